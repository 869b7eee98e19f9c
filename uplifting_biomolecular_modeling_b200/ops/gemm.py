"""Batched bf16 GEMM on the tcgen05 kernel (``csrc/gemm_sm100.cu``).

``gemm_tn`` contracts the last (contiguous) dimension of both operands; ``gemm_nt`` contracts
the second-to-last dimension (operands stored K x M / K x N).  Both accept an optional leading
batch dimension.  Replaces the cuBLAS strided-batched call of the reference's triangle
multiplication (common/opt_core/opt_core/kernels/fpf_trimul_v4/DESIGN.md:21-37).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import native

native.declare("ubm_gemm_fp8", [native.c_void_p] * 5 + [native.c_int] * 3 + [native.c_ll] * 4 +
               [native.c_int, native.c_float, native.c_void_p, native.c_void_p, native.c_void_p])

ACT = {None: 0, "none": 0, "silu": 1, "sigmoid": 2, "gelu": 3, "relu": 4, "swiglu3": 5, "swiglu": 6}


def pack_swiglu3(gate_w: torch.Tensor, value_w: torch.Tensor, value2_w: torch.Tensor) -> torch.Tensor:
    """Rows of three [H, K] projections interleaved in groups of 32 (gate | value | second value) as the
    ``act="swiglu3"`` epilogue reads them; H a multiple of 32.  Returns bf16 [3 * H, K]."""
    H, K = gate_w.shape
    if H % 32 or value_w.shape != (H, K) or value2_w.shape != (H, K):
        raise ValueError("pack_swiglu3 expects three [H, K] weights with H a multiple of 32")
    w = torch.stack([gate_w.view(H // 32, 32, K), value_w.view(H // 32, 32, K), value2_w.view(H // 32, 32, K)], 1)
    return w.reshape(3 * H, K).to(torch.bfloat16).contiguous()


def pack_swiglu(gate_w: torch.Tensor, value_w: torch.Tensor) -> torch.Tensor:
    """Rows of two [H, K] projections interleaved in groups of 32 (gate | value) as the ``act="swiglu"`` epilogue
    reads them; H a multiple of 32.  Returns bf16 [2 * H, K]."""
    H, K = gate_w.shape
    if H % 32 or value_w.shape != (H, K):
        raise ValueError("pack_swiglu expects two [H, K] weights with H a multiple of 32")
    w = torch.stack([gate_w.view(H // 32, 32, K), value_w.view(H // 32, 32, K)], 1)
    return w.reshape(2 * H, K).to(torch.bfloat16).contiguous()


def _as3(t: torch.Tensor) -> torch.Tensor:
    return t.unsqueeze(0) if t.dim() == 2 else t


def gemm(a: torch.Tensor, b: torch.Tensor, *, mn_major: bool = False, bias: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, act: Optional[str] = None, alpha: float = 1.0,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
         c_blocked: Optional[tuple] = None, gate: Optional[torch.Tensor] = None, act_from: int = 0) -> torch.Tensor:
    """C = act(alpha * A.B^T + bias) * gate + residual.

    ``act_from``: the activation applies to output columns >= act_from (a multiple of 32) only.
    ``act="swiglu3"`` (b packed by ``pack_swiglu3``, N a multiple of 96, no bias / gate / residual): the result is
    [.., M, N / 3] = silu(gate) * value * second value, computed in the epilogue on the accumulator;
    ``act="swiglu"`` (``pack_swiglu``, N a multiple of 64): [.., M, N / 2] = silu(gate) * value.
    ``gate`` (bf16 [rows, N], rows dividing M, row stride free): row m is multiplied by gate row m % rows -
    a conditioning gate shared by the samples stacked along M.

    ``c_blocked=(hi, lo, col)`` (with ``out`` given, N a multiple of 32, batch 1) stores element (m, n) at
    ``out.data_ptr + (m // 32) * hi + (m % 32) * lo + (n // 32) * col + n % 32`` elements: the product of two
    [(token, channel)] operands lands as [(i, j)][(c, d)] without a permuted copy.

    mn_major=False: a [.., M, K], b [.., N, K];  mn_major=True: a [.., K, M], b [.., K, N].
    The innermost dimension of a and b must be contiguous; other strides are free as long as
    they are multiples of 8 elements.
    """
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm expects bf16 operands")
    squeeze = a.dim() == 2
    a3, b3 = _as3(a), _as3(b)
    if a3.stride(-1) != 1 or b3.stride(-1) != 1:
        raise ValueError("innermost dimension must be contiguous")
    batch = a3.shape[0]
    if b3.shape[0] != batch:
        raise ValueError("batch mismatch")
    if mn_major:
        K, M = a3.shape[1], a3.shape[2]
        N = b3.shape[2]
        if b3.shape[1] != K:
            raise ValueError("K mismatch")
    else:
        M, K = a3.shape[1], a3.shape[2]
        N = b3.shape[1]
        if b3.shape[2] != K:
            raise ValueError("K mismatch")
    if c_blocked is not None:
        if out is None or batch != 1 or N % 32 or residual is not None:
            raise ValueError("c_blocked needs an output tensor, batch 1, N % 32 == 0 and no residual")
        out3 = out
    else:
        n_out = N
        if act in ("swiglu3", "swiglu"):
            group = 96 if act == "swiglu3" else 64
            if N % group or mn_major or bias is not None or gate is not None or residual is not None or act_from:
                raise ValueError(f"{act} needs a K-major product with N % {group} == 0 and no bias / gate / residual")
            n_out = N // 3 if act == "swiglu3" else N // 2
        if out is None:
            out = torch.empty((batch, M, n_out), dtype=torch.bfloat16 if n_out != N else out_dtype, device=a.device)
        out3 = _as3(out)
        if n_out != N and (out3.shape[-1] != n_out or out3.shape[-2] != M or out3.dtype != torch.bfloat16):
            raise ValueError(f"{act} output must be bf16 [.., {M}, {n_out}]")
        if out3.stride(-1) != 1:
            raise ValueError("output innermost dimension must be contiguous")
    res3 = None
    if residual is not None:
        res3 = _as3(residual)
        if res3.dtype != torch.bfloat16 or res3.stride(-1) != 1:
            raise ValueError("residual must be bf16 with contiguous rows")
    if bias is not None and bias.dtype != torch.float32:
        bias = bias.float()
    st = native.status_tensor(a.device)
    if gate is not None:
        if gate.dtype != torch.bfloat16 or gate.dim() != 2 or gate.shape[1] != N or gate.stride(1) != 1 or batch != 1:
            raise ValueError("gate must be bf16 [rows, N] with contiguous rows (batch 1)")
    cb = c_blocked if c_blocked is not None else (0, 0, 0)
    rc = native.lib().ubm_gemm_bf16_ex(
        native.ptr(a3), native.ptr(b3), native.ptr(out3), native.ptr(bias), native.ptr(res3),
        M, N, K, batch,
        a3.stride(1), b3.stride(1), 0 if c_blocked is not None else out3.stride(1),
        0 if res3 is None else res3.stride(1),
        a3.stride(0) if batch > 1 else 0, b3.stride(0) if batch > 1 else 0,
        out3.stride(0) if batch > 1 and c_blocked is None else 0,
        0 if res3 is None or batch == 1 else res3.stride(0),
        1 if mn_major else 0, 1 if out3.dtype == torch.float32 else 0, ACT[act], float(alpha),
        int(cb[0]), int(cb[1]), int(cb[2]), native.ptr(gate), 0 if gate is None else gate.stride(0),
        0 if gate is None else gate.shape[0], int(act_from), native.ptr(st), native.current_stream(a.device))
    native.check(rc, "ubm_gemm_bf16_ex")
    if c_blocked is not None:
        return out
    return out3[0] if squeeze and out.dim() == 3 else out


_E4M3 = (torch.uint8, torch.float8_e4m3fn)


def quantize_e4m3(w: torch.Tensor):
    """Per-tensor e4m3 form of a matrix: (bytes [rows, cols] as ``torch.float8_e4m3fn``, dequantisation factor
    max|w| / 448 as a Python float).  One host read of the maximum: meant for weights, once."""
    amax = float(w.detach().abs().max())
    amax = max(amax, 1e-12)
    q = (w.detach().float() * (448.0 / amax)).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn).contiguous()
    return q, amax / 448.0


def gemm_fp8(a8: torch.Tensor, b8: torch.Tensor, alpha: float = 1.0, alpha_dev: Optional[torch.Tensor] = None, *,
             bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None, act: Optional[str] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 [M, N] = act(alpha * alpha_dev * a8 @ b8^T + bias) (+ residual) with e4m3 operands a8 [M, K], b8 [N, K]
    (``torch.float8_e4m3fn`` or raw bytes, rows contiguous, K a multiple of 16) on the tcgen05 ``kind::f8f6f4`` path.
    ``alpha`` is the host-known dequantisation factor, ``alpha_dev`` (fp32 [1] on the device, optional) the one a
    kernel earlier in the stream wrote (:func:`ops.seq.rmsnorm_fp8`)."""
    if a8.dtype not in _E4M3 or b8.dtype not in _E4M3 or a8.dim() != 2 or b8.dim() != 2:
        raise TypeError("gemm_fp8 expects 2-D e4m3 (or uint8) operands")
    M, K = a8.shape
    N = b8.shape[0]
    if b8.shape[1] != K or a8.stride(1) != 1 or b8.stride(1) != 1 or act in ("swiglu", "swiglu3"):
        raise ValueError("gemm_fp8: K-major operands of equal K; no SwiGLU epilogue")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a8.device)
    if out.dtype != torch.bfloat16 or out.shape != (M, N) or out.stride(1) != 1:
        raise ValueError("gemm_fp8 output must be bf16 [M, N] with contiguous rows")
    if residual is not None and (residual.dtype != torch.bfloat16 or residual.shape != (M, N) or residual.stride(1) != 1):
        raise ValueError("residual must be bf16 [M, N] with contiguous rows")
    if bias is not None and bias.dtype != torch.float32:
        bias = bias.float()
    if alpha_dev is not None and (alpha_dev.dtype != torch.float32 or alpha_dev.numel() != 1 or alpha_dev.device != a8.device):
        raise ValueError("alpha_dev is one fp32 value on the operands' device")
    st = native.status_tensor(a8.device)
    rc = native.lib().ubm_gemm_fp8(native.ptr(a8), native.ptr(b8), native.ptr(out), native.ptr(bias),
                                   native.ptr(residual), M, N, K, a8.stride(0), b8.stride(0), out.stride(0),
                                   0 if residual is None else residual.stride(0), ACT[act], float(alpha),
                                   native.ptr(alpha_dev), native.ptr(st), native.current_stream(a8.device))
    native.check(rc, "ubm_gemm_fp8")
    return out


def gemm_tn(a, b, **kw):
    return gemm(a, b, mn_major=False, **kw)


def gemm_nt(a, b, **kw):
    return gemm(a, b, mn_major=True, **kw)
