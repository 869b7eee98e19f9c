"""Python face of the row / sequence kernels for the language-model and genomics families
(``csrc/seq_sm100.cu``): RMSNorm, the causal FIR stages of the Hyena operators with their gates folded in, the
FFT-convolution epilogue, the decode step of the pole-residue filter, and the exact elementwise sets (gelu_new,
residual adds, bias + residual, folded batch-norm + GELU, rotary split of a fused q|k|v row, softmax of a
three-term sum, width-2 pooling, residual + LayerNorm).  Every wrapper has a plain statement of the same name in
:mod:`ops.reference`.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import native
from .native import c_float, c_int, c_ll, c_void_p

native.declare("ubm_rmsnorm_rows", [c_void_p] * 3 + [c_ll, c_int, c_float, c_void_p])
native.declare("ubm_fir_gate3", [c_void_p] * 5 + [c_int] * 5 + [c_void_p])
native.declare("ubm_fir_step", [c_void_p] * 6 + [c_int] * 3 + [c_void_p])
native.declare("ubm_fir_inner_gate", [c_void_p] * 6 + [c_int] * 4 + [c_void_p])
native.declare("ubm_fftconv_epilogue", [c_void_p, c_int] + [c_void_p] * 4 + [c_int] * 3 + [c_void_p])
native.declare("ubm_pole_step", [c_void_p] * 7 + [c_int] * 3 + [c_void_p])
native.declare("ubm_elementwise", [c_int] + [c_void_p] * 6 + [c_ll, c_int, c_void_p])
native.declare("ubm_rotary_split_qkv", [c_void_p] * 5 + [c_ll, c_int, c_int, c_int, c_float, c_void_p])
native.declare("ubm_add2_softmax_rows", [c_void_p] * 4 + [c_ll, c_int, c_void_p])
native.declare("ubm_pool2", [c_void_p] * 3 + [c_int] * 4 + [c_void_p])
native.declare("ubm_residual_ln", [c_void_p] * 6 + [c_ll, c_int, c_float, c_void_p])

native.declare("ubm_gemv_fused", [c_void_p] * 2 + [c_float] + [c_void_p] * 5 + [c_int] * 3 + [c_void_p])
native.declare("ubm_gemv_fused_w8", [c_void_p] * 2 + [c_float, c_void_p, c_float] + [c_void_p] * 3 + [c_int] * 3 + [c_void_p])
native.declare("ubm_rmsnorm_fp8", [c_void_p] * 5 + [c_ll, c_int, c_float, c_void_p])
native.declare("ubm_pole_prefill_state", [c_void_p] * 4 + [c_int] * 5 + [c_void_p])
native.declare("ubm_fft_pad_transpose", [c_void_p] * 2 + [c_int] * 4 + [c_void_p])
native.declare("ubm_spectrum_mul", [c_void_p] * 2 + [c_int, c_ll, c_void_p])
native.declare("ubm_decode_attention", [c_void_p] * 7 + [c_int] * 4 + [c_float] * 2 + [c_void_p] * 2)
native.declare("ubm_column_attention", [c_void_p] * 6 + [c_ll, c_int, c_int, c_int, c_float, c_void_p])
native.declare("ubm_relshift_softmax", [c_void_p] * 3 + [c_ll, c_int, c_int, c_void_p])

EW = {"gelu_new": 0, "add2": 1, "bias_residual": 2, "scale_shift_gelu": 3, "silu_mul": 4}


def _bf16c(t: torch.Tensor) -> torch.Tensor:
    if t.dtype != torch.bfloat16:
        raise TypeError("bf16 activation expected")
    return t.contiguous()


_F32_CACHE: dict = {}


def _f32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """Contiguous fp32 form of a per-channel vector.  Parameters (leaf tensors that outlive the call) are converted
    once and kept until they are written again: a decode step reads dozens of them."""
    if t is None:
        return None
    if t.dtype == torch.float32 and t.is_contiguous():
        return t.detach()
    if not isinstance(t, torch.nn.Parameter):
        return t.detach().float().contiguous()
    ent = _F32_CACHE.get(id(t))
    if ent is None or ent[0] is not t or ent[1] != t._version or ent[2].device != t.device:
        if len(_F32_CACHE) > 4096:
            _F32_CACHE.clear()
        ent = (t, t._version, t.detach().float().contiguous())
        _F32_CACHE[id(t)] = ent
    return ent[2]


def _stream(t: torch.Tensor):
    return native.current_stream(t.device)


def rmsnorm_rows(x: torch.Tensor, scale: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    x = _bf16c(x)
    C = x.shape[-1]
    out = torch.empty_like(x)
    sc = _f32(scale)        # held in a variable: a temporary would be freed (and its block reused) before the launch
    rc = native.lib().ubm_rmsnorm_rows(native.ptr(x), native.ptr(sc), native.ptr(out), x.numel() // C, C,
                                       float(eps), _stream(x))
    native.check(rc, "ubm_rmsnorm_rows")
    return out


def rmsnorm_fp8(x: torch.Tensor, scale: torch.Tensor, eps: float = 1e-6):
    """RMSNorm rows as e4m3 for an fp8 projection, scaled by the tensor's own maximum.  x: bf16 [.., C], C <= 4096.
    Returns (``torch.float8_e4m3fn`` [R, C], fp32 [1] dequantisation factor on the device)."""
    x = _bf16c(x)
    C = x.shape[-1]
    R = x.numel() // C
    out = torch.empty((R, C), dtype=torch.float8_e4m3fn, device=x.device)
    work = torch.empty(2, dtype=torch.float32, device=x.device)          # [0]: bits of the maximum, [1]: max / 448
    sc = _f32(scale)
    rc = native.lib().ubm_rmsnorm_fp8(native.ptr(x), native.ptr(sc), native.ptr(work), native.ptr(out),
                                      native.ptr(work) + 4, R, C, float(eps), _stream(x))
    native.check(rc, "ubm_rmsnorm_fp8")
    return out, work[1:2]


def taps_major(h: torch.Tensor) -> torch.Tensor:
    """[C, K] filter -> fp32 [K, C] (tap-major, the layout the FIR kernels read)."""
    return h.detach().float().t().contiguous()


def fir_gate3(z: torch.Tensor, ht: torch.Tensor, tail: Optional[torch.Tensor] = None,
              push: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """z: [B, L, 3d]; ht: fp32 [K, 3d] from :func:`taps_major`; tail: [B, K-1, 3d].  Returns (u, x2), each [B, L, d].
    ``push`` (decode, L <= 32): ``tail`` (contiguous bf16) is replaced in place by the last K - 1 samples."""
    z = _bf16c(z)
    B, L, C = z.shape
    d = C // 3
    u = torch.empty((B, L, d), dtype=torch.bfloat16, device=z.device)
    x2 = torch.empty_like(u)
    if push and (tail is None or tail.dtype != torch.bfloat16 or not tail.is_contiguous()):
        raise ValueError("fir_gate3: push needs a contiguous bf16 tail")
    t = None if tail is None else _bf16c(tail)
    rc = native.lib().ubm_fir_gate3(native.ptr(z), native.ptr(ht), native.ptr(t), native.ptr(u), native.ptr(x2),
                                    B, L, d, ht.shape[0], 1 if push else 0, _stream(z))
    native.check(rc, "ubm_fir_gate3")
    return u, x2


def fir_step(u: torch.Tensor, ht: torch.Tensor, D: torch.Tensor, x2: Optional[torch.Tensor],
             tail: torch.Tensor) -> torch.Tensor:
    """Decode form of :func:`fir_inner_gate` for one new position per batch row.  u, x2: [B, 1, d]; ht: fp32 [K, d]
    (2 <= K <= 256); tail: contiguous bf16 [B, K-1, d], replaced in place by (tail[:, 1:], u)."""
    u = _bf16c(u)
    B, L, d = u.shape
    if L != 1 or tail.dtype != torch.bfloat16 or not tail.is_contiguous() or tail.shape != (B, ht.shape[0] - 1, d):
        raise ValueError("fir_step: one position per row and a contiguous bf16 tail [B, K-1, d]")
    out = torch.empty_like(u)
    x2c = None if x2 is None else _bf16c(x2)
    Df = _f32(D)
    rc = native.lib().ubm_fir_step(native.ptr(u), native.ptr(ht), native.ptr(Df), native.ptr(x2c), native.ptr(tail),
                                   native.ptr(out), B, d, ht.shape[0], _stream(u))
    native.check(rc, "ubm_fir_step")
    return out


def fir_inner_gate(u: torch.Tensor, ht: torch.Tensor, D: torch.Tensor, x2: Optional[torch.Tensor],
                   tail: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x2 * (causal_fir(u, h) + D * u); u, x2: [B, L, d]; ht: fp32 [K, d]; tail: [B, K-1, d]."""
    u = _bf16c(u)
    B, L, d = u.shape
    out = torch.empty_like(u)
    x2c = None if x2 is None else _bf16c(x2)
    t = None if tail is None else _bf16c(tail)
    Df = _f32(D)
    rc = native.lib().ubm_fir_inner_gate(native.ptr(u), native.ptr(ht), native.ptr(Df), native.ptr(x2c),
                                         native.ptr(t), native.ptr(out), B, L, d, ht.shape[0], _stream(u))
    native.check(rc, "ubm_fir_inner_gate")
    return out


def fftconv_epilogue(y: torch.Tensor, u: torch.Tensor, D: torch.Tensor, x2: Optional[torch.Tensor]) -> torch.Tensor:
    """y: fp32 [B, d, n] (inverse FFT output, first L samples used); u, x2: [B, L, d] -> x2 * (y^T + D * u)."""
    u = _bf16c(u)
    B, L, d = u.shape
    y = y.contiguous()
    if y.dtype != torch.float32 or y.shape[0] != B or y.shape[1] != d or y.shape[2] < L:
        raise ValueError("y must be fp32 [B, d, n >= L]")
    out = torch.empty_like(u)
    x2c = None if x2 is None else _bf16c(x2)
    Df = _f32(D)
    rc = native.lib().ubm_fftconv_epilogue(native.ptr(y), y.shape[2], native.ptr(u), native.ptr(Df),
                                           native.ptr(x2c), native.ptr(out), B, L, d, _stream(u))
    native.check(rc, "ubm_fftconv_epilogue")
    return out


def pole_step(state: torch.Tensor, lam: torch.Tensor, res: torch.Tensor, u: torch.Tensor, D: torch.Tensor,
              x2: Optional[torch.Tensor]) -> torch.Tensor:
    """state: fp32 [B, d, S], updated in place; u, x2: [B, d] -> x2 * (sum_s state * res + D * u)."""
    if state.dtype != torch.float32 or not state.is_contiguous():
        raise ValueError("state must be contiguous fp32")
    u = _bf16c(u)
    B, d, S = state.shape
    out = torch.empty_like(u)
    x2c = None if x2 is None else _bf16c(x2)
    lamf, resf, Df = _f32(lam), _f32(res), _f32(D)
    rc = native.lib().ubm_pole_step(native.ptr(state), native.ptr(lamf), native.ptr(resf), native.ptr(u),
                                    native.ptr(Df), native.ptr(x2c), native.ptr(out), B, d, S, _stream(u))
    native.check(rc, "ubm_pole_step")
    return out


def pole_prefill_state(u: torch.Tensor, lam: torch.Tensor) -> torch.Tensor:
    """The pole state a prefill leaves for decoding: fp32 [B, d, S] with state[b, c, k] = sum_t lam[c, k]^(L-1-t)
    u[b, t, c].  u: bf16 [B, L, d]; lam: [d, S], S <= 16."""
    u = _bf16c(u)
    B, L, d = u.shape
    lamf = _f32(lam)
    S = lamf.shape[1]
    chunks = max(1, min(64, (L + 1023) // 1024))
    part = torch.empty((B, chunks, d, S), dtype=torch.float32, device=u.device)
    state = torch.empty((B, d, S), dtype=torch.float32, device=u.device)
    rc = native.lib().ubm_pole_prefill_state(native.ptr(u), native.ptr(lamf), native.ptr(part), native.ptr(state),
                                             B, L, d, S, chunks, _stream(u))
    native.check(rc, "ubm_pole_prefill_state")
    return state


def fft_pad_transpose(u: torch.Tensor, n: int) -> torch.Tensor:
    """u: bf16 [B, L, d] -> fp32 [B, d, n], zero from position L on (the input layout of the long convolution's FFT)."""
    u = _bf16c(u)
    B, L, d = u.shape
    out = torch.empty((B, d, n), dtype=torch.float32, device=u.device)
    rc = native.lib().ubm_fft_pad_transpose(native.ptr(u), native.ptr(out), B, L, d, n, _stream(u))
    native.check(rc, "ubm_fft_pad_transpose")
    return out


def spectrum_mul_(X: torch.Tensor, H: torch.Tensor) -> torch.Tensor:
    """X: complex64 [B, d, m], multiplied in place by H: complex64 [d, m]."""
    if X.dtype != torch.complex64 or H.dtype != torch.complex64 or not X.is_contiguous() or not H.is_contiguous() \
            or X.shape[1:] != H.shape:
        raise ValueError("spectrum_mul_: contiguous complex64 [B, d, m] and [d, m]")
    rc = native.lib().ubm_spectrum_mul(native.ptr(X), native.ptr(H), X.shape[0], H.numel(), _stream(X))
    native.check(rc, "ubm_spectrum_mul")
    return X


def elementwise(op: str, x: torch.Tensor, a: Optional[torch.Tensor] = None, b: Optional[torch.Tensor] = None,
                v0: Optional[torch.Tensor] = None, v1: Optional[torch.Tensor] = None) -> torch.Tensor:
    x = _bf16c(x)
    C = x.shape[-1]
    out = torch.empty_like(x)
    aa = None if a is None else _bf16c(a)
    bb = None if b is None else _bf16c(b)
    # the converted vectors live in variables until the launch is queued: two temporaries in one argument list
    # would share one freed block
    v0f, v1f = _f32(v0), _f32(v1)
    rc = native.lib().ubm_elementwise(EW[op], native.ptr(x), native.ptr(aa), native.ptr(bb), native.ptr(v0f),
                                      native.ptr(v1f), native.ptr(out), x.numel() // C, C, _stream(x))
    native.check(rc, "ubm_elementwise")
    return out


def gelu_new(x):
    return elementwise("gelu_new", x)


def residual_add2(x, a, b=None):
    return elementwise("add2", x, a, b)


def bias_residual(x, bias, res=None):
    return elementwise("bias_residual", x, res, None, bias)


def scale_shift_gelu(x, scale, shift):
    return elementwise("scale_shift_gelu", x, None, None, scale, shift)


def silu_mul(x, a):
    return elementwise("silu_mul", x, a)


def rotary_split_qkv(qkv: torch.Tensor, pos: torch.Tensor, heads: int, rot: int, base: float = 10000.0):
    """qkv: [T, 3 * heads * Dh] -> (q, k, v) each [T, heads, Dh]; interleaved-pair rotary on the first ``rot`` dims."""
    qkv = _bf16c(qkv)
    T = qkv.shape[0]
    Dh = qkv.shape[1] // (3 * heads)
    q = torch.empty((T, heads, Dh), dtype=torch.bfloat16, device=qkv.device)
    k, v = torch.empty_like(q), torch.empty_like(q)
    p = pos.to(torch.int32).contiguous()
    rc = native.lib().ubm_rotary_split_qkv(native.ptr(qkv), native.ptr(p), native.ptr(q), native.ptr(k), native.ptr(v),
                                           T, heads, Dh, rot, float(base), _stream(qkv))
    native.check(rc, "ubm_rotary_split_qkv")
    return q, k, v


def add2_softmax_rows(x: torch.Tensor, a: Optional[torch.Tensor] = None, b: Optional[torch.Tensor] = None):
    x = x.float().contiguous()
    C = x.shape[-1]
    out = torch.empty_like(x)
    aa = None if a is None else a.float().contiguous()
    bb = None if b is None else b.float().contiguous()
    rc = native.lib().ubm_add2_softmax_rows(native.ptr(x), native.ptr(aa), native.ptr(bb), native.ptr(out),
                                            x.numel() // C, C, _stream(x))
    native.check(rc, "ubm_add2_softmax_rows")
    return out


def pool2(x: torch.Tensor, mode: str = "max", w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Width-2 pooling along dim 1 of [B, L, C]: ``max``, ``mean`` or ``softmax`` (weights from logits ``w``)."""
    x = _bf16c(x)
    B, L, C = x.shape
    out = torch.empty((B, L // 2, C), dtype=torch.bfloat16, device=x.device)
    ww = None if w is None else _bf16c(w)
    rc = native.lib().ubm_pool2(native.ptr(x), native.ptr(ww), native.ptr(out), B, L, C,
                                {"max": 0, "mean": 1, "softmax": 2}[mode], _stream(x))
    native.check(rc, "ubm_pool2")
    return out


def residual_ln(x: torch.Tensor, res: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor],
                eps: float = 1e-5, return_sum: bool = False):
    x, res = _bf16c(x), _bf16c(res)
    C = x.shape[-1]
    out = torch.empty_like(x)
    s = torch.empty_like(x) if return_sum else None
    gf, bf = _f32(gamma), _f32(beta)
    rc = native.lib().ubm_residual_ln(native.ptr(x), native.ptr(res), native.ptr(gf), native.ptr(bf),
                                      native.ptr(s), native.ptr(out), x.numel() // C, C, float(eps), _stream(x))
    native.check(rc, "ubm_residual_ln")
    return (out, s) if return_sum else out


def gemv_rows(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, *,
              gamma: Optional[torch.Tensor] = None, eps: float = 1e-6, w2: Optional[torch.Tensor] = None,
              res: Optional[torch.Tensor] = None, wscale: Optional[float] = None) -> torch.Tensor:
    """x: bf16 [M, K] with M <= 8 (decode rows); w: bf16 [N, K] contiguous; returns bf16 [M, N] = x^ @ w.T (+ bias).
    ``w`` may hold e4m3 values (``torch.float8_e4m3fn``, K a multiple of 16) with ``wscale`` their dequantisation
    factor: half the bytes per output row, activations still bf16 (not with ``w2``).

    The rows of a decode block fold into the same launch: ``gamma`` (fp32 [K]) puts RMSNorm in front
    (x^ = rmsnorm(x) * gamma, else x^ = x); ``w2`` makes the SwiGLU form silu(x^ @ w.T) * (x^ @ w2.T); ``res``
    (bf16 [M, N]) is added behind.  Every intermediate is rounded to bf16 where the separate kernels round it."""
    x = _bf16c(x)
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    if w2 is not None and (w2.shape != w.shape or not w2.is_contiguous()):
        raise ValueError("gemv_rows: w2 must match w")
    if res is not None:
        res = _bf16c(res.reshape(M, N))
    gamma = _f32(gamma)                  # a parameter in another type is converted once, not per decode step
    if w.dtype in (torch.float8_e4m3fn, torch.uint8):
        if w2 is not None or wscale is None or not w.is_contiguous():
            raise ValueError("gemv_rows: e4m3 weights come with wscale, contiguous, and without w2")
        rc = native.lib().ubm_gemv_fused_w8(native.ptr(x), native.ptr(gamma), float(eps), native.ptr(w), float(wscale),
                                            native.ptr(bias), native.ptr(res), native.ptr(out), M, N, K, _stream(x))
        native.check(rc, "ubm_gemv_fused_w8")
        return out
    rc = native.lib().ubm_gemv_fused(native.ptr(x), native.ptr(gamma), float(eps), native.ptr(w), native.ptr(w2),
                                     native.ptr(bias), native.ptr(res), native.ptr(out), M, N, K, _stream(x))
    native.check(rc, "ubm_gemv_fused")
    return out


def decode_attention(qkv: torch.Tensor, pos: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor,
                     rope_base: float, scale: Optional[float] = None) -> torch.Tensor:
    """One new token against a fixed-size cache (``csrc/decode_attn_sm100.cu``).  qkv: bf16 [B, 3 * H * 128]
    (q | k | v); pos: int64 [1] on the device, the cache row the new key / value take (keys 0..pos are attended);
    kc, vc: contiguous bf16 [B, Lmax, H, 128], written at row pos.  Rotary embedding (interleaved pairs) is applied
    to q and k.  Returns bf16 [B, H * 128].  No host value enters: the call can be captured in a CUDA graph."""
    qkv = _bf16c(qkv)
    B, Lmax, H, hd = kc.shape
    if hd != 128 or qkv.shape != (B, 3 * H * hd) or vc.shape != kc.shape or kc.dtype != torch.bfloat16 or \
            vc.dtype != torch.bfloat16 or not kc.is_contiguous() or not vc.is_contiguous():
        raise ValueError("decode_attention: bf16 caches [B, Lmax, H, 128] and qkv [B, 3*H*128]")
    if pos.dtype != torch.int64 or pos.numel() != 1 or pos.device != qkv.device:
        raise ValueError("decode_attention: pos is an int64 device tensor with one element")
    # one split per 1024 cache rows (sizing the split count for four full waves of CTAs instead measured slower:
    # 137 against 130 us at 33000 keys, 58 against 48 us at 8192)
    splits = max(1, min(64, (Lmax + 1023) // 1024))
    q_rot = torch.empty((B, H, hd), dtype=torch.bfloat16, device=qkv.device)
    part = torch.empty((B, H, splits, hd + 2), dtype=torch.float32, device=qkv.device)
    out = torch.empty((B, H * hd), dtype=torch.bfloat16, device=qkv.device)
    sc = float(hd) ** -0.5 if scale is None else float(scale)
    rc = native.lib().ubm_decode_attention(native.ptr(qkv), native.ptr(pos), native.ptr(kc), native.ptr(vc),
                                           native.ptr(q_rot), native.ptr(part), native.ptr(out), B, H, Lmax, splits,
                                           float(rope_base), sc, native.ptr(native.status_tensor(qkv.device)),
                                           _stream(qkv))
    native.check(rc, "ubm_decode_attention")
    return out


def column_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, index: torch.Tensor,
                     bias: Optional[torch.Tensor] = None, scale: Optional[float] = None) -> torch.Tensor:
    """Per-column attention over clade rows (``csrc/lmops_sm100.cu``).  q: bf16 [T, H, D]; k, v: bf16 [R, T, H, D]
    (one row per distinct alignment row); index: int [C] clade -> row; bias: fp32 [H, C] or None.  D is 32 or 64,
    C <= 256.  Returns bf16 [T, H, D]."""
    q, k, v = _bf16c(q), _bf16c(k), _bf16c(v)
    T, H, D = q.shape
    C = index.shape[0]
    idx = index.to(torch.int32).contiguous()
    out = torch.empty_like(q)
    sc = float(D) ** -0.5 if scale is None else float(scale)
    bf = _f32(bias)
    rc = native.lib().ubm_column_attention(native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(idx),
                                           native.ptr(bf), native.ptr(out), T, H, D, C, sc, _stream(q))
    native.check(rc, "ubm_column_attention")
    return out


def relshift_softmax(content: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    """softmax_j(content[..., i, j] + pos[..., i, j - i + L - 1]) for content fp32 [..., L, L] and relative-position
    logits pos fp32 [..., L, P] with P >= 2L - 1 (columns past 2L - 2 are padding; the row stride of ``pos`` may
    exceed P): the shift is an index, no shifted copy is made."""
    content = content.float().contiguous()
    L = content.shape[-1]
    if pos.dtype != torch.float32 or pos.stride(-1) != 1:
        pos = pos.float().contiguous()
    ldp = pos.stride(-2)
    flat = pos.dim() == 2 or all(pos.stride(i) == pos.stride(i + 1) * pos.shape[i + 1] for i in range(pos.dim() - 2))
    if not flat:
        pos = pos.contiguous()
        ldp = pos.stride(-2)
    if content.shape[-2] != L or pos.shape[-1] < 2 * L - 1 or pos.shape[:-1] != content.shape[:-1]:
        raise ValueError("relshift_softmax expects content [..., L, L] and pos [..., L, >= 2L - 1]")
    out = torch.empty_like(content)
    rc = native.lib().ubm_relshift_softmax(native.ptr(content), native.ptr(pos), native.ptr(out),
                                           content.numel() // L, L, ldp, _stream(content))
    native.check(rc, "ubm_relshift_softmax")
    return out
