"""Causal self-attention at head dimension 128 on the tcgen05 kernel (``csrc/causal_attn_sm100.cu``): the attention
layers of the StripedHyena-2 models (the protein language models of this package have head dimension 64 and stay on the library call).

The reference calls a library flash-attention at this site (evo2/opt/evo2_opt/kit/base.py).
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from . import native

HEAD_DIM = 128
# Measured on B200 at 32 heads x 128 (batch 1): this kernel runs at 1.05 PFLOP/s at 32768 tokens, the library's fused
# attention at 1.51; the models therefore take the kernel only when asked to (UBM_CAUSAL_KERNEL=1 or ``ENABLED``).
ENABLED = os.environ.get("UBM_CAUSAL_KERNEL") == "1"

native.declare("ubm_causal_attention_d128",
               [native.c_void_p] * 4 + [native.c_int] * 5 + [native.c_ll] * 3 + [native.c_float] +
               [native.c_void_p] * 2)


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> Optional[str]:
    """None when the kernel takes this call, else the reason it does not."""
    if not q.is_cuda:
        return "not_cuda"
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        return "dtype"
    if q.dim() != 4 or q.shape[-1] != HEAD_DIM or k.shape[-1] != HEAD_DIM or v.shape != k.shape:
        return f"head_dim_{q.shape[-1]}"
    if k.shape[1] < q.shape[1] or q.shape[2] % k.shape[2]:
        return "shape"
    return None


def _rows(t: torch.Tensor) -> torch.Tensor:
    """[B, T, H, 128] with unit channel stride, head stride 128, a row stride that is a multiple of 16 elements and
    batch stride = T rows (what one 3-d tensor map over [columns, rows, batch] can describe); else a packed copy."""
    B, T, H, D = t.shape
    ok = (t.stride(3) == 1 and t.stride(2) == D and t.stride(1) % 16 == 0 and t.stride(1) >= H * D and
          (B == 1 or t.stride(0) == T * t.stride(1)) and t.data_ptr() % 16 == 0)
    return t if ok else t.contiguous()


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q: bf16 [B, Tq, H, 128]; k, v: bf16 [B, Tk, Hkv, 128] (Hkv divides H, Tk >= Tq; query i sees keys
    0 .. i + Tk - Tq).  Returns bf16 [B, Tq, H, 128].  q / k / v may be column slices of one projection output."""
    why = supported(q, k, v)
    if why is not None:
        raise ValueError(f"causal_attention does not take this call: {why}")
    q, k, v = _rows(q), _rows(k), _rows(v)
    if k.stride(1) != v.stride(1):
        v = v.contiguous()
        k = k.contiguous()
    B, Tq, H, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    if out is None:
        out = torch.empty((B, Tq, H, D), dtype=torch.bfloat16, device=q.device)
    if not out.is_contiguous() or out.dtype != torch.bfloat16 or out.shape != (B, Tq, H, D):
        raise ValueError("out must be a contiguous bf16 [B, Tq, H, 128] tensor")
    st = native.status_tensor(q.device)
    rc = native.lib().ubm_causal_attention_d128(
        native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(out), B, H, Hkv, Tq, Tk,
        q.stride(1), k.stride(1), H * D, float(scale if scale is not None else 1.0 / math.sqrt(D)),
        native.ptr(st), native.current_stream(q.device))
    native.check(rc, "ubm_causal_attention_d128")
    return out


def reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """Plain fp32 statement of the same attention (tests, CPU)."""
    B, Tq, H, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    g = H // Hkv
    kf = k.float().repeat_interleave(g, 2)
    vf = v.float().repeat_interleave(g, 2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kf) * (scale if scale is not None else 1.0 / math.sqrt(D))
    qi = torch.arange(Tq, device=q.device)[:, None] + (Tk - Tq)
    ki = torch.arange(Tk, device=q.device)[None, :]
    s = s.masked_fill(ki > qi, float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vf)
