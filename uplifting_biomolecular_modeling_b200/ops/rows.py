"""Python face of the row kernels (``csrc/rows_sm100.cu``): LayerNorm rows, pair -> head-bias
planes, AdaLN, gated residual, SwiGLU.  Each wrapper has the same signature as its plain
statement in :mod:`ops.reference` where one exists."""
from __future__ import annotations

import weakref
from typing import Optional

import torch

from . import native
from .native import c_float, c_int, c_ll, c_void_p

native.declare("ubm_layernorm_rows", [c_void_p] * 4 + [c_ll, c_int, c_float, c_int, c_int, c_void_p])
native.declare("ubm_pair_head_bias", [c_void_p] * 5 + [c_int, c_int, c_int, c_int, c_void_p])
native.declare("ubm_adaln_rows", [c_void_p] * 4 + [c_ll, c_int, c_ll, c_ll, c_float, c_void_p])
native.declare("ubm_gate_residual", [c_void_p] * 4 + [c_ll, c_int, c_ll, c_ll, c_void_p])
native.declare("ubm_swiglu_rows", [c_void_p] * 2 + [c_ll, c_int, c_void_p])
native.declare("ubm_swiglu3_rows", [c_void_p] * 2 + [c_ll, c_int, c_void_p])
native.declare("ubm_segment_mean", [c_void_p] * 3 + [c_int] * 5 + [c_void_p])
native.declare("ubm_gather_rows_add", [c_void_p] * 4 + [c_int] * 4 + [c_void_p])

_DT = {torch.bfloat16: 0, torch.float32: 1}


_F32_CACHE: dict = {}


def _f32_param(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """Contiguous fp32 copy of an affine parameter, kept until the parameter is written again (the conversion was two
    small launches per LayerNorm call)."""
    if t is None:
        return None
    if t.dtype == torch.float32 and t.is_contiguous():
        return t.detach()
    ent = _F32_CACHE.get(id(t))
    if ent is None or ent[0] is not t or ent[1] != t._version or ent[2].device != t.device:
        if len(_F32_CACHE) > 4096:
            _F32_CACHE.clear()
        ent = (t, t._version, t.detach().float().contiguous())
        _F32_CACHE[id(t)] = ent
    return ent[2]


def layernorm_rows(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                   eps: float = 1e-5, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    if x.dtype not in _DT or not x.is_contiguous():
        raise ValueError("layernorm_rows expects contiguous bf16 / fp32 input")
    C = x.shape[-1]
    R = x.numel() // C
    out_dtype = out_dtype or x.dtype
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    w, b = _f32_param(weight), _f32_param(bias)
    rc = native.lib().ubm_layernorm_rows(native.ptr(x), native.ptr(w), native.ptr(b), native.ptr(out), R, C,
                                         float(eps), _DT[x.dtype], _DT[out_dtype], native.current_stream(x.device))
    native.check(rc, "ubm_layernorm_rows")
    return out


_HB_CACHE = {}


def pair_head_bias(z: torch.Tensor, ln_w, ln_b, w, scale: float = 1.0, transpose: bool = False,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """z: bf16 [N, N, 128]; w: [H, 128].  Returns bf16 [H, N, N] (a view of planes padded to a
    multiple of 8 columns) with ``scale * Linear(LN(z))`` laid out head-major."""
    N = z.shape[0]
    H = w.shape[0]
    Np = (N + 7) // 8 * 8
    # the cache entry is tied to the live weight tensor object (a freed tensor's address may be reused)
    key = (id(w), w._version, None if ln_w is None else ln_w._version, float(scale), str(z.device))
    entry = _HB_CACHE.get(key)
    packed = entry[1] if entry is not None and entry[0]() is w else None
    if packed is None:
        gam = torch.ones(128, device=z.device) if ln_w is None else ln_w.detach().float()
        wf = (w.detach().float() * gam[None, :] * scale).contiguous()
        colsum = wf.sum(1).contiguous()
        colbias = torch.zeros(H, device=z.device) if ln_b is None else \
            ((w.detach().float() @ ln_b.detach().float()) * scale).contiguous()
        packed = (wf, colsum, colbias)
        if len(_HB_CACHE) > 4096:
            _HB_CACHE.clear()
        _HB_CACHE[key] = (weakref.ref(w), packed)
    wf, colsum, colbias = packed
    if out is None:
        out = torch.zeros((H, N, Np), dtype=torch.bfloat16, device=z.device) if Np != N else \
            torch.empty((H, N, Np), dtype=torch.bfloat16, device=z.device)
    rc = native.lib().ubm_pair_head_bias(native.ptr(z), native.ptr(wf), native.ptr(colsum), native.ptr(colbias),
                                         native.ptr(out), N, Np, H, 1 if transpose else 0,
                                         native.current_stream(z.device))
    native.check(rc, "ubm_pair_head_bias")
    return out[:, :, :N]


def _cond2d(t: torch.Tensor, C: int) -> torch.Tensor:
    """Conditioning rows as a 2-D view [rows, C] whose rows may be strided (a column slice of a wider buffer)."""
    t2 = t.reshape(-1, C) if t.is_contiguous() else t.squeeze(0) if t.dim() == 3 and t.shape[0] == 1 else t
    if t2.dim() != 2 or t2.shape[1] != C or t2.stride(1) != 1:
        t2 = t.reshape(-1, C).contiguous()
    return t2


def adaln_rows(a: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """sigmoid(scale) * LN_noaffine(a) + shift; scale/shift rows are reused cyclically over a's rows and may be
    column slices of one wider buffer (equal row strides)."""
    C = a.shape[-1]
    R = a.numel() // C
    out = torch.empty_like(a)
    sc, sh = _cond2d(scale, C), _cond2d(shift, C)
    if sc.stride(0) != sh.stride(0) or sc.shape[0] != sh.shape[0]:
        sc, sh = sc.contiguous(), sh.contiguous()
    rc = native.lib().ubm_adaln_rows(native.ptr(a), native.ptr(sc), native.ptr(sh), native.ptr(out), R, C,
                                     sc.shape[0], sc.stride(0), float(eps), native.current_stream(a.device))
    native.check(rc, "ubm_adaln_rows")
    return out


def gate_residual(x: torch.Tensor, gate: torch.Tensor, res: Optional[torch.Tensor]) -> torch.Tensor:
    """res + sigmoid(gate) * x; gate rows reused cyclically, possibly a column slice of a wider buffer."""
    C = x.shape[-1]
    R = x.numel() // C
    out = torch.empty_like(x)
    g = _cond2d(gate, C)
    rc = native.lib().ubm_gate_residual(native.ptr(x), native.ptr(g), native.ptr(res), native.ptr(out), R, C,
                                        g.shape[0], g.stride(0), native.current_stream(x.device))
    native.check(rc, "ubm_gate_residual")
    return out


def swiglu3_rows(x: torch.Tensor) -> torch.Tensor:
    """x: [.., 3*Hd] = [u | g | w] -> silu(u) * g * w."""
    Hd = x.shape[-1] // 3
    R = x.numel() // (3 * Hd)
    out = torch.empty(x.shape[:-1] + (Hd,), dtype=x.dtype, device=x.device)
    rc = native.lib().ubm_swiglu3_rows(native.ptr(x), native.ptr(out), R, Hd, native.current_stream(x.device))
    native.check(rc, "ubm_swiglu3_rows")
    return out


def swiglu_rows(ab: torch.Tensor) -> torch.Tensor:
    Hd = ab.shape[-1] // 2
    R = ab.numel() // (2 * Hd)
    out = torch.empty(ab.shape[:-1] + (Hd,), dtype=ab.dtype, device=ab.device)
    rc = native.lib().ubm_swiglu_rows(native.ptr(ab), native.ptr(out), R, Hd, native.current_stream(ab.device))
    native.check(rc, "ubm_swiglu_rows")
    return out


def segment_mean(t: torch.Tensor, table: torch.Tensor, n_tokens: int) -> torch.Tensor:
    """Mean of atom rows per token.  t: bf16 [B, A, C]; table: int32 [N, M] atom indices (-1 = none)."""
    t = t.contiguous()
    B, A, C = t.shape
    out = torch.empty((B, n_tokens, C), dtype=t.dtype, device=t.device)
    rc = native.lib().ubm_segment_mean(native.ptr(t), native.ptr(table), native.ptr(out), B, A, n_tokens,
                                       table.shape[1], C, native.current_stream(t.device))
    native.check(rc, "ubm_segment_mean")
    return out


def gather_rows_add(q: Optional[torch.Tensor], a: torch.Tensor, a2t: torch.Tensor) -> torch.Tensor:
    """q + a[:, a2t] (token rows broadcast to their atoms).  q: bf16 [B, A, C] or None; a: [B, N, C]; a2t: int32 [A]."""
    a = a.contiguous()
    B, N, C = a.shape
    A = a2t.shape[0]
    out = torch.empty((B, A, C), dtype=a.dtype, device=a.device)
    qq = None if q is None else q.contiguous()
    rc = native.lib().ubm_gather_rows_add(native.ptr(qq), native.ptr(a), native.ptr(a2t), native.ptr(out), B, A, N, C,
                                          native.current_stream(a.device))
    native.check(rc, "ubm_gather_rows_add")
    return out
