"""Python face of the fused pair-stack kernels (triangle multiplication, pair transition,
triangle attention).  Weight preparation ("folding") happens once per module:

* LayerNorm is folded into the following Linear: ``W' = W * gamma`` (bf16), with the per-column
  constants ``colsum = rowsum(W')`` and ``colbias = W @ beta (+ bias)`` in fp32, so that
  ``Linear(LN(x)) = rstd * (W' x - mu * colsum) + colbias`` and the kernels feed raw rows to the
  tensor cores.
* Matrices that the kernels consume side by side are stacked in the order the kernel expects.

The reference performs the same kind of one-time weight work in its "castcache"/"interleave fold"
levers (common/opt_core/opt_core/of3_trunk/castcache.py, evo2/CHANGES.md lever L2).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import gemm as _gemm
from . import native
from .native import c_int, c_ll, c_void_p

native.declare("ubm_trimul_proj", [c_void_p] * 7 + [c_int, c_int, c_void_p, c_void_p])
native.declare("ubm_triatt_proj", [c_void_p] * 13 + [c_int, c_int, c_int, c_int, c_void_p, c_void_p])
native.declare("ubm_trimul_out", [c_void_p] * 9 + [c_int, c_int, c_int, c_void_p, c_void_p])
native.declare("ubm_transition", [c_void_p] * 8 + [c_ll, c_int, c_int, c_void_p, c_void_p])


def ceil_to(n: int, m: int) -> int:
    return (n + m - 1) // m * m


def fold_ln_linear(W: torch.Tensor, gamma: Optional[torch.Tensor], beta: Optional[torch.Tensor],
                   bias: Optional[torch.Tensor] = None, scale: float = 1.0):
    """Returns (W' bf16 [out, in], colsum fp32 [out], colbias fp32 [out]) for Linear(LN(x)) * scale."""
    Wf = W.detach().float()
    g = torch.ones(Wf.shape[1], device=Wf.device) if gamma is None else gamma.detach().float()
    Wg = (Wf * g[None, :]) * scale
    Wb = Wg.to(torch.bfloat16).contiguous()
    colsum = Wb.float().sum(dim=1).contiguous()
    colbias = torch.zeros(Wf.shape[0], device=Wf.device)
    if beta is not None:
        colbias = colbias + Wf @ beta.detach().float()
    if bias is not None:
        colbias = colbias + bias.detach().float()
    return Wb, colsum, (colbias * scale).contiguous()


# ------------------------------------------------------------------------------------------
@dataclass
class TransitionPacked:
    wab: torch.Tensor       # bf16 [(hidden/64)*128, 128]
    wo: torch.Tensor        # bf16 [128, hidden]
    colsum: torch.Tensor    # fp32 [(hidden/64)*128]
    colbias: torch.Tensor
    hidden: int

    @classmethod
    def pack(cls, norm_w, norm_b, fc1, fc2, fc3) -> "TransitionPacked":
        hidden, c = fc1.shape
        if c != 128 or hidden % 64 or hidden > 1024:
            raise ValueError(f"fused transition supports c=128 and hidden%64==0, <=1024 (got c={c}, hidden={hidden})")
        a, a_sum, a_bias = fold_ln_linear(fc1, norm_w, norm_b)
        b, b_sum, b_bias = fold_ln_linear(fc2, norm_w, norm_b)
        nch = hidden // 64
        wab = torch.stack([a.view(nch, 64, c), b.view(nch, 64, c)], dim=1).reshape(nch * 128, c).contiguous()
        colsum = torch.stack([a_sum.view(nch, 64), b_sum.view(nch, 64)], dim=1).reshape(-1).contiguous()
        colbias = torch.stack([a_bias.view(nch, 64), b_bias.view(nch, 64)], dim=1).reshape(-1).contiguous()
        return cls(wab, fc3.detach().to(torch.bfloat16).contiguous(), colsum, colbias, hidden)


def transition_fused(x: torch.Tensor, w: TransitionPacked, residual: bool = True,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x: bf16 [..., 128] contiguous.  Returns x + transition(x) (or the update alone)."""
    if x.dtype != torch.bfloat16 or x.shape[-1] != 128 or not x.is_contiguous():
        raise ValueError("transition_fused expects a contiguous bf16 tensor with 128 channels")
    R = x.numel() // 128
    out = torch.empty_like(x) if out is None else out
    st = native.status_tensor(x.device)
    rc = native.lib().ubm_transition(native.ptr(x), native.ptr(w.wab), native.ptr(w.wo), native.ptr(w.colsum),
                                     native.ptr(w.colbias), 0, 0, native.ptr(out), R, w.hidden,
                                     1 if residual else 0, native.ptr(st), native.current_stream(x.device))
    native.check(rc, "ubm_transition")
    return out


# ------------------------------------------------------------------------------------------
@dataclass
class TrimulPacked:
    w_in: torch.Tensor       # bf16 [512, 128] rows [p_a; g_a; p_b; g_b]
    in_colsum: torch.Tensor  # fp32 [512]
    in_colbias: torch.Tensor
    wo: torch.Tensor         # bf16 [128, 128]
    o_colsum: torch.Tensor
    o_colbias: torch.Tensor
    wg: torch.Tensor         # bf16 [128, 128]
    g_colsum: torch.Tensor
    g_colbias: torch.Tensor

    @classmethod
    def pack(cls, norm_in_w, norm_in_b, p_in, g_in, norm_out_w, norm_out_b, p_out, g_out) -> "TrimulPacked":
        two_h, c = p_in.shape
        if c != 128 or two_h != 256:
            raise ValueError("fused triangle multiplication supports c_z = c_hidden = 128")
        h = two_h // 2
        stacked = torch.cat([p_in[:h], g_in[:h], p_in[h:], g_in[h:]], dim=0)
        w_in, s_in, b_in = fold_ln_linear(stacked, norm_in_w, norm_in_b)
        wo, so, bo = fold_ln_linear(p_out, norm_out_w, norm_out_b)
        wg, sg, bg = fold_ln_linear(g_out, norm_in_w, norm_in_b)
        return cls(w_in, s_in, b_in, wo, so, bo, wg, sg, bg)


def trimul_fused(z: torch.Tensor, mask: Optional[torch.Tensor], w: TrimulPacked, outgoing: bool,
                 residual: bool = True, out: Optional[torch.Tensor] = None,
                 workspace: Optional[dict] = None) -> torch.Tensor:
    """z: bf16 [N, N, 128] contiguous; mask: [N, N] or None.  Three launches: projection ->
    batched tcgen05 contraction -> output stage."""
    if z.dtype != torch.bfloat16 or z.dim() != 3 or z.shape[-1] != 128 or not z.is_contiguous():
        raise ValueError("trimul_fused expects a contiguous bf16 [N, N, 128] tensor")
    N = z.shape[0]
    Np = ceil_to(N, 8)
    dev = z.device
    ws = workspace if workspace is not None else {}
    key = ("trimul", N, dev)
    if key not in ws:
        ws[key] = (torch.empty((2, 128, N, Np), dtype=torch.bfloat16, device=dev),
                   torch.empty((128, N, Np), dtype=torch.bfloat16, device=dev))
    planes, x = ws[key]
    st = native.status_tensor(dev)
    stream = native.current_stream(dev)
    m = None
    if mask is not None:
        m = mask.to(torch.float32).contiguous()
    rc = native.lib().ubm_trimul_proj(native.ptr(z), native.ptr(w.w_in), native.ptr(w.in_colsum),
                                      native.ptr(w.in_colbias), native.ptr(m), native.ptr(planes), 0, N, Np,
                                      native.ptr(st), stream)
    native.check(rc, "ubm_trimul_proj")
    _gemm.gemm(planes[0][:, :, :N], planes[1][:, :, :N], mn_major=not outgoing, out=x[:, :, :N])
    out = torch.empty_like(z) if out is None else out
    rc = native.lib().ubm_trimul_out(native.ptr(x), native.ptr(z), native.ptr(w.wo), native.ptr(w.wg),
                                     native.ptr(w.o_colsum), native.ptr(w.o_colbias), native.ptr(w.g_colsum),
                                     native.ptr(w.g_colbias), native.ptr(out), N, Np, 1 if residual else 0,
                                     native.ptr(st), stream)
    native.check(rc, "ubm_trimul_out")
    return out
