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
# row-block forms (also the per-rank forms of the row-sharded pair stack)
native.declare("ubm_trimul_proj_rows", [c_void_p] * 7 + [c_int, c_int, c_int, c_int, c_void_p, c_void_p])
native.declare("ubm_triatt_proj_rows", [c_void_p] * 13 + [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
native.declare("ubm_trimul_out_rows", [c_void_p] * 9 + [c_int, c_int, c_int, c_int, c_void_p, c_void_p])


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


def _trimul_blocked(z, m, w: TrimulPacked, outgoing: bool, residual: bool, out, ws: dict, rb: int):
    """Row-blocked triangle multiplication: the projected operand planes a, b exist whole (the contraction of a
    row block needs every row of the other operand), the contracted planes x only for ``rb`` rows of the update
    at a time - contraction and output stage alternate per block.  Same kernels, same sums as the whole form."""
    N = z.shape[0]
    Np = ceil_to(N, 8)
    dev = z.device
    key = ("trimul_blocked", N, rb, dev)
    if key not in ws:
        ws[key] = (torch.empty((2, 128, N, Np), dtype=torch.bfloat16, device=dev),
                   torch.empty((128, rb, Np), dtype=torch.bfloat16, device=dev))
    planes, xb = ws[key]
    st = native.status_tensor(dev)
    stream = native.current_stream(dev)
    lib = native.lib()
    rc = lib.ubm_trimul_proj(native.ptr(z), native.ptr(w.w_in), native.ptr(w.in_colsum), native.ptr(w.in_colbias),
                             native.ptr(m), native.ptr(planes), 0, N, Np, native.ptr(st), stream)
    native.check(rc, "ubm_trimul_proj")
    out = torch.empty_like(z) if out is None else out
    for r0 in range(0, N, rb):
        r1 = min(N, r0 + rb)
        xv = xb.view(-1)[: 128 * (r1 - r0) * Np].view(128, r1 - r0, Np)
        if outgoing:      # x[c, i, j] = sum_k a[c, i, k] b[c, j, k]: rows i of a against all of b
            _gemm.gemm(planes[0][:, r0:r1, :N], planes[1][:, :, :N], out=xv[:, :, :N])
        else:             # x[c, i, j] = sum_k a[c, k, i] b[c, k, j]: columns i of a (MN-major operands)
            _gemm.gemm(planes[0][:, :, r0:r1], planes[1][:, :, :N], mn_major=True, out=xv[:, :, :N])
        rc = lib.ubm_trimul_out_rows(native.ptr(xv), native.ptr(z[r0:r1]), native.ptr(w.wo), native.ptr(w.wg),
                                     native.ptr(w.o_colsum), native.ptr(w.o_colbias), native.ptr(w.g_colsum),
                                     native.ptr(w.g_colbias), native.ptr(out[r0:r1]), r1 - r0, N, Np,
                                     1 if residual else 0, native.ptr(st), stream)
        native.check(rc, "ubm_trimul_out_rows")
    return out


def trimul_fused(z: torch.Tensor, mask: Optional[torch.Tensor], w: TrimulPacked, outgoing: bool,
                 residual: bool = True, out: Optional[torch.Tensor] = None,
                 workspace: Optional[dict] = None) -> torch.Tensor:
    """z: bf16 [N, N, 128] contiguous; mask: [N, N] or None.  Three launches: projection ->
    batched tcgen05 contraction -> output stage.  With ``workspace["row_block"]`` set (the ``chunk_pair_ops`` lever)
    and smaller than N, contraction and output stage run per block of rows (see :func:`_trimul_blocked`)."""
    if z.dtype != torch.bfloat16 or z.dim() != 3 or z.shape[-1] != 128 or not z.is_contiguous():
        raise ValueError("trimul_fused expects a contiguous bf16 [N, N, 128] tensor")
    N = z.shape[0]
    Np = ceil_to(N, 8)
    dev = z.device
    ws = workspace if workspace is not None else {}
    rb = int(ws.get("row_block", 0) or 0)
    if 0 < rb < N:
        m = None if mask is None else mask.to(torch.float32).contiguous()
        return _trimul_blocked(z, m, w, outgoing, residual, out, ws, rb // 8 * 8 or 8)
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


# ------------------------------------------------------------------------------------------
_ATTN_SIG = [c_void_p] * 8 + [c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_ll, c_int, c_void_p, c_void_p]
native.declare("ubm_attention_d32", _ATTN_SIG)
native.declare("ubm_attention_d64", _ATTN_SIG)

native.declare("ubm_attention_set_variant", [c_int])

LOG2E = 1.4426950408889634


def set_attention_variant(v: int) -> None:
    """Low nibble, head dimension 32: 0 = choose by row count (four rows per CTA from four rows on), 5 = two rows
    with 128-key steps, 1 = two rows, P and bias through shared memory.  Bits 4-5: 0 = one exponential in four as a
    polynomial on the FMA pipe, 1 = all on the special-function unit."""
    native.lib().ubm_attention_set_variant(int(v))


MASK_STEP = 64          # the kernel's flags are per 64-key step
MASK_NEG = -1.0e30


@dataclass
class KeyMask:
    """A key mask laid out for the attention kernel: additive bf16 rows (0 keeps, -1e30 masks) padded to whole
    64-key steps, and one flag byte per (row, step) that is set when the step holds a masked key, so that rows and
    steps without masked keys run the mask-free loop (the reference skips the mask the same way for unmasked row
    groups: common/opt_core/opt_core/kernels/flash_triattn.py:35-37)."""
    add: torch.Tensor        # bf16 [rows, ld]
    flags: torch.Tensor      # uint8 [rows, ld / 64]

    @classmethod
    def pack(cls, keep: torch.Tensor) -> Optional["KeyMask"]:
        """keep: [rows, Nk], non-zero = attend.  Returns None when nothing is masked (one host read)."""
        keep = keep != 0
        if bool(keep.all()):
            return None
        rows, nk = keep.shape
        ld = ceil_to(nk, MASK_STEP)
        add = torch.zeros((rows, ld), dtype=torch.bfloat16, device=keep.device)
        add[:, :nk].masked_fill_(~keep, MASK_NEG)
        flags = (add.view(rows, ld // MASK_STEP, MASK_STEP) != 0).any(-1).to(torch.uint8).contiguous()
        return cls(add, flags)


@dataclass
class TriattPacked:
    w: torch.Tensor          # bf16 [512, 128] rows [q * log2e/sqrt(d); k; v; g], gamma folded
    colsum: torch.Tensor     # fp32 [512]
    colbias: torch.Tensor
    wb: torch.Tensor         # fp32 [H, 128] head-bias weights * gamma * log2e
    wb_colsum: torch.Tensor  # fp32 [H]
    wb_colbias: torch.Tensor
    wo: torch.Tensor         # bf16 [128, 128]
    bo: Optional[torch.Tensor]
    heads: int
    raw_bias: tuple = ()     # (ln_w, ln_b, w_bias) as given: the row-blocked form computes the bias planes first

    @classmethod
    def pack(cls, ln_w, ln_b, w_bias, w_q, w_k, w_v, w_g, b_g, w_o, b_o, heads: int) -> "TriattPacked":
        c = w_q.shape[1]
        if c != 128 or w_q.shape[0] != 128 or heads * 32 != 128:
            raise ValueError("fused triangle attention supports c_z = 128 and 4 heads of 32")
        qs = LOG2E / (32 ** 0.5)
        wq, sq, bq = fold_ln_linear(w_q, ln_w, ln_b, scale=qs)
        wk, sk, bk = fold_ln_linear(w_k, ln_w, ln_b)
        wv, sv, bv = fold_ln_linear(w_v, ln_w, ln_b)
        wg, sg, bg = fold_ln_linear(w_g, ln_w, ln_b, bias=b_g)
        w = torch.cat([wq, wk, wv, wg], 0).contiguous()
        colsum = torch.cat([sq, sk, sv, sg]).contiguous()
        colbias = torch.cat([bq, bk, bv, bg]).contiguous()
        gam = torch.ones(c, device=w_q.device) if ln_w is None else ln_w.detach().float()
        wb = (w_bias.detach().float() * gam[None, :] * LOG2E).contiguous()
        wb_colsum = wb.sum(1).contiguous()
        wb_colbias = torch.zeros(heads, device=w_q.device)
        if ln_b is not None:
            wb_colbias = (w_bias.detach().float() @ ln_b.detach().float()) * LOG2E
        return cls(w, colsum, colbias, wb, wb_colsum, wb_colbias.contiguous(),
                   w_o.detach().to(torch.bfloat16).contiguous(),
                   None if b_o is None else b_o.detach().float().contiguous(), heads, (ln_w, ln_b, w_bias))


def attention(q, k, v, bias, gate, out, rows: int, Nq: int, Nk: int, H: int, D: int = 32, ldb: int = 0,
              ld_in: int = 0, transpose_out: bool = False, ld_gate: int = 0, mask: Optional[KeyMask] = None):
    """Raw launch of the tcgen05 attention kernel (see csrc/attention_sm100.cu for the layout).
    D is the (padded) head dimension, 32 or 64; ld_in the row stride of q / k / v in elements, ld_gate that of
    the gate (0 = H * D); mask a :class:`KeyMask` over [rows, Nk] or None."""
    st = native.status_tensor(q.device)
    fn = native.lib().ubm_attention_d32 if D == 32 else native.lib().ubm_attention_d64
    if D not in (32, 64):
        raise ValueError("attention kernel supports head dimensions 32 and 64 (pad smaller heads)")
    if mask is not None and (mask.add.shape[0] != rows or mask.add.shape[1] < Nk):
        raise ValueError(f"key mask of shape {tuple(mask.add.shape)} does not cover [{rows}, {Nk}]")
    rc = fn(native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(bias), native.ptr(gate), native.ptr(out),
            native.ptr(None if mask is None else mask.add), native.ptr(None if mask is None else mask.flags), rows,
            Nq, Nk, H, ldb, ld_in, ld_gate, 0 if mask is None else mask.add.stride(0), 1 if transpose_out else 0,
            native.ptr(st), native.current_stream(q.device))
    native.check(rc, f"ubm_attention_d{D}")
    return out


def attention_d32(q, k, v, bias, gate, out, rows, Nq, Nk, H, ldb: int = 0, transpose_out: bool = False,
                  mask: Optional[KeyMask] = None):
    return attention(q, k, v, bias, gate, out, rows, Nq, Nk, H, 32, ldb, 0, transpose_out, mask=mask)


@dataclass
class ApbPacked:
    """Weights of attention-with-pair-bias for the fused path: heads padded to the kernel's head
    dimension (zero rows / columns), q scaled by log2(e)/sqrt(d), q|k|v stacked into one projection."""
    wqkv: torch.Tensor      # bf16 [3*H*Dp, c]
    bqkv: torch.Tensor      # fp32 [3*H*Dp]
    wg: torch.Tensor        # bf16 [H*Dp, c]
    wqkvg: torch.Tensor     # bf16 [4*H*Dp, c]: q|k|v|gate in one projection (sigmoid on the last quarter)
    bqkvg: torch.Tensor     # fp32 [4*H*Dp]
    wo: torch.Tensor        # bf16 [c, H*Dp]
    H: int
    Dp: int

    @classmethod
    def pack(cls, w_q, b_q, w_k, w_v, w_g, w_o, heads: int) -> "ApbPacked":
        c_out, c = w_q.shape
        D = c_out // heads
        Dp = 32 if D <= 32 else 64
        if D > 64:
            raise ValueError("head dimension above 64 is not supported by the attention kernel")

        def pad_rows(W, scale=1.0):
            Wp = torch.zeros((heads, Dp, W.shape[1]), dtype=torch.float32, device=W.device)
            Wp[:, :D] = W.detach().float().view(heads, D, -1) * scale
            return Wp.view(heads * Dp, -1)

        qs = LOG2E / (D ** 0.5)
        wqkv = torch.cat([pad_rows(w_q, qs), pad_rows(w_k), pad_rows(w_v)], 0).to(torch.bfloat16).contiguous()
        bq = torch.zeros((heads, Dp), device=w_q.device)
        if b_q is not None:
            bq[:, :D] = b_q.detach().float().view(heads, D) * qs
        bqkv = torch.cat([bq.view(-1), torch.zeros(2 * heads * Dp, device=w_q.device)]).contiguous()
        wg = pad_rows(w_g).to(torch.bfloat16).contiguous()
        wo = torch.zeros((w_o.shape[0], heads, Dp), dtype=torch.float32, device=w_o.device)
        wo[:, :, :D] = w_o.detach().float().view(w_o.shape[0], heads, D)
        wqkvg = torch.cat([wqkv, wg], 0).contiguous()
        bqkvg = torch.cat([bqkv, torch.zeros(heads * Dp, device=w_q.device)]).contiguous()
        return cls(wqkv, bqkv, wg, wqkvg, bqkvg,
                   wo.view(w_o.shape[0], heads * Dp).to(torch.bfloat16).contiguous(), heads, Dp)


def apb_fused(x: torch.Tensor, w: ApbPacked, bias_planes: torch.Tensor, ldb: int,
              out_gate: Optional[torch.Tensor] = None, out_residual: Optional[torch.Tensor] = None,
              mask: Optional[KeyMask] = None) -> torch.Tensor:
    """Gated attention with pair bias on rows x: bf16 [B, N, c]; bias_planes: bf16 [H, N, ldb] holding
    log2(e) * bias (shared by the B rows); mask: key mask over [B, N] or None.
    Returns proj_o(sigmoid(proj_g x) * attention) as [B, N, c];
    with ``out_gate`` ([N, c], shared by the B rows) and ``out_residual`` ([B*N, c]) the output projection's
    epilogue returns residual + gate * projection."""
    B, N, c = x.shape
    HD = w.H * w.Dp
    x2 = x.reshape(B * N, c)
    # q | k | v | gate from one GEMM (sigmoid on the gate columns); the attention kernel reads all four as column
    # slices of its output
    qkvg = _gemm.gemm(x2, w.wqkvg, bias=w.bqkvg, act="sigmoid", act_from=3 * HD)
    o = torch.empty((B * N, HD), dtype=torch.bfloat16, device=x.device)
    attention(qkvg[:, :HD], qkvg[:, HD:2 * HD], qkvg[:, 2 * HD:3 * HD], bias_planes, qkvg[:, 3 * HD:], o, rows=B,
              Nq=N, Nk=N, H=w.H, D=w.Dp, ldb=ldb, ld_in=4 * HD, ld_gate=4 * HD, mask=mask)
    return _gemm.gemm(o, w.wo, gate=out_gate, residual=out_residual).view(B, N, -1)


def _triatt_blocked(z, w: TriattPacked, starting: bool, residual: bool, out, ws: dict, mask, rb: int):
    """Row-blocked triangle attention: the per-head bias planes of the whole pair tensor first (one pass of a row
    kernel; transposed for the ending node), then projection -> attention -> output projection for ``rb``
    attention rows at a time, so q | k | v | gate | o exist for one block only.  For the ending node an attention
    row is a column of z: the block's columns are gathered to rows before the projection and the update is
    added back to those columns."""
    from . import rows as _rows
    N = z.shape[0]
    Np = ceil_to(N, 8)
    dev = z.device
    key = ("triatt_blocked", N, rb, dev)
    if key not in ws:
        ws[key] = (torch.empty((5, rb * N, 128), dtype=torch.bfloat16, device=dev),
                   torch.zeros((w.heads, N, Np), dtype=torch.bfloat16, device=dev),
                   torch.zeros((w.heads, rb, Np), dtype=torch.bfloat16, device=dev))
    qkvgo, hb, hb_scratch = ws[key]
    ln_w, ln_b, w_bias = w.raw_bias
    _rows.pair_head_bias(z, ln_w, ln_b, w_bias, scale=LOG2E, transpose=not starting, out=hb)
    st = native.status_tensor(dev)
    stream = native.current_stream(dev)
    lib = native.lib()
    out = torch.empty_like(z) if out is None else out
    for r0 in range(0, N, rb):
        r1 = min(N, r0 + rb)
        R = r1 - r0
        src = z[r0:r1] if starting else z[:, r0:r1].transpose(0, 1).contiguous()
        q, k, v, g, og = (qkvgo[i][: R * N] for i in range(5))
        rc = lib.ubm_triatt_proj_rows(native.ptr(src), native.ptr(w.w), native.ptr(w.colsum), native.ptr(w.colbias),
                                      native.ptr(w.wb), native.ptr(w.wb_colsum), native.ptr(w.wb_colbias),
                                      native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(g),
                                      native.ptr(hb_scratch), 0, R, rb, N, Np, w.heads, 0, native.ptr(st), stream)
        native.check(rc, "ubm_triatt_proj_rows")
        km = None if mask is None else KeyMask(mask.add[r0:r1], mask.flags[r0:r1])
        attention_d32(q, k, v, hb, g, og, rows=R, Nq=N, Nk=N, H=w.heads, ldb=Np, mask=km)
        if starting:
            _gemm.gemm(og, w.wo, bias=w.bo, residual=z[r0:r1].view(R * N, 128) if residual else None,
                       out=out[r0:r1].view(R * N, 128))
        else:
            upd = _gemm.gemm(og, w.wo, bias=w.bo).view(R, N, 128).transpose(0, 1)
            out[:, r0:r1] = (z[:, r0:r1] + upd) if residual else upd
    return out


def triangle_attention_fused(z: torch.Tensor, w: TriattPacked, starting: bool, residual: bool = True,
                             out: Optional[torch.Tensor] = None, workspace: Optional[dict] = None,
                             mask: Optional[KeyMask] = None) -> torch.Tensor:
    """z: bf16 [N, N, 128] contiguous; mask: key mask over [attention row, key] (for the ending node the
    attention rows are the columns of z, so the caller packs the transposed pair mask).  Three launches:
    projection (LN folded, q|k|v|gate rows + head bias planes, written at the transposed pair index for the
    ending node) -> attention -> output projection with residual."""
    if z.dtype != torch.bfloat16 or z.dim() != 3 or z.shape[-1] != 128 or not z.is_contiguous():
        raise ValueError("triangle_attention_fused expects a contiguous bf16 [N, N, 128] tensor")
    N = z.shape[0]
    Np = ceil_to(N, 8)
    dev = z.device
    ws = workspace if workspace is not None else {}
    rb = int(ws.get("row_block", 0) or 0)
    if 0 < rb < N:
        return _triatt_blocked(z, w, starting, residual, out, ws, mask, rb)
    key = ("triatt", N, dev)
    if key not in ws:
        ws[key] = (torch.empty((5, N * N, 128), dtype=torch.bfloat16, device=dev),
                   torch.zeros((w.heads, N, Np), dtype=torch.bfloat16, device=dev))
    qkvgo, hb = ws[key]
    q, k, v, g, og = qkvgo[0], qkvgo[1], qkvgo[2], qkvgo[3], qkvgo[4]
    st = native.status_tensor(dev)
    stream = native.current_stream(dev)
    rc = native.lib().ubm_triatt_proj(native.ptr(z), native.ptr(w.w), native.ptr(w.colsum), native.ptr(w.colbias),
                                      native.ptr(w.wb), native.ptr(w.wb_colsum), native.ptr(w.wb_colbias),
                                      native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(g), native.ptr(hb), 0,
                                      N, Np, w.heads, 0 if starting else 1, native.ptr(st), stream)
    native.check(rc, "ubm_triatt_proj")
    attention_d32(q, k, v, hb, g, og, rows=N, Nq=N, Nk=N, H=w.heads, ldb=Np, transpose_out=not starting, mask=mask)
    z2 = z.view(N * N, 128)
    out = torch.empty_like(z) if out is None else out
    _gemm.gemm(og, w.wo, bias=w.bo, residual=z2 if residual else None, out=out.view(N * N, 128))
    return out


# ------------------------------------------------------------------------------------------
native.declare("ubm_window_attention", [c_void_p] * 6 + [c_int, c_int, c_int, c_ll, c_int, c_void_p])
native.declare("ubm_window_attention_tc", [c_void_p] * 6 + [c_int, c_int, c_int, c_ll, c_int, c_void_p, c_void_p])

WINDOW_KERNEL = "tc"     # "tc": tcgen05 kernel (four windows per CTA); "simt": CUDA-core kernel (one window per CTA)


def window_attention_fused(x: torch.Tensor, w: ApbPacked, bias: Optional[torch.Tensor],
                           out_gate: Optional[torch.Tensor] = None,
                           out_residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gated atom attention in 32 x 128 windows.  x: bf16 [B, A, c] (A a multiple of 32); w: packed projections with
    4 x 32 heads; bias: bf16 [1 or B, H, A/32, 32, 128] already multiplied by log2(e).  Returns [B, A, c]."""
    B, A, c = x.shape
    if w.Dp != 32:
        raise ValueError("window attention supports head dimension 32")
    HD = w.H * 32
    x2 = x.reshape(B * A, c)
    qkv = _gemm.gemm(x2, w.wqkv, bias=w.bqkv)
    g = _gemm.gemm(x2, w.wg, act="sigmoid")
    o = torch.empty((B * A, HD), dtype=torch.bfloat16, device=x.device)
    if WINDOW_KERNEL == "tc":
        rc = native.lib().ubm_window_attention_tc(native.ptr(qkv), native.ptr(qkv) + HD * 2,
                                                  native.ptr(qkv) + 2 * HD * 2, native.ptr(bias), native.ptr(g),
                                                  native.ptr(o), B, A, w.H, 3 * HD,
                                                  1 if bias is None else bias.shape[0],
                                                  native.ptr(native.status_tensor(x.device)),
                                                  native.current_stream(x.device))
        native.check(rc, "ubm_window_attention_tc")
    else:
        rc = native.lib().ubm_window_attention(native.ptr(qkv), native.ptr(qkv) + HD * 2,
                                               native.ptr(qkv) + 2 * HD * 2, native.ptr(bias), native.ptr(g),
                                               native.ptr(o), B, A, w.H, 3 * HD,
                                               1 if bias is None else bias.shape[0], native.current_stream(x.device))
        native.check(rc, "ubm_window_attention")
    return _gemm.gemm(o, w.wo, gate=out_gate, residual=out_residual).view(B, A, -1)
