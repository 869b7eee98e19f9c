"""Pairformer stack (AF3 / Boltz-2 family) with the upstream parameter names.

Module and parameter names follow Boltz-2 so its checkpoints load unchanged
(boltz2/stock/src/boltz/model/layers/pairformer.py:41-62 ``pre_norm_s, attention, tri_mul_out,
tri_mul_in, tri_att_start, tri_att_end, transition_s, transition_z``; triangular_mult.py:49-54;
transition.py; attentionv2.py; triangular_attention/attention.py:44-50).  Every module has two
forwards: the plain statement (``ops.reference``, the ``off`` path and the CPU oracle) and the
fused sm_100a path (``ops.pair``) that a mode's levers switch on per module through
:func:`set_impl`.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import reference as R

IMPLS = ("reference", "fused")


class _Switchable(nn.Module):
    """A module with a per-instance implementation word and a lazily packed weight cache."""

    impl: str = "reference"
    lever: str = ""          # the lever whose ledger counts this module's calls (ops.dispatch.LEVERS)

    def __init__(self):
        super().__init__()
        self.impl = "reference"
        self._packed = None
        self._workspace: Optional[dict] = None

    def _decide(self, reason: Optional[str], klass: Optional[str] = None, tokens: Optional[int] = None,
                call: Optional[dict] = None, row: Optional[str] = None) -> bool:
        """Under the kernel implementation every call is decided and counted before it runs: ``reason`` None =
        the kernel serves, otherwise the plain statement runs as ``fallback:<reason>`` in the lever's ledger (an
        undeclared reason ends the run PARTIAL).  With the plain implementation there is nothing to count."""
        if self.impl != "fused":
            return False
        from ..ops import dispatch
        return dispatch.decide(self.lever, reason, klass, tokens, call, row)

    @staticmethod
    def _tensor_reason(x: torch.Tensor) -> Optional[str]:
        if not x.is_cuda:
            return "not_cuda"
        if x.dtype != torch.bfloat16:
            return f"dtype_{str(x.dtype).replace('torch.', '')}"
        return None

    def set_impl(self, impl: str, workspace: Optional[dict] = None):
        if impl not in IMPLS:
            raise ValueError(f"impl {impl!r} not in {IMPLS}")
        self.impl = impl
        self._packed = None
        self._workspace = workspace

    def _fusable(self, z: torch.Tensor) -> bool:
        return (self.impl == "fused" and z.is_cuda and z.dtype == torch.bfloat16 and z.shape[-1] == 128)


class Transition(_Switchable):
    """SwiGLU transition: ``fc3(silu(fc1 n) * fc2 n)``, n = LN(x)."""

    def __init__(self, dim: int, hidden: Optional[int] = None, out_dim: Optional[int] = None):
        super().__init__()
        hidden = hidden or 4 * dim
        out_dim = out_dim or dim
        self.norm = nn.LayerNorm(dim, eps=1e-5)
        self.fc1 = nn.Linear(dim, hidden, bias=False)
        self.fc2 = nn.Linear(dim, hidden, bias=False)
        self.fc3 = nn.Linear(hidden, out_dim, bias=False)
        self.dim, self.hidden, self.out_dim = dim, hidden, out_dim

    lever = "fused_transition"

    def forward(self, x: torch.Tensor, residual: bool = False) -> torch.Tensor:
        one_kernel = self.dim == 128 and self.out_dim == 128 and self.hidden % 64 == 0 and self.hidden <= 1024
        rows_ok = self.dim % 8 == 0 and self.dim <= 1024 and self.hidden % 8 == 0 and self.out_dim % 8 == 0
        why = self._tensor_reason(x) or (None if (one_kernel or rows_ok) else f"width_{self.dim}x{self.hidden}")
        tokens = x.shape[-2]
        served = self._decide(why, f"C{self.dim}X{max(1, self.hidden // max(1, self.dim))}", tokens,
                              {"c": self.dim, "expansion": self.hidden // max(1, self.dim), "dtype": "bf16"},
                              "tcgen05_fused" if one_kernel else "rows_gemm")
        if served and one_kernel:
            from ..ops import pair
            if self._packed is None:
                self._packed = pair.TransitionPacked.pack(self.norm.weight, self.norm.bias, self.fc1.weight,
                                                          self.fc2.weight, self.fc3.weight)
            return pair.transition_fused(x.contiguous(), self._packed, residual=residual)
        if served:
            # other widths (the MSA track at 64, the template stack): LayerNorm rows -> one GEMM for both hidden
            # projections -> SwiGLU rows -> output GEMM with the residual in its epilogue
            from ..ops import gemm, rows
            in_epilogue = self.hidden % 32 == 0     # silu(fc1) * fc2 formed on the accumulator of one product
            if self._packed is None:
                w12 = gemm.pack_swiglu(self.fc1.weight.detach(), self.fc2.weight.detach()) if in_epilogue else \
                    torch.cat([self.fc1.weight, self.fc2.weight], 0).detach().to(torch.bfloat16).contiguous()
                self._packed = (w12, self.fc3.weight.detach().to(torch.bfloat16).contiguous())
            w12, w3 = self._packed
            x2 = x.reshape(-1, self.dim).contiguous()
            n = rows.layernorm_rows(x2, self.norm.weight, self.norm.bias, self.norm.eps)
            h = gemm.gemm(n, w12, act="swiglu") if in_epilogue else rows.swiglu_rows(gemm.gemm(n, w12))
            y = gemm.gemm(h, w3, residual=x2 if residual and self.out_dim == self.dim else None)
            return y.view(*x.shape[:-1], self.out_dim)
        return R.transition(x, self.norm.weight, self.norm.bias, self.fc1.weight, self.fc2.weight, self.fc3.weight,
                            residual=residual)


class TriangleMultiplication(_Switchable):
    def __init__(self, dim: int = 128, outgoing: bool = True):
        super().__init__()
        self.outgoing = outgoing
        self.norm_in = nn.LayerNorm(dim, eps=1e-5)
        self.p_in = nn.Linear(dim, 2 * dim, bias=False)
        self.g_in = nn.Linear(dim, 2 * dim, bias=False)
        self.norm_out = nn.LayerNorm(dim)
        self.p_out = nn.Linear(dim, dim, bias=False)
        self.g_out = nn.Linear(dim, dim, bias=False)

    lever = "fused_trimul"

    def _rows_gemm_forward(self, z: torch.Tensor, mask: Optional[torch.Tensor], residual: bool) -> torch.Tensor:
        """Widths other than 128 (the template stack at 64, the ESM family at 256): LayerNorm rows -> one tcgen05
        GEMM for [p_in; g_in] with the sigmoid on the gate half in its epilogue -> channel-major operand planes ->
        the batched contraction GEMM (K-major for outgoing, MN-major for incoming) -> LayerNorm rows -> output GEMM
        whose epilogue applies the output gate and the residual.  Gating products and the two layout changes are
        plain tensor statements."""
        from ..ops import gemm, rows
        N, c = z.shape[1], z.shape[-1]
        h = self.p_in.weight.shape[0] // 2
        if self._packed is None:
            bf = lambda t: t.detach().to(torch.bfloat16).contiguous()  # noqa: E731
            self._packed = (bf(torch.cat([self.p_in.weight, self.g_in.weight], 0)), bf(self.g_out.weight),
                            bf(self.p_out.weight))
        w_in, w_go, w_po = self._packed
        x = z[0].reshape(N * N, c).contiguous()
        n = rows.layernorm_rows(x, self.norm_in.weight, self.norm_in.bias, self.norm_in.eps)
        pg = gemm.gemm(n, w_in, act="sigmoid", act_from=2 * h)                      # [N^2, 4h] = p | sigmoid(g)
        ab = pg[:, :2 * h] * pg[:, 2 * h:]
        if mask is not None:
            ab = ab * mask[0].reshape(N * N, 1).to(ab.dtype)
        Np = (N + 7) // 8 * 8
        planes = torch.zeros((2, h, N, Np), dtype=torch.bfloat16, device=z.device)
        planes[0, :, :, :N] = ab[:, :h].reshape(N, N, h).permute(2, 0, 1)
        planes[1, :, :, :N] = ab[:, h:].reshape(N, N, h).permute(2, 0, 1)
        xc = torch.zeros((h, N, Np), dtype=torch.bfloat16, device=z.device)
        gemm.gemm(planes[0][:, :, :N], planes[1][:, :, :N], mn_major=not self.outgoing, out=xc[:, :, :N])
        xr = xc[:, :, :N].permute(1, 2, 0).reshape(N * N, h).contiguous()
        xn = rows.layernorm_rows(xr, self.norm_out.weight, self.norm_out.bias, self.norm_out.eps)
        go = gemm.gemm(n, w_go, act="sigmoid")
        out = gemm.gemm(xn, w_po, gate=go, residual=x if residual else None)
        return out.view(1, N, N, c)

    def forward(self, z: torch.Tensor, mask: Optional[torch.Tensor], residual: bool = False) -> torch.Tensor:
        c = z.shape[-1]
        h2 = self.p_in.weight.shape[0]
        one_kernel_set = c == 128 and h2 == 256
        rows_ok = c % 32 == 0 and h2 % 64 == 0 and c <= 1024
        why = self._tensor_reason(z) or (None if (one_kernel_set or rows_ok) else f"width_{c}x{h2 // 2}") \
            or (f"batch_{z.shape[0]}" if z.shape[0] != 1 else None)
        served = self._decide(why, f"C{c}H{h2 // 2}", z.shape[1],
                              {"c_z": c, "c_hidden": h2 // 2, "dtype": "bf16"},
                              "tcgen05_3stage" if one_kernel_set else "rows_gemm")
        if served and not one_kernel_set:
            return self._rows_gemm_forward(z, mask, residual)
        if served:
            from ..ops import pair
            if self._packed is None:
                self._packed = pair.TrimulPacked.pack(self.norm_in.weight, self.norm_in.bias, self.p_in.weight,
                                                      self.g_in.weight, self.norm_out.weight, self.norm_out.bias,
                                                      self.p_out.weight, self.g_out.weight)
            m = None if mask is None else mask[0]
            out = pair.trimul_fused(z[0].contiguous(), m, self._packed, self.outgoing, residual=residual,
                                    workspace=self._workspace)
            return out.unsqueeze(0)
        return R.triangle_multiplication(z, mask, self.norm_in.weight, self.norm_in.bias, self.p_in.weight,
                                         self.g_in.weight, self.norm_out.weight, self.norm_out.bias,
                                         self.p_out.weight, self.g_out.weight, outgoing=self.outgoing,
                                         residual=residual)


class TriangleMultiplicationOutgoing(TriangleMultiplication):
    def __init__(self, dim: int = 128):
        super().__init__(dim, outgoing=True)


class TriangleMultiplicationIncoming(TriangleMultiplication):
    def __init__(self, dim: int = 128):
        super().__init__(dim, outgoing=False)


class _MHA(nn.Module):
    """Parameter holder with the OpenFold attention names used by Boltz-2's triangle attention.  Boltz-2 keeps no
    bias on the gate and output projections (boltz2/stock/src/boltz/model/layers/triangular_attention/
    primitives.py:259-267); ``bias=True`` gives the OpenFold / AF3-family form that has them."""

    def __init__(self, c_in: int, c_hidden: int, heads: int, bias: bool = False):
        super().__init__()
        self.linear_q = nn.Linear(c_in, c_hidden * heads, bias=False)
        self.linear_k = nn.Linear(c_in, c_hidden * heads, bias=False)
        self.linear_v = nn.Linear(c_in, c_hidden * heads, bias=False)
        self.linear_o = nn.Linear(c_hidden * heads, c_in, bias=bias)
        self.linear_g = nn.Linear(c_in, c_hidden * heads, bias=bias)


class TriangleAttention(_Switchable):
    def __init__(self, c_in: int = 128, c_hidden: int = 32, heads: int = 4, starting: bool = True):
        super().__init__()
        self.starting, self.heads, self.c_hidden = starting, heads, c_hidden
        self.layer_norm = nn.LayerNorm(c_in)
        self.linear = nn.Linear(c_in, heads, bias=False)
        self.mha = _MHA(c_in, c_hidden, heads)

    lever = "fused_triatt"

    def _rows_gemm_forward(self, z: torch.Tensor, mask: Optional[torch.Tensor], residual: bool) -> torch.Tensor:
        """Widths / head shapes other than 128 channels with 4 x 32: LayerNorm rows -> one tcgen05 GEMM for
        q | k | v | gate (heads padded to the kernel's head dimension 32 or 64, sigmoid on the gate columns) -> the
        attention kernel on column slices of that output with the head-bias planes and the key mask -> output GEMM
        with bias and residual.  The ending node runs on the transposed pair tensor (a tensor statement)."""
        from ..ops import gemm, pair, rows
        m = self.mha
        N, c = z.shape[1], z.shape[-1]
        H, D = self.heads, self.c_hidden
        if self._packed is None:
            w = pair.ApbPacked.pack(m.linear_q.weight, None, m.linear_k.weight, m.linear_v.weight, m.linear_g.weight,
                                    m.linear_o.weight, H)
            if m.linear_g.bias is not None:
                bg = torch.zeros((H, w.Dp), device=z.device)
                bg[:, :D] = m.linear_g.bias.detach().float().view(H, D)
                w.bqkvg[3 * H * w.Dp:] = bg.view(-1)
            self._packed = w
        w = self._packed
        HD = H * w.Dp
        src = z[0] if self.starting else z[0].transpose(0, 1)
        x = src.reshape(N * N, c).contiguous()
        n = rows.layernorm_rows(x, self.layer_norm.weight, self.layer_norm.bias, self.layer_norm.eps)
        qkvg = gemm.gemm(n, w.wqkvg, bias=w.bqkvg, act="sigmoid", act_from=3 * HD)
        Np = (N + 7) // 8 * 8
        hb = torch.zeros((H, N, Np), dtype=torch.bfloat16, device=z.device)
        hb[:, :, :N] = (F.linear(n, self.linear.weight.to(n.dtype)).float() * pair.LOG2E).view(N, N, H).permute(2, 0, 1)
        km = None
        if mask is not None:
            km = _cached_key_mask(self._workspace, mask[0], transposed=not self.starting)
        o = torch.empty((N * N, HD), dtype=torch.bfloat16, device=z.device)
        pair.attention(qkvg[:, :HD], qkvg[:, HD:2 * HD], qkvg[:, 2 * HD:3 * HD], hb, qkvg[:, 3 * HD:], o, rows=N, Nq=N,
                       Nk=N, H=H, D=w.Dp, ldb=Np, ld_in=4 * HD, ld_gate=4 * HD, mask=km)
        bo = None if m.linear_o.bias is None else m.linear_o.bias.float()
        upd = gemm.gemm(o, w.wo, bias=bo, residual=x if residual else None).view(N, N, c)
        if not self.starting:
            upd = upd.transpose(0, 1)
        return upd.unsqueeze(0)

    def forward(self, z: torch.Tensor, mask: Optional[torch.Tensor] = None, residual: bool = False) -> torch.Tensor:
        m = self.mha
        c = z.shape[-1]
        one_kernel_set = c == 128 and (self.heads, self.c_hidden) == (4, 32)
        rows_ok = c % 32 == 0 and c <= 1024 and self.c_hidden <= 64 and (self.heads * (32 if self.c_hidden <= 32 else 64)) % 32 == 0
        why = self._tensor_reason(z) or (None if (one_kernel_set or rows_ok) else
                                         f"shape_{c}_{self.heads}x{self.c_hidden}") \
            or (f"batch_{z.shape[0]}" if z.shape[0] != 1 else None)
        served = self._decide(why, f"D{self.c_hidden}H{self.heads}", z.shape[1],
                              {"head_dim": 32 if self.c_hidden <= 32 else 64, "dtype": "bf16"},
                              "tcgen05_4row" if one_kernel_set else "rows_gemm")
        if served and not one_kernel_set:
            return self._rows_gemm_forward(z, mask, residual)
        if served:
            from ..ops import pair
            km = None
            if mask is not None:
                km = _cached_key_mask(self._workspace, mask[0], transposed=not self.starting)
            if self._packed is None:
                self._packed = pair.TriattPacked.pack(self.layer_norm.weight, self.layer_norm.bias,
                                                      self.linear.weight, m.linear_q.weight, m.linear_k.weight,
                                                      m.linear_v.weight, m.linear_g.weight, m.linear_g.bias,
                                                      m.linear_o.weight, m.linear_o.bias, self.heads)
            out = pair.triangle_attention_fused(z[0].contiguous(), self._packed, self.starting, residual=residual,
                                                workspace=self._workspace, mask=km)
            return out.unsqueeze(0)
        outs = [R.triangle_attention(z[b], None if mask is None else mask[b], self.layer_norm.weight,
                                     self.layer_norm.bias, self.linear.weight, m.linear_q.weight, m.linear_k.weight,
                                     m.linear_v.weight, m.linear_g.weight, m.linear_g.bias, m.linear_o.weight,
                                     m.linear_o.bias, self.heads, starting=self.starting, residual=residual)
                for b in range(z.shape[0])]
        return torch.stack(outs, 0)


def _cached_key_mask(workspace: Optional[dict], mask: torch.Tensor, transposed: bool = False):
    """Key mask of the attention kernel for a [rows, keys] keep-mask, packed once per mask tensor: the same pair
    mask reaches every triangle attention of a stack, so the packed form is kept in the stack's workspace under the
    tensor's identity and version."""
    from ..ops import pair
    ws = workspace if workspace is not None else {}
    key = ("keymask", mask.data_ptr(), mask._version, tuple(mask.shape), transposed)
    if key not in ws:
        for k in [k for k in ws if isinstance(k, tuple) and k and k[0] == "keymask" and k[1] != mask.data_ptr()]:
            del ws[k]
        ws[key] = pair.KeyMask.pack(mask.t() if transposed else mask)
    return ws[key]


class TriangleAttentionStartingNode(TriangleAttention):
    def __init__(self, c_in=128, c_hidden=32, heads=4):
        super().__init__(c_in, c_hidden, heads, starting=True)


class TriangleAttentionEndingNode(TriangleAttention):
    def __init__(self, c_in=128, c_hidden=32, heads=4):
        super().__init__(c_in, c_hidden, heads, starting=False)


class BiasPlanes:
    """Pair bias laid out for the attention kernel: bf16 planes [H, N, ld] (ld a multiple of 8) that
    already carry the factor log2(e).  ``dense()`` gives the plain [1, H, N, N] bias back."""

    LOG2E = 1.4426950408889634

    def __init__(self, view: torch.Tensor):
        self.view = view                      # [H, N, N] view with stride(1) = ld
        self.ld = view.stride(1)

    def dense(self) -> torch.Tensor:
        return (self.view.float() / self.LOG2E).unsqueeze(0)


class AttentionPairBias(_Switchable):
    """Single-representation attention with a bias projected from the pair tensor."""

    def __init__(self, c_s: int = 384, c_z: int = 128, heads: int = 16, compute_pair_bias: bool = True):
        super().__init__()
        self.c_s, self.heads = c_s, heads
        self.head_dim = c_s // heads
        self.proj_q = nn.Linear(c_s, c_s)
        self.proj_k = nn.Linear(c_s, c_s, bias=False)
        self.proj_v = nn.Linear(c_s, c_s, bias=False)
        self.proj_g = nn.Linear(c_s, c_s, bias=False)
        self.compute_pair_bias = compute_pair_bias
        if compute_pair_bias:
            self.proj_z = nn.Sequential(nn.LayerNorm(c_z), nn.Linear(c_z, heads, bias=False))
        self.proj_o = nn.Linear(c_s, c_s, bias=False)

    lever = "fused_apb"

    def pair_bias(self, z: torch.Tensor):
        """[B, H, N, N] bias from the pair tensor (a :class:`BiasPlanes` on the fused path)."""
        if self._fusable(z) and z.shape[0] == 1:
            from ..ops import rows
            return BiasPlanes(rows.pair_head_bias(z[0].contiguous(), self.proj_z[0].weight, self.proj_z[0].bias,
                                                  self.proj_z[1].weight, scale=BiasPlanes.LOG2E))
        return self.proj_z[1](self.proj_z[0](z)).permute(0, 3, 1, 2)

    def _fused_forward(self, s: torch.Tensor, planes: "BiasPlanes", out_gate=None, out_residual=None,
                       mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        from ..ops import pair
        km = None
        if mask is not None:
            km = _cached_key_mask(self._workspace, mask if mask.shape[0] == s.shape[0] else
                                  mask.expand(s.shape[0], -1) if mask.shape[0] == 1 else
                                  mask.repeat_interleave(s.shape[0] // mask.shape[0], 0))
        if self._packed is None:
            self._packed = pair.ApbPacked.pack(self.proj_q.weight, self.proj_q.bias, self.proj_k.weight,
                                               self.proj_v.weight, self.proj_g.weight, self.proj_o.weight,
                                               self.heads)
        return pair.apb_fused(s.to(torch.bfloat16).contiguous(), self._packed, planes.view, planes.ld,
                              out_gate=out_gate, out_residual=out_residual, mask=km)

    def forward(self, s: torch.Tensor, z: Optional[torch.Tensor], mask: Optional[torch.Tensor],
                bias: Optional[torch.Tensor] = None, k_in: Optional[torch.Tensor] = None,
                multiplicity: int = 1) -> torch.Tensor:
        """s: [B*mult, N, c_s] already normalised by the caller; bias (if given) replaces proj_z(z)."""
        B, N, _ = s.shape
        kin = s if k_in is None else k_in
        if bias is None:
            bias = self.pair_bias(z)
        if self.impl == "fused":
            why = ("not_cuda" if not s.is_cuda else None) or ("cross_keys" if k_in is not None else None) \
                or (None if isinstance(bias, BiasPlanes) else "dense_bias") \
                or (f"head_dim_{self.head_dim}" if self.head_dim > 64 else None)
            Dp = 32 if self.head_dim <= 32 else 64
            if self._decide(why, f"D{Dp}H{self.heads}S{B}", N, {"head_dim": Dp, "dtype": "bf16"}):
                return self._fused_forward(s, bias, mask=mask).to(s.dtype)
        if isinstance(bias, BiasPlanes):
            bias = bias.dense()
        H, D = self.heads, self.head_dim
        q = self.proj_q(s).view(B, N, H, D).transpose(1, 2)
        k = self.proj_k(kin).view(B, kin.shape[1], H, D).transpose(1, 2)
        v = self.proj_v(kin).view(B, kin.shape[1], H, D).transpose(1, 2)
        g = torch.sigmoid(self.proj_g(s))
        b = bias[..., : kin.shape[1]].float()
        if multiplicity > 1:
            b = b.repeat_interleave(multiplicity, 0)
        if mask is not None:
            mm = mask if multiplicity == 1 else mask.repeat_interleave(multiplicity, 0)
            b = b + ((1.0 - mm.float()) * -1e6)[:, None, None, :]
        o = R.attention_with_bias(q, k, v, b)
        o = o.transpose(1, 2).reshape(B, N, H * D)
        return self.proj_o(g * o)


class PairformerLayer(nn.Module):
    def __init__(self, c_s: int = 384, c_z: int = 128, heads: int = 16, pair_heads: int = 4, no_seq: bool = False,
                 transition_n: int = 4):
        super().__init__()
        self.no_seq = no_seq
        if not no_seq:
            self.pre_norm_s = nn.LayerNorm(c_s)
            self.attention = AttentionPairBias(c_s, c_z, heads)
            self.transition_s = Transition(c_s, c_s * transition_n)
        self.tri_mul_out = TriangleMultiplicationOutgoing(c_z)
        self.tri_mul_in = TriangleMultiplicationIncoming(c_z)
        self.tri_att_start = TriangleAttentionStartingNode(c_z, c_z // pair_heads, pair_heads)
        self.tri_att_end = TriangleAttentionEndingNode(c_z, c_z // pair_heads, pair_heads)
        self.transition_z = Transition(c_z, c_z * transition_n)

    def pair_update(self, z: torch.Tensor, pair_mask: Optional[torch.Tensor]) -> torch.Tensor:
        z = self.tri_mul_out(z, pair_mask, residual=True)
        z = self.tri_mul_in(z, pair_mask, residual=True)
        z = self.tri_att_start(z, pair_mask, residual=True)
        z = self.tri_att_end(z, pair_mask, residual=True)
        z = self.transition_z(z, residual=True)
        return z

    def forward(self, s: Optional[torch.Tensor], z: torch.Tensor, mask: Optional[torch.Tensor],
                pair_mask: Optional[torch.Tensor]):
        z = self.pair_update(z, pair_mask)
        if self.no_seq:
            return s, z
        # single track in fp32, as upstream (pairformer.py:103-111)
        s32 = s.float()
        sn = F.layer_norm(s32, (s32.shape[-1],), self.pre_norm_s.weight.float(), self.pre_norm_s.bias.float())
        with torch.autocast(device_type=s.device.type, enabled=False):
            upd = _run_fp32(self.attention, sn, z, mask)
        s32 = s32 + upd
        s32 = s32 + _run_fp32(self.transition_s, s32)
        return s32.to(s.dtype), z


def _run_fp32(module: nn.Module, x: torch.Tensor, *args):
    """Run a module whose parameters may be bf16 on an fp32 activation (weights up-cast on the fly)."""
    p = next(module.parameters())
    if p.dtype == torch.float32:
        return module(x, *args)
    return module(x.to(p.dtype), *args).float()


class PairformerModule(nn.Module):
    def __init__(self, c_s: int = 384, c_z: int = 128, num_blocks: int = 48, heads: int = 16, pair_heads: int = 4,
                 no_seq: bool = False):
        super().__init__()
        self.layers = nn.ModuleList([PairformerLayer(c_s, c_z, heads, pair_heads, no_seq) for _ in range(num_blocks)])

    def forward(self, s, z, mask=None, pair_mask=None):
        for layer in self.layers:
            s, z = layer(s, z, mask, pair_mask)
        return s, z


def set_impl(module: nn.Module, impl: str, kinds=None, workspace: Optional[dict] = None) -> int:
    """Switch every :class:`_Switchable` below ``module`` (optionally only the given classes).
    All switched modules share one scratch workspace, so the pair stack's intermediates are
    allocated once per size.  Returns the number of modules switched."""
    ws = {} if workspace is None else workspace
    n = 0
    for m in module.modules():
        if isinstance(m, _Switchable) and (kinds is None or isinstance(m, tuple(kinds))):
            m.set_impl(impl, ws)
            n += 1
    return n
