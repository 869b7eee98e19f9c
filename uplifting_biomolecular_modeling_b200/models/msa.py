"""MSA module (AF3 / Boltz-2 family): outer-product mean, pair-weighted averaging, MSA transition
and a no-sequence Pairformer layer per block.

Names follow Boltz-2 (boltz2/stock/src/boltz/model/modules/trunkv2.py:512 ``MSAModule`` with
``s_proj, msa_proj, layers``; ``MSALayer:672`` = ``msa_transition, pair_weighted_averaging,
pairformer_layer, outer_product_mean``; layers/outer_product_mean.py ``norm, proj_a, proj_b,
proj_o``).  The fused path runs both contractions on the tcgen05 GEMM: the outer product as a
[N*c, S] x [S, N*c] product in row blocks so that the [N, N, c*c] tensor never exists whole (the
fusion boundary of the reference's ops.msa_opm, common/opt_core/opt_core/ops/msa_opm/__init__.py:106),
and the weighted average as one batched GEMM over heads (ops.msa_pwa, :40).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import reference as R
from .pairformer import PairformerLayer, Transition, _Switchable


class OuterProductMean(_Switchable):
    def __init__(self, c_in: int = 64, c_hidden: int = 32, c_out: int = 128):
        super().__init__()
        self.c_hidden = c_hidden
        self.norm = nn.LayerNorm(c_in)
        self.proj_a = nn.Linear(c_in, c_hidden, bias=False)
        self.proj_b = nn.Linear(c_in, c_hidden, bias=False)
        self.proj_o = nn.Linear(c_hidden * c_hidden, c_out)
        self.row_block = 128
        self.full_mask = False      # set by the caller when the MSA mask is known (on the host) to be all ones

    lever = "fused_opm"

    def forward(self, m: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        why = self._tensor_reason(m) or (f"batch_{m.shape[0]}" if m.shape[0] != 1 else None)
        if not self._decide(why, f"C{m.shape[-1]}H{self.c_hidden}S{m.shape[1]}", m.shape[2]):
            return R.outer_product_mean(m, mask, self.norm.weight, self.norm.bias, self.proj_a.weight,
                                        self.proj_b.weight, self.proj_o.weight, self.proj_o.bias)
        from ..ops import gemm, rows
        B, S, N, _ = m.shape
        c = self.c_hidden
        n = rows.layernorm_rows(m.contiguous(), self.norm.weight, self.norm.bias, self.norm.eps)
        mk = mask.unsqueeze(-1).to(n.dtype)
        # [S, N, c] seen as [S, N*c]: sequences (the contraction) along rows, (token, channel) contiguous - the
        # operand form of the MN-major GEMM, so no [N*c, S] transposed copies are made
        a2 = (self.proj_a(n) * mk)[0].reshape(S, N * c)
        b2 = (self.proj_b(n) * mk)[0].reshape(S, N * c)
        wo = self.proj_o.weight.to(torch.bfloat16).contiguous()
        bo = self.proj_o.bias.float()
        out = torch.empty((N, N, wo.shape[0]), dtype=torch.bfloat16, device=m.device)
        # The mean over sequences: the first GEMM carries 1/S; where sequences are masked the per-pair count
        # differs from S and the (linear) output projection is rescaled by S / count afterwards, on 128
        # channels instead of c*c.
        scale = None
        if not self.full_mask:
            cnt = torch.einsum("si,sj->ij", mask[0].float(), mask[0].float()).clamp(min=1.0)
            scale = (float(S) / cnt).unsqueeze(-1)
        rb = self.row_block
        blocked = c == 32 and (N * c) % 32 == 0
        t2 = torch.empty((rb * N, c * c), dtype=torch.bfloat16, device=m.device)
        for i0 in range(0, N, rb):
            i1 = min(N, i0 + rb)
            nr = (i1 - i0) * N
            if blocked:
                # product [(i, c), (j, d)] stored straight into [(i, j), (c, d)] by the kernel's epilogue
                gemm.gemm(a2[:, i0 * c:i1 * c], b2, mn_major=True, alpha=1.0 / S, out=t2,
                          c_blocked=(N * c * c, c, c * c))
                t = t2[:nr]
            else:
                t = gemm.gemm(a2[:, i0 * c:i1 * c], b2, mn_major=True, alpha=1.0 / S)
                t = t.view(i1 - i0, c, N, c).permute(0, 2, 1, 3).reshape(nr, c * c)
            if scale is None:
                gemm.gemm(t, wo, bias=bo, out=out[i0:i1].view(nr, -1))
            else:
                o = gemm.gemm(t, wo).view(i1 - i0, N, -1)
                out[i0:i1] = (o.float() * scale[i0:i1] + bo).to(torch.bfloat16)
        return out.unsqueeze(0)


class PairWeightedAveraging(_Switchable):
    def __init__(self, c_m: int = 64, c_z: int = 128, c_h: int = 32, heads: int = 8):
        super().__init__()
        self.heads, self.c_h = heads, c_h
        self.norm_m = nn.LayerNorm(c_m)
        self.norm_z = nn.LayerNorm(c_z)
        self.proj_m = nn.Linear(c_m, c_h * heads, bias=False)
        self.proj_g = nn.Linear(c_m, c_h * heads, bias=False)
        self.proj_z = nn.Linear(c_z, heads, bias=False)
        self.proj_o = nn.Linear(c_h * heads, c_m, bias=False)

    lever = "fused_pwa"

    def forward(self, m: torch.Tensor, z: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        why = self._tensor_reason(m) or (f"batch_{m.shape[0]}" if m.shape[0] != 1 else None)
        if not self._decide(why, f"C{m.shape[-1]}H{self.heads}x{self.c_h}S{m.shape[1]}", m.shape[2]):
            return R.pair_weighted_averaging(m, z, mask, self.norm_m.weight, self.norm_m.bias, self.norm_z.weight,
                                             self.norm_z.bias, self.proj_m.weight, self.proj_g.weight,
                                             self.proj_z.weight, self.proj_o.weight, self.heads)
        from ..ops import gemm, rows
        B, S, N, _ = m.shape
        H, c = self.heads, self.c_h
        mn = rows.layernorm_rows(m.contiguous(), self.norm_m.weight, self.norm_m.bias, self.norm_m.eps)
        b = rows.pair_head_bias(z[0].contiguous(), self.norm_z.weight, self.norm_z.bias, self.proj_z.weight).float()
        b = b + ((1.0 - mask[0].float()) * -1e6)[None]
        Np = (N + 7) // 8 * 8
        w = torch.zeros((H, N, Np), dtype=torch.bfloat16, device=m.device)
        w[:, :, :N] = torch.softmax(b, dim=-1).to(torch.bfloat16)
        v = self.proj_m(mn)[0].view(S, N, H, c)
        vt = torch.zeros((H, S * c, Np), dtype=torch.bfloat16, device=m.device)
        vt[:, :, :N] = v.permute(2, 0, 3, 1).reshape(H, S * c, N)
        o = gemm.gemm(w[:, :, :N], vt[:, :, :N])                       # [H, N(i), S*c]
        o = o.view(H, N, S, c).permute(2, 1, 0, 3).reshape(1, S, N, H * c)
        g = torch.sigmoid(self.proj_g(mn))
        return self.proj_o(g * o)


class MSALayer(nn.Module):
    def __init__(self, c_m: int = 64, c_z: int = 128):
        super().__init__()
        self.msa_transition = Transition(c_m, c_m * 4)
        self.pair_weighted_averaging = PairWeightedAveraging(c_m, c_z)
        self.pairformer_layer = PairformerLayer(c_s=384, c_z=c_z, no_seq=True)
        self.outer_product_mean = OuterProductMean(c_m, 32, c_z)

    def forward(self, z, m, token_mask, msa_mask, pair_mask):
        m = m + self.pair_weighted_averaging(m, z, token_mask if pair_mask is None else pair_mask)
        m = m + self.msa_transition(m)
        z = z + self.outer_product_mean(m, msa_mask).to(z.dtype)
        _, z = self.pairformer_layer(None, z, None, None if _all_ones(pair_mask) else pair_mask)
        return z, m


def _all_ones(mask) -> bool:
    return mask is None or getattr(mask, "_ubm_all_ones", False)


class MSAModule(nn.Module):
    def __init__(self, c_m: int = 64, c_z: int = 128, c_s_inputs: int = 384, num_blocks: int = 4, msa_feat: int = 34):
        super().__init__()
        self.s_proj = nn.Linear(c_s_inputs, c_m, bias=False)
        self.msa_proj = nn.Linear(msa_feat, c_m, bias=False)
        self.layers = nn.ModuleList([MSALayer(c_m, c_z) for _ in range(num_blocks)])

    def forward(self, z, s_inputs, msa_feat, msa_mask, token_mask, pair_mask=None):
        """msa_feat: [B, S, N, msa_feat]; msa_mask: [B, S, N]; token_mask: [B, N]."""
        m = self.msa_proj(msa_feat.to(z.dtype)) + self.s_proj(s_inputs.to(z.dtype)).unsqueeze(1)
        pm = token_mask[:, :, None] * token_mask[:, None, :]
        for layer in self.layers:
            z, m = layer(z, m, pm, msa_mask, pair_mask)
        return z
