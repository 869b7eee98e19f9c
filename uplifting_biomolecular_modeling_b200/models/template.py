"""Template embedder (AlphaFold3 Algorithm 16, the Boltz-2 ``TemplateV2Module`` family): per-template pair
features -> a small pair stack -> mean over templates -> relu -> projection added to the pair tensor.

Names follow the OpenFold3 family (``TemplatePairEmbedderAllAtom`` / ``TemplateEmbedderAllAtom``): eight bias-free
Linears build the pair stack's input (distogram, pseudo-beta pair mask, the two residue-type terms, the three
unit-vector components, the backbone pair mask) on top of ``linear_z(LayerNorm(z))``.  On the kernel path the
embedding is one launch and the tail one row kernel plus a tcgen05 GEMM (``ops/csrc/template_sm100.cu``; the
reference's kernels with the same boundary: common/opt_core/opt_core/kernels/templ_embed.py).  The pair stack itself
runs at width 64, where the fused Pairformer kernels (built for width 128) do not apply: plain statements.
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn as nn
import torch.nn.functional as F

from .pairformer import PairformerLayer, _Switchable

C_T, C_DG, C_AA = 64, 39, 32


class TemplateEmbedder(_Switchable):
    def __init__(self, c_z: int = 128, c_t: int = C_T, n_blocks: int = 2):
        super().__init__()
        self.c_z, self.c_t = c_z, c_t
        self.z_norm = nn.LayerNorm(c_z)
        self.linear_z = nn.Linear(c_z, c_t, bias=False)
        self.linear_dgram = nn.Linear(C_DG, c_t, bias=False)
        self.linear_pb = nn.Linear(1, c_t, bias=False)
        self.linear_aa1 = nn.Linear(C_AA, c_t, bias=False)
        self.linear_aa2 = nn.Linear(C_AA, c_t, bias=False)
        self.linear_x = nn.Linear(1, c_t, bias=False)
        self.linear_y = nn.Linear(1, c_t, bias=False)
        self.linear_z_vec = nn.Linear(1, c_t, bias=False)
        self.linear_bb = nn.Linear(1, c_t, bias=False)
        self.pair_stack = nn.ModuleList([PairformerLayer(c_s=c_t, c_z=c_t, no_seq=True, pair_heads=4)
                                         for _ in range(n_blocks)])
        self.v_norm = nn.LayerNorm(c_t)
        self.linear_t = nn.Linear(c_t, c_z, bias=False)

    # ---- plain statements
    def embed_reference(self, zp, f: Dict[str, torch.Tensor]) -> torch.Tensor:
        dt = zp.dtype
        asym = f["asym_id"]
        same = (asym[:, None] == asym[None, :]).to(dt)
        pbp = (f["template_pb_mask"][:, :, None] * f["template_pb_mask"][:, None, :]).to(dt) * same
        bbp = (f["template_bb_mask"][:, :, None] * f["template_bb_mask"][:, None, :]).to(dt) * same
        uv = f["template_unit_vector"].to(dt)
        a = self.linear_dgram(f["template_distogram"].to(dt)) + self.linear_pb(pbp[..., None])
        a = a + self.linear_aa1(f["template_restype"].to(dt))[:, :, None, :]
        a = a + self.linear_aa2(f["template_restype"].to(dt))[:, None, :, :]
        a = a + self.linear_x(uv[..., 0:1]) + self.linear_y(uv[..., 1:2]) + self.linear_z_vec(uv[..., 2:3])
        a = a + self.linear_bb(bbp[..., None])
        return zp[None] + a

    def _embed_fused(self, zp, f):
        from ..ops import native
        T, N = f["template_distogram"].shape[:2]
        dev = zp.device
        bf = torch.bfloat16
        ri = self.linear_aa1(f["template_restype"].to(zp.dtype)).to(bf).contiguous()
        rj = self.linear_aa2(f["template_restype"].to(zp.dtype)).to(bf).contiguous()
        w_dgram = self.linear_dgram.weight.detach().float().t().contiguous()                  # [39, 64]
        w_vec = torch.stack([self.linear_pb.weight[:, 0], self.linear_x.weight[:, 0], self.linear_y.weight[:, 0],
                             self.linear_z_vec.weight[:, 0], self.linear_bb.weight[:, 0]]).detach().float().contiguous()
        out = torch.empty((T, N, N, self.c_t), dtype=bf, device=dev)
        dg = f["template_distogram"].to(bf).contiguous()
        uv = f["template_unit_vector"].to(bf).contiguous()
        pbm = f["template_pb_mask"].float().contiguous()
        bbm = f["template_bb_mask"].float().contiguous()
        asym = f["asym_id"].to(torch.int32).contiguous()
        zpc = zp.to(bf).contiguous()
        rc = native.lib().ubm_template_embed(native.ptr(dg), native.ptr(uv), native.ptr(pbm), native.ptr(bbm),
                                             native.ptr(asym), native.ptr(ri), native.ptr(rj),
                                             native.ptr(zpc), native.ptr(w_dgram),
                                             native.ptr(w_vec), native.ptr(out), T, N, native.current_stream(dev))
        native.check(rc, "ubm_template_embed")
        return out.to(zp.dtype)

    def forward(self, z: torch.Tensor, f: Dict[str, torch.Tensor]) -> torch.Tensor:
        """z: [1, N, N, c_z]; f: template_distogram [T, N, N, 39], template_unit_vector [T, N, N, 3],
        template_pb_mask / template_bb_mask [T, N], template_restype [T, N, 32] (one-hot), asym_id [N].
        Returns the update to add to z."""
        zp = self.linear_z(self.z_norm(z[0]))                                               # [N, N, c_t]
        fused = self.impl == "fused" and z.is_cuda and self.c_t == C_T
        v = self._embed_fused(zp, f) if fused else self.embed_reference(zp, f)
        T = v.shape[0]
        outs = []
        for t in range(T):                       # templates go through the stack one at a time (memory)
            vt = v[t:t + 1]
            for blk in self.pair_stack:
                _, vt = blk(None, vt, None, None)
            outs.append(self.v_norm(vt[0]))
        s = torch.stack(outs, 0)                                                             # [T, N, N, c_t]
        if fused and s.dtype == torch.bfloat16:
            from ..ops import gemm, native
            N = s.shape[1]
            u = torch.empty((N * N, self.c_t), dtype=torch.bfloat16, device=s.device)
            sc = s.contiguous()
            rc = native.lib().ubm_template_tail(native.ptr(sc), native.ptr(u), T, N * N, self.c_t,
                                                native.current_stream(s.device))
            native.check(rc, "ubm_template_tail")
            out = gemm.gemm(u, self.linear_t.weight.detach().to(torch.bfloat16).contiguous()).view(N, N, -1)
        else:
            out = self.linear_t(F.relu(s.float().sum(0) / T).to(s.dtype))
        return out.unsqueeze(0)


def synthetic_template_features(n_tokens: int, n_templates: int, asym_id: torch.Tensor, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    T, N = n_templates, n_tokens
    bins = torch.randint(0, C_DG, (T, N, N), generator=g)
    uv = torch.randn(T, N, N, 3, generator=g)
    return {"template_distogram": F.one_hot(bins, C_DG).float(),
            "template_unit_vector": uv / uv.norm(dim=-1, keepdim=True).clamp(min=1e-6),
            "template_pb_mask": (torch.rand(T, N, generator=g) > 0.1).float(),
            "template_bb_mask": (torch.rand(T, N, generator=g) > 0.1).float(),
            "template_restype": F.one_hot(torch.randint(0, C_AA, (T, N), generator=g), C_AA).float(),
            "asym_id": asym_id}
