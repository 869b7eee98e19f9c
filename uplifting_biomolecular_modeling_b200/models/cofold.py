"""AF3-family cofolding model: input embedding, recycled trunk (MSA module + Pairformer), diffusion
sampler, distogram and confidence heads; plus the named configurations of the benchmarks and the
synthetic-input builders (random-init weights, synthetic features of the stated shapes).

Top-level wiring follows Boltz-2 (boltz2/stock/src/boltz/model/models/boltz2.py:182,421-455:
``z_init_1/z_init_2`` outer sum + ``rel_pos`` + ``token_bonds``; recycle loop
``s = s_init + s_recycle(s_norm(s))``, ``z = z_init + z_recycle(z_norm(z))``; then MSA module,
Pairformer, distogram, ``structure_module.sample``, confidence module).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .diffusion import AtomDiffusion, DiffusionModule
from .msa import MSAModule
from .pairformer import PairformerModule, set_impl


@dataclass(frozen=True)
class CofoldConfig:
    name: str = "af3"
    c_s: int = 384
    c_z: int = 128
    c_m: int = 64
    c_atom: int = 128
    c_atompair: int = 16
    pairformer_blocks: int = 48
    msa_blocks: int = 4
    recycles: int = 3                 # trunk passes = recycles + 1
    token_depth: int = 24
    token_heads: int = 16
    atom_depth: int = 3
    atom_heads: int = 4
    window_q: int = 32
    window_k: int = 128
    sampling_steps: int = 200
    samples: int = 5
    confidence_blocks: int = 4
    distogram_bins: int = 64
    token_feat: int = 36             # residue type one-hot (+ profile slots folded in by the embedder)
    msa_feat: int = 34
    atom_feat: int = 24
    relpos_bins: int = 139
    template_blocks: int = 0          # > 0 adds the template embedder (2 in the AF3 family); features optional
    align_reverse_diff: bool = False  # Boltz-2 sampler: rigid alignment of noisy onto denoised coordinates per step


CONFIGS: Dict[str, CofoldConfig] = {
    # BASELINE config 2: Boltz-2-shaped (64 Pairformer blocks, 3 recycles, 1 sample)
    "boltz2": CofoldConfig(name="boltz2", pairformer_blocks=64, recycles=3, samples=1),
    # BASELINE config 3: AF3 / Chai-1-shaped (48 blocks, 5 samples x 200 steps)
    "af3": CofoldConfig(name="af3", pairformer_blocks=48, recycles=3, samples=5),
    # BASELINE config 4: big mode, 1 recycle, single-sequence MSA
    "big4096": CofoldConfig(name="big4096", pairformer_blocks=48, recycles=0, samples=1),
    # diffusion design kits: a structure-module-heavy model (short trunk, no recycling, many samples per target)
    "design": CofoldConfig(name="design", pairformer_blocks=12, msa_blocks=1, recycles=0, samples=8,
                           sampling_steps=100, confidence_blocks=1),
    "tiny": CofoldConfig(name="tiny", pairformer_blocks=2, msa_blocks=1, recycles=1, token_depth=2,
                         atom_depth=1, sampling_steps=4, samples=2, confidence_blocks=1),
}


class RelativePositionEncoding(nn.Module):
    def __init__(self, c_z: int, bins: int = 139):
        super().__init__()
        self.linear_layer = nn.Linear(bins, c_z, bias=False)
        self.bins = bins

    def rows(self, residue_index, chain_id, r0: int, r1: int):
        return self.forward(residue_index, chain_id, rows=(r0, r1))

    def forward(self, residue_index, chain_id, entity_id=None, rows=None):
        r_max, s_max = 32, 2
        a0, a1 = (0, residue_index.shape[1]) if rows is None else rows
        chain_q, res_q = chain_id[:, a0:a1], residue_index[:, a0:a1]
        same_chain = chain_q[:, :, None] == chain_id[:, None, :]
        d = res_q[:, :, None] - residue_index[:, None, :]
        d_res = torch.where(same_chain, torch.clamp(d + r_max, 0, 2 * r_max), torch.full_like(d, 2 * r_max + 1))
        d_chain = torch.clamp(chain_q[:, :, None] - chain_id[:, None, :] + s_max, 0, 2 * s_max)
        d_chain = torch.where(same_chain, torch.full_like(d_chain, 2 * s_max + 1), d_chain)
        n_res, n_chain = 2 * r_max + 2, 2 * s_max + 2
        w = self.linear_layer.weight                                           # [c_z, bins]
        # sum of three one-hot projections == gather of weight columns (no [N, N, bins] tensor)
        out = w[:, :n_res].t()[d_res] + w[:, n_res:2 * n_res].t()[d_res] + \
            w[:, 2 * n_res + 1:2 * n_res + 1 + n_chain].t()[d_chain]
        out = out + w[:, 2 * n_res].t()[None, None, None, :] * same_chain[..., None].to(w.dtype)
        return out


class InputEmbedder(nn.Module):
    """Token features + atom encoder (no coordinates) -> s_inputs."""

    def __init__(self, cfg: CofoldConfig):
        super().__init__()
        from .diffusion import AtomAttentionEncoder
        self.cfg = cfg
        self.atom_embed = nn.Linear(cfg.atom_feat, cfg.c_atom, bias=False)
        self.atom_pair_embed = nn.Linear(4, cfg.c_atompair, bias=False)
        self.atom_attention_encoder = AtomAttentionEncoder(cfg.c_atom, cfg.c_s, cfg.atom_depth, cfg.atom_heads,
                                                           structure=False)
        self.atom_pair_bias = nn.ModuleList(
            [nn.Sequential(nn.LayerNorm(cfg.c_atompair), nn.Linear(cfg.c_atompair, cfg.atom_heads, bias=False))
             for _ in range(cfg.atom_depth)])
        self.token_embed = nn.Linear(cfg.token_feat, cfg.c_s, bias=False)

    def atom_tensors(self, feats):
        """c (atom single conditioning) and the windowed atom-pair representation."""
        cfg = self.cfg
        c = self.atom_embed(feats["atom_feat"].to(self.atom_embed.weight.dtype))       # [1, A, c_atom]
        ref = feats["ref_pos"]                                                           # [1, A, 3]
        A = ref.shape[1]
        wq, wk = cfg.window_q, cfg.window_k
        nw = A // wq
        pad = (wk - wq) // 2
        idx = (torch.arange(nw, device=ref.device) * wq)[:, None] + torch.arange(wk, device=ref.device)[None, :] - pad
        valid = (idx >= 0) & (idx < A)
        idxc = idx.clamp(0, A - 1)
        rq = ref[0].view(nw, wq, 3)
        rk = ref[0][idxc]                                                                # [nw, wk, 3]
        d = rq[:, :, None, :] - rk[:, None, :, :]
        same = (feats["ref_space_uid"][0].view(nw, wq)[:, :, None] == feats["ref_space_uid"][0][idxc][:, None, :])
        same = (same & valid[:, None, :]).to(ref.dtype)
        inv = 1.0 / (1.0 + (d * d).sum(-1, keepdim=True))
        pf = torch.cat([d * same[..., None], inv * same[..., None]], dim=-1)            # [nw, wq, wk, 4]
        p = self.atom_pair_embed(pf.to(self.atom_pair_embed.weight.dtype)).unsqueeze(0)
        return c, p

    def forward(self, feats):
        c, p = self.atom_tensors(feats)
        biases = [m(p).permute(0, 4, 1, 2, 3) for m in self.atom_pair_bias]
        layers = self.atom_attention_encoder.atom_transformer.layers
        if layers and layers[0].impl == "fused" and p.is_cuda and (self.cfg.window_q, self.cfg.window_k) == (32, 128):
            from .diffusion import WindowBias
            biases = [WindowBias(b) for b in biases]         # the window-attention kernel's bias layout
        n_tokens = feats["token_feat"].shape[1]
        a, _ = self.atom_attention_encoder(c, c, biases, torch.zeros_like(feats["ref_pos"]),
                                           feats["atom_to_token"][0], n_tokens)
        s_inputs = a + self.token_embed(feats["token_feat"].to(a.dtype))
        return s_inputs, c, p


class DistogramModule(nn.Module):
    def __init__(self, c_z: int, bins: int):
        super().__init__()
        self.distogram = nn.Linear(c_z, bins)

    def forward(self, z):
        z = z + z.transpose(1, 2)
        return self.distogram(z)


class ConfidenceModule(nn.Module):
    """Pairformer-based confidence head: pLDDT per token, PAE / PDE per pair."""

    def __init__(self, cfg: CofoldConfig):
        super().__init__()
        self.s_norm = nn.LayerNorm(cfg.c_s)
        self.z_norm = nn.LayerNorm(cfg.c_z)
        self.s_to_z = nn.Linear(cfg.c_s, cfg.c_z, bias=False)
        self.s_to_z_transpose = nn.Linear(cfg.c_s, cfg.c_z, bias=False)
        self.dist_bin_pairwise_embed = nn.Embedding(64, cfg.c_z)
        self.pairformer_stack = PairformerModule(cfg.c_s, cfg.c_z, cfg.confidence_blocks)
        self.to_plddt_logits = nn.Linear(cfg.c_s, 50)
        self.to_pae_logits = nn.Linear(cfg.c_z, 64)
        self.to_pde_logits = nn.Linear(cfg.c_z, 64)

    def forward(self, s, z, token_xyz):
        """s: [1, N, c_s]; z: [1, N, N, c_z]; token_xyz: [1, N, 3] representative-atom coordinates."""
        s = self.s_norm(s)
        z = self.z_norm(z) + self.s_to_z(s)[:, :, None, :] + self.s_to_z_transpose(s)[:, None, :, :]
        d = torch.cdist(token_xyz.float(), token_xyz.float())
        bins = torch.clamp(((d - 2.0) / (22.0 - 2.0) * 63).long(), 0, 63)
        z = z + self.dist_bin_pairwise_embed(bins).to(z.dtype)
        s, z = self.pairformer_stack(s, z)
        return {"plddt_logits": self.to_plddt_logits(s), "pae_logits": self.to_pae_logits(z),
                "pde_logits": self.to_pde_logits(z + z.transpose(1, 2))}


class CofoldModel(nn.Module):
    def __init__(self, cfg: CofoldConfig):
        super().__init__()
        self.cfg = cfg
        self.input_embedder = InputEmbedder(cfg)
        self.s_init = nn.Linear(cfg.c_s, cfg.c_s, bias=False)
        self.z_init_1 = nn.Linear(cfg.c_s, cfg.c_z, bias=False)
        self.z_init_2 = nn.Linear(cfg.c_s, cfg.c_z, bias=False)
        self.rel_pos = RelativePositionEncoding(cfg.c_z, cfg.relpos_bins)
        self.token_bonds = nn.Linear(1, cfg.c_z, bias=False)
        self.s_norm = nn.LayerNorm(cfg.c_s)
        self.z_norm = nn.LayerNorm(cfg.c_z)
        self.s_recycle = nn.Linear(cfg.c_s, cfg.c_s, bias=False)
        self.z_recycle = nn.Linear(cfg.c_z, cfg.c_z, bias=False)
        self.msa_module = MSAModule(cfg.c_m, cfg.c_z, cfg.c_s, cfg.msa_blocks, cfg.msa_feat)
        if cfg.template_blocks > 0:
            from .template import TemplateEmbedder
            self.template_embedder = TemplateEmbedder(cfg.c_z, n_blocks=cfg.template_blocks)
        self.pairformer_module = PairformerModule(cfg.c_s, cfg.c_z, cfg.pairformer_blocks)
        self.distogram_module = DistogramModule(cfg.c_z, cfg.distogram_bins)
        score = DiffusionModule(cfg.c_s, cfg.c_z, cfg.c_atom, cfg.c_atompair, cfg.token_depth, cfg.token_heads,
                                cfg.atom_depth, cfg.atom_heads, cfg.window_q, cfg.window_k)
        self.structure_module = AtomDiffusion(score, cfg.sampling_steps)
        self.structure_module.align_reverse_diff = cfg.align_reverse_diff
        self.z_cond_norm = nn.LayerNorm(cfg.c_z)
        self.confidence_module = ConfidenceModule(cfg)
        self.fused = False
        self.workspace: dict = {}
        # the ``trunk_graph`` lever: Pairformer stack passes replayed from a CUDA graph below this token count (the
        # stack is launch-bound there: ~40 launches per block); None = eager
        self.trunk_graphs = None
        self.trunk_graph_max_tokens = 512
        # the ``park_pair_init`` lever (big): the initial pair tensor, which every recycling pass reads once, waits in
        # pinned host memory between passes instead of holding N x N x c_z on the device for the whole trunk
        self.park_z_init = False

    # ------------------------------------------------------------------ implementation switch
    def set_impl(self, impl: str, kinds=None) -> int:
        self.fused = impl == "fused"
        return set_impl(self, impl, kinds, self.workspace)

    # ------------------------------------------------------------------ stages
    def embed(self, feats):
        s_inputs, atom_c, atom_p = self.input_embedder(feats)
        s_init = self.s_init(s_inputs)
        z_init = self.z_init_1(s_inputs)[:, :, None] + self.z_init_2(s_inputs)[:, None, :]
        z_init = z_init + self.rel_pos(feats["residue_index"], feats["chain_id"]).to(z_init.dtype)
        z_init = z_init + self.token_bonds(feats["token_bonds"].to(z_init.dtype))
        return s_inputs, s_init, z_init, atom_c, atom_p

    def z_init_rows(self, feats, s_inputs, r0: int, r1: int):
        """Rows [r0, r1) of the initial pair tensor without building the whole [N, N, c_z] tensor."""
        z = self.z_init_1(s_inputs)[:, r0:r1, None] + self.z_init_2(s_inputs)[:, None, :]
        ri, ci = feats["residue_index"], feats["chain_id"]
        rel = self.rel_pos.rows(ri, ci, r0, r1) if hasattr(self.rel_pos, "rows") else \
            self.rel_pos(ri, ci)[:, r0:r1]
        z = z + rel.to(z.dtype)
        return z + self.token_bonds(feats["token_bonds"][:, r0:r1].to(z.dtype))

    def trunk(self, feats, s_inputs, s_init, z_init, recycles: Optional[int] = None):
        cfg = self.cfg
        s = torch.zeros_like(s_init)
        z = torch.zeros_like(z_init)
        n = cfg.recycles if recycles is None else recycles
        tmask = feats["token_mask"]
        # without padding tokens the single-track attention needs no key mask (and may run fused)
        smask = None if feats.get("no_padding") is True else tmask
        # pair mask of the triangle updates, as upstream builds it (boltz2/stock/src/boltz/model/models/boltz2.py:
        # mask[:, :, None] * mask[:, None, :]); None only when the features say that no token is padding
        pmask = None if smask is None else tmask[:, :, None] * tmask[:, None, :]
        for layer in self.msa_module.layers:
            layer.outer_product_mean.full_mask = feats.get("msa_full") is True
        park = None
        if self.park_z_init and n > 0 and z_init.is_cuda:
            from ..mem.offload import HostPark
            park = HostPark(z_init)
            z_shape = z_init.shape
            del z_init
        for _ in range(n + 1):
            s = s_init + self.s_recycle(self.s_norm(s))
            zr = self.z_recycle(self.z_norm(z))
            if park is not None:
                z = park.fetch(zr.device)            # one pair tensor in from the host per pass
                z += zr
            else:
                z = z_init + zr
            del zr
            if self.cfg.template_blocks > 0 and "template_distogram" in feats:
                tf = {k: (v[0] if k.startswith("template_") else v) for k, v in feats.items()
                      if k.startswith("template_")}
                tf["asym_id"] = feats["chain_id"][0]
                z = z + self.template_embedder(z, tf).to(z.dtype)
            z = self.msa_module(z, s_inputs, feats["msa_feat"], feats["msa_mask"], tmask, pmask)
            if self.trunk_graphs is not None and smask is None and z.is_cuda and \
                    z.shape[1] <= self.trunk_graph_max_tokens:
                # capture-once, replay-many, first replay checked bit for bit against eager (capture.graphs)
                s, z = self.trunk_graphs.run(self._stack_unmasked, s, z)
            else:
                s, z = self.pairformer_module(s, z, smask, pmask)
        if park is not None:
            park.release()
        return s, z

    def _stack_unmasked(self, s, z):
        return self.pairformer_module(s, z, None, None)

    def structure(self, feats, s, z, s_inputs, atom_c, atom_p, samples=None, steps=None, generator=None,
                  step_fn=None, prep=None):
        cfg = self.cfg
        sm = self.structure_module
        if prep is None:
            prep = sm.score_model.prepare(s, s_inputs, self.z_cond_norm(z), atom_c, atom_c, atom_p, self.fused)
        A = feats["ref_pos"].shape[1]
        N = s.shape[1]
        x = sm.sample(prep, feats["atom_to_token"][0], N, A, samples or cfg.samples, steps or cfg.sampling_steps,
                      generator, step_fn)
        return x, prep

    @torch.no_grad()
    def forward(self, feats, recycles=None, samples=None, steps=None, generator=None, confidence: bool = True):
        s_inputs, s_init, z_init, atom_c, atom_p = self.embed(feats)
        s, z = self.trunk(feats, s_inputs, s_init, z_init, recycles)
        out = {"distogram_logits": self.distogram_module(z)}
        x, _ = self.structure(feats, s, z, s_inputs, atom_c, atom_p, samples, steps, generator)
        out["coords"] = x
        if confidence:
            rep = feats["token_rep_atom"][0]
            conf = self.confidence_module(s, z, x[:1, rep])
            out.update(conf)
            p = torch.softmax(conf["plddt_logits"].float(), -1)
            out["plddt"] = (p * (torch.arange(50, device=p.device) + 0.5) / 50).sum(-1)
        return out


# ----------------------------------------------------------------------------------- synthetic inputs
AA = 20


def synthetic_features(n_tokens: int, msa_depth: int, cfg: CofoldConfig, device="cpu", dtype=torch.float32,
                       seed: int = 0, chains=None, atoms_per_token: Optional[int] = None,
                       mutation_p: float = 0.3) -> Dict[str, torch.Tensor]:
    """Synthetic complex of the benchmark shapes: residues uniform over 20 amino acids, an MSA made by
    mutating the query per position with probability ``mutation_p``, atoms laid out token by token.

    ``chains`` is a list of (length, kind) with kind in {"protein", "dna", "ligand"}; by default one
    protein chain of ``n_tokens`` residues.  Atoms per token: protein 8, DNA 20, ligand 1 (heavy atoms).
    """
    g = torch.Generator().manual_seed(seed)
    chains = chains or [(n_tokens, "protein")]
    assert sum(c[0] for c in chains) == n_tokens
    per = {"protein": atoms_per_token or 8, "dna": atoms_per_token or 20, "ligand": 1}
    restype, chain_id, res_idx, atoms = [], [], [], []
    for ci, (length, kind) in enumerate(chains):
        if kind == "protein":
            rt = torch.randint(0, AA, (length,), generator=g)
        elif kind == "dna":
            rt = 22 + torch.randint(0, 4, (length,), generator=g)
        else:
            rt = torch.full((length,), 30, dtype=torch.long)
        restype.append(rt)
        chain_id.append(torch.full((length,), ci, dtype=torch.long))
        res_idx.append(torch.arange(length) if kind != "ligand" else torch.zeros(length, dtype=torch.long))
        atoms.append(torch.full((length,), per[kind], dtype=torch.long))
    restype, chain_id, res_idx, atoms = map(torch.cat, (restype, chain_id, res_idx, atoms))
    token_feat = F.one_hot(restype, cfg.token_feat).float()
    # MSA: depth x tokens, query first; non-protein columns are gaps except in the query
    msa = restype.unsqueeze(0).repeat(msa_depth, 1)
    if msa_depth > 1:
        mut = torch.rand((msa_depth, n_tokens), generator=g) < mutation_p
        mut[0] = False
        rnd = torch.randint(0, AA, (msa_depth, n_tokens), generator=g)
        is_prot = (restype < AA).unsqueeze(0)
        msa = torch.where(mut & is_prot, rnd, msa)
    msa_feat = torch.zeros((msa_depth, n_tokens, cfg.msa_feat))
    msa_feat.scatter_(2, msa.clamp(max=cfg.msa_feat - 3).unsqueeze(-1), 1.0)
    # atoms
    n_atoms_true = int(atoms.sum())
    A = (n_atoms_true + cfg.window_q - 1) // cfg.window_q * cfg.window_q
    atom_to_token = torch.repeat_interleave(torch.arange(n_tokens), atoms)
    atom_to_token = F.pad(atom_to_token, (0, A - n_atoms_true), value=n_tokens - 1)
    first_atom = torch.cumsum(atoms, 0) - atoms
    ref_pos = torch.randn((A, 3), generator=g) * 1.5
    atom_feat = torch.zeros((A, cfg.atom_feat))
    atom_feat.scatter_(1, torch.randint(0, 4, (A, 1), generator=g), 1.0)      # element one-hot (C/N/O/S)
    atom_feat[:, 4] = (torch.arange(A) < n_atoms_true).float()
    bonds = torch.zeros((n_tokens, n_tokens, 1))
    lig = (restype == 30).nonzero().flatten()
    for a, b in zip(lig[:-1].tolist(), lig[1:].tolist()):                     # random connected graph: a chain
        bonds[a, b, 0] = bonds[b, a, 0] = 1.0
    feats = {
        "token_feat": token_feat[None], "residue_index": res_idx[None], "chain_id": chain_id[None],
        "token_mask": torch.ones((1, n_tokens)), "token_bonds": bonds[None],
        "msa_feat": msa_feat[None], "msa_mask": torch.ones((1, msa_depth, n_tokens)),
        "atom_feat": atom_feat[None], "ref_pos": ref_pos[None], "ref_space_uid": atom_to_token[None].clone(),
        "atom_to_token": atom_to_token[None], "token_rep_atom": first_atom[None],
    }
    out = {}
    for k, v in feats.items():
        out[k] = v.to(device=device, dtype=dtype) if v.is_floating_point() else v.to(device)
    return out


def chains_for(config_name: str, n_tokens: int):
    """Chain composition of the named benchmark inputs."""
    if config_name == "af3" and n_tokens == 1536:
        # the stated chains give 1488 tokens; the named size is 1536, so 48 single-atom filler tokens
        # (a second ligand-like entity, unmasked) complete it and the compute is that of N = 1536
        return [(448, "protein")] * 3 + [(48, "dna")] * 2 + [(48, "ligand")] + [(48, "ligand")]
    if config_name == "big4096" and n_tokens == 4096:
        return [(512, "protein")] * 8
    return [(n_tokens, "protein")]


def build_model(config: str = "af3", device="cpu", dtype=torch.float32, seed: int = 0, **overrides) -> CofoldModel:
    cfg = CONFIGS[config]
    if overrides:
        cfg = replace(cfg, **overrides)
    torch.manual_seed(seed)
    model = CofoldModel(cfg).eval()
    for p in model.parameters():
        p.requires_grad_(False)
    return model.to(device=device, dtype=dtype)
