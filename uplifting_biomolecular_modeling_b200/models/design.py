"""Design-side models: sequence inversion through the structure trunk (the one workload with gradients) and a
message-passing inverse-folding decoder with batch-invariant sampling.

* :class:`SequenceInversion` - optimise a relaxed sequence (logits over 20 residue types per token) so that the
  trunk's distogram matches a target: forward through ``embed`` -> ``trunk`` -> distogram head, cross-entropy
  against the target bins, gradient with respect to the logits only.  Memory plan of the backward pass: every
  Pairformer block is an activation-checkpoint boundary (its inputs are kept, its inside is recomputed), the
  weights are frozen so every LayerNorm / Linear backward computes the input gradient only.
* :class:`InverseFoldingDecoder` - backbone coordinates -> k-nearest-neighbour graph with radial-basis edge
  features -> message-passing encoder -> autoregressive decoder over a random decoding order.  Every sample draws
  its decoding order and its sampling uniforms from its own generator stream *before* decoding, so a sample's
  sequence does not depend on which other samples share its batch (the property the reference gets from
  replaying per-sample Philox streams inside one captured graph).

Reference kits: ef2inv (``ef2_bwd_ckpt`` memory plan, dX-only LayerNorm backward), proteinmpnn (``--graph_rng``),
esm_if1.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

N_TYPES = 20


# ------------------------------------------------------------------------------------------ sequence inversion
def trunk_checkpointed(model, feats, s_inputs, s_init, z_init, recycles: int = 0, use_checkpoint: bool = True):
    """The trunk loop of :class:`models.cofold` with every Pairformer block as a checkpoint boundary."""
    s = torch.zeros_like(s_init)
    z = torch.zeros_like(z_init)
    tmask = feats["token_mask"]
    for _ in range(recycles + 1):
        s = s_init + model.s_recycle(model.s_norm(s))
        z = z_init + model.z_recycle(model.z_norm(z))
        z = model.msa_module(z, s_inputs, feats["msa_feat"], feats["msa_mask"], tmask, None)
        for layer in model.pairformer_module.layers:
            if use_checkpoint:
                s, z = checkpoint(layer, s, z, tmask, None, use_reentrant=False)
            else:
                s, z = layer(s, z, tmask, None)
    return s, z


class SequenceInversion:
    def __init__(self, model, feats: Dict[str, torch.Tensor], target_bins: torch.Tensor, recycles: int = 0,
                 use_checkpoint: bool = True, lr: float = 0.5, seed: int = 0):
        self.model, self.feats, self.target = model, dict(feats), target_bins
        self.recycles, self.use_checkpoint = recycles, use_checkpoint
        for p in model.parameters():                       # frozen weights: every backward is input-gradient only
            p.requires_grad_(False)
        N = feats["token_feat"].shape[1]
        g = torch.Generator().manual_seed(seed)
        self.logits = (0.01 * torch.randn(1, N, N_TYPES, generator=g)).to(feats["token_feat"].device).requires_grad_(True)
        self.opt = torch.optim.Adam([self.logits], lr=lr)
        self.history: List[float] = []

    def loss(self) -> torch.Tensor:
        f = dict(self.feats)
        tf = f["token_feat"].clone().float()
        tf[..., :N_TYPES] = torch.softmax(self.logits, -1)
        f["token_feat"] = tf.to(self.feats["token_feat"].dtype)
        s_inputs, s_init, z_init, _, _ = self.model.embed(f)
        _, z = trunk_checkpointed(self.model, f, s_inputs, s_init, z_init, self.recycles, self.use_checkpoint)
        d = self.model.distogram_module(z).float()
        return F.cross_entropy(d.reshape(-1, d.shape[-1]), self.target.reshape(-1))

    def step(self) -> float:
        self.opt.zero_grad(set_to_none=True)
        loss = self.loss()
        loss.backward()
        self.opt.step()
        self.history.append(float(loss.detach()))
        return self.history[-1]

    def sequence(self) -> torch.Tensor:
        return self.logits.detach().argmax(-1)


# ------------------------------------------------------------------------------------------ inverse-folding decoder
def rbf(d: torch.Tensor, n: int = 16, d_max: float = 20.0) -> torch.Tensor:
    mu = torch.linspace(0.0, d_max, n, device=d.device)
    return torch.exp(-((d[..., None] - mu) / (d_max / n)) ** 2)


def knn_graph(x: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """x: [B, N, 3] -> (neighbour index [B, N, k], distances [B, N, k]); a node is its own first neighbour."""
    d = torch.cdist(x, x)
    dist, idx = d.topk(min(k, x.shape[1]), dim=-1, largest=False)
    return idx, dist


def _gather_nodes(h: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    B, N, k = idx.shape
    return torch.gather(h[:, None].expand(B, N, N, h.shape[-1]), 2, idx[..., None].expand(B, N, k, h.shape[-1]))


class _MPLayer(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.msg = nn.Sequential(nn.Linear(3 * dim, dim), nn.GELU(), nn.Linear(dim, dim))
        self.norm1 = nn.LayerNorm(dim)
        self.ff = nn.Sequential(nn.Linear(dim, 4 * dim), nn.GELU(), nn.Linear(4 * dim, dim))
        self.norm2 = nn.LayerNorm(dim)

    def forward(self, h, e, idx, visible=None):
        """h: [B, N, d] nodes, e: [B, N, k, d] edges; ``visible`` [B, N, k] masks neighbour messages (decoder)."""
        hn = _gather_nodes(h, idx)
        m = self.msg(torch.cat([h[:, :, None].expand_as(hn), hn, e], -1))
        if visible is not None:
            m = m * visible[..., None].to(m.dtype)
        h = self.norm1(h + m.mean(2))
        return self.norm2(h + self.ff(h))


class InverseFoldingDecoder(nn.Module):
    def __init__(self, dim: int = 64, k: int = 12, enc_layers: int = 3, dec_layers: int = 3, n_rbf: int = 16):
        super().__init__()
        self.dim, self.k, self.n_rbf = dim, k, n_rbf
        self.edge_in = nn.Linear(n_rbf, dim)
        self.node_in = nn.Linear(n_rbf, dim)
        self.enc = nn.ModuleList([_MPLayer(dim) for _ in range(enc_layers)])
        self.seq_embed = nn.Embedding(N_TYPES + 1, dim)            # last index = "not decoded yet"
        self.dec = nn.ModuleList([_MPLayer(dim) for _ in range(dec_layers)])
        self.head = nn.Linear(dim, N_TYPES)

    def encode(self, x: torch.Tensor):
        idx, dist = knn_graph(x, self.k)
        e = self.edge_in(rbf(dist, self.n_rbf))
        h = self.node_in(rbf(dist.mean(-1), self.n_rbf))
        for layer in self.enc:
            h = layer(h, e, idx)
        return h, e, idx

    @staticmethod
    def draws(n_tokens: int, seeds: List[int], device="cpu") -> Tuple[torch.Tensor, torch.Tensor]:
        """Per-sample decoding order and sampling uniforms, each sample from its own generator stream."""
        orders, unis = [], []
        for sd in seeds:
            g = torch.Generator().manual_seed(int(sd))
            orders.append(torch.randperm(n_tokens, generator=g))
            unis.append(torch.rand(n_tokens, generator=g, dtype=torch.float64))
        return torch.stack(orders).to(device), torch.stack(unis).to(device)

    @torch.no_grad()
    def sample(self, x: torch.Tensor, seeds: List[int], temperature: float = 0.1) -> torch.Tensor:
        """x: [1 or B, N, 3] backbone; one sequence per seed -> [len(seeds), N] residue types."""
        B, N = len(seeds), x.shape[1]
        if x.shape[0] == 1 and B > 1:
            x = x.expand(B, N, 3)
        h, e, idx = self.encode(x)
        order, uni = self.draws(N, seeds, x.device)
        rank = torch.empty_like(order)
        rank.scatter_(1, order, torch.arange(N, device=x.device).expand(B, N))       # rank[b, i] = step at which i is decoded
        seq = torch.full((B, N), N_TYPES, dtype=torch.long, device=x.device)
        rows = torch.arange(B, device=x.device)
        for t in range(N):
            i = order[:, t]                                                          # token decoded at this step
            # a neighbour's residue is visible only if it was decoded earlier
            vis = _gather_nodes(rank[..., None].float(), idx)[..., 0] < t
            hd = h
            emb = _gather_nodes(self.seq_embed(seq), idx)
            for layer in self.dec:
                hd = layer(hd, e + emb, idx, vis)
            logits = self.head(hd[rows, i]).double() / max(temperature, 1e-6)
            cdf = torch.softmax(logits, -1).cumsum(-1)
            pick = (cdf < uni[rows, t][:, None] * cdf[:, -1:]).sum(-1).clamp(max=N_TYPES - 1)
            seq[rows, i] = pick
        return seq


def build_decoder(seed: int = 0, **kw) -> InverseFoldingDecoder:
    g = torch.Generator().manual_seed(seed)
    m = InverseFoldingDecoder(**kw)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g) / math.sqrt(p.shape[-1]))
    return m.eval()


LETTERS = "ACDEFGHIKLMNPQRSTVWY"


class DesignPipeline:
    """Backbone diffusion followed by inverse folding: the ``design`` verb of the diffusion design kits.

    A target of ``n_tokens`` residues is built with a fraction of its positions marked "to be designed" (their
    residue type is the unknown token, so the trunk conditions on the rest only); the structure module samples one
    backbone per design; the inverse-folding decoder gives each backbone a sequence from its own random stream.
    With ``dedup`` the designs are the samples of ONE prediction (one trunk pass, one set of step-invariant sampler
    tensors, every step batched over the designs); without it each design is a prediction of its own.  The
    reference's design kits get the same saving from their ``cond_dedup`` / ``sdedup`` levers and resident sampler
    graphs (boltzgen, rfdiffusion1 ``se3fast_addon``, pxdesign CHANGES.md)."""

    def __init__(self, predictor, seed: int = 0, dedup: bool = True, decoder: Optional[InverseFoldingDecoder] = None):
        self.pred, self.seed, self.dedup = predictor, seed, dedup
        self.decoder = decoder or build_decoder(seed=seed)

    def features(self, n_tokens: int, designed_fraction: float = 0.5):
        from . import cofold
        cfg = self.pred.cfg
        feats = cofold.synthetic_features(n_tokens, 1, cfg, seed=self.seed)
        g = torch.Generator().manual_seed(self.seed + 17)
        designed = torch.rand(n_tokens, generator=g) < designed_fraction
        tf = feats["token_feat"].clone()
        tf[:, designed, :] = 0
        tf[:, designed, min(20, tf.shape[-1] - 1)] = 1          # unknown-residue slot
        feats["token_feat"] = tf
        return feats, designed

    @torch.no_grad()
    def run(self, n_tokens: int, designs: int = 2, designed_fraction: float = 0.5) -> dict:
        feats, designed = self.features(n_tokens, designed_fraction)
        rep = feats["token_rep_atom"][0]
        if self.dedup:
            out = self.pred.predict(feats, samples=designs, confidence=False)
            coords = out["coords"]
            passes = 1
        else:
            coords = torch.cat([self.pred.predict(feats, samples=1, confidence=False, seed=self.seed + i)["coords"]
                                for i in range(designs)], 0)
            passes = designs
        backbones = coords[:, rep].float().cpu()                  # one representative atom per token
        dec = self.decoder
        seqs = torch.cat([dec.sample(backbones[i:i + 1], seeds=[self.seed + 1000 + i]) for i in range(designs)], 0)
        text = ["".join(LETTERS[int(t) % len(LETTERS)] for t in row.tolist()) for row in seqs]
        return {"coords": coords.cpu(), "sequences": text, "designed": designed, "trunk_passes": passes}
