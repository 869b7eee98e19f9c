"""Diffusion module (AF3 / Boltz-2 family) and its sampler.

Structure and names follow Boltz-2 (boltz2/stock/src/boltz/model/modules/diffusionv2.py:38-115
``single_conditioner, atom_attention_encoder, s_to_a_linear, token_transformer, a_norm,
atom_attention_decoder``; transformersv2.py:17-227 ``DiffusionTransformerLayer`` = ``adaln,
pair_bias_attn, output_projection, transition``; windows of 32 queries x 128 keys,
diffusionv2.py:44-56).  The sampler is the EDM roll-out of ``AtomDiffusion.sample``
(diffusionv2.py:295-396): per step a random rigid augmentation, noise injection, one denoiser
call over all samples, an Euler update.

What is step-invariant is computed once per prediction and reused by all steps: the pair biases of
the 24 token-transformer layers, the atom-pair biases of the 6 atom layers, and every
conditioning projection of s (the reference's ``apb_hoist`` / ``atom_hoist`` / ``dit_hoist``
levers, common/opt_core/opt_core/of3_sampler/atom_hoist.py, of3_trunk/apb_hoist.py).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import reference as R
from .pairformer import AttentionPairBias, _Switchable


class AdaLN(nn.Module):
    def __init__(self, dim: int, dim_s: int):
        super().__init__()
        self.a_norm = nn.LayerNorm(dim, elementwise_affine=False)
        self.s_norm = nn.LayerNorm(dim_s, bias=False)
        self.s_scale = nn.Linear(dim_s, dim)
        self.s_bias = nn.Linear(dim_s, dim, bias=False)

    def cond(self, s):
        sn = self.s_norm(s)
        return self.s_scale(sn), self.s_bias(sn)

    def forward(self, a, s=None, cond=None, fused: bool = False):
        scale, shift = self.cond(s) if cond is None else cond
        if fused and a.is_cuda and a.dtype == torch.bfloat16:
            from ..ops import rows
            return rows.adaln_rows(a.contiguous(), scale.contiguous(), shift.contiguous())
        return torch.sigmoid(scale) * self.a_norm(a) + shift


class ConditionedTransitionBlock(nn.Module):
    def __init__(self, dim: int, dim_s: int, expansion: int = 2):
        super().__init__()
        self.adaln = AdaLN(dim, dim_s)
        hidden = dim * expansion
        # parameter names and the SwiGLU halves as upstream (boltz2/stock/src/boltz/model/modules/transformersv2.py:
        # 34-65, utils.py:29-35): ``swish_gate.0`` projects to [values | gates] and the GATES half goes through silu;
        # ``output_projection.0`` is the conditioning gate's Linear (the Sequential's sigmoid is applied in forward)
        self.swish_gate = nn.Sequential(nn.Linear(dim, 2 * hidden, bias=False))
        self.a_to_b = nn.Linear(dim, hidden, bias=False)
        self.b_to_a = nn.Linear(hidden, dim, bias=False)
        self.output_projection = nn.Sequential(nn.Linear(dim_s, dim), nn.Sigmoid())
        nn.init.constant_(self.output_projection[0].bias, -2.0)

    def forward(self, a, s=None, cond=None, gate=None, fused: bool = False):
        x = self.adaln(a, s, cond, fused)
        vals, gates = self.swish_gate[0](x).chunk(2, dim=-1)
        b = F.silu(gates) * vals * self.a_to_b(x)
        gate = self.output_projection[0](s) if gate is None else gate
        return torch.sigmoid(gate) * self.b_to_a(b)


class WindowBias:
    """Atom-pair bias of one atom-transformer layer laid out for the window-attention kernel: bf16
    [1, H, windows, 32, 128] that already carries the factor log2(e)."""

    LOG2E = 1.4426950408889634

    def __init__(self, dense: torch.Tensor):
        self.data = (dense.float() * self.LOG2E).to(torch.bfloat16).contiguous()

    def dense(self) -> torch.Tensor:
        return self.data.float() / self.LOG2E


class DiffusionTransformerLayer(_Switchable):
    def __init__(self, dim: int = 768, dim_s: int = 768, heads: int = 16):
        super().__init__()
        self.adaln = AdaLN(dim, dim_s)
        self.pair_bias_attn = AttentionPairBias(dim, 128, heads, compute_pair_bias=False)
        self.output_projection_linear = nn.Linear(dim_s, dim)
        nn.init.constant_(self.output_projection_linear.bias, -2.0)
        # upstream registers the same Linear a second time inside a Sequential (transformersv2.py:159-165): its
        # checkpoints carry both names, so the alias is kept for strict loading
        self.output_projection = nn.Sequential(self.output_projection_linear, nn.Sigmoid())
        self.transition = ConditionedTransitionBlock(dim, dim_s)
        self.dim, self.heads = dim, heads

    def hoist(self, s):
        """Everything that depends only on the conditioning s (same for every layer call of a step)."""
        gate, t_gate = self.output_projection_linear(s), self.transition.output_projection[0](s)
        return {"adaln": self.adaln.cond(s), "gate": gate, "t_adaln": self.transition.adaln.cond(s),
                "t_gate": t_gate, "gate_sig": torch.sigmoid(gate), "t_gate_sig": torch.sigmoid(t_gate)}

    def cond_weights(self):
        """Rows of the batched conditioning GEMMs of this layer: (W [4C, dim_s], b [4C]) for
        scale | shift | transition scale | transition shift on the affine-free normalised s (the LayerNorm weight
        of each AdaLN is folded into its columns), and (W [2C, dim_s], b [2C]) for the two output gates on s."""
        def fold(ad):
            g = ad.s_norm.weight.detach().float()
            return (ad.s_scale.weight.detach().float() * g[None, :], ad.s_scale.bias.detach().float(),
                    ad.s_bias.weight.detach().float() * g[None, :])
        ws, bs, wb = fold(self.adaln)
        tws, tbs, twb = fold(self.transition.adaln)
        zc = torch.zeros_like(bs)
        w1 = torch.cat([ws, wb, tws, twb], 0)
        b1 = torch.cat([bs, zc, tbs, zc], 0)
        w2 = torch.cat([self.output_projection_linear.weight.detach().float(),
                        self.transition.output_projection[0].weight.detach().float()], 0)
        b2 = torch.cat([self.output_projection_linear.bias.detach().float(),
                        self.transition.output_projection[0].bias.detach().float()], 0)
        return w1, b1, w2, b2

    lever = "fused_dit"

    def _fused_token_layer(self, a, h, bias, mask=None):
        """Token-transformer layer on the fused path: AdaLN rows -> q|k|v and gate projections (tcgen05
        GEMM) -> attention with the hoisted pair-bias planes shared by all samples -> output projection whose
        epilogue applies the conditioning gate and the residual; then the conditioned SwiGLU transition the same
        way (one GEMM for swish_gated and a_to_b, a three-way row kernel, an output GEMM with gate and residual)."""
        from ..ops import gemm, pair, rows
        B, N, C = a.shape
        attn = self.pair_bias_attn
        a = a.contiguous()
        a2 = a.view(B * N, C)
        gate, t_gate = h["gate_sig"], h["t_gate_sig"]
        gate = gate.reshape(-1, C) if gate.dim() == 3 else gate
        t_gate = t_gate.reshape(-1, C) if t_gate.dim() == 3 else t_gate
        b = rows.adaln_rows(a, h["adaln"][0], h["adaln"][1])
        if isinstance(bias, WindowBias):
            if attn._packed is None:
                attn._packed = pair.ApbPacked.pack(attn.proj_q.weight, attn.proj_q.bias, attn.proj_k.weight,
                                                   attn.proj_v.weight, attn.proj_g.weight, attn.proj_o.weight,
                                                   attn.heads)
            a = pair.window_attention_fused(b, attn._packed, bias.data, out_gate=gate, out_residual=a2)
        else:
            a = attn._fused_forward(b, bias, out_gate=gate, out_residual=a2, mask=mask)
        a2 = a.view(B * N, C)
        tr = self.transition
        if self._packed is None:
            # silu(gates half) * values half * a_to_b: upstream's swish_gate stores the values first
            wsg = tr.swish_gate[0].weight.detach()
            hid = wsg.shape[0] // 2
            if hid % 32 == 0:
                # one projection whose epilogue forms the product on the accumulator (no [M, 3 * hid] intermediate)
                w_in = gemm.pack_swiglu3(wsg[hid:], wsg[:hid], tr.a_to_b.weight.detach())
            else:
                w_in = torch.cat([wsg[hid:], wsg[:hid], tr.a_to_b.weight.detach()], 0).to(torch.bfloat16).contiguous()
            self._packed = (w_in, tr.b_to_a.weight.detach().to(torch.bfloat16).contiguous(), hid % 32 == 0)
        w_in, w_ba, in_epilogue = self._packed
        x = rows.adaln_rows(a, h["t_adaln"][0], h["t_adaln"][1]).view(B * N, C)
        u = gemm.gemm(x, w_in, act="swiglu3") if in_epilogue else rows.swiglu3_rows(gemm.gemm(x, w_in))
        return gemm.gemm(u, w_ba, gate=t_gate, residual=a2).view(B, N, C)

    def forward(self, a, s, bias, mask=None, multiplicity: int = 1, hoisted: Optional[dict] = None,
                window: Optional[tuple] = None):
        fused = self.impl == "fused"
        h = hoisted if hoisted is not None else self.hoist(s)
        from .pairformer import BiasPlanes
        if fused:
            token = window is None and isinstance(bias, BiasPlanes)
            atoms = window == (32, 128) and isinstance(bias, WindowBias) and self.pair_bias_attn.head_dim == 32
            why = self._tensor_reason(a) or (None if (token or atoms) else "bias_layout") \
                or ("window_mask" if (atoms and mask is not None) else None)
            klass = f"WIN{window[0]}x{window[1]}" if window is not None else \
                f"D{64 if self.pair_bias_attn.head_dim > 32 else 32}H{self.pair_bias_attn.heads}S{a.shape[0]}"
            if self._decide(why, klass, a.shape[1], {"head_dim": self.pair_bias_attn.head_dim, "dtype": "bf16",
                                                     **({"window": tuple(window)} if window is not None else {})},
                            "tcgen05_window" if atoms else "tcgen05_2row"):
                return self._fused_token_layer(a, h, bias, mask)
        if isinstance(bias, WindowBias):
            bias = bias.dense()
        if isinstance(bias, BiasPlanes):
            bias = bias.dense()
        b = self.adaln(a, None, h["adaln"], fused)
        if window is None:
            b = self.pair_bias_attn(b, None, mask, bias=bias, multiplicity=multiplicity)
        else:
            b = _window_attention(self.pair_bias_attn, b, bias, window)
        a = a + torch.sigmoid(h["gate"]) * b
        a = a + self.transition(a, None, h["t_adaln"], h["t_gate"], fused)
        return a


def _window_attention(attn: AttentionPairBias, x, bias, window):
    """Atom attention in (wq, wk) windows; bias: [B, H, nw, wq, wk]."""
    wq, wk = window
    B, A, _ = x.shape
    H, D = attn.heads, attn.head_dim
    if isinstance(bias, WindowBias):
        bias = bias.dense().to(x.dtype)
    q = attn.proj_q(x).view(B, A, H, D).transpose(1, 2)
    k = attn.proj_k(x).view(B, A, H, D).transpose(1, 2)
    v = attn.proj_v(x).view(B, A, H, D).transpose(1, 2)
    g = torch.sigmoid(attn.proj_g(x))
    bb = bias
    if bb is not None and bb.shape[0] != B:
        bb = bb.repeat_interleave(B // bb.shape[0], 0)
    o = R.window_attention(q, k, v, bb, wq, wk)
    o = o.transpose(1, 2).reshape(B, A, H * D)
    return attn.proj_o(g * o)


class DiffusionTransformer(nn.Module):
    def __init__(self, depth: int, dim: int, dim_s: int, heads: int):
        super().__init__()
        self.layers = nn.ModuleList([DiffusionTransformerLayer(dim, dim_s, heads) for _ in range(depth)])
        self._cond_packed = None

    def hoist_all(self, s):
        """Conditioning of every layer from two GEMMs (fused path): the affine-free normalised s against the
        stacked AdaLN weights of all layers, and s against the stacked gate weights with the sigmoid in the
        epilogue.  Per-layer entries are column slices of the two outputs.  s: [1, N, dim_s] bf16 on the GPU."""
        from ..ops import gemm
        C = self.layers[0].dim
        if self._cond_packed is None:
            parts = [l.cond_weights() for l in self.layers]
            self._cond_packed = (torch.cat([p[0] for p in parts], 0).to(torch.bfloat16).contiguous(),
                                 torch.cat([p[1] for p in parts], 0).contiguous(),
                                 torch.cat([p[2] for p in parts], 0).to(torch.bfloat16).contiguous(),
                                 torch.cat([p[3] for p in parts], 0).contiguous())
        w1, b1, w2, b2 = self._cond_packed
        s2 = s.reshape(-1, s.shape[-1])
        sn = F.layer_norm(s2.float(), (s2.shape[-1],)).to(torch.bfloat16)
        cond = gemm.gemm(sn, w1, bias=b1)                                   # [N, L * 4C]
        gates = gemm.gemm(s2.to(torch.bfloat16).contiguous(), w2, bias=b2, act="sigmoid")   # [N, L * 2C]
        out = []
        for i in range(len(self.layers)):
            c0, g0 = i * 4 * C, i * 2 * C
            out.append({"adaln": (cond[:, c0:c0 + C], cond[:, c0 + C:c0 + 2 * C]),
                        "t_adaln": (cond[:, c0 + 2 * C:c0 + 3 * C], cond[:, c0 + 3 * C:c0 + 4 * C]),
                        "gate_sig": gates[:, g0:g0 + C], "t_gate_sig": gates[:, g0 + C:g0 + 2 * C],
                        "gate": None, "t_gate": None})
        return out

    def can_hoist_all(self, s, biases) -> bool:
        from .pairformer import BiasPlanes
        return (s.is_cuda and s.dtype == torch.bfloat16 and all(l.impl == "fused" for l in self.layers)
                and all(isinstance(b, BiasPlanes) for b in biases) and self.layers[0].dim % 8 == 0)

    def forward(self, a, s, biases, mask=None, multiplicity=1, hoisted=None, window=None):
        for i, layer in enumerate(self.layers):
            a = layer(a, s, biases[i], mask, multiplicity, None if hoisted is None else hoisted[i], window)
        return a


class FourierEmbedding(nn.Module):
    def __init__(self, dim: int = 256):
        super().__init__()
        self.proj = nn.Linear(1, dim)
        for p in self.proj.parameters():
            p.requires_grad_(False)
        nn.init.normal_(self.proj.weight)
        nn.init.normal_(self.proj.bias)

    def forward(self, t):
        x = F.linear(t.float().unsqueeze(-1), self.proj.weight.float(), self.proj.bias.float())
        return torch.cos(2 * math.pi * x)


class SingleConditioning(nn.Module):
    def __init__(self, c_s: int = 384, c_s_inputs: int = 384, dim_fourier: int = 256, sigma_data: float = 16.0):
        super().__init__()
        from .pairformer import Transition
        d = c_s + c_s_inputs
        self.sigma_data = sigma_data
        self.norm_single = nn.LayerNorm(d)
        self.single_embed = nn.Linear(d, 2 * c_s)
        self.fourier_embed = FourierEmbedding(dim_fourier)
        self.norm_fourier = nn.LayerNorm(dim_fourier)
        self.fourier_to_single = nn.Linear(dim_fourier, 2 * c_s, bias=False)
        self.transitions = nn.ModuleList([Transition(2 * c_s, 4 * c_s) for _ in range(2)])

    def static_part(self, s_trunk, s_inputs):
        return self.single_embed(self.norm_single(torch.cat([s_trunk, s_inputs], dim=-1)))

    def forward(self, times, static):
        """times: [B] (c_noise); static: [1, N, 2c_s] from :meth:`static_part`."""
        f = self.fourier_to_single(self.norm_fourier(self.fourier_embed(times).to(static.dtype)))
        s = static + f[:, None, :]
        for t in self.transitions:
            s = s + t(s)
        return s


_SEG_CACHE: dict = {}
_WEIGHT_CACHE: dict = {}


def _bf16_weight(lin: nn.Linear) -> torch.Tensor:
    """Contiguous bf16 copy of a bias-free Linear's weight for the GEMM kernel (refreshed when the weight changes)."""
    ent = _WEIGHT_CACHE.get(id(lin))
    if ent is None or ent[0] is not lin.weight or ent[1] != lin.weight._version:
        ent = (lin.weight, lin.weight._version, lin.weight.detach().to(torch.bfloat16).contiguous())
        _WEIGHT_CACHE[id(lin)] = ent
    return ent[2]



def build_segment_tables(atom_to_token: torch.Tensor, n_tokens: int, device) -> tuple:
    """Index tables of one atom layout: padded gather table [N, M], validity and counts for the plain statement,
    an int32 table (-1 = no atom) and an int32 atom -> token map for the kernels."""
    a2t = atom_to_token.detach().cpu()
    counts = torch.bincount(a2t, minlength=n_tokens)
    M = int(counts.max().item())
    order = torch.argsort(a2t, stable=True)
    starts = torch.cumsum(counts, 0) - counts
    idx = starts[:, None] + torch.arange(M)[None, :]
    valid = torch.arange(M)[None, :] < counts[:, None]
    idx = order[idx.clamp(max=a2t.shape[0] - 1)]
    table = torch.where(valid, idx, torch.full_like(idx, -1)).to(torch.int32).contiguous()
    return (idx.to(device), valid.to(device), counts.clamp(min=1).to(device), table.to(device),
            a2t.to(torch.int32).contiguous().to(device))


def _segment_tables(t: torch.Tensor, atom_to_token: torch.Tensor, n_tokens: int):
    """Tables of :func:`build_segment_tables`, built once per ``atom_to_token`` tensor.  A caller that rewrites that
    tensor in place (a captured graph's static input) refreshes the cached tables itself: see
    :func:`refresh_segment_tables`."""
    key = (atom_to_token.data_ptr(), atom_to_token.shape[0], n_tokens, str(t.device))
    tab = _SEG_CACHE.get(key)
    if tab is None:
        tab = build_segment_tables(atom_to_token, n_tokens, t.device)
        if len(_SEG_CACHE) > 64:
            _SEG_CACHE.clear()
        _SEG_CACHE[key] = tab
    return tab


def refresh_segment_tables(static_a2t: torch.Tensor, new_a2t: torch.Tensor, n_tokens: int) -> bool:
    """Rewrite, in place, the cached tables of ``static_a2t`` for a new atom layout (and ``static_a2t`` itself).
    Returns False when the new layout needs tables of another shape (more atoms in some token): the caller must
    then drop whatever captured the old tensors."""
    key = (static_a2t.data_ptr(), static_a2t.shape[0], n_tokens, str(static_a2t.device))
    old = _SEG_CACHE.get(key)
    new = build_segment_tables(new_a2t, n_tokens, static_a2t.device)
    if old is not None and any(o.shape != n.shape for o, n in zip(old, new)):
        return False
    static_a2t.copy_(new_a2t)
    if old is None:
        _SEG_CACHE[key] = new
    else:
        for o, n in zip(old, new):
            o.copy_(n)
    return True


def segment_mean(t: torch.Tensor, atom_to_token: torch.Tensor, n_tokens: int, fused: bool = False) -> torch.Tensor:
    """Mean of atom rows per token, deterministic (no atomics): atoms of a token are gathered through
    a padded [N, M] index table built once per atom layout.  t: [B, A, C] -> [B, N, C].
    Reference kernel with the same job: _seg_reduce_kernel (common/opt_core/opt_core/kernels/dtk_kernels.py)."""
    idx, valid, counts, table, _ = _segment_tables(t, atom_to_token, n_tokens)
    if fused and t.is_cuda and t.dtype == torch.bfloat16 and t.shape[-1] % 8 == 0:
        from ..ops import rows
        return rows.segment_mean(t, table, n_tokens)
    g = t[:, idx]                                              # [B, N, M, C]
    g = g * valid[None, :, :, None].to(t.dtype)
    return (g.float().sum(2) / counts[None, :, None].float()).to(t.dtype)


class AtomTransformer(nn.Module):
    """Holder with upstream's nesting: the windowed atom transformer's layers live under ``diffusion_transformer``
    (boltz2/stock/src/boltz/model/modules/transformersv2.py:211-262), so that checkpoints name them
    ``atom_encoder.diffusion_transformer.layers.N...`` / ``atom_decoder.diffusion_transformer.layers.N...``."""

    def __init__(self, depth: int, c_atom: int, heads: int):
        super().__init__()
        self.diffusion_transformer = DiffusionTransformer(depth, c_atom, c_atom, heads)

    def forward(self, *a, **kw):
        return self.diffusion_transformer(*a, **kw)


class AtomEncoderDecoderBase(nn.Module):
    _holder = "atom_encoder"

    def __init__(self, c_atom: int, c_token: int, depth: int, heads: int):
        super().__init__()
        self.c_atom = c_atom
        setattr(self, self._holder, AtomTransformer(depth, c_atom, heads))

    @property
    def atom_transformer(self) -> "DiffusionTransformer":
        return getattr(self, self._holder).diffusion_transformer


class AtomAttentionEncoder(AtomEncoderDecoderBase):
    def __init__(self, c_atom: int = 128, c_token: int = 768, depth: int = 3, heads: int = 4, structure: bool = True):
        super().__init__(c_atom, c_token, depth, heads)
        self.structure = structure
        if structure:
            self.r_to_q_trans = nn.Linear(3, c_atom, bias=False)
        self.atom_to_token_trans = nn.Sequential(nn.Linear(c_atom, c_token, bias=False), nn.ReLU())

    def forward(self, q0, c, biases, r, atom_to_token, n_tokens, hoisted=None, window=(32, 128)):
        """q0, c: [1, A, c_atom]; r: [B, A, 3]; atom_to_token: [A] long.  Returns (a [B, N, c_token], q, c)."""
        B = r.shape[0]
        q = q0.expand(B, -1, -1)
        if self.structure:
            q = q + self.r_to_q_trans(r.to(q0.dtype))
        q = self.atom_transformer(q, c, biases, hoisted=hoisted, window=window)
        fused = self.atom_transformer.layers[0].impl == "fused" and q.is_cuda and q.dtype == torch.bfloat16
        if fused:
            from ..ops import gemm
            lin = self.atom_to_token_trans[0]
            t = gemm.gemm(q.reshape(-1, q.shape[-1]), _bf16_weight(lin), act="relu").view(B, q.shape[1], -1)
        else:
            t = self.atom_to_token_trans(q)
        a = segment_mean(t, atom_to_token, n_tokens, fused=fused)
        return a, q


class AtomAttentionDecoder(AtomEncoderDecoderBase):
    _holder = "atom_decoder"

    def __init__(self, c_atom: int = 128, c_token: int = 768, depth: int = 3, heads: int = 4):
        super().__init__(c_atom, c_token, depth, heads)
        self.a_to_q_trans = nn.Linear(c_token, c_atom, bias=False)
        self.atom_feat_to_atom_pos_update = nn.Sequential(nn.LayerNorm(c_atom), nn.Linear(c_atom, 3, bias=False))

    def forward(self, a, q, c, biases, atom_to_token, hoisted=None, window=(32, 128)):
        if self.atom_transformer.layers[0].impl == "fused" and q.is_cuda and q.dtype == torch.bfloat16:
            from ..ops import gemm, rows
            B, N, _ = a.shape
            aq = gemm.gemm(a.reshape(B * N, -1), _bf16_weight(self.a_to_q_trans)).view(B, N, -1)
            a2t32 = _segment_tables(q, atom_to_token, N)[4]
            q = rows.gather_rows_add(q, aq, a2t32)
            q = self.atom_transformer(q, c, biases, hoisted=hoisted, window=window)
            # LayerNorm over the atom rows on the row kernel (the library's took 85 us for 63840 x 128), then the
            # 128 -> 3 projection
            ln, lin = self.atom_feat_to_atom_pos_update
            return F.linear(rows.layernorm_rows(q.contiguous(), ln.weight, ln.bias, ln.eps), lin.weight)
        q = q + self.a_to_q_trans(a)[:, atom_to_token]
        q = self.atom_transformer(q, c, biases, hoisted=hoisted, window=window)
        return self.atom_feat_to_atom_pos_update(q)


class DiffusionModule(nn.Module):
    """Denoiser network: atoms -> tokens -> 24-block token transformer -> atoms."""

    def __init__(self, c_s: int = 384, c_z: int = 128, c_atom: int = 128, c_atompair: int = 16,
                 token_depth: int = 24, token_heads: int = 16, atom_depth: int = 3, atom_heads: int = 4,
                 wq: int = 32, wk: int = 128, sigma_data: float = 16.0):
        super().__init__()
        self.c_token = 2 * c_s
        self.window = (wq, wk)
        self.sigma_data = sigma_data
        self.single_conditioner = SingleConditioning(c_s, c_s, sigma_data=sigma_data)
        self.atom_attention_encoder = AtomAttentionEncoder(c_atom, self.c_token, atom_depth, atom_heads)
        self.s_to_a_linear = nn.Sequential(nn.LayerNorm(2 * c_s), nn.Linear(2 * c_s, self.c_token, bias=False))
        self.token_transformer = DiffusionTransformer(token_depth, self.c_token, 2 * c_s, token_heads)
        self.a_norm = nn.LayerNorm(self.c_token)
        self.atom_attention_decoder = AtomAttentionDecoder(c_atom, self.c_token, atom_depth, atom_heads)
        # producers of the step-invariant biases
        self.token_pair_bias = nn.ModuleList(
            [nn.Sequential(nn.LayerNorm(c_z), nn.Linear(c_z, token_heads, bias=False)) for _ in range(token_depth)])
        self.atom_enc_pair_bias = nn.ModuleList(
            [nn.Sequential(nn.LayerNorm(c_atompair), nn.Linear(c_atompair, atom_heads, bias=False))
             for _ in range(atom_depth)])
        self.atom_dec_pair_bias = nn.ModuleList(
            [nn.Sequential(nn.LayerNorm(c_atompair), nn.Linear(c_atompair, atom_heads, bias=False))
             for _ in range(atom_depth)])

    # ---- once per prediction
    def prepare(self, s_trunk, s_inputs, z_cond, atom_q, atom_c, atom_pair, fused: bool = False) -> Dict:
        """Step-invariant tensors.  z_cond: [1, N, N, c_z]; atom_pair: [1, nw, wq, wk, c_atompair]."""
        if fused and z_cond.is_cuda and z_cond.dtype == torch.bfloat16 and z_cond.shape[-1] == 128:
            from ..ops import rows
            from .pairformer import BiasPlanes
            zc = z_cond[0].contiguous()
            tb = [BiasPlanes(rows.pair_head_bias(zc, m[0].weight, m[0].bias, m[1].weight, scale=BiasPlanes.LOG2E))
                  for m in self.token_pair_bias]
        else:
            tb = [m(z_cond).permute(0, 3, 1, 2) for m in self.token_pair_bias]
        eb = [m(atom_pair).permute(0, 4, 1, 2, 3) for m in self.atom_enc_pair_bias]
        db = [m(atom_pair).permute(0, 4, 1, 2, 3) for m in self.atom_dec_pair_bias]
        if fused and atom_pair.is_cuda and self.window == (32, 128):
            eb = [WindowBias(x) for x in eb]
            db = [WindowBias(x) for x in db]
        enc_h = [l.hoist(atom_c) for l in self.atom_attention_encoder.atom_transformer.layers]
        dec_h = [l.hoist(atom_c) for l in self.atom_attention_decoder.atom_transformer.layers]
        return {"token_bias": tb, "enc_bias": eb, "dec_bias": db, "enc_hoist": enc_h, "dec_hoist": dec_h,
                "s_static": self.single_conditioner.static_part(s_trunk, s_inputs), "atom_q": atom_q,
                "atom_c": atom_c}

    # ---- once per step
    def forward(self, r_noisy, times, prep: Dict, atom_to_token, n_tokens: int):
        """r_noisy: [B, A, 3] (already scaled by c_in); times: [B] = c_noise.  Returns r_update [B, A, 3]."""
        B = r_noisy.shape[0]
        r_noisy = r_noisy.to(prep["atom_q"].dtype)
        # every sample of a step sees the same noise level, so the conditioning (and everything hoisted from
        # it) is computed for one row and broadcast over the samples
        s = self.single_conditioner(times[:1], prep["s_static"])                   # [1, N, 2c_s]
        a, q = self.atom_attention_encoder(prep["atom_q"], prep["atom_c"], prep["enc_bias"], r_noisy,
                                           atom_to_token, n_tokens, prep["enc_hoist"], self.window)
        a = a + self.s_to_a_linear(s)
        tt = self.token_transformer
        hoisted = tt.hoist_all(s) if tt.can_hoist_all(s, prep["token_bias"]) else [l.hoist(s) for l in tt.layers]
        a = self.token_transformer(a, s, prep["token_bias"], None, multiplicity=B, hoisted=hoisted)
        a = self.a_norm(a)
        return self.atom_attention_decoder(a, q, prep["atom_c"], prep["dec_bias"], atom_to_token,
                                           prep["dec_hoist"], self.window)


def edm_schedule(num_steps: int, sigma_min=0.0004, sigma_max=160.0, sigma_data=16.0, rho=7.0, device=None):
    inv = 1.0 / rho
    steps = torch.arange(num_steps, device=device, dtype=torch.float32)
    sig = sigma_data * (sigma_max ** inv + steps / (num_steps - 1) * (sigma_min ** inv - sigma_max ** inv)) ** rho
    return F.pad(sig, (0, 1), value=0.0)


def random_rigid(batch: int, device, generator=None, s_trans: float = 1.0):
    """Uniform random rotations (from normalised quaternions) and Gaussian translations."""
    qd = torch.randn((batch, 4), device=device, generator=generator)
    qd = qd / qd.norm(dim=-1, keepdim=True)
    w, x, y, z = qd.unbind(-1)
    Rm = torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w),
                      2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w),
                      2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)], -1).view(batch, 3, 3)
    t = torch.randn((batch, 1, 3), device=device, generator=generator) * s_trans
    return Rm, t


class AtomDiffusion(nn.Module):
    """EDM preconditioning + sampler around :class:`DiffusionModule`."""

    def __init__(self, score_model: DiffusionModule, num_steps: int = 200, gamma_0: float = 0.8,
                 gamma_min: float = 1.0, noise_scale: float = 1.003, step_scale: float = 1.5):
        super().__init__()
        self.score_model = score_model
        self.num_steps, self.gamma_0, self.gamma_min = num_steps, gamma_0, gamma_min
        self.noise_scale, self.step_scale = noise_scale, step_scale
        self.sigma_data = score_model.sigma_data
        # Boltz-2's sampler aligns the noisy coordinates onto the denoised ones before the update
        # ("alignment_reverse_diff"); off unless a configuration asks for it.  The alignment is graph-safe
        # (models/align.py: fixed-sweep Jacobi SVD, no solver call between replays).
        self.align_reverse_diff = False

    def denoise(self, x_noisy, sigma, prep, atom_to_token, n_tokens):
        """Preconditioned network output D(x; sigma).  sigma: [B]."""
        sd = self.sigma_data
        s2 = sigma[:, None, None]
        c_in = 1.0 / torch.sqrt(s2 ** 2 + sd ** 2)
        c_skip = sd ** 2 / (s2 ** 2 + sd ** 2)
        c_out = s2 * sd / torch.sqrt(s2 ** 2 + sd ** 2)
        c_noise = torch.log(sigma / sd) * 0.25
        upd = self.score_model(x_noisy * c_in, c_noise, prep, atom_to_token, n_tokens)
        return c_skip * x_noisy + c_out * upd.float()

    def step(self, x, sigma_tm, sigma_t, gamma, prep, atom_to_token, n_tokens, generator=None):
        """One sampler step for all samples.  x: [B, A, 3] fp32."""
        B = x.shape[0]
        x = x - x.mean(dim=1, keepdim=True)
        Rm, t = random_rigid(B, x.device, generator)
        x = torch.einsum("bij,baj->bai", Rm, x) + t
        t_hat = sigma_tm * (1.0 + gamma)
        eps = self.noise_scale * torch.sqrt(torch.clamp(t_hat ** 2 - sigma_tm ** 2, min=0.0)) * \
            torch.randn(x.shape, device=x.device, generator=generator)
        x_noisy = x + eps
        den = self.denoise(x_noisy, t_hat.expand(B), prep, atom_to_token, n_tokens)
        if self.align_reverse_diff:
            from .align import weighted_rigid_align
            x_noisy = weighted_rigid_align(x_noisy, den)
        d = (x_noisy - den) / t_hat
        return x_noisy + self.step_scale * (sigma_t - t_hat) * d

    @torch.no_grad()
    def sample(self, prep, atom_to_token, n_tokens: int, n_atoms: int, multiplicity: int = 1, num_steps=None,
               generator=None, step_fn=None):
        """Roll the sampler out; ``step_fn`` (a captured CUDA graph wrapper) may replace :meth:`step`."""
        dev = prep["atom_q"].device
        steps = num_steps or self.num_steps
        sig = edm_schedule(steps, sigma_data=self.sigma_data, device=dev)
        gammas = torch.where(sig > self.gamma_min, torch.full_like(sig, self.gamma_0), torch.zeros_like(sig))
        x = sig[0] * torch.randn((multiplicity, n_atoms, 3), device=dev, generator=generator)
        fn = step_fn or (lambda x_, a_, b_, g_: self.step(x_, a_, b_, g_, prep, atom_to_token, n_tokens, generator))
        for i in range(steps):
            x = fn(x, sig[i], sig[i + 1], gammas[i + 1])
        return x
