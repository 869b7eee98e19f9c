"""Protein- and DNA-language-model families: ESM-C, E1, ProGen2 and GPN-Star.

Three block forms cover the four families:

* encoder block (ESM-C, E1, GPN-Star): pre-LayerNorm, one q|k|v projection, LayerNorm over q and over k,
  rotary embedding, bidirectional attention, SwiGLU feed-forward, residuals scaled by a constant.  E1 packs
  several sequences into one row and alternates within-sequence layers with layers that attend over the whole
  row; GPN-Star adds, after the self-attention, a column attention of every position over the clade rows of a
  whole-genome alignment (K / V rows stored once per distinct row, clade -> row index).
* parallel decoder block (ProGen2, GPT-J form): one LayerNorm feeds attention and MLP, rotary on the first
  ``rot`` dims in interleaved pairs, gelu_new MLP, ``x + attn + mlp``; static key / value slots for decoding.

Every block has two statements of the same arithmetic: plain PyTorch (``impl = "reference"``, any device and
dtype) and the kernel path (``impl = "fused"``, CUDA bf16): row kernels for LayerNorm / SwiGLU / gelu_new /
residual sums / rotary split, the tcgen05 GEMM for every projection (residual and bias in its epilogue) and the
tcgen05 attention kernel for bidirectional attention with head dimension 32 or 64.

Reference kits: esmc (residual + LayerNorm kernels, q / k LayerNorm + rotary), e1 (varlen packing, block masks,
key / value cache views), progen2 (kits/v0_ew/kernels.cu:37-209: gelu_new, rotary_split_qkv, residual_add2;
static key / value slots), gpnstar (accel/fused_col.py:56-195: clade K / V de-duplication, column attention).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import reference as ref

LOG2E = 1.4426950408889634


@dataclass(frozen=True)
class PLMConfig:
    name: str
    family: str                  # esmc | e1 | progen2 | gpnstar
    vocab: int
    d_model: int
    layers: int
    heads: int
    ffn: int                     # hidden width (per branch for SwiGLU)
    rot: int                     # rotary dims per head
    causal: bool = False
    global_every: int = 0        # e1: every n-th layer attends across the packed sequences of a row
    clades: int = 0              # gpnstar: clade rows attended per column
    align_rows: int = 0          # gpnstar: distinct alignment rows behind the clades
    eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.d_model // self.heads


CONFIGS: Dict[str, PLMConfig] = {c.name: c for c in [
    PLMConfig("esmc_300m", "esmc", 64, 960, 30, 15, 2560, 64),
    PLMConfig("esmc_600m", "esmc", 64, 1152, 36, 18, 3072, 64),
    PLMConfig("esmc_tiny", "esmc", 64, 128, 2, 2, 256, 64),
    PLMConfig("e1_300m", "e1", 40, 1024, 20, 16, 2816, 64, global_every=2),
    PLMConfig("e1_tiny", "e1", 40, 128, 2, 2, 256, 64, global_every=2),
    PLMConfig("progen2_small", "progen2", 32, 1024, 12, 16, 4096, 32, causal=True),
    PLMConfig("progen2_base", "progen2", 32, 1536, 27, 24, 6144, 48, causal=True),
    PLMConfig("progen2_tiny", "progen2", 32, 128, 2, 2, 512, 32, causal=True),
    PLMConfig("gpnstar_200m", "gpnstar", 8, 1024, 16, 16, 2816, 64, clades=28, align_rows=100),
    PLMConfig("gpnstar_tiny", "gpnstar", 8, 128, 2, 2, 256, 64, clades=6, align_rows=9),
]}

DEFAULT = {"esmc": "esmc_tiny", "e1": "e1_tiny", "progen2": "progen2_tiny", "gpnstar": "gpnstar_tiny"}

AMINO = "ACDEFGHIKLMNPQRSTVWY"
DNA = "ACGT"


def tokenize(text: str, cfg: PLMConfig, device="cpu") -> torch.Tensor:
    """Letters -> ids (4 + index in the family's alphabet; unknown letters map to id 3)."""
    alphabet = DNA if cfg.family == "gpnstar" else AMINO
    lut = {ch: 4 + i for i, ch in enumerate(alphabet)}
    ids = [min(lut.get(ch, 3), cfg.vocab - 1) for ch in text.upper() if not ch.isspace()]
    return torch.tensor([ids or [3]], dtype=torch.long, device=device)


def _kernels_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


def _bf16(w: torch.Tensor) -> torch.Tensor:
    return w.detach().to(torch.bfloat16).contiguous()


def _sdpa(q, k, v, B, L, mask=None, causal=False):
    """q, k, v: [T, H, D] with T = B * L -> [T, H * D]."""
    T, H, D = q.shape
    qh, kh, vh = (t.reshape(B, L, H, D).transpose(1, 2) for t in (q, k, v))
    o = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, is_causal=causal and mask is None)
    return o.transpose(1, 2).reshape(T, H * D)


class EncoderBlock(nn.Module):
    def __init__(self, cfg: PLMConfig, layer: int):
        super().__init__()
        d = cfg.d_model
        self.cfg, self.layer = cfg, layer
        self.ln1 = nn.LayerNorm(d, eps=cfg.eps)
        self.wqkv = nn.Linear(d, 3 * d, bias=False)
        self.q_ln = nn.LayerNorm(d, eps=cfg.eps, bias=False)
        self.k_ln = nn.LayerNorm(d, eps=cfg.eps, bias=False)
        self.wo = nn.Linear(d, d, bias=False)
        self.ln2 = nn.LayerNorm(d, eps=cfg.eps)
        self.w1 = nn.Linear(d, 2 * cfg.ffn, bias=False)
        self.w2 = nn.Linear(cfg.ffn, d, bias=False)
        self.scale = math.sqrt(cfg.layers / 36.0) if cfg.family == "esmc" else 1.0
        self.global_layer = cfg.global_every > 0 and (layer + 1) % cfg.global_every == 0
        if cfg.family == "gpnstar":
            self.ln_c = nn.LayerNorm(d, eps=cfg.eps)
            self.wq_c = nn.Linear(d, d, bias=False)
            self.wkv_c = nn.Linear(d, 2 * d, bias=False)
            self.wo_c = nn.Linear(d, d, bias=False)
            self.clade_bias = nn.Parameter(torch.zeros(cfg.heads, cfg.clades))
        self.impl = "reference"
        self._packed = None

    # -------------------------------------------------------------------------------- plain statements
    def _reference(self, x, pos, mask, align, clade_index):
        cfg = self.cfg
        B, L, d = x.shape
        T = B * L
        H, Dh = cfg.heads, cfg.head_dim
        n = self.ln1(x)
        q, k, v = self.wqkv(n).chunk(3, -1)
        qkv = torch.cat([self.q_ln(q), self.k_ln(k), v], -1).reshape(T, 3 * d)
        q, k, v = (t.to(x.dtype) for t in ref.rotary_split_qkv(qkv, pos, H, cfg.rot))
        x = x + self.wo(_sdpa(q, k, v, B, L, mask)).view(B, L, d) / self.scale
        if cfg.family == "gpnstar":
            R = align.shape[1]
            qc = self.wq_c(self.ln_c(x)).reshape(T, H, Dh)
            kc, vc = self.wkv_c(align).chunk(2, -1)                         # [B, R, L, d]
            kc = kc.permute(1, 0, 2, 3).reshape(R, T, H, Dh)
            vc = vc.permute(1, 0, 2, 3).reshape(R, T, H, Dh)
            oc = ref.column_attention(qc, kc, vc, clade_index, self.clade_bias).to(x.dtype)
            x = x + self.wo_c(oc.reshape(B, L, d))
        a, b = self.w1(self.ln2(x)).chunk(2, -1)
        return x + self.w2(F.silu(a) * b) / self.scale

    # -------------------------------------------------------------------------------- kernel path
    def _pack(self):
        if self._packed is None:
            qs = LOG2E / math.sqrt(self.cfg.head_dim)
            p = {"wqkv": _bf16(self.wqkv.weight), "wo": _bf16(self.wo.weight / self.scale),
                 "w1": _bf16(self.w1.weight), "w2": _bf16(self.w2.weight / self.scale),
                 "q_ln": self.q_ln.weight.detach().float(), "q_ln_scaled": self.q_ln.weight.detach().float() * qs}
            if self.cfg.family == "gpnstar":
                p.update(wq_c=_bf16(self.wq_c.weight), wkv_c=_bf16(self.wkv_c.weight), wo_c=_bf16(self.wo_c.weight))
            ffn = self.w1.weight.shape[0] // 2
            if ffn % 32 == 0:
                # gate | value rows interleaved in groups of 32: silu(a) * b is formed on the GEMM's accumulator
                from ..ops import gemm
                p["w1_swiglu"] = gemm.pack_swiglu(self.w1.weight.detach()[:ffn], self.w1.weight.detach()[ffn:])
            self._packed = p
        return self._packed

    def _fused(self, x, pos, mask, align, clade_index):
        from ..ops import gemm, pair, rows, seq
        cfg = self.cfg
        B, L, d = x.shape
        T = B * L
        H, Dh = cfg.heads, cfg.head_dim
        p = self._pack()
        x2 = x.reshape(T, d)
        n = rows.layernorm_rows(x2, self.ln1.weight, self.ln1.bias, cfg.eps)
        qkv = gemm.gemm(n, p["wqkv"])
        # the attention kernel takes q already multiplied by log2(e) / sqrt(D): folded into the q LayerNorm weight
        own = mask is None and Dh in (32, 64)
        qkv[:, :d] = rows.layernorm_rows(qkv[:, :d].contiguous(), p["q_ln_scaled"] if own else p["q_ln"], None, cfg.eps)
        qkv[:, d:2 * d] = rows.layernorm_rows(qkv[:, d:2 * d].contiguous(), self.k_ln.weight, None, cfg.eps)
        q, k, v = seq.rotary_split_qkv(qkv, pos, H, cfg.rot)
        if own:
            o = torch.empty((T, d), dtype=x.dtype, device=x.device)
            pair.attention(q.view(T, d), k.view(T, d), v.view(T, d), None, None, o, rows=B, Nq=L, Nk=L, H=H, D=Dh)
        else:
            o = _sdpa(q, k, v, B, L, mask)
        x2 = gemm.gemm(o, p["wo"], residual=x2)
        if cfg.family == "gpnstar":
            R = align.shape[1]
            nc = rows.layernorm_rows(x2, self.ln_c.weight, self.ln_c.bias, cfg.eps)
            qc = gemm.gemm(nc, p["wq_c"]).view(T, H, Dh)
            # rows-major alignment [R, T, d] -> K | V of every distinct row from one GEMM
            al = align.permute(1, 0, 2, 3).reshape(R * T, d).contiguous()
            kv = gemm.gemm(al, p["wkv_c"]).view(R, T, 2, H, Dh)
            oc = seq.column_attention(qc, kv[:, :, 0], kv[:, :, 1], clade_index, self.clade_bias)
            x2 = gemm.gemm(oc.view(T, d), p["wo_c"], residual=x2)
        n2 = rows.layernorm_rows(x2, self.ln2.weight, self.ln2.bias, cfg.eps)
        if "w1_swiglu" in p:
            g = gemm.gemm(n2, p["w1_swiglu"], act="swiglu")
        else:
            g = rows.swiglu_rows(gemm.gemm(n2, p["w1"]))
        return gemm.gemm(g, p["w2"], residual=x2).view(B, L, d)

    def forward(self, x, pos, mask=None, align=None, clade_index=None):
        if self.impl == "fused" and _kernels_ok(x):
            return self._fused(x, pos, mask, align, clade_index)
        return self._reference(x, pos, mask, align, clade_index)


class ParallelDecoderBlock(nn.Module):
    """GPT-J form: x + attention(LN x) + MLP(LN x)."""

    def __init__(self, cfg: PLMConfig, layer: int):
        super().__init__()
        d = cfg.d_model
        self.cfg = cfg
        self.ln = nn.LayerNorm(d, eps=cfg.eps)
        self.wqkv = nn.Linear(d, 3 * d, bias=False)
        self.wo = nn.Linear(d, d, bias=False)
        self.fc_in = nn.Linear(d, cfg.ffn)
        self.fc_out = nn.Linear(cfg.ffn, d)
        self.impl = "reference"
        self._packed = None

    def _attend(self, q, k, v, B, L, cache, start):
        """Causal attention; with ``cache`` = (K, V) static slots [B, Lmax, H, D] the new keys are written at
        ``start`` and the queries see slots [0, start + L)."""
        T, H, D = q.shape
        if cache is None:
            return _sdpa(q, k, v, B, L, causal=True)
        K, V = cache
        K[:, start:start + L] = k.view(B, L, H, D)
        V[:, start:start + L] = v.view(B, L, H, D)
        end = start + L
        qh = q.view(B, L, H, D).transpose(1, 2)
        kh, vh = K[:, :end].transpose(1, 2), V[:, :end].transpose(1, 2)
        if L == 1:
            # written out: the library's fused attention re-plans whenever the key length changes, which with a
            # growing prefix is every decode step (milliseconds of host time per call)
            sc = torch.matmul(qh.float(), kh.float().transpose(-1, -2)) * (D ** -0.5)
            o = torch.matmul(torch.softmax(sc, -1).to(vh.dtype), vh)
        else:
            i = torch.arange(L, device=q.device)[:, None] + start
            j = torch.arange(end, device=q.device)[None, :]
            o = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=j <= i)
        return o.transpose(1, 2).reshape(T, H * D)

    def forward(self, x, pos, cache=None, start: int = 0):
        cfg = self.cfg
        B, L, d = x.shape
        T = B * L
        if self.impl == "fused" and _kernels_ok(x):
            from ..ops import gemm, rows, seq
            if self._packed is None:
                self._packed = {"wqkv": _bf16(self.wqkv.weight), "wo": _bf16(self.wo.weight),
                                "fc_in": _bf16(self.fc_in.weight), "fc_out": _bf16(self.fc_out.weight)}
            p = self._packed
            x2 = x.reshape(T, d)
            n = rows.layernorm_rows(x2, self.ln.weight, self.ln.bias, cfg.eps)
            q, k, v = seq.rotary_split_qkv(gemm.gemm(n, p["wqkv"]), pos, cfg.heads, cfg.rot)
            a = gemm.gemm(self._attend(q, k, v, B, L, cache, start), p["wo"])
            h = seq.gelu_new(gemm.gemm(n, p["fc_in"], bias=self.fc_in.bias))
            m = gemm.gemm(h, p["fc_out"], bias=self.fc_out.bias)
            return seq.residual_add2(x2, a, m).view(B, L, d)
        n = self.ln(x)
        q, k, v = (t.to(x.dtype) for t in ref.rotary_split_qkv(self.wqkv(n).reshape(T, 3 * d), pos, cfg.heads, cfg.rot))
        a = self.wo(self._attend(q, k, v, B, L, cache, start)).view(B, L, d)
        m = self.fc_out(ref.gelu_new(self.fc_in(n)).to(x.dtype))
        return x + a + m


class ProteinLM(nn.Module):
    def __init__(self, cfg: PLMConfig):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab, cfg.d_model)
        block = ParallelDecoderBlock if cfg.family == "progen2" else EncoderBlock
        self.blocks = nn.ModuleList([block(cfg, i) for i in range(cfg.layers)])
        self.norm = nn.LayerNorm(cfg.d_model, eps=cfg.eps)
        self.head = nn.Linear(cfg.d_model, cfg.vocab)
        if cfg.family == "gpnstar":
            self.row_embed = nn.Embedding(cfg.vocab, cfg.d_model)
        self.impl = "reference"

    def set_impl(self, impl: str) -> "ProteinLM":
        if impl not in ("reference", "fused"):
            raise ValueError(f"unknown implementation {impl!r}")
        self.impl = impl
        for b in self.blocks:
            b.impl = impl
            b._packed = None
        return self

    @property
    def dtype(self):
        return self.embed.weight.dtype

    # ---------------------------------------------------------------------------------------- forward
    def _masks(self, tokens, seq_ids):
        """E1: sequences packed into one row.  Within-sequence layers see a block-diagonal mask, global layers
        see the whole row; a row holding one sequence needs no mask."""
        if self.cfg.family != "e1" or seq_ids is None:
            return None
        return (seq_ids[:, :, None] == seq_ids[:, None, :]).unsqueeze(1)

    @staticmethod
    def _positions(B, L, seq_ids, device):
        if seq_ids is None:
            return torch.arange(L, device=device).repeat(B)
        # position restarts at every packed sequence: index minus the index of the sequence's first token
        idx = torch.arange(L, device=device).expand(B, L)
        first = torch.where(F.pad(seq_ids[:, 1:] != seq_ids[:, :-1], (1, 0), value=True), idx, 0).cummax(1).values
        return (idx - first).reshape(-1)

    def hidden(self, tokens, seq_ids=None, alignment=None, clade_index=None):
        cfg = self.cfg
        B, L = tokens.shape
        x = self.embed(tokens)
        pos = self._positions(B, L, seq_ids, tokens.device)
        local = self._masks(tokens, seq_ids)
        align = None
        if cfg.family == "gpnstar":
            if alignment is None:
                raise ValueError("gpnstar needs the alignment rows [B, R, L] and the clade -> row index")
            # only the alignment rows that some clade refers to are embedded and projected (per layer the K | V
            # projection of the rows is the largest GEMM of this family): clade -> row becomes clade -> kept row
            uniq, clade_index = torch.unique(clade_index, return_inverse=True)
            align = self.row_embed(alignment[:, uniq])                       # [B, R', L, d], R' <= clades
        for blk in self.blocks:
            if cfg.family == "progen2":
                x = blk(x, pos)
            else:
                x = blk(x, pos, None if blk.global_layer else local, align, clade_index)
        return self.norm(x)

    def forward(self, tokens, seq_ids=None, alignment=None, clade_index=None):
        return self.head(self.hidden(tokens, seq_ids, alignment, clade_index))

    @torch.no_grad()
    def score(self, tokens, **kw) -> torch.Tensor:
        """Mean log-probability of the given tokens: next-token for the causal family, in-place for the masked
        families (one unmasked pass)."""
        logp = torch.log_softmax(self.forward(tokens, **kw).float(), -1)
        if self.cfg.causal:
            return logp[:, :-1].gather(-1, tokens[:, 1:, None]).squeeze(-1).mean(1)
        return logp.gather(-1, tokens[:, :, None]).squeeze(-1).mean(1)

    @torch.no_grad()
    def variant_effect(self, tokens, alignment, clade_index) -> torch.Tensor:
        """GPN-Star ``vep``: per position, log p(allele) - log p(reference allele) for the four bases."""
        logp = torch.log_softmax(self.forward(tokens, alignment=alignment, clade_index=clade_index).float(), -1)
        base = logp[..., 4:8]
        refp = logp.gather(-1, tokens[:, :, None])
        return base - refp

    # ---------------------------------------------------------------------------------------- decoding
    def make_cache(self, batch: int, max_len: int, device=None):
        cfg = self.cfg
        device = device or self.embed.weight.device
        shape = (batch, max_len, cfg.heads, cfg.head_dim)
        return [(torch.zeros(shape, dtype=self.dtype, device=device), torch.zeros(shape, dtype=self.dtype, device=device))
                for _ in range(cfg.layers)]

    @torch.no_grad()
    def generate(self, tokens, max_new_tokens: int, temperature: float = 0.0, top_p: float = 1.0,
                 generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """Static key / value slots sized once for prompt + new tokens; greedy at temperature 0, otherwise
        nucleus sampling from ``generator`` (the draws depend only on the generator state, not on the path)."""
        if self.cfg.family != "progen2":
            raise ValueError("generate is defined for the causal family")
        B, L0 = tokens.shape
        cache = self.make_cache(B, L0 + max_new_tokens, tokens.device)
        out = [tokens]
        cur, start = tokens, 0
        for _ in range(max_new_tokens):
            L = cur.shape[1]
            x = self.embed(cur)
            pos = (torch.arange(L, device=tokens.device) + start).repeat(B)
            for blk, c in zip(self.blocks, cache):
                x = blk(x, pos, c, start)
            logits = self.head(self.norm(x[:, -1])).float()
            if temperature <= 0.0:
                nxt = logits.argmax(-1, keepdim=True)
            else:
                pr = torch.softmax(logits / temperature, -1)
                sp, si = pr.sort(-1, descending=True)
                keep = sp.cumsum(-1) - sp < top_p
                sp = torch.where(keep, sp, torch.zeros_like(sp))
                nxt = si.gather(-1, torch.multinomial(sp / sp.sum(-1, keepdim=True), 1, generator=generator))
            out.append(nxt)
            start += L
            cur = nxt
        return torch.cat(out, 1)


def build(config: str, device="cpu", dtype=torch.float32, seed: int = 0, impl: Optional[str] = None) -> ProteinLM:
    cfg = CONFIGS[config]
    g = torch.Generator().manual_seed(seed)
    m = ProteinLM(cfg)
    with torch.no_grad():
        for name, p in m.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g) * (0.5 / math.sqrt(p.shape[-1])))
            elif name.endswith("clade_bias"):
                p.copy_(torch.randn(p.shape, generator=g) * 0.1)
    m = m.to(device=device, dtype=dtype).eval()
    if impl is None:
        impl = "fused" if (str(device).startswith("cuda") and dtype == torch.bfloat16) else "reference"
    return m.set_impl(impl)


def synthetic_alignment(cfg: PLMConfig, tokens: torch.Tensor, seed: int = 0):
    """Alignment rows [B, R, L] that agree with the target at most columns, and a clade -> row index [C]."""
    g = torch.Generator().manual_seed(seed)
    B, L = tokens.shape
    R, C = cfg.align_rows, cfg.clades
    noise = torch.randint(4, 8, (B, R, L), generator=g)
    keep = torch.rand((B, R, L), generator=g) < 0.8
    align = torch.where(keep, tokens.cpu()[:, None, :].expand(B, R, L), noise)
    index = torch.randint(0, R, (C,), generator=g).sort().values
    return align.to(tokens.device), index.to(tokens.device)


def with_layers(cfg: PLMConfig, layers: int) -> PLMConfig:
    return replace(cfg, layers=layers)
