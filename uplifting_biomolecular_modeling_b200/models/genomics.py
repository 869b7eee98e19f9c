"""Genomic track models: Enformer, Borzoi / Flashzoi and ChromBPNet.

Activations are channels-last ``[B, L, C]`` everywhere, which turns every convolution into a GEMM on the
tcgen05 kernel without an im2col copy: a width-K convolution reads the (zero-padded) sequence through an
overlapping-row view ``A[l, (t, c)] = x[l + t, c]`` (row stride C, row length K * C) against the weight
``[C_out, K * C]``.  Dilated convolutions concatenate their taps (three shifted views) and put ReLU and the
cropped residual into the GEMM epilogue.  Around the GEMMs run the row kernels: folded batch-norm + GELU,
attention pooling / max pooling of width 2, bias + residual, and the softmax over content + relative-position
logits that reads the positional logits at their shifted index.

Each model has two statements of the same arithmetic: ``impl = "reference"`` (plain PyTorch convolutions, any
device / dtype) and ``impl = "fused"`` (CUDA bf16, the kernels above).

Reference kits: enformer (kits/v0_2/enformer_xattn.cu:24-99 content + positional softmax and band GEMM,
enformer_fastkit.py:96-157 bn_gelu / pool / bias_residual), enformer_deepmind (ops/edm_*.cc: scale-shift-GELU,
softmax pooling, relative-shift softmax, bias + residual), borzoi / flashzoi, chrombpnet (im2col dot, serial
head and global-average-pool kernels).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import reference as ref


def _kernels_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


def _bf16(w: torch.Tensor) -> torch.Tensor:
    return w.detach().to(torch.bfloat16).contiguous()


_ONE_HOT_LUT = None


def one_hot_dna(text: str, device="cpu", dtype=torch.float32, channels: int = 8) -> torch.Tensor:
    """ACGT -> one-hot [1, L, channels] (channels >= 4; the extra channels stay zero so rows are 16 bytes; any other
    letter is an all-zero row).  One table lookup over the raw bytes: no per-character loop."""
    global _ONE_HOT_LUT
    if _ONE_HOT_LUT is None:
        lut = torch.zeros((256, 4))
        for i, ch in enumerate("ACGT"):
            lut[ord(ch), i] = 1
            lut[ord(ch.lower()), i] = 1
        _ONE_HOT_LUT = lut
    raw = torch.frombuffer(bytearray(text.encode("latin-1", "replace")), dtype=torch.uint8).long()
    x = torch.zeros((1, raw.numel(), channels), dtype=dtype)
    x[0, :, :4] = _ONE_HOT_LUT[raw].to(dtype)
    return x.to(device)


# ------------------------------------------------------------------------------------------ convolution as a GEMM
class ConvCL(nn.Module):
    """1-D convolution on channels-last rows.  weight: [C_out, K, C_in]; ``same`` padding unless ``valid``."""

    def __init__(self, c_in: int, c_out: int, k: int, dilation: int = 1, bias: bool = True, valid: bool = False):
        super().__init__()
        self.c_in, self.c_out, self.k, self.dilation, self.valid = c_in, c_out, k, dilation, valid
        self.weight = nn.Parameter(torch.empty(c_out, k, c_in))
        self.bias = nn.Parameter(torch.zeros(c_out)) if bias else None
        self._w2 = None

    def out_len(self, L: int) -> int:
        return L - (self.k - 1) * self.dilation if self.valid else L

    def reference(self, x, act=None, residual=None):
        pad = 0 if self.valid else (self.k // 2) * self.dilation
        y = F.conv1d(x.transpose(1, 2), self.weight.permute(0, 2, 1).to(x.dtype),
                     None if self.bias is None else self.bias.to(x.dtype), padding=pad, dilation=self.dilation)
        y = y.transpose(1, 2)
        if act == "relu":
            y = F.relu(y)
        elif act == "gelu":
            y = F.gelu(y)
        return y if residual is None else y + residual

    def fused(self, x, act=None, residual=None):
        """x: bf16 [B, L, C_in] -> bf16 [B, L_out, C_out] = act(conv(x) + bias) + residual."""
        from ..ops import gemm
        B, L, C = x.shape
        k, d = self.k, self.dilation
        if self._w2 is None:
            cp = (self.c_out + 7) // 8 * 8                     # pad tiny heads (one output channel) to 8 columns
            w2 = torch.zeros((cp, k * C), dtype=x.dtype, device=x.device)
            w2[:self.c_out] = self.weight.detach().reshape(self.c_out, k * C).to(x.dtype)
            b2 = None
            if self.bias is not None:
                b2 = torch.zeros(cp, dtype=torch.float32, device=x.device)
                b2[:self.c_out] = self.bias.detach().float()
            self._w2 = (w2, b2, cp)
        w2, b2, cp = self._w2
        Lo = self.out_len(L)
        if not self.valid and k > 1:
            x = F.pad(x, (0, 0, (k // 2) * d, (k // 2) * d))
        Lp = x.shape[1]
        res2 = None if residual is None else residual.reshape(B * Lo, cp)
        if k == 1:
            y = gemm.gemm(x.reshape(B * Lp, C), w2, bias=b2, act=act, residual=res2)
            return y.view(B, Lo, cp)[..., :self.c_out]
        x = x.contiguous()
        if d == 1 and C % 8 == 0:
            # overlapping-row view over the flattened batch: windows that straddle two sequences are computed and
            # dropped (k - 1 rows per sequence)
            rows_all = B * Lp - (k - 1)
            a = x.as_strided((rows_all, k * C), (C, 1))
            if B == 1:
                y = gemm.gemm(a, w2, bias=b2, act=act, residual=res2)
                return y.view(1, Lo, cp)[..., :self.c_out]
            y = torch.empty((B * Lp, cp), dtype=x.dtype, device=x.device)
            gemm.gemm(a, w2, bias=b2, act=act, out=y[:rows_all])
            y = y.view(B, Lp, cp)[:, :Lo]
            if residual is not None:
                y = y + residual
            return y[..., :self.c_out]
        # dilated taps: shifted views side by side, one GEMM, activation and residual in its epilogue
        a = torch.cat([x[:, t * d:t * d + Lo] for t in range(k)], -1).reshape(B * Lo, k * C)
        y = gemm.gemm(a, w2, bias=b2, act=act, residual=res2)
        return y.view(B, Lo, cp)[..., :self.c_out]


class BNAct(nn.Module):
    """Inference batch-norm folded to scale / shift, followed by GELU (erf form)."""

    def __init__(self, c: int):
        super().__init__()
        self.register_buffer("scale", torch.ones(c))
        self.register_buffer("shift", torch.zeros(c))

    def forward(self, x, fused: bool):
        if fused:
            from ..ops import seq
            return seq.scale_shift_gelu(x, self.scale, self.shift)
        return F.gelu(x.float() * self.scale.float() + self.shift.float()).to(x.dtype)


class ConvBlock(nn.Module):
    """batch-norm -> GELU -> convolution (+ residual)."""

    def __init__(self, c_in, c_out, k, residual: bool = False):
        super().__init__()
        self.norm = BNAct(c_in)
        self.conv = ConvCL(c_in, c_out, k)
        self.residual = residual

    def forward(self, x, fused: bool):
        h = self.norm(x, fused)
        r = x if self.residual else None
        return self.conv.fused(h, residual=r) if fused else self.conv.reference(h, residual=r)


class Pool2(nn.Module):
    """Width-2 pooling along the sequence: ``attention`` (softmax of per-channel logits x W, W near 2 I) or ``max``."""

    def __init__(self, c: int, mode: str):
        super().__init__()
        self.mode = mode
        if mode == "attention":
            self.logit = nn.Linear(c, c, bias=False)
        self._w = None

    def forward(self, x, fused: bool):
        if x.shape[1] % 2:
            x = x[:, :-1]
        if self.mode == "max":
            if fused:
                from ..ops import seq
                return seq.pool2(x, "max")
            return ref.pool2(x, "max").to(x.dtype)
        if fused:
            from ..ops import gemm, seq
            if self._w is None:
                self._w = _bf16(self.logit.weight)
            B, L, C = x.shape
            w = gemm.gemm(x.reshape(B * L, C), self._w).view(B, L, C)
            return seq.pool2(x, "softmax", w)
        return ref.pool2(x, "softmax", self.logit(x)).to(x.dtype)


# ------------------------------------------------------------------------------------------ relative-position attention
def positional_features(L: int, feats: int, device, dtype=torch.float32) -> torch.Tensor:
    """[2L - 1, feats]: exponential-decay and central-mask bases of |distance| and their signed copies."""
    if feats % 4:
        raise ValueError("the number of positional features must be a multiple of 4")
    nb = feats // 4
    dist = torch.arange(-(L - 1), L, device=device, dtype=torch.float32)
    a = dist.abs()
    half = torch.exp(torch.linspace(math.log(3.0), math.log(max(4.0, float(L))), nb, device=device))
    expo = torch.exp(-math.log(2.0) / half[None, :] * a[:, None])
    width = 2.0 ** torch.arange(1, nb + 1, device=device, dtype=torch.float32) - 1
    mask = (width[None, :] > a[:, None]).float()
    base = torch.cat([expo, mask], -1)
    return torch.cat([base, torch.sign(dist)[:, None] * base], -1).to(dtype)


class RelPosAttention(nn.Module):
    """Multi-head attention with content and relative-position logits:
    softmax((q + u) k^T + shift((q + w) r^T)) v, r = W_r positional_features."""

    def __init__(self, dim: int, heads: int, dim_key: int, dim_value: int, feats: int):
        super().__init__()
        self.heads, self.dk, self.dv, self.feats = heads, dim_key, dim_value, feats
        self.wq = nn.Linear(dim, heads * dim_key, bias=False)
        self.wk = nn.Linear(dim, heads * dim_key, bias=False)
        self.wv = nn.Linear(dim, heads * dim_value, bias=False)
        self.wr = nn.Linear(feats, heads * dim_key, bias=False)
        self.wo = nn.Linear(heads * dim_value, dim)
        self.u = nn.Parameter(torch.zeros(heads, dim_key))
        self.w = nn.Parameter(torch.zeros(heads, dim_key))
        self._packed = None

    def reference(self, x):
        B, L, _ = x.shape
        H, dk, dv = self.heads, self.dk, self.dv
        q = self.wq(x).view(B, L, H, dk).transpose(1, 2).float() * dk ** -0.5
        k = self.wk(x).view(B, L, H, dk).transpose(1, 2).float()
        v = self.wv(x).view(B, L, H, dv).transpose(1, 2).float()
        r = self.wr(positional_features(L, self.feats, x.device, x.dtype)).view(2 * L - 1, H, dk).transpose(0, 1).float()
        content = torch.einsum("bhid,bhjd->bhij", q + self.u.float()[None, :, None], k)
        pos = torch.einsum("bhid,hpd->bhip", q + self.w.float()[None, :, None], r)
        p = ref.relshift_softmax(content, pos)
        o = torch.einsum("bhij,bhjd->bhid", p, v).transpose(1, 2).reshape(B, L, H * dv)
        return self.wo(o.to(x.dtype))

    def fused(self, x, residual):
        """x: LayerNorm output, residual: the block input; returns residual + attention(x)."""
        from ..ops import gemm, seq
        B, L, dim = x.shape
        H, dk, dv = self.heads, self.dk, self.dv
        if self._packed is None:
            wqk = torch.cat([self.wq.weight * dk ** -0.5, self.wk.weight], 0)
            self._packed = {"wqk": _bf16(wqk), "wv": _bf16(self.wv.weight), "wr": _bf16(self.wr.weight),
                            "wo": _bf16(self.wo.weight), "rel": {}}
        p = self._packed
        if L not in p["rel"]:
            # relative-position keys depend on the length only: [H, 2L, dk] (one zero row of padding keeps rows of
            # the positional logits a multiple of 8 wide)
            f = positional_features(L, self.feats, x.device, x.dtype)
            r = gemm.gemm(f, p["wr"]).view(2 * L - 1, H, dk).permute(1, 0, 2)
            rp = torch.zeros((H, 2 * L, dk), dtype=x.dtype, device=x.device)
            rp[:, :2 * L - 1] = r
            p["rel"][L] = rp
        rel = p["rel"][L]
        x2 = x.reshape(B * L, dim)
        qk = gemm.gemm(x2, p["wqk"]).view(B, L, 2, H, dk)
        v = gemm.gemm(x2, p["wv"]).view(B, L, H, dv)
        outs = []
        for b in range(B):
            q = qk[b, :, 0].permute(1, 0, 2).float()                                  # [H, L, dk]
            k = qk[b, :, 1].permute(1, 0, 2).contiguous()
            qu = (q + self.u.float()[:, None]).to(x.dtype)
            qw = (q + self.w.float()[:, None]).to(x.dtype)
            content = gemm.gemm(qu, k, out_dtype=torch.float32)                       # [H, L, L]
            pos = gemm.gemm(qw, rel, out_dtype=torch.float32)                         # [H, L, 2L]
            prob = seq.relshift_softmax(content, pos).to(x.dtype)
            vt = v[b].permute(1, 2, 0)                                                # [H, dv, L]
            if L % 8:
                # operand rows of the GEMM are multiples of 8 elements: zero keys at the end
                prob, vt = F.pad(prob, (0, 8 - L % 8)), F.pad(vt, (0, 8 - L % 8))
            vt = vt.contiguous()
            outs.append(gemm.gemm(prob, vt).permute(1, 0, 2).reshape(L, H * dv))      # [L, H * dv]
        o = torch.cat(outs, 0) if B > 1 else outs[0]
        return gemm.gemm(o, p["wo"], bias=self.wo.bias, residual=residual.reshape(B * L, dim)).view(B, L, dim)


class TrackTransformerLayer(nn.Module):
    def __init__(self, dim, heads, dim_key, feats, rotary: bool = False):
        super().__init__()
        self.ln1 = nn.LayerNorm(dim)
        self.rotary = rotary
        if rotary:
            self.heads = heads
            self.wqkv = nn.Linear(dim, 3 * dim, bias=False)
            self.wo = nn.Linear(dim, dim)
        else:
            self.attn = RelPosAttention(dim, heads, dim_key, dim // heads, feats)
        self.ln2 = nn.LayerNorm(dim)
        self.fc1 = nn.Linear(dim, 2 * dim)
        self.fc2 = nn.Linear(2 * dim, dim)
        self._packed = None

    def _rotary_attention(self, n, x, fused):
        """Flashzoi form: rotary q / k and plain softmax attention."""
        B, L, dim = n.shape
        H = self.heads
        pos = torch.arange(L, device=n.device).repeat(B)
        if fused:
            from ..ops import gemm, pair, seq
            Dh = dim // H
            own = Dh in (32, 64)
            p = self._packed
            q, k, v = seq.rotary_split_qkv(gemm.gemm(n.reshape(B * L, dim), p["wqkv_s" if own else "wqkv"]), pos, H, Dh)
            if own:
                o = torch.empty((B * L, dim), dtype=n.dtype, device=n.device)
                pair.attention(q.view(B * L, dim), k.view(B * L, dim), v.view(B * L, dim), None, None, o, rows=B,
                               Nq=L, Nk=L, H=H, D=Dh)
            else:
                qh, kh, vh = (t.view(B, L, H, Dh).transpose(1, 2) for t in (q, k, v))
                o = F.scaled_dot_product_attention(qh, kh, vh).transpose(1, 2).reshape(B * L, dim)
            return gemm.gemm(o, p["wo"], bias=self.wo.bias, residual=x.reshape(B * L, dim)).view(B, L, dim)
        Dh = dim // H
        q, k, v = (t.to(n.dtype) for t in ref.rotary_split_qkv(self.wqkv(n).reshape(B * L, 3 * dim), pos, H, Dh))
        qh, kh, vh = (t.view(B, L, H, Dh).transpose(1, 2) for t in (q, k, v))
        o = F.scaled_dot_product_attention(qh, kh, vh).transpose(1, 2).reshape(B, L, dim)
        return x + self.wo(o)

    def forward(self, x, fused: bool):
        B, L, dim = x.shape
        if fused:
            from ..ops import gemm, rows
            if self._packed is None:
                self._packed = {"fc1": _bf16(self.fc1.weight), "fc2": _bf16(self.fc2.weight)}
                if self.rotary:
                    Dh = dim // self.heads
                    ws = self.wqkv.weight.detach().clone()
                    ws[:dim] *= 1.4426950408889634 / math.sqrt(Dh)     # the attention kernel's q scale
                    self._packed.update(wqkv=_bf16(self.wqkv.weight), wqkv_s=_bf16(ws), wo=_bf16(self.wo.weight))
            p = self._packed
            x = x.contiguous()
            n = rows.layernorm_rows(x, self.ln1.weight, self.ln1.bias, self.ln1.eps)
            x = self._rotary_attention(n, x, True) if self.rotary else self.attn.fused(n, x)
            x2 = x.reshape(B * L, dim)
            n2 = rows.layernorm_rows(x2, self.ln2.weight, self.ln2.bias, self.ln2.eps)
            h = gemm.gemm(n2, p["fc1"], bias=self.fc1.bias, act="relu")
            return gemm.gemm(h, p["fc2"], bias=self.fc2.bias, residual=x2).view(B, L, dim)
        n = self.ln1(x)
        x = self._rotary_attention(n, x, False) if self.rotary else x + self.attn.reference(n)
        return x + self.fc2(F.relu(self.fc1(self.ln2(x))))


# ------------------------------------------------------------------------------------------ models
@dataclass(frozen=True)
class TrackConfig:
    name: str
    family: str                  # enformer | borzoi | flashzoi | chrombpnet
    dim: int = 1536
    tower: int = 6               # pooling stages after the stem (each halves the length)
    layers: int = 11
    heads: int = 8
    dim_key: int = 64
    feats: int = 192             # positional features (enformer: dim / heads)
    tracks: int = 5313
    crop: int = 320              # bins dropped on each side of the transformer output
    unet: int = 0                # borzoi: up-sampling stages with skips
    filters: int = 512           # chrombpnet
    dilated: int = 8
    out_len: int = 1000


CONFIGS: Dict[str, TrackConfig] = {c.name: c for c in [
    TrackConfig("enformer", "enformer"),
    TrackConfig("enformer_tiny", "enformer", dim=128, tower=2, layers=1, heads=2, dim_key=64, feats=64, tracks=16, crop=2),
    TrackConfig("borzoi", "borzoi", dim=1536, tower=6, layers=8, heads=8, dim_key=64, feats=32, tracks=7611, crop=0, unet=2),
    TrackConfig("borzoi_tiny", "borzoi", dim=128, tower=3, layers=1, heads=2, dim_key=64, feats=32, tracks=16, crop=0, unet=2),
    TrackConfig("flashzoi", "flashzoi", dim=1536, tower=6, layers=8, heads=24, dim_key=64, tracks=7611, crop=0, unet=2),
    TrackConfig("flashzoi_tiny", "flashzoi", dim=128, tower=3, layers=1, heads=2, dim_key=64, tracks=16, crop=0, unet=2),
    TrackConfig("chrombpnet", "chrombpnet", filters=512, dilated=8, out_len=1000),
    TrackConfig("chrombpnet_tiny", "chrombpnet", filters=64, dilated=3, out_len=64),
]}

DEFAULT = {"enformer": "enformer_tiny", "enformer_deepmind": "enformer_tiny", "borzoi": "borzoi_tiny",
           "flashzoi": "flashzoi_tiny", "chrombpnet": "chrombpnet_tiny"}


class TrackModel(nn.Module):
    """Enformer / Borzoi / Flashzoi: convolutional tower with width-2 pooling, transformer over the pooled bins,
    optional U-net up-sampling with skips (Borzoi), pointwise convolution + GELU, softplus track heads."""

    def __init__(self, cfg: TrackConfig):
        super().__init__()
        self.cfg = cfg
        dim = cfg.dim
        half = dim // 2
        pool = "attention" if cfg.family == "enformer" else "max"
        self.stem = ConvCL(8, half, 15)
        self.stem_res = ConvBlock(half, half, 1, residual=True)
        self.stem_pool = Pool2(half, pool)
        widths = [int(round(half * (dim / half) ** (i / max(1, cfg.tower - 1)) / 8)) * 8 for i in range(cfg.tower)]
        widths[-1] = dim
        self.tower = nn.ModuleList()
        c = half
        for w in widths:
            self.tower.append(nn.ModuleList([ConvBlock(c, w, 5), ConvBlock(w, w, 1, residual=True), Pool2(w, pool)]))
            c = w
        self.widths = widths
        rotary = cfg.family == "flashzoi"
        self.layers = nn.ModuleList([TrackTransformerLayer(dim, cfg.heads, cfg.dim_key, cfg.feats, rotary)
                                     for _ in range(cfg.layers)])
        if cfg.unet:
            # stage s fuses the up-sampled trunk with the tower output that has the same length
            self.up_trunk = nn.ModuleList([ConvBlock(dim, dim, 1) for _ in range(cfg.unet)])
            self.up_skip = nn.ModuleList([ConvBlock(widths[-1 - s], dim, 1) for s in range(cfg.unet)])
            self.up_mix = nn.ModuleList([ConvBlock(dim, dim, 3) for _ in range(cfg.unet)])
        self.final = ConvBlock(dim, 2 * dim, 1)
        self.head = nn.Linear(2 * dim, cfg.tracks)
        self.impl = "reference"
        self._head_w = None

    def set_impl(self, impl):
        self.impl = impl
        return self

    def forward(self, x):
        """x: one-hot [B, L, 8] (channels 4..7 zero) -> tracks [B, bins, tracks]."""
        cfg = self.cfg
        fused = self.impl == "fused" and _kernels_ok(x)
        x = self.stem.fused(x) if fused else self.stem.reference(x)
        x = self.stem_pool(self.stem_res(x, fused), fused)
        skips: List[torch.Tensor] = []
        for conv, res, pool in self.tower:
            x = res(conv(x, fused), fused)
            skips.append(x)
            x = pool(x, fused)
        for layer in self.layers:
            x = layer(x, fused)
        for s in range(cfg.unet):
            # the tower output before pooling stage -(s + 1) is twice as long as the trunk at this point
            x = self.up_trunk[s](x, fused).repeat_interleave(2, dim=1)
            skip = skips[-1 - s]
            x = x[:, :skip.shape[1]] + self._skip(s, skip, fused)
            x = self.up_mix[s](x, fused)
        if cfg.crop:
            x = x[:, cfg.crop:x.shape[1] - cfg.crop]
        x = self.final(x, fused)
        B, L, C = x.shape
        if fused:
            from ..ops import gemm
            if self._head_w is None:
                self._head_w = _bf16(self.head.weight)
            h = F.gelu(x.float()).to(x.dtype).reshape(B * L, C)
            y = gemm.gemm(h, self._head_w, bias=self.head.bias, out_dtype=torch.float32).view(B, L, -1)
        else:
            y = self.head(F.gelu(x.float()).to(x.dtype)).float()
        return F.softplus(y)

    def _skip(self, s, skip, fused):
        blk = self.up_skip[s]
        if blk.conv.c_in != skip.shape[-1]:
            raise ValueError("skip width does not match the up-sampling stage")
        return blk(skip, fused)


class ChromBPNet(nn.Module):
    """BPNet-form bias-factorised accessibility model: first convolution (width 21), dilated residual tower
    (width 3, dilation 2^i, valid padding, cropped residual), profile head (width 75) and count head (global
    average pool + linear)."""

    def __init__(self, cfg: TrackConfig):
        super().__init__()
        self.cfg = cfg
        f = cfg.filters
        self.first = ConvCL(8, f, 21, valid=True)
        self.dilated = nn.ModuleList([ConvCL(f, f, 3, dilation=2 ** (i + 1), valid=True) for i in range(cfg.dilated)])
        self.profile = ConvCL(f, 1, 75, valid=True)
        self.count = nn.Linear(f, 1)
        self.impl = "reference"

    def set_impl(self, impl):
        self.impl = impl
        return self

    @property
    def receptive_trim(self) -> int:
        return 20 + sum(2 * 2 ** (i + 1) for i in range(self.cfg.dilated)) + 74

    def forward(self, x):
        """x: one-hot [B, L, 8] -> (profile logits [B, out_len], log counts [B])."""
        fused = self.impl == "fused" and _kernels_ok(x)
        x = self.first.fused(x, act="relu") if fused else self.first.reference(x, act="relu")
        for conv in self.dilated:
            d = conv.dilation
            Lo = conv.out_len(x.shape[1])
            crop = x[:, d:d + Lo]
            x = conv.fused(x, act="relu", residual=crop.contiguous()) if fused else conv.reference(x, "relu", crop)
        prof = (self.profile.fused(x) if fused else self.profile.reference(x)).squeeze(-1).float()
        start = (prof.shape[1] - self.cfg.out_len) // 2
        prof = prof[:, start:start + self.cfg.out_len]
        pooled = x.float().mean(1)
        counts = (pooled @ self.count.weight.float().t() + self.count.bias.float()).squeeze(-1)
        return prof, counts


def build(config: str, device="cpu", dtype=torch.float32, seed: int = 0, impl: Optional[str] = None):
    cfg = CONFIGS[config]
    g = torch.Generator().manual_seed(seed)
    m = ChromBPNet(cfg) if cfg.family == "chrombpnet" else TrackModel(cfg)
    with torch.no_grad():
        for name, p in m.named_parameters():
            if name.endswith(("logit.weight",)):
                p.copy_(2.0 * torch.eye(p.shape[0]) + 0.01 * torch.randn(p.shape, generator=g))
            elif p.dim() >= 2:
                fan = p[0].numel()
                p.copy_(torch.randn(p.shape, generator=g) * (0.7 / math.sqrt(fan)))
            elif name.endswith((".u", ".w")):
                p.copy_(torch.randn(p.shape, generator=g) * 0.1)
        for name, b in m.named_buffers():
            if name.endswith("scale"):
                b.copy_(1.0 + 0.1 * torch.randn(b.shape, generator=g))
            elif name.endswith("shift"):
                b.copy_(0.1 * torch.randn(b.shape, generator=g))
    m = m.to(device=device, dtype=dtype).eval()
    if impl is None:
        impl = "fused" if (str(device).startswith("cuda") and dtype == torch.bfloat16) else "reference"
    return m.set_impl(impl)


def input_length(cfg: TrackConfig, bins: int = 8) -> int:
    """A sequence length that the configuration accepts: ``bins`` transformer bins for the tower models, the
    output window plus the receptive-field trim for ChromBPNet."""
    if cfg.family == "chrombpnet":
        return cfg.out_len + 20 + sum(2 * 2 ** (i + 1) for i in range(cfg.dilated)) + 74
    return (bins + 2 * cfg.crop) * 2 ** (cfg.tower + 1)
