"""Evo2-shaped genomic language model: a StripedHyena-2 decoder (gated short / medium / long
convolution operators interleaved with multi-head attention, SwiGLU MLPs, byte vocabulary).

Shape facts follow the reference's stock configuration (evo2/stock/src/evo2/configs/evo2-7b-1m.yml:
hidden 4096, 32 layers, attention at layers 3/10/17/24/31 with 32 heads, the remaining layers cycling
short (7-tap FIR), medium (128-tap FIR) and long (implicit, pole/residue) Hyena operators, vocabulary
512) and the benchmark configuration (SwiGLU width 11008).  Each Hyena operator is
``out( x2 * conv(x1 * v) )`` after a 3-tap depthwise FIR on the 3d-wide input projection (the reference's
kernels for the same pieces: evo2/opt/evo2_opt/kit/base.py:55 ``_fir3_kernel``, :160 ``_hcs7_kernel_s``,
:219/:242 FFT-convolution epilogues, gen/hyenafuse for the decode-step state update).

Prefill runs the medium / long operators as FFT convolutions; decoding keeps per-layer state (FIR
tails, pole states, attention KV cache) and advances one token per step.  Tensor parallelism shards
the channel dimension of every operator (``parallel.tp``): column-parallel input projections, row-parallel
output projections whose reduce-scatter is done by the GEMM epilogue over peer memory.  The causal attention
of the five attention layers is the library's fused attention; the package's own tcgen05 causal kernel
(``ops/causal.py``, head dimension 128) is measured slower than it and is taken only on request.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, replace
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass(frozen=True)
class Evo2Config:
    name: str = "evo2_7b"
    d_model: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    ffn: int = 11008
    vocab: int = 512
    attn_layers: Tuple[int, ...] = (3, 10, 17, 24, 31)
    short_len: int = 7
    medium_len: int = 128
    state_dim: int = 16            # poles per channel of the long operator
    fir_len: int = 3               # depthwise FIR on the input projection
    rope_base: float = 10000.0
    eps: float = 1e-6

    def layer_kind(self, i: int) -> str:
        if i in self.attn_layers:
            return "attn"
        k = [j for j in range(self.n_layers) if j not in self.attn_layers].index(i) % 3
        return ("hcs", "hcm", "hcl")[k]


CONFIGS: Dict[str, Evo2Config] = {
    "evo2_7b": Evo2Config(),
    "evo2_1b": Evo2Config(name="evo2_1b", d_model=1920, n_layers=25, n_heads=15, ffn=5120,
                          attn_layers=(3, 10, 17, 24)),
    "evo2_tiny": Evo2Config(name="evo2_tiny", d_model=128, n_layers=4, n_heads=4, ffn=256, attn_layers=(3,),
                            medium_len=16, state_dim=4),
}


def _fusable(mod, x: torch.Tensor) -> bool:
    """The kernel path serves bf16 activations on the GPU whose channel count is a multiple of 8."""
    return getattr(mod, "impl", "torch") == "fused" and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0


class RMSNorm(nn.Module):
    def __init__(self, d: int, eps: float = 1e-6):
        super().__init__()
        self.scale = nn.Parameter(torch.ones(d))
        self.eps = eps
        self.impl = "torch"

    def forward(self, x):
        if _fusable(self, x):
            from ..ops import seq
            return seq.rmsnorm_rows(x, self.scale, self.eps)
        x32 = x.float()
        y = x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + self.eps)
        return (y * self.scale.float()).to(x.dtype)


def causal_fir(x: torch.Tensor, h: torch.Tensor, tail: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Depthwise causal FIR.  x: [B, L, C]; h: [C, K] (h[:, 0] multiplies the current sample); tail: the
    K-1 samples before x ([B, K-1, C]) or None for zeros."""
    B, L, C = x.shape
    K = h.shape[1]
    pad = x.new_zeros((B, K - 1, C)) if tail is None else tail.to(x.dtype)
    xp = torch.cat([pad, x], dim=1).transpose(1, 2)                      # [B, C, L+K-1]
    w = h.flip(1).unsqueeze(1).to(x.dtype)                                # conv1d correlates: flip for convolution
    return F.conv1d(xp, w, groups=C).transpose(1, 2)


SPECTRUM_CACHE_MAX_BYTES = 2 << 30


def fft_size(L: int, Lh: int) -> int:
    return 1 << (L + Lh - 1).bit_length()


def fft_causal_conv(x: torch.Tensor, h: Optional[torch.Tensor], spectrum: Optional[torch.Tensor] = None,
                    n: Optional[int] = None) -> torch.Tensor:
    """Depthwise causal convolution with a filter as long as the sequence.  x: [B, L, C]; h: [C, Lh], or its
    spectrum ``rfft(h, n)`` ([C, n/2 + 1]) with the transform size ``n``."""
    B, L, C = x.shape
    if spectrum is None:
        n = fft_size(L, h.shape[1])
        spectrum = torch.fft.rfft(h.float(), n=n)
    X = torch.fft.rfft(x.float().transpose(1, 2), n=n)
    y = torch.fft.irfft(X * spectrum.unsqueeze(0), n=n)[..., :L]
    return y.transpose(1, 2).to(x.dtype)


class HyenaOperator(nn.Module):
    """Gated convolution operator; ``kind`` in {hcs, hcm, hcl}."""

    def __init__(self, cfg: Evo2Config, kind: str):
        super().__init__()
        d = cfg.d_model
        self.kind, self.d, self.cfg = kind, d, cfg
        self.in_proj = nn.Linear(d, 3 * d, bias=False)
        self.fir = nn.Parameter(torch.randn(3 * d, cfg.fir_len) * 0.3)
        if kind == "hcs":
            self.h = nn.Parameter(torch.randn(d, cfg.short_len) * 0.2)
        elif kind == "hcm":
            self.h = nn.Parameter(torch.randn(d, cfg.medium_len) * (1.0 / math.sqrt(cfg.medium_len)))
        else:
            self.log_poles = nn.Parameter(torch.log(torch.rand(d, cfg.state_dim) * 0.5 + 0.45))
            self.residues = nn.Parameter(torch.randn(d, cfg.state_dim) * (1.0 / cfg.state_dim))
        self.D = nn.Parameter(torch.ones(d))
        self.out_proj = nn.Linear(d, d, bias=True)
        self.impl = "torch"
        self._taps = None           # tap-major fp32 copies of the filters for the kernels
        self._lam_cache = None
        self.fp8 = False            # prefill: the input projection in e4m3 (see forward)

    # ---- filters
    def filter_spectrum(self, L: int):
        """(rfft of this operator's long / medium filter at the transform size for length L, that size).  The
        weights are constants at inference, so the spectrum is computed once per sequence length and kept (two
        lengths per operator; each entry is d x (n/2 + 1) complex64); a changed parameter version drops it."""
        h_len = L if self.kind == "hcl" else self.h.shape[1]
        n = fft_size(L, h_len)
        # version counter, shape and storage address: a sharded copy (tensor parallelism swaps ``.data``) or an
        # in-place update both drop the entry
        ver = tuple((p._version, tuple(p.shape), p.data_ptr())
                    for p in ((self.log_poles, self.residues) if self.kind == "hcl" else (self.h,)))
        cache = self.__dict__.setdefault("_spectra", {})
        ent = cache.get((L, n))
        dev = self.D.device
        if ent is None or ent[0] != ver or ent[1].device != dev:
            h = self.long_filter(L) if self.kind == "hcl" else self.h
            spec = torch.fft.rfft(h.float(), n=n)
            # an entry is d x (n/2 + 1) complex64: kept only below a size limit (million-token contexts would pin tens
            # of GB per operator); above it the spectrum is rebuilt per call as before
            if spec.numel() * 8 > SPECTRUM_CACHE_MAX_BYTES:
                return spec, n
            if len(cache) >= 2:
                cache.pop(next(iter(cache)))
            ent = (ver, spec)
            cache[(L, n)] = ent
        return ent[1], n

    def long_filter(self, L: int) -> torch.Tensor:
        t = torch.arange(L, device=self.residues.device, dtype=torch.float32)
        lam = torch.exp(self.log_poles.float())                                   # in (0, 1)
        return torch.einsum("cs,cst->ct", self.residues.float(), lam.unsqueeze(-1) ** t)

    def inner(self, u: torch.Tensor, state: Optional[dict]) -> torch.Tensor:
        """conv(u) + D*u for the operator's filter.  u: [B, L, d]."""
        if self.kind in ("hcs", "hcm"):
            tail = None if state is None else state.get("inner_tail")
            if self.kind == "hcm" and u.shape[1] > 4 * self.h.shape[1] and tail is None:
                y = fft_causal_conv(u, None, *self.filter_spectrum(u.shape[1]))
            else:
                y = causal_fir(u, self.h, tail)
        else:
            y = fft_causal_conv(u, None, *self.filter_spectrum(u.shape[1]))
        return y + u * self.D.to(u.dtype)

    def _lam(self) -> torch.Tensor:
        """exp(log_poles) in fp32, kept until the parameter is written again (three launches per decode step)."""
        ent = self._lam_cache
        if ent is None or ent[0] != self.log_poles._version or ent[1].device != self.log_poles.device:
            ent = (self.log_poles._version, torch.exp(self.log_poles.detach().float()).contiguous())
            self._lam_cache = ent
        return ent[1]

    def _kernel_taps(self):
        if self._taps is None:
            from ..ops import seq
            self._taps = (seq.taps_major(self.fir), None if self.kind == "hcl" else seq.taps_major(self.h))
        return self._taps

    def _fused_inner(self, u, x2, tail):
        """x2 * (conv(u) + D u) with the gate folded into the convolution's epilogue."""
        from ..ops import seq
        if self.kind in ("hcs", "hcm") and self.h.shape[1] <= 512:
            # short filters from a register window, the medium filter (128 taps) as a tiled direct convolution:
            # 17 G multiply-adds per operator at the 7B shape against three FFT-sized fp32 passes
            return seq.fir_inner_gate(u, self._kernel_taps()[1], self.D, x2, tail)
        Hf, n = self.filter_spectrum(u.shape[1])
        X = torch.fft.rfft(seq.fft_pad_transpose(u, n))          # channel-major fp32, zero-padded to the transform size
        y = torch.fft.irfft(seq.spectrum_mul_(X, Hf.contiguous()), n=n)                   # [B, d, n] fp32
        return seq.fftconv_epilogue(y, u, self.D, x2)

    def forward(self, x: torch.Tensor, state: Optional[dict] = None, linear=None,
                residual: Optional[torch.Tensor] = None, pre_norm: Optional["RMSNorm"] = None) -> torch.Tensor:
        """Prefill form.  When ``state`` is a dict it is filled with what decoding needs.  ``residual`` (only with a
        ``linear`` hook that takes one) is added behind the output projection, in its epilogue.  ``pre_norm``: x is
        the block's input before its RMSNorm and the input projection runs in fp8 (the norm emits e4m3 rows, the
        weights are held in e4m3: upstream's fp8 input projections)."""
        lin = linear or (lambda m, t: m(t))
        z = fp8_projection(self.in_proj, x, pre_norm) if pre_norm is not None else lin(self.in_proj, x)
        fused = _fusable(self, z) and self.cfg.fir_len <= 4
        if fused:
            from ..ops import seq
            u, x2 = seq.fir_gate3(z, self._kernel_taps()[0])
            gated = self._fused_inner(u, x2, None)
        else:
            zf = causal_fir(z, self.fir)
            x1, x2, v = zf.chunk(3, dim=-1)
            u = x1 * v
            gated = x2 * self.inner(u, None)
        if state is not None:
            K = self.cfg.fir_len
            state["fir_tail"] = _last(z, K - 1)
            if self.kind in ("hcs", "hcm"):
                state["inner_tail"] = _last(u, self.h.shape[1] - 1)
            elif fused and self.log_poles.shape[1] <= 16:
                from ..ops import seq
                state["poles"] = seq.pole_prefill_state(u, self._lam())           # sum_t lam^(L-1-t) u_t
            else:
                lam = torch.exp(self.log_poles.float())                           # [d, S]
                L = u.shape[1]
                w = lam.unsqueeze(0) ** torch.arange(L - 1, -1, -1, device=u.device, dtype=torch.float32).view(L, 1, 1)
                state["poles"] = torch.einsum("bld,lds->bds", u.float(), w)       # sum_t lam^(L-1-t) u_t
        return lin(self.out_proj, gated) if residual is None else lin(self.out_proj, gated, residual)

    def step(self, x: torch.Tensor, state: dict, linear=None) -> torch.Tensor:
        """One token.  x: [B, 1, d]."""
        lin = linear or (lambda m, t: m(t))
        z = lin(self.in_proj, x)
        if _fusable(self, z) and self.cfg.fir_len <= 4:
            from ..ops import seq
            # a static state (fixed-address buffers that only this decode loop holds) is moved on inside the
            # kernels; any other state may be shared with a snapshot and is replaced, not written
            inplace = bool(state.get("static")) and z.shape[1] == 1 and _kernel_tail(state["fir_tail"])
            u, x2 = seq.fir_gate3(z, self._kernel_taps()[0], state["fir_tail"], push=inplace)
            if not inplace:
                _push(state, "fir_tail", z)
            if self.kind in ("hcs", "hcm"):
                taps = self._kernel_taps()[1]
                if inplace and 2 <= taps.shape[0] <= 256 and _kernel_tail(state["inner_tail"]):
                    gated = seq.fir_step(u, taps, self.D, x2, state["inner_tail"])
                else:
                    gated = seq.fir_inner_gate(u, taps, self.D, x2, state["inner_tail"])
                    _push(state, "inner_tail", u)
            else:
                st = state["poles"]
                if st.dtype != torch.float32 or not st.is_contiguous():
                    st = st.float().contiguous()
                    state["poles"] = st
                gated = seq.pole_step(st, self._lam(), self.residues, u[:, 0], self.D,
                                      x2[:, 0]).unsqueeze(1)          # updates st in place
            return lin(self.out_proj, gated)
        zf = causal_fir(z, self.fir, state["fir_tail"])
        _push(state, "fir_tail", z)
        x1, x2, v = zf.chunk(3, dim=-1)
        u = x1 * v
        if self.kind in ("hcs", "hcm"):
            y = causal_fir(u, self.h, state["inner_tail"]) + u * self.D.to(u.dtype)
            _push(state, "inner_tail", u)
        else:
            lam = torch.exp(self.log_poles.float())
            s = state["poles"] * lam.unsqueeze(0) + u[:, 0].float().unsqueeze(-1)     # [B, d, S]
            if state.get("static"):
                state["poles"].copy_(s)
                s = state["poles"]
            else:
                state["poles"] = s
            y = (s * self.residues.float().unsqueeze(0)).sum(-1).unsqueeze(1).to(u.dtype) + u * self.D.to(u.dtype)
        return lin(self.out_proj, x2 * y)

    # ---- multi-token continuation (speculative decoding): k tokens after an existing state, then keep j of them
    def extend(self, x: torch.Tensor, state: dict, linear=None) -> torch.Tensor:
        """x: [B, k, d] continuing ``state`` (not a static one).  The state itself is left as it was; what a later
        :meth:`commit` needs (projected inputs, gated inputs, the pole state after every token) is parked under
        ``state["pending"]``."""
        lin = linear or (lambda m, t: m(t))
        z = lin(self.in_proj, x)
        zf = causal_fir(z, self.fir, state["fir_tail"])
        x1, x2, v = zf.chunk(3, dim=-1)
        u = x1 * v
        pend = {"z": z, "u": u}
        if self.kind in ("hcs", "hcm"):
            y = causal_fir(u, self.h, state["inner_tail"]) + u * self.D.to(u.dtype)
        else:
            lam = torch.exp(self.log_poles.float()).unsqueeze(0)
            res = self.residues.float().unsqueeze(0)
            s = state["poles"].float()
            ys, ss = [], []
            for t in range(u.shape[1]):
                s = s * lam + u[:, t].float().unsqueeze(-1)
                ss.append(s)
                ys.append((s * res).sum(-1))
            pend["poles"] = ss
            y = torch.stack(ys, 1).to(u.dtype) + u * self.D.to(u.dtype)
        state["pending"] = pend
        return lin(self.out_proj, x2 * y)

    def commit(self, state: dict, j: int) -> None:
        """Make the first ``j`` tokens of the last :meth:`extend` part of the state; drop the rest."""
        pend = state.pop("pending")
        if j <= 0:
            return
        K = self.cfg.fir_len
        state["fir_tail"] = _last(torch.cat([state["fir_tail"], pend["z"][:, :j].to(state["fir_tail"].dtype)], 1), K - 1)
        if self.kind in ("hcs", "hcm"):
            state["inner_tail"] = _last(torch.cat([state["inner_tail"], pend["u"][:, :j].to(state["inner_tail"].dtype)], 1),
                                        self.h.shape[1] - 1)
        else:
            state["poles"] = pend["poles"][j - 1]


def _kernel_tail(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous() and t.shape[1] >= 1


def _push(state: dict, key: str, new: torch.Tensor) -> None:
    """Shift a [B, K-1, C] tail by one position and append ``new`` ([B, 1, C]).  A static state (one that a
    captured decode graph reads and writes at fixed addresses) is rewritten in place."""
    nxt = torch.cat([state[key], new.to(state[key].dtype)], 1)[:, 1:]
    if state.get("static"):
        state[key].copy_(nxt)
    else:
        state[key] = nxt


def _last(t: torch.Tensor, n: int) -> torch.Tensor:
    B, L, C = t.shape
    if n <= 0:
        return t.new_zeros((B, 0, C))
    if L >= n:
        return t[:, L - n:].clone()
    return torch.cat([t.new_zeros((B, n - L, C)), t], 1)


def rope(x: torch.Tensor, pos: torch.Tensor, base: float) -> torch.Tensor:
    """x: [B, L, H, D]; pos: [L]."""
    D = x.shape[-1]
    inv = 1.0 / (base ** (torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D))
    ang = pos.float().unsqueeze(-1) * inv                                  # [L, D/2]
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    x1, x2 = x.float()[..., 0::2], x.float()[..., 1::2]
    out = torch.stack([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1).flatten(-2)
    return out.to(x.dtype)


def _few_query_attention(q, kc, vc, mask=None):
    """q: [B, k, H, D] (a handful of decode queries), kc / vc: [B, L, H, D], mask: bool [k, L] (True = visible) or
    None.  Written out instead of calling the library's fused attention: with a cache that grows every step the
    library re-plans its kernel per call (about 7 ms of host time per call on a B200 box), which made an eager decode
    step 8 times slower than its kernels."""
    sc = torch.einsum("bqhd,bkhd->bhqk", q, kc).float() * (q.shape[-1] ** -0.5)
    if mask is not None:
        sc = sc.masked_fill(~mask[None, None], float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc, -1).to(vc.dtype), vc)


class AttentionOperator(nn.Module):
    def __init__(self, cfg: Evo2Config):
        super().__init__()
        self.cfg = cfg
        d = cfg.d_model
        self.qkv = nn.Linear(d, 3 * d, bias=False)
        self.out_proj = nn.Linear(d, d, bias=True)
        self.impl = "torch"

    def _causal(self, q, k, v):
        """q, k, v: [B, L, H, hd] -> [B, L, H, hd].  The library's fused attention by default (it is the faster of
        the two on B200: 1.51 against 1.05 PFLOP/s at 32768 tokens); with ``ops.causal.ENABLED`` the kernel path
        takes the package's tcgen05 causal kernel at head dimension 128."""
        if self.impl == "fused":
            from ..ops import causal
            if causal.ENABLED and causal.supported(q, k, v) is None:
                return causal.causal_attention(q, k, v)
        return F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                              is_causal=True).transpose(1, 2)

    def _qkv(self, x, pos, lin):
        """q, k, v as [B, L, heads held here, head_dim]; under tensor parallelism the projection returns only
        this rank's heads."""
        B, L, d = x.shape
        hd = self.cfg.d_model // self.cfg.n_heads
        qkv = lin(self.qkv, x)
        H = qkv.shape[-1] // (3 * hd)
        if _fusable(self, qkv) and L > 8 and hd % 2 == 0:
            # one pass over the projection: rotary embedding of q and k, the three tensors written apart
            from ..ops import seq
            q, k, v = seq.rotary_split_qkv(qkv.view(B * L, -1), pos.to(torch.int32).repeat(B), H, hd,
                                           self.cfg.rope_base)
            return q.view(B, L, H, hd), k.view(B, L, H, hd), v.view(B, L, H, hd)
        q, k, v = qkv.view(B, L, 3, H, hd).unbind(2)
        return rope(q, pos, self.cfg.rope_base), rope(k, pos, self.cfg.rope_base), v

    def forward(self, x, state: Optional[dict] = None, linear=None, residual=None):
        lin = linear or (lambda m, t: m(t))
        B, L, d = x.shape
        pos = torch.arange(L, device=x.device)
        q, k, v = self._qkv(x, pos, lin)
        o = self._causal(q, k, v)
        if state is not None:
            state["k"], state["v"] = k, v
        o = o.reshape(B, L, -1)
        return lin(self.out_proj, o) if residual is None else lin(self.out_proj, o, residual)

    def step(self, x, state: dict, linear=None):
        lin = linear or (lambda m, t: m(t))
        B, _, d = x.shape
        if state.get("static"):
            # fixed-size cache, the position is a device tensor: no host value enters the step, so it can be
            # captured in a CUDA graph.  Keys past the position are masked.
            pos = state["pos"]                                              # int64 [1]
            hd = self.cfg.d_model // self.cfg.n_heads
            if _fusable(self, x) and x.shape[1] == 1 and hd == 128 and state["k"].dtype == torch.bfloat16 and \
                    state["k"].is_contiguous() and state["v"].is_contiguous():
                # rotary embedding, cache write and the masked attention as three launches of the kernel path
                from ..ops import seq
                o = seq.decode_attention(lin(self.qkv, x).view(B, -1), pos, state["k"], state["v"],
                                         self.cfg.rope_base)
                return lin(self.out_proj, o.view(B, 1, -1))
            q, k, v = self._qkv(x, pos, lin)
            state["k"].index_copy_(1, pos, k.to(state["k"].dtype))
            state["v"].index_copy_(1, pos, v.to(state["v"].dtype))
            kc, vc = state["k"], state["v"]                                 # [B, Lmax, H, hd]
            sc = torch.einsum("bqhd,bkhd->bhqk", q, kc).float() * (q.shape[-1] ** -0.5)
            dead = torch.arange(kc.shape[1], device=x.device) > pos
            sc = sc.masked_fill(dead[None, None, None, :], float("-inf"))
            o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc, -1).to(vc.dtype), vc)
            return lin(self.out_proj, o.reshape(B, 1, -1))
        pos = torch.full((1,), state["k"].shape[1], dtype=torch.long, device=x.device)      # no host-to-device copy
        q, k, v = self._qkv(x, pos, lin)
        state["k"] = torch.cat([state["k"], k], 1)
        state["v"] = torch.cat([state["v"], v], 1)
        o = _few_query_attention(q, state["k"], state["v"])
        return lin(self.out_proj, o.reshape(B, 1, -1))

    def extend(self, x, state: dict, linear=None):
        """k tokens after the cached ones (dynamic cache): the new keys are appended, each new query sees the cache
        and the new keys up to itself.  :meth:`commit` keeps the first j of them."""
        lin = linear or (lambda m, t: m(t))
        B, k, d = x.shape
        L0 = state["k"].shape[1]
        pos = torch.arange(L0, L0 + k, device=x.device)
        q, kk, vv = self._qkv(x, pos, lin)
        state["pending"] = {"len0": L0}
        state["k"] = torch.cat([state["k"], kk], 1)
        state["v"] = torch.cat([state["v"], vv], 1)
        mask = torch.arange(L0 + k, device=x.device)[None, :] <= pos[:, None]
        o = _few_query_attention(q, state["k"], state["v"], mask)
        return lin(self.out_proj, o.reshape(B, k, -1))

    def commit(self, state: dict, j: int) -> None:
        keep = state.pop("pending")["len0"] + max(j, 0)
        state["k"], state["v"] = state["k"][:, :keep], state["v"][:, :keep]


class SwiGLU(nn.Module):
    def __init__(self, d: int, ffn: int):
        super().__init__()
        self.l1 = nn.Linear(d, ffn, bias=False)     # gate
        self.l2 = nn.Linear(d, ffn, bias=False)     # up
        self.l3 = nn.Linear(ffn, d, bias=False)     # down
        self.impl = "torch"

    def forward(self, x, linear=None, residual=None):
        lin = linear or (lambda m, t: m(t))
        if residual is not None:
            inner = lin
            lin = lambda m, t: inner(m, t, residual) if m is self.l3 else inner(m, t)   # noqa: E731
        if _fusable(self, x) and linear is not None and x.numel() // x.shape[-1] > 8 and \
                self.l1.out_features % 32 == 0 and self.l1.bias is None and self.l2.bias is None:
            # both projections as one product whose epilogue forms silu(gate) * value on the accumulator (the
            # interleaved weight is a second copy of the two matrices, kept until either is written again)
            from ..ops import gemm
            x2 = x.reshape(-1, x.shape[-1])
            h = gemm.gemm(x2 if x2.is_contiguous() else x2.contiguous(), self._swiglu_weight(), act="swiglu")
            return lin(self.l3, h.view(*x.shape[:-1], h.shape[-1]))
        g, up = lin(self.l1, x), lin(self.l2, x)
        if _fusable(self, g):
            from ..ops import seq
            return lin(self.l3, seq.silu_mul(g, up))
        return lin(self.l3, F.silu(g) * up)

    def _swiglu_weight(self) -> torch.Tensor:
        ver = tuple((p._version, p.data_ptr(), tuple(p.shape)) for p in (self.l1.weight, self.l2.weight))
        ent = self.__dict__.get("_packed_w")
        if ent is None or ent[0] != ver:
            from ..ops import gemm
            ent = (ver, gemm.pack_swiglu(self.l1.weight.detach(), self.l2.weight.detach()))
            self.__dict__["_packed_w"] = ent
        return ent[1]


class Block(nn.Module):
    def __init__(self, cfg: Evo2Config, kind: str):
        super().__init__()
        self.kind = kind
        self.pre_norm = RMSNorm(cfg.d_model, cfg.eps)
        self.mixer = AttentionOperator(cfg) if kind == "attn" else HyenaOperator(cfg, kind)
        self.post_norm = RMSNorm(cfg.d_model, cfg.eps)
        self.mlp = SwiGLU(cfg.d_model, cfg.ffn)

    def forward(self, x, state=None, linear=None):
        if linear is not None and getattr(linear, "takes_residual", False) and _fusable(self.pre_norm, x):
            # the residual stream is added in the epilogue of the projection that closes each half of the block
            if getattr(self.mixer, "fp8", False) and x.shape[-1] <= 4096 and x.shape[0] * x.shape[1] > 8:
                x = self.mixer(x, state, linear, x, self.pre_norm)
            else:
                x = self.mixer(self.pre_norm(x), state, linear, x)
            return self.mlp(self.post_norm(x), linear, x)
        x = x + self.mixer(self.pre_norm(x), state, linear)
        return x + self.mlp(self.post_norm(x), linear)

    def step(self, x, state, linear=None, folded=None):
        if folded is not None and _decode_rows(self, x):
            return self._folded(x, state, self.mixer.step, folded)
        x = x + self.mixer.step(self.pre_norm(x), state, linear)
        return x + self.mlp(self.post_norm(x), linear)

    def extend(self, x, state, linear=None, folded=None):
        if folded is not None and _decode_rows(self, x):
            return self._folded(x, state, self.mixer.extend, folded)
        x = x + self.mixer.extend(self.pre_norm(x), state, linear)
        return x + self.mlp(self.post_norm(x), linear)

    def _folded(self, x, state, mixer_fn, folded):
        """The block on at most 8 rows with four weight-streaming launches instead of eleven: both RMSNorms run in
        front of the projection that reads them, both residual additions behind the projection that feeds them and
        the two halves of SwiGLU in one pass over their weights.  ``folded(module, rows, gamma=, eps=, res=,
        second=)`` is the model's hook for such a projection (:func:`folded_linear`, or the tensor-parallel form);
        on one GPU every intermediate is rounded where the separate kernels round it, so the tokens are the same."""
        B, L, d = x.shape
        rows = x.reshape(B * L, d)
        first = self.mixer.qkv if self.kind == "attn" else self.mixer.in_proj
        last = self.mixer.out_proj

        def lin(mod, t):
            t2 = t.reshape(-1, t.shape[-1])
            if mod is first:
                y = folded(mod, t2, gamma=self.pre_norm.scale, eps=self.pre_norm.eps)
            elif mod is last:
                y = folded(mod, t2, res=rows)
            else:
                y = folded(mod, t2)
            return y.view(*t.shape[:-1], y.shape[-1])

        x1 = mixer_fn(x, state, lin)                                     # x + mixer(norm(x))
        r1 = x1.reshape(B * L, d)
        h = folded(self.mlp.l1, r1, gamma=self.post_norm.scale, eps=self.post_norm.eps, second=self.mlp.l2)
        return folded(self.mlp.l3, h, res=r1).view(B, L, d)


class StripedHyena2(nn.Module):
    def __init__(self, cfg: Evo2Config):
        super().__init__()
        self.cfg = cfg
        self.embedding = nn.Embedding(cfg.vocab, cfg.d_model)
        self.blocks = nn.ModuleList([Block(cfg, cfg.layer_kind(i)) for i in range(cfg.n_layers)])
        self.norm = RMSNorm(cfg.d_model, cfg.eps)
        self.linear = None          # optional callable (module, x) -> y replacing nn.Linear calls (fused / TP GEMMs)
        self.folded = None          # optional hook of the folded decode block (see Block._folded)

    def set_impl(self, impl: str) -> int:
        """``fused``: RMSNorm, the FIR / gate stages, the convolution epilogues, the decode state step and SwiGLU
        run as kernels and every nn.Linear goes through the tcgen05 GEMM; ``torch``: the plain statements.
        Returns the number of modules switched."""
        n = 0
        for m in self.modules():
            if hasattr(m, "impl"):
                m.impl = impl
                n += 1
        self.linear = fused_linear if impl == "fused" else None
        self.folded = folded_linear if impl == "fused" else None
        return n

    def set_fp8_input_projections(self, on: bool = True) -> int:
        """The input projections of the Hyena operators in e4m3 (kernel path, d_model <= 4096): both operands in
        the prefill, the weights in the folded decode block.  Returns the number of operators switched."""
        n = 0
        for blk in self.blocks:
            if isinstance(blk.mixer, HyenaOperator):
                blk.mixer.fp8 = bool(on)
                blk.mixer.in_proj.fp8_weights = bool(on)     # read by the folded decode block
                n += 1
        return n

    def logits(self, x):
        return F.linear(self.norm(x), self.embedding.weight)

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, states: Optional[List[dict]] = None) -> torch.Tensor:
        """tokens: [B, L] -> logits [B, L, vocab].  ``states`` (a list of dicts, one per block) is filled for decoding."""
        x = self.embedding(tokens)
        for i, blk in enumerate(self.blocks):
            x = blk(x, None if states is None else states[i], self.linear)
        return self.logits(x)

    @torch.no_grad()
    def step(self, token: torch.Tensor, states: List[dict]) -> torch.Tensor:
        x = self.embedding(token)
        for i, blk in enumerate(self.blocks):
            x = blk.step(x, states[i], self.linear, self.folded)
        return self.logits(x)

    @torch.no_grad()
    def extend(self, tokens: torch.Tensor, states: List[dict]) -> torch.Tensor:
        """tokens: [B, k] continuing ``states`` -> logits [B, k, vocab]; one pass over the weights for k tokens.
        The states change only at :meth:`commit`."""
        x = self.embedding(tokens)
        for i, blk in enumerate(self.blocks):
            x = blk.extend(x, states[i], self.linear, self.folded)
        return self.logits(x)

    def commit(self, states: List[dict], j: int) -> None:
        for blk, st in zip(self.blocks, states):
            blk.mixer.commit(st, j)

    def make_static_states(self, states: List[dict], max_len: int) -> torch.Tensor:
        """Turn the states a prefill produced into fixed-address buffers (attention caches of ``max_len``
        positions, tails and pole states updated in place) and return the shared position tensor."""
        dev = self.embedding.weight.device
        pos = None
        for blk, st in zip(self.blocks, states):
            st["static"] = True
            if blk.kind == "attn":
                k, v = st["k"], st["v"]
                B, L = k.shape[:2]
                if pos is None:
                    pos = torch.full((1,), L, dtype=torch.long, device=dev)
                for name, t in (("k", k), ("v", v)):
                    buf = t.new_zeros((B, max_len) + tuple(t.shape[2:]))
                    buf[:, :L] = t
                    st[name] = buf
                st["pos"] = pos
            else:
                for name in ("fir_tail", "inner_tail"):
                    if name in st:
                        st[name] = st[name].contiguous().clone()
                if "poles" in st:
                    st["poles"] = st["poles"].float().contiguous().clone()
        if pos is None:
            pos = torch.zeros((1,), dtype=torch.long, device=dev)
        return pos

    @torch.no_grad()
    def generate(self, tokens: torch.Tensor, max_new_tokens: int, graph: bool = False) -> torch.Tensor:
        """Greedy decoding: prefill, then ``max_new_tokens`` single-token steps.  ``graph=True`` (GPU): the decode
        step is captured once in a CUDA graph over fixed-address states and replayed per token."""
        states = [dict() for _ in self.blocks]
        logits = self.forward(tokens, states)
        nxt = logits[:, -1:].argmax(-1)
        if graph and tokens.is_cuda and max_new_tokens > 2:
            return self._generate_graph(tokens, states, nxt, max_new_tokens)
        out = [nxt]
        for _ in range(max_new_tokens - 1):
            logits = self.step(nxt, states)
            nxt = logits[:, -1:].argmax(-1)
            out.append(nxt)
        return torch.cat(out, 1)

    @torch.no_grad()
    def generate_speculative(self, draft: "StripedHyena2", tokens: torch.Tensor, max_new_tokens: int, k: int = 6):
        """Greedy decoding of this model with ``draft`` proposing ``k`` tokens per round (batch 1).  Each round
        costs k single-token passes of the draft and ONE pass of this model over k + 1 tokens; the proposals are
        kept up to the first one this model would not have chosen, and this model's own choice follows them, so
        the output is the plain greedy sequence.  Returns (new tokens [1, max_new_tokens], statistics)."""
        if tokens.shape[0] != 1:
            raise ValueError("speculative decoding runs one sequence at a time")
        t_states = [dict() for _ in self.blocks]
        d_states = [dict() for _ in draft.blocks]
        cur = self.forward(tokens, t_states)[:, -1:].argmax(-1)
        draft.forward(tokens, d_states)
        out = [cur]
        n_out = 1
        stats = {"rounds": 0, "proposed": 0, "accepted": 0}
        while n_out < max_new_tokens:
            # the draft consumes cur, p1 .. p(k-1) and proposes p1 .. pk.  Continuation never writes a state tensor
            # in place (tails, pole states and caches are replaced by new tensors), so a shallow copy of the
            # dicts is a snapshot.
            snap = [dict(st) for st in d_states]
            consumed, props, tok = [], [], cur
            for _ in range(k):
                lg = draft.extend(tok, d_states)
                draft.commit(d_states, 1)
                consumed.append(tok)
                tok = lg[:, -1:].argmax(-1)
                props.append(tok)
            seq = torch.cat([cur] + props, 1)                               # [1, k + 1]
            choice = self.extend(seq, t_states).argmax(-1)                  # this model's token after each prefix
            agree = (choice[:, :k] == seq[:, 1:]).long()[0]
            j = int(agree.cumprod(0).sum())                                 # accepted proposals
            self.commit(t_states, j + 1)                                    # cur, p1 .. pj are now consumed
            new = [seq[:, i:i + 1] for i in range(1, j + 1)] + [choice[:, j:j + 1]]
            out.extend(new)
            n_out += len(new)
            stats["rounds"] += 1
            stats["proposed"] += k
            stats["accepted"] += j
            cur = new[-1]
            # the draft must have consumed exactly cur_old, p1 .. pj: it has consumed k tokens
            if j == k:
                draft.extend(props[-1], d_states)
                draft.commit(d_states, 1)
            elif j < k - 1:
                for st, old in zip(d_states, snap):
                    st.clear()
                    st.update(old)
                draft.extend(torch.cat(consumed[:j + 1], 1), d_states)
                draft.commit(d_states, j + 1)
        return torch.cat(out, 1)[:, :max_new_tokens], stats

    def _generate_graph(self, tokens, states, first, max_new_tokens):
        dev = tokens.device
        B, L = tokens.shape
        pos = self.make_static_states(states, L + max_new_tokens)
        tok = first.clone()                                               # static input / feedback buffer
        out = torch.zeros((B, max_new_tokens), dtype=first.dtype, device=dev)
        out[:, 0:1] = first
        cnt = torch.ones((1,), dtype=torch.long, device=dev)

        def one_step():
            nxt = self.step(tok, states)[:, -1:].argmax(-1)
            out.index_copy_(1, cnt, nxt)
            tok.copy_(nxt)
            pos.add_(1)
            cnt.add_(1)

        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            one_step()                                                    # eager step: warms every kernel up
        torch.cuda.current_stream(dev).wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            one_step()
        for _ in range(max_new_tokens - 2):
            g.replay()
        return out

    @torch.no_grad()
    def score(self, tokens: torch.Tensor) -> torch.Tensor:
        """Mean log-likelihood per sequence (the kit's ``score`` verb)."""
        lp = torch.log_softmax(self.forward(tokens).float(), -1)
        tgt = tokens[:, 1:]
        return lp[:, :-1].gather(-1, tgt.unsqueeze(-1)).squeeze(-1).mean(-1)


BYTE_LUT = {c: i for i, c in enumerate("ACGTN")}


_W_CACHE: dict = {}


def _bf16_weight(module: nn.Linear):
    """(contiguous bf16 weight, fp32 bias or None) of a linear layer, kept until the weight is written again."""
    key = id(module)
    ent = _W_CACHE.get(key)
    if ent is None or ent[0] is not module.weight or ent[1] != module.weight._version:
        ent = (module.weight, module.weight._version, module.weight.detach().to(torch.bfloat16).contiguous(),
               None if module.bias is None else module.bias.detach().float().contiguous())
        _W_CACHE[key] = ent
    return ent[2], ent[3]


def _decode_rows(block: "Block", x: torch.Tensor) -> bool:
    """At most 8 bf16 rows on the GPU with the kernel path on, and the widest projection input of the block
    staged in one CTA's shared memory: the folded decode block serves them."""
    if not (_fusable(block.pre_norm, x) and x.dim() == 3 and x.shape[0] * x.shape[1] <= 8):
        return False
    rows = x.shape[0] * x.shape[1]
    mb = 1 if rows == 1 else 2 if rows <= 2 else 4 if rows <= 4 else 8
    widest = max(x.shape[-1], block.mlp.l3.in_features)
    return widest % 8 == 0 and mb * widest * 2 <= 200 * 1024 and os.environ.get("UBM_EVO2_FOLDED_DECODE", "1") != "0"


_W8_CACHE: dict = {}


def fp8_projection(module: nn.Linear, x: torch.Tensor, norm: "RMSNorm") -> torch.Tensor:
    """module(norm(x)) with both operands in e4m3: the normalised rows are written as 8-bit floats scaled by their
    own maximum (``ops.seq.rmsnorm_fp8``), the weight is quantised once per version with its maximum, the product
    accumulates in fp32 and is scaled back in the epilogue.  x: bf16 [B, L, d] on the GPU."""
    from ..ops import gemm, seq
    q, dq, bias = _e4m3_weight(module)
    x8, dq_x = seq.rmsnorm_fp8(x, norm.scale, norm.eps)
    y = gemm.gemm_fp8(x8, q, alpha=dq, alpha_dev=dq_x, bias=bias)
    return y.view(*x.shape[:-1], y.shape[-1])


def _e4m3_weight(module: nn.Linear):
    """(e4m3 weight, its dequantisation factor, fp32 bias or None), quantised once per weight version."""
    from ..ops import gemm
    w = module.weight
    ent = _W8_CACHE.get(id(module))
    ver = (w._version, w.data_ptr(), tuple(w.shape))
    if ent is None or ent[0] is not w or ent[1] != ver:
        q, dq = gemm.quantize_e4m3(w)
        ent = (w, ver, q, dq, None if module.bias is None else module.bias.detach().float().contiguous())
        _W8_CACHE[id(module)] = ent
    return ent[2], ent[3], ent[4]


def folded_linear(module: nn.Linear, rows: torch.Tensor, gamma=None, eps: float = 1e-6, res=None,
                  second: Optional[nn.Linear] = None) -> torch.Tensor:
    """A projection of the folded decode block on one GPU: rows [M <= 8, K] -> [M, N] on the weight-streaming
    kernel with RMSNorm (``gamma``) in front, the residual (``res``) behind and, with ``second``, the SwiGLU of
    two projections."""
    from ..ops import seq
    if getattr(module, "fp8_weights", False) and second is None and rows.shape[-1] % 16 == 0:
        q, dq, b8 = _e4m3_weight(module)          # the prefill's e4m3 weights: half the bytes of the step
        return seq.gemv_rows(rows, q, b8, gamma=gamma, eps=eps, res=res, wscale=dq)
    w, b = _bf16_weight(module)
    w2 = None if second is None else _bf16_weight(second)[0]
    return seq.gemv_rows(rows, w, b, gamma=gamma, eps=eps, w2=w2, res=res)


def fused_linear(module: nn.Linear, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """nn.Linear on the tcgen05 GEMM for bf16 GPU activations (weights cached as contiguous bf16); anything
    else takes the module's own forward.  ``residual`` (the shape of the result) is added in the epilogue."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0):
        y = module(x)
        return y if residual is None else y + residual
    from ..ops import gemm
    w, b = _bf16_weight(module)
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    r2 = None
    if residual is not None:
        r2 = residual.reshape(-1, w.shape[0])
        if r2.dtype != torch.bfloat16 or not r2.is_contiguous():
            r2 = r2.to(torch.bfloat16).contiguous()
    if x2.shape[0] <= 8:                      # decode rows: stream the weights once (memory bound)
        from ..ops import seq
        return seq.gemv_rows(x2, w, b, res=r2).view(*x.shape[:-1], w.shape[0])
    return gemm.gemm(x2, w, bias=b, residual=r2).view(*x.shape[:-1], w.shape[0])


fused_linear.takes_residual = True


def tokenize(seq: str, device="cpu") -> torch.Tensor:
    """Byte tokenizer (vocabulary 512; DNA letters map to their byte values)."""
    return torch.tensor([[min(ord(c), 511) for c in seq]], dtype=torch.long, device=device)


def build(config: str = "evo2_7b", device="cpu", dtype=torch.float32, seed: int = 0, **overrides) -> StripedHyena2:
    cfg = CONFIGS[config]
    if overrides:
        cfg = replace(cfg, **overrides)
    torch.manual_seed(seed)
    with torch.device(device):
        m = StripedHyena2(cfg)
    m = m.to(dtype=dtype).eval()
    for p in m.parameters():
        p.requires_grad_(False)
    return m
