"""Kernel self-verification at load: before a mode that uses the kernels serves its first call on a GPU, every
kernel family runs one small fixed case and is held to the fp32 statement of the same op.  A family that misses
its tolerance (or whose launch leaves a non-zero status word) is a *refusal by name*: the activation reports
``KERNELS-REFUSED`` with the family and the process exits 5 instead of producing numbers from a kernel that does
not reproduce its statement on this driver / GPU.

The probes are deterministic (fixed generator seeds), take well under a second together, and need no files: the
reference side is computed on the spot in fp32, so there are no recorded vectors to go stale.  ``run_all`` caches
its verdict per device for the life of the process.  The pair-layer probes seed the global generators
(``torch.manual_seed(3)``) to build their weights: code that depends on the global random state seeds it after
the first kernel-mode ``Predictor`` has been constructed (``Predictor.predict`` seeds every call itself).

Reference: recorded test vectors + byte gates of the native kernels (triattn_native testvectors/cases.py,
apb/fpf_apb/loadcheck.py), warm probes against fp64 (fpf_trimul_v4/DESIGN.md:39-45).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..core import report

_VERDICT: Dict[str, "LoadCheck"] = {}


class KernelsRefused(RuntimeError):
    def __init__(self, failed: List["Probe"]):
        super().__init__("kernel self-verification failed: " + ", ".join(f"{p.family}({p.detail})" for p in failed))
        self.failed = failed


@dataclass
class Probe:
    family: str
    ok: bool
    error: float
    tolerance: float
    detail: str = ""


@dataclass
class LoadCheck:
    device: str
    probes: List[Probe]

    @property
    def ok(self) -> bool:
        return all(p.ok for p in self.probes)

    @property
    def failed(self) -> List[Probe]:
        return [p for p in self.probes if not p.ok]

    def line(self, tag: str = "opt_core") -> str:
        verb = "KERNELS-VERIFIED" if self.ok else "KERNELS-REFUSED"
        worst = max(self.probes, key=lambda p: p.error / max(p.tolerance, 1e-30)) if self.probes else None
        safe = [p.family for p in self.probes if p.ok and p.detail == "safe"]
        return report.line(tag, verb, ("families", len(self.probes)), ("failed", ",".join(p.family for p in self.failed) or "none"),
                           ("worst", f"{worst.family}:{worst.error:.2e}/{worst.tolerance:.0e}" if worst else "none"),
                           ("settings", "tuned" if not safe else "safe:" + ",".join(safe)))


def _rel(out: torch.Tensor, ref: torch.Tensor) -> float:
    scale = max(ref.float().abs().max().item(), 1.0)
    return (out.float() - ref.float()).abs().max().item() / scale


def _gen(dev, seed):
    return torch.Generator(device=dev).manual_seed(seed)


def _probe_gemm(dev) -> Tuple[float, float]:
    from . import gemm
    g = _gen(dev, 1)
    a = torch.randn(300, 192, device=dev, generator=g).bfloat16()
    w = (torch.randn(136, 192, device=dev, generator=g) / 14).bfloat16()
    bias = torch.randn(136, device=dev, generator=g)
    res = torch.randn(300, 136, device=dev, generator=g).bfloat16()
    out = gemm.gemm(a, w, bias=bias, residual=res, act="silu")
    ref = torch.nn.functional.silu(a.float() @ w.float().t() + bias) + res.float()
    return _rel(out, ref), 2e-2


def _probe_layernorm(dev) -> Tuple[float, float]:
    from . import rows
    g = _gen(dev, 2)
    worst = 0.0
    for C in (64, 128, 384, 1536):
        x = (torch.randn(77, C, device=dev, generator=g) * 2 + 0.5).bfloat16()
        w = 1 + 0.1 * torch.randn(C, device=dev, generator=g)
        b = 0.1 * torch.randn(C, device=dev, generator=g)
        worst = max(worst, _rel(rows.layernorm_rows(x, w, b), torch.nn.functional.layer_norm(x.float(), (C,), w, b)))
    return worst, 2e-2


def _pair_layer_probe(dev, pick, call) -> Tuple[float, float]:
    """One sub-module of a Pairformer layer: kernel path in bf16 against the fp32 statements of the same weights."""
    import copy
    from ..models import pairformer
    torch.manual_seed(3)
    layer = pairformer.PairformerLayer().to(dev).eval()
    for p in layer.parameters():
        p.requires_grad_(False)
    mod = pick(layer)
    fused = copy.deepcopy(mod).to(torch.bfloat16)
    pairformer.set_impl(fused, "fused")
    z = torch.randn(1, 72, 72, 128, device=dev, generator=_gen(dev, 4))
    with torch.no_grad():
        ref = call(mod, z)
        out = call(fused, z.bfloat16())
    return _rel(out, ref), 4e-2


def _probe_triattn(dev):
    return _pair_layer_probe(dev, lambda l: l.tri_att_start, lambda m, z: m(z, None))


def _probe_trimul(dev):
    return _pair_layer_probe(dev, lambda l: l.tri_mul_out, lambda m, z: m(z, None))


def _probe_transition(dev):
    return _pair_layer_probe(dev, lambda l: l.transition_z, lambda m, z: m(z))


def _probe_seq(dev) -> Tuple[float, float]:
    from . import reference as R, seq
    g = _gen(dev, 5)
    x = torch.randn(19, 512, device=dev, generator=g).bfloat16()
    sc = 1 + 0.1 * torch.randn(512, device=dev, generator=g)
    e1 = _rel(seq.rmsnorm_rows(x, sc), R.rmsnorm_rows(x, sc))
    z = torch.randn(2, 41, 3 * 64, device=dev, generator=g).bfloat16()
    h = torch.randn(3 * 64, 3, device=dev, generator=g) * 0.4
    u, x2 = seq.fir_gate3(z, seq.taps_major(h))
    ur, x2r = R.fir_gate3(z, h)
    return max(e1, _rel(u, ur), _rel(x2, x2r)), 2e-2


def _probe_column_attention(dev) -> Tuple[float, float]:
    from . import reference as R, seq
    g = _gen(dev, 6)
    q = torch.randn(33, 2, 64, device=dev, generator=g).bfloat16()
    k = torch.randn(9, 33, 2, 64, device=dev, generator=g).bfloat16()
    v = torch.randn(9, 33, 2, 64, device=dev, generator=g).bfloat16()
    idx = torch.randint(0, 9, (6,), device=dev, generator=g)
    return _rel(seq.column_attention(q, k, v, idx), R.column_attention(q, k, v, idx)), 2e-2


def _probe_window(dev) -> Tuple[float, float]:
    """Atom attention in 32 x 128 windows (4 heads of 32) against the windowed fp32 statement."""
    import copy
    from ..models import diffusion, pairformer
    from . import pair
    torch.manual_seed(7)
    B, A, c, H = 2, 160, 128, 4
    attn = pairformer.AttentionPairBias(c, 128, H, compute_pair_bias=False).to(dev).eval()
    x = torch.randn(B, A, c, device=dev, generator=_gen(dev, 8))
    bias = torch.randn(1, H, A // 32, 32, 128, device=dev, generator=_gen(dev, 9))
    with torch.no_grad():
        ref = diffusion._window_attention(attn, x, bias, (32, 128))
        ab = copy.deepcopy(attn).to(torch.bfloat16)
        w = pair.ApbPacked.pack(ab.proj_q.weight, ab.proj_q.bias, ab.proj_k.weight, ab.proj_v.weight,
                                ab.proj_g.weight, ab.proj_o.weight, H)
        out = pair.window_attention_fused(x.bfloat16(), w, diffusion.WindowBias(bias).data)
    return _rel(out, ref), 4e-2


PROBES: Dict[str, Callable] = {
    "gemm": _probe_gemm, "ln": _probe_layernorm, "triattn": _probe_triattn, "trimul": _probe_trimul,
    "transition": _probe_transition, "window": _probe_window, "seq": _probe_seq,
    "column_attention": _probe_column_attention,
}


def _run_probe(family: str, fn: Callable, device) -> Probe:
    from . import native
    try:
        err, tol = fn(device)
        if str(device).startswith("cuda"):
            torch.cuda.synchronize(device)
            native.raise_on_status(device, f"load check {family}")
        ok = err == err and err <= tol            # NaN fails
        return Probe(family, ok, float(err), tol, "" if ok else f"error {err:.3e} > {tol:.0e}")
    except Exception as e:  # noqa: BLE001 - any failure of a probe is a refusal of that family
        return Probe(family, False, float("inf"), 0.0, f"{type(e).__name__}: {str(e)[:80]}")


def run_all(device="cuda:0", probes: Optional[Dict[str, Callable]] = None, use_cache: bool = True,
            safe: Optional[Dict[str, Callable]] = None) -> LoadCheck:
    """Run every probe on ``device``; a probe that raises counts as failed with the exception's name.  A family that
    fails under the tuned settings and has a safe setting (``ops.safe_settings``) is switched to it and probed once
    more; passing then, it serves with the safe setting (``detail == "safe"``)."""
    key = str(device)
    if use_cache and probes is None and key in _VERDICT:
        return _VERDICT[key]
    from . import safe_settings
    results = []
    for family, fn in (probes or PROBES).items():
        pr = _run_probe(family, fn, device)
        if not pr.ok:
            applied = safe[family]() is None if (safe is not None and family in safe) else \
                (safe is None and safe_settings.apply(family))
            if applied:
                again = _run_probe(family, fn, device)
                if again.ok:
                    again.detail = "safe"
                    pr = again
        results.append(pr)
    lc = LoadCheck(key, results)
    if use_cache and probes is None:
        _VERDICT[key] = lc
    return lc


def require(device="cuda:0", tag: str = "opt_core") -> LoadCheck:
    """Run (or recall) the check, print its line, raise :class:`KernelsRefused` when a family failed."""
    lc = run_all(device)
    report.emit(lc.line(tag))
    if not lc.ok:
        raise KernelsRefused(lc.failed)
    return lc
