"""Same-box timings of the reference's own Blackwell rows, next to this library's kernels.

    python benchmarks/reference_kernels.py [--n 1536] [--iters 5] [--warmup 3] [--cases attention,trimul,...]

The reference serves sm_100 parts with Triton kernels that carry cc 10.0 launch cells; they are installed
unmodified under ``baseline/_ref`` (``opt_core``) and are called here through their public entry points:

* triangle attention  ``opt_core.kernels.flash_triattn.flash_triangle_attention`` (grid at flash_triattn.py:852)
  and the base-2 form ``opt_core.kernels.fpf_triatt_k2b.triatt_k2b``;
* triangle multiplication ``opt_core.kernels.fpf_trimul_v4.generic.trimul`` (K1 / cuBLAS bmm / K3);
* pair transition ``opt_core.kernels.fpf_transition_v2.kernel.fused_transition``;
* pair LayerNorm ``opt_core.kernels.ln.fastln.fastln.fast_layer_norm_triton``.

Each case runs the reference row and this library's kernel on the same tensors in one process, in interleaved
rounds (reference, ours, reference, ...), CUDA events around each call, a 160 MB write between calls so that no
call starts with its inputs in L2, median over the rounds.  One line per case:

    REFCASE <case> N=<n> ref_ms=<..> ours_ms=<..> ratio=<ref/ours> ref_impl=<row> max_abs_diff=<..>

A reference row that cannot run on this stack prints ``REFCASE <case> unavailable: <reason>`` (the reason is the
exception the reference raised); nothing is substituted for it.
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
REF = os.path.join(ROOT, "baseline", "_ref")

import torch

from uplifting_biomolecular_modeling_b200.ops import native, pair, rows


def interleaved(fns, iters, warmup):
    """Median ms per function, measured in interleaved rounds with an L2 flush before every call."""
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        for f in fns:
            f()
    torch.cuda.synchronize()
    ts = [[] for _ in fns]
    for _ in range(iters):
        for i, f in enumerate(fns):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            ts[i].append(e0.elapsed_time(e1))
    return [sorted(t)[len(t) // 2] for t in ts]


def report(case, N, ref_ms, ours_ms, impl, diff):
    print(f"REFCASE {case} N={N} ref_ms={ref_ms:.4f} ours_ms={ours_ms:.4f} ratio={ref_ms / ours_ms:.3f} "
          f"ref_impl={impl} max_abs_diff={diff:.4g}", flush=True)


def case_attention(N, a, masked=False, k2b=False):
    H, D = 4, 32
    g = torch.Generator(device="cuda").manual_seed(0)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)  # noqa: E731
    q, k, v = [rn(N, N, H * D).bfloat16() for _ in range(3)]
    Np = pair.ceil_to(N, 8)
    bias = torch.zeros(H, N, Np, device="cuda")
    bias[:, :, :N] = rn(H, N, N)
    keep = None
    if masked:
        keep = torch.ones(N, N, device="cuda")
        keep[:, N - N // 10:] = 0               # a padded tail of a tenth of the keys
    # this library: q pre-scaled by log2(e)/sqrt(D), bias by log2(e), bf16 planes
    qs = (q.float() * (pair.LOG2E / D ** 0.5)).bfloat16()
    bs = (bias * pair.LOG2E).bfloat16()
    out = torch.empty_like(q)
    km = None if keep is None else pair.KeyMask.pack(keep)
    ours = lambda: pair.attention(qs, k, v, bs, None, out, N, N, N, H, D, ldb=Np, mask=km)  # noqa: E731
    # the reference: [B, N, H, S, D] operands, fp32 bias [B, 1, H, S, S], bool mask [B, N, 1, 1, S]
    q5 = q.view(1, N, N, H, D).permute(0, 1, 3, 2, 4)
    k5 = k.view(1, N, N, H, D).permute(0, 1, 3, 2, 4)
    v5 = v.view(1, N, N, H, D).permute(0, 1, 3, 2, 4)
    b5 = bias[:, :, :N].contiguous().view(1, 1, H, N, N)
    m5 = None if keep is None else (keep > 0).view(1, N, 1, 1, N)
    if k2b:
        from opt_core.kernels.fpf_triatt_k2b import triatt_k2b as mod
        name = "k2b"
    else:
        from opt_core.kernels import flash_triattn as mod
        name = "flash_triattn"
    fn = mod.flash_triangle_attention
    holder = {}

    def ref():
        holder["o"] = fn(q5, k5, v5, b5, m5)
    ref()
    ours()
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "attention")
    o_ref = holder["o"][0].permute(0, 2, 1, 3).reshape(N, N, H * D).float()
    diff = (o_ref - out.float()).abs().max().item()
    r, o = interleaved([ref, ours], a.iters, a.warmup)
    report(("attention_k2b" if k2b else "attention") + ("_masked" if masked else ""), N, r, o, name, diff)


def _trimul_weights(g, c=128):
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)  # noqa: E731
    return dict(niw=1 + 0.1 * rn(c), nib=0.1 * rn(c), now=1 + 0.1 * rn(c), nob=0.1 * rn(c),
                p_in=rn(2 * c, c) * c ** -0.5, g_in=rn(2 * c, c) * c ** -0.5,
                p_out=rn(c, c) * c ** -0.5, g_out=rn(c, c) * c ** -0.5)


def case_trimul(N, a, outgoing=True):
    from opt_core.kernels.fpf_trimul_v4 import generic
    c = 128
    g = torch.Generator(device="cuda").manual_seed(1)
    z = (torch.randn(N, N, c, device="cuda", generator=g) + 0.2).bfloat16()
    w = _trimul_weights(g)
    packed = pair.TrimulPacked.pack(w["niw"], w["nib"], w["p_in"], w["g_in"], w["now"], w["nob"], w["p_out"], w["g_out"])
    ws = {}
    out = torch.empty_like(z)
    ours = lambda: pair.trimul_fused(z, None, packed, outgoing, residual=True, out=out, workspace=ws)  # noqa: E731
    # Boltz-2 layout: p_in / g_in are [2c, c] with the a half first
    rw = generic.pack_weights(ln_in_w=w["niw"], ln_in_b=w["nib"], ln_out_w=w["now"], ln_out_b=w["nob"],
                              w_o=w["p_out"], w_og=w["g_out"], w_ag=w["g_in"][:c], w_ap=w["p_in"][:c],
                              w_bg=w["g_in"][c:], w_bp=w["p_in"][c:])
    holder = {}
    z4 = z.unsqueeze(0)

    def ref():
        holder["o"] = generic.trimul(z4, None, direction="outgoing" if outgoing else "incoming", weights=rw,
                                     residual=True)
    ref()
    ours()
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "trimul")
    diff = (holder["o"].float().reshape(N, N, c) - out.float()).abs().max().item()
    r, o = interleaved([ref, ours], a.iters, a.warmup)
    report("trimul_" + ("outgoing" if outgoing else "incoming"), N, r, o, "fpf_trimul_v4", diff)


def case_transition(N, a):
    from opt_core.kernels.fpf_transition_v2 import kernel as tk
    c, hidden = 128, 512
    g = torch.Generator(device="cuda").manual_seed(2)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)  # noqa: E731
    x = (rn(N * N, c) + 0.3).bfloat16()
    nw, nb = 1 + 0.1 * rn(c), 0.1 * rn(c)
    fc1, fc2, fc3 = rn(hidden, c) * c ** -0.5, rn(hidden, c) * c ** -0.5, rn(c, hidden) * hidden ** -0.5
    packed = pair.TransitionPacked.pack(nw, nb, fc1, fc2, fc3)
    out = torch.empty_like(x)
    ours = lambda: pair.transition_fused(x, packed, residual=True, out=out)  # noqa: E731
    rp = tk.pack_weights(nw, nb, fc1, fc2, fc3, 1e-5, x.device)
    out_r = torch.empty_like(x)
    ref = lambda: tk.fused_transition(x, rp, residual=True, out2d=out_r, numerics="fast")  # noqa: E731
    ref()
    ours()
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "transition")
    diff = (out_r.float() - out.float()).abs().max().item()
    r, o = interleaved([ref, ours], a.iters, a.warmup)
    report("transition", N, r, o, "fpf_transition_v2(numerics=fast)", diff)


def case_layernorm(N, a):
    from opt_core.kernels.ln.fastln import fastln
    c = 128
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(N * N, c, device="cuda", generator=g).bfloat16()
    w, b = torch.ones(c, device="cuda"), torch.zeros(c, device="cuda")
    holder = {}

    def ref():
        holder["o"] = fastln.fast_layer_norm_triton(x, (c,), w.bfloat16(), b.bfloat16())
    def ours():
        holder["m"] = rows.layernorm_rows(x, w, b, 1e-5)
    ref()
    ours()
    torch.cuda.synchronize()
    diff = (holder["o"].float() - holder["m"].float()).abs().max().item()
    r, o = interleaved([ref, ours], a.iters, a.warmup)
    report("layernorm", N, r, o, "fastln", diff)


CASES = {
    "attention": lambda N, a: case_attention(N, a),
    "attention_masked": lambda N, a: case_attention(N, a, masked=True),
    "attention_k2b": lambda N, a: case_attention(N, a, k2b=True),
    "trimul_outgoing": lambda N, a: case_trimul(N, a, True),
    "trimul_incoming": lambda N, a: case_trimul(N, a, False),
    "transition": case_transition,
    "layernorm": case_layernorm,
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=1536)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--cases", default=",".join(CASES))
    a = ap.parse_args()
    if not os.path.isdir(os.path.join(REF, "opt_core")):
        print("REFCASE all unavailable: baseline/_ref/opt_core is not installed", flush=True)
        return
    sys.path.insert(0, REF)
    from importlib.metadata import version
    print(f"REFSTACK torch={torch.__version__} triton={version('triton')} gpu={torch.cuda.get_device_name(0)} "
          f"cc={torch.cuda.get_device_capability(0)}", flush=True)
    for name in a.cases.split(","):
        try:
            with torch.no_grad():
                CASES[name](a.n, a)
        except Exception as e:  # the reference refuses by raising; report its words and go on
            print(f"REFCASE {name} unavailable: {type(e).__name__}: {str(e)[:300]}", flush=True)
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
