"""Run one kernel of the library on a named case, timed with CUDA events (and small enough for ncu).

    python benchmarks/kernel_cases.py <case> [--n N] [--iters K] [--warmup W]

Cases: ``attention`` (triangle-attention core, H=4 x D=32, rows = N), ``attention_d64`` (token attention,
16 heads x 64, 5 samples), ``trimul_proj``, ``trimul_gemm``, ``trimul_out``, ``triatt_proj``, ``transition``,
``out_gemm`` (the [N*N,128] x [128,128] output projection with residual), ``trimul`` (three launches),
``triatt`` (three launches), ``causal_attention`` (--n tokens, --heads, head dimension 128; --lib 1 = the
library call), ``gemm_rows`` (--m --k --nn: a row GEMM with bias), ``gemv_rows`` (--m <= 8 rows, --k, --nn, --form), ``decode_attention`` (--n cached keys, --heads), ``fir_inner_gate`` (--n positions, --k channels, --nn taps), ``window_attention`` (--m atoms,
5 samples, 4 heads x 32).  Inputs are larger than L2 for N >= 768.  Prints one line per case with the
mean time, the algorithmic bytes and FLOPs, and the fractions of the measured peaks in MEASURED_PEAKS.json
(fallback 6.65 TB/s, 1.59 PFLOP/s when the file is absent).
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch

from uplifting_biomolecular_modeling_b200.ops import gemm, native, pair


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


def timeit(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    ts = []
    for _ in range(iters):
        flush.zero_()                       # write a buffer larger than L2 between timed launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--n", type=int, default=768)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--attn-variant", type=int, default=0, help="attention: 0 = default (four rows per CTA from 4 rows on), 5 = two rows per CTA, 1 = P and bias through shared memory, +16 = no polynomial exponentials; window_attention: 1 = CUDA-core kernel")
    ap.add_argument("--m", type=int, default=7680, help="rows of the gemm_rows case / atoms of window_attention")
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--nn", type=int, default=3072)
    ap.add_argument("--heads", type=int, default=32, help="causal_attention: heads")
    ap.add_argument("--lib", type=int, default=0, help="causal_attention: 1 = time the library attention instead")
    ap.add_argument("--masked", type=int, default=0, help="attention: 1 = key mask with a padded tail of a tenth of the keys")
    ap.add_argument("--form", default="plain", help="gemv_rows: plain | norm (RMSNorm in front) | res (residual behind) | swiglu (RMSNorm + two matrices); gemm_rows: fp8 = e4m3 operands")
    ap.add_argument("--incoming", type=int, default=0, help="trimul / trimul_gemm: 1 = the incoming update (MN-major contraction)")
    a = ap.parse_args()
    N, c = a.n, 128
    pair.set_attention_variant(a.attn_variant)
    dev = "cuda"
    torch.manual_seed(0)
    r = lambda *s: torch.randn(*s, device=dev) * 0.08  # noqa: E731
    ones, zeros = torch.ones(c, device=dev), torch.zeros(c, device=dev)
    z = torch.randn(N, N, c, device=dev).bfloat16() if a.case not in ("causal_attention", "gemm_rows", "gemv_rows", "decode_attention", "fir_inner_gate") else None
    Np = pair.ceil_to(N, 8)
    st = native.status_tensor(dev)
    stream = native.current_stream(dev)
    lib = native.lib()
    byts = flops = 0
    if a.case in ("attention", "attention_d64"):
        if a.case == "attention":
            rows, H, D = N, 4, 32
        else:
            rows, H, D = 5, 16, 64
        q = torch.randn(rows, N, H * D, device=dev).bfloat16()
        k, v, g = torch.randn_like(q), torch.randn_like(q), torch.rand_like(q)
        bias = torch.randn(H, N, Np, device=dev).bfloat16()
        out = torch.empty_like(q)
        km = None
        if a.masked:
            keep = torch.ones(rows, N, device=dev)
            keep[:, N - N // 10:] = 0
            km = pair.KeyMask.pack(keep)
        fn = lambda: pair.attention(q, k, v, bias, g, out, rows, N, N, H, D, ldb=Np, mask=km)  # noqa: E731
        byts = 5 * q.numel() * 2 + bias.numel() * 2
        flops = 4.0 * rows * H * N * N * D
    elif a.case in ("trimul_proj", "trimul_gemm", "trimul_out", "trimul"):
        w = pair.TrimulPacked.pack(ones, zeros, r(256, c), r(256, c), ones, zeros, r(c, c), r(c, c))
        planes = torch.empty((2, 128, N, Np), dtype=torch.bfloat16, device=dev)
        x = torch.empty((128, N, Np), dtype=torch.bfloat16, device=dev)
        out = torch.empty_like(z)
        f1 = lambda: lib.ubm_trimul_proj(native.ptr(z), native.ptr(w.w_in), native.ptr(w.in_colsum),  # noqa: E731
                                         native.ptr(w.in_colbias), 0, native.ptr(planes), 0, N, Np, native.ptr(st),
                                         stream)
        f2 = lambda: gemm.gemm(planes[0][:, :, :N], planes[1][:, :, :N], mn_major=bool(a.incoming),  # noqa: E731
                               out=x[:, :, :N])
        f3 = lambda: lib.ubm_trimul_out(native.ptr(x), native.ptr(z), native.ptr(w.wo), native.ptr(w.wg),  # noqa: E731
                                        native.ptr(w.o_colsum), native.ptr(w.o_colbias), native.ptr(w.g_colsum),
                                        native.ptr(w.g_colbias), native.ptr(out), N, Np, 1, native.ptr(st), stream)
        f1(); f2()
        zb = z.numel() * 2
        if a.case == "trimul_proj":
            fn, byts, flops = f1, 3 * zb, 2.0 * N * N * 128 * 512
        elif a.case == "trimul_gemm":
            fn, byts, flops = f2, 3 * zb, 2.0 * 128 * N ** 3
        elif a.case == "trimul_out":
            fn, byts, flops = f3, 3 * zb, 2.0 * N * N * 128 * 256
        else:
            fn = lambda: (f1(), f2(), f3())  # noqa: E731
            byts, flops = 9 * zb, 2.0 * 128 * N ** 3 + 2.0 * N * N * 128 * 768
    elif a.case == "head_bias":
        from uplifting_biomolecular_modeling_b200.ops import rows as rows_ops
        wb = r(16, c)
        hb = torch.empty((16, N, Np), dtype=torch.bfloat16, device=dev)
        fn = lambda: rows_ops.pair_head_bias(z, ones, zeros, wb, out=hb)  # noqa: E731
        byts, flops = z.numel() * 2 + hb.numel() * 2, 2.0 * N * N * 128 * 16
    elif a.case in ("triatt_proj", "triatt"):
        w = pair.TriattPacked.pack(ones, zeros, r(4, c), r(c, c), r(c, c), r(c, c), r(c, c), r(c), r(c, c), r(c), 4)
        ws = {}
        out = torch.empty_like(z)
        if a.case == "triatt":
            fn = lambda: pair.triangle_attention_fused(z, w, True, out=out, workspace=ws)  # noqa: E731
            byts, flops = 11 * z.numel() * 2, 4.0 * N * 4 * N * N * 32 + 2.0 * N * N * 128 * 640
        else:
            bufs = torch.empty((4, N * N, 128), dtype=torch.bfloat16, device=dev)
            hb = torch.zeros((4, N, Np), dtype=torch.bfloat16, device=dev)
            fn = lambda: lib.ubm_triatt_proj(native.ptr(z), native.ptr(w.w), native.ptr(w.colsum),  # noqa: E731
                                             native.ptr(w.colbias), native.ptr(w.wb), native.ptr(w.wb_colsum),
                                             native.ptr(w.wb_colbias), native.ptr(bufs[0]), native.ptr(bufs[1]),
                                             native.ptr(bufs[2]), native.ptr(bufs[3]), native.ptr(hb), 0, N, Np, 4, 0,
                                             native.ptr(st), stream)
            byts, flops = 5 * z.numel() * 2, 2.0 * N * N * 128 * 512
    elif a.case == "transition":
        w = pair.TransitionPacked.pack(ones, zeros, r(512, c), r(512, c), r(c, 512))
        out = torch.empty_like(z)
        fn = lambda: pair.transition_fused(z, w, out=out)  # noqa: E731
        byts, flops = 2 * z.numel() * 2, 2.0 * N * N * (128 * 1024 + 512 * 128)
    elif a.case == "out_gemm":
        og = torch.randn(N * N, c, device=dev).bfloat16()
        wo = r(c, c).bfloat16()
        out = torch.empty_like(og)
        fn = lambda: gemm.gemm(og, wo, bias=zeros, residual=z.view(N * N, c), out=out)  # noqa: E731
        byts, flops = 3 * og.numel() * 2, 2.0 * N * N * c * c
    elif a.case == "gemm_rows":
        # plain row GEMM with bias, the shape family of the diffusion transformer: [m, k] x [nn, k]^T
        M, K, NN = a.m, a.k, a.nn
        x = torch.randn(M, K, device=dev).bfloat16()
        wt = r(NN, K).bfloat16()
        bvec = torch.zeros(NN, device=dev)
        out = torch.empty((M, NN), dtype=torch.bfloat16, device=dev)
        fn = lambda: gemm.gemm(x, wt, bias=bvec, out=out)  # noqa: E731
        byts, flops = (x.numel() + wt.numel() + out.numel()) * 2, 2.0 * M * K * NN
        if a.form == "fp8":             # the same product with e4m3 operands (kind::f8f6f4)
            x8, dqx = gemm.quantize_e4m3(x)
            w8, dqw = gemm.quantize_e4m3(wt)
            fn = lambda: gemm.gemm_fp8(x8, w8, alpha=dqx * dqw, bias=bvec, out=out)  # noqa: E731
            byts = x.numel() + wt.numel() + out.numel() * 2
    elif a.case == "gemv_rows":
        # decode projection: --m rows (<= 8) x [nn, k] weights streamed once; --form plain | norm | res | swiglu
        from uplifting_biomolecular_modeling_b200.ops import seq
        M, K, NN = a.m, a.k, a.nn
        x = torch.randn(M, K, device=dev).bfloat16()
        wt, w2 = r(NN, K).bfloat16(), r(NN, K).bfloat16()
        gamma = torch.ones(K, device=dev)
        res = torch.randn(M, NN, device=dev).bfloat16()
        kw = {"plain": {}, "norm": {"gamma": gamma}, "res": {"res": res}, "swiglu": {"gamma": gamma, "w2": w2}}[a.form]
        fn = lambda: seq.gemv_rows(x, wt, **kw)  # noqa: E731
        byts, flops = wt.numel() * 2 * (2 if a.form == "swiglu" else 1), 2.0 * M * K * NN
    elif a.case == "fir_inner_gate":
        # inner operator of a Hyena layer over --n positions x --k channels with --nn taps (128 = the medium filter:
        # the tiled direct convolution), gate included
        from uplifting_biomolecular_modeling_b200.ops import seq
        Lp, ch, taps = N, a.k, a.nn
        u = torch.randn(1, Lp, ch, device=dev).bfloat16()
        x2 = torch.randn(1, Lp, ch, device=dev).bfloat16()
        ht = seq.taps_major(torch.randn(ch, taps, device=dev) * taps ** -0.5)
        Dv = torch.randn(ch, device=dev)
        fn = lambda: seq.fir_inner_gate(u, ht, Dv, x2, None)  # noqa: E731
        byts, flops = 3 * u.numel() * 2, 2.0 * Lp * ch * taps
    elif a.case == "decode_attention":
        # one new token against a cache of --n keys (--heads heads of 128): rotary + cache write, split-key pass, merge
        from uplifting_biomolecular_modeling_b200.ops import seq
        Hh = a.heads
        kc = torch.randn(1, N + 1, Hh, 128, device=dev).bfloat16()
        vc = torch.randn(1, N + 1, Hh, 128, device=dev).bfloat16()
        qkv = torch.randn(1, 3 * Hh * 128, device=dev).bfloat16()
        pos = torch.full((1,), N, dtype=torch.long, device=dev)
        fn = lambda: seq.decode_attention(qkv, pos, kc, vc, 10000.0)  # noqa: E731
        byts, flops = 2 * (N + 1) * Hh * 128 * 2, 4.0 * (N + 1) * Hh * 128
    elif a.case == "causal_attention":
        # causal self-attention at head dimension 128: --n tokens, --heads heads, batch 1; --lib 1 times the library call
        import torch.nn.functional as F
        from uplifting_biomolecular_modeling_b200.ops import causal
        T, Hh = N, a.heads
        qkv = torch.randn(1, T, 3, Hh, 128, device=dev).bfloat16()
        q, k, v = qkv.unbind(2)
        out = torch.empty(1, T, Hh, 128, device=dev, dtype=torch.bfloat16)
        if a.lib:
            qh, kh, vh = (t.transpose(1, 2) for t in (q, k, v))
            fn = lambda: F.scaled_dot_product_attention(qh, kh, vh, is_causal=True)  # noqa: E731
        else:
            fn = lambda: causal.causal_attention(q, k, v, out=out)  # noqa: E731
        byts, flops = 4 * T * Hh * 128 * 2, 4.0 * T * T * 128 * Hh / 2
    elif a.case == "window_attention":
        B, A, H = 5, a.m // 32 * 32, 4
        xw = torch.randn(B * A, 3 * H * 32, device=dev).bfloat16()
        bias = torch.randn(1, H, A // 32, 32, 128, device=dev).bfloat16()
        gate = torch.rand(B * A, H * 32, device=dev).bfloat16()
        out = torch.empty_like(gate)
        native.declare("ubm_window_attention", [native.c_void_p] * 6 + [native.c_int, native.c_int, native.c_int,
                                                                       native.c_ll, native.c_int, native.c_void_p])
        if a.attn_variant == 1:       # CUDA-core kernel, one window per CTA
            fn = lambda: lib.ubm_window_attention(native.ptr(xw), native.ptr(xw) + H * 64,  # noqa: E731
                                                  native.ptr(xw) + H * 128, native.ptr(bias), native.ptr(gate),
                                                  native.ptr(out), B, A, H, 3 * H * 32, 1, stream)
        else:                         # tcgen05 kernel, four windows per CTA
            fn = lambda: lib.ubm_window_attention_tc(native.ptr(xw), native.ptr(xw) + H * 64,  # noqa: E731
                                                     native.ptr(xw) + H * 128, native.ptr(bias), native.ptr(gate),
                                                     native.ptr(out), B, A, H, 3 * H * 32, 1, native.ptr(st), stream)
        byts = (xw.numel() + bias.numel() + 2 * gate.numel()) * 2
        flops = 4.0 * B * A * H * 128 * 32
    else:
        raise SystemExit(f"unknown case {a.case}")
    ms = timeit(fn, a.iters, a.warmup)
    native.raise_on_status(dev, a.case)
    bw, fl, src = peaks()
    print(f"CASE {a.case} N={N} ms={ms:.4f} GB/s={byts / ms / 1e6:.0f} ({byts / ms / 1e-3 / bw:.3f} of {src} HBM) "
          f"TFLOP/s={flops / ms / 1e9:.0f} ({flops / ms / 1e-3 / fl:.3f} of {src} bf16)", flush=True)


if __name__ == "__main__":
    main()
