"""Forward passes of the protein-LM and genomic-track families: kernel path against the plain PyTorch statements.

    python benchmarks/sequence_families.py --model esmc_300m --batch 8 --length 2048
    python benchmarks/sequence_families.py --model progen2_small --batch 8 --length 1024
    python benchmarks/sequence_families.py --model gpnstar_200m --batch 4 --length 512
    python benchmarks/sequence_families.py --model enformer --batch 1 --length 196608
    python benchmarks/sequence_families.py --model chrombpnet --batch 64

bf16, random-init weights of the named configuration, synthetic inputs.  Both arms run the same module with the
same weights; ``reference`` is the plain PyTorch statement list in bf16 (library convolutions / SDPA), ``fused`` the
kernel path.  CUDA-event times after warm-up; one JSON line per run.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="esmc_300m")
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--length", type=int, default=0, help="tokens / bases per sequence (0 = the model's natural input)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    from uplifting_biomolecular_modeling_b200.models import genomics, plm
    from uplifting_biomolecular_modeling_b200.ops import native
    dev = "cuda:0"
    g = torch.Generator().manual_seed(0)
    if a.model in plm.CONFIGS:
        m = plm.build(a.model, device=dev, dtype=torch.bfloat16, seed=0)
        cfg = m.cfg
        L = a.length or 1024
        hi = 8 if cfg.family == "gpnstar" else min(cfg.vocab, 24)
        toks = torch.randint(4, hi, (a.batch, L), generator=g).to(dev)
        kw = {}
        if cfg.family == "gpnstar":
            al, idx = plm.synthetic_alignment(cfg, toks)
            kw = {"alignment": al, "clade_index": idx}
        run = lambda: m(toks, **kw)
        units = a.batch * L
    else:
        m = genomics.build(a.model, device=dev, dtype=torch.bfloat16, seed=0)
        cfg = m.cfg
        L = a.length or genomics.input_length(cfg, bins=1536 - 2 * cfg.crop if cfg.family != "chrombpnet" else 8)
        idx = torch.randint(0, 4, (a.batch, L), generator=g)
        x = torch.zeros(a.batch, L, 8).scatter_(2, idx[..., None], 1.0).to(dev).bfloat16()
        run = lambda: m(x)
        units = a.batch * L
    res = {"model": a.model, "batch": a.batch, "length": L, "dtype": "bf16", "data": "synthetic"}
    for impl in ("reference", "fused"):
        m.set_impl(impl)
        n0 = native.launch_count()
        with torch.no_grad():
            for _ in range(a.warmup):
                run()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.iters):
                run()
            e1.record()
            torch.cuda.synchronize()
        native.raise_on_status(dev)
        ms = e0.elapsed_time(e1) / a.iters
        res[f"{impl}_ms"] = round(ms, 3)
        res[f"{impl}_units_per_s"] = round(units / ms * 1e3, 1)
        res[f"{impl}_kernel_launches"] = (native.launch_count() - n0) // (a.warmup + a.iters)
    res["speedup"] = round(res["reference_ms"] / res["fused_ms"], 3)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
