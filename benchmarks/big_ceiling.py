"""Largest token count whose Pairformer pair block runs on ONE GPU, for the `fast` and the `big` pair stack.

    python benchmarks/big_ceiling.py [--start 4096] [--step 512] [--max 14336] [--modes fast,big] [--row-block 512]

The peak of a prediction's trunk is that of one pair block (blocks do not accumulate memory), so one block of the
Pairformer (no single track) is run at growing N until the allocator raises its out-of-memory exception; that
exception is caught, the buffers are dropped and the sweep ends for that mode - nothing faults.  The sweep is
bounded by ``--max``.  Per size: one warm run and one timed run, CUDA events, allocator peak.  Prints

    CEILING mode=<m> N=<n> ms_per_block=<..> peak_gb=<..>            per size that ran
    CEILING mode=<m> largest_N=<n> first_oom_N=<n|none>              per mode

The reference states single-GPU `big` ceilings of 2,000-6,000 tokens on an 80 GB H100 (per kit README).
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch

from uplifting_biomolecular_modeling_b200.models import pairformer
from uplifting_biomolecular_modeling_b200.ops import native


def one_size(layer, N, ws):
    z = torch.empty((1, N, N, 128), dtype=torch.bfloat16, device="cuda").normal_()
    ms = None
    for rep in range(2):
        torch.cuda.reset_peak_memory_stats()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = layer.pair_update(z, None)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        del out
    native.raise_on_status("cuda", "pair block")
    return ms, torch.cuda.max_memory_allocated() / 2 ** 30


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--start", type=int, default=4096)
    ap.add_argument("--step", type=int, default=512)
    ap.add_argument("--max", type=int, default=14336)
    ap.add_argument("--modes", default="fast,big")
    ap.add_argument("--row-block", type=int, default=512)
    a = ap.parse_args()
    torch.manual_seed(0)
    layer = pairformer.PairformerLayer(no_seq=True).to("cuda").to(torch.bfloat16).eval()
    for p in layer.parameters():
        p.requires_grad_(False)
    for mode in a.modes.split(","):
        largest, first_oom = None, None
        N = a.start
        while N <= a.max:
            ws = {"row_block": a.row_block} if mode == "big" else {}
            pairformer.set_impl(layer, "fused", workspace=ws)
            try:
                with torch.no_grad():
                    ms, peak = one_size(layer, N, ws)
            except torch.cuda.OutOfMemoryError:
                first_oom = N
                ws.clear()
                torch.cuda.empty_cache()
                break
            print(f"CEILING mode={mode} N={N} ms_per_block={ms:.1f} peak_gb={peak:.1f}", flush=True)
            largest = N
            ws.clear()
            torch.cuda.empty_cache()
            N += a.step
        print(f"CEILING mode={mode} largest_N={largest} first_oom_N={first_oom if first_oom else 'none'} "
              f"(sweep bound {a.max})", flush=True)


if __name__ == "__main__":
    main()
