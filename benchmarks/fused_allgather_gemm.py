"""All-gather -> triangle-contraction GEMM, fused versus NCCL, on P GPUs (run under torchrun).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 --master-port 29541 \
        benchmarks/fused_allgather_gemm.py [--tokens 4096] [--iters 5]

Every rank holds R = N / P rows of the projected operands a, b as channel-major planes [128][R][N] and
computes x[c][i][j] = sum_k a[c][i][k] * b[c][j][k] for its rows i and ALL j, which needs every other rank's b
rows.  Arms: ``fused`` (one kernel: copy CTAs pull each remote block over NVLink once while the compute CTAs
start on the local shard), ``direct`` (the GEMM's TMA loads read remote tiles in place, once per m-tile),
``nccl`` (all_gather_into_tensor, then the local GEMM).  Times are CUDA-event times, max over ranks.
Roofline of the step: the slower of FLOPs / measured bf16 peak and bytes over NVLink / 770 GB/s per direction.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from uplifting_biomolecular_modeling_b200.ops import gemm, native, peer
from uplifting_biomolecular_modeling_b200.parallel.symm import SymmHeap


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--copy-ctas", type=int, default=16)
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    heap = SymmHeap(device=dev)
    N, C = a.tokens, 128
    R = N // world
    planes = heap.alloc((2, C, R, N), torch.bfloat16)
    torch.manual_seed(rank)
    planes.local.copy_(torch.randn(2, C, R, N, device=dev).bfloat16())
    x = torch.empty((C, R, N), dtype=torch.bfloat16, device=dev)
    heap.barrier()
    b_off = C * R * N * 2
    ptrs = [planes.ptr(q, b_off) for q in range(world)]
    counts = [R] * world
    gs = peer.GatherState(C, N, N, dev, copy_ctas=a.copy_ctas)
    b_all = torch.empty((world, C, R, N), dtype=torch.bfloat16, device=dev)

    def fused():
        heap.barrier()
        peer.gemm_allgather_b(planes.local[0], ptrs, counts, x, K=N, ldb=N, stride_b=R * N, my_rank=rank, gather=gs)
        heap.barrier()

    def direct():
        heap.barrier()
        peer.gemm_allgather_b(planes.local[0], ptrs, counts, x, K=N, ldb=N, stride_b=R * N, my_rank=rank)
        heap.barrier()

    def nccl():
        dist.all_gather_into_tensor(b_all, planes.local[1])
        bf = b_all.permute(1, 0, 2, 3).reshape(C, N, N)          # view-compatible: [C][P*R][N] needs a copy
        gemm.gemm(planes.local[0], bf.contiguous() if not bf.is_contiguous() else bf, out=x)

    def timeit(fn):
        for _ in range(2):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        ts = []
        for _ in range(a.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.barrier()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    res = {}
    ref = None
    for name, fn in (("nccl", nccl), ("fused", fused), ("direct", direct)):
        if name == "direct" and world > 2 and N > 2048:
            continue                                  # re-reads every remote tile per m-tile: only worth timing small
        ms = timeit(fn)
        native.raise_on_status(dev, name)
        chk = float(x.float().abs().mean())
        if ref is None:
            ref = x.clone()
        err = float((x.float() - ref.float()).abs().max())
        res[name] = {"ms": round(ms, 3), "max_abs_diff_vs_nccl": err, "mean_abs": round(chk, 4)}
    flops = 2.0 * C * R * N * N
    nv_bytes = (world - 1) * C * R * N * 2
    peaks = os.path.join(ROOT, "MEASURED_PEAKS.json")
    pf = json.load(open(peaks))["bf16_tflops"] * 1e12 if os.path.exists(peaks) else 1.59e15
    roof_ms = max(flops / pf, nv_bytes / 770e9) * 1e3
    if rank == 0:
        for k, v in res.items():
            v["fraction_of_roofline"] = round(roof_ms / v["ms"], 3)
        print("FUSED-AG-GEMM " + json.dumps({"world": world, "N": N, "rows_per_rank": R, "tflop_per_rank": flops / 1e12,
                                             "nvlink_gb_per_rank": nv_bytes / 1e9, "roofline_ms": round(roof_ms, 3),
                                             "bound": "compute" if flops / pf > nv_bytes / 770e9 else "nvlink",
                                             "arms": res}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
