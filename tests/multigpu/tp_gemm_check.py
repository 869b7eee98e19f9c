"""GEMM -> reduce-scatter fused over peer memory against NCCL (run under torchrun, one rank per GPU).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29541 \
        tests/multigpu/tp_gemm_check.py [tokens] [d_model] [ffn] [iters]

Checks the fused row-parallel linear (each rank's epilogue stores its partial rows into the owner's slots, the
owner adds the slots) against torch.matmul + dist.reduce_scatter_tensor, then times both with CUDA events
(max over ranks).  Prints one line per rank 0.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def main():
    tokens = int(sys.argv[1]) if len(sys.argv) > 1 else 8192
    d = int(sys.argv[2]) if len(sys.argv) > 2 else 4096
    ffn = int(sys.argv[3]) if len(sys.argv) > 3 else 11264
    iters = int(sys.argv[4]) if len(sys.argv) > 4 else 10
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    from uplifting_biomolecular_modeling_b200.ops import native, peer
    from uplifting_biomolecular_modeling_b200.parallel import symm
    heap = symm.SymmHeap()
    kl = ffn // world                                   # this rank's slice of the contraction dimension
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    x = (torch.randn(tokens, kl, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(d, kl, device="cuda", generator=g) * kl ** -0.5).bfloat16()
    rows = tokens // world
    state = peer.ReduceScatterState(heap, rows, d)

    def fused():
        return peer.gemm_reduce_scatter(x, w, state)

    def nccl():
        part = x @ w.t()
        out = torch.empty((rows, d), dtype=torch.bfloat16, device="cuda")
        dist.reduce_scatter_tensor(out, part)
        return out

    a, b = fused(), nccl()
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "gemm_reduce_scatter")
    # fp32 oracle of this rank's rows
    parts = [torch.empty_like(x) for _ in range(world)]
    wparts = [torch.empty_like(w) for _ in range(world)]
    dist.all_gather(parts, x)
    dist.all_gather(wparts, w)
    ref = sum(p[rank * rows:(rank + 1) * rows].float() @ q.float().t() for p, q in zip(parts, wparts))
    err_f = (a.float() - ref).abs().max().item() / ref.abs().max().item()
    err_n = (b.float() - ref).abs().max().item() / ref.abs().max().item()

    def timeit(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    tf, tn = timeit(fused), timeit(nccl)
    native.raise_on_status("cuda", "gemm_reduce_scatter timing")
    if rank == 0:
        flops = 2.0 * tokens * d * kl
        nv_bytes = tokens * d * 2 * (world - 1) / world
        print(f"TP_GEMM_RS world={world} tokens={tokens} d={d} k_local={kl} fused_ms={tf:.3f} nccl_ms={tn:.3f} "
              f"err_fused={err_f:.2e} err_nccl={err_n:.2e} gemm_tflops={flops / tf / 1e9:.0f} "
              f"nvlink_GBs={nv_bytes / tf / 1e6:.0f}", flush=True)
    assert err_f < 2e-2, err_f
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
