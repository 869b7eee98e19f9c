"""Run under torchrun on P GPUs: the fused row-sharded Pairformer pair block against the dense block.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 --master-port 29531 \
        tests/multigpu/rowpair_fused_check.py [N]

Every rank builds the same layer (seed 0), rank r runs its row shard through ``FusedRowPair`` and the
gathered result is compared with the single-GPU fused block and with the plain fp32 statement.  Prints one
``ROWPAIR-FUSED ok ...`` line on rank 0 and exits non-zero on mismatch or on a non-zero kernel status word.
"""
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from uplifting_biomolecular_modeling_b200.models import pairformer
from uplifting_biomolecular_modeling_b200.ops import native
from uplifting_biomolecular_modeling_b200.parallel import comm as C
from uplifting_biomolecular_modeling_b200.parallel import rowpair
from uplifting_biomolecular_modeling_b200.parallel.layout import Layout
from uplifting_biomolecular_modeling_b200.parallel.rowpair_fused import FusedRowPair
from uplifting_biomolecular_modeling_b200.parallel.symm import SymmHeap


def main():
    N = int(sys.argv[1]) if len(sys.argv) > 1 else 384
    iters = int(sys.argv[2]) if len(sys.argv) > 2 else 0
    gather = sys.argv[3] if len(sys.argv) > 3 else "peer"
    check = N <= 1024                      # the fp32 dense statement needs O(N^3) memory-time; skip when large
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    comm = C.GroupComm()
    heap = SymmHeap(device=dev)
    torch.manual_seed(0)
    layer = pairformer.PairformerLayer(no_seq=True).to(dev).eval()
    for p in layer.parameters():
        p.requires_grad_(False)
    z = torch.randn(N, N, 128, device=dev)
    lay = Layout(N, world, align=128)
    with torch.no_grad():
        ref32 = layer.pair_update(z.unsqueeze(0), None)[0] if check else z
        lb = layer.to(torch.bfloat16)
        zb = z.bfloat16()
        fr = FusedRowPair(lay, comm, heap, gather=gather)
        z_loc = rowpair.shard_rows(zb, lay, rank)
        out_loc = fr.pair_block_(lb, z_loc)
        torch.cuda.synchronize()
        native.raise_on_status(dev, "fused rowpair block")
        e_dense = e_ref = 0.0
        if check:
            full = comm.all_gather_rows(out_loc.contiguous())
            pairformer.set_impl(lb, "fused")
            for m in lb.modules():
                if hasattr(m, "_packed"):
                    m._packed = None
            dense = lb.pair_update(zb.unsqueeze(0), None)[0]
            torch.cuda.synchronize()
            upd_ref = (ref32 - z)
            e_dense = ((full.float() - dense.float()).abs().mean() / upd_ref.abs().mean()).item()
            e_ref = ((full.float() - ref32).abs().mean() / upd_ref.abs().mean()).item()
            del full, dense
        del ref32
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
    ms = None
    if iters:
        with torch.no_grad():
            for _ in range(2):
                fr.pair_block_(lb, z_loc)
            dist.barrier(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fr.pair_block_(lb, z_loc)
            e1.record(); torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            native.raise_on_status(dev, "fused rowpair block (timed)")
    ok = e_dense < 2e-2 and e_ref < 6e-2
    if rank == 0:
        print(f"ROWPAIR-FUSED {'ok' if ok else 'MISMATCH'} world={world} N={N} gather={gather} err_vs_single_gpu_fused={e_dense:.4f} "
              f"err_vs_fp32={e_ref:.4f} ms_per_block={ms} peak_GB={torch.cuda.max_memory_allocated() / 2**30:.2f}",
              flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
