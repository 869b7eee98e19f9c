"""Run as P rank processes (one per GPU): the outer product mean of an MSA sharded over sequences, with the
reduce-scatter in the projection GEMM's epilogue, against the plain sharded statement (NCCL exchange) and the dense
fp32 module.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 --master-port 29571 \
        tests/multigpu/opm_seqshard_check.py [N] [S] [masked]

Prints ``OPM-SEQSHARD ok ...`` on rank 0; exits non-zero on mismatch or a non-zero kernel status word.
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from uplifting_biomolecular_modeling_b200.models import msa
from uplifting_biomolecular_modeling_b200.ops import native
from uplifting_biomolecular_modeling_b200.parallel import comm as C
from uplifting_biomolecular_modeling_b200.parallel import rowpair
from uplifting_biomolecular_modeling_b200.parallel.layout import Layout
from uplifting_biomolecular_modeling_b200.parallel.rowpair_fused import FusedRowPair
from uplifting_biomolecular_modeling_b200.parallel.symm import SymmHeap


def main():
    N = int(sys.argv[1]) if len(sys.argv) > 1 else 256
    S = int(sys.argv[2]) if len(sys.argv) > 2 else 96
    masked = bool(int(sys.argv[3])) if len(sys.argv) > 3 else False
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    comm = C.GroupComm()
    heap = SymmHeap(device=dev)
    torch.manual_seed(0)
    mod = msa.OuterProductMean(64, 32, 128).to(dev).eval()
    with torch.no_grad():
        for p in mod.parameters():
            p.normal_(0, 0.15)
        mod.norm.weight.add_(1.0)
    m = torch.randn(1, S, N, 64, device=dev)
    mask = torch.ones(1, S, N, device=dev)
    if masked:
        mask = (torch.rand(1, S, N, device=dev) > 0.2).float()
    mod.full_mask = not masked
    lay = Layout(N, world, align=128)
    a, b = lay.rows(rank)
    s0, s1 = rowpair.seq_bounds(S, world)[rank]
    with torch.no_grad():
        dense = mod(m, mask)[0]                                                      # fp32 plain statement, all rows
        fr = FusedRowPair(lay, comm, heap, gather="peer")
        import copy
        mb = copy.deepcopy(mod).to(torch.bfloat16)
        mb.full_mask = not masked
        got = fr.opm_seqshard_(m[:, s0:s1].bfloat16(), mask[:, s0:s1], mb, S)
        plain = rowpair.opm_seqshard(m[:, s0:s1], mask[:, s0:s1], mod, lay, comm, S)
        torch.cuda.synchronize()
        native.raise_on_status(dev, "opm seqshard")
        ref = dense[a:b]
        scale = ref.abs().mean().clamp(min=1e-6)
        e_fused = float(((got.float() - ref).abs().mean() / scale)) if b > a else 0.0
        e_plain = float(((plain.float() - ref).abs().mean() / scale)) if b > a else 0.0
    t = torch.tensor([e_fused, e_plain], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = float(t[0]) < 3e-2 and float(t[1]) < 1e-4
    if rank == 0:
        print(f"OPM-SEQSHARD {'ok' if ok else 'MISMATCH'} world={world} N={N} S={S} masked={int(masked)} "
              f"err_fused={float(t[0]):.4f} err_plain={float(t[1]):.2e}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
