"""Run as P rank processes (one per GPU): the token transformer of the sampler on token-row shards (one all-gather
of the AdaLN-normalised rows per layer over NCCL; queries, gates, transition and residuals local to the shard)
against the dense transformer on the same GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 --master-port 29573 \
        tests/multigpu/dit_rows_check.py [N] [depth]

Prints ``DIT-ROWS ok ...`` on rank 0; exits non-zero on mismatch.
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from uplifting_biomolecular_modeling_b200.models import diffusion
from uplifting_biomolecular_modeling_b200.parallel import comm as C
from uplifting_biomolecular_modeling_b200.parallel import rowpair
from uplifting_biomolecular_modeling_b200.parallel.layout import Layout


def main():
    N = int(sys.argv[1]) if len(sys.argv) > 1 else 200
    depth = int(sys.argv[2]) if len(sys.argv) > 2 else 3
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    comm = C.GroupComm()
    torch.manual_seed(0)                                   # same weights and inputs on every rank
    tr = diffusion.DiffusionTransformer(depth=depth, dim=256, dim_s=128, heads=8).to(dev).eval()
    with torch.no_grad():
        for p in tr.parameters():
            if p.dim() > 1:
                p.normal_(0, 0.08)
    a = torch.randn(3, N, 256, device=dev)                 # three samples
    s = torch.randn(1, N, 128, device=dev)
    bias = torch.randn(1, 8, N, N, device=dev)
    lay = Layout(N, world)
    r0, r1 = lay.rows(rank)
    with torch.no_grad():
        want = tr(a, s, [bias] * depth)
        got = rowpair.dit_rows(tr, a[:, r0:r1], s[:, r0:r1], bias[:, :, r0:r1], comm)
    torch.cuda.synchronize()
    err = float((got - want[:, r0:r1]).abs().max()) if r1 > r0 else 0.0
    t = torch.tensor([err], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = float(t[0]) < 2e-4
    if rank == 0:
        print(f"DIT-ROWS {'ok' if ok else 'MISMATCH'} world={world} N={N} depth={depth} max_abs_err={float(t[0]):.3e}",
              flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
