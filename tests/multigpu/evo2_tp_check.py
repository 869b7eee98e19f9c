"""Run as P rank processes (one per GPU): StripedHyena-2 under tensor parallelism against the same model on one GPU -
prefill logits, then decode steps through the folded decode block (column-parallel projections with RMSNorm / SwiGLU
folded in on this rank's slice, row-parallel projections as partial rows + all-reduce + bias and residual) and the
single-query cache attention on this rank's heads, eagerly and as a captured graph.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 --master-port 29574 \
        tests/multigpu/evo2_tp_check.py [tokens] [steps]

Prints ``EVO2-TP ok ...`` on rank 0; exits non-zero on mismatch.
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from uplifting_biomolecular_modeling_b200.models import evo2
from uplifting_biomolecular_modeling_b200.ops import native
from uplifting_biomolecular_modeling_b200.parallel import comm as C
from uplifting_biomolecular_modeling_b200.parallel import tp


def build(dev):
    # head dimension 128 (the decode attention kernels), every operator kind, an attention layer
    m = evo2.build("evo2_tiny", device=dev, dtype=torch.bfloat16, seed=7, d_model=512, n_heads=4, ffn=1024, n_layers=5,
                   attn_layers=(3,))
    m.set_impl("fused")
    return m


def main():
    L = int(sys.argv[1]) if len(sys.argv) > 1 else 192
    steps = int(sys.argv[2]) if len(sys.argv) > 2 else 4
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    g = torch.Generator(device=dev).manual_seed(3)
    tok = torch.randint(0, 512, (1, L), device=dev, generator=g)
    feed = torch.randint(0, 512, (1, steps), device=dev, generator=g)

    one = build(dev)
    st1 = [dict() for _ in one.blocks]
    want = [one(tok, st1).float()[:, -1]]
    for i in range(steps):
        want.append(one.step(feed[:, i:i + 1], st1).float()[:, -1])
    want_tokens = one.generate(tok, steps + 2, graph=True)

    par = tp.TensorParallel(C.GroupComm(), None)
    many = build(dev)
    par.shard_evo2(many)
    assert many.folded is not None
    stp = [dict() for _ in many.blocks]
    got = [many(tok, stp).float()[:, -1]]
    for i in range(steps):
        got.append(many.step(feed[:, i:i + 1], stp).float()[:, -1])
    got_tokens = many.generate(tok, steps + 2, graph=True)
    torch.cuda.synchronize()
    native.raise_on_status(dev, "evo2 tensor parallel")

    scale = max(float(w.abs().max()) for w in want)
    err = max(float((a - b).abs().max()) for a, b in zip(got, want))
    same = int(torch.equal(got_tokens, want_tokens))
    t = torch.tensor([err, float(1 - same)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = float(t[0]) <= 6e-2 * scale
    if rank == 0:
        print(f"EVO2-TP {'ok' if ok else 'MISMATCH'} world={world} tokens={L} steps={steps} "
              f"max_abs_err={float(t[0]):.3e} scale={scale:.3e} graph_tokens_equal={int(float(t[1]) == 0)} "
              f"reduce_calls={par.reduce_calls}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
