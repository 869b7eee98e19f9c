"""Rank process of the StripedHyena-2 kit under tensor parallelism (``run.sh score|generate --mode fast --n_gpu P``).

Every rank builds the same model (same seed, or the same checkpoint), keeps its slice of every operator
(``parallel.tp.TensorParallel.shard_evo2``: channels of the Hyena operators, heads of the attention layers, columns /
rows of the projections) and runs the verb on the same tokens; row-parallel projections meet in a GEMM with the
reduce-scatter in its epilogue (prefill) or an all-reduce (decode).  Rank 0 writes the result.  On a machine without
GPUs the ranks run the plain statements over gloo, which is how the CPU suite holds this path.

Reference: the 2-device split of evo2's 40b kit (evo2/opt/evo2_opt/kit/multidev.py, kit/pipelined.py) is the
reference's multi-device form of this family; here the devices share every layer instead of dividing the layers.
"""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="evo2_7b")
    ap.add_argument("--verb", default="score")
    ap.add_argument("--prompt", default="ACGT" * 16)
    ap.add_argument("--input", default=None)
    ap.add_argument("--max_new_tokens", type=int, default=32)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--allow-partial", action="store_true")
    ap.add_argument("--fp8", type=int, default=0)
    ap.add_argument("--out", default=None, help="rank 0 writes the result here (JSON)")
    a = ap.parse_args(argv)

    import torch

    from ..kits.run import _sequence_records
    from ..models import lm, weights
    from . import launch, symm, tp

    comm = launch.init_from_env()
    cuda = torch.cuda.is_available()
    device = f"cuda:{torch.cuda.current_device()}" if cuda else "cpu"
    runner = lm.build("evo2", a.config, device=device, mode="fast", seed=a.seed, kit="evo2")
    if a.checkpoint:
        weights.load_checkpoint(runner.model, a.checkpoint, strict=not a.allow_partial)
    if cuda:
        runner.model.set_impl("fused")
        runner.decode_graph = True
        if a.fp8:
            runner.model.set_fp8_input_projections(True)
    par = tp.TensorParallel(comm, symm.SymmHeap() if cuda else None)
    par.shard_evo2(runner.model)
    records = _sequence_records(a.input) or [("prompt", a.prompt)]
    per = [dict(runner.run(a.verb, seq, max_new_tokens=a.max_new_tokens), id=name) for name, seq in records]
    if cuda:
        from ..ops import native
        native.raise_on_status(device, "tensor-parallel sequence kit")
    if comm.rank == 0:
        res = dict(per[0], records=len(per), world=comm.world, reduce_calls=par.reduce_calls,
                   fused_reduce_scatter_calls=par.fused_calls,
                   per_record=[{k: v for k, v in r.items() if isinstance(v, (int, float, str))} for r in per])
        if a.out:
            with open(a.out, "w") as f:
                json.dump(res, f)
        print("LM-WORKER " + json.dumps({k: v for k, v in res.items() if k != "per_record"}), flush=True)
    comm.barrier()          # nobody leaves while a peer still reads its symmetric buffers
    return 0


if __name__ == "__main__":
    sys.exit(main())
