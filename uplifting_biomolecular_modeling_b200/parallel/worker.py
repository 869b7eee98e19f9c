"""Rank worker of a row-sharded prediction (``pred --mode big --n_gpu P``).

Every rank builds the same model (same seed), rank 0 builds the features and broadcasts them, all ranks
check that replicated inputs agree, then the trunk runs with the pair tensor row-sharded: embedding
and MSA module replicated, the Pairformer stack through :class:`parallel.rowpair_fused.FusedRowPair`
on GPUs (plain sharded statements on CPU / gloo).  Rank 0 gathers the pair tensor for the heads and
writes the outputs; each rank prints its SCHEDULE and MEMSTATS lines.
Reference: common/opt_core/opt_core/mem/rowpair/trunk.py:1131, evidence.py:163,187.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

from ..core import det, report
from ..models import cofold
from . import launch, rowpair
from .ckpt import TrunkCheckpointer, feature_digest
from .layout import Layout

TAG = "rowpair"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="tiny")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--msa_depth", type=int, default=1)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--recycles", type=int, default=None)
    ap.add_argument("--out_dir", default=None)
    ap.add_argument("--gather", default="peer")
    ap.add_argument("--blocks", type=int, default=None, help="override the number of Pairformer blocks")
    ap.add_argument("--json", action="store_true", help="rank 0 prints one BIGMODE json line (device-timed)")
    ap.add_argument("--repeat", type=int, default=1, help="run the trunk this many times; the last run is the timed one")
    a = ap.parse_args(argv)
    comm = launch.init_from_env()
    cuda = comm.backend == "nccl"
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    dtype = torch.bfloat16 if cuda else torch.float32
    over = {} if a.blocks is None else {"pairformer_blocks": a.blocks}
    model = cofold.build_model(a.config, device=dev, dtype=dtype, seed=a.seed, **over)
    comm.check_replicated(next(model.parameters()).float(), "model weights")
    feats = cofold.synthetic_features(a.tokens, a.msa_depth, model.cfg, device=dev, dtype=dtype, seed=a.seed,
                                      chains=cofold.chains_for(a.config, a.tokens))
    comm.check_replicated(feats["token_feat"].float(), "features")
    N = a.tokens
    lay = Layout(N, comm.world, align=128 if cuda else 1)
    r0, r1 = lay.rows(comm.rank)
    report.emit(report.line(TAG, "SCHEDULE", ("rank", comm.rank), ("rows", f"{r0}:{r1}"), ("world", comm.world),
                            ("backend", comm.backend), ("gather", a.gather if cuda else "none")))
    fused = None
    if cuda:
        from .rowpair_fused import FusedRowPair
        from .symm import SymmHeap
        fused = FusedRowPair(lay, comm, SymmHeap(device=dev), gather=a.gather)      # symmetric buffers: once per process
    cold_ms = None
    for rep in range(max(1, a.repeat)):
        t0 = time.time()
        if cuda:
            torch.cuda.reset_peak_memory_stats(dev)
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            comm.barrier()
            ev0.record()
        with torch.no_grad():
            s_inputs, atom_c, atom_p = model.input_embedder(feats)
            s_init = model.s_init(s_inputs)
            z_init_loc = model.z_init_rows(feats, s_inputs, r0, r1)[0]          # only this rank's rows ever exist
            recycles = model.cfg.recycles if a.recycles is None else a.recycles
            ck = TrunkCheckpointer.from_env(comm.rank, comm.world, det.numerics_signature(det.Policy()))
            fd = feature_digest({k: v for k, v in feats.items() if isinstance(v, torch.Tensor)}) if ck else ""
            s = torch.zeros_like(s_init)
            z_loc = torch.zeros_like(z_init_loc)
            msa = model.msa_module
            for cyc in range(recycles + 1):
                s = s_init + model.s_recycle(model.s_norm(s))
                z_loc = z_init_loc + model.z_recycle(model.z_norm(z_loc))
                m = msa.msa_proj(feats["msa_feat"].to(dtype)) + msa.s_proj(s_inputs.to(dtype)).unsqueeze(1)
                for ml in msa.layers:
                    z_loc, m = rowpair.msa_layer_rows(ml, z_loc, m, feats["msa_mask"], lay, comm, comm.rank,
                                                      None if fused is None else fused.pair_block_)
                del m
                for bi, layer in enumerate(model.pairformer_module.layers):
                    if fused is not None:
                        z_loc = fused.pair_block_(layer, z_loc.contiguous())
                        s32 = s.float() + rowpair.apb_rows(s, z_loc, layer.attention, layer.pre_norm_s, lay, comm, comm.rank)
                        s = (s32 + layer.transition_s(s32.to(s.dtype)).float()).to(s.dtype)
                    else:
                        s, z_loc = rowpair.pairformer_layer_rows(layer, s, z_loc, lay, comm, comm.rank)
                if ck is not None:
                    ck.save(cyc, z_loc, (r0, r1), fd, {"s": s}, comm.barrier)
            # distogram on the local rows (z + z^T needs the transposed rows: one all-to-all)
            zt = rowpair.transpose_shard(z_loc.contiguous(), lay, comm)
            dist = model.distogram_module.distogram(z_loc + zt)
            dist_mean = comm.all_reduce_scalar(float(dist.float().sum()), "sum") / float(N * N * dist.shape[-1])
        if cuda and rep == 0 and a.repeat > 1:
            ev1.record()
            torch.cuda.synchronize()
            cold_ms = ev0.elapsed_time(ev1)
    ms = None
    if cuda:
        ev1.record()
        torch.cuda.synchronize()
        tms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
        import torch.distributed as tdist
        tdist.all_reduce(tms, op=tdist.ReduceOp.MAX)
        ms = float(tms.item())
        from ..ops import native
        native.raise_on_status(dev, "sharded trunk")
        peak = torch.cuda.max_memory_allocated(dev)
    else:
        peak = 0
    report.emit(report.line(TAG, "MEMSTATS", ("rank", comm.rank), ("peak_bytes", peak),
                            ("seconds", round(time.time() - t0, 3))))
    peaks = comm.all_gather(torch.tensor([float(peak)], device=dev))
    if a.json and comm.rank == 0:
        print("BIGMODE " + json.dumps({"n_gpus": comm.world, "tokens": N, "blocks": len(model.pairformer_module.layers),
                                       "msa_blocks": len(model.msa_module.layers), "trunk_passes": recycles + 1,
                                       "gather": a.gather if cuda else "none", "latency_ms_max_over_ranks": ms,
                                       "first_run_ms_rank0": cold_ms,
                                       "peak_gb_per_gpu_max": round(max(float(p.item()) for p in peaks) / 2 ** 30, 3),
                                       "mean_distogram_logit": dist_mean}), flush=True)
    if comm.rank == 0 and a.out_dir:
        os.makedirs(a.out_dir, exist_ok=True)
        torch.save({"s": s.float().cpu(), "distogram_logits_mean": dist_mean},
                   os.path.join(a.out_dir, "trunk.pt"))
        with open(os.path.join(a.out_dir, "sharding.json"), "w") as f:
            json.dump({"n_gpu": comm.world, "sharding": "rowpair", "bounds": lay.bounds()}, f)
    comm.barrier()
    return 0


if __name__ == "__main__":
    sys.exit(main())
