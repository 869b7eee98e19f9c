"""Rank worker of a row-sharded prediction (``pred --mode big --n_gpu P``).

Every rank builds the same model (same seed, same checkpoint), rank 0 reads or builds the features and
broadcasts them, all ranks check that replicated inputs agree, then the trunk runs with the pair tensor
row-sharded: embedding and MSA representation replicated, the Pairformer stack through
:class:`parallel.rowpair_fused.FusedRowPair` on GPUs (plain sharded statements on CPU / gloo), transitions of
the MSA and single tracks on the kernel path.  With ``--structure 1`` the row shards are then sent to rank 0,
which runs the diffusion sampler and the confidence head on the whole pair tensor (the kernel path and the
sampler graph of a single-GPU prediction) and writes coordinates; the other ranks hold no copy of the whole
tensor.  Each rank prints its SCHEDULE and MEMSTATS lines.
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
    ap.add_argument("--structure", type=int, default=0, help="1 = sampler and confidence head on rank 0 after the trunk")
    ap.add_argument("--input", default=None, help="feature file (.pt) or complex description (.json), read by rank 0")
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--kit", default="", help="kit name: selects the checkpoint name mapper of its upstream, if any")
    ap.add_argument("--allow-partial", action="store_true")
    ap.add_argument("--sampling_steps", type=int, default=None)
    ap.add_argument("--diffusion_samples", type=int, default=None)
    a = ap.parse_args(argv)
    comm = launch.init_from_env()
    cuda = comm.backend == "nccl"
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    dtype = torch.bfloat16 if cuda else torch.float32
    over = {} if a.blocks is None else {"pairformer_blocks": a.blocks}
    model = cofold.build_model(a.config, device=dev, dtype=dtype, seed=a.seed, **over)
    if a.checkpoint:
        from ..models import weights
        from ..models import mappers
        rep = weights.load_checkpoint(model, a.checkpoint, strict=not a.allow_partial, mapper=mappers.for_kit(a.kit))
        report.emit(report.line(TAG, "WEIGHTS", ("rank", comm.rank), ("matched", rep.matched),
                                ("missing", len(rep.missing)), ("unexpected", len(rep.unexpected))))
    comm.check_replicated(next(model.parameters()).float(), "model weights")
    if a.input:
        # rank 0 reads the file; the tensors travel as coalesced byte chunks, the table through the host store
        feats0 = None
        if comm.rank == 0:
            from ..kits import run as kit_run
            ns = argparse.Namespace(input=a.input, tokens=a.tokens, msa_depth=a.msa_depth, seed=a.seed)
            feats0 = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v)
                      for k, v in kit_run._load_features(ns, model.cfg, a.config).items()}
        feats = rowpair.broadcast_features(feats0 or {}, comm, 0, device=dev)
        feats = {k: (v.to(dtype) if isinstance(v, torch.Tensor) and v.is_floating_point() else v)
                 for k, v in feats.items()}
    else:
        feats = cofold.synthetic_features(a.tokens, a.msa_depth, model.cfg, device=dev, dtype=dtype, seed=a.seed,
                                          chains=cofold.chains_for(a.config, a.tokens))
    comm.check_replicated(feats["token_feat"].float(), "features")
    N = int(feats["token_feat"].shape[1])
    if cuda:
        # transitions of the MSA and single tracks (and, on rank 0, the sampler and the confidence head) on the
        # kernel path; the pair stack of the trunk goes through FusedRowPair below
        from ..models import pairformer as _pf
        _pf.set_impl(model, "fused", kinds=(_pf.Transition,), workspace=model.workspace)
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
        recycles = model.cfg.recycles if a.recycles is None else a.recycles
        s, z_loc, s_inputs, atom_c, atom_p, dist_mean = sharded_trunk(model, feats, comm, lay, fused, recycles, dtype)
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
    # one census point of the per-rank model peak = a(N) + b(N) / P (fitted over runs at several P by mem.peak.fit_a_b)
    from ..mem import peak as _peak
    sys.stderr.write(_peak.census_line(TAG, "trunk", comm.rank, int(peak), N, comm.world) + "\n")
    peaks = comm.all_gather(torch.tensor([float(peak)], device=dev))
    if a.json and comm.rank == 0:
        print("BIGMODE " + json.dumps({"n_gpus": comm.world, "tokens": N, "blocks": len(model.pairformer_module.layers),
                                       "msa_blocks": len(model.msa_module.layers), "trunk_passes": recycles + 1,
                                       "gather": a.gather if cuda else "none", "latency_ms_max_over_ranks": ms,
                                       "first_run_ms_rank0": cold_ms,
                                       "peak_gb_per_gpu_max": round(max(float(p.item()) for p in peaks) / 2 ** 30, 3),
                                       "mean_distogram_logit": dist_mean}), flush=True)
    structure = None
    if a.structure:
        structure = _structure_on_rank0(a, comm, model, feats, s, z_loc, lay, dev, cuda, s_inputs, atom_c, atom_p)
    if comm.rank == 0 and a.out_dir:
        os.makedirs(a.out_dir, exist_ok=True)
        torch.save({"s": s.float().cpu(), "distogram_logits_mean": dist_mean},
                   os.path.join(a.out_dir, "trunk.pt"))
        if structure is not None:
            torch.save(structure, os.path.join(a.out_dir, "prediction.pt"))
            with open(os.path.join(a.out_dir, "confidence.json"), "w") as f:
                json.dump({"plddt_mean": float(structure["plddt"].mean()) if "plddt" in structure else None,
                           "pae_mean": float(structure["pae_mean"]) if "pae_mean" in structure else None}, f)
        with open(os.path.join(a.out_dir, "sharding.json"), "w") as f:
            json.dump({"n_gpu": comm.world, "sharding": "rowpair", "bounds": lay.bounds()}, f)
    comm.barrier()
    return 0


@torch.no_grad()
def sharded_trunk(model, feats, comm, lay: Layout, fused, recycles: int, dtype, checkpoint: bool = True):
    """Embedding, recycling loop, MSA module and Pairformer stack with the pair tensor row-sharded over the ranks of
    ``comm`` (rows of this rank only ever exist here), then the mean distogram logit as a checksum all ranks agree
    on.  ``fused``: a :class:`parallel.rowpair_fused.FusedRowPair` (GPU kernel path) or None (plain sharded
    statements).  Returns (s, z_loc, s_inputs, atom_c, atom_p, mean distogram logit)."""
    r0, r1 = lay.rows(comm.rank)
    N = lay.n
    s_inputs, atom_c, atom_p = model.input_embedder(feats)
    s_init = model.s_init(s_inputs)
    z_init_loc = model.z_init_rows(feats, s_inputs, r0, r1)[0]          # only this rank's rows ever exist
    ck = TrunkCheckpointer.from_env(comm.rank, comm.world, det.numerics_signature(det.Policy())) if checkpoint else None
    fd = feature_digest({k: v for k, v in feats.items() if isinstance(v, torch.Tensor)}) if ck else ""
    s = torch.zeros_like(s_init)
    z_loc = torch.zeros_like(z_init_loc)
    first_cycle = 0
    if ck is not None and os.environ.get("ROWPAIR_RESUME") == "1":
        step = ck.latest()
        if step is not None:
            # resume after the last complete cycle: refused by name when features, layout, dtype or numerics differ
            z_loc, repl, rng = ck.load(step, fd, (r0, r1), z_loc.dtype, device=z_loc.device)
            s = repl["s"].to(s.dtype)
            ck.restore_rng(rng)
            first_cycle = step + 1
            report.emit(report.line(TAG, "RESUME", ("rank", comm.rank), ("from_cycle", step)))
    msa = model.msa_module
    for cyc in range(first_cycle, recycles + 1):
        s = s_init + model.s_recycle(model.s_norm(s))
        z_loc = z_init_loc + model.z_recycle(model.z_norm(z_loc))
        m = msa.msa_proj(feats["msa_feat"].to(dtype)) + msa.s_proj(s_inputs.to(dtype)).unsqueeze(1)
        for ml in msa.layers:
            z_loc, m = rowpair.msa_layer_rows(ml, z_loc, m, feats["msa_mask"], lay, comm, comm.rank,
                                              None if fused is None else fused.pair_block_)
        del m
        for layer in model.pairformer_module.layers:
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
    return s, z_loc, s_inputs, atom_c, atom_p, dist_mean


def _structure_on_rank0(a, comm, model, feats, s, z_loc, lay, dev, cuda, s_inputs, atom_c, atom_p):
    """Send the row shards to rank 0 (point to point, straight into their rows of the whole tensor) and run the
    sampler and the confidence head there.  Returns the host result on rank 0, None elsewhere."""
    N = lay.n
    z = None
    if comm.world == 1:
        z = z_loc
    else:
        import torch.distributed as tdist
        if comm.rank == 0:
            z = torch.empty((N, N, z_loc.shape[-1]), dtype=z_loc.dtype, device=dev)
            r0, r1 = lay.rows(0)
            z[r0:r1].copy_(z_loc)
            for q in range(1, comm.world):
                q0, q1 = lay.rows(q)
                if q1 > q0:
                    tdist.recv(z[q0:q1], src=q)
        elif z_loc.shape[0] > 0:
            tdist.send(z_loc.contiguous(), dst=0)
    out = None
    if comm.rank == 0:
        from .. import api
        t0 = time.time()
        pred = api.Predictor(a.config, mode="off", device=str(dev), dtype=z.dtype, seed=a.seed, model=model,
                             use_graphs=cuda)
        if cuda:
            pred.set_mode("big")
            model.set_impl("fused")
        res = pred.structure_and_confidence(feats, s, z.unsqueeze(0), s_inputs, atom_c, atom_p,
                                            a.diffusion_samples, a.sampling_steps, True, a.seed)
        out = {k: v.float().cpu() for k, v in res.items()}
        report.emit(report.line(TAG, "STRUCTURE", ("rank", 0), ("samples", out["coords"].shape[0]),
                                ("atoms", out["coords"].shape[1]), ("seconds", round(time.time() - t0, 3))))
    comm.barrier()
    return out


if __name__ == "__main__":
    sys.exit(main())
