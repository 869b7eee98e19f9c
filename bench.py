"""Headline benchmark: AF3 / Chai-1-shaped cofolding at N = 1536 tokens, fast mode.

``python bench.py --gpus N --steps K --warmup W`` runs one independent prediction per GPU per step
(weak scaling: per-GPU work is fixed) and reports predictions/hour over all GPUs.  A step is one
whole prediction: feature copy host->device, input embedding, MSA module + 48 Pairformer blocks per
trunk pass, 5 samples x 200 sampler steps, confidence head, result copy device->host.  Weights are
random-init, features synthetic (3 x 448-residue proteins, 2 x 48-nt DNA, a 48-atom ligand, MSA depth
1024).  Timing: CUDA events on the launching stream, barrier + synchronize on both sides, max over
ranks.  The working set of a step (pair tensor 604 MB, pair-bias planes 1.8 GB, MSA) is far larger
than the 126 MB L2, so no explicit flush is needed between timed steps.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIG = {"model": "af3-shaped cofold (48 Pairformer blocks, 4 MSA blocks, 24-block DiT, 5x200 sampling)",
          "tokens": 1536, "msa_depth": 1024, "mode": "fast", "l2": "inputs larger than L2"}


def clock_sampler(stop, samples, gpu_index):
    q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    while not stop.is_set():
        try:
            out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i",
                                  str(gpu_index)], capture_output=True, text=True, timeout=5).stdout.strip()
            if out:
                samples.append([x.strip() for x in out.split(",")])
        except Exception:
            pass
        stop.wait(0.5)


def summarize_clocks(samples):
    if not samples:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
    sm = sorted(int(s[0]) for s in samples if s[0].isdigit())
    mx = max(int(s[1]) for s in samples if s[1].isdigit()) if samples else None
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    reasons = [n for i, n in enumerate(names) if any(len(s) > 2 + i and s[2 + i].startswith("Active") for s in samples)]
    return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": reasons}


def reference_arm(args):
    """The reference's own public path for this metric is a kit's ``pred`` verb (``boltz predict`` patched in
    memory by ``boltz2_opt``).  It is tried as it stands: the stock package ships in the reference as a pure-Python
    wheel and is installed without dependencies under ``baseline/_ref``; whatever import stops it is named in the
    ``unavailable`` line.  Nothing of this repository's models, kernels or engine is put in its place.  As context
    (never as the headline), the stock trunk modules that do import - ``PairformerModule`` and ``MSAModule``, the
    Pairformer part of the same N = 1536 workload - are timed unmodified and reported under ``stock_trunk``."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    line = {"impl": "reference"}
    if not os.path.isdir(os.path.join(ref, "boltz")):
        line["unavailable"] = ("baseline/_ref holds no stock model package: install the wheel the reference ships "
                               "(boltz2/stock/boltz-2.2.1-py3-none-any.whl) with pip --no-deps --target baseline/_ref")
        print(json.dumps(line))
        return 0
    sys.path.insert(0, ref)
    failing = []
    for mod in ("boltz.main", "boltz.model.models.boltz2", "boltz.model.modules.diffusionv2"):
        try:
            __import__(mod)
        except Exception as e:  # noqa: BLE001 - the reason is the answer
            failing.append(f"{mod}: {type(e).__name__}: {e}")
    if not failing:
        failing.append("imports succeed but `boltz predict` needs its checkpoint and CCD downloads (no network)")
    line["unavailable"] = ("the stock prediction path does not import here: " + "; ".join(failing) +
                           " (none of pytorch_lightning, einx, rdkit, cuequivariance is in the offline wheelhouse)")
    try:
        import torch
        if torch.cuda.is_available() and os.environ.get("UBM_BENCH_STOCK_TRUNK", "1") != "0":
            sys.path.insert(0, os.path.join(ROOT, "benchmarks"))
            import trunk_vs_reference as tvr
            ok, why = tvr.stock_available()
            if ok:
                blocks = 48
                res = tvr.measure(args.tokens, blocks, 4, args.msa_depth, rounds=1, ours=False,
                                  log=lambda *_: None)
                passes = (3 if args.recycles is None else args.recycles) + 1
                line["stock_trunk"] = {
                    "what": "unmodified stock boltz-2.2.1 PairformerModule(v2, 48 blocks) and MSAModule(4 blocks), "
                            "eval, bf16 autocast, use_kernels=False, random-init, one pass each; not the headline metric",
                    "tokens": args.tokens, "msa_depth": args.msa_depth,
                    "pairformer_ms_per_pass": res["pairformer"]["stock_ms"],
                    "msa_module_ms_per_pass": res["msa_module"]["stock_ms"],
                    "trunk_ms_for_passes": round(passes * (res["pairformer"]["stock_ms"] + res["msa_module"]["stock_ms"]), 1),
                    "trunk_passes": passes}
            else:
                line["stock_trunk"] = {"unavailable": why}
    except Exception as e:  # noqa: BLE001 - context only; the unavailable line stands
        line["stock_trunk"] = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
    print(json.dumps(line))
    return 0


def big_mode(args, world, rank, dev):
    """BASELINE's second metric: one N = 4096 prediction trunk (48 Pairformer blocks, single-sequence MSA, one pass)
    with the pair tensor held by the run's P GPUs - latency (device-timed, max over ranks, second run) and peak GB
    per GPU.  P = 1: the single-GPU ``big`` mode (row-blocked kernel path).  P > 1: row-sharded over the ranks, once
    with the gathers fused into the kernels (``peer``) and once with NCCL gathers (``nccl``)."""
    import torch
    import torch.distributed as dist
    from uplifting_biomolecular_modeling_b200.models import cofold
    N = int(os.environ.get("UBM_BENCH_BIG_TOKENS", "4096"))
    out = {"tokens": N, "config": "big4096: 8 chains x 512 residues, single-sequence MSA, 48 Pairformer blocks, 1 pass",
           "n_gpus": world}
    torch.cuda.empty_cache()
    if world == 1:
        from uplifting_biomolecular_modeling_b200 import api
        pred = api.Predictor("big4096", mode="big", device=str(dev), dtype=torch.bfloat16, seed=0)
        feats = pred.to_device(cofold.synthetic_features(N, 1, pred.cfg, seed=0, chains=cofold.chains_for("big4096", N)))
        ms = None
        for rep in range(2):
            torch.cuda.reset_peak_memory_stats(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            with torch.no_grad():
                s_inputs, s_init, z_init, _, _ = pred.model.embed(feats)
                s, z = pred.model.trunk(feats, s_inputs, s_init, z_init, 0)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            del s, z, z_init
        out["single_gpu_big"] = {"latency_ms": round(ms, 1), "row_block": pred.row_block,
                                 "peak_gb": round(torch.cuda.max_memory_allocated(dev) / 2 ** 30, 2)}
        return out
    from uplifting_biomolecular_modeling_b200.parallel import comm as C
    from uplifting_biomolecular_modeling_b200.parallel import worker
    from uplifting_biomolecular_modeling_b200.parallel.layout import Layout
    from uplifting_biomolecular_modeling_b200.parallel.rowpair_fused import FusedRowPair
    from uplifting_biomolecular_modeling_b200.parallel.symm import SymmHeap
    from uplifting_biomolecular_modeling_b200.models import pairformer as pf
    from uplifting_biomolecular_modeling_b200.ops import native
    comm = C.GroupComm()
    model = cofold.build_model("big4096", device=dev, dtype=torch.bfloat16, seed=0)
    pf.set_impl(model, "fused", kinds=(pf.Transition,), workspace=model.workspace)
    feats = cofold.synthetic_features(N, 1, model.cfg, device=dev, dtype=torch.bfloat16, seed=0,
                                      chains=cofold.chains_for("big4096", N))
    lay = Layout(N, world, align=128)
    heap = SymmHeap(device=dev)
    for gather in ("peer", "nccl"):
        fused = FusedRowPair(lay, comm, heap, gather=gather)
        ms = None
        for rep in range(2):
            torch.cuda.reset_peak_memory_stats(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.barrier()
            torch.cuda.synchronize()
            e0.record()
            worker.sharded_trunk(model, feats, comm, lay, fused, 0, torch.bfloat16, checkpoint=False)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
        native.raise_on_status(dev, "big mode")
        t = torch.tensor([ms, torch.cuda.max_memory_allocated(dev) / 2 ** 30], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[f"rowpair_{gather}"] = {"latency_ms_max_over_ranks": round(float(t[0]), 1),
                                    "peak_gb_per_gpu_max": round(float(t[1]), 2)}
        del fused
        torch.cuda.empty_cache()
    return out


def second_metric_then_line(line: dict, measure, rank: int, limit_s: float, key: str = "big_mode",
                            leave=os._exit):
    """Run the optional second measurement and print the benchmark's one JSON line (rank 0) exactly once.

    The second measurement may not cost the line: an exception is recorded in its place, and a rank that is still
    inside it after ``limit_s`` (a peer that never arrives at a collective) prints the line with the time-out
    recorded and leaves the process through ``leave(0)``.  Returns what was recorded under ``key``."""
    once = threading.Lock()

    def emit(value) -> None:
        if not once.acquire(blocking=False):
            return
        if rank == 0:
            line[key] = value
            print(json.dumps(line), flush=True)

    if measure is None:
        emit(None)
        return None

    def give_up():
        emit({"error": f"the measurement was still running after {limit_s:.0f} s; abandoned"})
        leave(0)
    timer = threading.Timer(limit_s, give_up)
    timer.daemon = True
    timer.start()
    try:
        value = measure()
    except Exception as e:  # noqa: BLE001 - the headline line must still be printed
        value = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
    timer.cancel()
    emit(value)
    return value


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="fast")
    ap.add_argument("--tokens", type=int, default=1536)
    ap.add_argument("--msa-depth", type=int, default=1024)
    ap.add_argument("--config", default="af3")
    ap.add_argument("--sampling-steps", type=int, default=None)
    ap.add_argument("--recycles", type=int, default=None)
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist
    from uplifting_biomolecular_modeling_b200 import api
    from uplifting_biomolecular_modeling_b200.models import cofold
    from uplifting_biomolecular_modeling_b200.ops import native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")      # the package's kernels use plain peer loads and stores
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=600))

    pred = api.Predictor(args.config, mode=args.mode, device=str(dev), dtype=torch.bfloat16, seed=rank)
    chains = cofold.chains_for(args.config, args.tokens)
    feats = cofold.synthetic_features(args.tokens, args.msa_depth, pred.cfg, seed=rank, chains=chains)
    feats = {k: v.pin_memory() for k, v in feats.items()}
    kw = dict(steps=args.sampling_steps, recycles=args.recycles)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        pred.predict(feats, **kw)
    barrier()
    samples, stop = [], threading.Event()
    th = threading.Thread(target=clock_sampler, args=(stop, samples, local), daemon=True)
    th.start()
    # (1) device-timed value: K predictions with the features resident on the device and the result left there
    feats_dev = pred.to_device(feats)
    pred.predict(feats_dev, to_host=False, **kw)
    native.reset_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        out = pred.predict(feats_dev, to_host=False, **kw)
    e1.record()
    barrier()
    launches = native.launch_count() // max(args.steps, 1)
    # (2) end to end through the public call: every step copies the features in from pinned host memory and the
    # result out
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    f0.record()
    for _ in range(args.steps):
        out = pred.predict(feats, **kw)
    f1.record()
    barrier()
    stop.set()
    th.join(timeout=2)
    t = torch.tensor([e0.elapsed_time(e1) / args.steps, f0.elapsed_time(f1) / args.steps], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = (float(v) for v in t.tolist())
    value = world * 3600.0 * 1000.0 / ms
    value_e2e = world * 3600.0 * 1000.0 / ms_e2e
    finite = bool(torch.isfinite(out["coords"]).all())
    ledgers = {}
    try:
        from uplifting_biomolecular_modeling_b200.core import counters
        ledgers = {k: {"served": v["served"], "fallback": v["fallback"], **({"fallback_by": v["fallback_by"]}
                                                                                if v["fallback"] else {})}
                   for k, v in counters.BOOK.stats().items()}
    except Exception:  # noqa: BLE001
        pass
    cfg, h2d_bytes, d2h_bytes = pred.cfg, pred.h2d_bytes, pred.d2h_bytes
    c = cfg
    shape = "AF3-shaped" if args.config == "af3" else f"{args.config}-shaped"
    model = (f"{shape} cofold ({c.pairformer_blocks} Pairformer blocks, {c.msa_blocks} MSA blocks, "
             f"{c.token_depth}-block DiT, {c.samples}x{args.sampling_steps or c.sampling_steps} sampling)")
    line = {"metric": f"predictions/hour at N={args.tokens} ({shape} cofold, {args.mode} mode)",
            "value": round(value, 3),
            "unit": "predictions/hour", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms, 3), "sec_per_prediction": round(ms / 1000.0, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic features, random-init weights", "impl": "ours",
            "config": dict(CONFIG, model=model, tokens=args.tokens, msa_depth=args.msa_depth, mode=args.mode,
                           global_batch=world, seq_len=args.tokens, parallelism=f"dp{world}",
                           sampling_steps=args.sampling_steps or cfg.sampling_steps,
                           samples=cfg.samples, trunk_passes=(cfg.recycles if args.recycles is None
                                                                   else args.recycles) + 1),
            "clocks": summarize_clocks(samples),
            "e2e": {"value": round(value_e2e, 3), "unit": "predictions/hour", "ms_per_step": round(ms_e2e, 3),
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                    "note": "Predictor.predict(host features): pinned-host feature copy in, coordinates / "
                            "confidence copy out, every step; `value` is the same call on device-resident "
                            "features with the result left on the device"},
            "gpu_launches": launches, "finite_output": finite, "kernel_ledgers": ledgers, "big_mode": None}
    big = None
    if os.environ.get("UBM_BENCH_BIG", "1") != "0" and args.tokens == 1536:
        # the second metric of the baseline (big-mode latency and peak memory at this run's P); measured after the
        # headline regions, never inside them
        del pred, feats_dev, out
        big = second_metric_then_line(line, lambda: big_mode(args, world, rank, dev), rank,
                                      float(os.environ.get("UBM_BENCH_BIG_LIMIT_S", "420")))
    else:
        second_metric_then_line(line, None, rank, 0.0)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
