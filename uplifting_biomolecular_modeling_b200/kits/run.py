"""Run commands of the kits: build the family's model under the activation, run it, write outputs.

Cofolding kits (``pred``): features come from ``--input`` (a ``.pt`` / ``.json`` feature file) or are
synthetic of ``--tokens`` / ``--msa_depth``; ``--mode off`` runs the plain statements in this process
after proving the process clean (the reference runs stock in a clean subprocess:
boltz2/opt/boltz2_opt/stock_pred.py).  ``--n_gpu P`` hands the prediction to the row-sharded launcher.
"""
from __future__ import annotations

import json
import os
import sys
import time

from ..core import counters, report, stock_proof
from . import base


def _load_features(args, cfg, config_name):
    import torch
    from ..models import cofold
    if args.input and args.input.endswith(".pt") and os.path.exists(args.input):
        return torch.load(args.input, map_location="cpu")
    n = args.tokens or 128
    return cofold.synthetic_features(n, args.msa_depth or 16, cfg, seed=args.seed,
                                     chains=cofold.chains_for(config_name, n))


def run(spec, act: "base.Activation", args, allow_partial: bool) -> int:
    if spec.name in ("proteinmpnn", "esm_if1", "ef2inv"):
        return _run_design(spec, act, args, allow_partial)
    if spec.family in ("cofold", "design"):
        return _run_cofold(spec, act, args, allow_partial)
    if spec.family == "evo2":
        return _run_lm(spec, act, args, allow_partial, "evo2")
    return _run_lm(spec, act, args, allow_partial, spec.family)


def _run_cofold(spec, act, args, allow_partial) -> int:
    import torch
    from .. import api
    config = args.model_config or (spec.config if spec.family == "cofold" else "tiny")
    if config not in __import__("uplifting_biomolecular_modeling_b200.models.cofold", fromlist=["CONFIGS"]).CONFIGS:
        config = "af3"
    if act.mode == "off":
        proof = stock_proof.env_proof([spec.env], [], {k: v for k, v in os.environ.items() if k != spec.env}, {}, [])
        report.emit(stock_proof.proof_line(spec.tag, proof))
    if act.n_gpu > 1:
        from ..parallel import launch
        try:
            act.plan()
        except base.ActivationError:
            return report.EXIT_NOT_ACTIVE
        return launch.run_prediction_sharded(spec, act, args, config, allow_partial)
    device = "cuda:0" if torch.cuda.is_available() else "cpu"
    dtype = torch.bfloat16 if device != "cpu" else torch.float32
    overrides = {}
    if args.recycling_steps is not None:
        overrides["recycles"] = args.recycling_steps
    if args.sampling_steps is not None:
        overrides["sampling_steps"] = args.sampling_steps
    if args.diffusion_samples is not None:
        overrides["samples"] = args.diffusion_samples
    try:
        pred = api.Predictor(config, mode="off", device=device, dtype=dtype, seed=args.seed, **overrides)
        pred.mode = act.mode
        if args.checkpoint:
            from ..models import weights
            weights.load_checkpoint(pred.model, args.checkpoint)
        if getattr(args, "upstream_fix", None):
            from ..core import upstream_fix
            act.words = list(getattr(act, "words", [])) + upstream_fix.apply_all(
                pred.model, upstream_fix.parse(args.upstream_fix), spec.tag, spec.name)
        act.apply(pred)
        if act.mode in ("fast", "big") and device != "cpu" and os.environ.get("UBM_LOADCHECK", "1") != "0":
            from ..ops import loadcheck
            try:
                loadcheck.require(device, tag=spec.tag)
            except loadcheck.KernelsRefused:
                return report.EXIT_KERNELS_REFUSED
    except base.ActivationError:
        return report.EXIT_NOT_ACTIVE
    except api.NotActive as e:
        act.refuse(str(e))
        return report.EXIT_NOT_ACTIVE
    act.register_exit()
    feats = _load_features(args, pred.cfg, config)
    t0 = time.time()
    try:
        out = pred.predict(feats)
    except Exception as e:  # noqa: BLE001
        report.emit(report.line(spec.tag, "FAILED", ("error", type(e).__name__), ("detail", report.token(str(e))[:200])))
        return act.finish(report.EXIT_FAIL, allow_partial, args.out_dir)
    dt = time.time() - t0
    incomplete = None
    if args.out_dir:
        os.makedirs(args.out_dir, exist_ok=True)
        torch.save({k: v for k, v in out.items()}, os.path.join(args.out_dir, "prediction.pt"))
        with open(os.path.join(args.out_dir, "confidence.json"), "w") as f:
            json.dump({"plddt_mean": float(out["plddt"].mean()) if "plddt" in out else None,
                       "pae_mean": float(out["pae_mean"]) if "pae_mean" in out else None}, f)
        if not os.path.exists(os.path.join(args.out_dir, "prediction.pt")):
            incomplete = "prediction.pt missing"
    report.emit(report.line(spec.tag, "DONE", ("seconds", round(dt, 3)), ("tokens", feats["token_feat"].shape[1]),
                            ("samples", out["coords"].shape[0])))
    return act.finish(0, allow_partial, args.out_dir, incomplete)


def _run_design(spec, act, args, allow_partial) -> int:
    """``design`` verb of the sequence-design kits: inverse folding of a synthetic backbone (proteinmpnn, esm_if1) or
    sequence inversion through the structure trunk (ef2inv)."""
    import torch
    from ..models import cofold, design
    try:
        act.apply(None)
    except base.ActivationError:
        return report.EXIT_NOT_ACTIVE
    act.register_exit()
    n = args.tokens or 32
    t0 = time.time()
    if spec.name == "ef2inv":
        model = cofold.build_model("tiny", device="cpu", dtype=torch.float32, seed=args.seed)
        feats = cofold.synthetic_features(n, 4, model.cfg, seed=args.seed)
        g = torch.Generator().manual_seed(args.seed)
        target = torch.randint(0, model.cfg.distogram_bins, (1, n, n), generator=g)
        inv = design.SequenceInversion(model, feats, target, seed=args.seed)
        losses = [inv.step() for _ in range(4)]
        res = {"loss_first": round(losses[0], 4), "loss_last": round(losses[-1], 4), "tokens": n}
        seqs = inv.sequence()
    else:
        dec = design.build_decoder(seed=args.seed)
        x = torch.randn(1, n, 3, generator=torch.Generator().manual_seed(args.seed)) * 6.0
        k = args.diffusion_samples or 2
        seqs = dec.sample(x, seeds=[args.seed + i for i in range(k)])
        res = {"sequences": k, "tokens": n}
    letters = "ACDEFGHIKLMNPQRSTVWY"
    text = ["".join(letters[int(t)] for t in row.tolist()) for row in seqs]
    report.emit(report.line(spec.tag, "DONE", ("seconds", round(time.time() - t0, 3)), ("verb", args.verb),
                            *res.items(), ("first", text[0][:40])))
    if args.out_dir:
        os.makedirs(args.out_dir, exist_ok=True)
        with open(os.path.join(args.out_dir, "design.json"), "w") as f:
            json.dump(dict(res, sequences_text=text), f)
    return act.finish(0, allow_partial, args.out_dir)


def _run_lm(spec, act, args, allow_partial, family) -> int:
    import torch
    from ..models import lm
    device = "cuda:0" if torch.cuda.is_available() else "cpu"
    try:
        act.apply(None)
    except base.ActivationError:
        return report.EXIT_NOT_ACTIVE
    act.register_exit()
    model = lm.build(family, spec.config if args.model_config is None else args.model_config, device=device,
                     mode=act.mode, seed=args.seed, kit=spec.name, specdec=getattr(args, "specdec", 0))
    protein = family == "protein_lm" and spec.name != "gpnstar"
    prompt = args.prompt or ("MKTAYIAKQRQISFVKSHFSRQLEERLGLIEVQ" * 2 if protein else "ACGT" * 16)
    t0 = time.time()
    res = model.run(args.verb, prompt, max_new_tokens=args.max_new_tokens)
    report.emit(report.line(spec.tag, "DONE", ("seconds", round(time.time() - t0, 3)), ("verb", args.verb),
                            *[(k, v) for k, v in res.items() if isinstance(v, (int, float, str))]))
    if args.out_dir:
        os.makedirs(args.out_dir, exist_ok=True)
        with open(os.path.join(args.out_dir, f"{args.verb}.json"), "w") as f:
            json.dump({k: (v if isinstance(v, (int, float, str, list)) else str(v)) for k, v in res.items()}, f)
    return act.finish(0, allow_partial, args.out_dir)
