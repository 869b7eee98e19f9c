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


class InputError(ValueError):
    """``--input`` / ``--model_config`` / ``--checkpoint`` cannot be honoured as given (exit 2, never a substitute)."""


REQUIRED_FEATURES = ("token_feat", "token_mask", "residue_index", "chain_id", "token_bonds", "msa_feat", "msa_mask",
                     "ref_pos", "atom_to_token", "token_rep_atom")


def _load_features(args, cfg, config_name):
    """Features of one prediction: a ``.pt`` feature dict or a ``.json`` description of a synthetic complex
    (``{"tokens": N, "msa_depth": S, "chains": [[length, kind], ...], "seed": k}``); without ``--input`` a synthetic
    complex of ``--tokens`` / ``--msa_depth``.  A path that cannot be read, or a file of another kind, is an error:
    nothing is substituted for a named input."""
    import torch
    from ..models import cofold
    if args.input:
        if not os.path.exists(args.input):
            raise InputError(f"--input {args.input}: no such file")
        if args.input.endswith(".pt"):
            feats = torch.load(args.input, map_location="cpu", weights_only=True)
            missing = [k for k in REQUIRED_FEATURES if k not in feats]
            if missing:
                raise InputError(f"--input {args.input}: feature(s) {','.join(missing)} missing")
            return feats
        if args.input.endswith(".json"):
            with open(args.input) as f:
                spec = json.load(f)
            n = int(spec.get("tokens") or sum(int(c[0]) for c in spec.get("chains", [])) or 0)
            if n <= 0:
                raise InputError(f"--input {args.input}: gives neither tokens nor chains")
            chains = [(int(c[0]), str(c[1])) for c in spec["chains"]] if "chains" in spec else \
                cofold.chains_for(config_name, n)
            return cofold.synthetic_features(n, int(spec.get("msa_depth", args.msa_depth or 16)), cfg,
                                             seed=int(spec.get("seed", args.seed)), chains=chains)
        raise InputError(f"--input {args.input}: expected a .pt feature file or a .json complex description")
    n = args.tokens or 128
    return cofold.synthetic_features(n, args.msa_depth or 16, cfg, seed=args.seed,
                                     chains=cofold.chains_for(config_name, n))


def run(spec, act: "base.Activation", args, allow_partial: bool) -> int:
    if spec.name in ("proteinmpnn", "esm_if1", "ef2inv"):
        return _run_design(spec, act, args, allow_partial)
    if spec.family == "design":
        return _run_diffusion_design(spec, act, args, allow_partial)
    if spec.family == "cofold":
        return _run_cofold(spec, act, args, allow_partial)
    if spec.family == "evo2":
        return _run_lm(spec, act, args, allow_partial, "evo2")
    return _run_lm(spec, act, args, allow_partial, spec.family)


def _run_cofold(spec, act, args, allow_partial) -> int:
    import torch
    from .. import api
    from ..models import cofold as _cofold
    config = args.model_config or spec.config
    if config not in _cofold.CONFIGS:
        if args.model_config:
            report.emit(report.line(spec.tag, "USAGE", ("error", "unknown_model_config"), ("given", config),
                                    ("known", ",".join(sorted(_cofold.CONFIGS)))))
            return report.EXIT_USAGE
        config = "af3"          # kits of the AF3 family without a configuration of their own share this one
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
        if getattr(args, "det", 0):
            from ..core import det
            det.apply_switches(det.Recipe(seed=args.seed))       # seeds, deterministic algorithms, no TF32
        ckpt = args.checkpoint or _weights_file(args.weights)
        init_skipped = 0
        if ckpt and not allow_partial:
            # cold start (host.coldstart): a strict load overwrites every parameter, so the random initialisation is
            # skipped while the model is built; a checkpoint that misses a parameter is refused below by name, so
            # no unfilled tensor survives
            from ..host import coldstart
            with coldstart.no_init() as skipped:
                pred = api.Predictor(config, mode="off", device=device, dtype=dtype, seed=args.seed, **overrides)
            init_skipped = skipped.n
        else:
            pred = api.Predictor(config, mode="off", device=device, dtype=dtype, seed=args.seed, **overrides)
        pred.set_mode(act.mode)
        act.manifest_extra = {"numerics": pred.numerics, "det": int(getattr(args, "det", 0))}
        if ckpt:
            from ..models import mappers, weights
            try:
                # kits of another upstream translate its parameter names first (models/mappers.py)
                rep = weights.load_checkpoint(pred.model, ckpt, strict=not allow_partial,
                                              mapper=mappers.for_kit(spec.name))
            except (ValueError, OSError) as e:
                act.refuse(f"checkpoint {ckpt}: {e}")
                return report.EXIT_NOT_ACTIVE
            act.manifest_extra = dict(getattr(act, "manifest_extra", {}))
            act.manifest_extra["checkpoint"] = {"path": ckpt, "matched": rep.matched, "missing": rep.missing[:50],
                                                 "unexpected": rep.unexpected[:50],
                                                 "shape_mismatch": rep.shape_mismatch[:50]}
            report.emit(report.line(spec.tag, "WEIGHTS", ("path", ckpt), ("matched", rep.matched),
                                    ("missing", len(rep.missing)), ("unexpected", len(rep.unexpected)),
                                    ("shape_mismatch", len(rep.shape_mismatch)), ("init_skipped", init_skipped)))
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
    # Resident loop: the model is built and activated once; inputs (one file, a comma list, or every .pt / .json of
    # a directory) are featurised ahead on a helper thread, predicted on this thread, written behind on a writer
    # thread (reference: <kit>_opt/worker.py + prefetch.py + writer.py of the cofolding kits).
    from ..host import resident
    try:
        items = _input_items(args)
    except InputError as e:
        report.emit(report.line(spec.tag, "USAGE", ("error", "input"), ("detail", report.token(str(e))[:200])))
        return act.finish(report.EXIT_USAGE, allow_partial, None)
    multi = len(items) > 1
    done, errors = [], []

    # items that name the same input bytes (a complex listed twice, or under two names) are featurised once: keyed by
    # the file's sha256, never by its path or time stamp (host.memo)
    from ..host import memo as _memo
    feature_memo = _memo.Memo("features", max_items=8)

    def prepare(item):
        ns = type(args)(**dict(vars(args), input=item[1]))
        if item[1] is None or not os.path.isfile(item[1]):
            return item, _load_features(ns, pred.cfg, config)          # synthetic, or the error path names the input
        parts = {"file": _memo.file_digest(item[1]), "kind": os.path.splitext(item[1])[1], "config": config,
                 "msa_depth": args.msa_depth, "seed": args.seed}
        return item, dict(feature_memo.get_or_build(parts, lambda: _load_features(ns, pred.cfg, config)))

    def forward(prepared):
        item, feats = prepared
        t0 = time.time()
        out = pred.predict(feats)
        return {"out": out, "tokens": int(feats["token_feat"].shape[1]), "seconds": time.time() - t0}

    def write(pair):
        item, res = pair
        out = res["out"]
        if args.out_dir:
            d = os.path.join(args.out_dir, item[0]) if multi else args.out_dir
            os.makedirs(d, exist_ok=True)
            torch.save({k: v for k, v in out.items()}, os.path.join(d, "prediction.pt"))
            with open(os.path.join(d, "confidence.json"), "w") as f:
                json.dump({"plddt_mean": float(out["plddt"].mean()) if "plddt" in out else None,
                           "pae_mean": float(out["pae_mean"]) if "pae_mean" in out else None}, f)
            if getattr(pred, "stage_peaks", None):
                from ..mem import peak as _peak
                _peak.write(d, pred.stage_peaks)
        done.append(item[0])
        report.emit(report.line(spec.tag, "DONE", ("item", item[0]), ("seconds", round(res["seconds"], 3)),
                                ("tokens", res["tokens"]), ("samples", out["coords"].shape[0])))

    def on_error(item, e):
        errors.append((item[0], e))
        kind = "input" if isinstance(e, InputError) else type(e).__name__
        report.emit(report.line(spec.tag, "USAGE" if isinstance(e, InputError) else "FAILED", ("item", item[0]),
                                ("error", kind), ("detail", report.token(str(e))[:200])))

    stats = resident.run_resident(items, prepare, forward, write, workers=1, depth=2, on_error=on_error)
    if multi:
        report.emit(report.line(spec.tag, "RESIDENT", *stats.words().items(),
                                ("features_built", feature_memo.stats["build"]),
                                ("features_reused", feature_memo.stats["hit"])))
    if errors:
        bad_input = all(isinstance(e, InputError) for _, e in errors)
        return act.finish(report.EXIT_USAGE if bad_input else report.EXIT_FAIL, allow_partial, args.out_dir)
    incomplete = None
    if args.out_dir:
        first = os.path.join(args.out_dir, items[0][0]) if multi else args.out_dir
        if not os.path.exists(os.path.join(first, "prediction.pt")):
            incomplete = "prediction.pt missing"
    return act.finish(0, allow_partial, args.out_dir, incomplete)


def _input_items(args):
    """(name, path) pairs of a run: ``--input`` may name one file, several separated by commas, or a directory whose
    ``.pt`` / ``.json`` files are taken in sorted order; without ``--input`` one synthetic item."""
    if not args.input:
        return [("synthetic", None)]
    paths = []
    for part in str(args.input).split(","):
        part = part.strip()
        if os.path.isdir(part):
            found = sorted(f for f in os.listdir(part) if f.endswith((".pt", ".json")))
            if not found:
                raise InputError(f"--input {part}: directory holds no .pt / .json input")
            paths += [os.path.join(part, f) for f in found]
        elif part:
            paths.append(part)
    names, seen = [], {}
    for pth in paths:
        base = os.path.splitext(os.path.basename(pth))[0] or "input"
        seen[base] = seen.get(base, 0) + 1
        names.append(base if seen[base] == 1 else f"{base}_{seen[base]}")
    return list(zip(names, paths))


def _sequence_records(path):
    """``--input`` of the sequence kits: FASTA records (``>name`` lines) or one sequence per line -> [(name, sequence)];
    [] without a path.  A missing or empty file is an input error (exit 2), never a silent default prompt."""
    if not path:
        return []
    if not os.path.isfile(path):
        raise InputError(f"--input {path}: no such file")
    out, name, buf = [], None, []
    fasta = False
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            if line.startswith(">"):
                fasta = True
                if buf:
                    out.append((name or f"record{len(out)}", "".join(buf)))
                name, buf = line[1:].split()[0] if len(line) > 1 else None, []
            elif fasta:
                buf.append(line)
            else:
                out.append((f"line{len(out)}", line))
    if buf:
        out.append((name or f"record{len(out)}", "".join(buf)))
    if not out:
        raise InputError(f"--input {path}: holds no sequence")
    return out


def _weights_file(weights_dir):
    """``--weights D``: the one checkpoint file in D (``*.ckpt`` / ``*.pt`` / ``*.safetensors``); None without D.
    Several candidates are an error of the call, reported by the loader as an unreadable path."""
    if not weights_dir:
        return None
    if os.path.isfile(weights_dir):
        return weights_dir
    if not os.path.isdir(weights_dir):
        return weights_dir                      # the loader reports the missing path
    c = sorted(f for f in os.listdir(weights_dir) if f.endswith((".ckpt", ".pt", ".safetensors")))
    if len(c) == 1:
        return os.path.join(weights_dir, c[0])
    return None if not c else os.path.join(weights_dir, "<ambiguous:" + ",".join(c[:4]) + ">")


def _run_diffusion_design(spec, act, args, allow_partial) -> int:
    """``design`` verb of the diffusion design kits (BoltzGen, Complexa, PXDesign, Genie 3, RFdiffusion 1 / 3,
    Caliby, ColabDesign, mosaic): backbones of ``--diffusion_samples`` designs are sampled by the structure module
    on a target whose designed positions carry the unknown-residue token, then each backbone is given a sequence
    by the inverse-folding decoder.  One trunk pass and one set of step-invariant sampler tensors serve the whole
    design batch (``cond_dedup``); the sampler step replays from a CUDA graph under ``exact`` and above.
    Reference: the resident sampler-graph drivers of those kits (e.g. rfdiffusion1/opt/forward/se3fast_addon)."""
    import torch
    from .. import api
    from ..models import cofold, design
    device = "cuda:0" if torch.cuda.is_available() else "cpu"
    dtype = torch.bfloat16 if device != "cpu" else torch.float32
    config = args.model_config or spec.config
    if config not in cofold.CONFIGS:
        report.emit(report.line(spec.tag, "USAGE", ("error", "unknown_model_config"), ("given", config)))
        return report.EXIT_USAGE
    over = {}
    if args.sampling_steps is not None:
        over["sampling_steps"] = args.sampling_steps
    over["samples"] = args.diffusion_samples or 2
    try:
        pred = api.Predictor(config, mode="off", device=device, dtype=dtype, seed=args.seed, **over)
        pred.set_mode(act.mode)
        act.apply(pred)
    except base.ActivationError:
        return report.EXIT_NOT_ACTIVE
    except api.NotActive as e:
        act.refuse(str(e))
        return report.EXIT_NOT_ACTIVE
    act.register_exit()
    n = args.tokens or 48
    t0 = time.time()
    pipe = design.DesignPipeline(pred, seed=args.seed, dedup=bool(getattr(pred, "cond_dedup", False)))
    try:
        res = pipe.run(n_tokens=n, designs=over["samples"], designed_fraction=0.5)
    except Exception as e:  # noqa: BLE001
        report.emit(report.line(spec.tag, "FAILED", ("error", type(e).__name__), ("detail", report.token(str(e))[:200])))
        return act.finish(report.EXIT_FAIL, allow_partial, args.out_dir)
    report.emit(report.line(spec.tag, "DONE", ("seconds", round(time.time() - t0, 3)), ("verb", args.verb),
                            ("designs", len(res["sequences"])), ("tokens", n), ("trunk_passes", res["trunk_passes"]),
                            ("first", res["sequences"][0][:40])))
    if args.out_dir:
        os.makedirs(args.out_dir, exist_ok=True)
        torch.save({"coords": res["coords"]}, os.path.join(args.out_dir, "designs.pt"))
        with open(os.path.join(args.out_dir, "design.json"), "w") as f:
            json.dump({"sequences_text": res["sequences"], "tokens": n, "trunk_passes": res["trunk_passes"]}, f)
    return act.finish(0, allow_partial, args.out_dir)


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


def _run_lm_sharded(spec, act, args, allow_partial) -> int:
    """``--n_gpu P`` of the StripedHyena-2 kit: P ranks of ``parallel.lm_worker`` (tensor parallelism); the parent
    prints ACTIVE, the result of rank 0 and EXIT."""
    import tempfile
    from ..parallel import launch
    try:
        act.levers_on = act.plan()
    except base.ActivationError:
        return report.EXIT_NOT_ACTIVE
    ckpt = getattr(args, "checkpoint", None) or _weights_file(getattr(args, "weights", None))
    if ckpt:
        # held against the model's names and shapes here (meta device, nothing is allocated), so that a checkpoint
        # that does not fit is NOT ACTIVE with exit 3 before any rank starts
        import torch
        from ..models import evo2 as _evo2, weights
        cfg = args.model_config or spec.config
        try:
            with torch.device("meta"):
                probe = _evo2.StripedHyena2(_evo2.CONFIGS[cfg if cfg in _evo2.CONFIGS else "evo2_tiny"])
            rep = weights.load_checkpoint(probe, ckpt, strict=not allow_partial, dry_run=True)
        except (ValueError, OSError) as e:
            act.refuse(f"checkpoint {ckpt}: {e}")
            return report.EXIT_NOT_ACTIVE
        report.emit(report.line(spec.tag, "WEIGHTS", ("path", ckpt), ("matched", rep.matched),
                                ("missing", len(rep.missing)), ("unexpected", len(rep.unexpected)),
                                ("shape_mismatch", len(rep.shape_mismatch)), ("init_skipped", 0)))
    report.emit(report.with_words(report.line(spec.tag, "ACTIVE", ("mode", act.mode), ("levers", act.levers_on),
                                              ("source", act.source), ("n_gpu", act.n_gpu),
                                              ("sharding", "tensor_parallel")), act.words))
    act.register_exit()
    out = os.path.join(args.out_dir or tempfile.mkdtemp(prefix="ubm_lm_"), f"{args.verb}.json")
    os.makedirs(os.path.dirname(out), exist_ok=True)
    wargs = ["--config", args.model_config or spec.config, "--verb", args.verb, "--seed", str(args.seed),
             "--max_new_tokens", str(args.max_new_tokens), "--out", out,
             "--fp8", "1" if "fp8_input_proj" in act.levers_on else "0"]
    for flag, val in (("--prompt", args.prompt), ("--input", getattr(args, "input", None)), ("--checkpoint", ckpt)):
        if val:
            wargs += [flag, str(val)]
    if allow_partial:
        wargs += ["--allow-partial"]
    import torch
    t0 = time.time()
    try:
        launch.run_sharded(act.n_gpu, "uplifting_biomolecular_modeling_b200.parallel.lm_worker", wargs,
                           cpu_ok=not torch.cuda.is_available(), backend=None if torch.cuda.is_available() else "gloo",
                           echo_rank0=False)
    except launch.RankFailed as e:
        report.emit(report.line(spec.tag, "FAILED", ("rank", e.rank), ("rc", e.rc)))
        sys.stderr.write(e.tail)
        return act.finish(report.EXIT_FAIL, allow_partial, args.out_dir)
    res = json.load(open(out))
    report.emit(report.line(spec.tag, "DONE", ("seconds", round(time.time() - t0, 3)), ("verb", args.verb),
                            *[(k, v) for k, v in res.items() if isinstance(v, (int, float, str))]))
    return act.finish(0, allow_partial, args.out_dir)


def _run_lm(spec, act, args, allow_partial, family) -> int:
    import torch
    from ..models import lm
    if act.n_gpu > 1:
        return _run_lm_sharded(spec, act, args, allow_partial)
    device = "cuda:0" if torch.cuda.is_available() else "cpu"
    # the model is built on its plain statements; the mode's levers then switch the kernel path, the decode graph
    # and the tensor-parallel form on, each reporting what it did
    model = lm.build(family, spec.config if args.model_config is None else args.model_config, device=device,
                     mode="off", seed=args.seed, kit=spec.name, specdec=getattr(args, "specdec", 0))
    model.mode = act.mode
    ckpt = getattr(args, "checkpoint", None) or _weights_file(getattr(args, "weights", None))
    if ckpt:
        # loaded before the levers run, so that packed / quantised weights are made from the loaded parameters; a
        # checkpoint that does not fit ends the run by name (no run on partly random weights unless asked for)
        from ..models import weights
        try:
            rep = weights.load_checkpoint(model.model, ckpt, strict=not allow_partial)
        except (ValueError, OSError) as e:
            act.refuse(f"checkpoint {ckpt}: {e}")
            return report.EXIT_NOT_ACTIVE
        act.manifest_extra = dict(getattr(act, "manifest_extra", {}) or {})
        act.manifest_extra["checkpoint"] = {"path": ckpt, "matched": rep.matched, "missing": rep.missing[:50],
                                             "unexpected": rep.unexpected[:50],
                                             "shape_mismatch": rep.shape_mismatch[:50]}
        report.emit(report.line(spec.tag, "WEIGHTS", ("path", ckpt), ("matched", rep.matched),
                                ("missing", len(rep.missing)), ("unexpected", len(rep.unexpected)),
                                ("shape_mismatch", len(rep.shape_mismatch)), ("init_skipped", 0)))
    try:
        act.apply(model)
    except base.ActivationError:
        return report.EXIT_NOT_ACTIVE
    act.register_exit()
    protein = family == "protein_lm" and spec.name != "gpnstar"
    try:
        records = _sequence_records(getattr(args, "input", None))
    except InputError as e:
        report.emit(report.line(spec.tag, "USAGE", ("error", "input"), ("detail", report.token(str(e))[:200])))
        return act.finish(report.EXIT_USAGE, allow_partial, None)
    prompt = args.prompt or ("MKTAYIAKQRQISFVKSHFSRQLEERLGLIEVQ" * 2 if protein else "ACGT" * 16)
    t0 = time.time()
    if records:
        # --input: a FASTA (or one sequence per line) file; every record is run, the first one's result leads
        per = [dict(model.run(args.verb, seq, max_new_tokens=args.max_new_tokens), id=name) for name, seq in records]
        res = dict(per[0], records=len(per))
        if len(per) > 1 and all("score" in r for r in per):
            res["mean_score"] = sum(r["score"] for r in per) / len(per)
        res["per_record"] = [{k: v for k, v in r.items() if isinstance(v, (int, float, str))} for r in per]
    else:
        res = model.run(args.verb, prompt, max_new_tokens=args.max_new_tokens)
    report.emit(report.line(spec.tag, "DONE", ("seconds", round(time.time() - t0, 3)), ("verb", args.verb),
                            *[(k, v) for k, v in res.items() if isinstance(v, (int, float, str))]))
    if args.out_dir:
        os.makedirs(args.out_dir, exist_ok=True)
        tracks = getattr(model, "last_tracks", None)
        if tracks is not None:
            # genomic-track kits: the first predicted track of the window as a bedGraph, written on the writer
            # thread (host.tracks); the window of a synthetic prompt is named for what it is
            from ..host import tracks as _tracks
            tw = _tracks.TrackWriter(args.out_dir, bin_size=int(model.last_bin_size), columns=(0,))
            tw.submit("synthetic_window", 0, tracks)
            res["bedgraph_records"] = tw.close()
        with open(os.path.join(args.out_dir, f"{args.verb}.json"), "w") as f:
            json.dump({k: (v if isinstance(v, (int, float, str, list)) else str(v)) for k, v in res.items()}, f)
    return act.finish(0, allow_partial, args.out_dir)
