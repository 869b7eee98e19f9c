"""Kit surface on CPU: run.sh verbs, mode resolution, refusals with exit 3, LEVER lines, manifest."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

from uplifting_biomolecular_modeling_b200.core import gates, report
from uplifting_biomolecular_modeling_b200.kits import base, registry


def _b200(n=8):
    return lambda: [{"index": i, "name": "NVIDIA B200", "cc": "10.0", "sm": "sm100", "mem_mib": 183359}
                    for i in range(n)]


def test_registry_covers_the_reference_kits():
    assert len(registry.REGISTRY) == 36
    for k in ("boltz2", "protenix_v2", "openfold3", "af3_jax", "chai1", "evo2", "esmc", "enformer_deepmind",
              "chrombpnet", "proteinmpnn", "rfdiffusion3", "ef2inv"):
        assert k in registry.REGISTRY
    assert registry.get("boltz2").env == "BOLTZ2_OPT" and registry.get("boltz2").tag == "boltz2-opt"
    assert registry.get("chai1").n_gpu == (1,)
    assert registry.get("evo2").default == "exact" and registry.get("atlasfold").default == "off"
    assert registry.get("proteinmpnn").default is None
    for d in os.listdir(os.path.join(ROOT, "kits")):
        assert os.path.isfile(os.path.join(ROOT, "kits", d, "run.sh"))
        assert os.path.isfile(os.path.join(ROOT, "kits", d, "configs", "b200.env"))


def test_dry_run_lines_with_fake_gpu(capsys):
    act = base.Activation(registry.get("boltz2"), "fast", "cli", 1, probe=_b200(), environ={})
    act.apply(None, dry_run=True)
    assert act.lines[0].startswith("[boltz2-opt] DRY-RUN mode=fast levers=sampler_graph,graph_verify,trunk_graph,fused_transition,")
    lever_lines = [l for l in act.lines if " LEVER " in l]
    assert any("name=fused_triatt state=on impl=pair_proj+attention_sm100@1 origin=core "
               "strategy=F1.kernel_fusion" in l for l in lever_lines)
    assert act.finish(0) == 0


def test_levers_off_and_partial_exit():
    env = {"MODEL_OPT_LEVERS_OFF": "fused_opm"}
    act = base.Activation(registry.get("boltz2"), "fast", "cli", 1, probe=_b200(), environ=env)
    act.apply(None, dry_run=True)
    assert "fused_opm" not in act.levers_on
    assert any("name=fused_opm state=off reason=user" in l for l in act.lines)
    act.levers_skipped["fused_pwa"] = "compile_failed"
    assert act.finish(0, allow_partial=False) == report.EXIT_NOT_ACTIVE
    assert act.finish(0, allow_partial=True) == 0


def test_refusals():
    h100 = lambda: [{"index": 0, "name": "NVIDIA H100", "cc": "9.0", "sm": "sm90", "mem_mib": 81559}]  # noqa: E731
    act = base.Activation(registry.get("boltz2"), "fast", "cli", 1, probe=h100, environ={})
    with pytest.raises(base.ActivationError):
        act.apply(None, dry_run=True)
    assert act.lines[-1].startswith("[boltz2-opt] NOT ACTIVE: gate gpu:")
    act = base.Activation(registry.get("boltz2"), "fast", "cli", 4, probe=_b200(), environ={})
    with pytest.raises(base.ActivationError):
        act.plan()
    assert "big-mode feature" in act.lines[-1]
    act = base.Activation(registry.get("boltz2"), "big", "cli", 4, probe=_b200(2), environ={})
    with pytest.raises(base.ActivationError):
        act.plan()
    act = base.Activation(registry.get("boltz2"), "big", "cli", 4, probe=_b200(8), environ={})
    assert "rowpair_tp" in act.plan()


def _run(args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run(["bash"] + args, capture_output=True, text=True, env=e, cwd=ROOT, timeout=120)


def test_run_sh_exit_codes(tmp_path):
    r = _run(["kits/boltz2/run.sh", "check", "--mode", "off"])
    assert r.returncode == 0 and "[boltz2-opt] DRY-RUN mode=off" in r.stderr
    r = _run(["kits/boltz2/run.sh", "check"], {"BOLTZ2_OPT": "turbo"})
    assert r.returncode == 3 and "NOT ACTIVE" in r.stderr
    r = _run(["kits/boltz2/run.sh", "frobnicate"])
    assert r.returncode == 2
    r = _run(["kits/proteinmpnn/run.sh", "check"])          # no default mode: every call names its mode
    assert r.returncode == 3 and "no mode given" in r.stderr
    r = _run(["kits/boltz2/run.sh", "check"], {"BOLTZ2_OPT_BOGUS": "1"})
    assert r.returncode == 3 and "undeclared" in r.stderr


def test_pred_off_on_cpu_writes_outputs_and_manifest(tmp_path):
    out = tmp_path / "o"
    r = _run(["kits/boltz2/run.sh", "pred", "--mode", "off", "--model_config", "tiny", "--tokens", "32",
              "--msa_depth", "4", "--out_dir", str(out)])
    assert r.returncode == 0, r.stderr[-2000:]
    assert "[boltz2-opt] STOCK clean=True" in r.stderr
    assert "[boltz2-opt] ACTIVE mode=off" in r.stderr and "[boltz2-opt] EXIT pid=" in r.stderr
    m = json.load(open(out / "opt_manifest.json"))
    assert m["mode"] == "off" and m["verdict"]["exit_code"] == 0
    assert (out / "prediction.pt").exists()


def test_lever_descriptors_can_be_written_on_a_lever_line():
    """Strategy ids are catalogued and no value that goes on a LEVER line holds a blank (the line grammar refuses it
    at the moment the lever engages, which is on the GPU for most of them)."""
    from uplifting_biomolecular_modeling_b200.core import strategies
    from uplifting_biomolecular_modeling_b200.kits import levers
    for name, lv in levers.LEVERS.items():
        assert strategies.is_known(lv.strategy), (name, lv.strategy)
        for field in (name, lv.strategy, lv.impl):
            assert field and " " not in str(field), (name, field)


def test_no_lever_is_a_no_op():
    """Every lever of the table has an ``apply`` that changes the object it is given (or raises): a table of names
    that do nothing cannot come back."""
    import types
    from uplifting_biomolecular_modeling_b200.kits import levers
    used = {n for spec in registry.REGISTRY.values() for names in spec.levers.values() for n in names}
    assert used <= set(levers.LEVERS), used - set(levers.LEVERS)
    for name, lv in levers.LEVERS.items():
        assert lv.apply is not None and lv.apply.__name__ != "_noop", name
        if lv.needs_gpu or name == "expandable_segments":
            continue                                  # these need a device (or the live allocator) to act on
        obj = types.SimpleNamespace(model=types.SimpleNamespace(workspace={}), n_gpu=1)
        snap = lambda: (sorted((k, repr(v)) for k, v in vars(obj).items() if k != "model"),  # noqa: E731
                        sorted((k, repr(v)) for k, v in vars(obj.model).items()))
        before = snap()
        ev = lv.apply(obj)
        assert ev and snap() != before, name


def test_pred_refuses_unreadable_input_and_unknown_config(tmp_path):
    r = _run(["kits/boltz2/run.sh", "pred", "--mode", "off", "--model_config", "tiny", "--input",
              str(tmp_path / "missing.pt")])
    assert r.returncode == 2 and "error=input" in r.stderr and "no_such_file" in r.stderr.replace(" ", "_")
    r = _run(["kits/boltz2/run.sh", "pred", "--mode", "off", "--model_config", "nonesuch", "--tokens", "16"])
    assert r.returncode == 2 and "unknown_model_config" in r.stderr
    spec = tmp_path / "complex.json"
    spec.write_text(json.dumps({"chains": [[12, "protein"], [8, "protein"]], "msa_depth": 2}))
    out = tmp_path / "o"
    r = _run(["kits/boltz2/run.sh", "pred", "--mode", "off", "--model_config", "tiny", "--input", str(spec),
              "--out_dir", str(out)])
    assert r.returncode == 0 and "tokens=20" in r.stderr, r.stderr[-1500:]


def test_partial_checkpoint_is_not_active(tmp_path):
    import torch
    from uplifting_biomolecular_modeling_b200.models import cofold
    m = cofold.build_model("tiny", seed=1)
    sd = m.state_dict()
    k0 = next(iter(sd))
    torch.save({"state_dict": {k0: sd[k0]}}, tmp_path / "one.ckpt")
    args = ["kits/boltz2/run.sh", "pred", "--mode", "off", "--model_config", "tiny", "--tokens", "16", "--msa_depth",
            "2", "--checkpoint", str(tmp_path / "one.ckpt")]
    r = _run(args)
    assert r.returncode == 3 and "NOT ACTIVE" in r.stderr and "missing" in r.stderr
    r = _run(args + ["--allow-partial", "--out_dir", str(tmp_path / "o")])
    assert r.returncode == 0 and "[boltz2-opt] WEIGHTS" in r.stderr and "matched=1" in r.stderr
    man = json.load(open(tmp_path / "o" / "opt_manifest.json"))
    assert man["checkpoint"]["matched"] == 1 and man["checkpoint"]["missing"]


def test_sequence_kit_checkpoint_is_loaded_strictly(tmp_path):
    """The language-model kits take --checkpoint too: a full state loads and changes the score, a partial one is
    NOT ACTIVE with exit 3 unless --allow-partial."""
    import torch
    from uplifting_biomolecular_modeling_b200.models import evo2
    m = evo2.build("evo2_tiny", seed=123)
    torch.save(m.state_dict(), tmp_path / "full.pt")
    k0 = next(iter(m.state_dict()))
    torch.save({k0: m.state_dict()[k0]}, tmp_path / "one.pt")
    base_args = ["kits/evo2/run.sh", "score", "--mode", "off", "--model_config", "evo2_tiny", "--prompt", "ACGTACGTAC"]
    r0 = _run(base_args)
    r1 = _run(base_args + ["--checkpoint", str(tmp_path / "full.pt")])
    assert r0.returncode == 0 and r1.returncode == 0, r1.stderr[-1500:]
    assert "[evo2-opt] WEIGHTS" in r1.stderr and "missing=0" in r1.stderr and "unexpected=0" in r1.stderr
    score = lambda r: [l for l in r.stderr.splitlines() if " DONE " in l][0].split("score=")[1].split()[0]  # noqa: E731
    assert score(r0) != score(r1)                     # other weights (seed 123 against the kit's seed), other score
    r2 = _run(base_args + ["--checkpoint", str(tmp_path / "one.pt")])
    assert r2.returncode == 3 and "NOT ACTIVE" in r2.stderr and "missing" in r2.stderr
    r3 = _run(base_args + ["--checkpoint", str(tmp_path / "one.pt"), "--allow-partial"])
    assert r3.returncode == 0 and "matched=1" in r3.stderr


def test_sequence_kit_reads_fasta_input_and_refuses_a_missing_file(tmp_path):
    fa = tmp_path / "two.fa"
    fa.write_text(">first some description\nACGTACGT\nACGT\n>second\nTTTTACGTAA\n")
    out = tmp_path / "o"
    r = _run(["kits/evo2/run.sh", "score", "--mode", "off", "--model_config", "evo2_tiny", "--input", str(fa),
              "--out_dir", str(out)])
    assert r.returncode == 0, r.stderr[-1500:]
    res = json.load(open(out / "score.json"))
    assert res["records"] == 2 and [p["id"] for p in res["per_record"]] == ["first", "second"]
    assert res["per_record"][0]["tokens"] == 12 and res["per_record"][1]["tokens"] == 10
    assert abs(res["mean_score"] - sum(p["score"] for p in res["per_record"]) / 2) < 1e-9
    r = _run(["kits/evo2/run.sh", "score", "--mode", "off", "--model_config", "evo2_tiny", "--input",
              str(tmp_path / "absent.fa")])
    assert r.returncode == 2 and "USAGE" in r.stderr and "no_such_file" in r.stderr.replace(" ", "_")


def test_full_checkpoint_loads_cold_and_reproduces_the_weights(tmp_path):
    """With a checkpoint that carries every parameter the model is built without its random initialisation (the fillers
    are skipped and counted) and the prediction equals the one of the model that wrote the checkpoint."""
    import torch
    from uplifting_biomolecular_modeling_b200.models import cofold
    m = cofold.build_model("tiny", seed=5)
    torch.save({"state_dict": m.state_dict()}, tmp_path / "full.ckpt")
    base_args = ["kits/boltz2/run.sh", "pred", "--mode", "off", "--model_config", "tiny", "--tokens", "16",
                 "--msa_depth", "2", "--seed", "5"]
    a = _run(base_args + ["--out_dir", str(tmp_path / "a")])
    b = _run(base_args + ["--checkpoint", str(tmp_path / "full.ckpt"), "--out_dir", str(tmp_path / "b")])
    assert a.returncode == 0 and b.returncode == 0, b.stderr[-1500:]
    word = [w for w in b.stderr.split() if w.startswith("init_skipped=")]
    assert word and int(word[0].split("=")[1]) > 0
    pa = torch.load(tmp_path / "a" / "prediction.pt", weights_only=True)
    pb = torch.load(tmp_path / "b" / "prediction.pt", weights_only=True)
    assert torch.equal(pa["coords"], pb["coords"])


def test_design_verb_runs_the_design_pipeline(tmp_path):
    out = tmp_path / "d"
    r = _run(["kits/boltzgen/run.sh", "design", "--mode", "off", "--model_config", "tiny", "--tokens", "24",
              "--diffusion_samples", "2", "--out_dir", str(out)])
    assert r.returncode == 0, r.stderr[-2000:]
    assert "designs=2" in r.stderr and "verb=design" in r.stderr
    d = json.load(open(out / "design.json"))
    assert len(d["sequences_text"]) == 2 and len(d["sequences_text"][0]) == 24


def test_resident_loop_over_a_directory_of_inputs(tmp_path):
    """Several inputs through one activation: featurised ahead, predicted in order, written behind; a bad item is
    reported and the others still run."""
    inp = tmp_path / "in"
    inp.mkdir()
    for i, n in enumerate((12, 16)):
        (inp / f"c{i}.json").write_text(json.dumps({"tokens": n, "msa_depth": 2}))
    (inp / "broken.json").write_text(json.dumps({"msa_depth": 2}))
    out = tmp_path / "o"
    r = _run(["kits/boltz2/run.sh", "pred", "--mode", "off", "--model_config", "tiny", "--input", str(inp),
              "--out_dir", str(out)])
    assert r.returncode == 2, r.stderr[-1500:]                       # the broken item makes the run a usage error ...
    assert "item=broken error=input" in r.stderr
    assert (out / "c0" / "prediction.pt").exists() and (out / "c1" / "prediction.pt").exists()   # ... the rest ran
    assert "RESIDENT items=2 failed=1" in r.stderr


def test_resident_loop_featurises_equal_inputs_once(tmp_path):
    """Two items with the same bytes under different names are featurised once (keyed by the file's digest) and both
    predicted."""
    inp = tmp_path / "in"
    inp.mkdir()
    spec = json.dumps({"tokens": 12, "msa_depth": 2})
    (inp / "a.json").write_text(spec)
    (inp / "b.json").write_text(spec)
    (inp / "c.json").write_text(json.dumps({"tokens": 16, "msa_depth": 2}))
    out = tmp_path / "o"
    r = _run(["kits/boltz2/run.sh", "pred", "--mode", "off", "--model_config", "tiny", "--input", str(inp),
              "--out_dir", str(out)])
    assert r.returncode == 0, r.stderr[-1500:]
    assert "features_built=2 features_reused=1" in r.stderr
    for name in "abc":
        assert (out / name / "prediction.pt").exists()


def test_genomic_track_kit_writes_a_bedgraph(tmp_path):
    """``predict`` of a genomic-track kit leaves the first predicted track as a bedGraph beside its JSON."""
    out = tmp_path / "t"
    r = _run(["kits/flashzoi/run.sh", "predict", "--mode", "off", "--out_dir", str(out)])
    assert r.returncode == 0, r.stderr[-2000:]
    res = json.load(open(out / "predict.json"))
    lines = [ln for ln in (out / "track_0.bedGraph").read_text().splitlines() if not ln.startswith("track")]
    assert 1 <= res["bedgraph_records"] == len(lines) <= res["bins"]          # equal neighbours are merged into one record
    rows = [ln.split("\t") for ln in lines]
    assert all(r[0] == "synthetic_window" for r in rows)
    assert int(rows[0][1]) == 0 and all(int(a[2]) == int(b[1]) for a, b in zip(rows, rows[1:]))   # contiguous
    assert int(rows[-1][2]) % res["bins"] == 0 and int(rows[-1][2]) > 0                            # bins x bin size


def test_install_places_the_pth_hook_and_the_variable_activates_in_process(tmp_path):
    site_dir = tmp_path / "site"
    r = _run(["kits/boltz2/run.sh", "install", "--pth-dir", str(site_dir)])
    assert r.returncode == 0 and "pth=" in r.stderr, r.stderr[-1500:]
    pth = site_dir / "boltz2_opt_autoload.pth"
    assert pth.exists() and "BOLTZ2_OPT" in pth.read_text()
    code = (f"import site, sys; site.addsitedir({str(site_dir)!r}); "
            "import uplifting_biomolecular_modeling_b200.models.cofold as c; "
            "print('loaded', 'uplifting_biomolecular_modeling_b200.kits.base' in sys.modules)")
    env = {k: v for k, v in os.environ.items() if not k.startswith("BOLTZ2_OPT")}
    # variable unset: the hook imports nothing of the kit layer
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=str(tmp_path))
    assert r.returncode == 0 and "loaded False" in r.stdout, r.stderr[-1500:]
    # an unknown mode is refused before anything runs
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True,
                       env=dict(env, BOLTZ2_OPT="turbo"), cwd=str(tmp_path))
    assert r.returncode == 3 and "NOT ACTIVE" in r.stderr
    # a mode whose gates fail on this machine is NOT ACTIVE with exit 3 at the trigger import (the probe asks
    # nvidia-smi, so a machine that has a B200 passes the gates whatever CUDA_VISIBLE_DEVICES says)
    if any(g.get("sm") == "sm100" for g in gates.probe_gpus()):
        return
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True,
                       env=dict(env, BOLTZ2_OPT="fast", CUDA_VISIBLE_DEVICES=""), cwd=str(tmp_path))
    assert r.returncode == 3 and "[boltz2-opt] NOT ACTIVE" in r.stderr, (r.returncode, r.stderr[-1500:])


def test_sequence_kit_tensor_parallel_worker_on_two_gloo_ranks(tmp_path):
    """``--n_gpu P`` of the StripedHyena-2 kit: two ranks of the worker (gloo, plain statements) return the single-
    process score and tokens; the plan accepts several GPUs in the mode that has the tensor-parallel lever only."""
    import sys
    from uplifting_biomolecular_modeling_b200.models import lm
    from uplifting_biomolecular_modeling_b200.parallel import launch
    prompt = "ACGTTGCAACGTTTGACCA"
    one = lm.build("evo2", "evo2_tiny", seed=0, kit="evo2")
    want_score = one.run("score", prompt)["score"]
    want_text = one.run("generate", prompt, 6)["text"]
    for verb in ("score", "generate"):
        out = tmp_path / f"{verb}.json"
        launch.run_rank_processes(2, [sys.executable, "-m", "uplifting_biomolecular_modeling_b200.parallel.lm_worker",
                                      "--config", "evo2_tiny", "--verb", verb, "--prompt", prompt, "--max_new_tokens",
                                      "6", "--out", str(out)], cpu=True, run_timeout_s=240,
                                  log_dir=str(tmp_path / f"logs_{verb}"), extra_env={"PYTHONPATH": ROOT},
                                  echo_rank0=False)
        res = json.load(open(out))
        assert res["world"] == 2 and res["reduce_calls"] > 0
        if verb == "score":
            assert abs(res["score"] - want_score) <= 1e-4 * max(1.0, abs(want_score))
        else:
            assert res["text"] == want_text
    spec = registry.get("evo2")
    base.Activation(spec, "fast", "cli", 2, probe=_b200(), environ={}).plan()
    with pytest.raises(base.ActivationError):
        base.Activation(spec, "exact", "cli", 2, probe=_b200(), environ={}).plan()


def test_sequence_kit_sharded_launcher_checks_the_checkpoint_before_it_starts_ranks(tmp_path, capsys):
    """The parent of ``--n_gpu P``: a fitting checkpoint goes to the ranks (gloo here), one that does not fit is
    NOT ACTIVE with exit 3 and no rank process is started."""
    import argparse
    import torch
    from uplifting_biomolecular_modeling_b200.core import report
    from uplifting_biomolecular_modeling_b200.kits import run
    from uplifting_biomolecular_modeling_b200.models import evo2
    m = evo2.build("evo2_tiny", seed=5)
    torch.save(m.state_dict(), tmp_path / "full.pt")
    k0 = next(iter(m.state_dict()))
    torch.save({k0: m.state_dict()[k0]}, tmp_path / "one.pt")
    spec = registry.get("evo2")

    def args(ckpt, out):
        return argparse.Namespace(verb="score", model_config="evo2_tiny", prompt="ACGTTGCAAC", input=None, seed=0,
                                  max_new_tokens=4, checkpoint=str(ckpt), weights=None, out_dir=str(out))

    def activation():
        act = base.Activation(spec, "fast", "cli", 2, probe=_b200(), environ={})
        act.register_exit = lambda: None            # no exit hook in the test process
        return act

    rc = run._run_lm_sharded(spec, activation(), args(tmp_path / "one.pt", tmp_path / "o1"), False)
    assert rc == report.EXIT_NOT_ACTIVE and not os.path.exists(tmp_path / "o1" / "score.json")
    rc = run._run_lm_sharded(spec, activation(), args(tmp_path / "full.pt", tmp_path / "o2"), False)
    res = json.load(open(tmp_path / "o2" / "score.json"))
    m.eval()
    want = float(m.score(evo2.tokenize("ACGTTGCAAC"))[0])
    assert res["world"] == 2 and abs(res["score"] - want) <= 1e-4 * max(1.0, abs(want))
    err = capsys.readouterr().err
    assert "WEIGHTS" in err and "sharding=tensor_parallel" in err and "NOT ACTIVE" in err


def test_sharded_cofold_launcher_refuses_a_checkpoint_that_does_not_fit_before_it_starts_ranks(tmp_path, capsys):
    import argparse
    import torch
    from uplifting_biomolecular_modeling_b200.core import report
    from uplifting_biomolecular_modeling_b200.models import cofold
    from uplifting_biomolecular_modeling_b200.parallel import launch
    m = cofold.build_model("tiny", seed=1)
    k0 = next(iter(m.state_dict()))
    torch.save({"state_dict": {k0: m.state_dict()[k0]}}, tmp_path / "one.ckpt")
    spec = registry.get("boltz2")
    act = base.Activation(spec, "big", "cli", 2, probe=_b200(), environ={})
    act.register_exit = lambda: None
    args = argparse.Namespace(checkpoint=str(tmp_path / "one.ckpt"), weights=None, tokens=32, msa_depth=2, seed=0,
                              out_dir=None, recycling_steps=None, input=None, sampling_steps=None,
                              diffusion_samples=None)
    started = []
    real = launch.run_sharded
    launch.run_sharded = lambda *a, **k: started.append(a)
    try:
        rc = launch.run_prediction_sharded(spec, act, args, "tiny", False)
    finally:
        launch.run_sharded = real
    assert rc == report.EXIT_NOT_ACTIVE and not started
    assert "NOT ACTIVE" in capsys.readouterr().err
