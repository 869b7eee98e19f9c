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
    assert act.lines[0].startswith("[boltz2-opt] DRY-RUN mode=fast levers=hoist_pair_bias,")
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
