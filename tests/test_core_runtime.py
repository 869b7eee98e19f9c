"""Contract runtime on CPU: line grammar, mode resolution, exit rule, gates, arch, ledgers, manifest,
autoload, census, environment scripts."""
import json
import os
import sys
import types

import pytest

from uplifting_biomolecular_modeling_b200.core import (arch, autoload, cell_census, counters, gates, jit_cache,
                                                       manifest, modes, oom, report, shape_policy, stock_proof)


def test_line_grammar_and_words():
    assert report.line("boltz2-opt", "ACTIVE", ("mode", "fast"), levers=["a", "b"]) == \
        "[boltz2-opt] ACTIVE mode=fast levers=a,b"
    assert report.kv(x=None, y=[], z={"a": 1}) == "x=none y=none z=a:1"
    assert report.word("card", "uncertified", "NVIDIA L4", "22731MiB") == "card=uncertified(NVIDIA_L4,22731MiB)"
    line = report.active_line("k-opt", "fast", ["l1"], words=[report.word("cache", "miss", 3)])
    assert line == "[k-opt] ACTIVE mode=fast levers=l1 cache=miss(3)"
    assert report.not_active_line("k-opt", "no GPU", "mode=fast") == "[k-opt] NOT ACTIVE: no GPU (mode=fast)"


def test_lever_line_rules():
    s = report.lever_line("k-opt", "fused_trimul", "on", impl="trimul_sm100@1", origin="core",
                          strategy="F1.kernel_fusion", served=3)
    assert s == "[k-opt] LEVER name=fused_trimul state=on impl=trimul_sm100@1 origin=core " \
                "strategy=F1.kernel_fusion served=3"
    with pytest.raises(ValueError):
        report.lever_line("k", "x", "skipped", impl="i", origin="core")          # reason missing
    with pytest.raises(ValueError):
        report.lever_line("k", "x", "on", impl="i", origin="elsewhere")
    with pytest.raises(ValueError):
        report.lever_line("k", "x", "on", impl="has blank", origin="core")
    with pytest.raises(ValueError):
        report.lever_line("k", "x", "on", impl="i", origin="kit", strategy="bogus")


def test_exit_rule():
    v = report.verdict(0, {"partial": ["a"]}, False)
    assert v["exit_code"] == report.EXIT_NOT_ACTIVE
    assert report.verdict(0, {"partial": ["a"]}, True)["exit_code"] == 0
    assert report.verdict(0, {}, False, incomplete="2 of 3 outputs")["exit_code"] == report.EXIT_FAIL
    assert report.verdict(1, {"partial": ["a"]}, False)["exit_code"] == 1
    assert "NOT ACTIVE: partial activation" in report.partial_line("k", v, {"a": "no kernel"})
    assert report.tally_fields({"m": {"zeta": 1, "rank": 0, "alpha": 2}}, max_fields=2) == ["m={rank=0,alpha=2,...+1}"]


def test_modes_resolution_precedence():
    t = modes.ModeTable("boltz2", {"off": [], "exact": ["a"], "fast": ["b"], "big": ["c"]}, default="fast",
                        bases={"fast": "exact", "big": "fast"})
    assert t.levers("big") == ("a", "b", "c")
    assert modes.resolve_mode(t, "exact", "BOLTZ2_OPT", {"BOLTZ2_OPT": "big"}).mode == "exact"
    r = modes.resolve_mode(t, None, "BOLTZ2_OPT", {"BOLTZ2_OPT": "big"})
    assert (r.mode, r.source) == ("big", "env:BOLTZ2_OPT")
    assert modes.resolve_mode(t, None, "BOLTZ2_OPT", {}).source == "default"
    with pytest.raises(modes.ModeError):
        modes.resolve_mode(t, "turbo", "BOLTZ2_OPT", {})
    with pytest.raises(modes.ModeError):
        modes.ModeTable("x", {"fast": []})
    assert modes.levers_off({"MODEL_OPT_LEVERS_OFF": "a, b"}) == ("a", "b")
    assert modes.check_declared_env("K_OPT", ["K_OPT"], {"K_OPT": "fast", "K_OPT_X": "1"}) == ["K_OPT_X"]


def test_env_script():
    s = modes.EnvScript('# card\nexport MODEL_OPT_TARGET_GPU=b200\nFOO="${BAR:-dflt}/x"\n')
    env = {}
    s.apply(env)
    assert env == {"MODEL_OPT_TARGET_GPU": "b200", "FOO": "dflt/x"}


def test_gates_with_fake_probe():
    b200 = lambda: [{"index": 0, "name": "NVIDIA B200", "cc": "10.0", "sm": "sm100", "mem_mib": 183359}]  # noqa: E731
    h100 = lambda: [{"index": 0, "name": "NVIDIA H100 80GB HBM3", "cc": "9.0", "sm": "sm90", "mem_mib": 81559}]  # noqa: E731
    assert gates.gpu_gate(probe=b200).ok
    g = gates.gpu_gate(probe=h100)
    assert not g.ok and "sm100" in g.detail
    assert not gates.gpu_gate(probe=lambda: [], n_required=1).ok
    assert not gates.gpu_gate(probe=b200, n_required=2).ok
    assert gates.gpu_class("NVIDIA GB200") == "gb200"
    ok, gs = gates.run_gates([lambda: gates.Gate("a", True), lambda: 1 / 0])
    assert not ok and gates.first_failure(gs).name
    assert gates.version_gate("torch", "2.11.0", minimum="2.8").ok
    assert not gates.version_gate("torch", "2.1.0", minimum="2.8").ok
    assert not gates.core_pin_check("0.0.9", "0.1.0").ok
    e = gates.cannot_run(RuntimeError("x"))
    assert gates.is_cannot_run(e) and gates.is_cannot_run(gates.CannotRun("y"))


def test_nvidia_smi_probe_parses(tmp_path):
    class R:
        returncode = 0
        stdout = "0, NVIDIA B200, 10.0, 183359\n1, NVIDIA B200, 10.0, 183359\n"
    out = gates.nvidia_smi_probe(run=lambda *a, **k: R(), which=lambda n: "/usr/bin/nvidia-smi")
    assert [g["sm"] for g in out] == ["sm100", "sm100"]
    assert gates.nvidia_smi_probe(which=lambda n: None) == []


def test_sums_and_binary_refusal(tmp_path):
    f = tmp_path / "lib.so"
    f.write_bytes(b"abc")
    d = gates.sha256_file(f)
    (tmp_path / "SHA256SUMS").write_text(f"{d}  lib.so\n")
    assert gates.sums_gate(tmp_path / "SHA256SUMS").ok
    assert gates.binary_refusal(f, d) is None
    assert gates.binary_refusal(f, "0" * 64).startswith("binary_digest_mismatch")
    f.write_bytes(b"abd")
    assert not gates.sums_gate(tmp_path / "SHA256SUMS").ok
    assert gates.binary_refusal(tmp_path / "nope.so", None).startswith("binary_missing")


def test_arch_support_words():
    assert arch.supports("fused_trimul", "sm100") == "supported"
    assert arch.supports("fused_trimul", "sm90").startswith("unsupported:needs_sm100")
    assert arch.supports("fused_trimul", "sm103") == "uncertified"
    with pytest.raises(arch.ArchRefused) as ei:
        arch.require("fused_trimul", "sm90")
    assert gates.is_cannot_run(ei.value)
    with pytest.raises(ValueError):
        arch.declare("x", certified=("sm999",))


def test_ledger_fail_closed():
    lg = counters.Ledger("fused_trimul", "trimul_sm100@1", declared_fallbacks=["below_min_tokens"], min_tokens=64)
    lg.serve("N1536")
    lg.fallback("below_min_tokens")
    assert lg.gate() is None
    assert "served=1 fallback=1 fallback_by=below_min_tokens:1 min_tokens=64" in lg.line("k")
    lg.fallback("dtype_fp64")
    assert lg.gate() == "undeclared_fallback:dtype_fp64"
    lg.error(ValueError("x"))
    assert lg.gate().startswith("error:ValueError")
    book = counters.LedgerBook()
    book.get("a", "impl").fallback("r")
    assert "a" in book.partial()


def test_manifest_roundtrip(tmp_path):
    m = manifest.build("boltz2", "fast", "cli", ["a"], {"b": "no kernel"}, words=["card=uncertified(x)"],
                       verdict={"exit_code": 0})
    p = manifest.write(tmp_path, m)
    assert os.path.basename(p) == "opt_manifest.json"
    assert manifest.read(tmp_path)["levers_skipped"] == {"b": "no kernel"}
    assert manifest.read(tmp_path / "missing") is None


def test_autoload_fires_on_trigger_and_refuses(tmp_path, monkeypatch):
    pkgdir = tmp_path / "pkgs"
    pkgdir.mkdir()
    (pkgdir / "fake_upstream.py").write_text("VALUE = 1\n")
    (pkgdir / "fake_kit.py").write_text(
        "CALLS = []\n"
        "def enable(mode, strict=False, trigger=None):\n"
        "    if mode == 'big':\n        raise RuntimeError('needs 2 GPUs')\n"
        "    CALLS.append((mode, strict, trigger))\n")
    monkeypatch.syspath_prepend(str(pkgdir))
    exits = []
    spec = autoload.AutoloadSpec("fake-opt", "FAKE_OPT", "fake_kit", ("fake_upstream",), exit_fn=exits.append)
    mp = []
    assert autoload.install(spec, {}, mp) is None and mp == []            # variable unset: nothing installed
    finder = autoload.install(spec, {"FAKE_OPT": "exact"}, mp)
    assert mp == [finder]
    monkeypatch.setattr(sys, "meta_path", [finder] + sys.meta_path)
    import importlib
    up = importlib.import_module("fake_upstream")
    assert up.VALUE == 1
    assert sys.modules["fake_kit"].CALLS == [("exact", True, "fake_upstream")]
    # unknown mode and failing enable -> NOT ACTIVE + exit 3
    autoload.install(spec, {"FAKE_OPT": "turbo"}, [])
    assert exits == [3]
    autoload.fire(spec, "big", trigger="fake_upstream")
    assert exits == [3, 3]
    for m in ("fake_upstream", "fake_kit"):
        sys.modules.pop(m, None)


def test_census_and_nearest():
    cell_census.reset()
    assert cell_census.record("triattn", "10.0|bf16|D32|H4|N<=1536", "cell_hit", row="attention_sm100")
    assert not cell_census.record("triattn", "10.0|bf16|D32|H4|N<=1536", "cell_hit")
    cell_census.record("trimul", "x", "named_fallback", reason="c_z=256")
    assert cell_census.summary()["triattn"]["cell_hit"] == 1
    assert any("family=trimul" in l and "named_fallback=1" in l for l in cell_census.exit_lines())
    assert cell_census.nearest([800, 1536, 2048], 1000) == 1536
    assert cell_census.nearest([800, 1536, 2048], 5000) == 2048
    assert cell_census.nearest([800, 1536], 1000, "floor") == 800
    with pytest.raises(ValueError):
        cell_census.record("a", "b", "maybe")


def test_small_helpers(tmp_path):
    assert oom.is_oom_text("RuntimeError: CUDA out of memory. Tried to allocate")
    assert not oom.is_oom(ValueError("shape"))
    assert shape_policy.pad_to_tile(1488) == 1536 and shape_policy.bucket(1500) == 1536
    assert shape_policy.plane_leading_dim(1489) == 1496
    assert jit_cache.stack_key("2.11.0", "12.8", "sm100") == "torch2.11.0-cu128-sm100"
    assert jit_cache.root({"MODEL_OPT_JIT_ROOT": "/x"}) == "/x"
    pr = stock_proof.env_proof(["BOLTZ2_OPT"], ["boltz2_opt"], {"BOLTZ2_OPT": "fast"}, {"boltz2_opt.cli": 1}, [])
    assert not pr["clean"] and pr["env"] == ["BOLTZ2_OPT"] and pr["modules"] == ["boltz2_opt.cli"]
    assert stock_proof.env_proof(["BOLTZ2_OPT"], ["boltz2_opt"], {}, {}, [])["clean"]
