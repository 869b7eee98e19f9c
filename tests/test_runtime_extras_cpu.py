"""Upstream-fix registry, external digests, the pre-import pin gate, warm imports, worker packing."""
import sys

import pytest
import torch

from uplifting_biomolecular_modeling_b200.core import core_gate, extern, report, upstream_fix, warm
from uplifting_biomolecular_modeling_b200.host import packing


def test_upstream_fix_registry(capsys):
    upstream_fix._clear_for_tests()
    hit = []
    upstream_fix.register(upstream_fix.Fix("mask_sign", "flip the sign of the padding mask", lambda m: hit.append(m) or True,
                                           kits=("boltz2",)))
    upstream_fix.register(upstream_fix.Fix("noop", "nothing to do here", lambda m: False))
    assert upstream_fix.parse("mask_sign, noop") == ["mask_sign", "noop"]
    words = upstream_fix.apply_all("model", ["mask_sign", "noop"], tag="boltz2-opt", kit="boltz2")
    assert words == ["fix:mask_sign", "fix:noop:nothing_to_fix"] and hit == ["model"]
    assert "UPSTREAM-FIX name=mask_sign" in capsys.readouterr().err
    with pytest.raises(upstream_fix.UnknownFix, match="known: noop"):
        upstream_fix.resolve(["mask_sign"], kit="chai1")
    with pytest.raises(upstream_fix.UnknownFix):
        upstream_fix.resolve(["bogus"])
    upstream_fix._clear_for_tests()


def test_weight_digest_is_container_independent(tmp_path):
    a = {"w": torch.arange(6.0).view(2, 3), "b": torch.zeros(3, dtype=torch.bfloat16)}
    b = dict(reversed(list(a.items())))
    assert extern.weight_digest(a) == extern.weight_digest(b)
    c = {"w": a["w"].clone(), "b": a["b"].clone()}
    c["w"][0, 0] = 1
    assert extern.weight_digest(c) != extern.weight_digest(a)
    p = tmp_path / "f.bin"
    p.write_bytes(b"abc" * 1000)
    d = extern.file_digest(str(p))
    extern.check("f.bin", d, d)
    with pytest.raises(extern.DigestMismatch, match="f.bin"):
        extern.check("f.bin", d, "0" * 64)


def test_core_gate_exits_3_on_a_pin_mismatch(capsys):
    versions = {"opt_core": "0.5.228.0", "torch": "2.11.0+cu128"}
    assert core_gate.satisfies("2.11.0+cu128", "2.11.*") and core_gate.satisfies("2.11.0", ">=2.4")
    assert not core_gate.satisfies("2.3.1", ">=2.4") and not core_gate.satisfies(None, "1.0")
    assert core_gate.check("boltz2-opt", {"opt_core": "0.5.228.0", "torch": "2.11.*"}, versions.get)
    codes = []
    ok = core_gate.check("boltz2-opt", {"opt_core": "0.6.*"}, versions.get, exit_fn=codes.append)
    assert not ok and codes == [report.EXIT_NOT_ACTIVE]
    assert "[boltz2-opt] NOT ACTIVE reason=core_pin name=opt_core pinned=0.6.* found=0.5.228.0" in capsys.readouterr().err


def test_warm_imports_run_off_thread():
    w = warm.warm(["json", "no_such_module_xyz"])
    secs = w.join(10)
    assert set(secs) == {"json", "no_such_module_xyz"} and "no_such_module_xyz" in w.errors


def test_worker_packing_reports_oom_as_rc_6(tmp_path):
    py = sys.executable
    ok = [py, "-c", "import os; print('worker', os.environ['UBM_WORKER_INDEX'], 'of', os.environ['UBM_WORKER_COUNT'])"]
    res = packing.run_workers([ok, ok], str(tmp_path / "a"))
    assert res.exit_code == 0 and "worker 1 of 2" in open(res.logs[1]).read()
    boom = [py, "-c", "import sys; print('torch.OutOfMemoryError: CUDA out of memory. Tried to allocate'); sys.exit(1)"]
    res = packing.run_workers([ok, boom], str(tmp_path / "b"))
    assert res.exit_code == packing.EXIT_OOM and res.oom_workers == [1]
    bad = [py, "-c", "import sys; sys.exit(4)"]
    assert packing.run_workers([bad], str(tmp_path / "c")).exit_code == 1
    assert packing.mps_available({}) is False


def test_roomy_call_runs_from_a_frame_larger_than_a_stack_chunk():
    import sys
    from uplifting_biomolecular_modeling_b200.core import pystack, warm

    def depth():
        f, n = sys._getframe(), 0
        while f is not None:
            n += 1
            f = f.f_back
        return n

    assert pystack.roomy_call(lambda a, b=1: a + b, 2, b=3) == 5
    assert pystack.frame_slots() * 8 > 16 * 1024                      # bigger than one 16 KiB chunk
    assert pystack.roomy_call(depth) == depth() + 2                  # the large frame and the callee sit above the caller
    try:
        pystack.roomy_call(lambda: 1 / 0)
        raise AssertionError("exception swallowed")
    except ZeroDivisionError:
        pass
    assert pystack.call_cost_us(200) < 1000.0
    w = warm.warm(["json", "no_such_module_xyz"])
    w.join(10)
    assert "json" in w.seconds and "no_such_module_xyz" in w.errors
