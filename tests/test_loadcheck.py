"""Verdict logic of the kernel self-verification (the probes themselves need a GPU)."""
import pytest

from uplifting_biomolecular_modeling_b200.ops import loadcheck


def test_verdict_line_and_refusal(capsys):
    good = loadcheck.run_all("cpu", probes={"a": lambda d: (1e-3, 2e-2), "b": lambda d: (0.0, 1e-2)})
    assert good.ok and "KERNELS-VERIFIED families=2 failed=none" in good.line("boltz2-opt")

    def boom(dev):
        raise RuntimeError("launch failed")
    bad = loadcheck.run_all("cpu", probes={"a": lambda d: (1e-3, 2e-2), "b": lambda d: (0.5, 2e-2),
                                           "c": lambda d: (float("nan"), 1.0), "d": boom})
    assert not bad.ok and [p.family for p in bad.failed] == ["b", "c", "d"]
    assert "KERNELS-REFUSED" in bad.line() and "failed=b,c,d" in bad.line()
    assert "RuntimeError" in bad.failed[2].detail
    with pytest.raises(loadcheck.KernelsRefused, match="b\\("):
        raise loadcheck.KernelsRefused(bad.failed)




def test_a_family_that_fails_tuned_is_retried_under_its_safe_setting():
    state = {"safe": False}

    def flaky(dev):
        return (1e-3, 2e-2) if state["safe"] else (0.9, 2e-2)
    lc = loadcheck.run_all("cpu", probes={"triattn": flaky, "gemm": lambda d: (0.0, 1e-2)},
                           safe={"triattn": lambda: state.__setitem__("safe", True)})
    assert lc.ok and "settings=safe:triattn" in lc.line("x")
    state["safe"] = False
    lc = loadcheck.run_all("cpu", probes={"triattn": lambda d: (0.9, 2e-2)}, safe={"triattn": lambda: None})
    assert not lc.ok and "KERNELS-REFUSED" in lc.line() and "settings=tuned" in lc.line()     # safe form failed too


@pytest.mark.gpu
def test_every_family_verifies_on_the_gpu():
    lc = loadcheck.run_all("cuda:0", use_cache=False)
    assert lc.ok, lc.line()
    # the probes sit well inside their tolerances (a false refusal would take a working GPU out of service)
    assert all(p.error <= 0.5 * p.tolerance for p in lc.probes), [(p.family, p.error) for p in lc.probes]
    assert "settings=tuned" in lc.line()
