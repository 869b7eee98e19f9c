"""Counted dispatch: every call of a switched module is served or a named fallback; undeclared reasons fail closed."""
import torch

from uplifting_biomolecular_modeling_b200.core import cell_census, counters, report
from uplifting_biomolecular_modeling_b200.kits import base, registry
from uplifting_biomolecular_modeling_b200.models import pairformer
from uplifting_biomolecular_modeling_b200.models import weights
from uplifting_biomolecular_modeling_b200.ops import dispatch


def _fresh():
    counters.BOOK._ledgers.clear()
    cell_census.reset()
    dispatch.reset()


def test_cpu_call_under_the_kernel_implementation_is_a_counted_fallback_and_exits_3():
    _fresh()
    torch.manual_seed(0)
    layer = pairformer.PairformerLayer(no_seq=True).eval()
    pairformer.set_impl(layer, "fused")
    z = torch.randn(1, 8, 8, 128)
    with torch.no_grad():
        out = layer.pair_update(z, None)
    assert out.shape == z.shape
    lg = counters.BOOK.get("fused_triatt")
    assert lg.served == 0 and lg.fallbacks == {"not_cuda": 2}
    assert lg.gate() == "undeclared_fallback:not_cuda"
    recs = [r for r in cell_census.records() if r["family"] == "triattn"]
    assert recs and recs[0]["outcome"] == "named_fallback" and recs[0]["reason"] == "not_cuda"
    # the activation turns the open ledgers into PARTIAL / exit 3, and into 0 under --allow-partial
    act = base.Activation(registry.get("boltz2"), "off", "cli", 1, environ={})
    assert "fused_triatt" in act.report_dict()["partial"]
    assert act.finish(0, allow_partial=False) == report.EXIT_NOT_ACTIVE
    assert act.finish(0, allow_partial=True) == 0
    _fresh()


def test_declared_reason_closes_the_ledger_and_plain_modules_are_not_counted():
    _fresh()
    assert dispatch.decide("fused_apb", "cross_keys", "D32H16S1", 64) is False
    assert dispatch.decide("fused_apb", None, "D32H16S1", 64) is True
    assert counters.BOOK.get("fused_apb").gate() is None
    layer = pairformer.PairformerLayer(no_seq=True).eval()           # implementation "reference": nothing to count
    with torch.no_grad():
        layer.pair_update(torch.randn(1, 4, 4, 128), None)
    assert "fused_trimul" not in dict(counters.BOOK.items())
    _fresh()


def test_checkpoint_key_collisions_and_shape_mismatches_are_named(tmp_path):
    import pytest
    lin = torch.nn.Linear(4, 4)
    sd = {"model.weight": torch.zeros(4, 4), "ema.model.weight": torch.ones(4, 4), "model.bias": torch.zeros(4)}
    with pytest.raises(weights.KeyCollision):
        weights.strip_prefixes(sd)
    assert torch.equal(weights.strip_prefixes(sd, ema=True)["weight"], torch.ones(4, 4))
    assert torch.equal(weights.strip_prefixes(sd, ema=False)["weight"], torch.zeros(4, 4))
    torch.save({"state_dict": {"weight": torch.zeros(4, 3), "bias": torch.zeros(4)}}, tmp_path / "c.pt")
    with pytest.raises(ValueError, match="shape-mismatched"):
        weights.load_checkpoint(lin, str(tmp_path / "c.pt"))
    rep = weights.load_checkpoint(lin, str(tmp_path / "c.pt"), strict=False)
    assert rep.matched == 1 and rep.shape_mismatch and rep.shape_mismatch[0].startswith("weight:")


def test_token_window_of_a_lever_is_a_declared_counted_fallback(monkeypatch):
    """The ``below_min`` rung: a call outside a lever's token window runs the plain statement, is counted under its
    own reason and leaves the ledger closed (the window is a setting, not a degradation)."""
    monkeypatch.setenv("UBM_MIN_TOKENS_FUSED_TRIMUL", "128")
    monkeypatch.setenv("UBM_MAX_TOKENS", "4096")
    _fresh()
    assert dispatch.decide("fused_trimul", None, "c128", 64) is False
    assert dispatch.decide("fused_trimul", None, "c128", 256) is True
    assert dispatch.decide("fused_trimul", None, "c128", 8192) is False
    assert dispatch.decide("fused_transition", None, "c128", 64) is True       # the general window has no minimum
    lg = counters.BOOK.get("fused_trimul")
    assert lg.served == 1 and lg.fallbacks == {"below_min_tokens": 1, "above_max_tokens": 1}
    assert lg.gate() is None
    gate = dispatch.size_gate("fused_trimul")
    assert gate.total == 3 and "below_min_tokens:128=1" in gate.words()
    reasons = {r["reason"] for r in cell_census.records() if r["family"] == "trimul" and r["outcome"] == "named_fallback"}
    assert reasons == {"below_min_tokens", "above_max_tokens"}
    _fresh()
