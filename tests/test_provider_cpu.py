"""Provider selection over the measured table, census outcomes, named refusals, the size gate."""
import pytest

from uplifting_biomolecular_modeling_b200.core import cell_census
from uplifting_biomolecular_modeling_b200.ops import provider as pv


def setup_function(_):
    cell_census.reset()


def test_select_is_pure_and_records_outcomes():
    a = pv.select("triattn", "sm100", "D32H4", 1536, "fast", {"head_dim": 32, "dtype": "bf16"})
    b = pv.select("triattn", "sm100", "D32H4", 1536, "fast", {"head_dim": 32, "dtype": "bf16"})
    assert a == b and a.row == "tcgen05_4row" and a.outcome == "cell_hit" and a.expected_ms == pytest.approx(4.98)
    inh = pv.select("triattn", "sm100", "D32H4", 1000, "fast", {"head_dim": 32, "dtype": "bf16"})
    assert inh.outcome == "inherited" and inh.key.endswith("N1536")
    ex = pv.select("triattn", "sm100", "D32H4", 1536, "exact")
    assert ex.row == "stock"
    out = pv.select("triattn", "sm100", "D16H8", 768, "fast")
    assert out.row == "stock" and out.outcome == "stock" and "not measured" in out.reason
    s = cell_census.summary()["triattn"]
    assert s["cell_hit"] >= 1 and s["inherited"] == 1 and s["stock"] == 1
    with pytest.raises(ValueError):
        pv.select("triattn", "sm100", "D32H4", 768, "turbo")


def test_named_refusal_falls_to_the_next_measured_row():
    sel = pv.select("transition", "sm100", "C128X4", 1536, "fast", {"c": 128, "expansion": 2, "dtype": "bf16"})
    assert sel.row == "rows_gemm" and sel.outcome == "named_fallback" and "expansion=2" in sel.reason
    sel = pv.select("transition", "sm100", "C128X4", 1536, "fast", {"c": 128, "expansion": 4, "dtype": "fp32"})
    assert sel.row == "stock" and sel.outcome == "named_fallback"


def test_every_serving_row_of_the_table_is_measured_and_registered():
    for fam, cells in pv.table().items():
        if fam == "note":
            continue
        for key, cell in cells.items():
            assert len(key.split("|")) == 3
            for tier, row in cell["serve"].items():
                assert tier in pv.TIERS and row in cell["rows"], (fam, key, tier, row)
                assert row == "stock" or (fam, row) in pv._ROWS, (fam, row)
            assert set(cell["order"]) == set(cell["rows"]), (fam, key)


def test_size_gate_accounts_for_every_call():
    g = pv.SizeGate("trimul_fused", min_tokens=64, max_tokens=4096)
    assert [g.admit(n) for n in (32, 64, 5000, 1536, 16)] == [False, True, False, True, False]
    assert g.total == 5 and g.served == 2
    assert "below_min_tokens:64=2" in g.words() and "above_max_tokens:4096=1" in g.words()


def test_predictor_plan_names_a_row_for_every_call_class():
    from uplifting_biomolecular_modeling_b200 import api
    pred = api.Predictor("tiny", mode="exact", device="cpu", dtype=__import__("torch").float32)
    plan = pred.provider_plan(1536, 12768)
    assert plan and all(sel.row == "stock" for sel in plan.values())          # exact = the plain statements
    assert api.Predictor("tiny", mode="off", device="cpu", dtype=__import__("torch").float32).provider_plan(64) == {}
    pred.mode = "fast"                                                         # table lookup only, nothing runs
    pred.dtype = __import__("torch").bfloat16
    fast = pred.provider_plan(1536, 12768)
    assert fast["triattn|D32H4"].row in ("tcgen05_4row", "stock")              # stock when the table has no cpu cells
