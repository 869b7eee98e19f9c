"""Capture-safety instruments and the host-side exchange-plan check."""
import pytest
import torch

from uplifting_biomolecular_modeling_b200.capture import audit
from uplifting_biomolecular_modeling_b200.ops import native
from uplifting_biomolecular_modeling_b200.parallel import plan_check as pc
from uplifting_biomolecular_modeling_b200.parallel.plan_check import Transfer as T


def test_launch_counter_counts_by_entry_point():
    with audit.LaunchCounter() as lc:
        native.add_launches(3, "ubm_gemm_bf16_ex")
        native.add_launches(10)
    assert lc.by_entry == {"ubm_gemm_bf16_ex": 3, "graph_replay": 10}
    assert lc.total == 13 and lc.replays == 10


def test_rng_guard():
    with audit.RNGGuard() as g:
        torch.zeros(3) + 1
    assert not g.advanced
    with pytest.raises(audit.AuditError):
        with audit.RNGGuard(expect="unchanged"):
            torch.randn(2)
    with audit.RNGGuard(expect="advanced") as g:
        torch.randn(2)
    assert g.cpu_advanced
    with pytest.raises(audit.AuditError):
        with audit.RNGGuard(expect="advanced"):
            pass


def test_audit_capture_safety_findings():
    x = torch.arange(8.0)
    ok = audit.audit_capture_safety(lambda: {"y": x * 2})
    assert ok.safe and "CAPTURE-SAFE" in ok.line("double")
    noisy = audit.audit_capture_safety(lambda: x + torch.randn(8))
    assert not noisy.safe and noisy.rng_advanced and "NOT-CAPTURE-SAFE" in noisy.line()
    assert audit.audit_capture_safety(lambda: x + torch.randn(8), allow_rng=True).safe
    state = {"n": 0}

    def drifting():
        state["n"] += 1
        return x + state["n"]
    rep = audit.audit_capture_safety(drifting)
    assert not rep.deterministic and not rep.safe


def test_exchange_plan_matches_and_refuses():
    good = {0: [T("send", 1, "a", 64), T("recv", 1, "b", 32)], 1: [T("recv", 0, "a", 64), T("send", 0, "b", 32)]}
    assert pc.check_exchange_plan(good) == 2
    with pytest.raises(pc.PlanMismatch, match="do not pair up"):
        pc.check_exchange_plan({0: [T("send", 1, "a", 64)], 1: [T("recv", 0, "a", 48)]})
    with pytest.raises(pc.PlanMismatch, match="different orders"):
        pc.check_exchange_plan({0: [T("send", 1, "a", 8), T("send", 1, "b", 8)],
                                1: [T("recv", 0, "b", 8), T("recv", 0, "a", 8)]})
    with pytest.raises(pc.PlanMismatch, match="both start by receiving"):
        pc.check_exchange_plan({0: [T("recv", 1, "a", 8), T("send", 1, "b", 8)],
                                1: [T("recv", 0, "b", 8), T("send", 0, "a", 8)]})
    with pytest.raises(pc.PlanMismatch, match="outside the group"):
        pc.check_exchange_plan({0: [T("put", 3, "a", 8)], 1: []})


def test_one_sided_plans_of_the_fused_collectives():
    world, rows, rb = 4, [6, 6, 6, 5], 256
    gather = pc.row_gather_plan(world, rows, rb)
    sizes = {(q, "rows"): rows[q] * rb for q in range(world)}
    assert pc.check_exchange_plan(gather, sizes) == world * (world - 1)
    rs = pc.reduce_scatter_plan(world, rows, rb)
    slot_sizes = {(q, "slots"): world * rows[q] * rb for q in range(world)}
    assert pc.check_exchange_plan(rs, slot_sizes) == world * world
    with pytest.raises(pc.PlanMismatch, match="exceeds"):
        pc.check_exchange_plan(rs, {k: v - 1 for k, v in slot_sizes.items()})
    clash = {0: [T("put", 1, "slots", 64, 0)], 1: [], 2: [T("put", 1, "slots", 64, 32)]}
    with pytest.raises(pc.PlanMismatch, match="overlap"):
        pc.check_exchange_plan(clash)


def test_canary_buffer_names_the_overwritten_side():
    b = pc.CanaryBuffer(100)
    b.payload.fill_(7)
    b.check()
    b.raw[b.guard + b.payload.numel()] = 0
    with pytest.raises(pc.PlanMismatch, match="after"):
        b.check("gathered rows")
