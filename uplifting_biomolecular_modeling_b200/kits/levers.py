"""Levers: individually switchable optimisations a mode is made of.

Each lever has a name, a strategy id, the implementation it stands for, and ``apply(model)`` which
returns evidence or raises.  A lever that cannot run raises a cannot-run exception (the mode is
refused by name); a lever the user switched off through ``MODEL_OPT_LEVERS_OFF`` is reported
``state=off``.  Reference: per-kit ``registry.py`` / ``modes.py`` tables and
common/opt_core/opt_core/mem/registry.py:145,201,305.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional

from ..core import arch, gates


@dataclass
class Lever:
    name: str
    strategy: str
    impl: str
    origin: str = "core"
    needs_gpu: bool = False
    apply: Optional[Callable] = None          # (predictor) -> dict of evidence


def _fused(kinds_fn, lever_name):
    def apply(pred):
        import torch
        if pred.device.type != "cuda":
            raise gates.CannotRun(f"{lever_name}: needs a CUDA device")
        sm = arch.device_sm(pred.device.index or 0)
        arch.require(lever_name if arch.declaration(lever_name) else "fused_transition", sm or "sm0")
        from ..models import pairformer
        n = pairformer.set_impl(pred.model, "fused", kinds_fn(), pred.model.workspace)
        pred.model.fused = True
        if n == 0:
            raise gates.CannotRun(f"{lever_name}: the model has no module of this kind")
        return {"modules": n}
    return apply


def _kinds_transition():
    from ..models import pairformer as p
    return (p.Transition,)


def _kinds_trimul():
    from ..models import pairformer as p
    return (p.TriangleMultiplication,)


def _kinds_triatt():
    from ..models import pairformer as p
    return (p.TriangleAttention,)


def _kinds_apb():
    from ..models import pairformer as p
    return (p.AttentionPairBias,)


def _kinds_opm():
    from ..models import msa
    return (msa.OuterProductMean,)


def _kinds_pwa():
    from ..models import msa
    return (msa.PairWeightedAveraging,)


def _kinds_dit():
    from ..models import diffusion
    return (diffusion.DiffusionTransformerLayer,)


def _flag(attr, value=True):
    def apply(pred):
        setattr(pred, attr, value)
        return {attr: value}
    return apply


def _noop(pred):
    return {}


LEVERS: Dict[str, Lever] = {l.name: l for l in [
    Lever("fused_transition", "F1.kernel_fusion", "transition_sm100@1", needs_gpu=True,
          apply=_fused(_kinds_transition, "fused_transition")),
    Lever("fused_trimul", "F1.kernel_fusion", "pair_proj+gemm+trimul_out_sm100@1", needs_gpu=True,
          apply=_fused(_kinds_trimul, "fused_trimul")),
    Lever("fused_triatt", "F1.kernel_fusion", "pair_proj+attention_sm100@1", needs_gpu=True,
          apply=_fused(_kinds_triatt, "fused_triatt")),
    Lever("fused_apb", "F1.kernel_fusion", "attention_sm100@1", needs_gpu=True, apply=_fused(_kinds_apb, "fused_apb")),
    Lever("fused_opm", "F1.kernel_fusion", "gemm_sm100@1", needs_gpu=True, apply=_fused(_kinds_opm, "fused_opm")),
    Lever("fused_pwa", "F1.kernel_fusion", "gemm_sm100@1", needs_gpu=True, apply=_fused(_kinds_pwa, "fused_pwa")),
    Lever("fused_dit", "F1.kernel_fusion", "attention_d64+rows_sm100@1", needs_gpu=True,
          apply=_fused(_kinds_dit, "fused_dit")),
    Lever("bf16_pair_stack", "F4.precision", "models.cofold", apply=_noop),
    Lever("hoist_pair_bias", "F3.hoisting", "models.diffusion.prepare", apply=_noop),
    Lever("hoist_conditioning", "F3.hoisting", "models.diffusion.hoist", apply=_noop),
    Lever("sampler_graph", "F2.graph_capture", "api.Predictor._step_fn", needs_gpu=True, apply=_flag("use_graphs")),
    Lever("segment_mean_det", "F1.kernel_fusion", "models.diffusion.segment_mean", apply=_noop),
    Lever("chunk_pair_ops", "F5.memory", "mem.chunk", apply=_flag("chunk_rows", 256)),
    Lever("release_intermediates", "F5.memory", "mem.release", apply=_flag("release", True)),
    Lever("expandable_segments", "F5.memory", "mem.allocator", apply=_noop),
    Lever("rowpair_tp", "F7.tensor_parallel", "parallel.rowpair", needs_gpu=True, apply=_noop),
    Lever("cond_dedup", "F3.hoisting", "models.design", apply=_noop),
    Lever("attn_bf16", "F4.precision", "attention_sm100@1", needs_gpu=True, apply=_noop),
    Lever("graph_rng", "F2.graph_capture", "capture.rng", apply=_noop),
    Lever("resident_weights", "F6.host_overlap", "models.lm", apply=_noop),
    Lever("forward_graph", "F2.graph_capture", "capture.graphs", needs_gpu=True, apply=_noop),
    Lever("fused_rows", "F1.kernel_fusion", "rows_sm100@1", needs_gpu=True, apply=_noop),
    Lever("tc_gemm", "F1.kernel_fusion", "gemm_sm100@1", needs_gpu=True, apply=_noop),
    Lever("fused_conv", "F1.kernel_fusion", "hyena_sm100@1", needs_gpu=True, apply=_noop),
    Lever("tp_fused", "F7.tensor_parallel", "parallel.tp", needs_gpu=True, apply=_noop),
]}
