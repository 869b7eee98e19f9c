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
    droppable: bool = False                   # a refusal of this lever leaves the mode whole (reported, not PARTIAL)


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
    apply.__doc__ = ("Switches the model's modules of this kind to their sm_100a kernel implementation; every call is "
                     "then counted served or fallback in the lever's ledger.")
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


def _flag(attr, value=True, doc=""):
    def apply(pred):
        setattr(pred, attr, value)
        return {attr: value}
    apply.__doc__ = doc
    return apply


def _expandable(pred):
    """Allocator policy of ``big``: expandable segments requested and read back (a process whose allocator already
    runs without them reports ``skipped`` with the reason; the lever is droppable)."""
    from ..mem import allocator
    ok = allocator.want_expandable()
    live = allocator.verify_expandable()
    if live is False:
        raise RuntimeError("allocator_already_initialised_without_expandable_segments")
    return {"requested": ok, "verified": live}


def _chunk_pair_ops(pred):
    """Pair operations of the kernel path run in row blocks: the triangle-attention q|k|v|gate|o rows and the
    contracted planes of the triangle multiplication exist for one block of rows at a time."""
    rows = int(getattr(pred, "row_block", 0) or 512)
    pred.row_block = rows
    pred.model.workspace["row_block"] = rows
    return {"row_block": rows}


def _release(pred):
    """The trunk's scratch buffers are returned to the allocator before the sampler starts."""
    pred.release = True
    return {"release": True}


def _park_pair_init(pred):
    """The initial pair tensor waits in pinned host memory between recycling passes (one fetch per pass)."""
    pred.model.park_z_init = True
    return {"park_z_init": True}


def _rowpair(pred):
    """Row-sharded prediction over the ranks of ``--n_gpu P`` (the activation hands the run to the launcher)."""
    import torch
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    want = int(getattr(pred, "n_gpu", 1) or 1)
    if want > 1 and n < want:
        raise gates.CannotRun(f"rowpair_tp: {want} GPUs requested, {n} visible")
    pred.sharding = "rowpair"
    return {"visible_gpus": n, "n_gpu": want}


def _graph_verify(pred):
    """The first replay of every captured graph is compared bit for bit with the eager step on the same inputs."""
    pred.verify_graphs = 1
    return {"verify": 1}


def _trunk_graph(pred):
    """Pairformer stack passes of small inputs replay from a CUDA graph (capture once per shape, first replay
    verified against eager, byte budget on the static buffers)."""
    from ..capture import pool
    gp = getattr(pred, "graph_pool", None)
    if gp is None:
        gp = pred.graph_pool = pool.GraphPool(budget_bytes=4 << 30, default_policy=pool.FixedK(2))
    gp.site("pairformer_stack", verify=1)
    pred.model.trunk_graphs = gp.handle("pairformer_stack")
    return {"max_tokens": pred.model.trunk_graph_max_tokens, "site": "pairformer_stack"}


def _cond_dedup(pred):
    """Design batches share one trunk pass and one set of step-invariant sampler tensors."""
    pred.cond_dedup = True
    return {"cond_dedup": True}


def _kernel_path(pred):
    """Sequence models: row kernels, tcgen05 GEMMs and the convolution kernels replace the plain statements."""
    import torch
    model = getattr(pred, "model", None)
    if model is None or not hasattr(model, "set_impl"):
        raise gates.CannotRun("kernel_path: no switchable model")
    if not torch.cuda.is_available():
        raise gates.CannotRun("kernel_path: needs a CUDA device")
    model.set_impl("fused")
    return {"impl": "fused"}


def _decode_graph(pred):
    """Generation: the decode step is captured once and replayed per token."""
    pred.decode_graph = True
    return {"decode_graph": True}


def _forward_graph(pred):
    """Scoring: the forward of a recurring input shape (at most ``forward_graph_max_tokens`` tokens) is captured at
    its second sighting and replayed afterwards; the first replay is compared with the eager result."""
    from ..capture import pool
    gp = getattr(pred, "graph_pool", None)
    if gp is None:
        gp = pred.graph_pool = pool.GraphPool(budget_bytes=8 << 30, default_policy=pool.FixedK(2))
    gp.site("score_forward", verify=1)
    pred.forward_graphs = gp.handle("score_forward")
    return {"max_tokens": pred.forward_graph_max_tokens, "site": "score_forward"}


def _fp8_input_proj(pred):
    """StripedHyena-2 prefill: the input projections of the Hyena operators run in e4m3 (upstream's fp8 input
    projections): RMSNorm emits 8-bit rows scaled by their maximum, the weights are quantised once."""
    import torch
    model = getattr(pred, "model", None)
    if model is None or not hasattr(model, "set_fp8_input_projections"):
        raise gates.CannotRun("fp8_input_proj: the model has no Hyena operators")
    if not torch.cuda.is_available():
        raise gates.CannotRun("fp8_input_proj: needs a CUDA device")
    return {"operators": model.set_fp8_input_projections(True)}


def _tp_fused(pred):
    """Tensor parallelism of the sequence models with the collectives fused into the GEMM kernels.  It engages in the
    rank processes that ``--n_gpu P`` starts (``parallel.lm_worker``); a single-process run has nothing to shard."""
    raise RuntimeError("single_process_run_needs_--n_gpu_above_1")


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
    Lever("sampler_graph", "F2.graph_capture", "api.Predictor._step_fn", needs_gpu=True, apply=_flag("use_graphs", True, "The sampler step is captured once per shape in a CUDA graph and replayed for every "
                                            "step and every later prediction.")),
    Lever("graph_verify", "F2.graph_capture", "capture.graphs.verify", needs_gpu=True, apply=_graph_verify),
    Lever("trunk_graph", "F2.graph_capture", "capture.graphs.GraphCache", needs_gpu=True, apply=_trunk_graph),
    Lever("chunk_pair_ops", "F5.memory", "models.pairformer.row_blocks", apply=_chunk_pair_ops),
    Lever("release_intermediates", "F5.memory", "api.Predictor.release", apply=_release),
    Lever("park_pair_init", "F5.memory", "mem.offload.HostPark", apply=_park_pair_init),
    Lever("expandable_segments", "F5.memory", "mem.allocator", apply=_expandable, droppable=True),
    Lever("rowpair_tp", "F7.tensor_parallel", "parallel.rowpair", needs_gpu=True, apply=_rowpair),
    Lever("cond_dedup", "F3.hoisting", "models.design.DesignPipeline", apply=_cond_dedup),
    Lever("kernel_path", "F1.kernel_fusion", "rows+gemm+seq_sm100@1", needs_gpu=True, apply=_kernel_path),
    Lever("decode_graph", "F2.graph_capture", "models.evo2.generate", needs_gpu=True, apply=_decode_graph),
    Lever("forward_graph", "F2.graph_capture", "capture.pool.GraphPool", needs_gpu=True, apply=_forward_graph),
    Lever("fp8_input_proj", "F4.precision", "gemm_sm100.f8f6f4+seq_sm100.rmsnorm_fp8@1", needs_gpu=True,
          apply=_fp8_input_proj, droppable=True),
    Lever("tp_fused", "F7.tensor_parallel", "parallel.tp", needs_gpu=True, apply=_tp_fused, droppable=True),
]}
