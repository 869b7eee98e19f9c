"""Checkpoint names of upstream Pairformer stacks -> this package's parameter names.

This package's trunk modules carry Boltz-2's parameter names (a Boltz-2 ``state_dict`` loads with ``strict=True``).
Other upstreams of the AF3 family hold the same tensors under other names and, for the triangle multiplication,
split over more matrices.  A mapper renames and merges them; what it does not know it leaves untouched, so a strict
load still fails loudly on anything unexpected.

Name sources (read as text, nothing is imported from them):

* Protenix: ``protenix/model/modules/pairformer.py`` (``PairformerBlock``: ``tri_mul_out/in``, ``tri_att_start/end``,
  ``pair_transition``, ``attention_pair_bias``, ``single_transition``; ``PairformerStack.blocks``),
  ``protenix/model/triangular/triangular.py`` (``linear_a_p / linear_a_g / linear_b_p / linear_b_g / linear_g /
  linear_z``, ``layer_norm_in / layer_norm_out``; ``TriangleAttention``: ``layer_norm``, ``linear``, ``mha.linear_*``),
  ``protenix/model/modules/primitives.py`` (``Transition``: ``layernorm1``, ``linear_no_bias_a / _b``,
  ``linear_no_bias``), ``protenix/model/modules/transformer.py`` (``AttentionPairBias``: ``layernorm_a``,
  ``layernorm_z``, ``linear_nobias_z``, ``attention.linear_q / k / v / g / o``).
* OpenFold3: ``openfold3/core/model/latent/pairformer.py`` (``PairFormerBlock``: ``pair_stack``, ``attn_pair_bias``,
  ``single_transition``), ``latent/base_blocks.py`` (``PairBlock``), ``layers/triangular_multiplicative_update.py``,
  ``layers/triangular_attention.py`` (bias projection ``linear_z``), ``layers/transition.py`` (``SwiGLUTransition``:
  ``layer_norm``, ``swiglu.linear_a / linear_b``, ``linear_out``), ``layers/attention_pair_bias.py``
  (``layer_norm_a``, ``layer_norm_z``, ``linear_z``, ``mha.linear_*``).

Semantics held by the merge: the first half of ``p_in`` / ``g_in`` is the ``a`` operand, the second half ``b``
(``models/pairformer.py`` chunks the gated projection in that order); ``fc1`` of a transition is the SiLU branch.
"""
from __future__ import annotations

import re
from typing import Callable, Dict, List, Optional, Tuple

import torch

State = Dict[str, torch.Tensor]


class MapperError(ValueError):
    """A block of the upstream checkpoint is incomplete (one of the matrices to merge is absent)."""


def _trimul(prefix_src: str, prefix_dst: str, st: State, out: State, used: set) -> None:
    """One triangle multiplication: four operand matrices -> two stacked ones; names of the rest."""
    def take(name):
        k = prefix_src + name
        if k not in st:
            raise MapperError(f"{k} is missing from the checkpoint")
        used.add(k)
        return st[k]

    out[prefix_dst + "p_in.weight"] = torch.cat([take("linear_a_p.weight"), take("linear_b_p.weight")], 0)
    out[prefix_dst + "g_in.weight"] = torch.cat([take("linear_a_g.weight"), take("linear_b_g.weight")], 0)
    out[prefix_dst + "p_out.weight"] = take("linear_z.weight")
    out[prefix_dst + "g_out.weight"] = take("linear_g.weight")
    for src, dst in (("layer_norm_in", "norm_in"), ("layer_norm_out", "norm_out")):
        for leaf in ("weight", "bias"):
            out[prefix_dst + f"{dst}.{leaf}"] = take(f"{src}.{leaf}")


def _rename(prefix_src: str, prefix_dst: str, table: List[Tuple[str, str]], st: State, out: State, used: set,
            optional: Tuple[str, ...] = ()) -> None:
    for src, dst in table:
        k = prefix_src + src
        if k in st:
            out[prefix_dst + dst] = st[k]
            used.add(k)
        elif src.endswith(".bias") and k[:-len("bias")] + "weight" in st and st[k[:-len("bias")] + "weight"].dim() == 1:
            # a LayerNorm built without its offset: the same function as one with a zero offset
            out[prefix_dst + dst] = torch.zeros_like(st[k[:-len("bias")] + "weight"])
        elif src not in optional:
            raise MapperError(f"{k} is missing from the checkpoint")


_LN = lambda a, b: [(f"{a}.weight", f"{b}.weight"), (f"{a}.bias", f"{b}.bias")]   # noqa: E731

_TRIATT_COMMON = [(f"mha.linear_{x}.weight", f"mha.linear_{x}.weight") for x in "qkvog"] + _LN("layer_norm", "layer_norm")

_PROTENIX = {
    "triatt": _TRIATT_COMMON + [("linear.weight", "linear.weight")],
    "transition": _LN("layernorm1", "norm") + [("linear_no_bias_a.weight", "fc1.weight"),
                                               ("linear_no_bias_b.weight", "fc2.weight"),
                                               ("linear_no_bias.weight", "fc3.weight")],
    "apb_src": "attention_pair_bias.",
    "apb": [("attention.linear_q.weight", "attention.proj_q.weight"), ("attention.linear_q.bias", "attention.proj_q.bias"),
            ("attention.linear_k.weight", "attention.proj_k.weight"), ("attention.linear_v.weight", "attention.proj_v.weight"),
            ("attention.linear_g.weight", "attention.proj_g.weight"), ("attention.linear_o.weight", "attention.proj_o.weight"),
            ("linear_nobias_z.weight", "attention.proj_z.1.weight")]
           + _LN("layernorm_z", "attention.proj_z.0") + _LN("layernorm_a", "pre_norm_s"),
    "pair_prefix": "",
}

_OPENFOLD3 = {
    "triatt": _TRIATT_COMMON + [("linear_z.weight", "linear.weight")],
    "transition": _LN("layer_norm", "norm") + [("swiglu.linear_a.weight", "fc1.weight"),
                                               ("swiglu.linear_b.weight", "fc2.weight"),
                                               ("linear_out.weight", "fc3.weight")],
    "apb_src": "attn_pair_bias.",
    "apb": [("mha.linear_q.weight", "attention.proj_q.weight"), ("mha.linear_q.bias", "attention.proj_q.bias"),
            ("mha.linear_k.weight", "attention.proj_k.weight"), ("mha.linear_v.weight", "attention.proj_v.weight"),
            ("mha.linear_g.weight", "attention.proj_g.weight"), ("mha.linear_o.weight", "attention.proj_o.weight"),
            ("linear_z.weight", "attention.proj_z.1.weight")]
           + _LN("layer_norm_z", "attention.proj_z.0") + _LN("layer_norm_a", "pre_norm_s"),
    "pair_prefix": "pair_stack.",
}

UPSTREAMS = {"protenix": _PROTENIX, "openfold3": _OPENFOLD3}


def map_pairformer_block(st: State, upstream: str, src: str, dst: str, out: State, used: set,
                         with_single: Optional[bool] = None) -> None:
    """One block: keys under ``src`` (upstream names) -> keys under ``dst`` (this package's).  ``with_single`` None:
    the single track is mapped when the block has one."""
    spec = UPSTREAMS[upstream]
    pp = src + spec["pair_prefix"]
    _trimul(pp + "tri_mul_out.", dst + "tri_mul_out.", st, out, used)
    _trimul(pp + "tri_mul_in.", dst + "tri_mul_in.", st, out, used)
    _rename(pp + "tri_att_start.", dst + "tri_att_start.", spec["triatt"], st, out, used)
    _rename(pp + "tri_att_end.", dst + "tri_att_end.", spec["triatt"], st, out, used)
    _rename(pp + "pair_transition.", dst + "transition_z.", spec["transition"], st, out, used)
    has_single = any(k.startswith(src + spec["apb_src"]) for k in st)
    if with_single is None:
        with_single = has_single
    if with_single:
        _rename(src + spec["apb_src"], dst, spec["apb"], st, out, used)
        _rename(src + "single_transition.", dst + "transition_s.", spec["transition"], st, out, used)


def map_pairformer_stack(state: State, upstream: str, src_prefix: str = "", dst_prefix: str = "") -> State:
    """Every ``<src_prefix>blocks.<i>.`` of an upstream Pairformer stack -> ``<dst_prefix>layers.<i>.``.  Keys outside
    the stack (and keys of a block that the tables do not name, e.g. a bias this package has no parameter for) are
    passed through unchanged, so a strict load reports them."""
    if upstream not in UPSTREAMS:
        raise KeyError(f"unknown upstream {upstream!r}; known: {sorted(UPSTREAMS)}")
    pat = re.compile(re.escape(src_prefix) + r"blocks\.(\d+)\.")
    blocks = sorted({int(m.group(1)) for k in state for m in [pat.match(k)] if m})
    out: State = {}
    used: set = set()
    for i in blocks:
        map_pairformer_block(state, upstream, f"{src_prefix}blocks.{i}.", f"{dst_prefix}layers.{i}.", out, used)
    for k, v in state.items():
        if k not in used:
            out.setdefault(k, v)
    return out


# the trunk's Pairformer stack inside the whole-model checkpoints: (upstream prefix, this package's prefix)
TRUNK_PREFIX = {"protenix": ("pairformer_stack.", "pairformer_module."),
                "openfold3": ("pairformer_stack.", "pairformer_module.")}

KIT_UPSTREAM = {"protenix_v1": "protenix", "protenix_v2": "protenix", "pxdesign": "protenix",
                "openfold3": "openfold3", "openfold3_ob0": "openfold3"}


def for_kit(kit: str) -> Optional[Callable[[State], State]]:
    """The checkpoint mapper of a cofold kit, or None for the kits whose checkpoints carry this package's names
    (Boltz-2 and the kits served by the same model under their own descriptor)."""
    up = KIT_UPSTREAM.get(kit)
    if up is None:
        return None
    src, dst = TRUNK_PREFIX[up]
    return lambda state: map_pairformer_stack(state, up, src, dst)
