"""The kits: one entry per upstream tool the reference ships a kit for (README.md:284-321 of the
reference), re-expressed on this framework's PyTorch model layer.

A :class:`KitSpec` is data: the tag of its lines, the variable that selects its mode, the modes it
ships and its default, which model family serves it, its commands, and whether ``--n_gpu P`` is
offered.  JAX and TensorFlow kits of the reference (af3_jax, colabfold, af2ig, colabdesign, mosaic,
enformer_deepmind, ...) are served by the same PyTorch families here.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

# Every name below is a lever of kits/levers.py whose ``apply`` changes what runs; work that every mode does
# (step-invariant hoists in the sampler, bf16 storage of the pair stack) is not a lever and is not listed.
COFOLD_LEVERS_EXACT = ("sampler_graph", "graph_verify", "trunk_graph")
COFOLD_LEVERS_FAST = ("fused_transition", "fused_trimul", "fused_triatt", "fused_apb", "fused_opm", "fused_pwa",
                      "fused_dit")
COFOLD_LEVERS_BIG = ("chunk_pair_ops", "release_intermediates", "park_pair_init", "expandable_segments", "rowpair_tp")
LM_LEVERS_EXACT = ("kernel_path", "decode_graph", "forward_graph")
LM_LEVERS_FAST = ("tp_fused", "fp8_input_proj")


@dataclass(frozen=True)
class KitSpec:
    name: str
    upstream: str
    family: str                          # cofold | design | evo2 | protein_lm | genomic_track
    modes: Tuple[str, ...]
    default: Optional[str]
    commands: Tuple[str, ...]
    config: str = "af3"                  # model configuration key of the family
    n_gpu: Tuple[int, ...] = (1,)
    library_style: bool = False
    big_token_ceiling: Optional[int] = None   # single-GPU ceiling the reference states (H100 80 GB)
    levers: Dict[str, Tuple[str, ...]] = field(default_factory=dict)

    @property
    def tag(self) -> str:
        return f"{self.name}-opt"

    @property
    def env(self) -> str:
        return f"{self.name.upper()}_OPT"


def _cofold(name, upstream, config="af3", n_gpu=(1, 2, 4, 8), ceiling=None, default="fast", commands=("pred",)):
    return KitSpec(name, upstream, "cofold", ("off", "exact", "fast", "big"), default,
                   ("install", "check") + tuple(commands), config, n_gpu, False, ceiling,
                   {"off": (), "exact": COFOLD_LEVERS_EXACT, "fast": COFOLD_LEVERS_FAST, "big": COFOLD_LEVERS_BIG})


def _design(name, upstream, modes=("off", "exact", "fast"), default="fast", commands=("design",)):
    lv = {"off": (), "exact": ("sampler_graph", "cond_dedup"),
          "fast": ("fused_transition", "fused_trimul", "fused_triatt", "fused_apb", "fused_dit"),
          "big": ("chunk_pair_ops",)}
    return KitSpec(name, upstream, "design", modes, default, ("install", "check") + tuple(commands), "design", (1,),
                   False, None, {m: lv[m] for m in modes})


def _lm(name, upstream, family, modes=("off", "exact"), default="exact", commands=("score",), library=False,
        config="lm", n_gpu=(1,)):
    # only levers that change what this family runs: the decode graph, the tensor-parallel form and the e4m3 input
    # projections belong to StripedHyena-2; the other sequence families take the kernel path and the forward graph
    evo = family == "evo2"
    lv = {"off": (), "exact": LM_LEVERS_EXACT if evo else tuple(l for l in LM_LEVERS_EXACT if l != "decode_graph"),
          "fast": LM_LEVERS_FAST if evo else ()}
    return KitSpec(name, upstream, family, modes, default if not library else None,
                   ("install", "check") + tuple(commands), config, n_gpu, library, None, {m: lv[m] for m in modes})


REGISTRY: Dict[str, KitSpec] = {k.name: k for k in [
    # AF3-family cofolding / structure prediction
    _cofold("boltz2", "Boltz-2 2.2.1", "boltz2", ceiling=3000),
    _cofold("protenix_v2", "Protenix 2.0.0", ceiling=3000),
    _cofold("protenix_v1", "Protenix 1.1.0", ceiling=4000),
    _cofold("openfold3", "OpenFold3 0.4.1", ceiling=6000),
    _cofold("openfold3_ob0", "OpenFold3 0.5.0", ceiling=5000),
    _cofold("af3_torch", "xfold on OpenFold3 weights", ceiling=4000),
    _cofold("af3_jax", "AlphaFold 3 (JAX fork)", ceiling=6000),
    _cofold("chai1", "Chai-1 0.6.1", n_gpu=(1,), ceiling=2000),
    _cofold("opendde", "OpenDDE 1.1.1", ceiling=4000),
    _cofold("esmfold2", "ESMFold2", ceiling=3000),
    _cofold("rosettafold3", "RoseTTAFold 3 (foundry)", ceiling=4000),
    _cofold("colabfold", "ColabFold / AF2-multimer v3", ceiling=4000),
    _cofold("af2ig", "AF2 initial guess", n_gpu=(1,), ceiling=3000),
    _cofold("atlasfold", "AtlasFold", n_gpu=(1,), ceiling=4000, default="off"),
    # design tools
    _design("colabdesign", "ColabDesign", ("off", "exact", "fast", "big")),
    _design("mosaic", "mosaic / joltz", ("off", "exact", "fast", "big")),
    _design("boltzgen", "BoltzGen"), _design("complexa", "Complexa"), _design("pxdesign", "PXDesign"),
    _design("genie3", "Genie 3"), _design("rfdiffusion1", "RFdiffusion"), _design("rfdiffusion3", "RFdiffusion3"),
    _design("caliby", "Caliby"), _design("esm_if1", "ESM-IF1", ("off", "exact"), "exact"),
    _design("ef2inv", "ESMFold2 inversion"),
    KitSpec("proteinmpnn", "ProteinMPNN", "design", ("off", "exact", "fast"), None, ("install", "check", "design"),
            "design", (1,), False, None, {"off": (), "exact": ("cond_dedup",), "fast": ()}),
    # genomic / protein language models
    _lm("evo2", "Evo 2 7b/40b (StripedHyena-2)", "evo2", ("off", "exact", "fast"), "exact", ("score", "generate"),
        config="evo2_7b", n_gpu=(1, 2, 4, 8)),
    _lm("esmc", "ESM C", "protein_lm", library=True), _lm("e1", "E1", "protein_lm"),
    _lm("progen2", "ProGen2", "protein_lm", commands=("generate",)),
    _lm("gpnstar", "GPN-Star", "protein_lm", library=True),
    # genomic track models
    _lm("enformer", "Enformer (PyTorch)", "genomic_track", ("off", "exact", "fast"), library=True, commands=("predict",)),
    _lm("enformer_deepmind", "Enformer (DeepMind TF)", "genomic_track", library=True, commands=("predict",)),
    _lm("borzoi", "Borzoi", "genomic_track", commands=("predict",)),
    _lm("flashzoi", "Flashzoi", "genomic_track", ("off", "exact", "fast"), library=True, commands=("predict",)),
    _lm("chrombpnet", "ChromBPNet", "genomic_track", ("off", "exact", "fast"), commands=("predict",)),
]}


def get(name: str) -> KitSpec:
    try:
        return REGISTRY[name]
    except KeyError:
        raise KeyError(f"unknown kit {name!r}; known: {', '.join(sorted(REGISTRY))}") from None


def names():
    return sorted(REGISTRY)
