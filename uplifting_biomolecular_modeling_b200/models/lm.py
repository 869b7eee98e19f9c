"""Sequence-model families behind the language-model and genomic-track kits (``score`` / ``generate`` /
``predict`` verbs): ``evo2`` is the StripedHyena-2 decoder of :mod:`models.evo2`, the protein / DNA language
models (ESM-C, E1, ProGen2, GPN-Star) live in :mod:`models.plm`, the genomic track models (Enformer, Borzoi,
Flashzoi, ChromBPNet) in :mod:`models.genomics`.  ``build`` returns a runner with one ``run(verb, prompt)``
method so the kit command line does not depend on the family."""
from __future__ import annotations

import torch

from . import evo2, genomics, plm


class _Runner:
    def __init__(self, model, device, mode):
        self.model, self.device, self.mode = model, device, mode
        self.draft = None                 # a smaller model of the family: generate() then decodes speculatively
        self.specdec_k = 0
        self.decode_graph = False         # the ``decode_graph`` lever: replay the decode step from a CUDA graph
        self.forward_graphs = None        # the ``forward_graph`` lever: a capture site (``run(fn, *tensors)``)
        self.forward_graph_max_tokens = 16384

    def run(self, verb: str, prompt: str, max_new_tokens: int = 32) -> dict:
        toks = evo2.tokenize(prompt, self.device)
        if verb == "generate":
            extra = {}
            if self.draft is not None and self.specdec_k > 0:
                out, stats = self.model.generate_speculative(self.draft, toks, max_new_tokens, k=self.specdec_k)
                extra = {"specdec_rounds": stats["rounds"], "specdec_accepted": stats["accepted"],
                         "specdec_proposed": stats["proposed"]}
            else:
                out = self.model.generate(toks, max_new_tokens, graph=self.decode_graph)
            return {"new_tokens": int(out.shape[1]), "text": "".join(chr(int(t)) if 32 <= int(t) < 127 else "?"
                                                                      for t in out[0].tolist()), **extra}
        if verb in ("score", "predict"):
            return {"score": float(self._score(toks)[0]), "tokens": int(toks.shape[1])}
        raise ValueError(f"unknown verb {verb!r}")

    def _score(self, toks, **kw):
        """``model.score`` - through the capture site for GPU inputs of a recurring shape that is small enough."""
        if self.forward_graphs is not None and toks.is_cuda and not kw and toks.shape[1] <= self.forward_graph_max_tokens:
            return self.forward_graphs.run(lambda t: self.model.score(t), toks)
        return self.model.score(toks, **kw)


class _PLMRunner(_Runner):
    def run(self, verb: str, prompt: str, max_new_tokens: int = 32) -> dict:
        cfg = self.model.cfg
        toks = plm.tokenize(prompt, cfg, self.device)
        kw = {}
        if cfg.family == "gpnstar":
            align, index = plm.synthetic_alignment(cfg, toks)
            kw = {"alignment": align, "clade_index": index}
        if verb == "generate":
            out = self.model.generate(toks, max_new_tokens)
            letters = plm.AMINO
            return {"new_tokens": int(out.shape[1] - toks.shape[1]),
                    "text": "".join(letters[int(t) - 4] if 4 <= int(t) < 4 + len(letters) else "X"
                                    for t in out[0].tolist())}
        if verb in ("score", "predict", "embedding", "logits", "vep"):
            res = {"score": float(self._score(toks, **kw)[0]), "tokens": int(toks.shape[1])}
            if verb == "vep" and cfg.family == "gpnstar":
                res["vep_min"] = float(self.model.variant_effect(toks, **kw).min())
            return res
        raise ValueError(f"unknown verb {verb!r}")


class _TrackRunner(_Runner):
    def run(self, verb: str, prompt: str, max_new_tokens: int = 32) -> dict:
        if verb not in ("predict", "score"):
            raise ValueError(f"unknown verb {verb!r}")
        cfg = self.model.cfg
        need = genomics.input_length(cfg)
        text = (prompt * (need // max(1, len(prompt)) + 1))[:need]
        x = genomics.one_hot_dna(text, self.device, next(self.model.parameters()).dtype)
        with torch.no_grad():
            if self.forward_graphs is not None and x.is_cuda:
                # the window length is fixed, so every call after the first has the same shape: captured at the second
                # sighting, replayed afterwards (the ``forward_graph`` lever)
                out = self.forward_graphs.run(lambda t: self.model(t), x)
            else:
                out = self.model(x)
        if cfg.family == "chrombpnet":
            prof, counts = out
            # kept for the kit's track writer: base-pair profile of the window, one column
            self.last_tracks, self.last_bin_size = prof[0].reshape(-1, 1), 1
            return {"score": float(counts[0]), "bins": int(prof.shape[1]), "tokens": need}
        self.last_tracks = out[0]                                              # [bins, tracks]
        self.last_bin_size = 2 ** (cfg.tower + 1)                              # base pairs per output bin
        return {"score": float(out.mean()), "bins": int(out.shape[1]), "tracks": int(out.shape[2]), "tokens": need}


DRAFT_OF = {"evo2_7b": "evo2_1b", "evo2_1b": "evo2_tiny", "evo2_tiny": "evo2_tiny"}


def build(family: str, config: str, device="cpu", mode: str = "exact", seed: int = 0, kit: str = "",
          specdec: int = 0) -> _Runner:
    """``family`` is the kit's model family (evo2 | protein_lm | genomic_track), ``kit`` its name (which model of the
    family), ``config`` a configuration key of that model (unknown keys fall back to the model's small default)."""
    dtype = torch.bfloat16 if str(device).startswith("cuda") else torch.float32
    if family == "protein_lm" or kit in plm.DEFAULT:
        name = config if config in plm.CONFIGS else plm.DEFAULT.get(kit, "esmc_tiny")
        impl = "reference" if mode == "off" else None
        return _PLMRunner(plm.build(name, device=device, dtype=dtype, seed=seed, impl=impl), device, mode)
    if family == "genomic_track" or kit in genomics.DEFAULT:
        name = config if config in genomics.CONFIGS else genomics.DEFAULT.get(kit, "enformer_tiny")
        impl = "reference" if mode == "off" else None
        return _TrackRunner(genomics.build(name, device=device, dtype=dtype, seed=seed, impl=impl), device, mode)
    cfg = config if config in evo2.CONFIGS else "evo2_tiny"
    m = evo2.build(cfg, device=device, dtype=dtype, seed=seed)
    r = _Runner(m, device, mode)
    if specdec > 0:
        # ``specdec`` k > 0: the family's next smaller configuration proposes k tokens per round (greedy output is
        # unchanged; see StripedHyena2.generate_speculative)
        r.draft = evo2.build(DRAFT_OF.get(cfg, "evo2_tiny"), device=device, dtype=dtype, seed=seed + 1)
        r.specdec_k = specdec
    return r
