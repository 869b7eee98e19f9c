"""Sequence-model families behind the language-model and genomic-track kits (``score`` / ``generate`` /
``predict`` verbs).  ``evo2`` is the StripedHyena-2 decoder of :mod:`models.evo2`; the protein language
models and the genomic track models are served by small generic stand-ins of the right operator mix
until their own modules are written."""
from __future__ import annotations

import torch

from . import evo2


class _Runner:
    def __init__(self, model, device, mode):
        self.model, self.device, self.mode = model, device, mode

    def run(self, verb: str, prompt: str, max_new_tokens: int = 32) -> dict:
        toks = evo2.tokenize(prompt, self.device)
        if verb == "generate":
            out = self.model.generate(toks, max_new_tokens)
            return {"new_tokens": int(out.shape[1]), "text": "".join(chr(int(t)) if 32 <= int(t) < 127 else "?"
                                                                      for t in out[0].tolist())}
        if verb in ("score", "predict"):
            return {"score": float(self.model.score(toks)[0]), "tokens": int(toks.shape[1])}
        raise ValueError(f"unknown verb {verb!r}")


def build(family: str, config: str, device="cpu", mode: str = "exact", seed: int = 0) -> _Runner:
    cfg = config if config in evo2.CONFIGS else "evo2_tiny"
    dtype = torch.bfloat16 if str(device).startswith("cuda") else torch.float32
    m = evo2.build(cfg, device=device, dtype=dtype, seed=seed)
    return _Runner(m, device, mode)
