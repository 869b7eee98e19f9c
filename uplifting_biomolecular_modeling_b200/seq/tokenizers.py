"""Byte -> row lookup tokenisers: a 256-entry table maps every byte of the input to its vocabulary row, so that
tokenising a sequence is one ``frombuffer`` and one gather (no per-character Python loop)."""
from __future__ import annotations

from typing import Mapping, Optional

import torch


class ByteLUT:
    def __init__(self, alphabet: Mapping[str, int], unknown: Optional[int] = None, fold_case: bool = True):
        lut = torch.full((256,), -1 if unknown is None else unknown, dtype=torch.long)
        for ch, row in alphabet.items():
            b = ch.encode("latin-1")
            if len(b) != 1:
                raise ValueError(f"alphabet entry {ch!r} is not a single byte")
            lut[b[0]] = row
            if fold_case:
                lut[ord(ch.lower())] = row
                lut[ord(ch.upper())] = row
        self.lut = lut

    def encode(self, text: str, device="cpu") -> torch.Tensor:
        raw = torch.frombuffer(bytearray(text.encode("latin-1")), dtype=torch.uint8).long()
        ids = self.lut[raw]
        if (ids < 0).any():
            bad = text[int((ids < 0).nonzero()[0])]
            raise ValueError(f"character {bad!r} is not in the alphabet")
        return ids.to(device)


DNA = ByteLUT({"A": 0, "C": 1, "G": 2, "T": 3, "N": 4}, unknown=4)
