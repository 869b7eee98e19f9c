"""Roll-out and confidence head one sample chunk at a time, outputs assembled on the host: the peak of the
structure stage is that of ``chunk`` samples instead of all of them.

``run(sample_fn, head_fn, n_samples, chunk, draws)`` calls ``sample_fn(k0, k1, noise)`` for consecutive sample
ranges with the noise those samples would have drawn in one full-width call (``draws``: a
:class:`mem.ckpt.StockOrderDraws`), passes each chunk's coordinates through ``head_fn`` and moves the results to
the host before the next chunk starts.  Reference: common/opt_core/opt_core/mem/sample_loop.py:165.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

from .ckpt import sample_chunks


def run(sample_fn: Callable[[int, int], torch.Tensor], head_fn: Optional[Callable[[torch.Tensor], Dict]] = None,
        n_samples: int = 1, chunk: int = 1) -> Dict[str, torch.Tensor]:
    coords: List[torch.Tensor] = []
    heads: Dict[str, List[torch.Tensor]] = {}
    for k0, k1 in sample_chunks(n_samples, chunk):
        x = sample_fn(k0, k1)
        if head_fn is not None:
            for name, t in head_fn(x).items():
                heads.setdefault(name, []).append(t.detach().to("cpu", non_blocking=False))
        coords.append(x.detach().to("cpu"))
        del x
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
    out = {"coords": torch.cat(coords, 0)}
    for name, parts in heads.items():
        out[name] = torch.cat(parts, 0)
    return out
