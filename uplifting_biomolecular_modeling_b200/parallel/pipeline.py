"""Pipeline parallelism for deep sequence models: the layer stack split over devices, micro-batches of the
sequence batch kept in flight so that every device works while another one's output is in transit.

The reference has one such site (the 40b StripedHyena's two-device layer split with a two-in-flight window on
per-device streams: evo2/opt/evo2_opt/kit/pipelined.py:1-8, kit/multidev.py:1).  Here: ``LayerPipeline`` places
consecutive blocks on a list of devices (one process, several GPUs - activations cross with non-blocking peer
copies on the consumer's stream, ordered by events) and ``forward`` runs ``window`` micro-batches through the
stages in the order of a software pipeline.  On CPU devices the same schedule runs sequentially (tests).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.nn as nn


def split_layers(n_layers: int, n_stages: int, weights: Optional[Sequence[float]] = None) -> List[range]:
    """Contiguous layer ranges per stage, balanced by per-layer cost ``weights`` (default: equal)."""
    w = list(weights) if weights is not None else [1.0] * n_layers
    total, out, start, acc = sum(w), [], 0, 0.0
    for s in range(n_stages):
        target = total * (s + 1) / n_stages
        end = start
        while end < n_layers and (acc + w[end] <= target + 1e-9 or end == start) and n_layers - end > n_stages - 1 - s:
            acc += w[end]
            end += 1
        if s == n_stages - 1:
            end = n_layers
        out.append(range(start, end))
        start = end
    return out


class LayerPipeline:
    def __init__(self, blocks: Sequence[nn.Module], devices: Sequence, weights: Optional[Sequence[float]] = None):
        self.devices = [torch.device(d) for d in devices]
        self.ranges = split_layers(len(blocks), len(self.devices), weights)
        self.stages: List[List[nn.Module]] = []
        for dev, rg in zip(self.devices, self.ranges):
            self.stages.append([blocks[i].to(dev) for i in rg])
        self.streams = [torch.cuda.Stream(d) if d.type == "cuda" else None for d in self.devices]

    def _run_stage(self, s: int, x: torch.Tensor, ready) -> tuple:
        dev, stream = self.devices[s], self.streams[s]
        if stream is None:
            x = x.to(dev)
            for blk in self.stages[s]:
                x = blk(x)
            return x, None
        with torch.cuda.stream(stream):
            if ready is not None:
                stream.wait_event(ready)
            x = x.to(dev, non_blocking=True)
            for blk in self.stages[s]:
                x = blk(x)
            ev = torch.cuda.Event()
            ev.record(stream)
        return x, ev

    @torch.no_grad()
    def forward(self, x: torch.Tensor, window: int = 2) -> torch.Tensor:
        """x: [B, L, d]; the batch is cut into ``window`` micro-batches that travel through the stages one stage
        apart (micro-batch m enters stage s at tick m + s)."""
        micro = list(torch.chunk(x, min(window, x.shape[0]), dim=0))
        S, M = len(self.stages), len(micro)
        act = list(micro)
        ready = [None] * M
        for tick in range(M + S - 1):
            for s in reversed(range(S)):                 # later stages first: they consume last tick's outputs
                m = tick - s
                if 0 <= m < M:
                    act[m], ready[m] = self._run_stage(s, act[m], ready[m])
        last = self.devices[-1]
        if last.type == "cuda":
            for ev in ready:
                if ev is not None:
                    torch.cuda.current_stream(last).wait_event(ev)
        return torch.cat(act, 0)
