"""Writers for genomic track predictions: bedGraph text (the plain-text sibling of bigWig: one
``chrom start end value`` line per run of equal values) and ``.npy`` arrays, submitted to a background writer so
that post-processing of one window overlaps the forward of the next.  Reference: the genomics kits' pipelined
post-processing and their bigWig / HDF5 writer re-implementations (enformer / borzoi / chrombpnet CHANGES)."""
from __future__ import annotations

import os
from typing import Optional, Sequence

import numpy as np
import torch

from .outputs import AsyncWriter


def bedgraph_lines(chrom: str, start: int, bin_size: int, values: Sequence[float], precision: int = 5):
    """Run-length merged bedGraph records for consecutive bins starting at ``start``."""
    v = np.asarray(values, dtype=np.float64).round(precision)
    if v.size == 0:
        return []
    cut = np.flatnonzero(np.diff(v) != 0) + 1
    starts = np.concatenate([[0], cut])
    ends = np.concatenate([cut, [v.size]])
    return [f"{chrom}\t{start + int(s) * bin_size}\t{start + int(e) * bin_size}\t{v[s]:.{precision}g}"
            for s, e in zip(starts, ends)]


def write_bedgraph(path: str, chrom: str, start: int, bin_size: int, values, track_name: Optional[str] = None,
                   append: bool = False) -> int:
    lines = bedgraph_lines(chrom, start, bin_size, values)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "a" if append else "w") as f:
        if track_name and not append:
            f.write(f'track type=bedGraph name="{track_name}"\n')
        f.write("\n".join(lines) + ("\n" if lines else ""))
    return len(lines)


class TrackWriter:
    """``submit(chrom, start, tracks)`` with tracks [bins, n_tracks] (tensor or array): the chosen track columns go
    to ``<out_dir>/track_<k>.bedGraph`` (appended window by window) and, when ``save_arrays``, the whole window to
    ``<out_dir>/<chrom>_<start>.npy`` - on a writer thread."""

    def __init__(self, out_dir: str, bin_size: int, columns: Sequence[int] = (0,), save_arrays: bool = False):
        self.out_dir, self.bin_size, self.columns, self.save_arrays = out_dir, bin_size, tuple(columns), save_arrays
        os.makedirs(out_dir, exist_ok=True)
        self._started = set()
        self.records = 0
        self._writer = AsyncWriter(self._write, workers=1, depth=4)

    def _write(self, item) -> None:
        chrom, start, arr = item
        for k in self.columns:
            path = os.path.join(self.out_dir, f"track_{k}.bedGraph")
            self.records += write_bedgraph(path, chrom, start, self.bin_size, arr[:, k], f"track_{k}",
                                           append=path in self._started)
            self._started.add(path)
        if self.save_arrays:
            np.save(os.path.join(self.out_dir, f"{chrom}_{start}.npy"), arr)

    def submit(self, chrom: str, start: int, tracks) -> None:
        arr = tracks.detach().float().cpu().numpy() if isinstance(tracks, torch.Tensor) else np.asarray(tracks)
        self._writer.submit((chrom, start, arr))

    def close(self) -> int:
        self._writer.drain()
        return self.records
