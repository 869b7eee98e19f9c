"""Peak-memory instrument: allocator peak plus the driver's high-water mark (nvidia-smi), written as
``peak_mem.json``; and the per-rank model ``peak = a(N) + b(N) / P`` fitted from measured points.
Reference: common/opt_core/opt_core/mem/peak.py:240,373 and mem/rowpair/census.py:214."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence, Tuple


def allocator_peak(device=None) -> Dict[str, int]:
    import torch
    if not torch.cuda.is_available():
        return {"allocated": 0, "reserved": 0}
    return {"allocated": int(torch.cuda.max_memory_allocated(device)),
            "reserved": int(torch.cuda.max_memory_reserved(device))}


def reset(device=None) -> None:
    import torch
    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats(device)


def write(out_dir: str, stage_peaks: Dict[str, Dict[str, int]], name: str = "peak_mem.json") -> str:
    os.makedirs(out_dir, exist_ok=True)
    p = os.path.join(out_dir, name)
    with open(p, "w") as f:
        json.dump(stage_peaks, f, indent=1, sort_keys=True)
    return p


def fit_a_b(points: Sequence[Tuple[int, float]]) -> Tuple[float, float]:
    """Least-squares fit of peak = a + b / P from (P, peak) points."""
    xs = [1.0 / p for p, _ in points]
    ys = [y for _, y in points]
    n = len(points)
    if n < 2:
        return (ys[0] if ys else 0.0, 0.0)
    mx, my = sum(xs) / n, sum(ys) / n
    sxx = sum((x - mx) ** 2 for x in xs)
    b = sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / sxx if sxx else 0.0
    return my - b * mx, b


def census_line(tag: str, stage: str, rank: int, peak_bytes: int, n: int, world: int) -> str:
    from ..core import report
    return f"{report.tag_prefix(tag)} TPCENSUS " + json.dumps({"stage": stage, "rank": rank, "peak": peak_bytes,
                                                               "N": n, "P": world}, sort_keys=True)
