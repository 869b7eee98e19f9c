"""RNG discipline around captured and batched sampling steps: the same draws as the plain loop.

(1) Warm-up does not move the stream: :func:`generator_checkpoint` snapshots the state of every generator it is
    given and restores it on exit, so the warm-up a CUDA-graph capture requires consumes no draws the plain loop
    would have made.
(2) The capture contract is declared: ``RNG_NONE`` (no draw inside the captured region), ``RNG_OUTSIDE`` (draws
    stay outside: noise is an input of the captured step), ``RNG_REGISTERED`` (the generator is registered with
    the graph so replays advance it).  :func:`capture_contract_gate` refuses an undeclared contract and modules
    left in training mode (dropout draws).
(3) Batched items draw what they would have drawn alone: :func:`fork_at_offsets` positions one generator per
    item at the Philox offset its first draw has in the plain order; :func:`philox_increment` measures the
    offset one unit of the plain loop consumes.
Reference: common/opt_core/opt_core/diffusion_loop/rng.py, mem/ckpt.py:318 (StockOrderDraws).
"""
from __future__ import annotations

import contextlib
from typing import Callable, Iterable, List, Optional, Sequence

import torch

from ..core.gates import Gate

RNG_NONE, RNG_OUTSIDE, RNG_REGISTERED = "none", "outside", "registered"
CONTRACTS = (RNG_NONE, RNG_OUTSIDE, RNG_REGISTERED)


def default_generator(device=None) -> torch.Generator:
    if device is None or torch.device(device).type == "cpu":
        return torch.default_generator
    idx = torch.device(device).index
    return torch.cuda.default_generators[torch.cuda.current_device() if idx is None else idx]


@contextlib.contextmanager
def generator_checkpoint(generators: Sequence[Optional[torch.Generator]], device=None):
    gens = [default_generator(device) if g is None else g for g in generators]
    states = [g.get_state() for g in gens]
    try:
        yield gens
    finally:
        for g, s in zip(gens, states):
            g.set_state(s)


def train_mode_modules(modules: Iterable[torch.nn.Module]) -> List[str]:
    out = []
    for m in modules:
        for name, sub in m.named_modules():
            if sub.training and any(isinstance(sub, t) for t in (torch.nn.Dropout, torch.nn.Dropout1d,
                                                                 torch.nn.Dropout2d, torch.nn.Dropout3d)):
                out.append(name or type(sub).__name__)
    return out


def capture_contract_gate(contract: str, modules: Iterable[torch.nn.Module] = ()) -> Gate:
    if contract not in CONTRACTS:
        return Gate("rng_contract", False, f"undeclared contract {contract!r}; one of {CONTRACTS}")
    bad = train_mode_modules(modules)
    if bad and contract != RNG_REGISTERED:
        return Gate("rng_contract", False, f"dropout in training mode inside a {contract} region: {bad[0]}")
    return Gate("rng_contract", True, contract)


def offsets_moved(fn: Callable, generators: Sequence[torch.Generator]):
    """Run ``fn()`` and report which generators it advanced: (result, [(index, changed), ...])."""
    before = [g.get_state().clone() for g in generators]
    out = fn()
    moved = [(i, not torch.equal(b, g.get_state())) for i, (b, g) in enumerate(zip(before, generators))]
    return out, moved


def positioned_generator(seed: int, offset: int = 0, device="cpu") -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    if offset:
        if hasattr(g, "set_offset") and torch.device(device).type == "cuda":
            g.set_offset(offset)
        else:
            # CPU generators have no offset API: advance by drawing
            torch.empty(offset, device=device).normal_(generator=g)
    return g


def philox_increment(draw: Callable[[torch.Generator], object], device="cuda") -> int:
    """Philox offset one unit of the plain loop consumes (CUDA generators)."""
    g = torch.Generator(device=device)
    g.manual_seed(0)
    o0 = g.get_offset()
    draw(g)
    return int(g.get_offset() - o0)


def fork_at_offsets(seed: int, offsets: Sequence[int], device="cpu") -> List[torch.Generator]:
    return [positioned_generator(seed, int(o), device) for o in offsets]
