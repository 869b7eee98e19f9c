"""Row-chunked forms of the pair operations: the same statement applied to blocks of rows so that only
one block's intermediates exist at a time.  Transition, triangle attention (per block of rows ``i``; the
bias is computed once) and the row-local part of triangle multiplication are bitwise equal to the
unchunked statement ("bitwise" label); chunking the contraction dimension is not offered (it would
reorder sums).  Reference: common/opt_core/opt_core/mem/chunk.py:370,424,526,689,751 and
mem/torch_rowchunk.py:80.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ..ops import reference as R
from .registry import Ctx, Refusal, register


def rowchunk_apply(fn: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, rows: int, dim: int = 0,
                   out: Optional[torch.Tensor] = None, inplace: bool = False) -> torch.Tensor:
    """Apply ``fn`` to blocks of ``rows`` rows along ``dim`` and assemble (in place when asked)."""
    n = x.shape[dim]
    if rows <= 0 or rows >= n:
        return fn(x)
    dst = x if inplace else (out if out is not None else None)
    pieces = []
    for a in range(0, n, rows):
        sl = [slice(None)] * x.dim()
        sl[dim] = slice(a, min(n, a + rows))
        y = fn(x[tuple(sl)])
        if dst is not None:
            dst[tuple(sl)] = y
        else:
            pieces.append(y)
    return dst if dst is not None else torch.cat(pieces, dim=dim)


def rows_within(budget_bytes: int, bytes_per_row: int, minimum: int = 1, multiple: int = 1) -> int:
    """Largest row block (a multiple of ``multiple``) whose intermediates fit the budget."""
    r = max(minimum, budget_bytes // max(1, bytes_per_row))
    return max(minimum, r // multiple * multiple)


def transition_chunked(x, mod, rows: int, residual: bool = True):
    return rowchunk_apply(lambda b: mod(b, residual=residual), x, rows, dim=1 if x.dim() == 4 else 0)


def triangle_attention_chunked(z, mod, rows: int, residual: bool = True):
    """Starting-node triangle attention in blocks of rows i; the [H, N, N] bias is computed once.
    z: [N, N, c] (single batch)."""
    m = mod.mha
    H = mod.heads
    src = z if mod.starting else z.transpose(0, 1)
    n = R.layer_norm(src, mod.layer_norm.weight, mod.layer_norm.bias)
    bias = torch.nn.functional.linear(n, mod.linear.weight).permute(2, 0, 1).unsqueeze(0)
    N = src.shape[0]
    out = torch.empty_like(src)
    for a in range(0, N, max(1, rows)):
        b = min(N, a + max(1, rows))
        nb = n[a:b]
        q = torch.nn.functional.linear(nb, m.linear_q.weight).view(b - a, N, H, -1).transpose(1, 2)
        k = torch.nn.functional.linear(nb, m.linear_k.weight).view(b - a, N, H, -1).transpose(1, 2)
        v = torch.nn.functional.linear(nb, m.linear_v.weight).view(b - a, N, H, -1).transpose(1, 2)
        g = torch.sigmoid(torch.nn.functional.linear(nb, m.linear_g.weight, m.linear_g.bias))
        o = R.attention_with_bias(q, k, v, bias).transpose(1, 2).reshape(b - a, N, -1)
        out[a:b] = torch.nn.functional.linear(o * g, m.linear_o.weight, m.linear_o.bias)
    if not mod.starting:
        out = out.transpose(0, 1)
    return z + out if residual else out


@register("chunk_transition", label="bitwise")
def _lever_chunk_transition(ctx: Ctx):
    """Pair transitions run in row blocks (setting ``chunk_rows``)."""
    model = ctx.need("model")
    rows = int(ctx.settings.get("chunk_rows", 256))
    from ..models import pairformer
    n = 0
    for mod in model.modules():
        if isinstance(mod, pairformer.Transition) and mod.dim == 128 and not getattr(mod, "_chunked", False):
            orig = mod.forward
            mod.forward = (lambda x, residual=False, _o=orig, _r=rows:
                           rowchunk_apply(lambda b: _o(b, residual=residual), x, _r, dim=1 if x.dim() == 4 else 0))
            mod._chunked = True
            n += 1
    if n == 0:
        raise Refusal("no_pair_transition")
    return {"modules": n, "rows": rows}


@register("chunk_triatt", label="bitwise")
def _lever_chunk_triatt(ctx: Ctx):
    """Triangle attention (plain-statement path) runs in blocks of rows."""
    model = ctx.need("model")
    rows = int(ctx.settings.get("chunk_rows", 128))
    from ..models import pairformer
    n = 0
    for mod in model.modules():
        if isinstance(mod, pairformer.TriangleAttention) and not getattr(mod, "_chunked", False):
            orig = mod.forward

            def fwd(z, mask=None, residual=False, _m=mod, _o=orig, _r=rows):
                if _m.impl == "fused" or mask is not None or z.shape[0] != 1:
                    return _o(z, mask, residual)
                return triangle_attention_chunked(z[0], _m, _r, residual).unsqueeze(0)
            mod.forward = fwd
            mod._chunked = True
            n += 1
    if n == 0:
        raise Refusal("no_triangle_attention")
    return {"modules": n, "rows": rows}
