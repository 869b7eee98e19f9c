"""Tensor parallelism for the sequence models (StripedHyena-2 / Evo2): every operator is sharded over its
channel dimension.

Column-parallel projections (Hyena ``in_proj``, attention ``qkv``, the MLP's ``l1`` / ``l2``) keep a slice of
their output rows, so each rank computes its own channels / heads / hidden units from the replicated input and
everything per-channel in between (FIR stages, gates, convolutions, pole states, attention heads) runs on the
slice with no communication.  Row-parallel projections (``out_proj``, ``l3``) hold the matching slice of their
input columns; their partial products have to be summed over the ranks.  On GPUs that sum is the fused kernel
of :func:`ops.peer.gemm_reduce_scatter` (the GEMM epilogue stores every output row into the memory of the rank
that owns it, the owner adds the slots) followed by an all-gather of the rows; small row counts (decode steps)
and CPU tensors take a local GEMM and an all-reduce.

Reference: the tensor-parallel plan of the evo2 kit (evo2/opt/evo2_opt/kit, vortex model parallel layers).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from .comm import Comm


def _rows_of_thirds(n: int, lo: int, hi: int) -> torch.Tensor:
    """Indices [lo, hi) of each of the three n-wide thirds of a 3n-wide dimension."""
    base = torch.arange(lo, hi)
    return torch.cat([base, n + base, 2 * n + base])


class TensorParallel:
    def __init__(self, comm: Comm, heap=None, min_fused_rows: int = 1024):
        self.comm, self.heap = comm, heap
        self.rank, self.world = comm.rank, comm.world
        self.min_fused_rows = min_fused_rows
        self._rs: Dict[Tuple[int, int], object] = {}
        self.fused_calls = 0
        self.reduce_calls = 0

    # ------------------------------------------------------------------ sharding
    def shard_evo2(self, model) -> None:
        """Replace the parameters of a replicated model by this rank's slices, in place."""
        from ..models import evo2
        P, r = self.world, self.rank
        cfg = model.cfg
        d = cfg.d_model
        if d % P or cfg.n_heads % P or cfg.ffn % P:
            raise ValueError(f"d_model {d}, heads {cfg.n_heads} and ffn {cfg.ffn} must be divisible by {P} ranks")
        dl = d // P
        lo, hi = r * dl, (r + 1) * dl

        def keep(param: nn.Parameter, t: torch.Tensor):
            param.data = t.contiguous().clone()

        for blk in model.blocks:
            mx = blk.mixer
            if isinstance(mx, evo2.HyenaOperator):
                rows = _rows_of_thirds(d, lo, hi).to(mx.in_proj.weight.device)
                keep(mx.in_proj.weight, mx.in_proj.weight.data[rows])
                keep(mx.fir, mx.fir.data[rows])
                if mx.kind == "hcl":
                    keep(mx.log_poles, mx.log_poles.data[lo:hi])
                    keep(mx.residues, mx.residues.data[lo:hi])
                else:
                    keep(mx.h, mx.h.data[lo:hi])
                keep(mx.D, mx.D.data[lo:hi])
                mx._taps = None
            else:
                hd = d // cfg.n_heads
                w = mx.qkv.weight.data.view(3, cfg.n_heads, hd, d)
                hl = cfg.n_heads // P
                keep(mx.qkv.weight, w[:, r * hl:(r + 1) * hl].reshape(3 * hl * hd, d))
            keep(mx.out_proj.weight, mx.out_proj.weight.data[:, lo:hi])
            mx.out_proj._tp_row = True
            fl = cfg.ffn // P
            keep(blk.mlp.l1.weight, blk.mlp.l1.weight.data[r * fl:(r + 1) * fl])
            keep(blk.mlp.l2.weight, blk.mlp.l2.weight.data[r * fl:(r + 1) * fl])
            keep(blk.mlp.l3.weight, blk.mlp.l3.weight.data[:, r * fl:(r + 1) * fl])
            blk.mlp.l3._tp_row = True
        evo2._W_CACHE.clear()
        model.linear = self.linear
        model.folded = self.folded_linear if getattr(model, "folded", None) is not None else None

    # ------------------------------------------------------------------ the Linear hook
    def _sum(self, t: torch.Tensor) -> torch.Tensor:
        self.reduce_calls += 1
        dist = getattr(self.comm, "dist", None)
        if dist is not None:
            t = t.contiguous()
            dist.all_reduce(t, group=self.comm.group)
            return t
        parts = self.comm.all_gather(t.unsqueeze(0))
        return torch.stack([p_[0] for p_ in parts], 0).sum(0)

    def folded_linear(self, module: nn.Linear, rows: torch.Tensor, gamma=None, eps: float = 1e-6, res=None,
                      second=None) -> torch.Tensor:
        """The projection hook of the folded decode block (``models.evo2.Block._folded``) under tensor parallelism.
        Column-parallel projections take the one-GPU form on this rank's slice (their input is replicated, so the
        RMSNorm in front and the SwiGLU of two slices fold as they do there); a row-parallel projection streams
        its slice, the partial rows are summed over the ranks and bias and residual are added once behind the sum."""
        from ..models.evo2 import _bf16_weight, folded_linear
        if not getattr(module, "_tp_row", False):
            return folded_linear(module, rows, gamma=gamma, eps=eps, res=res, second=second)
        from ..ops import seq
        w, b = _bf16_weight(module)
        y = self._sum(seq.gemv_rows(rows, w))
        if b is not None:
            return seq.elementwise("bias_residual", y, a=res, v0=b)
        return y if res is None else seq.elementwise("add2", y, a=res)

    def linear(self, module: nn.Linear, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Replacement of ``module(x)`` under tensor parallelism (installed as the model's ``linear`` hook).
        ``residual`` (replicated, the shape of the result) is added once, behind the sum over the ranks."""
        y = self._linear(module, x)
        if residual is None:
            return y
        if y.is_cuda and y.dtype == torch.bfloat16 and residual.dtype == torch.bfloat16 and y.shape[-1] % 8 == 0:
            from ..ops import seq
            return seq.elementwise("add2", y.contiguous(), a=residual.contiguous().view(y.shape))
        return y + residual

    def _linear(self, module: nn.Linear, x: torch.Tensor) -> torch.Tensor:
        from ..models.evo2 import fused_linear
        if not getattr(module, "_tp_row", False):
            return fused_linear(module, x)                       # column-parallel: this rank's output slice
        P = self.world
        x2 = x.reshape(-1, x.shape[-1])
        M, N = x2.shape[0], module.weight.shape[0]
        gpu = x.is_cuda and x.dtype == torch.bfloat16 and x2.shape[1] % 8 == 0
        if gpu and self.heap is not None and M % P == 0 and M >= self.min_fused_rows and N % 8 == 0:
            from ..ops import peer
            key = (M // P, N)
            st = self._rs.get(key)
            if st is None:
                st = peer.ReduceScatterState(self.heap, M // P, N)
                self._rs[key] = st
            w = module.weight.detach()
            if w.dtype != torch.bfloat16 or not w.is_contiguous():
                w = w.to(torch.bfloat16).contiguous()
            rows = peer.gemm_reduce_scatter(x2.contiguous(), w, st, bias=module.bias)
            self.fused_calls += 1
            full = torch.empty((M, N), dtype=rows.dtype, device=rows.device)
            self.comm.dist.all_gather_into_tensor(full, rows, group=self.comm.group)
            return full.view(*x.shape[:-1], N)
        # partial product without the bias, summed over the ranks, bias once
        if gpu:
            from ..ops import gemm
            w = module.weight.detach()
            if w.dtype != torch.bfloat16 or not w.is_contiguous():
                w = w.to(torch.bfloat16).contiguous()
            if M <= 8:
                from ..ops import seq
                part = seq.gemv_rows(x2.contiguous(), w)
            else:
                part = gemm.gemm(x2.contiguous(), w)
        else:
            part = torch.nn.functional.linear(x2, module.weight)
        y = self._sum(part)
        if module.bias is not None:
            y = y + module.bias.to(y.dtype)
        return y.view(*x.shape[:-1], N)


TensorParallel.linear.takes_residual = True
