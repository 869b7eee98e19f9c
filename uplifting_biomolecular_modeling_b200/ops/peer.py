"""Python face of the kernels that read other GPUs' memory themselves (collective fused with compute):
the all-gather -> triangle contraction GEMM and the attention kernel with its pair-bias all-gather."""
from __future__ import annotations

import ctypes
import os
from typing import Sequence

import torch

from . import native
from .native import c_float, c_int, c_ll, c_void_p

native.declare("ubm_gemm_bf16_allgather_b",
               [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll,
                c_int, c_float, c_int, c_int, c_void_p, c_ll, c_ll, c_void_p, ctypes.c_uint, c_void_p, c_void_p])
native.declare("ubm_attention_d32_peer_bias",
               [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_ll, c_void_p, c_void_p, c_int, c_int, c_int,
                c_int, c_ll, c_ll, c_void_p, c_void_p])
native.declare("ubm_trimul_proj_rows", [c_void_p] * 7 + [c_int, c_int, c_int, c_int, c_void_p, c_void_p])
native.declare("ubm_triatt_proj_rows", [c_void_p] * 13 + [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
native.declare("ubm_trimul_out_rows", [c_void_p] * 9 + [c_int, c_int, c_int, c_int, c_void_p, c_void_p])


def _ptrs(ptrs: Sequence[int]):
    return (ctypes.c_void_p * len(ptrs))(*[ctypes.c_void_p(int(p)) for p in ptrs])


def _ints(vals: Sequence[int]):
    return (ctypes.c_int * len(vals))(*[int(v) for v in vals])


class GatherState:
    """Per-buffer state of the gather-once mode: the local gathered copy, its ready flags and the epoch."""

    def __init__(self, batch: int, total_rows: int, ld: int, device, copy_ctas: int = 16):
        self.buf = torch.empty((batch, total_rows, ld), dtype=torch.bfloat16, device=device)
        self.flags = torch.zeros(batch * ((total_rows + 255) // 256 + 8), dtype=torch.int32, device=device)
        self.epoch = 0
        self.copy_ctas = copy_ctas


def gemm_allgather_b(a: torch.Tensor, b_ptrs: Sequence[int], rows: Sequence[int], out: torch.Tensor, K: int,
                     ldb: int, stride_b: int, alpha: float = 1.0, my_rank: int = 0,
                     gather: "GatherState | None" = None) -> torch.Tensor:
    """out[c][m][col0_q + n] = sum_k a[c][m][k] * B_q[c][n][k]; B_q = bf16 [batch][rows[q]][K] at b_ptrs[q]
    (possibly on another GPU) with leading dimension ldb and batch stride stride_b (elements).  With a
    :class:`GatherState` the kernel's copy CTAs bring each remote block into local memory once."""
    batch, M = a.shape[0], a.shape[1]
    st = native.status_tensor(a.device)
    if gather is not None:
        gather.epoch += 1
        g_args = (gather.copy_ctas, native.ptr(gather.buf), gather.buf.stride(1), gather.buf.stride(0),
                  native.ptr(gather.flags), gather.epoch)
    else:
        g_args = (0, 0, 0, 0, 0, 0)
    rc = native.lib().ubm_gemm_bf16_allgather_b(native.ptr(a), _ptrs(b_ptrs), _ints(rows), len(rows), native.ptr(out),
                                                M, K, batch, a.stride(1), ldb, out.stride(1), a.stride(0), stride_b,
                                                out.stride(0), 1 if out.dtype == torch.float32 else 0, float(alpha),
                                                my_rank, *g_args,
                                                native.ptr(st), native.current_stream(a.device))
    native.check(rc, "ubm_gemm_bf16_allgather_b")
    return out


native.declare("ubm_attention_d32_gather_bias",
               [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, ctypes.c_uint, c_void_p,
                c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_ll, c_int, c_void_p,
                c_void_p])


native.declare("ubm_triatt_proj_rows_peer",
               [c_void_p, c_void_p, c_int, c_int] + [c_void_p] * 11 + [c_int] * 5 + [c_void_p, c_void_p])
native.declare("ubm_trimul_proj_rows_peer",
               [c_void_p, c_void_p, c_int, c_int] + [c_void_p] * 5 + [c_int] * 4 + [c_void_p, c_void_p])


class BiasGatherState:
    """Counter and launch count of the in-kernel pair-bias gather (one per symmetric bias buffer)."""

    def __init__(self, device):
        self.done = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0


def attention_gather_bias(q, k, v, bias_bufs: Sequence[int], rows_per_gpu: Sequence[int], me: int,
                          state: BiasGatherState, gate, out, rows: int, N: int, H: int, ldb: int,
                          transpose_out: bool = False, mask=None):
    """Triangle-attention core whose launch also performs the all-gather of the pair-bias planes: ``bias_bufs[i]`` is
    GPU i's [H, N, ldb] buffer (symmetric memory) holding the rows it owns; the kernel completes this GPU's buffer
    from the peers' and attends on it.  Needs at least four rows."""
    st = native.status_tensor(q.device)
    state.epoch += 1
    rc = native.lib().ubm_attention_d32_gather_bias(
        native.ptr(q), native.ptr(k), native.ptr(v), _ptrs(bias_bufs), _ints(rows_per_gpu), len(rows_per_gpu), me,
        native.ptr(state.done), state.epoch, native.ptr(gate), native.ptr(out),
        native.ptr(None if mask is None else mask.add), native.ptr(None if mask is None else mask.flags), rows, N, N, H,
        ldb, 0, 0, 0 if mask is None else mask.add.stride(0), 1 if transpose_out else 0, native.ptr(st),
        native.current_stream(q.device))
    native.check(rc, "ubm_attention_d32_gather_bias")
    return out


def attention_peer_bias(q, k, v, bias_ptrs: Sequence[int], peer_rows: Sequence[int], head_stride: int, gate, out,
                        rows: int, N: int, H: int, ldb: int):
    st = native.status_tensor(q.device)
    rc = native.lib().ubm_attention_d32_peer_bias(native.ptr(q), native.ptr(k), native.ptr(v), _ptrs(bias_ptrs),
                                                  _ints(peer_rows), len(peer_rows), head_stride, native.ptr(gate),
                                                  native.ptr(out), rows, N, N, H, ldb, 0, native.ptr(st),
                                                  native.current_stream(q.device))
    native.check(rc, "ubm_attention_d32_peer_bias")
    return out


native.declare("ubm_gemm_bf16_scatter_rows",
               [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_int, c_float,
                c_void_p, c_void_p])
native.declare("ubm_sum_slots", [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p])


class ReduceScatterState:
    """Slot buffers of the GEMM -> reduce-scatter: on every GPU two symmetric buffers [P][rows_per_rank][N] bf16
    (alternating between calls, so a sender never overwrites slots their owner is still adding)."""

    def __init__(self, heap, rows_per_rank: int, n: int):
        self.heap, self.rows, self.n = heap, rows_per_rank, n
        self.bufs = [heap.alloc((heap.world, rows_per_rank, n), torch.bfloat16) for _ in range(2)]
        self.calls = 0
        if os.environ.get("UBM_P2P_CHECK", "0") == "1":
            # every rank's puts of one call against the slot buffer sizes, before any kernel stores to a peer
            from ..parallel import plan_check
            P, row_bytes = heap.world, n * 2
            plan = plan_check.reduce_scatter_plan(P, [rows_per_rank] * P, row_bytes)
            plan_check.check_exchange_plan(plan, {(q, "slots"): P * rows_per_rank * row_bytes for q in range(P)})


def gemm_reduce_scatter(x: torch.Tensor, w: torch.Tensor, state: ReduceScatterState, bias=None, residual=None,
                        alpha: float = 1.0) -> torch.Tensor:
    """Row-parallel linear of a tensor-parallel layer.  x: bf16 [M, K_local]; w: bf16 [N, K_local] (this rank's
    slice of the contraction dimension).  Every rank's GEMM epilogue stores its partial product straight into
    the slot it owns in the memory of the GPU that owns those output rows (rows m of GPU m // rows_per_rank);
    after a barrier that orders the stores each GPU adds its P slots in rank order (deterministic) with bias and
    residual.  Returns this rank's rows [rows_per_rank, N] of sum_over_ranks(x @ w.T)."""
    heap = state.heap
    P, r = heap.world, heap.rank
    M, K = x.shape
    N = w.shape[0]
    if M > P * state.rows or N != state.n:
        raise ValueError("shape does not fit the slot buffers")
    buf = state.bufs[state.calls & 1]
    state.calls += 1
    slot_bytes = state.rows * N * 2
    ptrs = _ptrs([buf.ptr(q, r * slot_bytes) for q in range(P)])
    st = native.status_tensor(x.device)
    rc = native.lib().ubm_gemm_bf16_scatter_rows(native.ptr(x), native.ptr(w), ptrs, P, state.rows, M, N, K,
                                                 x.stride(0), w.stride(0), N, 0, float(alpha), native.ptr(st),
                                                 native.current_stream(x.device))
    native.check(rc, "ubm_gemm_bf16_scatter_rows")
    heap.barrier()
    out = torch.empty((state.rows, N), dtype=torch.bfloat16, device=x.device)
    b32 = None if bias is None else bias.float().contiguous()
    rc = native.lib().ubm_sum_slots(native.ptr(buf.local), state.rows * N, P, native.ptr(b32), native.ptr(residual),
                                    native.ptr(out), state.rows, N, native.current_stream(x.device))
    native.check(rc, "ubm_sum_slots")
    return out
