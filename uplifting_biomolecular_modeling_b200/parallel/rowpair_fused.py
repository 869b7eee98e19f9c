"""Row-sharded pair stack on the sm_100a kernels, with the gathers fused into the compute kernels.

Per rank: rows [r0, r1) of z (bf16 [R, N, 128]).  Buffers that peers read live in symmetric memory:
the projected triangle-multiplication operands (``planes``) and the per-head triangle-attention bias
(``headbias``).  The schedule of one Pairformer block:

  trimul outgoing : projection (local rows) -> barrier -> contraction GEMM whose B tiles are TMA-loaded from
                    the owners' planes (all-gather fused into the GEMM) -> barrier -> output stage (local)
  trimul incoming : the projection kernel fetches its input tiles - columns of z - from the owners' shards
                    (distributed transpose + LayerNorm + gated projections in one kernel), then the outgoing
                    schedule; all-to-all + local projection when N or a shard is not a multiple of 128
  triatt starting : projection (q|k|v|gate rows + this rank's rows of the bias planes) -> barrier -> attention
                    launch whose prologue copies the peers' bias rows into the local planes with plain peer loads
                    (the all-gather is part of the kernel; the tiles then read local memory) -> barrier -> output GEMM
  triatt ending   : projection fetching columns of z from the owners (as above), attention, output GEMM, the
                    update transposed back by all-to-all
  transition      : local

The barriers are stream-ordered kernels with bounded waits (``parallel.symm``).  The two transposes use
the process group's all-to-all.  Same statements as ``parallel.rowpair`` (which is the NCCL-only
baseline of every step).  Reference schedule: common/opt_core/opt_core/mem/rowpair/pairstack.py:195-251.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import gemm as _gemm
from ..ops import native, pair, peer
from .comm import Comm
from .layout import Layout
from .rowpair import transpose_shard
from .symm import SymmHeap


class FusedRowPair:
    def __init__(self, layout: Layout, comm: Comm, heap: SymmHeap, heads: int = 4, gather: str = "peer"):
        """``gather="peer"``: the GEMM / attention kernels read the owners' shards themselves (fused);
        ``gather="peer_direct"``: as "peer" but the GEMM re-reads remote tiles per m-tile instead of copying them once;
        ``gather="nccl"``: the shards are first all-gathered into local buffers with NCCL and the same
        kernels run on the gathered copy - the NCCL-only baseline of the same schedule."""
        if gather not in ("peer", "peer_direct", "nccl"):
            raise ValueError("gather must be 'peer', 'peer_direct' or 'nccl'")
        self.gather = gather
        self.layout, self.comm, self.heap = layout, comm, heap
        self.rank, self.world = comm.rank, comm.world
        self.N = layout.n
        self.Np = pair.ceil_to(self.N, 8)
        self.rows = layout.count(self.rank)
        self.counts = [b - a for a, b in layout.bounds()]
        self.Rmax = max(max(self.counts), 1)
        dev = heap.device
        self.H = heads
        self.planes = heap.alloc((2, 128, self.Rmax, self.Np), torch.bfloat16)
        self.headbias = heap.alloc((heads, self.Rmax, self.Np), torch.bfloat16)
        self.planes.local.zero_()
        self.headbias.local.zero_()
        # whole bias planes [H, N, Np] in symmetric memory: every rank writes the rows it owns into its own copy and
        # the attention launch completes the copy from the peers' ("peer" mode: the all-gather is the kernel's prologue)
        self.row0 = layout.rows(self.rank)[0]
        self.hb_full = None
        if gather == "peer" and self.world > 1 and min(self.counts) >= 0:
            self.hb_full = heap.alloc((heads, self.N, self.Np), torch.bfloat16)
            self.hb_full.local.zero_()
            self._hb_state = peer.BiasGatherState(dev)
        # "peer" mode, N and every shard a multiple of 128: the projections of the transposed forms (incoming
        # triangle multiplication, ending-node attention) fetch their input tiles - columns of z - from the owners'
        # shards themselves, so z shards are staged in symmetric memory and no all-to-all precedes the projection
        self.zsym = None
        if gather == "peer" and self.world > 1 and self.N % 128 == 0 and all(c % 128 == 0 and c > 0 for c in self.counts):
            self.zsym = heap.alloc((self.Rmax, self.N, 128), torch.bfloat16)
        self.x = torch.empty((128, self.Rmax, self.Np), dtype=torch.bfloat16, device=dev)
        self.qkvgo = torch.empty((5, self.Rmax * self.N, 128), dtype=torch.bfloat16, device=dev)
        self.dev = dev
        heap.barrier()

    # ------------------------------------------------------------------ triangle multiplication
    def trimul_(self, z_loc: torch.Tensor, w: pair.TrimulPacked, outgoing: bool) -> torch.Tensor:
        R, N, Np, Rmax = self.rows, self.N, self.Np, self.Rmax
        st = native.status_tensor(self.dev)
        stream = native.current_stream(self.dev)
        lib = native.lib()
        if not outgoing and self.zsym is not None:
            # transpose + LayerNorm + gated projections in one kernel: tiles of z^T come from the owners' shards
            self._stage_z(z_loc)
            rc = lib.ubm_trimul_proj_rows_peer(self._z_ptrs(), self._counts_arr(), self.world, self.rank,
                                               native.ptr(w.w_in), native.ptr(w.in_colsum), native.ptr(w.in_colbias),
                                               0, native.ptr(self.planes.local), R, Rmax, N, Np, native.ptr(st), stream)
            native.check(rc, "ubm_trimul_proj_rows_peer")
        else:
            src = z_loc if outgoing else transpose_shard(z_loc, self.layout, self.comm)
            if R > 0:
                rc = lib.ubm_trimul_proj_rows(native.ptr(src), native.ptr(w.w_in), native.ptr(w.in_colsum),
                                              native.ptr(w.in_colbias), 0, native.ptr(self.planes.local), 0, R, Rmax, N,
                                              Np, native.ptr(st), stream)
                native.check(rc, "ubm_trimul_proj_rows")
        xv = self.x.view(-1)[: 128 * max(R, 1) * Np].view(128, max(R, 1), Np)   # [128][rows][Np] for the output stage
        a_loc = self.planes.local[0][:, :R, :N]
        if self.gather in ("peer", "peer_direct"):
            self.heap.barrier()                  # every owner's b rows are written and visible
            if R > 0:
                b_off = 128 * Rmax * Np * 2      # byte offset of plane b inside each rank's buffer
                gs = None
                if self.gather == "peer" and self.world > 1:
                    if not hasattr(self, "_gather_b"):
                        self._gather_b = peer.GatherState(128, N, Np, self.dev)
                    gs = self._gather_b
                peer.gemm_allgather_b(a_loc, [self.planes.ptr(q, b_off) for q in range(self.world)], self.counts,
                                      xv[:, :, :N], K=N, ldb=Np, stride_b=Rmax * Np, my_rank=self.rank, gather=gs)
            self.heap.barrier()                  # nobody still reads my planes when I overwrite them
        else:
            import torch.distributed as dist
            if not hasattr(self, "_b_all"):
                self._b_all = torch.empty((self.world, 128, Rmax, Np), dtype=torch.bfloat16, device=self.dev)
            dist.all_gather_into_tensor(self._b_all, self.planes.local[1].contiguous())
            if R > 0:
                b_full = torch.cat([self._b_all[q][:, :self.counts[q], :N] for q in range(self.world)], dim=1)
                _gemm.gemm(a_loc, b_full, out=xv[:, :, :N])
        if R > 0:
            out = torch.empty_like(z_loc)
            rc = lib.ubm_trimul_out_rows(native.ptr(self.x), native.ptr(z_loc), native.ptr(w.wo), native.ptr(w.wg),
                                         native.ptr(w.o_colsum), native.ptr(w.o_colbias), native.ptr(w.g_colsum),
                                         native.ptr(w.g_colbias), native.ptr(out), R, N, Np, 1, native.ptr(st), stream)
            native.check(rc, "ubm_trimul_out_rows")
            return out
        return z_loc

    # ------------------------------------------------------------------ z shards readable by the peers
    def _stage_z(self, z_loc: torch.Tensor) -> None:
        """Copy this rank's rows of z into its symmetric staging buffer and order the ranks: after the barrier
        every shard is written and visible, and (the barrier being the first since the previous reader's last
        barrier) nobody still reads the old contents."""
        self.zsym.local[: self.rows].copy_(z_loc)
        self.heap.barrier()

    def _z_ptrs(self):
        from . import symm as _symm
        return _symm.ptr_array([self.zsym.ptr(q) for q in range(self.world)])

    def _counts_arr(self):
        from . import symm as _symm
        return _symm.int_array(self.counts)

    # ------------------------------------------------------------------ triangle attention
    def triatt_(self, z_loc: torch.Tensor, w: pair.TriattPacked, starting: bool) -> torch.Tensor:
        R, N, Np, Rmax, H = self.rows, self.N, self.Np, self.Rmax, self.H
        st = native.status_tensor(self.dev)
        stream = native.current_stream(self.dev)
        q, k, v, g, og = (self.qkvgo[i][: R * N] for i in range(5))
        lib = native.lib()
        fused_gather = self.hb_full is not None and min(self.counts) >= 4
        peer_src = (not starting) and self.zsym is not None
        src = None
        if peer_src:
            # ending node: transpose + LayerNorm + q|k|v|gate + head-bias projection in one kernel
            self._stage_z(z_loc)
            hb_ptr = (self.hb_full.ptr(self.rank, self.row0 * Np * 2), N) if fused_gather else \
                (native.ptr(self.headbias.local), Rmax)
            rc = lib.ubm_triatt_proj_rows_peer(self._z_ptrs(), self._counts_arr(), self.world, self.rank,
                                               native.ptr(w.w), native.ptr(w.colsum), native.ptr(w.colbias),
                                               native.ptr(w.wb), native.ptr(w.wb_colsum), native.ptr(w.wb_colbias),
                                               native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(g), hb_ptr[0],
                                               R, hb_ptr[1], N, Np, H, native.ptr(st), stream)
            native.check(rc, "ubm_triatt_proj_rows_peer")
        else:
            src = z_loc if starting else transpose_shard(z_loc, self.layout, self.comm)
        if R > 0 and not peer_src:
            # in the fused-gather mode the projection writes this rank's bias rows straight into its rows of the
            # whole planes (plane stride N rows); otherwise into the [H, Rmax, Np] shard buffer
            hb_ptr = (self.hb_full.ptr(self.rank, self.row0 * Np * 2), N) if fused_gather else \
                (native.ptr(self.headbias.local), Rmax)
            rc = lib.ubm_triatt_proj_rows(native.ptr(src), native.ptr(w.w), native.ptr(w.colsum), native.ptr(w.colbias),
                                          native.ptr(w.wb), native.ptr(w.wb_colsum), native.ptr(w.wb_colbias),
                                          native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(g),
                                          hb_ptr[0], 0, R, hb_ptr[1], N, Np, H, 0, native.ptr(st), stream)
            native.check(rc, "ubm_triatt_proj_rows")
        # the bias tiles are reused by every row pair: reading them in-kernel from the owner crosses NVLink once
        # per reuse, so only the "peer_direct" mode does that; otherwise the planes are gathered once
        if fused_gather:
            self.heap.barrier()                  # every owner's bias rows are written and visible
            peer.attention_gather_bias(q, k, v, [self.hb_full.ptr(p) for p in range(self.world)], self.counts,
                                       self.rank, self._hb_state, g, og, rows=R, N=N, H=H, ldb=Np)
            self.heap.barrier()                  # nobody still reads my rows when the next projection overwrites them
        elif self.gather == "peer_direct":
            self.heap.barrier()
            if R > 0:
                peer.attention_peer_bias(q, k, v, [self.headbias.ptr(p) for p in range(self.world)], self.counts,
                                         Rmax * Np, g, og, rows=R, N=N, H=H, ldb=Np)
            self.heap.barrier()
        else:
            import torch.distributed as dist
            if not hasattr(self, "_hb_all"):
                self._hb_all = torch.empty((self.world, H, Rmax, Np), dtype=torch.bfloat16, device=self.dev)
            dist.all_gather_into_tensor(self._hb_all, self.headbias.local)
            if R > 0:
                hb_full = torch.cat([self._hb_all[p][:, :self.counts[p]] for p in range(self.world)], dim=1).contiguous()
                pair.attention(q, k, v, hb_full, g, og, rows=R, Nq=N, Nk=N, H=H, D=32, ldb=Np)
        if starting:
            out = torch.empty_like(z_loc)
            if R > 0:
                _gemm.gemm(og, w.wo, bias=w.bo, residual=z_loc.view(R * N, 128), out=out.view(R * N, 128))
            return out
        upd_t = torch.empty_like(z_loc)
        if R > 0:
            _gemm.gemm(og, w.wo, bias=w.bo, out=upd_t.view(R * N, 128))
        upd = transpose_shard(upd_t, self.layout, self.comm)
        return z_loc + upd

    # ------------------------------------------------------------------ outer product mean, MSA sharded over sequences
    def opm_seqshard_(self, m_loc: torch.Tensor, mask_loc: torch.Tensor, mod, n_seq: int,
                      row_block: int = 128) -> torch.Tensor:
        """Outer product mean of an MSA sharded over sequences, GEMM -> reduce-scatter in one kernel: per block of
        pair rows every rank contracts its own sequences (MN-major tcgen05 GEMM with the blocked epilogue), then the
        projection GEMM's epilogue stores the rank's partial update straight into the slot it owns in the memory of
        the GPU that owns those rows (plain peer stores); a stream barrier orders the stores and the owner adds the P
        slots in rank order.  m_loc: bf16 [1, S_loc, N, c_m]; mask_loc: [1, S_loc, N].  Returns the update of the
        local rows, bf16 [R, N, c_z].  Plain statement: ``rowpair.opm_seqshard``."""
        from ..ops import rows as _rows
        from . import symm as _symm
        P, me, N, dev = self.world, self.rank, self.N, self.dev
        S_loc = m_loc.shape[1]
        c = mod.c_hidden
        cz = mod.proj_o.weight.shape[0]
        if c != 32 or S_loc == 0 or (N * c) % 32:
            raise ValueError("fused sequence-sharded outer product mean needs c_hidden = 32 and sequences on every rank")
        rb = max(8, min(row_block, self.Rmax))
        if not hasattr(self, "_opm_slots"):
            self._opm_slots = [self.heap.alloc((P, rb * N, cz), torch.bfloat16) for _ in range(2)]
            self._opm_t = torch.empty((rb * N, c * c), dtype=torch.bfloat16, device=dev)
            self._opm_calls = 0
        n = _rows.layernorm_rows(m_loc.contiguous(), mod.norm.weight, mod.norm.bias, mod.norm.eps)
        mk = mask_loc.unsqueeze(-1).to(n.dtype)
        a2 = (mod.proj_a(n) * mk)[0].reshape(S_loc, N * c)
        b2 = (mod.proj_b(n) * mk)[0].reshape(S_loc, N * c)
        wo = mod.proj_o.weight.detach().to(torch.bfloat16).contiguous()
        full = bool(getattr(mod, "full_mask", False))
        bias = mod.proj_o.bias.float().contiguous()
        cnt_rows = None
        if not full:
            # pairs with masked sequences: per-pair counts over all ranks (the mean's denominator); the first GEMM
            # carries 1 / S and the summed update is rescaled by S / count on c_z channels
            import torch.distributed as dist
            cnt = torch.einsum("si,sj->ij", mask_loc[0].float(), mask_loc[0].float())
            dist.all_reduce(cnt)
            r0, r1 = self.layout.rows(me)
            cnt_rows = (float(n_seq) / cnt[r0:r1].clamp(min=1.0)).unsqueeze(-1)
        out = torch.empty((max(self.rows, 0), N, cz), dtype=torch.bfloat16, device=dev)
        st = native.status_tensor(dev)
        stream = native.current_stream(dev)
        lib = native.lib()
        slot_elems = rb * N * cz
        for q in range(P):
            q0, q1 = self.layout.rows(q)
            for i0 in range(q0, q1, rb):
                i1 = min(q1, i0 + rb)
                nr = (i1 - i0) * N
                buf = self._opm_slots[self._opm_calls & 1]
                self._opm_calls += 1
                _gemm.gemm(a2[:, i0 * c:i1 * c], b2, mn_major=True, alpha=1.0 / n_seq, out=self._opm_t,
                           c_blocked=(N * c * c, c, c * c))
                dst = _symm.ptr_array([buf.ptr(q, me * slot_elems * 2)])
                rc = lib.ubm_gemm_bf16_scatter_rows(native.ptr(self._opm_t), native.ptr(wo), dst, 1, nr, nr, cz, c * c,
                                                    c * c, c * c, cz, 0, 1.0, native.ptr(st), stream)
                native.check(rc, "ubm_gemm_bf16_scatter_rows")
                self.heap.barrier()              # every rank's partial of this block is in the owner's slots
                if q == me:
                    o = out[i0 - q0:i1 - q0].view(nr, cz)
                    rc = lib.ubm_sum_slots(native.ptr(buf.local), slot_elems, P, native.ptr(bias) if full else 0, 0,
                                           native.ptr(o), nr, cz, stream)
                    native.check(rc, "ubm_sum_slots")
        if cnt_rows is not None and self.rows > 0:
            out = (out.float() * cnt_rows + bias).to(torch.bfloat16)
        return out

    # ------------------------------------------------------------------ one Pairformer block (pair part)
    def pair_block_(self, layer, z_loc: torch.Tensor) -> torch.Tensor:
        def packed(mod, maker):
            if mod._packed is None:
                mod._packed = maker()
            return mod._packed

        tmo, tmi, tas, tae, tr = (layer.tri_mul_out, layer.tri_mul_in, layer.tri_att_start, layer.tri_att_end,
                                  layer.transition_z)
        w_tmo = packed(tmo, lambda: pair.TrimulPacked.pack(tmo.norm_in.weight, tmo.norm_in.bias, tmo.p_in.weight,
                                                           tmo.g_in.weight, tmo.norm_out.weight, tmo.norm_out.bias,
                                                           tmo.p_out.weight, tmo.g_out.weight))
        w_tmi = packed(tmi, lambda: pair.TrimulPacked.pack(tmi.norm_in.weight, tmi.norm_in.bias, tmi.p_in.weight,
                                                           tmi.g_in.weight, tmi.norm_out.weight, tmi.norm_out.bias,
                                                           tmi.p_out.weight, tmi.g_out.weight))

        def tri(m):
            a = m.mha
            return pair.TriattPacked.pack(m.layer_norm.weight, m.layer_norm.bias, m.linear.weight, a.linear_q.weight,
                                          a.linear_k.weight, a.linear_v.weight, a.linear_g.weight, a.linear_g.bias,
                                          a.linear_o.weight, a.linear_o.bias, m.heads)
        w_tas, w_tae = packed(tas, lambda: tri(tas)), packed(tae, lambda: tri(tae))
        w_tr = packed(tr, lambda: pair.TransitionPacked.pack(tr.norm.weight, tr.norm.bias, tr.fc1.weight,
                                                             tr.fc2.weight, tr.fc3.weight))
        import os
        timing = os.environ.get("ROWPAIR_PAIRSTACK_TIMES") == "1"
        marks = []

        def mark(name):
            if timing:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                marks.append((name, e))

        mark("start")
        z_loc = self.trimul_(z_loc, w_tmo, True)
        mark("trimul_out")
        z_loc = self.trimul_(z_loc, w_tmi, False)
        mark("trimul_in")
        z_loc = self.triatt_(z_loc, w_tas, True)
        mark("triatt_start")
        z_loc = self.triatt_(z_loc, w_tae, False)
        mark("triatt_end")
        if self.rows > 0:
            z_loc = pair.transition_fused(z_loc.contiguous(), w_tr, residual=True)
        mark("transition")
        if timing:
            torch.cuda.synchronize()
            self.block_count = getattr(self, "block_count", 0) + 1
            if self.rank == 0 and self.block_count % 8 == 0:
                from ..core import report
                report.emit(report.line("rowpair", "BLOCKTIMES", ("block", self.block_count),
                                        *[(marks[i][0], round(marks[i - 1][1].elapsed_time(marks[i][1]), 2))
                                          for i in range(1, len(marks))]))
        return z_loc
