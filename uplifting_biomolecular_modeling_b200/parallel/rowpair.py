"""Row-sharded pair stack ("rowpair"): one prediction over P GPUs of one host (``big --n_gpu P``).

Every rank owns rows [r0, r1) of the pair tensor z[N, N, C] from its birth to its last reader; the
single representation and the MSA are replicated.  Each sharded statement equals its dense statement:
the full-k sum of every output element happens inside one matmul on one rank - no split-K across
ranks, no partial-sum all-reduce (the reference's P-invariance rule,
common/opt_core/opt_core/mem/rowpair/trimul.py:15-18).

What crosses ranks, per Pairformer block (collective sites C1-C7 of the reference,
common/opt_core/opt_core/mem/rowpair/dist.py, ring.py, triatt.py, trimul.py):

* triangle multiplication, outgoing : all-gather of the projected ``b`` rows feeding a_ik . b_jk
* triangle multiplication, incoming : transpose of z (all-to-all), then the outgoing schedule on z^T rows
* triangle attention, starting node : all-gather of the per-head pair bias rows
* triangle attention, ending node   : transpose (all-to-all), starting-node schedule, transpose back
* single attention with pair bias   : local query rows, all-gather of the updated single rows

``impl="reference"`` runs plain PyTorch statements on the shards through the :class:`Comm` surface
(the NCCL baseline, also what the CPU tests check against the dense model); ``impl="fused"`` runs the
sm_100a kernels on the shards and lets the contraction GEMM and the attention kernel read the other
ranks' projected rows / bias planes straight from peer memory (see ``parallel.symm`` and
``ops.peer``), so the gather overlaps the math tile by tile.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F

from ..ops import reference as R
from .comm import Comm
from .layout import Layout


# ------------------------------------------------------------------------------- data movement
def shard_rows(z: torch.Tensor, layout: Layout, rank: int) -> torch.Tensor:
    a, b = layout.rows(rank)
    return z[a:b].contiguous()


def transpose_shard(z_loc: torch.Tensor, layout: Layout, comm: Comm) -> torch.Tensor:
    """Rows [r0, r1) of z -> rows [r0, r1) of z^T (z^T[i, k] = z[k, i]) by one all-to-all of blocks."""
    parts = [z_loc[:, a:b].contiguous() for (a, b) in layout.bounds()]          # to rank q: my rows x its columns
    got = comm.all_to_all(parts)                                                # from q: its rows x my columns
    col = torch.cat(got, dim=0)                                                 # [N, R_p, ...]
    return col.transpose(0, 1).contiguous()


# ------------------------------------------------------------------------------- sharded statements
def trimul_rows(z_loc, mask_loc, mod, layout: Layout, comm: Comm, outgoing: bool = True, residual: bool = True,
                mask_t_loc=None):
    """Triangle multiplication on local rows.  ``mod`` is a models.pairformer.TriangleMultiplication."""
    w = mod
    x_in = R.layer_norm(z_loc, w.norm_in.weight, w.norm_in.bias)
    if outgoing:
        src, src_mask = x_in, mask_loc
    else:
        zt = transpose_shard(z_loc, layout, comm)
        src = R.layer_norm(zt, w.norm_in.weight, w.norm_in.bias)
        src_mask = mask_t_loc
    ab = F.linear(src, w.p_in.weight) * torch.sigmoid(F.linear(src, w.g_in.weight))
    if src_mask is not None:
        ab = ab * src_mask.unsqueeze(-1).to(ab.dtype)
    a, b = torch.chunk(ab.float(), 2, dim=-1)
    b_all = comm.all_gather_rows(b.contiguous())                                # [N, N, c]
    x = torch.einsum("ikd,jkd->ijd", a, b_all).to(z_loc.dtype)
    out = F.linear(R.layer_norm(x, w.norm_out.weight, w.norm_out.bias), w.p_out.weight) * \
        torch.sigmoid(F.linear(x_in, w.g_out.weight))
    return z_loc + out if residual else out


def triatt_rows(z_loc, mod, layout: Layout, comm: Comm, starting: bool = True, residual: bool = True):
    """Triangle attention on local rows.  ``mod`` is a models.pairformer.TriangleAttention."""
    m = mod.mha
    H = mod.heads
    src = z_loc if starting else transpose_shard(z_loc, layout, comm)
    n = R.layer_norm(src, mod.layer_norm.weight, mod.layer_norm.bias)
    bias_loc = F.linear(n, mod.linear.weight)                                   # [R, N, H]
    bias = comm.all_gather_rows(bias_loc.contiguous()).permute(2, 0, 1)         # [H, N, N]
    Rr, N, _ = n.shape
    q = F.linear(n, m.linear_q.weight).view(Rr, N, H, -1).transpose(1, 2)
    k = F.linear(n, m.linear_k.weight).view(Rr, N, H, -1).transpose(1, 2)
    v = F.linear(n, m.linear_v.weight).view(Rr, N, H, -1).transpose(1, 2)
    g = torch.sigmoid(F.linear(n, m.linear_g.weight, m.linear_g.bias))
    o = R.attention_with_bias(q, k, v, bias.unsqueeze(0)).transpose(1, 2).reshape(Rr, N, -1)
    o = F.linear(o * g, m.linear_o.weight, m.linear_o.bias)
    if not starting:
        o = transpose_shard(o, layout, comm)
    return z_loc + o if residual else o


def transition_rows(z_loc, mod, residual: bool = True):
    return mod(z_loc, residual=residual)


def apb_rows(s, z_loc, mod, pre_norm, layout: Layout, comm: Comm, rank: int):
    """Single attention with pair bias: queries of the local token rows, keys of all tokens (s is
    replicated), bias from the local pair rows; the updated rows are all-gathered."""
    a, b = layout.rows(rank)
    s32 = s.float()
    sn = F.layer_norm(s32, (s32.shape[-1],), pre_norm.weight.float(), pre_norm.bias.float())
    H, D = mod.heads, mod.head_dim
    N = sn.shape[1]
    ql = sn[:, a:b]
    q = F.linear(ql, mod.proj_q.weight.float(), mod.proj_q.bias.float()).view(1, b - a, H, D).transpose(1, 2)
    k = F.linear(sn, mod.proj_k.weight.float()).view(1, N, H, D).transpose(1, 2)
    v = F.linear(sn, mod.proj_v.weight.float()).view(1, N, H, D).transpose(1, 2)
    g = torch.sigmoid(F.linear(ql, mod.proj_g.weight.float()))
    zl = z_loc.float()
    bias = F.linear(R.layer_norm(zl, mod.proj_z[0].weight.float(), mod.proj_z[0].bias.float()),
                    mod.proj_z[1].weight.float()).permute(2, 0, 1).unsqueeze(0)           # [1, H, R, N]
    o = R.attention_with_bias(q, k, v, bias).transpose(1, 2).reshape(1, b - a, H * D)
    upd_loc = F.linear(g * o, mod.proj_o.weight.float())[0]                              # [R, c_s]
    upd = comm.all_gather_rows(upd_loc.contiguous()).unsqueeze(0)
    return upd


def pairformer_layer_rows(layer, s, z_loc, layout: Layout, comm: Comm, rank: int, mask_loc=None, mask_t_loc=None):
    """One PairformerLayer on a row shard (block order as in the dense layer)."""
    z_loc = trimul_rows(z_loc, mask_loc, layer.tri_mul_out, layout, comm, True, True)
    z_loc = trimul_rows(z_loc, mask_loc, layer.tri_mul_in, layout, comm, False, True, mask_t_loc)
    z_loc = triatt_rows(z_loc, layer.tri_att_start, layout, comm, True, True)
    z_loc = triatt_rows(z_loc, layer.tri_att_end, layout, comm, False, True)
    z_loc = transition_rows(z_loc, layer.transition_z, True)
    if layer.no_seq:
        return s, z_loc
    s32 = s.float() + apb_rows(s, z_loc, layer.attention, layer.pre_norm_s, layout, comm, rank)
    t = layer.transition_s
    s32 = s32 + R.transition(s32, t.norm.weight.float(), t.norm.bias.float(), t.fc1.weight.float(),
                             t.fc2.weight.float(), t.fc3.weight.float())
    return s32.to(s.dtype), z_loc


def pair_stack_rows(module, s, z_loc, layout: Layout, comm: Comm, rank: int):
    for layer in module.layers:
        s, z_loc = pairformer_layer_rows(layer, s, z_loc, layout, comm, rank)
    return s, z_loc


def opm_rows(m, mask, mod, layout: Layout, rank: int):
    """Outer product mean: output rows [r0, r1) only (m replicated, so no traffic at all; contraction over
    the MSA depth is whole per (i, j))."""
    a0, a1 = layout.rows(rank)
    n = R.layer_norm(m, mod.norm.weight, mod.norm.bias)
    mk = mask.unsqueeze(-1).to(n.dtype)
    a = (F.linear(n, mod.proj_a.weight) * mk)[0, :, a0:a1]
    b = (F.linear(n, mod.proj_b.weight) * mk)[0]
    cnt = torch.einsum("si,sj->ij", mask[0, :, a0:a1].float(), mask[0].float()).clamp(min=1.0)
    out = []
    step = max(1, min(a1 - a0, (1 << 28) // max(1, b.shape[1] * a.shape[-1] * b.shape[-1])))   # <= 1 GiB fp32 per block
    for i0 in range(0, a1 - a0, step):
        i1 = min(a1 - a0, i0 + step)
        num = torch.einsum("sic,sjd->ijcd", a[:, i0:i1].float(), b.float())
        zz = (num / cnt[i0:i1, :, None, None]).reshape(i1 - i0, b.shape[1], -1).to(m.dtype)
        out.append(F.linear(zz, mod.proj_o.weight, mod.proj_o.bias))
    return torch.cat(out, 0) if out else a.new_zeros((0, b.shape[1], mod.proj_o.weight.shape[0]))


def pwa_rows(m, z_loc, mod, layout: Layout, comm: Comm, rank: int):
    """Pair-weighted averaging with local query rows: the softmax over j of the bias of rows [r0, r1) is whole
    on this rank; the averaged rows are all-gathered to update the replicated MSA representation."""
    a0, a1 = layout.rows(rank)
    mn = R.layer_norm(m, mod.norm_m.weight, mod.norm_m.bias)
    zn = R.layer_norm(z_loc, mod.norm_z.weight, mod.norm_z.bias)
    B, S, N, _ = mn.shape
    H, c = mod.heads, mod.c_h
    v = F.linear(mn, mod.proj_m.weight).view(B, S, N, H, c)[0]                       # [S, N, H, c]
    w = torch.softmax(F.linear(zn, mod.proj_z.weight).permute(2, 0, 1).float(), dim=-1)   # [H, R, N]
    o = torch.einsum("hij,sjhd->sihd", w, v.float()).to(m.dtype)                       # [S, R, H, c]
    g = torch.sigmoid(F.linear(mn[0, :, a0:a1], mod.proj_g.weight))                   # [S, R, H*c]
    upd_loc = F.linear(g * o.reshape(S, a1 - a0, H * c), mod.proj_o.weight)            # [S, R, c_m]
    upd = comm.all_gather_rows(upd_loc.transpose(0, 1).contiguous()).transpose(0, 1)   # [S, N, c_m]
    return upd.unsqueeze(0)


def msa_layer_rows(layer, z_loc, m, msa_mask, layout: Layout, comm: Comm, rank: int, pair_block=None):
    """One MSA block on a row shard: m replicated, z rows local.  ``pair_block(layer, z_loc)`` may replace the
    plain sharded pair update (the fused GPU path)."""
    m = m + pwa_rows(m, z_loc, layer.pair_weighted_averaging, layout, comm, rank)
    m = m + layer.msa_transition(m)
    z_loc = z_loc + opm_rows(m, msa_mask, layer.outer_product_mean, layout, rank).to(z_loc.dtype)
    if pair_block is not None:
        z_loc = pair_block(layer.pairformer_layer, z_loc.contiguous())
    else:
        _, z_loc = pairformer_layer_rows(layer.pairformer_layer, None, z_loc, layout, comm, rank)
    return z_loc, m


# ------------------------------------------------------------------------------- MSA sharded over sequences
def seq_bounds(n_seq: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous sequence ranges of the ranks (the first ``n_seq % world`` ranks hold one more)."""
    base, extra = divmod(n_seq, world)
    out, a = [], 0
    for r in range(world):
        b = a + base + (1 if r < extra else 0)
        out.append((a, b))
        a = b
    return out


def opm_seqshard(m_loc, mask_loc, mod, layout: Layout, comm: Comm, n_seq: int, row_block: int = 64):
    """Outer product mean with the MSA sharded over SEQUENCES: every rank contracts its own sequences for every
    pair (i, j), projects the partial sum (the projection is linear) and the partial updates are reduce-scattered
    onto the row owners - rank q receives the sum over ranks of rows [r0_q, r1_q).  This is the plain statement of
    the schedule (partials exchanged with the comm surface's all-to-all and added in rank order); the GPU form puts
    the scatter into the projection GEMM's epilogue (``FusedRowPair.opm_seqshard_``).  The reference keeps m
    replicated or token-sharded and has no reduce-scatter (common/opt_core/opt_core/mem/rowpair/msa.py:157); a deep
    MSA then costs every rank the whole [S, N, c_m] tensor, which this schedule divides by P.

    m_loc: [1, S_loc, N, c_m]; mask_loc: [1, S_loc, N].  Returns the update of the local pair rows [R, N, c_z].
    The mean divides by the per-pair count of unmasked sequences over ALL ranks."""
    n = R.layer_norm(m_loc, mod.norm.weight, mod.norm.bias)
    mk = mask_loc.unsqueeze(-1).to(n.dtype)
    a = (F.linear(n, mod.proj_a.weight) * mk)[0]                     # [S_loc, N, c]
    b = (F.linear(n, mod.proj_b.weight) * mk)[0]
    N = a.shape[1]
    cnt_part = torch.einsum("si,sj->ij", mask_loc[0].float(), mask_loc[0].float())      # [N, N] partial counts
    parts_out, parts_cnt = [], []
    for (q0, q1) in layout.bounds():
        rows = []
        for i0 in range(q0, q1, max(1, row_block)):
            i1 = min(q1, i0 + max(1, row_block))
            num = torch.einsum("sic,sjd->ijcd", a[:, i0:i1].float(), b.float()).reshape(i1 - i0, N, -1)
            rows.append(F.linear(num.to(mod.proj_o.weight.dtype), mod.proj_o.weight))     # partial, no bias
        parts_out.append(torch.cat(rows, 0) if rows else a.new_zeros((0, N, mod.proj_o.weight.shape[0])))
        parts_cnt.append(cnt_part[q0:q1].contiguous())
    got = comm.all_to_all([p.float().contiguous() for p in parts_out])        # from rank q: its partial of MY rows
    gotc = comm.all_to_all(parts_cnt)
    tot = got[0]
    cnt = gotc[0]
    for q in range(1, comm.world):                                             # rank order: deterministic
        tot = tot + got[q]
        cnt = cnt + gotc[q]
    out = tot / cnt.clamp(min=1.0).unsqueeze(-1) + mod.proj_o.bias.float()
    return out.to(m_loc.dtype)


def pwa_seqshard(m_loc, z_loc, mod, layout: Layout, comm: Comm):
    """Pair-weighted averaging with the MSA sharded over sequences: the softmax weights of the local pair rows are
    all-gathered (every rank needs the weights of every query token), the average itself is local to the rank's
    sequences - the MSA rows never travel."""
    mn = R.layer_norm(m_loc, mod.norm_m.weight, mod.norm_m.bias)
    zn = R.layer_norm(z_loc, mod.norm_z.weight, mod.norm_z.bias)
    B, S, N, _ = mn.shape
    H, c = mod.heads, mod.c_h
    w_loc = torch.softmax(F.linear(zn, mod.proj_z.weight).float(), dim=1)                 # [R, N, H] over j
    w = comm.all_gather_rows(w_loc.contiguous()).permute(2, 0, 1)                          # [H, N, N]
    v = F.linear(mn, mod.proj_m.weight).view(B, S, N, H, c)[0]                             # [S_loc, N, H, c]
    o = torch.einsum("hij,sjhd->sihd", w, v.float()).to(m_loc.dtype)
    g = torch.sigmoid(F.linear(mn[0], mod.proj_g.weight))
    return F.linear(g * o.reshape(S, N, H * c), mod.proj_o.weight).unsqueeze(0)


def msa_layer_seqshard(layer, z_loc, m_loc, msa_mask_loc, layout: Layout, comm: Comm, rank: int, n_seq: int,
                       pair_block=None, opm=None):
    """One MSA block with the MSA sharded over sequences and the pair tensor over rows.  ``opm(m_loc, mask_loc,
    module)`` may replace :func:`opm_seqshard` (the fused GEMM -> reduce-scatter form)."""
    m_loc = m_loc + pwa_seqshard(m_loc, z_loc, layer.pair_weighted_averaging, layout, comm)
    m_loc = m_loc + layer.msa_transition(m_loc)
    upd = opm(m_loc, msa_mask_loc, layer.outer_product_mean) if opm is not None else \
        opm_seqshard(m_loc, msa_mask_loc, layer.outer_product_mean, layout, comm, n_seq)
    z_loc = z_loc + upd.to(z_loc.dtype)
    if pair_block is not None:
        z_loc = pair_block(layer.pairformer_layer, z_loc.contiguous())
    else:
        _, z_loc = pairformer_layer_rows(layer.pairformer_layer, None, z_loc, layout, comm, rank)
    return z_loc, m_loc


def gather_pair(z_loc, comm: Comm) -> torch.Tensor:
    return comm.all_gather_rows(z_loc)


# ------------------------------------------------------------------------------- memory model
def shard_bytes(n: int, c: int, elt: int, world: int) -> int:
    """u = N^2 * C * elt / P, the unit of the per-rank peak model peak = a(N) + b(N) / P
    (common/opt_core/opt_core/mem/rowpair/API.md:174)."""
    return n * n * c * elt // world


# ------------------------------------------------------------------------------------------ heads, gathers, features
def sym_logit_rows(z_loc: torch.Tensor, linear, layout: Layout, comm: Comm) -> torch.Tensor:
    """Rows of ``linear(z + z^T)`` (distogram / contact heads) from a row shard: the transposed shard arrives by the
    same distributed transpose the ending-node attention uses; the sum and the projection are local.
    Reference: heads.sym_logit_rows (mem/rowpair/heads.py:150)."""
    zt = transpose_shard(z_loc, layout, comm)
    return linear(z_loc + zt)


def gather_rows_to_rank0_host(x_loc: torch.Tensor, comm: Comm, block_cols: Optional[int] = None,
                              max_block_bytes: int = 64 << 20) -> Optional[torch.Tensor]:
    """Row shards ``[rows_r, N, ...]`` -> the whole tensor in host memory on rank 0 (None elsewhere), gathered in
    column blocks of at most ``max_block_bytes`` per rank so that no rank ever stages the whole tensor on its
    device.  Reference: dist.gather_rows_to_rank0_host (mem/rowpair/dist.py:1686)."""
    rows = [int(t.item()) for t in comm.all_gather(torch.tensor([x_loc.shape[0]], dtype=torch.long, device=x_loc.device))]
    N = x_loc.shape[1]
    tail = tuple(x_loc.shape[2:])
    per_col = max(1, x_loc.shape[0]) * x_loc.element_size()
    for d in tail:
        per_col *= int(d)
    if block_cols is None:
        block_cols = max(1, min(N, max_block_bytes // max(1, per_col)))
    out = None
    if comm.rank == 0:
        pin = torch.cuda.is_available() and x_loc.is_cuda
        out = torch.empty((sum(rows), N) + tail, dtype=x_loc.dtype, pin_memory=pin)
    starts = [sum(rows[:r]) for r in range(comm.world)]
    for c0 in range(0, N, block_cols):
        c1 = min(N, c0 + block_cols)
        parts = comm.all_gather(x_loc[:, c0:c1].contiguous())
        if comm.rank == 0:
            for r, p in enumerate(parts):
                out[starts[r]:starts[r] + rows[r], c0:c1].copy_(p, non_blocking=True)
    if comm.rank == 0 and x_loc.is_cuda:
        torch.cuda.current_stream(x_loc.device).synchronize()
    return out


def broadcast_features(feats, comm: Comm, src: int = 0, chunk_bytes: int = 64 << 20, device=None):
    """Rank ``src`` featurises, every rank receives: the key / shape / dtype table travels through the host store,
    the tensors as coalesced byte chunks of at most ``chunk_bytes`` (small tensors share a chunk, large ones are
    split).  Returns the feature dict on every rank.  Reference: bcast.broadcast_tensordict
    (mem/rowpair/bcast.py:118)."""
    import json
    if comm.world == 1:
        return feats
    key = "ubm_features_table"
    if comm.rank == src:
        table = [(k, list(v.shape), str(v.dtype).replace("torch.", "")) for k, v in feats.items()
                 if isinstance(v, torch.Tensor)]
        extras = {k: v for k, v in feats.items() if not isinstance(v, torch.Tensor)}
        comm.host_signal(key, json.dumps({"table": table, "extras": extras}))
    meta = json.loads(comm.host_wait(key))
    table = meta["table"]
    dev = device if device is not None else (next(iter(feats.values())).device if comm.rank == src and feats else "cpu")
    sizes = []
    for k, shape, dt in table:
        n = 1
        for s in shape:
            n *= s
        sizes.append(n * torch.empty((), dtype=getattr(torch, dt)).element_size())
    # every tensor starts on a 16-byte boundary of the wire buffer (views of wider element types need it)
    offsets, total = [], 0
    for nbytes in sizes:
        offsets.append(total)
        total += (nbytes + 15) // 16 * 16
    flat = torch.zeros(total, dtype=torch.uint8, device=dev)
    if comm.rank == src:
        for (k, _, _), o, nbytes in zip(table, offsets, sizes):
            if nbytes:
                flat[o:o + nbytes].copy_(feats[k].contiguous().view(-1).view(torch.uint8))
    for o in range(0, total, chunk_bytes):
        piece = flat[o:o + chunk_bytes]
        got = comm.broadcast(piece.contiguous(), src)
        if comm.rank != src:
            piece.copy_(got)
    out = dict(meta["extras"])
    for (k, shape, dt), o, nbytes in zip(table, offsets, sizes):
        out[k] = flat[o:o + nbytes].view(getattr(torch, dt)).view(*shape) if nbytes else \
            torch.empty(shape, dtype=getattr(torch, dt), device=dev)
    return out


# ------------------------------------------------------------------------------------------ token transformer (DiT)
def dit_layer_rows(layer, a_loc: torch.Tensor, s_loc: torch.Tensor, bias_loc: torch.Tensor, comm: Comm):
    """One diffusion-transformer token layer on a token-row shard.  a_loc: [B, R, c] activations of the local
    token rows, s_loc: [B or 1, R, c_s] their conditioning, bias_loc: [1, H, R, N] the bias rows of the local
    queries.  Per layer one all-gather of the AdaLN-normalised rows (keys / values of every token); queries, the
    gate, the conditioned transition and both residuals are local to the shard.
    Reference: diffusion.dit_block_sharded (mem/rowpair/diffusion.py:545)."""
    h = layer.hoist(s_loc)
    b_loc = layer.adaln(a_loc, None, h["adaln"], False)
    parts = comm.all_gather(b_loc.transpose(0, 1).contiguous())                # token rows lead for the gather
    b_all = torch.cat(parts, 0).transpose(0, 1)                                 # [B, N, c]
    o_loc = layer.pair_bias_attn(b_loc, None, None, bias=bias_loc, k_in=b_all)
    a_loc = a_loc + torch.sigmoid(h["gate"]) * o_loc
    return a_loc + layer.transition(a_loc, None, h["t_adaln"], h["t_gate"], False)


def dit_rows(transformer, a_loc, s_loc, bias_loc, comm: Comm):
    """All token layers on a token-row shard (see :func:`dit_layer_rows`)."""
    for layer in transformer.layers:
        a_loc = dit_layer_rows(layer, a_loc, s_loc, bias_loc, comm)
    return a_loc
