"""Row-sharded statements equal the dense statements (rank threads on CPU; P in {2, 3, 4}, uneven N)."""
import pytest
import torch

from uplifting_biomolecular_modeling_b200.core.testing import RankFailure, run_ranks
from uplifting_biomolecular_modeling_b200.models import pairformer
from uplifting_biomolecular_modeling_b200.parallel import comm as C
from uplifting_biomolecular_modeling_b200.parallel import rowpair
from uplifting_biomolecular_modeling_b200.parallel.layout import Layout


def test_layout_bounds():
    assert Layout(10, 3).bounds() == [(0, 4), (4, 7), (7, 10)]
    assert Layout(1000, 4, align=128).bounds() == [(0, 256), (256, 512), (512, 768), (768, 1000)]
    assert Layout(100, 4, align=128).bounds() == [(0, 100), (100, 100), (100, 100), (100, 100)]
    assert Layout(100, 4, align=128).empty_ranks() == [1, 2, 3]
    assert Layout(10, 3).owner(6) == 1 and Layout(10, 3).max_count() == 4


@pytest.mark.parametrize("P,N", [(2, 12), (3, 11), (4, 13)])
def test_transpose_shard(P, N):
    z = torch.randn(N, N, 3, dtype=torch.float64)
    lay = Layout(N, P)

    def fn(comm):
        zt = rowpair.transpose_shard(rowpair.shard_rows(z, lay, comm.rank), lay, comm)
        a, b = lay.rows(comm.rank)
        assert torch.equal(zt, z.transpose(0, 1)[a:b])
        return True

    assert all(run_ranks(P, fn))


@pytest.mark.parametrize("P,N", [(2, 16), (3, 13)])
def test_pairformer_layer_sharded_equals_dense(P, N):
    torch.manual_seed(0)
    layer = pairformer.PairformerLayer(c_s=32, c_z=16, heads=4, pair_heads=2).double().eval()
    s = torch.randn(1, N, 32, dtype=torch.float64)
    z = torch.randn(1, N, N, 16, dtype=torch.float64)
    with torch.no_grad():
        s_ref, z_ref = layer(s, z, None, None)
    lay = Layout(N, P)

    def fn(comm):
        with torch.no_grad():
            zl = rowpair.shard_rows(z[0], lay, comm.rank)
            s2, zl = rowpair.pairformer_layer_rows(layer, s, zl, lay, comm, comm.rank)
            zfull = rowpair.gather_pair(zl, comm)
        return s2, zfull

    for s2, zfull in run_ranks(P, fn):
        assert torch.allclose(zfull, z_ref[0], atol=1e-9, rtol=1e-9)
        assert torch.allclose(s2, s_ref, atol=1e-5, rtol=1e-5)      # single track runs in fp32 by design


def test_solo_comm_is_identity_and_failures_surface():
    c = C.SoloComm()
    t = torch.arange(6.).view(3, 2)
    assert torch.equal(c.all_gather_rows(t), t) and c.all_reduce_scalar(3.0) == 3.0

    def bad(comm):
        if comm.rank == 1:
            raise ValueError("boom")
        comm.barrier()

    with pytest.raises(RankFailure) as ei:
        run_ranks(2, bad, timeout_s=20)
    assert "boom" in str(ei.value)

    def guard(comm):
        comm.check_replicated(torch.ones(3) * (1 + comm.rank), "weights")

    with pytest.raises(RankFailure) as ei:
        run_ranks(2, guard, timeout_s=20)
    assert "replication guard" in str(ei.value)


def test_host_wait_times_out_by_name():
    hub = C.ThreadHub(2)

    def fn(comm):
        if comm.rank == 0:
            with pytest.raises(C.CommAborted):
                comm.host_wait("never", timeout_s=0.3)
        return True

    assert all(run_ranks(2, fn, hub=hub))


@pytest.mark.parametrize("P,N", [(2, 10), (3, 11)])
def test_heads_gather_and_feature_broadcast(P, N):
    from uplifting_biomolecular_modeling_b200.core.testing import run_ranks
    from uplifting_biomolecular_modeling_b200.parallel import rowpair
    from uplifting_biomolecular_modeling_b200.parallel.layout import Layout
    torch.manual_seed(0)
    z = torch.randn(N, N, 8)
    lin = torch.nn.Linear(8, 5)
    want = lin(z + z.transpose(0, 1))
    feats0 = {"a": torch.arange(7.0), "b": torch.randint(0, 9, (3, 4)), "big": torch.randn(50, 33), "flag": True}
    layout = Layout(N, P)

    def body(comm):
        z_loc = rowpair.shard_rows(z, layout, comm.rank)
        logits = rowpair.sym_logit_rows(z_loc, lin, layout, comm)
        whole = rowpair.gather_rows_to_rank0_host(logits, comm, block_cols=3)
        feats = rowpair.broadcast_features(feats0 if comm.rank == 0 else None, comm, chunk_bytes=256)
        return whole, feats

    for r, (whole, feats) in enumerate(run_ranks(P, body)):
        if r == 0:
            torch.testing.assert_close(whole, want, atol=1e-5, rtol=1e-5)
        else:
            assert whole is None
        assert feats["flag"] is True and set(feats) == set(feats0)
        for k in ("a", "b", "big"):
            assert feats[k].dtype == feats0[k].dtype and torch.equal(feats[k], feats0[k])


@pytest.mark.parametrize("P,N", [(2, 12), (3, 10)])
def test_token_transformer_on_row_shards_equals_dense(P, N):
    from uplifting_biomolecular_modeling_b200.core.testing import run_ranks
    from uplifting_biomolecular_modeling_b200.models import diffusion
    from uplifting_biomolecular_modeling_b200.parallel import rowpair
    from uplifting_biomolecular_modeling_b200.parallel.layout import Layout
    torch.manual_seed(1)
    tr = diffusion.DiffusionTransformer(depth=2, dim=32, dim_s=24, heads=4).eval()
    a = torch.randn(2, N, 32)
    s = torch.randn(1, N, 24)
    bias = torch.randn(1, 4, N, N)
    with torch.no_grad():
        want = tr(a, s, [bias, bias])
    layout = Layout(N, P)

    def body(comm):
        r0, r1 = layout.rows(comm.rank)
        with torch.no_grad():
            return rowpair.dit_rows(tr, a[:, r0:r1], s[:, r0:r1], bias[:, :, r0:r1], comm)

    got = torch.cat(run_ranks(P, body), 1)
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)


def test_msa_block_sharded_over_sequences_matches_dense():
    """MSA sharded over sequences + pair tensor over rows (outer-product mean by reduce-scatter of partial updates,
    pair-weighted averaging with gathered weights) against the dense MSA block, uneven shards, masked sequences."""
    import torch
    from uplifting_biomolecular_modeling_b200.core import testing
    from uplifting_biomolecular_modeling_b200.models import msa
    from uplifting_biomolecular_modeling_b200.parallel import rowpair
    from uplifting_biomolecular_modeling_b200.parallel.layout import Layout
    torch.manual_seed(3)
    N, S, P = 13, 7, 3
    layer = msa.MSALayer(16, 128).double().eval()
    with torch.no_grad():
        for p_ in layer.parameters():
            p_.normal_(0, 0.2)
    z = torch.randn(1, N, N, 128, dtype=torch.float64)
    m = torch.randn(1, S, N, 16, dtype=torch.float64)
    msa_mask = (torch.rand(1, S, N) > 0.2).double()
    pm = torch.ones(1, N, N, dtype=torch.float64)
    with torch.no_grad():
        z_ref, m_ref = layer(z, m, pm, msa_mask, None)
    lay = Layout(N, P)
    sb = rowpair.seq_bounds(S, P)

    def rank_fn(comm):
        r = comm.rank
        a, b = lay.rows(r)
        s0, s1 = sb[r]
        with torch.no_grad():
            z_loc, m_loc = rowpair.msa_layer_seqshard(layer, z[0, a:b].clone(), m[:, s0:s1].clone(),
                                                      msa_mask[:, s0:s1], lay, comm, r, S)
        return z_loc, m_loc

    outs = testing.run_ranks(P, rank_fn)
    z_got = torch.cat([o[0] for o in outs], 0)
    m_got = torch.cat([o[1] for o in outs], 1)
    # partial sums and counts travel in fp32 (the wire format of the schedule), hence fp32-level agreement
    assert torch.allclose(z_got, z_ref[0], atol=2e-5, rtol=2e-5), (z_got - z_ref[0]).abs().max()
    assert torch.allclose(m_got, m_ref, atol=2e-5, rtol=2e-5)
