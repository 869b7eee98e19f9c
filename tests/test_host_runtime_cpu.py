"""Host-side runtime helpers on CPU: memo, prefetcher, outputs, cold start, capture policies, loop helpers,
sequence helpers, layer pipeline, sample loop."""
import os
import time

import pytest
import torch
import torch.nn as nn


def test_memo_keys_on_content_and_counts_bypasses(tmp_path):
    from uplifting_biomolecular_modeling_b200.host import memo
    calls = []
    m = memo.Memo("feat", disk_dir=str(tmp_path))
    build = lambda: calls.append(1) or {"x": torch.arange(4)}
    a = m.get_or_build({"seq": "ACDE", "seed": 1, "v": "1.0"}, build)
    b = m.get_or_build({"v": "1.0", "seed": 1, "seq": "ACDE"}, build)          # order of parts does not matter
    assert len(calls) == 1 and torch.equal(a["x"], b["x"])
    m.get_or_build({"seq": "ACDF", "seed": 1, "v": "1.0"}, build)
    assert len(calls) == 2
    m2 = memo.Memo("feat", disk_dir=str(tmp_path))                              # second process: from disk
    m2.get_or_build({"seq": "ACDE", "seed": 1, "v": "1.0"}, build)
    assert len(calls) == 2 and m2.stats["disk_hit"] == 1
    m.get_or_build({"seq": "ACDE"}, build, bypass="no_seed_known")
    assert m.bypasses == {"no_seed_known": 1}
    with pytest.raises(memo.Undigestible):
        m.get_or_build({"obj": object()}, build)
    f = tmp_path / "in.fa"
    f.write_text(">a\nACDE\n")
    assert memo.file_digest(str(f)) == memo.file_digest(str(f))


def test_prefetcher_is_ordered_bounded_and_raises_in_turn():
    from uplifting_biomolecular_modeling_b200.host import workers
    running = []

    def build(i):
        running.append(i)
        time.sleep(0.01)
        if i == 3:
            raise ValueError("bad item")
        return i * i

    got = []
    with pytest.raises(workers.WorkerError) as ei:
        for item, val in workers.Prefetcher(build, range(6), workers=2, depth=2):
            got.append((item, val))
            assert max(running) <= item + 2           # never more than `depth` items ahead
    assert got == [(0, 0), (1, 1), (2, 4)] and ei.value.index == 3


def test_to_host_and_async_writer(tmp_path):
    from uplifting_biomolecular_modeling_b200.host import outputs
    tree = {"a": torch.arange(6).view(2, 3), "b": [torch.ones(2), 5], "c": (torch.zeros(1),)}
    host = outputs.to_host(tree, outputs.PinnedPool())
    assert torch.equal(host["a"], tree["a"]) and host["b"][1] == 5 and isinstance(host["c"], tuple)
    written = []
    w = outputs.AsyncWriter(lambda it: written.append(float(it["x"].sum())), workers=2, depth=2)
    x = torch.ones(4)
    w.submit({"x": x})
    x.mul_(100)                                      # the writer owns a snapshot taken at submit time
    w.submit({"x": x})
    assert w.drain() == 2 and sorted(written) == [4.0, 400.0]
    bad = outputs.AsyncWriter(lambda it: 1 / 0)
    bad.submit({})
    with pytest.raises(ZeroDivisionError):
        bad.drain()


def test_coldstart_forms(tmp_path):
    from uplifting_biomolecular_modeling_b200.host import coldstart
    ref = nn.Sequential(nn.Linear(8, 16), nn.LayerNorm(16), nn.Linear(16, 4))
    path = tmp_path / "w.pt"
    torch.save(ref.state_dict(), path)
    with coldstart.no_init() as c:
        m = nn.Sequential(nn.Linear(8, 16), nn.LayerNorm(16), nn.Linear(16, 4))
    assert c.n > 0
    assert coldstart.load_total(m, coldstart.mmap_state_dict(str(path))) == 6
    assert coldstart.state_digest(m) == coldstart.state_digest(ref)
    with coldstart.meta_init():
        mm = nn.Sequential(nn.Linear(8, 16), nn.LayerNorm(16), nn.Linear(16, 4))
    coldstart.materialize(mm, torch.load(path, weights_only=True))
    assert coldstart.state_digest(mm) == coldstart.state_digest(ref)
    part = {k: v for k, v in ref.state_dict().items() if not k.startswith("2.")}
    with pytest.raises(coldstart.PartialLoad):
        coldstart.load_total(m, part)


def test_graph_pool_site_handle_counts_calls():
    """The object a model calls (``run`` / ``stats`` / ``words``) is a site of the pool: counted in its census; on a
    machine without CUDA every call runs eagerly."""
    import torch
    from uplifting_biomolecular_modeling_b200.capture import pool
    gp = pool.GraphPool(budget_bytes=1 << 20, default_policy=pool.FixedK(2))
    gp.site("stack", verify=1)
    h = gp.handle("stack")
    x = torch.ones(3)
    for _ in range(3):
        assert torch.equal(h.run(lambda t: t * 2, x), x * 2)
    assert gp.census() == {"stack": {"calls": 3, "replays": 0}}
    assert h.stats["eager"] == 3 and h.words()[0].startswith("graphs=")


def test_capture_policies():
    from uplifting_biomolecular_modeling_b200.capture import pool
    assert pool.break_even_k(3.0, 0.5) == 6 and pool.break_even_k(1.0, 0.0) is None
    assert pool.FixedK(2).decide("k", 1)[0] == "eager" and pool.FixedK(2).decide("k", 2)[0] == "capture"
    be = pool.BreakEven(capture_s=1.0, saving_s=0.25)
    assert be.decide("k", 3)[0] == "eager" and be.decide("k", 4)[0] == "capture"
    be.observe("k", capture_s=2.0, eager_s=1.0, replay_s=0.5)
    assert be.k("k") == 4
    t = pool.Table({"a": 1}, default_k=None)
    assert t.decide("a", 1)[0] == "capture" and t.decide("b", 9) == ("eager", "no_row", True)
    p = pool.Planned({"a": 10, "b": 2}, capture_s=1.0, saving_s=0.25)
    assert p.decide("a", 1)[0] == "capture" and p.decide("b", 1)[2] is True
    gp = pool.GraphPool(budget_bytes=1 << 20)
    gp.site("step", per_item=True, enabled=False)
    assert gp.call("step", lambda x: x + 1, torch.zeros(2)).sum() == 2
    gp.new_item()
    assert gp.census()["step"]["calls"] == 1


def test_rng_discipline_and_guards():
    from uplifting_biomolecular_modeling_b200.diffusion_loop import rng, source_guard, sync_census
    g = torch.Generator().manual_seed(5)
    with rng.generator_checkpoint([g]):
        torch.randn(10, generator=g)                 # warm-up draws
    a = torch.randn(3, generator=g)
    assert torch.equal(a, torch.randn(3, generator=torch.Generator().manual_seed(5)))
    assert not rng.capture_contract_gate("whatever").ok
    drop = nn.Sequential(nn.Dropout(0.1)).train()
    assert not rng.capture_contract_gate(rng.RNG_OUTSIDE, [drop]).ok
    assert rng.capture_contract_gate(rng.RNG_OUTSIDE, [drop.eval()]).ok
    _, moved = rng.offsets_moved(lambda: torch.randn(2, generator=g), [g, torch.Generator().manual_seed(1)])
    assert moved == [(0, True), (1, False)]
    # batched items draw what they would have drawn alone
    solo = torch.Generator().manual_seed(9)
    first, second = torch.randn(4, generator=solo), torch.randn(4, generator=solo)
    forks = rng.fork_at_offsets(9, [0, 4])
    assert torch.equal(torch.randn(4, generator=forks[0]), first)
    assert torch.equal(torch.randn(4, generator=forks[1]), second)

    def stock(x):
        return x + 1
    sha = source_guard.source_sha256(stock)
    assert source_guard.source_guard(stock, [sha]).ok
    assert not source_guard.source_guard(stock, ["0" * 64]).ok
    assert not source_guard.source_guard(stock).ok
    assert source_guard.source_guard(stock, required_text=["x + 1"]).ok
    c = sync_census.sync_census(lambda: 7)
    assert c.result == 7 and c.total == 0 and c.at_most(0).ok


def test_seq_helpers():
    from uplifting_biomolecular_modeling_b200 import seq
    plans = seq.plan_batches([100, 30, 31, 500, 29], max_tokens=256, multiple=8)
    assert sorted(i for p in plans for i in p.indices) == [0, 1, 2, 3, 4]
    assert all(p.tokens <= 256 or len(p.indices) == 1 for p in plans)
    big = seq.plan_batches([4096] * 8, max_tokens=1 << 40, width=1 << 20)
    assert all(p.tokens * (1 << 20) <= 2 ** 31 - 1 or len(p.indices) == 1 for p in big)
    tab = seq.RotaryTable.get(8)
    cos, sin = tab.upto(10)
    assert cos.shape == (10, 4) and tab.builds == 1 and tab.upto(5)[0].shape == (5, 4) and tab.builds == 1
    x = torch.randn(1, 6, 2, 8)
    y = tab.apply(x, torch.arange(6))
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    assert seq.tokenizers.DNA.encode("acgtN").tolist() == [0, 1, 2, 3, 4]
    with pytest.raises(ValueError):
        seq.ByteLUT({"A": 0}).encode("AB")
    m = torch.tensor([[1, 1, 1, 0], [1, 0, 0, 0]])
    assert seq.cu_seqlens(m).tolist() == [0, 3, 4]
    assert seq.pad_to_multiple(torch.ones(2, 5, 3), 4).shape == (2, 8, 3)


def test_layer_pipeline_matches_sequential():
    from uplifting_biomolecular_modeling_b200.parallel import pipeline
    torch.manual_seed(0)
    blocks = [nn.Sequential(nn.Linear(16, 16), nn.Tanh()) for _ in range(7)]
    x = torch.randn(4, 5, 16)
    ref = x
    with torch.no_grad():
        for b in blocks:
            ref = b(ref)
    pp = pipeline.LayerPipeline(blocks, ["cpu", "cpu", "cpu"], weights=[1, 1, 1, 3, 1, 1, 1])
    assert [len(r) for r in pp.ranges] and sum(len(r) for r in pp.ranges) == 7
    assert torch.allclose(pp.forward(x, window=2), ref, atol=1e-6)
    assert [list(r) for r in pipeline.split_layers(4, 2)] == [[0, 1], [2, 3]]


def test_sample_loop_chunks():
    from uplifting_biomolecular_modeling_b200.mem import sample_loop
    seen = []

    def sample(k0, k1):
        seen.append((k0, k1))
        return torch.arange(k0, k1).float().view(-1, 1, 1).expand(-1, 3, 3).clone()

    out = sample_loop.run(sample, lambda x: {"plddt": x.mean((1, 2))}, n_samples=5, chunk=2)
    assert seen == [(0, 2), (2, 4), (4, 5)]
    assert out["coords"].shape == (5, 3, 3) and out["plddt"].tolist() == [0.0, 1.0, 2.0, 3.0, 4.0]


def test_track_writer_and_one_hot_lookup(tmp_path):
    import numpy as np
    import torch
    from uplifting_biomolecular_modeling_b200.host import tracks
    from uplifting_biomolecular_modeling_b200.models import genomics
    x = genomics.one_hot_dna("ACGTNacgt-")
    assert x.shape == (1, 10, 8) and x[0, :, 4:].sum() == 0
    assert x[0, :4, :4].equal(torch.eye(4)) and x[0, 5:9, :4].equal(torch.eye(4))
    assert x[0, 4].sum() == 0 and x[0, 9].sum() == 0
    lines = tracks.bedgraph_lines("chr1", 1000, 128, [0.5, 0.5, 0.25, 0.25, 0.25, 1.0])
    assert lines == ["chr1\t1000\t1256\t0.5", "chr1\t1256\t1640\t0.25", "chr1\t1640\t1768\t1"]
    w = tracks.TrackWriter(str(tmp_path), bin_size=128, columns=(0, 2), save_arrays=True)
    w.submit("chr1", 0, torch.tensor([[1.0, 9, 3], [1.0, 9, 4]]))
    w.submit("chr1", 256, np.array([[2.0, 9, 4], [2.0, 9, 4]]))
    assert w.close() == 5
    t0 = open(tmp_path / "track_0.bedGraph").read().splitlines()
    assert t0[0].startswith("track type=bedGraph") and t0[1:] == ["chr1\t0\t256\t1", "chr1\t256\t512\t2"]
    assert np.load(tmp_path / "chr1_256.npy").shape == (2, 3)
