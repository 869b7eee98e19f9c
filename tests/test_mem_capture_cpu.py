"""Memory levers and capture helpers on CPU."""
import torch

from uplifting_biomolecular_modeling_b200 import mem
from uplifting_biomolecular_modeling_b200.capture import graphs, hoist
from uplifting_biomolecular_modeling_b200.mem import chunk, ckpt, offload, peak, registry
from uplifting_biomolecular_modeling_b200.models import pairformer


def test_rowchunk_is_bitwise():
    torch.manual_seed(0)
    t = pairformer.Transition(16, 32).eval()
    x = torch.randn(1, 10, 10, 16)
    with torch.no_grad():
        ref = t(x, residual=True)
        out = chunk.transition_chunked(x, t, 3, residual=True)
    assert torch.equal(out, ref)
    assert chunk.rows_within(1000, 30, multiple=8) == 32 and chunk.rows_within(10, 30, minimum=8) == 8


def test_triatt_chunked_equals_unchunked():
    torch.manual_seed(0)
    for starting in (True, False):
        m = pairformer.TriangleAttention(16, 8, 2, starting=starting).double().eval()
        z = torch.randn(9, 9, 16, dtype=torch.float64)
        with torch.no_grad():
            ref = m(z.unsqueeze(0), None, residual=True)[0]
            out = chunk.triangle_attention_chunked(z, m, 4, residual=True)
        assert torch.allclose(out, ref, atol=1e-12)


def test_registry_apply_and_gate():
    model = pairformer.PairformerLayer(c_s=32, c_z=128, heads=4, pair_heads=4, no_seq=True)
    ctx = registry.Ctx(hooks={"model": model}, settings={"chunk_rows": 4})
    rec = mem.apply("chunk_transition,chunk_triatt,nonexistent", ctx)
    assert rec.applied == ["chunk_transition", "chunk_triatt"] and rec.refused == {"nonexistent": "unknown_lever"}
    assert rec.active_fields().startswith("mode=big:chunk_transition,chunk_triatt base=fast exact=true")
    assert rec.gate() == "refused:nonexistent"
    rec2 = mem.apply("chunk_transition", registry.Ctx())
    assert rec2.refused == {"chunk_transition": "hook_missing:model"}
    assert "chunk_transition" in registry.compose_big({"fast": ["a"]}, "fast", drop=["cache_release"])


def test_offload_stream_blocks_cpu():
    x = torch.arange(20.).view(10, 2)
    p = offload.HostPark(x)
    offload.stream_blocks(p, lambda b, a0, a1: b * 2, rows=3, device="cpu")
    assert torch.equal(p.host, x * 2)


def test_sample_chunks_draw_order():
    assert ckpt.sample_chunks(5, 2) == [(0, 2), (2, 4), (4, 5)]
    g = torch.Generator().manual_seed(1)
    ref = torch.randn((5, 3), generator=torch.Generator().manual_seed(1))
    d = ckpt.StockOrderDraws(5, g)
    got = torch.cat([d.draw("eps0", (3,), a, b) for a, b in ckpt.sample_chunks(5, 2)])
    assert torch.equal(got, ref)


def test_peak_fit_and_memo():
    a, b = peak.fit_a_b([(1, 110.0), (2, 60.0), (4, 35.0)])
    assert abs(a - 10.0) < 1e-6 and abs(b - 100.0) < 1e-6
    memo = hoist.ConstMemo()
    t = torch.ones(3)
    calls = []
    f = lambda x: (calls.append(1), x * 2)[1]  # noqa: E731
    memo.get("k", f, t); memo.get("k", f, t)
    assert len(calls) == 1
    t.add_(1)
    memo.get("k", f, t)
    assert len(calls) == 2
    x = torch.tensor([[1., 2.], [1., 2.], [3., 4.]])
    assert torch.equal(hoist.RowDedup.apply(lambda r: r * 10, x), x * 10)
    gc = graphs.GraphCache(enabled=False)
    assert torch.equal(gc.run(lambda u: u + 1, t), t + 1) and gc.stats["eager"] == 1
