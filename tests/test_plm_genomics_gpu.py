"""Kernel path of the language-model and genomic-track families on a B200 against the plain fp32 statements."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(out, ref, tol=2e-2):
    err = (out.float() - ref.float()).abs().max().item()
    scale = max(ref.float().abs().max().item(), 1.0)
    assert err <= tol * scale, (err, scale)


@pytest.mark.parametrize("D,C,R,bias", [(32, 6, 9, True), (64, 28, 100, True), (64, 70, 40, False), (32, 256, 256, True)])
def test_column_attention(D, C, R, bias):
    from uplifting_biomolecular_modeling_b200.ops import reference as Rf, seq
    g = torch.Generator(device="cuda").manual_seed(0)
    T, H = 53, 3
    q = torch.randn(T, H, D, device="cuda", generator=g).bfloat16()
    k = torch.randn(R, T, H, D, device="cuda", generator=g).bfloat16()
    v = torch.randn(R, T, H, D, device="cuda", generator=g).bfloat16()
    idx = torch.randint(0, R, (C,), device="cuda", generator=g)
    b = torch.randn(H, C, device="cuda", generator=g) if bias else None
    _close(seq.column_attention(q, k, v, idx, b), Rf.column_attention(q, k, v, idx, b))


@pytest.mark.parametrize("L,pad", [(7, 0), (96, 1), (1536, 1)])
def test_relshift_softmax(L, pad):
    from uplifting_biomolecular_modeling_b200.ops import reference as Rf, seq
    g = torch.Generator(device="cuda").manual_seed(1)
    H = 2
    content = torch.randn(H, L, L, device="cuda", generator=g) * 3
    pos = torch.randn(H, L, 2 * L - 1 + pad, device="cuda", generator=g) * 3
    out = seq.relshift_softmax(content, pos)
    ref = Rf.relshift_softmax(content, pos)
    assert (out - ref).abs().max().item() < 1e-5


def _pair(build, name, seed):
    ref = build(name, device="cuda", dtype=torch.float32, seed=seed, impl="reference")
    fused = copy.deepcopy(ref).to(torch.bfloat16).set_impl("fused")
    return ref, fused


@pytest.mark.parametrize("name,L", [("esmc_tiny", 200), ("e1_tiny", 136), ("progen2_tiny", 77), ("gpnstar_tiny", 130)])
def test_plm_fused_vs_reference(name, L):
    from uplifting_biomolecular_modeling_b200.models import plm
    from uplifting_biomolecular_modeling_b200.ops import native
    ref, fused = _pair(plm.build, name, 3)
    cfg = ref.cfg
    g = torch.Generator().manual_seed(4)
    hi = 8 if cfg.family == "gpnstar" else min(cfg.vocab, 24)
    toks = torch.randint(4, hi, (2, L), generator=g).cuda()
    kw = {}
    if cfg.family == "gpnstar":
        a, i = plm.synthetic_alignment(cfg, toks)
        kw = dict(alignment=a, clade_index=i)
    if cfg.family == "e1":
        kw = dict(seq_ids=torch.tensor([[0] * 50 + [1] * (L - 50), [0] * L]).cuda())
    n0 = native.launch_count()
    with torch.no_grad():
        got = fused(toks, **kw)
        want = ref(toks, **kw)
    torch.cuda.synchronize()
    native.raise_on_status("cuda")
    assert native.launch_count() > n0
    _close(got, want, 4e-2)


def test_progen2_fused_generate_matches_reference_greedy():
    from uplifting_biomolecular_modeling_b200.models import plm
    ref, fused = _pair(plm.build, "progen2_tiny", 5)
    toks = torch.randint(4, 24, (1, 12), generator=torch.Generator().manual_seed(6)).cuda()
    a = fused.generate(toks, 4)
    assert a.shape == (1, 16)
    # bf16 can flip near-ties; the first new token comes from a well-separated prefill distribution
    logits = ref(toks)[:, -1]
    top2 = logits.topk(2).values[0]
    if (top2[0] - top2[1]).item() > 0.05:
        assert a[0, 12].item() == logits.argmax(-1).item()


@pytest.mark.parametrize("name", ["enformer_tiny", "borzoi_tiny", "flashzoi_tiny", "chrombpnet_tiny"])
def test_track_model_fused_vs_reference(name):
    from uplifting_biomolecular_modeling_b200.models import genomics
    from uplifting_biomolecular_modeling_b200.ops import native
    ref, fused = _pair(genomics.build, name, 7)
    L = genomics.input_length(ref.cfg, bins=40)
    idx = torch.randint(0, 4, (2, L), generator=torch.Generator().manual_seed(8))
    x = torch.zeros(2, L, 8).scatter_(2, idx[..., None], 1.0).cuda()
    n0 = native.launch_count()
    with torch.no_grad():
        got = fused(x.bfloat16())
        want = ref(x)
    torch.cuda.synchronize()
    native.raise_on_status("cuda")
    assert native.launch_count() > n0
    if isinstance(want, tuple):
        _close(got[0], want[0], 4e-2)
        _close(got[1], want[1], 4e-2)
    else:
        _close(got, want, 4e-2)


@pytest.mark.parametrize("kit", ["enformer", "chrombpnet", "borzoi"])
def test_forward_graph_lever_replays_the_track_forward(kit):
    from uplifting_biomolecular_modeling_b200.kits import levers
    from uplifting_biomolecular_modeling_b200.models import lm
    from uplifting_biomolecular_modeling_b200.ops import native
    r = lm.build("genomic_track", "lm", device="cuda", kit=kit)
    want = r.run("predict", "ACGTTGCA" * 8)
    levers.LEVERS["forward_graph"].apply(r)
    got = [r.run("predict", "ACGTTGCA" * 8) for _ in range(4)]
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "forward graph")
    assert all(abs(g["score"] - want["score"]) <= 1e-3 * max(1.0, abs(want["score"])) for g in got), (want, got)
    assert r.graph_pool.census()["score_forward"]["replays"] >= 2
    assert r.last_tracks is not None and torch.isfinite(r.last_tracks.float()).all()


@pytest.mark.parametrize("family,kit", [("evo2", "evo2"), ("protein_lm", "esmc")])
def test_forward_graph_lever_replays_the_score_of_a_recurring_shape(family, kit):
    """Second sighting of a shape is captured, the third call replays; every call returns the eager score."""
    from uplifting_biomolecular_modeling_b200.kits import levers
    from uplifting_biomolecular_modeling_b200.models import lm
    from uplifting_biomolecular_modeling_b200.ops import native
    r = lm.build(family, "lm", device="cuda", kit=kit)
    if hasattr(r.model, "set_impl"):
        r.model.set_impl("fused")
    want = r.run("score", "ACGTMKV" * 9)["score"]
    ev = levers.LEVERS["forward_graph"].apply(r)
    assert ev["site"] == "score_forward"
    got = [r.run("score", "ACGTMKV" * 9)["score"] for _ in range(4)]
    other = r.run("score", "ACGT" * 5)["score"]                       # another shape: its own entry, eager first
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "forward graph")
    assert all(abs(g - want) <= 1e-3 * max(1.0, abs(want)) for g in got), (want, got)
    assert r.graph_pool.census()["score_forward"]["replays"] >= 2
    assert other == other                                             # a number, not NaN
