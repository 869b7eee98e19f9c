"""StripedHyena-2 decoder on CPU: decode steps reproduce the prefill, FFT convolution equals the FIR."""
import pytest
import torch

from uplifting_biomolecular_modeling_b200.models import evo2


def test_layer_pattern_of_the_7b_shape():
    cfg = evo2.CONFIGS["evo2_7b"]
    kinds = [cfg.layer_kind(i) for i in range(cfg.n_layers)]
    assert kinds.count("attn") == 5 and kinds[3] == "attn" and kinds[31] == "attn"
    assert kinds[:3] == ["hcs", "hcm", "hcl"] and kinds.count("hcs") == 9


def test_fft_conv_equals_fir():
    torch.manual_seed(0)
    x = torch.randn(2, 50, 6, dtype=torch.float64)
    h = torch.randn(6, 9, dtype=torch.float64)
    assert torch.allclose(evo2.fft_causal_conv(x, h), evo2.causal_fir(x, h), atol=1e-5)


def test_decode_steps_match_prefill():
    m = evo2.build("evo2_tiny", dtype=torch.float64)
    toks = torch.randint(0, 512, (1, 24))
    full = m.forward(toks)
    states = [dict() for _ in m.blocks]
    pre = m.forward(toks[:, :16], states)
    assert torch.allclose(pre, full[:, :16], atol=2e-4)     # long filters run as fp32 FFT convolutions
    for t in range(16, 24):
        lg = m.step(toks[:, t:t + 1], states)
        assert torch.allclose(lg[:, 0], full[:, t], atol=2e-4), t
    out = m.generate(toks[:, :8], 5)
    assert out.shape == (1, 5)
    assert torch.isfinite(m.score(toks)).all()


def test_static_state_decode_equals_plain_decode():
    """Fixed-address states (what a captured decode graph uses) give the same tokens as the growing ones."""
    import torch
    from uplifting_biomolecular_modeling_b200.models import evo2
    m = evo2.build("evo2_tiny", device="cpu", dtype=torch.float32, seed=2)
    tok = torch.randint(0, m.cfg.vocab, (1, 30), generator=torch.Generator().manual_seed(3))
    ref = m.generate(tok, 8)
    states = [dict() for _ in m.blocks]
    nxt = m(tok, states)[:, -1:].argmax(-1)
    pos = m.make_static_states(states, 30 + 8)
    outs = [nxt]
    for _ in range(7):
        nxt = m.step(nxt, states)[:, -1:].argmax(-1)
        pos.add_(1)
        outs.append(nxt)
    assert torch.equal(torch.cat(outs, 1), ref)


def test_multi_token_continuation_equals_single_steps():
    """extend(k tokens) + commit(j) leaves the states where j single-token steps would, and gives their logits."""
    from uplifting_biomolecular_modeling_b200.models import evo2
    m = evo2.build("evo2_tiny", seed=3)
    toks = torch.randint(0, 4, (1, 37), generator=torch.Generator().manual_seed(0))
    nxt = torch.randint(0, 4, (1, 5), generator=torch.Generator().manual_seed(1))
    a = [dict() for _ in m.blocks]
    b = [dict() for _ in m.blocks]
    m.forward(toks, a)
    m.forward(toks, b)
    step_logits = torch.cat([m.step(nxt[:, i:i + 1], a) for i in range(3)], 1)
    ext = m.extend(nxt, b)
    torch.testing.assert_close(ext[:, :3], step_logits, atol=2e-4, rtol=2e-4)
    m.commit(b, 3)
    # both state sets now continue identically
    torch.testing.assert_close(m.step(nxt[:, 3:4], a), m.step(nxt[:, 3:4], b), atol=2e-4, rtol=2e-4)


def test_speculative_decoding_reproduces_greedy_decoding():
    from uplifting_biomolecular_modeling_b200.models import evo2
    target = evo2.build("evo2_tiny", seed=3)
    toks = torch.randint(0, 4, (1, 29), generator=torch.Generator().manual_seed(2))
    want = target.generate(toks, 20)
    # a draft with other weights: proposals are mostly rejected, the output must not change
    other = evo2.build("evo2_tiny", seed=11)
    got, stats = target.generate_speculative(other, toks, 20, k=4)
    assert torch.equal(got, want), (got, want)
    assert stats["proposed"] == 4 * stats["rounds"]
    # the target as its own draft: every proposal is accepted, k + 1 tokens per round
    got2, stats2 = target.generate_speculative(target, toks, 20, k=4)
    assert torch.equal(got2, want)
    assert stats2["accepted"] == stats2["proposed"] and stats2["rounds"] == 4


def test_filter_spectra_are_cached_per_length_and_follow_the_weights():
    from uplifting_biomolecular_modeling_b200.models import evo2
    m = evo2.build("evo2_tiny", seed=5)
    toks = torch.randint(0, 4, (1, 96), generator=torch.Generator().manual_seed(0))
    a = m(toks)
    ops = [b.mixer for b in m.blocks if getattr(b.mixer, "kind", None) in ("hcm", "hcl")]
    assert ops and all(len(o.__dict__.get("_spectra", {})) == 1 for o in ops)
    first = [next(iter(o._spectra.values()))[1] for o in ops]
    b = m(toks)
    assert torch.equal(a, b)
    assert all(next(iter(o._spectra.values()))[1] is f for o, f in zip(ops, first))       # reused, not recomputed
    m(toks[:, :80])
    m(toks[:, :72])
    assert all(len(o._spectra) == 2 for o in ops)                                          # bounded
    hcl = next(o for o in ops if o.kind == "hcl")
    with torch.no_grad():
        hcl.residues.mul_(1.5)                                                             # bumps the version
    c = m(toks)
    assert not torch.equal(a, c)


def test_oversized_filter_spectra_are_not_kept(monkeypatch):
    from uplifting_biomolecular_modeling_b200.models import evo2
    m = evo2.build("evo2_tiny", seed=5)
    toks = torch.randint(0, 4, (1, 96), generator=torch.Generator().manual_seed(0))
    want = m(toks)
    for b in m.blocks:
        b.mixer.__dict__.pop("_spectra", None)
    monkeypatch.setattr(evo2, "SPECTRUM_CACHE_MAX_BYTES", 16)
    got = m(toks)
    assert torch.equal(got, want)
    assert all(not b.mixer.__dict__.get("_spectra") for b in m.blocks)


def test_e4m3_weight_quantisation_bounds():
    """Per-tensor e4m3 form of a weight: the maximum maps to 448, every value is within half a 3-bit mantissa step."""
    from uplifting_biomolecular_modeling_b200.ops import gemm
    g = torch.Generator().manual_seed(0)
    w = torch.randn(64, 96, generator=g) * 0.07
    q, dq = gemm.quantize_e4m3(w)
    assert q.dtype == torch.float8_e4m3fn and q.shape == w.shape
    amax = w.abs().max().item()
    assert abs(dq * 448.0 - amax) < 1e-6 * amax
    back = q.float() * dq
    assert back.abs().max().item() == pytest.approx(amax, rel=1e-6)
    assert ((back - w).abs() <= 0.0625 * w.abs() + 2.0 ** -9 * amax).all()


def test_runner_scores_through_the_capture_site_only_when_it_may():
    """The ``forward_graph`` site is asked for GPU inputs below the token limit; on the CPU the model scores directly."""
    from uplifting_biomolecular_modeling_b200.models import lm

    class Site:
        calls = 0

        def run(self, fn, *tensors):
            Site.calls += 1
            return fn(*tensors)

    r = lm.build("evo2", "evo2_tiny", seed=0, kit="evo2")
    want = r.run("score", "ACGTACGTAC")["score"]
    r.forward_graphs = Site()
    assert r.run("score", "ACGTACGTAC")["score"] == want and Site.calls == 0        # CPU tensors: never captured


def test_checkpoint_dry_run_against_a_meta_model(tmp_path):
    """A launcher's check before rank processes start: names and shapes against a model that holds no memory."""
    from uplifting_biomolecular_modeling_b200.models import weights
    m = evo2.build("evo2_tiny", seed=3)
    torch.save(m.state_dict(), tmp_path / "full.pt")
    k0 = next(iter(m.state_dict()))
    torch.save({k0: m.state_dict()[k0]}, tmp_path / "one.pt")
    with torch.device("meta"):
        probe = evo2.StripedHyena2(evo2.CONFIGS["evo2_tiny"])
    rep = weights.load_checkpoint(probe, str(tmp_path / "full.pt"), strict=True, dry_run=True)
    assert rep.complete and rep.matched == len(m.state_dict())
    assert all(p.is_meta for p in probe.parameters())                  # nothing was written
    with pytest.raises(ValueError, match="missing"):
        weights.load_checkpoint(probe, str(tmp_path / "one.pt"), strict=True, dry_run=True)
    assert weights.load_checkpoint(probe, str(tmp_path / "one.pt"), strict=False, dry_run=True).matched == 1
