"""Language-model and genomic-track families on the CPU: the plain statements (shapes, decoding, packing,
clade de-duplication) and the wiring of the kernel path against them (kernel entry points replaced by PyTorch
stand-ins of the same contracts)."""
import dataclasses

import pytest
import torch

from tests import fake_kernels
from uplifting_biomolecular_modeling_b200.models import genomics, lm, plm
from uplifting_biomolecular_modeling_b200.ops import reference as ref


def _inputs(m, B=2, L=24, seed=0):
    g = torch.Generator().manual_seed(seed)
    cfg = m.cfg
    hi = 8 if cfg.family == "gpnstar" else min(cfg.vocab, 24)
    toks = torch.randint(4, hi, (B, L), generator=g)
    kw = {}
    if cfg.family == "gpnstar":
        a, i = plm.synthetic_alignment(cfg, toks)
        kw = dict(alignment=a, clade_index=i)
    if cfg.family == "e1":
        kw = dict(seq_ids=torch.tensor([[0] * 10 + [1] * (L - 10), [0] * L][:B]))
    return toks, kw


@pytest.mark.parametrize("name", ["esmc_tiny", "e1_tiny", "progen2_tiny", "gpnstar_tiny"])
def test_plm_kernel_path_wiring(name):
    m = plm.build(name, seed=1)
    toks, kw = _inputs(m)
    want = m.set_impl("reference")(toks, **kw)
    with fake_kernels.patched(plm):
        got = m.set_impl("fused")(toks, **kw)
    assert got.shape == (2, 24, m.cfg.vocab)
    torch.testing.assert_close(got, want, atol=2e-4, rtol=2e-4)


def test_progen2_static_slots_match_full_forward():
    m = plm.build("progen2_tiny", seed=2)
    toks, _ = _inputs(m, L=9)
    out = m.generate(toks, 5)
    assert out.shape == (2, 14)
    for t in range(9, 14):
        assert torch.equal(m(out[:, :t])[:, -1].argmax(-1), out[:, t])
    g1 = m.generate(toks, 5, temperature=0.8, top_p=0.9, generator=torch.Generator().manual_seed(3))
    g2 = m.generate(toks, 5, temperature=0.8, top_p=0.9, generator=torch.Generator().manual_seed(3))
    assert torch.equal(g1, g2)


def test_e1_packed_sequences_match_separate_runs():
    cfg = dataclasses.replace(plm.CONFIGS["e1_tiny"], name="e1_local", global_every=0)
    plm.CONFIGS[cfg.name] = cfg
    try:
        m = plm.build(cfg.name, seed=4)
    finally:
        del plm.CONFIGS[cfg.name]
    toks, _ = _inputs(m, B=1, L=24)
    ids = torch.tensor([[0] * 10 + [1] * 14])
    packed = m(toks, seq_ids=ids)
    torch.testing.assert_close(packed[:, :10], m(toks[:, :10]), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(packed[:, 10:], m(toks[:, 10:]), atol=1e-5, rtol=1e-5)


def test_gpnstar_clade_index_equals_expanded_rows():
    m = plm.build("gpnstar_tiny", seed=5)
    toks, kw = _inputs(m)
    a, idx = kw["alignment"], kw["clade_index"]
    expanded = a[:, idx]                                   # one row per clade, duplicates materialised
    same = m(toks, alignment=expanded, clade_index=torch.arange(idx.numel()))
    torch.testing.assert_close(m(toks, **kw), same, atol=1e-5, rtol=1e-5)
    vep = m.variant_effect(toks, a, idx)
    assert vep.shape == (2, 24, 4)
    # the reference allele's own entry is zero
    assert torch.allclose(vep.gather(-1, (toks - 4)[..., None]), torch.zeros(2, 24, 1), atol=1e-6)


def test_relative_shift_statement():
    L = 5
    pos = torch.arange(L * (2 * L - 1), dtype=torch.float32).view(1, L, 2 * L - 1)
    out = ref.relative_shift(pos)
    for i in range(L):
        for j in range(L):
            assert out[0, i, j] == pos[0, i, j - i + L - 1]


@pytest.mark.parametrize("name", ["enformer_tiny", "borzoi_tiny", "flashzoi_tiny", "chrombpnet_tiny"])
def test_track_model_kernel_path_wiring(name):
    m = genomics.build(name, seed=6)
    L = genomics.input_length(m.cfg)
    idx = torch.randint(0, 4, (2, L), generator=torch.Generator().manual_seed(7))
    x = torch.zeros(2, L, 8).scatter_(2, idx[..., None], 1.0)
    want = m.set_impl("reference")(x)
    with fake_kernels.patched(genomics):
        got = m.set_impl("fused")(x)
    if name.startswith("chrombpnet"):
        assert want[0].shape == (2, m.cfg.out_len) and want[1].shape == (2,)
        torch.testing.assert_close(got[0], want[0], atol=2e-4, rtol=2e-4)
        torch.testing.assert_close(got[1], want[1], atol=2e-4, rtol=2e-4)
    else:
        assert want.shape[0] == 2 and want.shape[2] == m.cfg.tracks
        torch.testing.assert_close(got, want, atol=2e-4, rtol=2e-4)


def test_conv_as_gemm_view_matches_conv1d():
    torch.manual_seed(0)
    for k, d, valid, B in [(5, 1, False, 3), (15, 1, False, 1), (3, 4, True, 2), (21, 1, True, 2), (1, 1, False, 2)]:
        conv = genomics.ConvCL(16, 24, k, dilation=d, valid=valid)
        with torch.no_grad():
            conv.weight.normal_()
            conv.bias.normal_()
        x = torch.randn(B, 40, 16)
        res = torch.randn(B, conv.out_len(40), 24)
        with fake_kernels.patched(genomics):
            got = conv.fused(x, act="relu", residual=res)
        torch.testing.assert_close(got, conv.reference(x, "relu", res), atol=1e-4, rtol=1e-4)


def test_kit_runners_cover_every_family():
    for kit, fam, verb in [("esmc", "protein_lm", "score"), ("e1", "protein_lm", "score"),
                           ("progen2", "protein_lm", "generate"), ("gpnstar", "protein_lm", "vep"),
                           ("enformer", "genomic_track", "predict"), ("borzoi", "genomic_track", "predict"),
                           ("flashzoi", "genomic_track", "predict"), ("chrombpnet", "genomic_track", "predict"),
                           ("evo2", "evo2", "score")]:
        res = lm.build(fam, "lm", kit=kit).run(verb, "ACGTMKV" * 3, 3)
        assert res and all(v == v for v in res.values() if isinstance(v, float))     # no NaN
