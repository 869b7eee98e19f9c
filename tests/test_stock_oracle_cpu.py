"""Parity with the upstream model code: the stock Boltz-2 modules (installed unmodified from the reference's wheel
under ``baseline/_ref``) give their ``state_dict()`` to this package's modules with ``strict=True``, and both run
the same fp32 inputs on CPU, with padding masks.  One test proves parameter names, shapes and the arithmetic.
Skipped when the stock package is not installed."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "boltz")),
                                reason="stock boltz package not installed under baseline/_ref")


@pytest.fixture(scope="module")
def stock():
    sys.path.insert(0, REF)
    try:
        from boltz.model.layers import pairformer as sp
        from boltz.model.modules import trunkv2 as st
        yield sp, st
    finally:
        sys.path.remove(REF)


def _randomize(module):
    """Upstream zero-initialises its output projections ("final" init): with fresh weights every update would be
    zero and any two implementations would agree.  Give every parameter a random value instead."""
    g = torch.Generator().manual_seed(123)
    with torch.no_grad():
        for p in module.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * (0.3 if p.dim() == 1 else p.shape[-1] ** -0.5))
    return module


def _masks(N, pad):
    mask = torch.ones(1, N)
    mask[:, N - pad:] = 0
    return mask, mask[:, :, None] * mask[:, None, :]


def test_pairformer_stack_matches_stock_with_masks(stock):
    sp, _ = stock
    from uplifting_biomolecular_modeling_b200.models import pairformer
    torch.manual_seed(0)
    ref = _randomize(sp.PairformerModule(384, 128, num_blocks=2, v2=True)).eval()
    own = pairformer.PairformerModule(384, 128, num_blocks=2).eval()
    own.load_state_dict(ref.state_dict(), strict=True)
    N = 40
    s, z = torch.randn(1, N, 384), torch.randn(1, N, N, 128)
    mask, pm = _masks(N, 6)
    with torch.no_grad():
        s1, z1 = ref(s, z, mask, pm)
        s2, z2 = own(s, z, mask, pm)
    assert torch.allclose(s1, s2, atol=2e-4, rtol=1e-4), (s1 - s2).abs().max()
    assert torch.allclose(z1, z2, atol=2e-4, rtol=1e-4), (z1 - z2).abs().max()
    # the mask matters: without it the valid rows change
    with torch.no_grad():
        _, z3 = own(s, z, None, None)
    assert (z3[:, :N - 6, :N - 6] - z2[:, :N - 6, :N - 6]).abs().max() > 1e-3


def test_no_seq_pairformer_matches_stock(stock):
    sp, _ = stock
    from uplifting_biomolecular_modeling_b200.models import pairformer
    torch.manual_seed(1)
    ref = _randomize(sp.PairformerNoSeqModule(128, num_blocks=1)).eval()
    own = pairformer.PairformerModule(384, 128, num_blocks=1, no_seq=True).eval()
    own.load_state_dict(ref.state_dict(), strict=True)
    N = 24
    z = torch.randn(1, N, N, 128)
    _, pm = _masks(N, 3)
    with torch.no_grad():
        z1 = ref(z, pm)
        _, z2 = own(None, z, None, pm)
    assert torch.allclose(z1, z2, atol=2e-4, rtol=1e-4), (z1 - z2).abs().max()


def test_msa_module_matches_stock(stock):
    _, st = stock
    from boltz.data import const
    from uplifting_biomolecular_modeling_b200.models import msa
    torch.manual_seed(2)
    ref = _randomize(st.MSAModule(msa_s=64, token_z=128, token_s=384, msa_blocks=2, msa_dropout=0.0, z_dropout=0.0)).eval()
    nfeat = const.num_tokens + 3
    own = msa.MSAModule(64, 128, 384, num_blocks=2, msa_feat=nfeat).eval()
    own.load_state_dict(ref.state_dict(), strict=True)
    N, S = 20, 5
    z, emb = torch.randn(1, N, N, 128), torch.randn(1, N, 384)
    mask, pm = _masks(N, 4)
    msa_mask = (torch.rand(1, S, N) > 0.1).float() * mask[:, None, :]
    feats = {"msa": torch.randint(0, const.num_tokens, (1, S, N)), "has_deletion": torch.randint(0, 2, (1, S, N)).float(),
             "deletion_value": torch.rand(1, S, N), "msa_paired": torch.randint(0, 2, (1, S, N)).float(),
             "msa_mask": msa_mask, "token_pad_mask": mask}
    msa_feat = torch.cat([torch.nn.functional.one_hot(feats["msa"], const.num_tokens).float(),
                          feats["has_deletion"][..., None], feats["deletion_value"][..., None],
                          feats["msa_paired"][..., None]], -1)
    with torch.no_grad():
        z1 = ref(z, emb, feats)
        z2 = own(z, emb, msa_feat, msa_mask, mask, pm)
    assert torch.allclose(z1, z2, atol=2e-4, rtol=1e-4), (z1 - z2).abs().max()


def test_diffusion_transformer_matches_stock(stock):
    """Token transformer of the diffusion module: stock ``DiffusionTransformer`` (AdaLN, pair-bias attention shared
    over the samples, conditioned SwiGLU transition) against this package's, same weights by strict load - the
    parameter names (``output_projection.0``, ``swish_gate.0``) and which SwiGLU half is the gate are upstream's."""
    from boltz.model.modules import transformersv2 as st
    from uplifting_biomolecular_modeling_b200.models import diffusion
    torch.manual_seed(4)
    depth, heads, dim, N, mult = 2, 16, 768, 10, 3
    ref = _randomize(st.DiffusionTransformer(depth=depth, heads=heads, dim=dim, dim_single_cond=dim)).eval()
    own = diffusion.DiffusionTransformer(depth, dim, dim, heads).eval()
    own.load_state_dict(ref.state_dict(), strict=True)
    a, s = torch.randn(mult, N, dim), torch.randn(mult, N, dim)
    bias = torch.randn(1, N, N, depth * heads)
    mask = torch.ones(mult, N)
    with torch.no_grad():
        out_ref = ref(a, s, bias=bias, mask=mask, multiplicity=mult)
        b5 = bias.view(1, N, N, depth, heads)
        biases = [b5[:, :, :, i].permute(0, 3, 1, 2) for i in range(depth)]          # [1, H, N, N] per layer
        out_own = own(a, s, biases, mask[:1], multiplicity=mult)        # this package repeats the mask over samples itself
    assert torch.allclose(out_ref, out_own, atol=3e-4, rtol=1e-4), (out_ref - out_own).abs().max()
