"""Design-side models on the CPU: gradients through the trunk with checkpointed blocks, batch-invariant decoding."""
import torch

from uplifting_biomolecular_modeling_b200.models import cofold, design


def _tiny():
    m = cofold.build_model("tiny", device="cpu", dtype=torch.float32, seed=0)
    feats = cofold.synthetic_features(16, 4, m.cfg, seed=0)
    return m, feats


def test_checkpointed_backward_equals_plain_backward_and_weights_get_no_gradient():
    m, feats = _tiny()
    target = torch.randint(0, m.cfg.distogram_bins, (1, 16, 16), generator=torch.Generator().manual_seed(1))
    a = design.SequenceInversion(m, feats, target, use_checkpoint=True, seed=3)
    b = design.SequenceInversion(m, feats, target, use_checkpoint=False, seed=3)
    la, lb = a.loss(), b.loss()
    la.backward()
    lb.backward()
    torch.testing.assert_close(la, lb)
    torch.testing.assert_close(a.logits.grad, b.logits.grad, atol=1e-6, rtol=1e-5)
    assert a.logits.grad.abs().sum() > 0
    assert all(p.grad is None for p in m.parameters())                # input gradients only


def test_inversion_lowers_its_loss():
    m, feats = _tiny()
    with torch.no_grad():                                             # a reachable target: the model's own distogram
        f = dict(feats)
        s_in, s0, z0, _, _ = m.embed(f)
        _, z = design.trunk_checkpointed(m, f, s_in, s0, z0, 0, False)
        target = m.distogram_module(z).argmax(-1)
    inv = design.SequenceInversion(m, feats, target, lr=0.3, seed=5)
    losses = [inv.step() for _ in range(6)]
    assert losses[-1] < losses[0]
    assert inv.sequence().shape == (1, 16)


def test_decoder_sampling_does_not_depend_on_batch_composition():
    dec = design.build_decoder(seed=0, dim=32, k=6, enc_layers=2, dec_layers=2)
    x = torch.randn(1, 14, 3, generator=torch.Generator().manual_seed(2)) * 4
    together = dec.sample(x, seeds=[11, 12, 13], temperature=0.5)
    alone = torch.cat([dec.sample(x, seeds=[s], temperature=0.5) for s in (11, 12, 13)])
    assert together.shape == (3, 14) and torch.equal(together, alone)
    assert not torch.equal(together[0], together[1])                  # different streams, different sequences
    assert torch.equal(dec.sample(x, seeds=[11], temperature=0.5), together[:1])
    assert int(together.max()) < design.N_TYPES


def test_decoder_never_sees_residues_that_are_not_decoded_yet():
    dec = design.build_decoder(seed=1, dim=32, k=5, enc_layers=1, dec_layers=1)
    x = torch.randn(1, 9, 3, generator=torch.Generator().manual_seed(3)) * 4
    order, _ = dec.draws(9, [7])
    seq = dec.sample(x, seeds=[7], temperature=0.5)
    # changing what the decoder would embed for the LAST decoded token cannot change any earlier choice
    last = int(order[0, -1])
    emb = dec.seq_embed.weight.data
    saved = emb[seq[0, last]].clone()
    emb[seq[0, last]] += 5.0 if (seq[0] == seq[0, last]).sum() == 1 else 0.0
    again = dec.sample(x, seeds=[7], temperature=0.5)
    emb[seq[0, last]] = saved
    keep = torch.ones(9, dtype=torch.bool)
    keep[last] = False
    if (seq[0] == seq[0, last]).sum() == 1:
        assert torch.equal(again[0, keep], seq[0, keep])
