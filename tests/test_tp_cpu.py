"""Tensor-parallel sharding of the StripedHyena-2 model: rank threads on CPU against the replicated model."""
import torch

from uplifting_biomolecular_modeling_b200.core.testing import run_ranks
from uplifting_biomolecular_modeling_b200.models import evo2
from uplifting_biomolecular_modeling_b200.parallel import tp


def test_sharded_evo2_matches_replicated():
    ref_model = evo2.build("evo2_tiny", device="cpu", dtype=torch.float32, seed=5)
    tok = torch.randint(0, ref_model.cfg.vocab, (2, 40), generator=torch.Generator().manual_seed(0))
    ref = ref_model(tok)
    ref_gen = ref_model.generate(tok, 6)

    import copy
    copies = [copy.deepcopy(ref_model) for _ in range(2)]      # built once: rank threads share the global RNG

    def body(comm):
        m = copies[comm.rank]
        par = tp.TensorParallel(comm)
        par.shard_evo2(m)
        # a Hyena layer now holds half of the channels, an attention layer half of the heads
        assert m.blocks[0].mixer.in_proj.weight.shape[0] == 3 * m.cfg.d_model // comm.world
        return m(tok), m.generate(tok, 6), par.reduce_calls

    for out, gen, calls in run_ranks(2, body):
        assert calls > 0
        assert torch.allclose(out, ref, atol=2e-4, rtol=2e-4)
        assert torch.equal(gen, ref_gen)
