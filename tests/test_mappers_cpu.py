"""Upstream Pairformer checkpoints (Protenix, OpenFold3) through the name mappers into this package's modules: every
upstream key of the written-down key lists is consumed, the mapped state loads with ``strict=True``, the merged
triangle-multiplication matrices hold the ``a`` operand first, and anything the tables do not name stays visible."""
import os

import pytest
import torch

from uplifting_biomolecular_modeling_b200.models import mappers, pairformer, weights

DATA = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data")


def _block_keys(upstream):
    out = []
    for line in open(os.path.join(DATA, f"{upstream}_pairformer_block_keys.txt")):
        if line.startswith("#") or not line.strip():
            continue
        name, *shape = line.split()
        out.append((name, tuple(int(s) for s in shape)))
    return out


def _stack_state(upstream, blocks, prefix=""):
    g = torch.Generator().manual_seed(5)
    return {f"{prefix}blocks.{i}.{k}": torch.randn(shape, generator=g) for i in range(blocks) for k, shape in _block_keys(upstream)}


@pytest.mark.parametrize("upstream", ["protenix", "openfold3"])
def test_every_upstream_key_is_consumed_and_the_stack_loads_strictly(upstream):
    st = _stack_state(upstream, 2)
    mapped = mappers.map_pairformer_stack(st, upstream)
    own = pairformer.PairformerModule(384, 128, num_blocks=2)
    assert not any(k.startswith("blocks.") for k in mapped), [k for k in mapped if k.startswith("blocks.")][:3]
    own.load_state_dict(mapped, strict=True)
    # a operand first, then b; the output projection and its gate keep their roles
    pre = "blocks.1." + mappers.UPSTREAMS[upstream]["pair_prefix"]
    w = own.layers[1].tri_mul_in
    assert torch.equal(w.p_in.weight[:128], st[pre + "tri_mul_in.linear_a_p.weight"])
    assert torch.equal(w.p_in.weight[128:], st[pre + "tri_mul_in.linear_b_p.weight"])
    assert torch.equal(w.g_in.weight[:128], st[pre + "tri_mul_in.linear_a_g.weight"])
    assert torch.equal(w.p_out.weight, st[pre + "tri_mul_in.linear_z.weight"])
    assert torch.equal(w.g_out.weight, st[pre + "tri_mul_in.linear_g.weight"])
    tr = own.layers[0].transition_z
    names = {"protenix": ("linear_no_bias_a", "linear_no_bias_b", "linear_no_bias"),
             "openfold3": ("swiglu.linear_a", "swiglu.linear_b", "linear_out")}[upstream]
    p0 = "blocks.0." + mappers.UPSTREAMS[upstream]["pair_prefix"] + "pair_transition."
    assert torch.equal(tr.fc1.weight, st[p0 + names[0] + ".weight"])       # the SiLU branch
    assert torch.equal(tr.fc2.weight, st[p0 + names[1] + ".weight"])
    assert torch.equal(tr.fc3.weight, st[p0 + names[2] + ".weight"])


def test_an_unknown_key_and_a_missing_matrix_are_not_hidden():
    st = _stack_state("protenix", 1)
    st["blocks.0.tri_att_start.mha.linear_o.bias"] = torch.zeros(128)      # this package has no such parameter
    mapped = mappers.map_pairformer_stack(st, "protenix")
    assert "blocks.0.tri_att_start.mha.linear_o.bias" in mapped           # passed through: a strict load reports it
    with pytest.raises(RuntimeError):
        pairformer.PairformerModule(384, 128, num_blocks=1).load_state_dict(mapped, strict=True)
    del st["blocks.0.tri_mul_out.linear_b_g.weight"]
    with pytest.raises(mappers.MapperError, match="linear_b_g"):
        mappers.map_pairformer_stack(st, "protenix")


def test_a_layer_norm_without_offset_maps_to_a_zero_offset():
    st = _stack_state("protenix", 1)
    del st["blocks.0.attention_pair_bias.layernorm_z.bias"]
    mapped = mappers.map_pairformer_stack(st, "protenix")
    assert not mapped["layers.0.attention.proj_z.0.bias"].any()


def test_kit_mapper_feeds_the_checkpoint_loader(tmp_path):
    """A whole-model style checkpoint: the trunk stack under the upstream's prefix, loaded into a model that has the
    stack under this package's prefix."""
    class Trunk(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.pairformer_module = pairformer.PairformerModule(384, 128, num_blocks=1)

    assert mappers.for_kit("boltz2") is None
    st = _stack_state("openfold3", 1, prefix="pairformer_stack.")
    path = tmp_path / "of3.pt"
    torch.save(st, path)
    m = Trunk()
    rep = weights.load_checkpoint(m, str(path), strict=True, mapper=mappers.for_kit("openfold3"))
    assert rep.complete and rep.matched == len(m.state_dict())
    with pytest.raises(ValueError):                                        # without the mapper nothing matches
        weights.load_checkpoint(Trunk(), str(path), strict=True)
