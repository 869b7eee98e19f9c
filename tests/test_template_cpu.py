"""Template embedder: shapes and the mean-over-templates contract on CPU (plain statements)."""
import torch

from uplifting_biomolecular_modeling_b200.models import template


def test_template_embedder_forward_cpu():
    torch.manual_seed(0)
    N, T = 24, 3
    asym = torch.tensor([0] * 14 + [1] * 10)
    m = template.TemplateEmbedder(c_z=128, n_blocks=1).eval()
    f = template.synthetic_template_features(N, T, asym)
    z = torch.randn(1, N, N, 128)
    with torch.no_grad():
        out = m(z, f)
        # identical templates: the mean over templates equals the single-template result
        f1 = {k: (v[:1] if v.dim() > 1 and v.shape[0] == T else v) for k, v in f.items()}
        f3 = {k: (v[:1].expand(T, *v.shape[1:]) if v.dim() > 1 and v.shape[0] == T else v) for k, v in f.items()}
        a, b = m(z, f1), m(z, f3)
    assert out.shape == (1, N, N, 128) and torch.isfinite(out).all()
    assert torch.allclose(a, b, atol=1e-5, rtol=1e-5)


def test_cofold_trunk_uses_templates_when_given():
    from uplifting_biomolecular_modeling_b200.models import cofold
    m = cofold.build_model("tiny", device="cpu", dtype=torch.float32, seed=0, template_blocks=1)
    f = cofold.synthetic_features(32, 4, m.cfg)
    tf = template.synthetic_template_features(32, 2, f["chain_id"][0])
    with torch.no_grad():
        si, s0, z0, _, _ = m.embed(f)
        _, z_plain = m.trunk(f, si, s0, z0, 0)
        f.update({k: v[None] for k, v in tf.items() if k.startswith("template_")})
        _, z_tmpl = m.trunk(f, si, s0, z0, 0)
    assert torch.isfinite(z_tmpl).all()
    assert (z_tmpl - z_plain).abs().max().item() > 0
