"""Causal attention at head dimension 128 (tcgen05 kernel) against the plain fp32 statement of the same attention."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,Tq,Tk,H,Hkv", [(1, 128, 128, 2, 2), (2, 384, 384, 3, 3), (1, 200, 200, 4, 2),
                                           (1, 1000, 1000, 2, 1), (1, 64, 448, 2, 2), (2, 130, 517, 2, 2),
                                           (1, 2048, 2048, 2, 2)])
def test_causal_attention_matches_fp32(B, Tq, Tk, H, Hkv):
    from uplifting_biomolecular_modeling_b200.ops import causal, native
    g = torch.Generator(device="cuda").manual_seed(Tq + Tk)
    q = torch.randn(B, Tq, H, 128, device="cuda", generator=g).bfloat16()
    k = torch.randn(B, Tk, Hkv, 128, device="cuda", generator=g).bfloat16()
    v = torch.randn(B, Tk, Hkv, 128, device="cuda", generator=g).bfloat16()
    out = causal.causal_attention(q, k, v)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "causal attention")
    ref = causal.reference(q, k, v)
    assert out.shape == ref.shape and out.dtype == torch.bfloat16
    err = (out.float() - ref).abs().max().item()
    assert err < 3e-2, err
    assert ((out.float() - ref).abs().mean() / ref.abs().mean()).item() < 1.5e-2


def test_causal_attention_on_column_slices_of_one_projection_and_a_scale():
    """q | k | v as views of one [B, T, 3 * H * 128] projection output (row stride 3 * H * 128), custom scale."""
    from uplifting_biomolecular_modeling_b200.ops import causal, native
    B, T, H = 1, 512, 4
    g = torch.Generator(device="cuda").manual_seed(9)
    qkv = torch.randn(B, T, 3, H, 128, device="cuda", generator=g).bfloat16()
    q, k, v = qkv.unbind(2)
    out = causal.causal_attention(q, k, v, scale=0.05)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "causal attention")
    ref = causal.reference(q, k, v, scale=0.05)
    assert (out.float() - ref).abs().max().item() < 3e-2


def test_evo2_attention_layer_on_the_causal_kernel_matches_the_library_path(monkeypatch):
    """The attention operator of the StripedHyena-2 model with the kernel path switched on against the same module
    on the plain path (head dimension 128, rotary positions, 300 tokens)."""
    from uplifting_biomolecular_modeling_b200.models import evo2
    from uplifting_biomolecular_modeling_b200.ops import causal, native
    monkeypatch.setattr(causal, "ENABLED", True)
    torch.manual_seed(0)
    cfg = evo2.Evo2Config(d_model=512, n_heads=4, n_layers=4, ffn=1024)
    op = evo2.AttentionOperator(cfg).cuda().to(torch.bfloat16).eval()
    x = torch.randn(1, 300, 512, device="cuda").bfloat16()
    with torch.no_grad():
        want = op(x)
        op.impl = "fused"
        before = native.launch_count()
        got = op(x)
        assert native.launch_count() > before
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "evo2 attention")
    assert (got.float() - want.float()).abs().max().item() < 3e-2
