"""tcgen05 GEMM against a plain fp32 PyTorch reference of the same contraction."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, mn_major):
    a32, b32 = a.float(), b.float()
    if mn_major:
        return torch.einsum("bkm,bkn->bmn", a32, b32)
    return torch.einsum("bmk,bnk->bmn", a32, b32)


@pytest.mark.parametrize("mn_major", [False, True])
@pytest.mark.parametrize("shape", [(1, 128, 128, 64), (2, 256, 256, 128), (3, 384, 320, 192), (2, 200, 136, 72),
                                   (4, 512, 512, 512)])
def test_gemm_matches_fp32(shape, mn_major):
    from uplifting_biomolecular_modeling_b200.ops import gemm, native
    batch, M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(1)
    if mn_major:
        a = torch.randn(batch, K, M, device="cuda", generator=g).bfloat16()
        b = torch.randn(batch, K, N, device="cuda", generator=g).bfloat16()
    else:
        a = torch.randn(batch, M, K, device="cuda", generator=g).bfloat16()
        b = torch.randn(batch, N, K, device="cuda", generator=g).bfloat16()
    out = gemm.gemm(a, b, mn_major=mn_major, out_dtype=torch.float32)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "gemm")
    ref = _ref(a, b, mn_major)
    err = (out - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 2e-3 * max(scale, 1.0), (err, scale)


def test_gemm_epilogue_bias_residual_act():
    from uplifting_biomolecular_modeling_b200.ops import gemm, native
    g = torch.Generator(device="cuda").manual_seed(2)
    a = torch.randn(300, 128, device="cuda", generator=g).bfloat16()
    b = torch.randn(264, 128, device="cuda", generator=g).bfloat16()
    bias = torch.randn(264, device="cuda", generator=g)
    res = torch.randn(300, 264, device="cuda", generator=g).bfloat16()
    out = gemm.gemm(a, b, bias=bias, residual=res, act="silu", alpha=0.5)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "gemm")
    ref = torch.nn.functional.silu(0.5 * (a.float() @ b.float().T) + bias) + res.float()
    assert out.dtype == torch.bfloat16
    assert torch.allclose(out.float(), ref, atol=6e-2, rtol=2e-2)
