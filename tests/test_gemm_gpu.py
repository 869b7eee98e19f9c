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


@pytest.mark.parametrize("act", ["silu", "sigmoid", "gelu", "relu"])
def test_gemm_activation_from_a_column(act):
    """Every activation of the epilogue, applied from column 64 on (the q | k | v | gate projection's form)."""
    from uplifting_biomolecular_modeling_b200.ops import gemm, native
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randn(520, 192, device="cuda", generator=g).bfloat16()
    b = (torch.randn(320, 192, device="cuda", generator=g) * 0.1).bfloat16()
    bias = torch.randn(320, device="cuda", generator=g) * 0.1
    out = gemm.gemm(a, b, bias=bias, act=act, act_from=64, out_dtype=torch.float32)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "gemm")
    y = a.float() @ b.float().T + bias
    fn = {"silu": torch.nn.functional.silu, "sigmoid": torch.sigmoid, "gelu": torch.nn.functional.gelu,
          "relu": torch.relu}[act]
    ref = torch.cat([y[:, :64], fn(y[:, 64:])], 1)
    assert torch.allclose(out, ref, atol=4e-3, rtol=4e-3), (out - ref).abs().max().item()


@pytest.mark.parametrize("M,H,K", [(640, 192, 128), (1000, 96, 256), (7680, 1536, 768), (130, 32, 64)])
def test_gemm_swiglu3_epilogue(M, H, K):
    """silu(x Wg^T) * (x Wv^T) * (x Wb^T) formed on the accumulator of one 192-wide-tile product against the three
    separate fp32 products (H = 96 and 32 leave a tile with one column triple / part of the tile empty)."""
    from uplifting_biomolecular_modeling_b200.ops import gemm, native
    g = torch.Generator(device="cuda").manual_seed(6)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    wg, wv, wb = ((torch.randn(H, K, device="cuda", generator=g) * K ** -0.5).bfloat16() for _ in range(3))
    out = gemm.gemm(x, gemm.pack_swiglu3(wg, wv, wb), act="swiglu3")
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "gemm")
    assert out.shape == (M, H) and out.dtype == torch.bfloat16
    xf = x.float()
    ref = torch.nn.functional.silu(xf @ wg.float().T) * (xf @ wv.float().T) * (xf @ wb.float().T)
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2 * max(ref.abs().max().item(), 1.0), err
    assert ((out.float() - ref).abs().mean() / ref.abs().mean()).item() < 8e-3


@pytest.mark.parametrize("M,H,K", [(640, 256, 128), (1000, 96, 256), (4096, 11008, 512), (130, 32, 64)])
def test_gemm_swiglu_epilogue(M, H, K):
    """silu(x Wg^T) * (x Wv^T) formed on the accumulator of one 256-wide-tile product against the two separate fp32
    products (H = 96 and 32 leave the last tile partly empty)."""
    from uplifting_biomolecular_modeling_b200.ops import gemm, native
    g = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    wg, wv = ((torch.randn(H, K, device="cuda", generator=g) * K ** -0.5).bfloat16() for _ in range(2))
    out = gemm.gemm(x, gemm.pack_swiglu(wg, wv), act="swiglu")
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "gemm")
    assert out.shape == (M, H) and out.dtype == torch.bfloat16
    xf = x.float()
    ref = torch.nn.functional.silu(xf @ wg.float().T) * (xf @ wv.float().T)
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2 * max(ref.abs().max().item(), 1.0), err
    assert ((out.float() - ref).abs().mean() / ref.abs().mean()).item() < 8e-3


@pytest.mark.parametrize("M,N,K", [(300, 520, 256), (1024, 1536, 4096), (130, 96, 208), (4096, 12288, 512)])
def test_gemm_fp8_against_the_product_of_the_dequantised_operands(M, N, K):
    """e4m3 operands on the kind::f8f6f4 path: the result is the fp32 product of the very same 8-bit values (K = 208
    leaves a k-block partly empty, N = 96 / 520 a tile), with bias, activation and residual in the epilogue."""
    from uplifting_biomolecular_modeling_b200.ops import gemm, native
    g = torch.Generator(device="cuda").manual_seed(8)
    a = torch.randn(M, K, device="cuda", generator=g)
    w = torch.randn(N, K, device="cuda", generator=g) * K ** -0.5
    a8, dqa = gemm.quantize_e4m3(a)
    w8, dqw = gemm.quantize_e4m3(w)
    ref = (a8.float() * dqa) @ (w8.float() * dqw).t()
    out = gemm.gemm_fp8(a8, w8, alpha=dqa * dqw)
    dev_scale = torch.full((1,), dqa, device="cuda")
    bias = torch.randn(N, device="cuda", generator=g)
    res = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    out2 = gemm.gemm_fp8(a8, w8, alpha=dqw, alpha_dev=dev_scale, bias=bias, residual=res, act="silu")
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "gemm_fp8")
    scale = max(ref.abs().max().item(), 1.0)
    assert (out.float() - ref).abs().max().item() <= 1e-2 * scale          # bf16 rounding of the output
    ref2 = torch.nn.functional.silu(ref + bias) + res.float()
    assert (out2.float() - ref2).abs().max().item() <= 1.5e-2 * max(ref2.abs().max().item(), 1.0)
    # and the quantisation itself stays within e4m3's precision of the unquantised product
    full = a @ w.t()
    assert ((out.float() - full).abs().mean() / full.abs().mean()).item() < 6e-2


@pytest.mark.parametrize("M,N,K", [(1000, 128, 128), (384, 96, 256), (257, 128, 64)])
def test_gemm_residual_tiles_by_tma(M, N, K):
    """N <= 128 takes the 128-wide tile whose residual arrives through the shared-memory ring."""
    from uplifting_biomolecular_modeling_b200.ops import gemm, native
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = (torch.randn(N, K, device="cuda", generator=g) * K ** -0.5).bfloat16()
    bias = torch.randn(N, device="cuda", generator=g)
    res = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    out = gemm.gemm(a, b, bias=bias, residual=res)
    inplace = res.clone()
    gemm.gemm(a, b, bias=bias, residual=inplace, out=inplace)      # output over the residual
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "gemm")
    ref = a.float() @ b.float().T + bias + res.float()
    assert torch.allclose(out.float(), ref, atol=4e-2, rtol=2e-2)
    assert torch.equal(out, inplace)


def test_gemm_blocked_output_is_the_permuted_product():
    """c_blocked writes [(i, c), (j, d)] products as [(i, j), (c, d)] rows."""
    from uplifting_biomolecular_modeling_b200.ops import gemm, native
    g = torch.Generator(device="cuda").manual_seed(4)
    I, J, c, S = 6, 40, 32, 72
    a = torch.randn(I * c, S, device="cuda", generator=g).bfloat16()
    b = torch.randn(J * c, S, device="cuda", generator=g).bfloat16()
    out = torch.zeros(I * J, c * c, device="cuda", dtype=torch.bfloat16)
    gemm.gemm(a, b, alpha=0.25, out=out, c_blocked=(J * c * c, c, c * c))
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "gemm")
    ref = 0.25 * (a.float() @ b.float().T)                                  # [(i, c), (j, d)]
    ref = ref.view(I, c, J, c).permute(0, 2, 1, 3).reshape(I * J, c * c)
    assert torch.allclose(out.float(), ref, atol=5e-2, rtol=2e-2)
