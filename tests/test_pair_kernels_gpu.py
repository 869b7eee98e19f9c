"""Fused pair-stack kernels against the plain PyTorch fp32 statements of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(out, ref):
    return ((out.float() - ref.float()).abs().max() / ref.float().abs().max().clamp(min=1e-6)).item()


def _rand(shape, g, scale=1.0):
    return torch.randn(shape, device="cuda", generator=g) * scale


@pytest.mark.parametrize("N", [64, 200, 384])
@pytest.mark.parametrize("hidden", [512, 256])
def test_transition(N, hidden):
    from uplifting_biomolecular_modeling_b200.ops import native, pair, reference
    g = torch.Generator(device="cuda").manual_seed(3)
    c = 128
    x = (_rand((N, N, c), g) + 0.3).bfloat16()
    nw, nb = 1.0 + 0.1 * _rand((c,), g), 0.1 * _rand((c,), g)
    fc1, fc2 = _rand((hidden, c), g, c ** -0.5), _rand((hidden, c), g, c ** -0.5)
    fc3 = _rand((c, hidden), g, hidden ** -0.5)
    w = pair.TransitionPacked.pack(nw, nb, fc1, fc2, fc3)
    out = pair.transition_fused(x, w, residual=True)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "transition")
    ref = reference.transition(x.float(), nw, nb, fc1, fc2, fc3, residual=True)
    assert _rel_err(out, ref) < 2e-2
    upd = (out.float() - x.float())
    upd_ref = ref - x.float()
    assert ((upd - upd_ref).abs().mean() / upd_ref.abs().mean()).item() < 2e-2


@pytest.mark.parametrize("outgoing", [True, False])
@pytest.mark.parametrize("N", [64, 136, 320])
def test_trimul(N, outgoing):
    from uplifting_biomolecular_modeling_b200.ops import native, pair, reference
    g = torch.Generator(device="cuda").manual_seed(4)
    c = 128
    z = (_rand((N, N, c), g) + 0.2).bfloat16()
    mask = (torch.rand((N, N), device="cuda", generator=g) > 0.1).float()
    niw, nib = 1.0 + 0.1 * _rand((c,), g), 0.1 * _rand((c,), g)
    now, nob = 1.0 + 0.1 * _rand((c,), g), 0.1 * _rand((c,), g)
    p_in, g_in = _rand((2 * c, c), g, c ** -0.5), _rand((2 * c, c), g, c ** -0.5)
    p_out, g_out = _rand((c, c), g, c ** -0.5), _rand((c, c), g, c ** -0.5)
    w = pair.TrimulPacked.pack(niw, nib, p_in, g_in, now, nob, p_out, g_out)
    out = pair.trimul_fused(z, mask, w, outgoing=outgoing, residual=False)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "trimul")
    ref = reference.triangle_multiplication(z.float(), mask, niw, nib, p_in, g_in, now, nob, p_out, g_out,
                                            outgoing=outgoing)
    err = (out.float() - ref).abs().mean() / ref.abs().mean()
    assert err.item() < 3e-2, err.item()
    assert _rel_err(out, ref) < 6e-2


def _attention_case(rows, N, H, D, g, masked):
    """Inputs, the kernel's scaled operands and the fp32 statement of one attention call."""
    from uplifting_biomolecular_modeling_b200.ops import pair, reference
    q = _rand((rows, N, H * D), g).bfloat16()
    k = _rand((rows, N, H * D), g).bfloat16()
    v = _rand((rows, N, H * D), g).bfloat16()
    gate = torch.rand((rows, N, H * D), device="cuda", generator=g).bfloat16()
    Np = (N + 7) // 8 * 8
    bias = torch.zeros((H, N, Np), device="cuda", dtype=torch.bfloat16)
    bias[:, :, :N] = _rand((H, N, N), g).bfloat16()
    qs = (q.float() * (pair.LOG2E / D ** 0.5)).bfloat16()
    bs = (bias.float() * pair.LOG2E).bfloat16()
    keep = None
    if masked:
        # some rows unmasked, some with scattered masked keys, some with a masked tail (padding)
        keep = torch.ones((rows, N), device="cuda")
        keep[1::3] = (torch.rand((len(range(1, rows, 3)), N), device="cuda", generator=g) > 0.3).float()
        keep[2::3, N - N // 5:] = 0
        keep[0, N - 3:] = 0
        keep[:, 0] = 1
    refs = []
    for r0 in range(0, rows, 64):     # the fp32 statement in row chunks (its score tensor is rows x H x N x N)
        sl = slice(r0, min(rows, r0 + 64))
        qh = qs[sl].float().view(-1, N, H, D).transpose(1, 2) / pair.LOG2E
        kh = k[sl].float().view(-1, N, H, D).transpose(1, 2)
        vh = v[sl].float().view(-1, N, H, D).transpose(1, 2)
        b = bs.float()[None, :, :, :N] / pair.LOG2E
        if keep is not None:
            b = b + ((1.0 - keep[sl]) * -1e9)[:, None, None, :]
        o = reference.attention_with_bias(qh, kh, vh, b, scale=1.0)
        refs.append(o.transpose(1, 2).reshape(-1, N, H * D) * gate[sl].float())
    return qs, k, v, bs, gate, Np, keep, torch.cat(refs, 0)


@pytest.mark.parametrize("variant", [0, 0x10])
@pytest.mark.parametrize("rows,N,H,D", [(7, 200, 4, 32), (9, 384, 2, 32), (1, 136, 4, 32), (5, 200, 4, 64)])
def test_attention_masked(rows, N, H, D, variant, request):
    """Key masks per row (scattered keys, padded tails, unmasked rows) in every tile shape and with the polynomial
    exponentials, against the fp32 statement with the same mask."""
    from uplifting_biomolecular_modeling_b200.ops import native, pair
    pair.set_attention_variant(variant)
    request.addfinalizer(lambda: pair.set_attention_variant(0))
    g = torch.Generator(device="cuda").manual_seed(15)
    qs, k, v, bs, gate, Np, keep, ref = _attention_case(rows, N, H, D, g, masked=True)
    km = pair.KeyMask.pack(keep)
    assert km is not None and int(km.flags.sum()) < km.flags.numel()      # some steps take the mask-free loop
    out = torch.empty_like(qs)
    pair.attention(qs, k, v, bs, gate, out, rows, N, N, H, D, ldb=Np, mask=km)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "attention")
    err = (out.float() - ref).abs().max().item()
    assert err < 3e-2, err
    assert pair.KeyMask.pack(torch.ones((rows, N), device="cuda")) is None


@pytest.mark.parametrize("masked", [False, True])
def test_attention_core_n1536(masked):
    """The benchmark size (1536 rows x 1536 keys, 4 heads x 32): every row against fp32 computed in row chunks."""
    from uplifting_biomolecular_modeling_b200.ops import native, pair
    g = torch.Generator(device="cuda").manual_seed(16)
    rows = N = 1536
    qs, k, v, bs, gate, Np, keep, ref = _attention_case(rows, N, 4, 32, g, masked)
    out = torch.empty_like(qs)
    pair.attention(qs, k, v, bs, gate, out, rows, N, N, 4, 32, ldb=Np,
                   mask=None if keep is None else pair.KeyMask.pack(keep))
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "attention")
    err = (out.float() - ref).abs().max().item()
    assert err < 3e-2, err


@pytest.mark.parametrize("variant", [0, 1, 5, 0x10])
@pytest.mark.parametrize("rows,N,H", [(2, 128, 4), (5, 200, 4), (8, 384, 2)])
def test_attention_core(rows, N, H, variant, request):
    """The attention kernel alone: base-2 softmax with shared bias, gate and tail masking.  Variant 0 takes the
    four-rows-per-CTA form for rows >= 4, variant 5 always the two-row form."""
    from uplifting_biomolecular_modeling_b200.ops import native, pair, reference
    pair.set_attention_variant(variant)
    request.addfinalizer(lambda: pair.set_attention_variant(0))
    g = torch.Generator(device="cuda").manual_seed(5)
    D = 32
    q = _rand((rows, N, H * D), g).bfloat16()
    k = _rand((rows, N, H * D), g).bfloat16()
    v = _rand((rows, N, H * D), g).bfloat16()
    gate = torch.rand((rows, N, H * D), device="cuda", generator=g).bfloat16()
    Np = (N + 7) // 8 * 8
    bias = torch.zeros((H, N, Np), device="cuda", dtype=torch.bfloat16)
    bias[:, :, :N] = _rand((H, N, N), g).bfloat16()
    out = torch.empty_like(q)
    qs = (q.float() * (pair.LOG2E / D ** 0.5)).bfloat16()
    bs = (bias.float() * pair.LOG2E).bfloat16()
    pair.attention_d32(qs, k, v, bs, gate, out, rows, N, N, H, ldb=Np)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "attention")
    qh = qs.float().view(rows, N, H, D).transpose(1, 2) / pair.LOG2E
    kh = k.float().view(rows, N, H, D).transpose(1, 2)
    vh = v.float().view(rows, N, H, D).transpose(1, 2)
    ref = reference.attention_with_bias(qh, kh, vh, bs.float()[None, :, :, :N] / pair.LOG2E, scale=1.0)
    ref = ref.transpose(1, 2).reshape(rows, N, H * D) * gate.float()
    err = (out.float() - ref).abs().max().item()
    assert err < 3e-2, err


@pytest.mark.parametrize("starting", [True, False])
@pytest.mark.parametrize("N", [64, 200])
def test_triangle_attention(N, starting):
    from uplifting_biomolecular_modeling_b200.ops import native, pair, reference
    g = torch.Generator(device="cuda").manual_seed(6)
    c, H = 128, 4
    z = (_rand((N, N, c), g) + 0.2).bfloat16()
    ln_w, ln_b = 1.0 + 0.1 * _rand((c,), g), 0.1 * _rand((c,), g)
    w_bias = _rand((H, c), g, c ** -0.5)
    w_q, w_k, w_v, w_g = [_rand((c, c), g, c ** -0.5) for _ in range(4)]
    b_g = 0.1 * _rand((c,), g)
    w_o, b_o = _rand((c, c), g, c ** -0.5), 0.1 * _rand((c,), g)
    w = pair.TriattPacked.pack(ln_w, ln_b, w_bias, w_q, w_k, w_v, w_g, b_g, w_o, b_o, H)
    out = pair.triangle_attention_fused(z, w, starting=starting, residual=False)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "triangle attention")
    ref = reference.triangle_attention(z.float(), None, ln_w, ln_b, w_bias, w_q, w_k, w_v, w_g, b_g, w_o, b_o, H,
                                       starting=starting)
    err = (out.float() - ref).abs().mean() / ref.abs().mean()
    assert err.item() < 3e-2, err.item()
    assert _rel_err(out, ref) < 6e-2
    # with a pair mask (padding tail + scattered pairs): the ending node attends over the transposed mask
    tok = torch.ones(N, device="cuda")
    tok[N - N // 6:] = 0
    pm = tok[:, None] * tok[None, :] * (torch.rand((N, N), device="cuda", generator=g) > 0.05).float()
    pm[:, 0] = 1
    pm[0, :] = 1
    km = pair.KeyMask.pack(pm if starting else pm.t())
    out = pair.triangle_attention_fused(z, w, starting=starting, residual=False, mask=km)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "triangle attention (masked)")
    ref = reference.triangle_attention(z.float(), pm, ln_w, ln_b, w_bias, w_q, w_k, w_v, w_g, b_g, w_o, b_o, H,
                                       starting=starting)
    err = (out.float() - ref).abs().mean() / ref.abs().mean()
    assert err.item() < 3e-2, err.item()


@pytest.mark.parametrize("B,N,H,D,c", [(3, 200, 16, 48, 768), (1, 136, 16, 24, 384)])
def test_apb_fused_matches_reference(B, N, H, D, c):
    """Gated attention with pair bias (DiT token attention 16 x 48 padded to 64; single attention 16 x 24
    padded to 32) against the plain statement."""
    from uplifting_biomolecular_modeling_b200.models import pairformer
    from uplifting_biomolecular_modeling_b200.ops import native, rows
    torch.manual_seed(7)
    attn = pairformer.AttentionPairBias(c, 128, H).cuda().eval()
    x = torch.randn(B, N, c, device="cuda")
    z = torch.randn(1, N, N, 128, device="cuda")
    with torch.no_grad():
        bias_dense = attn.pair_bias(z)
        ref = attn(x, None, None, bias=bias_dense, multiplicity=B)
        ab = attn.to(torch.bfloat16)
        ab.set_impl("fused")
        planes = ab.pair_bias(z.bfloat16())
        assert isinstance(planes, pairformer.BiasPlanes)
        out = ab(x.bfloat16(), None, None, bias=planes, multiplicity=B)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "apb")
    err = ((out.float() - ref).abs().mean() / ref.abs().mean()).item()
    assert err < 4e-2, err


def test_row_kernels():
    from uplifting_biomolecular_modeling_b200.ops import reference, rows
    g = torch.Generator(device="cuda").manual_seed(8)
    x = _rand((1000, 384), g) * 2 + 0.5
    w, b = 1 + 0.1 * _rand((384,), g), 0.1 * _rand((384,), g)
    out = rows.layernorm_rows(x, w, b)
    assert torch.allclose(out, reference.layer_norm(x, w, b), atol=2e-5, rtol=1e-5)
    xb = x.bfloat16()
    outb = rows.layernorm_rows(xb, w, b)
    assert torch.allclose(outb.float(), reference.layer_norm(xb.float(), w, b), atol=3e-2, rtol=2e-2)
    a = _rand((64, 768), g).bfloat16()
    sc, sh = _rand((64, 768), g).bfloat16(), _rand((64, 768), g).bfloat16()
    ref = torch.sigmoid(sc.float()) * torch.nn.functional.layer_norm(a.float(), (768,)) + sh.float()
    assert torch.allclose(rows.adaln_rows(a, sc, sh).float(), ref, atol=5e-2, rtol=3e-2)
    # 128 channels (atom track): half a warp per row; odd row count, conditioning rows shared by three samples
    a1 = _rand((3 * 333, 128), g).bfloat16()
    sc1, sh1 = _rand((333, 128), g).bfloat16(), _rand((333, 128), g).bfloat16()
    ref = (torch.sigmoid(sc1.float()) * torch.nn.functional.layer_norm(a1.float(), (128,)).view(3, 333, 128)
           + sh1.float()).view(-1, 128)
    assert torch.allclose(rows.adaln_rows(a1, sc1, sh1).float(), ref, atol=5e-2, rtol=3e-2)
    ab = _rand((64, 512), g).bfloat16()
    ref = torch.nn.functional.silu(ab[:, :256].float()) * ab[:, 256:].float()
    assert torch.allclose(rows.swiglu_rows(ab).float(), ref, atol=3e-2, rtol=3e-2)
    ref = a.float() + torch.sigmoid(sc.float()) * sh.float()
    assert torch.allclose(rows.gate_residual(sh, sc, a).float(), ref, atol=5e-2, rtol=3e-2)


@pytest.mark.parametrize("kernel", ["tc", "simt"])
@pytest.mark.parametrize("A", [320, 96, 800])
def test_window_attention_matches_reference(A, kernel, monkeypatch):
    from uplifting_biomolecular_modeling_b200.models import diffusion, pairformer
    from uplifting_biomolecular_modeling_b200.ops import native, pair
    monkeypatch.setattr(pair, "WINDOW_KERNEL", kernel)
    torch.manual_seed(9)
    B, c, H = 3, 128, 4
    attn = pairformer.AttentionPairBias(c, 128, H, compute_pair_bias=False).cuda().eval()
    x = torch.randn(B, A, c, device="cuda")
    bias = torch.randn(1, H, A // 32, 32, 128, device="cuda")
    with torch.no_grad():
        ref = diffusion._window_attention(attn, x, bias, (32, 128))
        ab = attn.to(torch.bfloat16)
        w = pair.ApbPacked.pack(ab.proj_q.weight, ab.proj_q.bias, ab.proj_k.weight, ab.proj_v.weight, ab.proj_g.weight,
                                ab.proj_o.weight, H)
        out = pair.window_attention_fused(x.bfloat16(), w, diffusion.WindowBias(bias).data)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "window attention")
    err = ((out.float() - ref).abs().mean() / ref.abs().mean()).item()
    assert err < 4e-2, err


def test_segment_mean_and_gather_rows():
    from uplifting_biomolecular_modeling_b200.models import diffusion
    from uplifting_biomolecular_modeling_b200.ops import rows
    g = torch.Generator(device="cuda").manual_seed(11)
    B, N, C = 3, 37, 768
    counts = torch.randint(1, 9, (N,), generator=torch.Generator().manual_seed(1))
    a2t = torch.repeat_interleave(torch.arange(N), counts).cuda()
    A = a2t.shape[0]
    t = torch.randn(B, A, C, device="cuda", generator=g).bfloat16()
    ref = diffusion.segment_mean(t, a2t, N, fused=False)
    out = diffusion.segment_mean(t, a2t, N, fused=True)
    assert torch.allclose(out.float(), ref.float(), atol=2e-2, rtol=2e-2)
    a = torch.randn(B, N, 128, device="cuda", generator=g).bfloat16()
    q = torch.randn(B, A, 128, device="cuda", generator=g).bfloat16()
    got = rows.gather_rows_add(q, a, a2t.to(torch.int32))
    assert torch.equal(got, q + a[:, a2t])
    assert torch.equal(rows.gather_rows_add(None, a, a2t.to(torch.int32)), a[:, a2t])


@pytest.mark.parametrize("N", [37, 136, 200])
@pytest.mark.parametrize("H", [4, 16, 32])
@pytest.mark.parametrize("transpose", [False, True])
def test_pair_head_bias_planes(N, H, transpose):
    """LN(z) -> H head-bias planes, several pair rows per thread (vector stores when 4 rows share a plane row)."""
    from uplifting_biomolecular_modeling_b200.ops import rows
    g = torch.Generator(device="cuda").manual_seed(N + H)
    z = (torch.randn(N, N, 128, device="cuda", generator=g) * 1.5 + 0.3).bfloat16()
    lw = 1 + 0.1 * torch.randn(128, device="cuda", generator=g)
    lb = 0.1 * torch.randn(128, device="cuda", generator=g)
    w = torch.randn(H, 128, device="cuda", generator=g) / 128 ** 0.5
    out = rows.pair_head_bias(z, lw, lb, w, scale=1.3, transpose=transpose)
    ref = 1.3 * torch.nn.functional.layer_norm(z.float(), (128,), lw, lb) @ w.t()          # [N, N, H]
    ref = ref.permute(2, 1, 0) if transpose else ref.permute(2, 0, 1)
    assert out.shape == (H, N, N)
    assert (out.float() - ref).abs().max().item() < 4e-2


@pytest.mark.parametrize("N,outgoing", [(1536, True), (1536, False), (4096, True)])
def test_trimul_large_sampled_rows(N, outgoing):
    """Benchmark sizes: the fused triangle multiplication at 1536 and 4096 tokens (pair planes pass 2^31 elements at
    4096: the 64-bit index paths run here) against fp32 computed for a sample of output rows."""
    from uplifting_biomolecular_modeling_b200.ops import native, pair, reference
    g = torch.Generator(device="cuda").manual_seed(21)
    c = 128
    z = (_rand((N, N, c), g) + 0.2).bfloat16()
    niw, nib = 1.0 + 0.1 * _rand((c,), g), 0.1 * _rand((c,), g)
    now, nob = 1.0 + 0.1 * _rand((c,), g), 0.1 * _rand((c,), g)
    p_in, g_in = _rand((2 * c, c), g, c ** -0.5), _rand((2 * c, c), g, c ** -0.5)
    p_out, g_out = _rand((c, c), g, c ** -0.5), _rand((c, c), g, c ** -0.5)
    w = pair.TrimulPacked.pack(niw, nib, p_in, g_in, now, nob, p_out, g_out)
    out = pair.trimul_fused(z, None, w, outgoing=outgoing, residual=False, workspace={})
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "trimul")
    # fp32 statement for a few output rows i: projections of the operand rows that those outputs read
    rows = [0, N // 3, N - 1]
    F = torch.nn.functional

    def proj(x):                                     # x: [..., c] fp32 rows of z -> gated a | b
        n = F.layer_norm(x, (c,), niw, nib)
        return F.linear(n, p_in) * torch.sigmoid(F.linear(n, g_in))
    errs = []
    for i in rows:
        if outgoing:          # x[i, j] = sum_k a[i, k] b[j, k]
            a_i = proj(z[i].float())[:, :c]                                   # [N(k), c]
            xi = torch.empty((N, c), device="cuda")
            for j0 in range(0, N, 256):
                b_j = proj(z[j0:j0 + 256].float())[..., c:]                   # [256, N(k), c]
                xi[j0:j0 + 256] = torch.einsum("kc,jkc->jc", a_i, b_j)
        else:                 # x[i, j] = sum_k a[k, i] b[k, j]
            a_i = proj(z[:, i].float())[:, :c]                                # [N(k), c]
            xi = torch.zeros((N, c), device="cuda")
            for k0 in range(0, N, 256):
                b_k = proj(z[k0:k0 + 256].float())[..., c:]                   # [256(k), N(j), c]
                xi += torch.einsum("kc,kjc->jc", a_i[k0:k0 + 256], b_k)
        ni = F.layer_norm(z[i].float(), (c,), niw, nib)
        ref_i = F.linear(F.layer_norm(xi, (c,), now, nob), p_out) * torch.sigmoid(F.linear(ni, g_out))
        errs.append(((out[i].float() - ref_i).abs().mean() / ref_i.abs().mean()).item())
    assert max(errs) < 3e-2, errs


def test_transition_n1536():
    from uplifting_biomolecular_modeling_b200.ops import native, pair, reference
    g = torch.Generator(device="cuda").manual_seed(22)
    N, c, hidden = 1536, 128, 512
    x = (_rand((N, N, c), g) + 0.3).bfloat16()
    nw, nb = 1.0 + 0.1 * _rand((c,), g), 0.1 * _rand((c,), g)
    fc1, fc2 = _rand((hidden, c), g, c ** -0.5), _rand((hidden, c), g, c ** -0.5)
    fc3 = _rand((c, hidden), g, hidden ** -0.5)
    out = pair.transition_fused(x, pair.TransitionPacked.pack(nw, nb, fc1, fc2, fc3), residual=True)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "transition")
    worst = 0.0
    for r0 in (0, 700, N - 64):                       # row chunks of the fp32 statement
        ref = reference.transition(x[r0:r0 + 64].float(), nw, nb, fc1, fc2, fc3, residual=True)
        upd_ref = ref - x[r0:r0 + 64].float()
        upd = out[r0:r0 + 64].float() - x[r0:r0 + 64].float()
        worst = max(worst, ((upd - upd_ref).abs().mean() / upd_ref.abs().mean()).item())
    assert worst < 2e-2, worst
