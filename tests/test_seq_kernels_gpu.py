"""Row / sequence kernels of the LM and genomics families against plain fp32 PyTorch statements."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(out, ref, tol=2e-2):
    err = (out.float() - ref.float()).abs().max().item()
    scale = max(ref.float().abs().max().item(), 1.0)
    assert err <= tol * scale, (err, scale)


@pytest.mark.parametrize("C", [256, 4096, 8192])
def test_rmsnorm(C):
    from uplifting_biomolecular_modeling_b200.ops import reference as R, seq
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(37, C, device="cuda", generator=g).bfloat16()
    sc = 1 + 0.1 * torch.randn(C, device="cuda", generator=g)
    _close(seq.rmsnorm_rows(x, sc), R.rmsnorm_rows(x, sc))


@pytest.mark.parametrize("K,tail", [(3, False), (3, True), (4, True)])
def test_fir_gate3(K, tail):
    from uplifting_biomolecular_modeling_b200.ops import reference as R, seq
    g = torch.Generator(device="cuda").manual_seed(1)
    B, L, d = 2, 77, 64
    z = torch.randn(B, L, 3 * d, device="cuda", generator=g).bfloat16()
    h = torch.randn(3 * d, K, device="cuda", generator=g) * 0.4
    t = torch.randn(B, K - 1, 3 * d, device="cuda", generator=g).bfloat16() if tail else None
    u, x2 = seq.fir_gate3(z, seq.taps_major(h), t)
    ur, x2r = R.fir_gate3(z, h, t)
    _close(u, ur)
    _close(x2, x2r)


@pytest.mark.parametrize("K,L,d", [(128, 1100, 96), (40, 513, 32), (17, 64, 40), (128, 4096, 256)])
def test_fir_inner_gate_tiled_direct_convolution(K, L, d):
    """Filters of more than 8 taps over a sequence without a tail take the shared-memory tiled kernel (taps padded to
    16, ragged channel and position tiles)."""
    from uplifting_biomolecular_modeling_b200.ops import reference as R, seq
    g = torch.Generator(device="cuda").manual_seed(24)
    B = 2
    u = torch.randn(B, L, d, device="cuda", generator=g).bfloat16()
    x2 = torch.randn(B, L, d, device="cuda", generator=g).bfloat16()
    h = torch.randn(d, K, device="cuda", generator=g) * K ** -0.5
    D = torch.randn(d, device="cuda", generator=g)
    out = seq.fir_inner_gate(u, seq.taps_major(h), D, x2, None)
    _close(out, R.fir_inner_gate(u, h, D, x2, None))
    _close(seq.fir_inner_gate(u, seq.taps_major(h), D, None, None), R.fir_inner_gate(u, h, D, None, None))


@pytest.mark.parametrize("K,tail", [(7, False), (7, True), (40, False), (40, True)])
def test_fir_inner_gate(K, tail):
    from uplifting_biomolecular_modeling_b200.ops import reference as R, seq
    g = torch.Generator(device="cuda").manual_seed(2)
    B, L, d = 2, 90, 128
    u = torch.randn(B, L, d, device="cuda", generator=g).bfloat16()
    x2 = torch.randn(B, L, d, device="cuda", generator=g).bfloat16()
    h = torch.randn(d, K, device="cuda", generator=g) * K ** -0.5
    D = torch.randn(d, device="cuda", generator=g)
    t = torch.randn(B, K - 1, d, device="cuda", generator=g).bfloat16() if tail else None
    _close(seq.fir_inner_gate(u, seq.taps_major(h), D, x2, t), R.fir_inner_gate(u, h, D, x2, t), 3e-2)


def test_fftconv_epilogue_and_pole_step():
    from uplifting_biomolecular_modeling_b200.ops import reference as R, seq
    g = torch.Generator(device="cuda").manual_seed(3)
    B, L, d, n, S = 2, 70, 96, 128, 8
    y = torch.randn(B, d, n, device="cuda", generator=g)
    u = torch.randn(B, L, d, device="cuda", generator=g).bfloat16()
    x2 = torch.randn(B, L, d, device="cuda", generator=g).bfloat16()
    D = torch.randn(d, device="cuda", generator=g)
    _close(seq.fftconv_epilogue(y, u, D, x2), R.fftconv_epilogue(y, u, D, x2), 3e-2)
    state = torch.randn(B, d, S, device="cuda", generator=g)
    lam = torch.rand(d, S, device="cuda", generator=g) * 0.5 + 0.45
    res = torch.randn(d, S, device="cuda", generator=g) / S
    u1, g1 = u[:, 0].contiguous(), x2[:, 0].contiguous()
    ref, sref = R.pole_step(state.clone(), lam, res, u1, D, g1)
    out = seq.pole_step(state, lam, res, u1, D, g1)
    _close(out, ref, 3e-2)
    _close(state, sref, 1e-5)


def test_elementwise_sets():
    from uplifting_biomolecular_modeling_b200.ops import reference as R, seq
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(33, 512, device="cuda", generator=g).bfloat16()
    a = torch.randn(33, 512, device="cuda", generator=g).bfloat16()
    b = torch.randn(33, 512, device="cuda", generator=g).bfloat16()
    v0 = torch.randn(512, device="cuda", generator=g)
    v1 = torch.randn(512, device="cuda", generator=g)
    _close(seq.gelu_new(x), R.gelu_new(x))
    _close(seq.residual_add2(x, a, b), x.float() + a.float() + b.float())
    _close(seq.bias_residual(x, v0, a), x.float() + v0 + a.float())
    _close(seq.scale_shift_gelu(x, v0, v1), torch.nn.functional.gelu(x.float() * v0 + v1))
    _close(seq.silu_mul(x, a), torch.nn.functional.silu(x.float()) * a.float())
    _close(seq.add2_softmax_rows(x, a, b), torch.softmax(x.float() + a.float() + b.float(), -1), 1e-5)
    xs = torch.randn(2, 40, 64, device="cuda", generator=g).bfloat16()
    ws = torch.randn(2, 40, 64, device="cuda", generator=g).bfloat16()
    for mode in ("max", "mean", "softmax"):
        _close(seq.pool2(xs, mode, ws), R.pool2(xs, mode, ws))
    out, s = seq.residual_ln(x, a, 1 + 0.1 * v0, v1, return_sum=True)
    _close(out, R.residual_ln(x, a, 1 + 0.1 * v0, v1), 3e-2)
    assert torch.equal(s, (x.float() + a.float()).bfloat16())


def test_rotary_split_qkv():
    from uplifting_biomolecular_modeling_b200.ops import reference as R, seq
    g = torch.Generator(device="cuda").manual_seed(5)
    T, H, Dh, rot = 50, 4, 64, 32
    qkv = torch.randn(T, 3 * H * Dh, device="cuda", generator=g).bfloat16()
    pos = torch.arange(T, device="cuda")
    q, k, v = seq.rotary_split_qkv(qkv, pos, H, rot)
    qr, kr, vr = R.rotary_split_qkv(qkv, pos, H, rot)
    _close(q, qr)
    _close(k, kr)
    assert torch.equal(v.float(), vr)


def test_evo2_fused_matches_plain_statements():
    """Prefill logits and greedy decoding of the kernel path against the plain statements (bf16 weights)."""
    from uplifting_biomolecular_modeling_b200.models import evo2
    from uplifting_biomolecular_modeling_b200.ops import native
    m = evo2.build("evo2_tiny", device="cuda", dtype=torch.bfloat16, seed=3)
    tok = torch.randint(0, m.cfg.vocab, (2, 96), device="cuda")
    ref = m(tok).float()
    ref_states = [dict() for _ in m.blocks]
    m(tok, ref_states)
    ref_step = m.step(tok[:, -1:], ref_states).float()
    assert m.set_impl("fused") > 0
    out = m(tok).float()
    states = [dict() for _ in m.blocks]
    m(tok, states)
    out_step = m.step(tok[:, -1:], states).float()
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "evo2")
    scale = ref.abs().max().item()
    assert (out - ref).abs().max().item() < 6e-2 * scale
    assert (out_step - ref_step).abs().max().item() < 6e-2 * scale


@pytest.mark.parametrize("M", [1, 3, 8])
def test_gemv_rows(M):
    from uplifting_biomolecular_modeling_b200.ops import seq
    g = torch.Generator(device="cuda").manual_seed(6)
    K, N = 4096, 1000
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * K ** -0.5).bfloat16()
    b = torch.randn(N, device="cuda", generator=g)
    _close(seq.gemv_rows(x, w, b), x.float() @ w.float().t() + b)


@pytest.mark.parametrize("M,K", [(1, 4096), (2, 1024), (5, 11008)])
def test_gemv_rows_folded_forms_return_the_bits_of_the_separate_kernels(M, K):
    """SwiGLU over two weight matrices and the residual behind return the bits of the chain of separate kernels;
    RMSNorm in front agrees to the last place of its scale."""
    from uplifting_biomolecular_modeling_b200.ops import seq
    g = torch.Generator(device="cuda").manual_seed(16)
    N = 776
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * K ** -0.5).bfloat16()
    w2 = (torch.randn(N, K, device="cuda", generator=g) * K ** -0.5).bfloat16()
    gamma = 1 + 0.1 * torch.randn(K, device="cuda", generator=g)
    res = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, device="cuda", generator=g)
    xn = seq.rmsnorm_rows(x, gamma, 1e-6)
    # the sum of squares is taken in another order than the row kernel's: a last-place difference of the scale
    _close(seq.gemv_rows(x, w, b, gamma=gamma, eps=1e-6), seq.gemv_rows(xn, w, b), 4e-3)
    assert torch.equal(seq.gemv_rows(x, w, b, res=res), seq.gemv_rows(x, w, b) + res)
    sep = seq.silu_mul(seq.gemv_rows(xn, w), seq.gemv_rows(xn, w2))
    _close(seq.gemv_rows(x, w, gamma=gamma, eps=1e-6, w2=w2), sep, 4e-3)
    assert torch.equal(seq.gemv_rows(xn, w, w2=w2), sep)
    _close(seq.gemv_rows(x, w, b, gamma=gamma, res=res), xn.float() @ w.float().t() + b + res.float())


@pytest.mark.parametrize("K", [3, 4])
def test_fir_gate3_moves_the_tail_on_in_place(K):
    from uplifting_biomolecular_modeling_b200.ops import seq
    g = torch.Generator(device="cuda").manual_seed(17)
    B, d = 2, 64
    h = seq.taps_major(torch.randn(3 * d, K, device="cuda", generator=g) * 0.4)
    tail = torch.randn(B, K - 1, 3 * d, device="cuda", generator=g).bfloat16()
    for _ in range(3):
        z = torch.randn(B, 1, 3 * d, device="cuda", generator=g).bfloat16()
        u0, x0 = seq.fir_gate3(z, h, tail)
        want = torch.cat([tail, z], 1)[:, 1:].contiguous()
        u1, x1 = seq.fir_gate3(z, h, tail, push=True)
        assert torch.equal(u0, u1) and torch.equal(x0, x1) and torch.equal(tail, want)


@pytest.mark.parametrize("K,d", [(7, 64), (128, 4096), (40, 200)])
def test_fir_step_equals_the_inner_stage_and_moves_the_tail_on(K, d):
    from uplifting_biomolecular_modeling_b200.ops import reference as R, seq
    g = torch.Generator(device="cuda").manual_seed(18)
    B = 2
    hraw = torch.randn(d, K, device="cuda", generator=g) * K ** -0.5
    h = seq.taps_major(hraw)
    D = torch.randn(d, device="cuda", generator=g)
    tail = torch.randn(B, K - 1, d, device="cuda", generator=g).bfloat16()
    for _ in range(3):
        u = torch.randn(B, 1, d, device="cuda", generator=g).bfloat16()
        x2 = torch.randn(B, 1, d, device="cuda", generator=g).bfloat16()
        ref = R.fir_inner_gate(u, hraw, D, x2, tail)
        want = torch.cat([tail, u], 1)[:, 1:].contiguous()
        out = seq.fir_step(u, h, D, x2, tail)
        _close(out, ref)
        assert torch.equal(tail, want)


@pytest.mark.parametrize("heads", [4, 1])          # head dimension 32 (plain attention step) and 128 (decode kernels)
def test_evo2_graph_decode_on_the_folded_block_emits_the_tokens_of_the_separate_kernels(monkeypatch, heads):
    from uplifting_biomolecular_modeling_b200.models import evo2
    from uplifting_biomolecular_modeling_b200.ops import native
    m = evo2.build("evo2_tiny", device="cuda", dtype=torch.bfloat16, seed=4, n_heads=heads)
    m.set_impl("fused")
    tok = torch.randint(0, m.cfg.vocab, (1, 64), device="cuda")
    monkeypatch.setenv("UBM_EVO2_FOLDED_DECODE", "0")
    want = m.generate(tok, 12, graph=True)
    plain = m.generate(tok, 12, graph=False)
    monkeypatch.setenv("UBM_EVO2_FOLDED_DECODE", "1")
    got = m.generate(tok, 12, graph=True)
    got_eager = m.generate(tok, 12, graph=False)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "evo2 decode")
    assert torch.equal(plain, want)
    assert torch.equal(got, want) and torch.equal(got_eager, want)


@pytest.mark.parametrize("B,H,Lmax,pos", [(1, 4, 300, 0), (2, 3, 5000, 4097), (1, 32, 2048, 2047)])
def test_decode_attention_against_the_masked_softmax(B, H, Lmax, pos):
    from uplifting_biomolecular_modeling_b200.models import evo2
    from uplifting_biomolecular_modeling_b200.ops import native, seq
    g = torch.Generator(device="cuda").manual_seed(19)
    hd = 128
    kc = torch.randn(B, Lmax, H, hd, device="cuda", generator=g).bfloat16()
    vc = torch.randn(B, Lmax, H, hd, device="cuda", generator=g).bfloat16()
    qkv = torch.randn(B, 3 * H * hd, device="cuda", generator=g).bfloat16()
    p = torch.full((1,), pos, dtype=torch.long, device="cuda")
    q, k, v = qkv.view(B, 1, 3, H, hd).unbind(2)
    qr, kr = evo2.rope(q, p, 10000.0), evo2.rope(k, p, 10000.0)
    kref, vref = kc.clone(), vc.clone()
    kref[:, pos] = kr[:, 0]
    vref[:, pos] = v[:, 0]
    sc = torch.einsum("bqhd,bkhd->bhqk", qr.float(), kref[:, :pos + 1].float()) * hd ** -0.5
    ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc, -1), vref[:, :pos + 1].float()).reshape(B, H * hd)
    out = seq.decode_attention(qkv, p, kc, vc, 10000.0)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "decode attention")
    _close(out, ref)
    _close(kc[:, pos], kref[:, pos], 1e-2)
    assert torch.equal(vc, vref) and torch.equal(kc[:, :pos], kref[:, :pos]) and torch.equal(kc[:, pos + 1:], kref[:, pos + 1:])


def test_decode_attention_reports_a_full_cache_in_the_status_word():
    from uplifting_biomolecular_modeling_b200.ops import native, seq
    kc = torch.zeros(1, 16, 2, 128, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    qkv = torch.ones(1, 3 * 2 * 128, device="cuda", dtype=torch.bfloat16)
    seq.decode_attention(qkv, torch.full((1,), 16, dtype=torch.long, device="cuda"), kc, vc, 10000.0)
    code, where, _, aux = native.read_status("cuda")
    assert (code, where, aux) == (3, 120, 16)
    assert not kc.any() and not vc.any()


@pytest.mark.parametrize("B,L,d,S", [(1, 3000, 256, 16), (2, 77, 40, 4), (1, 1024, 128, 8)])
def test_pole_prefill_state_against_the_written_out_powers(B, L, d, S):
    from uplifting_biomolecular_modeling_b200.ops import seq
    g = torch.Generator(device="cuda").manual_seed(20)
    u = torch.randn(B, L, d, device="cuda", generator=g).bfloat16()
    lam = torch.rand(d, S, device="cuda", generator=g) * 0.5 + 0.45
    w = lam.double().unsqueeze(0) ** torch.arange(L - 1, -1, -1, device="cuda", dtype=torch.float64).view(L, 1, 1)
    ref = torch.einsum("bld,lds->bds", u.double(), w)
    out = seq.pole_prefill_state(u, lam)
    assert out.dtype == torch.float32 and out.shape == (B, d, S)
    _close(out, ref, 1e-4)


def test_fft_prologue_and_spectrum_product_equal_the_plain_statements():
    from uplifting_biomolecular_modeling_b200.ops import seq
    g = torch.Generator(device="cuda").manual_seed(21)
    B, L, d, n = 2, 300, 72, 640
    u = torch.randn(B, L, d, device="cuda", generator=g).bfloat16()
    pad = seq.fft_pad_transpose(u, n)
    assert torch.equal(pad[..., :L], u.float().transpose(1, 2)) and not pad[..., L:].any()
    H = torch.fft.rfft(torch.randn(d, 100, device="cuda", generator=g), n=n)
    X = torch.fft.rfft(pad)
    want = X * H.unsqueeze(0)
    got = seq.spectrum_mul_(X.clone(), H.contiguous())
    assert (got - want).abs().max().item() <= 1e-5 * want.abs().max().item()


@pytest.mark.parametrize("M,K,N", [(1, 4096, 1000), (3, 1040, 77), (8, 256, 300)])
def test_gemv_rows_with_e4m3_weights(M, K, N):
    from uplifting_biomolecular_modeling_b200.ops import gemm, seq
    g = torch.Generator(device="cuda").manual_seed(23)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = torch.randn(N, K, device="cuda", generator=g) * K ** -0.5
    gamma = 1 + 0.1 * torch.randn(K, device="cuda", generator=g)
    res = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, device="cuda", generator=g)
    q, dq = gemm.quantize_e4m3(w)
    _close(seq.gemv_rows(x, q, b, wscale=dq), x.float() @ (q.float() * dq).t() + b, 1e-2)
    xn = seq.rmsnorm_rows(x, gamma, 1e-6)
    _close(seq.gemv_rows(x, q, b, gamma=gamma, res=res, wscale=dq),
           xn.float() @ (q.float() * dq).t() + b + res.float(), 1e-2)


@pytest.mark.parametrize("R,C", [(37, 256), (300, 4096), (5, 1024)])
def test_rmsnorm_fp8_rows_and_their_dequantisation_factor(R, C):
    from uplifting_biomolecular_modeling_b200.ops import reference as Rf, seq
    g = torch.Generator(device="cuda").manual_seed(22)
    x = (torch.randn(R, C, device="cuda", generator=g) * 3).bfloat16()
    sc = 1 + 0.1 * torch.randn(C, device="cuda", generator=g)
    ref = Rf.rmsnorm_rows(x, sc).float()
    y8, dq = seq.rmsnorm_fp8(x, sc)
    torch.cuda.synchronize()
    assert y8.dtype == torch.float8_e4m3fn and y8.shape == (R, C)
    amax = ref.abs().max().item()
    assert abs(dq.item() * 448.0 - amax) <= 1e-2 * amax            # ref is rounded to bf16, the kernel's maximum is not
    back = y8.float() * dq
    # three mantissa bits: a relative step of 1/8 at most, half of it as rounding error (plus the subnormal floor)
    assert ((back - ref).abs() <= 0.0625 * ref.abs() + 2.0 ** -9 * amax + 1e-2 * amax / 448).all()


def test_evo2_fp8_input_projections_stay_close_to_the_bf16_prefill():
    from uplifting_biomolecular_modeling_b200.models import evo2
    from uplifting_biomolecular_modeling_b200.ops import native
    m = evo2.build("evo2_tiny", device="cuda", dtype=torch.bfloat16, seed=9, d_model=256, n_heads=2, ffn=512)
    m.set_impl("fused")
    tok = torch.randint(0, m.cfg.vocab, (2, 200), device="cuda")
    want = m(tok).float()
    assert m.set_fp8_input_projections(True) == 3
    states = [dict() for _ in m.blocks]
    got = m(tok, states).float()
    step = m.step(tok[:, -1:], states)                              # the folded block reads the e4m3 weights
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "evo2 fp8")
    assert torch.isfinite(got).all() and torch.isfinite(step.float()).all()
    rel = ((got - want).abs().mean() / want.abs().mean()).item()
    assert 0.0 < rel < 8e-2, rel                                    # differs (8-bit operands) but stays close


def test_evo2_speculative_decoding_on_the_kernel_path_returns_the_greedy_tokens():
    """Multi-token continuation (``extend`` / ``commit`` through the folded block with several rows) and the draft's
    single-token steps against plain greedy decoding of the target."""
    from uplifting_biomolecular_modeling_b200.models import evo2
    from uplifting_biomolecular_modeling_b200.ops import native
    target = evo2.build("evo2_tiny", device="cuda", dtype=torch.bfloat16, seed=11, n_heads=1)
    draft = evo2.build("evo2_tiny", device="cuda", dtype=torch.bfloat16, seed=12, n_heads=1, n_layers=2, attn_layers=())
    target.set_impl("fused")
    draft.set_impl("fused")
    tok = torch.randint(0, target.cfg.vocab, (1, 48), device="cuda")
    want = target.generate(tok, 10, graph=False)
    got, stats = target.generate_speculative(draft, tok, 10, k=3)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "evo2 speculative")
    assert torch.equal(got, want), (got, want)
    assert stats["proposed"] >= stats["accepted"] >= 0 and stats["rounds"] >= 1


def test_per_channel_vectors_given_in_bf16():
    """Per-channel vectors that need a conversion are converted into tensors that outlive the launch."""
    from uplifting_biomolecular_modeling_b200.ops import reference as R, seq
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(3, 50, 64, device="cuda", generator=g).bfloat16()
    sc = (1 + 0.1 * torch.randn(64, device="cuda", generator=g)).bfloat16()
    sh = (0.5 * torch.randn(64, device="cuda", generator=g)).bfloat16()
    want = torch.nn.functional.gelu(x.float() * sc.float() + sh.float())
    _close(seq.scale_shift_gelu(x, sc, sh), want)
    res = torch.randn(3, 50, 64, device="cuda", generator=g).bfloat16()
    _close(seq.residual_ln(x, res, sc, sh), R.residual_ln(x, res, sc, sh))
