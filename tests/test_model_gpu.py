"""End-to-end model on the GPU: fused (fast) path against the plain statements (off path)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_pairformer_layer_fast_vs_off():
    from uplifting_biomolecular_modeling_b200.models import pairformer
    from uplifting_biomolecular_modeling_b200.ops import native
    torch.manual_seed(0)
    N = 192
    layer = pairformer.PairformerLayer().cuda().eval()
    for p in layer.parameters():
        p.requires_grad_(False)
    s = torch.randn(1, N, 384, device="cuda")
    z = torch.randn(1, N, N, 128, device="cuda")
    mask = torch.ones(1, N, device="cuda")
    with torch.no_grad():
        s_ref, z_ref = layer(s, z, mask, None)
        lb = layer.to(torch.bfloat16)
        pairformer.set_impl(lb, "fused")
        s_f, z_f = lb(s.bfloat16(), z.bfloat16(), mask, None)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "pairformer layer")
    dz = ((z_f.float() - z_ref).abs().mean() / (z_ref - z).abs().mean()).item()
    ds = ((s_f.float() - s_ref).abs().mean() / (s_ref - s).abs().mean()).item()
    assert dz < 5e-2, dz
    assert ds < 5e-2, ds


def test_predictor_fast_runs_and_uses_kernels():
    from uplifting_biomolecular_modeling_b200 import api
    from uplifting_biomolecular_modeling_b200.models import cofold
    from uplifting_biomolecular_modeling_b200.ops import native
    pred = api.Predictor("tiny", mode="fast", device="cuda:0", seed=0)
    feats = cofold.synthetic_features(128, 16, pred.cfg, seed=0)
    native.reset_launch_count()
    out = pred.predict(feats)
    assert torch.isfinite(out["coords"]).all()
    assert native.launch_count() > 0
    out2 = pred.predict(feats)            # second call replays the cached sampler graph
    assert torch.isfinite(out2["coords"]).all()
    assert torch.equal(out["coords"], out2["coords"])      # same seed, same kernels: run-to-run bitwise


def test_exact_is_bitwise_off():
    from uplifting_biomolecular_modeling_b200 import api
    from uplifting_biomolecular_modeling_b200.models import cofold
    off = api.Predictor("tiny", mode="off", device="cuda:0", seed=0)
    exact = api.Predictor("tiny", mode="exact", device="cuda:0", seed=0)
    feats = cofold.synthetic_features(96, 8, off.cfg, seed=1)
    a = off.predict(feats)
    b = exact.predict(feats)
    assert torch.equal(a["coords"], b["coords"])
    assert torch.equal(a["plddt"], b["plddt"])


@pytest.mark.parametrize("full", [True, False])
def test_outer_product_mean_fused_vs_reference(full):
    from uplifting_biomolecular_modeling_b200.models import msa
    from uplifting_biomolecular_modeling_b200.ops import native
    torch.manual_seed(1)
    S, N = 40, 200
    opm = msa.OuterProductMean().cuda().eval()
    m = torch.randn(1, S, N, 64, device="cuda")
    mask = torch.ones(1, S, N, device="cuda")
    if not full:
        mask = (torch.rand(1, S, N, device="cuda") > 0.2).float()
    with torch.no_grad():
        ref = opm(m, mask)
        ob = opm.to(torch.bfloat16)
        ob.impl = "fused"
        ob.row_block = 64
        ob.full_mask = full
        out = ob(m.bfloat16(), mask)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "outer product mean")
    err = ((out.float() - ref).abs().mean() / ref.abs().mean()).item()
    assert err < 3e-2, err


def test_template_embedder_fused_vs_reference():
    from uplifting_biomolecular_modeling_b200.models import template
    from uplifting_biomolecular_modeling_b200.ops import native
    torch.manual_seed(2)
    N, T = 72, 3
    asym = torch.tensor([0] * 40 + [1] * 32)
    m = template.TemplateEmbedder(c_z=128, n_blocks=1).cuda().eval()
    f = {k: v.cuda() for k, v in template.synthetic_template_features(N, T, asym).items()}
    z = torch.randn(1, N, N, 128, device="cuda")
    with torch.no_grad():
        ref = m(z, f)
        zp = m.linear_z(m.z_norm(z[0]))
        v_ref = m.embed_reference(zp, f)
        v_fused = m._embed_fused(zp, f)
        mb = m.to(torch.bfloat16)
        mb.impl = "fused"
        out = mb(z.bfloat16(), f)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "template")
    assert (v_fused - v_ref).abs().max().item() < 3e-2 * v_ref.abs().max().item()
    err = ((out.float() - ref).abs().mean() / ref.abs().mean()).item()
    assert err < 5e-2, err


@pytest.mark.parametrize("dim", [64, 256])
def test_transition_other_widths_fused_vs_reference(dim):
    from uplifting_biomolecular_modeling_b200.models import pairformer
    from uplifting_biomolecular_modeling_b200.ops import native
    torch.manual_seed(3)
    t = pairformer.Transition(dim).cuda().eval()
    x = torch.randn(3, 700, dim, device="cuda")
    with torch.no_grad():
        ref = t(x, residual=True)
        tb = t.to(torch.bfloat16)
        tb.impl = "fused"
        out = tb(x.bfloat16(), residual=True)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "transition")
    err = ((out.float() - ref).abs().mean() / (ref - x).abs().mean()).item()
    assert err < 5e-2, err


def test_layernorm_rows_narrow():
    from uplifting_biomolecular_modeling_b200.ops import rows
    g = torch.Generator(device="cuda").manual_seed(4)
    for C in (64, 128, 256, 384, 768, 960, 1152, 1536, 2048):
        x = (torch.randn(1001, C, device="cuda", generator=g) * 2 + 0.5).bfloat16()
        w = 1 + 0.1 * torch.randn(C, device="cuda", generator=g)
        b = 0.1 * torch.randn(C, device="cuda", generator=g)
        ref = torch.nn.functional.layer_norm(x.float(), (C,), w, b)
        out = rows.layernorm_rows(x, w, b)
        assert torch.allclose(out.float(), ref, atol=3e-2, rtol=2e-2), C


@pytest.mark.parametrize("c,heads,N", [(64, 4, 72), (256, 8, 100)])
def test_pair_block_at_other_widths_runs_on_the_kernel_path(c, heads, N):
    """Triangle multiplication, triangle attention and the transition at widths other than 128 (template stack 64,
    ESM family 256; head dimension 16 padded to 32): rows + GEMM forms of the kernel path against the fp32
    statements, with a pair mask, every call counted as served."""
    import torch
    from uplifting_biomolecular_modeling_b200.core import counters
    from uplifting_biomolecular_modeling_b200.models import pairformer
    from uplifting_biomolecular_modeling_b200.ops import dispatch, native
    counters.BOOK._ledgers.clear()
    dispatch.reset()
    torch.manual_seed(0)
    layer = pairformer.PairformerLayer(c_s=384, c_z=c, pair_heads=heads, no_seq=True).cuda().eval()
    with torch.no_grad():
        for p in layer.parameters():
            p.normal_(0, 0.5 * p.shape[-1] ** -0.5 if p.dim() > 1 else 0.1)
        for mod in layer.modules():
            if isinstance(mod, torch.nn.LayerNorm):
                mod.weight.add_(1.0)
    z = torch.randn(1, N, N, c, device="cuda")
    tok = torch.ones(N, device="cuda")
    tok[N - 9:] = 0
    pm = (tok[:, None] * tok[None, :]).unsqueeze(0)
    with torch.no_grad():
        ref = layer.pair_update(z, pm)
        lb = layer.to(torch.bfloat16)
        pairformer.set_impl(lb, "fused", workspace={})
        out = lb.pair_update(z.bfloat16(), pm)
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "pair block at other widths")
    v = tok.bool()
    r, o = ref[0][v][:, v], out[0][v][:, v].float()
    upd = r - z[0][v][:, v]
    err = ((o - r).abs().mean() / upd.abs().mean()).item()
    assert err < 4e-2, err
    for lever in ("fused_trimul", "fused_triatt", "fused_transition"):
        lg = counters.BOOK.get(lever)
        assert lg.served >= 1 and not lg.fallbacks, (lever, lg.stats())
    counters.BOOK._ledgers.clear()
    dispatch.reset()


def test_exact_is_bitwise_off_on_the_af3_shape():
    """The flagship model's shapes (48-block configuration cut to 4 blocks and 6 sampler steps to keep the test
    short): 256 tokens, no padding, so the Pairformer stack passes replay from the verified graph cache and the
    sampler step from its verified graph; coordinates and confidence equal `off` bit for bit."""
    from uplifting_biomolecular_modeling_b200 import api
    from uplifting_biomolecular_modeling_b200.models import cofold
    kw = dict(pairformer_blocks=4, msa_blocks=1, sampling_steps=6, samples=2, recycles=2, confidence_blocks=1,
              token_depth=4)
    off = api.Predictor("af3", mode="off", device="cuda:0", seed=0, **kw)
    exact = api.Predictor("af3", mode="exact", device="cuda:0", seed=0, **kw)
    feats = cofold.synthetic_features(256, 8, off.cfg, seed=2)
    a = off.predict(feats)
    b = exact.predict(feats)
    b2 = exact.predict(feats)                    # second call: every stack pass and sampler step is a replay
    assert torch.equal(a["coords"], b["coords"]) and torch.equal(a["coords"], b2["coords"])
    assert torch.equal(a["plddt"], b["plddt"])
    g = exact.model.trunk_graphs
    assert g is not None and g.stats["captured"] >= 1 and g.stats["retired"] == 0 and g.stats["replayed"] >= 3
    assert exact.graph_verified >= 1


def test_big_mode_matches_fast_and_lowers_the_peak():
    """`big` on one GPU: row-blocked pair operations give the numbers of `fast` (same kernels, same sums per output)
    with a lower allocator peak; a padded input exercises the key masks of the blocked attention."""
    from uplifting_biomolecular_modeling_b200.models import pairformer
    from uplifting_biomolecular_modeling_b200.ops import native
    torch.manual_seed(1)
    N = 320
    layer = pairformer.PairformerLayer(no_seq=True).cuda().to(torch.bfloat16).eval()
    with torch.no_grad():
        for p in layer.parameters():
            p.normal_(0, 0.5 * p.shape[-1] ** -0.5 if p.dim() > 1 else 0.1)
        for mod in layer.modules():
            if isinstance(mod, torch.nn.LayerNorm):
                mod.weight.add_(1.0)
    z = torch.randn(1, N, N, 128, device="cuda").bfloat16()
    tok = torch.ones(N, device="cuda")
    tok[N - 30:] = 0
    pm = (tok[:, None] * tok[None, :]).unsqueeze(0)
    peaks, outs = [], []
    for rb in (0, 64):
        ws = {"row_block": rb} if rb else {}
        pairformer.set_impl(layer, "fused", workspace=ws)
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        with torch.no_grad():
            outs.append(layer.pair_update(z, pm))
        torch.cuda.synchronize()
        peaks.append(torch.cuda.max_memory_allocated() - base)
        ws.clear()
    native.raise_on_status("cuda", "big mode block")
    v = tok.bool()
    a, b = outs[0][0][v][:, v].float(), outs[1][0][v][:, v].float()
    assert ((a - b).abs().mean() / a.abs().mean()).item() < 5e-3
    assert peaks[1] < 0.7 * peaks[0], peaks


def test_rigid_alignment_runs_inside_the_sampler_graph():
    """The sampler's alignment of the noisy coordinates onto the denoised ones (fixed-sweep fp64 Jacobi SVD, no solver
    call) on the GPU: same rotation as on the CPU, and a captured sampler step with the alignment switched on replays
    bit for bit (the predictor compares the first replay with the eager step and refuses the graph otherwise)."""
    from uplifting_biomolecular_modeling_b200 import api
    from uplifting_biomolecular_modeling_b200.models import align, cofold
    g = torch.Generator().manual_seed(3)
    x = torch.randn(4, 200, 3, generator=g)
    y = torch.randn(4, 200, 3, generator=g)
    w = torch.rand(4, 200, generator=g)
    ref = align.weighted_rigid_align(x, y, w)
    got = align.weighted_rigid_align(x.cuda(), y.cuda(), w.cuda())
    assert (got.cpu() - ref).abs().max() < 1e-4
    pred = api.Predictor("tiny", mode="exact", device="cuda:0", seed=0)
    pred.model.structure_module.align_reverse_diff = True
    feats = cofold.synthetic_features(96, 8, pred.cfg, seed=1)
    out = pred.predict(feats, steps=6)
    assert torch.isfinite(out["coords"]).all()
    assert getattr(pred, "graph_verified", 0) >= 1
    off = api.Predictor("tiny", mode="off", device="cuda:0", seed=0)
    off.model.structure_module.align_reverse_diff = True
    want = off.predict(feats, steps=6)
    assert torch.equal(out["coords"], want["coords"])
