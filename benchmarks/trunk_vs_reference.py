"""The Pairformer trunk of this framework against the unmodified stock Boltz-2 modules, same GPU, same weights.

    python benchmarks/trunk_vs_reference.py [--n 1536] [--blocks 48] [--msa-blocks 4] [--msa-depth 1024]
                                            [--rounds 3] [--masked 0|1]

The stock side is ``boltz.model.layers.pairformer.PairformerModule`` (v2) and
``boltz.model.modules.trunkv2.MSAModule`` from the wheel the reference ships
(``boltz2/stock/boltz-2.2.1-py3-none-any.whl``, installed without dependencies under ``baseline/_ref``), run the way
upstream runs them at inference: eval mode, ``torch.autocast("cuda", torch.bfloat16)``, its own chunking rule
(boltz2/stock/src/boltz/model/layers/pairformer.py:180-186), ``use_kernels=False`` (cuEquivariance is not
installed here).  Its parameters are given random values (upstream zero-initialises output projections) and then
loaded into this package's modules with ``strict=True``, so both sides compute the same function.  Timing:
interleaved rounds (stock, ours, stock, ...), CUDA events, a write larger than L2 before every run; prints

    TRUNKREF <stage> N=<n> blocks=<b> stock_ms=<..> ours_ms=<..> ratio=<stock/ours> rel_err_mean=<..>

``rel_err_mean`` is mean |ours - stock| / mean |stock| of the pair output (both sides compute in bf16).
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
REF = os.path.join(ROOT, "baseline", "_ref")

import torch

from uplifting_biomolecular_modeling_b200.models import msa as own_msa
from uplifting_biomolecular_modeling_b200.models import pairformer as own_pf


def randomize(module, seed=123):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p in module.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * (0.1 if p.dim() == 1 else 0.5 * p.shape[-1] ** -0.5))
        for m in module.modules():
            if isinstance(m, torch.nn.LayerNorm) and m.weight is not None:
                m.weight.add_(1.0)
    return module


def timed(fns, rounds):
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    ts = [[] for _ in fns]
    for _ in range(rounds):
        for i, f in enumerate(fns):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            ts[i].append(e0.elapsed_time(e1))
    return [sorted(t)[len(t) // 2] for t in ts]


def stock_available():
    """(True, "") or (False, reason naming what is missing)."""
    if not os.path.isdir(os.path.join(REF, "boltz")):
        return False, "baseline/_ref/boltz is not installed (pip install --no-deps --target baseline/_ref of the stock wheel)"
    if REF not in sys.path:
        sys.path.insert(0, REF)
    try:
        import boltz.model.layers.pairformer  # noqa: F401
        import boltz.model.modules.trunkv2  # noqa: F401
    except Exception as e:  # noqa: BLE001
        return False, f"stock trunk modules do not import: {type(e).__name__}: {e}"
    return True, ""


def measure(n=1536, blocks=48, msa_blocks=4, msa_depth=1024, rounds=3, masked=False, ours=True, log=print):
    """Returns {"pairformer": {...}, "msa_module": {...}} with stock (and, if asked, own) times in ms."""
    from boltz.data import const
    from boltz.model.layers import pairformer as sp
    from boltz.model.modules import trunkv2 as st
    dev = "cuda"
    res = {}
    torch.manual_seed(0)
    mask = torch.ones(1, n, device=dev)
    if masked:
        mask[:, n - n // 10:] = 0
    pm = mask[:, :, None] * mask[:, None, :]
    s = torch.randn(1, n, 384, device=dev)
    z = torch.randn(1, n, n, 128, device=dev)
    with torch.no_grad():
        # ------------------------------------------------------------------ Pairformer stack
        ref = randomize(sp.PairformerModule(384, 128, num_blocks=blocks, v2=True)).eval().to(dev)
        holder = {}

        def run_stock():
            with torch.autocast("cuda", dtype=torch.bfloat16):
                holder["ref"] = ref(s, z, mask, pm)
        fns = [run_stock]
        if ours:
            own = own_pf.PairformerModule(384, 128, num_blocks=blocks).eval()
            own.load_state_dict({k: v.cpu() for k, v in ref.state_dict().items()}, strict=True)
            own = own.to(dev).to(torch.bfloat16)
            ws = {}
            own_pf.set_impl(own, "fused", workspace=ws)
            sb, zb = s.bfloat16(), z.bfloat16()
            use_mask = masked

            def run_own():
                holder["own"] = own(sb, zb, mask if use_mask else None, pm if use_mask else None)
            fns.append(run_own)
        for f in fns:
            f()                                  # warm-up (weight packing, Triton-free: nothing compiles)
        torch.cuda.synchronize()
        t = timed(fns, rounds)
        entry = {"stock_ms": round(t[0], 2), "n": n, "blocks": blocks, "masked": bool(masked)}
        if ours:
            zr, zo = holder["ref"][1].float(), holder["own"][1].float()
            v = mask[0].bool()
            zr, zo = zr[0][v][:, v], zo[0][v][:, v]
            entry.update(ours_ms=round(t[1], 2), ratio=round(t[0] / t[1], 3),
                         rel_err_mean=float((zr - zo).abs().mean() / zr.abs().mean()))
        res["pairformer"] = entry
        log("TRUNKREF pairformer " + " ".join(f"{k}={v}" for k, v in entry.items()))
        del ref, holder
        if ours:
            del own, ws
        torch.cuda.empty_cache()
        # ------------------------------------------------------------------ MSA module
        if msa_blocks > 0:
            S = msa_depth
            refm = randomize(st.MSAModule(msa_s=64, token_z=128, token_s=384, msa_blocks=msa_blocks, msa_dropout=0.0,
                                          z_dropout=0.0)).eval().to(dev)
            feats = {"msa": torch.randint(0, const.num_tokens, (1, S, n), device=dev),
                     "has_deletion": torch.zeros(1, S, n, device=dev), "deletion_value": torch.zeros(1, S, n, device=dev),
                     "msa_paired": torch.zeros(1, S, n, device=dev), "msa_mask": torch.ones(1, S, n, device=dev),
                     "token_pad_mask": mask}
            emb = torch.randn(1, n, 384, device=dev)
            holder = {}

            def run_stock_msa():
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    holder["ref"] = refm(z, emb, feats)
            fns = [run_stock_msa]
            if ours:
                nfeat = const.num_tokens + 3
                ownm = own_msa.MSAModule(64, 128, 384, num_blocks=msa_blocks, msa_feat=nfeat).eval()
                ownm.load_state_dict({k: v.cpu() for k, v in refm.state_dict().items()}, strict=True)
                ownm = ownm.to(dev).to(torch.bfloat16)
                own_pf.set_impl(ownm, "fused", workspace={})
                for layer in ownm.layers:
                    layer.outer_product_mean.full_mask = True
                msa_feat = torch.cat([torch.nn.functional.one_hot(feats["msa"], const.num_tokens).bfloat16(),
                                      torch.zeros(1, S, n, 3, device=dev, dtype=torch.bfloat16)], -1)
                zb, eb = z.bfloat16(), emb.bfloat16()

                def run_own_msa():
                    holder["own"] = ownm(zb, eb, msa_feat, feats["msa_mask"], mask, pm if masked else None)
                fns.append(run_own_msa)
            for f in fns:
                f()
            torch.cuda.synchronize()
            t = timed(fns, rounds)
            entry = {"stock_ms": round(t[0], 2), "n": n, "blocks": msa_blocks, "msa_depth": S}
            if ours:
                zr, zo = holder["ref"].float(), holder["own"].float()
                entry.update(ours_ms=round(t[1], 2), ratio=round(t[0] / t[1], 3),
                             rel_err_mean=float((zr - zo).abs().mean() / zr.abs().mean()))
            res["msa_module"] = entry
            log("TRUNKREF msa_module " + " ".join(f"{k}={v}" for k, v in entry.items()))
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=1536)
    ap.add_argument("--blocks", type=int, default=48)
    ap.add_argument("--msa-blocks", type=int, default=4)
    ap.add_argument("--msa-depth", type=int, default=1024)
    ap.add_argument("--rounds", type=int, default=3)
    ap.add_argument("--masked", type=int, default=0)
    a = ap.parse_args()
    ok, why = stock_available()
    if not ok:
        print(f"TRUNKREF unavailable: {why}")
        return 0
    print(f"TRUNKREF stack torch={torch.__version__} gpu={torch.cuda.get_device_name(0)} stock=boltz-2.2.1 "
          f"(use_kernels=False, bf16 autocast)")
    measure(a.n, a.blocks, a.msa_blocks, a.msa_depth, a.rounds, bool(a.masked))
    return 0


if __name__ == "__main__":
    sys.exit(main())
