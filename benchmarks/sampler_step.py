"""One sampler step of the flagship model (24-block diffusion transformer over 5 samples, atom encoder / decoder) in
isolation: the trunk is skipped (random single / pair representations of the right shapes), the step-invariant
part is prepared once, then

* ``--mode time`` (default) times the graph-replayed step with CUDA events (``--iters`` replays between the events,
  the step's working set of activations and weights exceeds L2), and the same step launched eagerly;
* ``--mode list`` runs ``--eager-steps`` eager steps and exits, for a one-pass launch list under a profiler
  (kernels are serialised there, so programmatic dependent launch does not blur the per-kernel durations).

    python benchmarks/sampler_step.py --tokens 1536
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch

from uplifting_biomolecular_modeling_b200 import api
from uplifting_biomolecular_modeling_b200.models import cofold


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=1536)
    ap.add_argument("--config", default="af3")
    ap.add_argument("--mode", default="time", choices=["time", "list"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--eager-steps", type=int, default=2)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    pred = api.Predictor(a.config, mode="fast", device="cuda:0")
    cfg, m = pred.cfg, pred.model
    N = a.tokens
    feats = pred.to_device(cofold.synthetic_features(N, 8, cfg, chains=cofold.chains_for(a.config, N)))
    with torch.no_grad():
        s_inputs, s_init, z_init, atom_c, atom_p = m.embed(feats)
        s = torch.randn_like(s_init)
        z = torch.randn_like(z_init)
        sm = m.structure_module
        prep = sm.score_model.prepare(s, s_inputs, m.z_cond_norm(z), atom_c, atom_c, atom_p, m.fused)
        a2t = feats["atom_to_token"][0]
        A = feats["ref_pos"].shape[1]
        x = torch.randn((cfg.samples, A, 3), device=dev)
        t = [torch.tensor(v, device=dev) for v in (1.5, 0.75, 0.0)]
        if a.mode == "list":
            for _ in range(a.eager_steps):
                x = sm.step(x, *t, prep, a2t, N)
            torch.cuda.synchronize()
            print(f"SAMPLER-STEP list tokens={N} atoms={A} samples={cfg.samples} eager_steps={a.eager_steps}")
            return
        fn = pred._step_fn(prep, feats, N, cfg.samples)
        for _ in range(3):
            fn(x, *t)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.iters):
            fn(x, *t)
        e1.record()
        torch.cuda.synchronize()
        graph_ms = e0.elapsed_time(e1) / a.iters
        for _ in range(2):
            sm.step(x, *t, prep, a2t, N)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.iters):
            sm.step(x, *t, prep, a2t, N)
        e1.record()
        torch.cuda.synchronize()
        eager_ms = e0.elapsed_time(e1) / a.iters
    print(f"SAMPLER-STEP tokens={N} atoms={A} samples={cfg.samples} graph_ms={graph_ms:.3f} eager_ms={eager_ms:.3f}")


if __name__ == "__main__":
    main()
