"""Public prediction API: ``Predictor(config, mode).predict(features)``.

One object owns a model on one GPU under one mode word:

* ``off``   - the plain PyTorch statements (``ops.reference``), eager.
* ``exact`` - the same statements, with what is step-invariant hoisted and the sampler step replayed
              from a CUDA graph: bitwise identical to ``off`` by construction (same kernels, same order).
* ``fast``  - the fused sm_100a kernels in the pair stack / MSA module / diffusion transformer, plus graphs.
* ``big``   - ``fast`` plus the memory levers: triangle attention and the triangle-multiplication contraction run
              per block of ``row_block`` rows (q|k|v|gate and the contracted planes exist for one block), the trunk's
              scratch is released before the sampler; with ``n_gpu > 1`` the pair tensor is row-sharded over the
              ranks (``parallel.rowpair``).

``predict`` takes a feature dict on the host (pinned memory is used for the copy), runs embed ->
trunk -> sampler -> confidence, and returns host tensors.  It is the call the benchmarks time end to end.
Mode vocabulary and the no-silent-fallback rule are those of the reference kits (README.md:24-50).
"""
from __future__ import annotations

import os
import sys
import time
from typing import Dict, Optional

import torch

from .models import cofold

MODES = ("off", "exact", "fast", "big")


class NotActive(RuntimeError):
    """The requested mode cannot engage on this machine (exit code 3 at the CLI)."""


def _tree_copy(dst, src) -> None:
    """Copy every tensor of ``src`` into the tensor at the same place of ``dst`` (dicts / lists / tuples)."""
    if isinstance(dst, torch.Tensor):
        dst.copy_(src)
    elif hasattr(dst, "view") and isinstance(getattr(dst, "view"), torch.Tensor) and not isinstance(dst, dict):
        dst.view.copy_(src.view)              # models.pairformer.BiasPlanes
    elif hasattr(dst, "data") and isinstance(getattr(dst, "data"), torch.Tensor) and not isinstance(dst, dict):
        dst.data.copy_(src.data)              # models.diffusion.WindowBias
    elif isinstance(dst, dict):
        for k in dst:
            _tree_copy(dst[k], src[k])
    elif isinstance(dst, (list, tuple)):
        for d, s_ in zip(dst, src):
            _tree_copy(d, s_)


class Predictor:
    def __init__(self, config: str = "af3", mode: str = "fast", device: str = "cuda:0",
                 dtype: torch.dtype = torch.bfloat16, seed: int = 0, use_graphs: Optional[bool] = None,
                 model=None, **overrides):
        """``model``: an already built model of ``config`` (the row-sharded worker hands its replica over for the
        structure and confidence stages); otherwise the model is built here."""
        if mode not in MODES:
            raise ValueError(f"mode {mode!r} not in {MODES}")
        self.mode, self.device, self.dtype, self.seed = mode, torch.device(device), dtype, seed
        self.model = model if model is not None else \
            cofold.build_model(config, device=self.device, dtype=dtype, seed=seed, **overrides)
        self.cfg = self.model.cfg
        self.levers = []
        # numerics of every mode: no TF32 in the fp32 parts, highest matmul precision; applied around each prediction
        # and restored afterwards (core.det.NumericsGuard), recorded in manifests and trunk checkpoints
        from .core import det
        self.policy = det.Policy(compute_dtype="bf16" if dtype == torch.bfloat16 else str(dtype).replace("torch.", ""),
                                 allow_tf32=False, autocast=False, matmul_precision="highest")
        self.numerics = det.numerics_signature(self.policy)
        if mode in ("fast", "big"):
            if self.device.type != "cuda":
                raise NotActive(f"mode {mode} needs a CUDA device (sm_100a); got {self.device}")
            from .ops import native
            try:
                native.lib()
            except native.NativeUnavailable as e:
                raise NotActive(f"mode {mode}: {e}") from e
            if os.environ.get("UBM_LOADCHECK", "1") != "0":
                # every kernel family reproduces its fp32 statement on this GPU before it serves (once per process)
                from .ops import loadcheck
                try:
                    loadcheck.require(self.device, tag="ubm")
                except loadcheck.KernelsRefused as e:
                    raise NotActive(f"mode {mode}: {e}") from e
            n = self.model.set_impl("fused")
            self.levers.append(f"fused_kernels:{n}")
        self.use_graphs = (mode != "off" and self.device.type == "cuda") if use_graphs is None else use_graphs
        self.verify_graphs = 1 if mode != "off" else 0      # first replay of a captured graph checked against eager
        self.row_block = 0          # ``big``: pair operations of the kernel path in blocks of this many rows
        self.release = False        # ``big``: trunk scratch returned to the allocator before the sampler
        if mode == "big":
            self.row_block = int(os.environ.get("UBM_BIG_ROW_BLOCK", "512"))
            self.model.workspace["row_block"] = self.row_block
            self.release = True
            self.model.park_z_init = True
        if mode in ("fast", "big"):
            from .ops import dispatch
            dispatch.set_tier(mode)
        self.graph_pool = None
        if self.use_graphs and self.device.type == "cuda":
            # capture sites of this predictor under one byte budget and one census (capture.pool); the Pairformer
            # stack is the first site: captured at the second sighting of a shape, first replay verified
            from .capture import pool as _pool
            self.graph_pool = _pool.GraphPool(budget_bytes=4 << 30, default_policy=_pool.FixedK(2))
            self.graph_pool.site("pairformer_stack", verify=self.verify_graphs)
            self.model.trunk_graphs = self.graph_pool.handle("pairformer_stack")
        self.sample_chunk = int(os.environ.get("UBM_BIG_SAMPLE_CHUNK", "0")) if mode == "big" else 0
        self.stage_peaks: Dict[str, Dict[str, int]] = {}
        self._graph = None
        self._graph_key = None
        self._pinned: Dict[str, torch.Tensor] = {}
        self.last_timing: Dict[str, float] = {}

    def set_mode(self, mode: str) -> None:
        """Change the mode word of a predictor built under ``off`` (the kit runner builds the plain model first and
        lets the activation's levers switch implementations on one by one)."""
        if mode not in MODES:
            raise ValueError(f"mode {mode!r} not in {MODES}")
        self.mode = mode
        if mode in ("fast", "big"):
            from .ops import dispatch
            dispatch.set_tier(mode)

    # ------------------------------------------------------------------ provider decisions
    def provider_plan(self, n_tokens: int, n_atoms: Optional[int] = None) -> Dict[str, object]:
        """The row of every op family that serves this model's call classes at ``n_tokens`` under the current mode,
        looked up in the measured table and recorded in the cell census (once per call class).  ``off`` has no
        providers."""
        if self.mode == "off":
            return {}
        from .core import arch
        from .ops import provider
        sm = (arch.device_sm(self.device.index or 0) if self.device.type == "cuda" else None) or "cpu"
        c = self.cfg
        dt = "bf16" if self.dtype == torch.bfloat16 else str(self.dtype).replace("torch.", "")
        tri_heads, d_tri = 4, 32                                   # triangle attention: 4 heads of 32 channels
        d_tok = 64                                                  # token attention: 768 / 16 = 48, padded to 64
        calls = [
            ("triattn", f"D{d_tri}H{tri_heads}", n_tokens, {"head_dim": d_tri, "dtype": dt}),
            ("trimul", f"C{c.c_z}H{c.c_z}", n_tokens, {"c_z": c.c_z, "c_hidden": c.c_z, "dtype": dt}),
            ("transition", f"C{c.c_z}X4", n_tokens, {"c": c.c_z, "expansion": 4, "dtype": dt}),
            ("transition", f"C{c.c_s}X4", n_tokens, {"c": c.c_s, "expansion": 4, "dtype": dt}),
            ("transition", f"C{c.c_m}X4", n_tokens, {"c": c.c_m, "expansion": 4, "dtype": dt}),
            ("apb", f"D{d_tok}H{c.token_heads}S{c.samples}", n_tokens, {"head_dim": d_tok, "dtype": dt}),
            ("ln", f"C{c.c_z}", n_tokens, {"c": c.c_z, "dtype": dt}),
            ("ln", f"C{c.c_m}", n_tokens, {"c": c.c_m, "dtype": dt}),
        ]
        if n_atoms:
            calls.append(("apb", "WIN32x128", n_atoms, {"head_dim": c.c_atom // c.atom_heads, "window": (32, 128),
                                                        "dtype": dt}))
        plan = {}
        for fam, klass, n, call in calls:
            plan[f"{fam}|{klass}"] = provider.select(fam, sm, klass, n, self.mode, call)
        self.last_plan = plan
        return plan

    # ------------------------------------------------------------------ host <-> device
    def to_device(self, feats: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        out = {}
        self.h2d_bytes = 0
        no_padding = bool(feats["token_mask"].min() > 0) if "token_mask" in feats else False
        msa_full = bool(feats["msa_mask"].min() > 0) if "msa_mask" in feats else False
        for k, v in feats.items():
            if self.device.type == "cuda":
                pin = self._pinned.get(k)
                if pin is None or pin.shape != v.shape or pin.dtype != v.dtype:
                    pin = torch.empty(v.shape, dtype=v.dtype, pin_memory=True)
                    self._pinned[k] = pin
                pin.copy_(v)
                d = pin.to(self.device, non_blocking=True)
                self.h2d_bytes += v.numel() * v.element_size()
            else:
                d = v
            out[k] = d.to(self.dtype) if d.is_floating_point() else d
        out["no_padding"] = no_padding
        out["msa_full"] = msa_full      # host-side facts about the masks: they select mask-free kernels
        out["_on_device"] = True
        return out

    # ------------------------------------------------------------------ sampler step graph
    def _step_fn(self, prep, feats, n_tokens, samples):
        """Sampler step as a CUDA graph.  The graph is captured once per (tokens, atoms, samples) on the
        first prediction's step-invariant tensors; later predictions copy theirs into those buffers and
        replay (capture-once, replay-many; reference: common/opt_core/opt_core/capture/graphs.py:569)."""
        if not self.use_graphs:
            return None
        sm = self.model.structure_module
        A = feats["ref_pos"].shape[1]
        key = (n_tokens, A, samples)
        if self._graph is not None and self._graph_key == key:
            from .models import diffusion
            # the captured step reads the atom -> token tables of its static a2t tensor: rewrite them in place
            if diffusion.refresh_segment_tables(self._graph["a2t"], feats["atom_to_token"][0], n_tokens):
                _tree_copy(self._graph["prep"], prep)
                return self._graph["fn"]
            self._graph = None          # a token with more atoms than any before: tables change shape, recapture
        a2t = feats["atom_to_token"][0].clone()
        static_x = torch.zeros((samples, A, 3), device=self.device)
        static_s = torch.zeros(3, device=self.device)
        # RNG discipline of the captured step (diffusion_loop.rng): the step draws from the device's default
        # generator, which the graph registers, so replays advance it (contract ``registered``); a module left in
        # training mode under another contract, or an undeclared contract, refuses the capture
        from .diffusion_loop import rng as _rng
        gate = _rng.capture_contract_gate(_rng.RNG_REGISTERED, [sm])
        if not gate.ok:
            raise NotActive(f"sampler graph refused: {gate.detail}")
        if os.environ.get("UBM_GRAPH_AUDIT") == "1":
            # opt-in audit before the capture (capture.audit): host synchronisations, allocator growth between warm
            # runs; draws are allowed under the registered contract
            from .capture import audit as _audit
            rep = _audit.audit_capture_safety(
                lambda: sm.step(static_x, static_s[0] + 1.0, static_s[1] + 0.5, static_s[2], prep, a2t, n_tokens),
                allow_rng=True, check_determinism=False)
            print(rep.line("sampler_step"), file=sys.stderr, flush=True)
            if not rep.safe:
                raise NotActive("sampler graph refused by the capture audit: " + "; ".join(rep.findings))
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                sm.step(static_x, static_s[0] + 1.0, static_s[1] + 0.5, static_s[2], prep, a2t, n_tokens)
        torch.cuda.current_stream(self.device).wait_stream(side)
        from .ops import native
        before = native.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_out = sm.step(static_x, static_s[0], static_s[1], static_s[2], prep, a2t, n_tokens)
        per_replay = native.launch_count() - before      # kernels of this library inside one replay

        def fn(x, sig_tm, sig_t, gamma):
            static_x.copy_(x)
            static_s[0].copy_(sig_tm)
            static_s[1].copy_(sig_t)
            static_s[2].copy_(gamma)
            graph.replay()
            if per_replay:
                native.add_launches(per_replay)
            return static_out

        if self.verify_graphs:
            # replay against the eager step on the same inputs and random state: bit for bit, or the graph is not used
            # (reference: common/opt_core/opt_core/capture/graphs.py:569, ``verify >= 1``)
            gen = torch.Generator(device=self.device).manual_seed(97)
            x0 = torch.randn((samples, A, 3), device=self.device, generator=gen)
            args = (x0, torch.tensor(1.5, device=self.device), torch.tensor(0.75, device=self.device),
                    torch.tensor(0.0, device=self.device))
            torch.cuda.manual_seed(4242)
            got = fn(*args).clone()
            torch.cuda.manual_seed(4242)
            want = sm.step(*args, prep, a2t, n_tokens)
            if not torch.equal(got, want):
                worst = float((got - want).abs().max())
                raise NotActive(f"sampler graph replay differs from the eager step (max abs {worst:.3e})")
            self.graph_verified = getattr(self, "graph_verified", 0) + 1
        self._graph = {"graph": graph, "prep": prep, "a2t": a2t, "fn": fn}
        self._graph_key = key
        return fn

    # ------------------------------------------------------------------ one prediction
    @torch.no_grad()
    def predict(self, feats_host: Dict[str, torch.Tensor], recycles: Optional[int] = None,
                samples: Optional[int] = None, steps: Optional[int] = None, confidence: bool = True,
                seed: Optional[int] = None, to_host: bool = True) -> Dict[str, torch.Tensor]:
        from .core import det
        with det.NumericsGuard(self.policy):
            return self._predict(feats_host, recycles, samples, steps, confidence, seed, to_host)

    def _predict(self, feats_host, recycles, samples, steps, confidence, seed, to_host):
        m = self.model
        dev = self.device
        if dev.type == "cuda":
            torch.cuda.manual_seed(self.seed if seed is None else seed)
        else:
            torch.manual_seed(self.seed if seed is None else seed)
        timing = os.environ.get("UBM_STAGE_TIMES") == "1" and dev.type == "cuda"
        marks = []

        census = self.mode == "big" and dev.type == "cuda"
        if census:
            from .mem import peak as _peak
            _peak.reset(dev)

        def mark(name):
            if timing:
                torch.cuda.synchronize(dev)
                marks.append((name, time.perf_counter()))
            if census and name != "start":
                # per-stage peak of the allocator (``big`` only): what the memory levers are judged by
                self.stage_peaks[name] = _peak.allocator_peak(dev)
                _peak.reset(dev)

        mark("start")
        # features already on the device (a dict produced by to_device) skip the host copy; with
        # to_host=False the result stays on the device as well: the device-only form of the same call
        feats = feats_host if feats_host.get("_on_device") is True else self.to_device(feats_host)
        s_inputs, s_init, z_init, atom_c, atom_p = m.embed(feats)
        mark("embed")
        s, z = m.trunk(feats, s_inputs, s_init, z_init, recycles)
        mark("trunk")
        out = self.structure_and_confidence(feats, s, z, s_inputs, atom_c, atom_p, samples, steps, confidence, seed,
                                            mark)
        host = {k: v.float().cpu() for k, v in out.items()} if to_host else {k: v.float() for k, v in out.items()}
        mark("confidence_and_copy")
        if timing:
            self.last_timing = {marks[i][0]: round((marks[i][1] - marks[i - 1][1]) * 1e3, 2)
                                for i in range(1, len(marks))}
            import sys
            print(f"[ubm] STAGES ms {self.last_timing}", file=sys.stderr, flush=True)
        self.d2h_bytes = sum(v.numel() * 4 for v in host.values()) if to_host else 0
        if dev.type == "cuda" and m.fused:
            from .ops import native
            native.raise_on_status(dev, "predict")
        return host

    @torch.no_grad()
    def structure_and_confidence(self, feats, s, z, s_inputs, atom_c, atom_p, samples=None, steps=None,
                                 confidence: bool = True, seed: Optional[int] = None, mark=lambda name: None):
        """Sampler and confidence head on a finished trunk (s [1, N, c_s], z [1, N, N, c_z] on this device); returns
        device tensors.  ``predict`` calls it after its own trunk; the row-sharded worker calls it on rank 0 with the
        gathered pair tensor."""
        m = self.model
        dev = self.device
        N = s.shape[1]
        nsamp = samples or self.cfg.samples
        if getattr(self, "_plan_key", None) != N:
            self._plan_key = N
            self.provider_plan(N, feats["ref_pos"].shape[1] if "ref_pos" in feats else None)
        sm = m.structure_module
        if self.release:
            # ``big``: the pair stack's scratch (projection planes, q|k|v|gate rows) goes back to the allocator
            keep = {k: v for k, v in m.workspace.items() if k == "row_block"}
            m.workspace.clear()
            m.workspace.update(keep)
            if dev.type == "cuda":
                torch.cuda.empty_cache()
        prep = sm.score_model.prepare(s, s_inputs, m.z_cond_norm(z), atom_c, atom_c, atom_p, m.fused)
        step_fn = self._step_fn(prep, feats, N, nsamp)
        # the sampler's random stream starts here in every mode (graph warm-up / capture draw numbers too)
        if dev.type == "cuda":
            torch.cuda.manual_seed(self.seed if seed is None else seed)
        else:
            torch.manual_seed(self.seed if seed is None else seed)
        mark("sampler_setup")
        if self.sample_chunk and nsamp > self.sample_chunk:
            # ``big``: the samples are rolled out a chunk at a time (peak of the structure stage = one chunk); every
            # chunk continues the same random stream, so the samples differ from an unchunked run's
            from .mem import sample_loop
            chunk_fn = self._step_fn(prep, feats, N, self.sample_chunk) if self.use_graphs else None

            def roll(k0, k1):
                fn = chunk_fn if (k1 - k0) == self.sample_chunk else None
                return m.structure(feats, s, z, s_inputs, atom_c, atom_p, k1 - k0, steps, None, fn, prep)[0]
            x = sample_loop.run(roll, None, nsamp, self.sample_chunk)["coords"].to(dev)
        else:
            x, _ = m.structure(feats, s, z, s_inputs, atom_c, atom_p, nsamp, steps, None, step_fn, prep)
        mark("sampler")
        out = {"coords": x}
        if confidence:
            rep = feats["token_rep_atom"][0]
            conf = m.confidence_module(s, z, x[:1, rep].to(s.dtype))
            p = torch.softmax(conf["plddt_logits"].float(), -1)
            out["plddt"] = (p * (torch.arange(50, device=p.device) + 0.5) / 50).sum(-1)
            pae = torch.softmax(conf["pae_logits"].float(), -1)
            out["pae_mean"] = (pae * (torch.arange(64, device=p.device) + 0.5) * 0.5).sum(-1).mean()
        return out
