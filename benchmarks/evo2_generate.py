"""Evo2-shaped generation: one long prefill and a run of single-token decode steps, optionally tensor parallel.

    python benchmarks/evo2_generate.py --config evo2_7b --prefill 32768 --new 256                      # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 --master-port 29561 \
        benchmarks/evo2_generate.py --config evo2_7b --prefill 32768 --new 256                         # TP = P

bf16, random-init weights of the named configuration, a random byte prompt.  The kernel path is on
(``set_impl("fused")``: RMSNorm, FIR / gate stages, convolution epilogues, decode state step, tcgen05 GEMMs; under
tensor parallelism the row-parallel projections use the GEMM whose epilogue does the reduce-scatter over peer
memory).  Times are CUDA-event times, max over ranks; rank 0 prints one JSON line.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="evo2_7b")
    ap.add_argument("--prefill", type=int, default=32768)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = the configuration's)")
    ap.add_argument("--impl", default="fused", choices=["fused", "torch"])
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--graph", type=int, default=1, help="1: decode step captured in a CUDA graph and replayed")
    ap.add_argument("--fp8", type=int, default=0, help="1: the input projections of the Hyena operators in e4m3 during the prefill")
    ap.add_argument("--kernel-table", type=int, default=0, help="1: after two warm prefills, run one prefill under the torch profiler, print its kernel times by name and stop")
    ap.add_argument("--specdec", type=int, default=0, help="k > 0: also time speculative decoding with k proposals per round")
    ap.add_argument("--draft", default="evo2_1b", help="configuration of the draft model for --specdec")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from uplifting_biomolecular_modeling_b200.models import evo2
    from uplifting_biomolecular_modeling_b200.ops import native
    over = {"n_layers": a.layers, "attn_layers": tuple(i for i in evo2.CONFIGS[a.config].attn_layers if i < a.layers)} \
        if a.layers else {}
    model = evo2.build(a.config, device=dev, dtype=torch.bfloat16, seed=0, **over)
    par = None
    if a.impl == "fused":
        model.set_impl("fused")
        if a.fp8:
            model.set_fp8_input_projections(True)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        from uplifting_biomolecular_modeling_b200.parallel import comm, symm, tp
        par = tp.TensorParallel(comm.GroupComm(), symm.SymmHeap())
        par.shard_evo2(model)
    g = torch.Generator(device=dev).manual_seed(1)
    tokens = torch.randint(0, model.cfg.vocab, (1, a.prefill), device=dev, generator=g)

    if a.kernel_table:
        # shares of one warm prefill by kernel name (torch profiler: not a timing, the timed numbers come from the
        # CUDA events of the normal run)
        import collections
        import re
        from torch.profiler import ProfilerActivity, profile
        for _ in range(2):
            model(tokens, [dict() for _ in model.blocks])
        torch.cuda.synchronize(dev)
        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            model(tokens, [dict() for _ in model.blocks])
            torch.cuda.synchronize(dev)
        agg = collections.defaultdict(lambda: [0, 0.0])
        for ev in prof.events():
            if ev.device_type == torch.autograd.DeviceType.CUDA:
                k = re.sub(r"\(.*", "", re.sub(r"<.*", "", ev.name))[-70:]
                agg[k][0] += 1
                agg[k][1] += ev.device_time_total
        if rank == 0:
            print(f"KERNELS total_ms={sum(v[1] for v in agg.values()) / 1e3:.2f} prefill_tokens={a.prefill}")
            for k, (c, t) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:30]:
                print(f"KERNELS {t / 1e3:9.2f} ms {c:5d}  {k}")
        return

    def run():
        states = [dict() for _ in model.blocks]
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        logits = model(tokens, states)
        nxt = logits[:, -1:].argmax(-1)
        e[1].record()
        if a.graph:
            # capture (one eager step + one captured step) is inside the timed decode region
            nxt = model._generate_graph(tokens, states, nxt, a.new)[:, -1:]
        else:
            for _ in range(a.new - 1):
                nxt = model.step(nxt, states)[:, -1:].argmax(-1)
        e[2].record()
        torch.cuda.synchronize(dev)
        return e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2]), int(nxt.item())

    for _ in range(a.warmup):
        run()
    if world > 1:
        torch.distributed.barrier()
    pre, dec, last = run()
    native.raise_on_status(dev, "evo2 generate")
    t = torch.tensor([pre, dec], device=dev)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    spec = None
    if a.specdec > 0 and world == 1:
        # Random-init weights make the acceptance rate meaningless (target and draft agree by chance); what the
        # run measures is the cost of a round: k draft steps + one target pass over k + 1 tokens, against the
        # target's single-token step (both eager).
        draft = evo2.build(a.draft, device=dev, dtype=torch.bfloat16, seed=1)
        if a.impl == "fused":
            draft.set_impl("fused")
        short = tokens[:, :min(a.prefill, 4096)]
        model.generate_speculative(draft, short, 2 * (a.specdec + 1), k=a.specdec)          # warm-up
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        states = [dict() for _ in model.blocks]
        nxt = model(short, states)[:, -1:].argmax(-1)
        ev[0].record()
        for _ in range(16):
            nxt = model.step(nxt, states)[:, -1:].argmax(-1)
        ev[1].record()
        seq = torch.randint(0, model.cfg.vocab, (1, a.specdec + 1), device=dev, generator=g)
        for _ in range(16):
            model.extend(seq, states)
            model.commit(states, 1)
        ev[2].record()
        _, stats = model.generate_speculative(draft, short, 16 * (a.specdec + 1), k=a.specdec)
        ev[3].record()
        torch.cuda.synchronize(dev)
        spec = {"k": a.specdec, "draft": a.draft, "target_step_ms_eager": round(ev[0].elapsed_time(ev[1]) / 16, 3),
                "target_pass_over_k_plus_1_ms": round(ev[1].elapsed_time(ev[2]) / 16, 3),
                "rounds": stats["rounds"], "accepted": stats["accepted"], "proposed": stats["proposed"],
                "ms_per_round_incl_prefill": round(ev[2].elapsed_time(ev[3]) / max(stats["rounds"], 1), 3)}
    if rank == 0:
        pre, dec = t.tolist()
        print(json.dumps({
            "bench": "evo2_generate", "config": a.config, "layers": model.cfg.n_layers, "tp": world, "impl": a.impl, "fp8_input_projections": bool(a.fp8), "decode_graph": bool(a.graph),
            "prefill_tokens": a.prefill, "new_tokens": a.new, "prefill_ms": round(pre, 2),
            "prefill_tokens_per_s": round(a.prefill / pre * 1e3, 1), "decode_ms_per_token": round(dec / max(a.new - 1, 1), 3),
            "decode_tokens_per_s": round((a.new - 1) / dec * 1e3, 1), "last_token": last,
            "fused_reduce_scatter_calls": 0 if par is None else par.fused_calls,
            "peak_gb": round(torch.cuda.max_memory_allocated(dev) / 2 ** 30, 2), "specdec": spec}), flush=True)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
