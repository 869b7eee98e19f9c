"""Multi-GPU checks as tests: each starts its ranks as child processes (one per GPU, NCCL over NVLink, NVLS off, the
package's kernels on plain peer loads) and asserts on the line rank 0 prints.  Skipped with fewer than two GPUs."""
import os
import re
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _run(script, args, world, tmp_path, timeout=600):
    from uplifting_biomolecular_modeling_b200.parallel import launch
    log_dir = str(tmp_path / "logs")
    launch.run_rank_processes(world, [sys.executable, os.path.join(ROOT, script), *map(str, args)], cpu=False,
                              run_timeout_s=timeout, log_dir=log_dir,
                              extra_env={"PYTHONPATH": ROOT, "NCCL_NVLS_ENABLE": "0"}, echo_rank0=False)
    return open(os.path.join(log_dir, "rank0.log")).read()


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("gather", ["peer", "nccl"])
def test_row_sharded_pair_block_matches_single_gpu(tmp_path, gather):
    world = 2
    log = _run("tests/multigpu/rowpair_fused_check.py", [384, 0, gather], world, tmp_path)
    m = re.search(r"ROWPAIR-FUSED ok world=(\d+) N=384 gather=(\w+) err_vs_single_gpu_fused=([0-9.e+-]+) "
                  r"err_vs_fp32=([0-9.e+-]+)", log)
    assert m, log[-2000:]
    assert int(m.group(1)) == world and m.group(2) == gather
    assert float(m.group(3)) < 5e-3 and float(m.group(4)) < 4e-2


@pytest.mark.skipif(_gpus() < 4, reason="needs four GPUs")
def test_row_sharded_pair_block_on_four_gpus_even_rows(tmp_path):
    """128 rows per rank: the transposed projections read z columns from the owners inside the kernel."""
    log = _run("tests/multigpu/rowpair_fused_check.py", [512, 0, "peer"], 4, tmp_path)
    assert "ROWPAIR-FUSED ok world=4 N=512" in log, log[-2000:]


@pytest.mark.skipif(_gpus() < 4, reason="needs four GPUs")
def test_row_sharded_pair_block_on_four_gpus_with_ragged_rows(tmp_path):
    log = _run("tests/multigpu/rowpair_fused_check.py", [328, 0, "peer"], 4, tmp_path)
    assert "ROWPAIR-FUSED ok world=4 N=328" in log, log[-2000:]


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("masked", [0, 1])
def test_outer_product_mean_over_sequence_shards_reduce_scatter(tmp_path, masked):
    log = _run("tests/multigpu/opm_seqshard_check.py", [256, 96, masked], 2, tmp_path)
    assert f"OPM-SEQSHARD ok world=2 N=256 S=96 masked={masked}" in log, log[-2000:]


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
def test_tensor_parallel_gemm_reduce_scatter_matches_nccl(tmp_path):
    log = _run("tests/multigpu/tp_gemm_check.py", [], 2, tmp_path)
    m = re.search(r"TP_GEMM_RS world=2 .* err_fused=([0-9.e+-]+) err_nccl=([0-9.e+-]+)", log)
    assert m, log[-2000:]
    assert float(m.group(1)) <= float(m.group(2)) * 1.5 + 1e-3


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
def test_big_mode_worker_returns_a_structure(tmp_path):
    """``pred --mode big --n_gpu 2`` end of the pipeline: sharded trunk, shards sent to rank 0, sampler and
    confidence head there."""
    from uplifting_biomolecular_modeling_b200.parallel import launch
    out = tmp_path / "o"
    launch.run_rank_processes(2, [sys.executable, "-m", "uplifting_biomolecular_modeling_b200.parallel.worker",
                                  "--config", "tiny", "--tokens", "256", "--msa_depth", "4", "--recycles", "0",
                                  "--structure", "1", "--out_dir", str(out)],
                              cpu=False, run_timeout_s=600, log_dir=str(tmp_path / "logs"),
                              extra_env={"PYTHONPATH": ROOT, "NCCL_NVLS_ENABLE": "0"}, echo_rank0=False)
    pred = torch.load(out / "prediction.pt")
    assert pred["coords"].dim() == 3 and torch.isfinite(pred["coords"]).all() and "plddt" in pred


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
def test_layer_pipeline_over_two_gpus_matches_one():
    """The layer split of the deep sequence models on two GPUs of one process: blocks placed by cost, two micro-batches
    in flight on per-device streams, activations crossing by asynchronous peer copies ordered by events."""
    from uplifting_biomolecular_modeling_b200.parallel import pipeline
    torch.manual_seed(0)
    blocks = [torch.nn.Sequential(torch.nn.Linear(256, 256), torch.nn.GELU()).eval() for _ in range(7)]
    x = torch.randn(6, 128, 256)
    with torch.no_grad():
        ref = x.cuda(0)
        for b in blocks:
            ref = b.cuda(0)(ref)
        ref = ref.cpu()
    pp = pipeline.LayerPipeline(blocks, ["cuda:0", "cuda:1"], weights=[1, 1, 1, 3, 1, 1, 1])
    assert [len(r) for r in pp.ranges] == [4, 3] or sum(len(r) for r in pp.ranges) == 7
    for window in (1, 2, 3):
        out = pp.forward(x.cuda(0), window=window)
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)
        assert out.device.index == 1
        assert torch.allclose(out.cpu(), ref, atol=1e-5, rtol=1e-5), window


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
def test_token_transformer_on_row_shards_over_nccl(tmp_path):
    """The sampler's token transformer with the token rows split over two GPUs (one all-gather of the normalised rows
    per layer) against the dense transformer."""
    log = _run("tests/multigpu/dit_rows_check.py", [200, 3], 2, tmp_path)
    assert "DIT-ROWS ok world=2 N=200 depth=3" in log, log[-2000:]


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
def test_evo2_tensor_parallel_prefill_and_folded_decode(tmp_path):
    """StripedHyena-2 over two GPUs against one: prefill logits and decode steps through the folded decode block."""
    log = _run("tests/multigpu/evo2_tp_check.py", [192, 4], 2, tmp_path)
    assert "EVO2-TP ok world=2 tokens=192 steps=4" in log, log[-2000:]


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
def test_evo2_kit_command_line_over_two_gpus(tmp_path):
    """``run.sh generate --mode fast --n_gpu 2``: two ranks of the tensor-parallel worker behind the kit's surface."""
    import json
    import subprocess
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    prompt = "ACGTACGTACGTACGTACGTACGTACGTACGTACGT"
    r = subprocess.run(["bash", "kits/evo2/run.sh", "generate", "--mode", "fast", "--n_gpu", "2", "--model_config",
                        "evo2_tiny", "--prompt", prompt, "--max_new_tokens", "8", "--out_dir", str(tmp_path / "o")],
                       capture_output=True, text=True, cwd=ROOT, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    assert "sharding=tensor_parallel" in r.stderr and " DONE " in r.stderr
    res = json.load(open(tmp_path / "o" / "generate.json"))
    assert res["world"] == 2 and res["new_tokens"] == 8 and res["reduce_calls"] > 0
    one = subprocess.run(["bash", "kits/evo2/run.sh", "generate", "--mode", "exact", "--model_config", "evo2_tiny",
                          "--prompt", prompt, "--max_new_tokens", "8"], capture_output=True, text=True, cwd=ROOT,
                         env=env, timeout=600)
    assert one.returncode == 0, one.stderr[-2000:]
    assert f"text={res['text']}" in one.stderr, (res["text"], one.stderr[-800:])
