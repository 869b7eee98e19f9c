"""Kit command lines on a B200: the modes whose levers need the GPU (the CPU suite can only see them refused)."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args):
    return subprocess.run(["bash"] + args, capture_output=True, text=True, cwd=ROOT, timeout=300)


def _done(r):
    lines = [l for l in r.stderr.splitlines() if " DONE " in l]
    assert lines, r.stderr[-2000:]
    return dict(kv.split("=", 1) for kv in lines[0].split()[2:] if "=" in kv)


def test_evo2_kit_modes_engage_their_levers_and_agree():
    prompt = "ACGTACGTACGTACGTACGTACGTACGTACGTACGT"
    base = ["kits/evo2/run.sh", "score", "--model_config", "evo2_tiny", "--prompt", prompt]
    off, exact, fast = (_run(base + ["--mode", m]) for m in ("off", "exact", "fast"))
    for r in (off, exact, fast):
        assert r.returncode == 0, r.stderr[-2000:]
    assert "LEVER name=kernel_path state=on" in exact.stderr and "LEVER name=forward_graph state=on" in exact.stderr
    assert "LEVER name=fp8_input_proj state=on" in fast.stderr
    assert "LEVER name=tp_fused state=" in fast.stderr            # on with several GPUs, skipped (declared) with one
    s_off, s_exact, s_fast = (float(_done(r)["score"]) for r in (off, exact, fast))
    assert abs(s_exact - s_off) <= 2e-2 * abs(s_off) and abs(s_fast - s_off) <= 5e-2 * abs(s_off)
    gen = [_run(["kits/evo2/run.sh", "generate", "--model_config", "evo2_tiny", "--prompt", prompt,
                 "--max_new_tokens", "8", "--mode", m]) for m in ("exact", "fast")]
    for r in gen:
        assert r.returncode == 0 and _done(r)["new_tokens"] == "8", r.stderr[-2000:]


def test_boltz2_kit_big_mode_on_one_gpu_reports_its_memory_levers(tmp_path):
    r = _run(["kits/boltz2/run.sh", "pred", "--mode", "big", "--tokens", "128", "--msa_depth", "8", "--model_config",
              "tiny", "--out_dir", str(tmp_path / "o")])
    assert r.returncode == 0, r.stderr[-2000:]
    assert "LEVER name=chunk_pair_ops state=on" in r.stderr and "LEVER name=release_intermediates state=on" in r.stderr
    assert os.path.isfile(tmp_path / "o" / "prediction.pt") and os.path.isfile(tmp_path / "o" / "peak_mem.json")
