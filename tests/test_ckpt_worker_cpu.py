"""Trunk checkpoints, upstream-name weight loading and the sharded worker on CPU (gloo)."""
import os
import sys

import pytest
import torch

from uplifting_biomolecular_modeling_b200.models import cofold, weights
from uplifting_biomolecular_modeling_b200.parallel import ckpt, launch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_checkpoint_roundtrip_and_refusals(tmp_path):
    c = ckpt.TrunkCheckpointer(str(tmp_path), 0, 1, "sigA", keep=1)
    z = torch.randn(4, 8, 3)
    c.save(0, z, (0, 4), "feat1", {"s": torch.ones(2)})
    c.save(1, z * 2, (0, 4), "feat1", {"s": torch.ones(2) * 2})
    assert c.latest() == 1 and not os.path.exists(tmp_path / "step000000")
    z2, rep, _ = c.load(1, "feat1", (0, 4), torch.float32)
    assert torch.equal(z2, z * 2) and torch.equal(rep["s"], torch.ones(2) * 2)
    with pytest.raises(ckpt.ResumeRefused, match="features differ"):
        c.load(1, "other", (0, 4), torch.float32)
    with pytest.raises(ckpt.ResumeRefused, match="layout differs"):
        c.load(1, "feat1", (0, 3), torch.float32)
    with pytest.raises(ckpt.ResumeRefused, match="dtype"):
        c.load(1, "feat1", (0, 4), torch.bfloat16)
    with pytest.raises(ckpt.ResumeRefused, match="signature"):
        ckpt.TrunkCheckpointer(str(tmp_path), 0, 1, "sigB").load(1, "feat1", (0, 4), torch.float32)
    with open(tmp_path / "step000001" / "z_rank0.pt", "ab") as f:
        f.write(b"x")
    with pytest.raises(ckpt.ResumeRefused, match="digest"):
        c.load(1, "feat1", (0, 4), torch.float32)


def test_weights_load_by_upstream_names(tmp_path):
    m = cofold.build_model("tiny", seed=1)
    state = {"model." + k: v.clone() for k, v in m.state_dict().items()}
    p = tmp_path / "boltz_like.ckpt"
    torch.save({"state_dict": state, "hyper_parameters": {}}, p)
    m2 = cofold.build_model("tiny", seed=2)
    n, missing, unexpected = weights.load_checkpoint(m2, str(p))
    assert n == len(m.state_dict()) and not missing and not unexpected
    k = "pairformer_module.layers.0.tri_mul_out.p_in.weight"
    assert torch.equal(m2.state_dict()[k], m.state_dict()[k])
    torch.save({"state_dict": {"nothing": torch.zeros(1)}}, p)
    with pytest.raises(ValueError):
        weights.load_checkpoint(m2, str(p))


def test_sharded_worker_on_gloo_matches_single_rank(tmp_path):
    common = ["--config", "tiny", "--tokens", "24", "--msa_depth", "2", "--recycles", "0", "--structure", "1"]
    outs = []
    for world in (1, 2):
        out = tmp_path / f"w{world}"
        launch.run_rank_processes(world, [sys.executable, "-m",
                                          "uplifting_biomolecular_modeling_b200.parallel.worker", *common,
                                          "--out_dir", str(out)],
                                  cpu=True, run_timeout_s=300, log_dir=str(tmp_path / f"log{world}"),
                                  extra_env={"PYTHONPATH": ROOT, "CUDA_VISIBLE_DEVICES": ""}, echo_rank0=False)
        outs.append(torch.load(out / "trunk.pt"))
    assert torch.allclose(outs[0]["s"], outs[1]["s"], atol=1e-4, rtol=1e-4)
    assert abs(outs[0]["distogram_logits_mean"] - outs[1]["distogram_logits_mean"]) < 1e-4
    # the sharded run returns a structure: rank 0 received the row shards and ran sampler + confidence head
    preds = [torch.load(tmp_path / f"w{w}" / "prediction.pt") for w in (1, 2)]
    assert preds[1]["coords"].shape == preds[0]["coords"].shape and preds[1]["coords"].dim() == 3
    assert torch.isfinite(preds[1]["coords"]).all() and "plddt" in preds[1]
    assert torch.allclose(preds[0]["coords"], preds[1]["coords"], atol=5e-2, rtol=1e-2)
    assert "[rowpair] STRUCTURE rank=0" in (tmp_path / "log2" / "rank0.log").read_text()
    log = (tmp_path / "log2" / "rank1.log").read_text()
    assert "[rowpair] SCHEDULE rank=1" in log and "[rowpair] MEMSTATS rank=1" in log
