"""Trunk-level checkpoint / resume of a row-sharded run.

Each rank writes its own z shard plus a digest of the features it ran on; rank 0 also writes the
replicated tensors (s, recycling state), the RNG state and the numerics signature; the manifest is
written last (atomically), with a sha256 per file.  Resume is refused by name when the features, the
numerics signature, the dtype, the layout or a file digest differ.  Environment: ``ROWPAIR_CKPT_DIR``,
``ROWPAIR_CKPT_EVERY`` (blocks), ``ROWPAIR_CKPT_KEEP``, ``ROWPAIR_RESUME``.
Reference: common/opt_core/opt_core/mem/rowpair/ckpt.py:242-292,422.
"""
from __future__ import annotations

import hashlib
import json
import os
import tempfile
from typing import Dict, Mapping, Optional, Tuple

import torch

from ..core.gates import sha256_file


class ResumeRefused(RuntimeError):
    pass


def feature_digest(feats: Mapping[str, torch.Tensor]) -> str:
    h = hashlib.sha256()
    for k in sorted(feats):
        v = feats[k]
        if not isinstance(v, torch.Tensor):
            continue
        h.update(k.encode())
        h.update(str(tuple(v.shape)).encode())
        h.update(v.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()
                 if v.numel() < (1 << 22) else str(float(v.double().sum())).encode())
    return h.hexdigest()


def _atomic_save(obj, path: str) -> None:
    d = os.path.dirname(path)
    fd, tmp = tempfile.mkstemp(prefix=".ckpt.", dir=d)
    os.close(fd)
    torch.save(obj, tmp)
    os.replace(tmp, path)


class TrunkCheckpointer:
    def __init__(self, directory: str, rank: int, world: int, signature: str, keep: int = 2):
        self.dir, self.rank, self.world, self.signature, self.keep = directory, rank, world, signature, keep
        os.makedirs(directory, exist_ok=True)

    @classmethod
    def from_env(cls, rank: int, world: int, signature: str, environ=None) -> Optional["TrunkCheckpointer"]:
        env = os.environ if environ is None else environ
        d = env.get("ROWPAIR_CKPT_DIR")
        if not d:
            return None
        return cls(d, rank, world, signature, int(env.get("ROWPAIR_CKPT_KEEP", "2")))

    def _step_dir(self, step: int) -> str:
        return os.path.join(self.dir, f"step{step:06d}")

    def save(self, step: int, z_loc: torch.Tensor, rows: Tuple[int, int], feats_digest: str,
             replicated: Optional[Dict[str, torch.Tensor]] = None, barrier=None) -> str:
        sd = self._step_dir(step)
        os.makedirs(sd, exist_ok=True)
        name = f"z_rank{self.rank}.pt"
        _atomic_save({"z": z_loc.detach().cpu(), "rows": tuple(rows), "features": feats_digest,
                      "dtype": str(z_loc.dtype)}, os.path.join(sd, name))
        # every rank hashes its own shard (rank 0 hashing all of them would leave the others seconds ahead, into
        # device-side waits on a rank that is still on the host)
        with open(os.path.join(sd, name + ".sha256"), "w") as f:
            f.write(sha256_file(os.path.join(sd, name)))
        if self.rank == 0:
            import random
            rng = {"cpu": torch.get_rng_state(), "python": random.getstate()}
            if torch.cuda.is_available():
                rng["cuda"] = torch.cuda.get_rng_state_all()
            _atomic_save({"replicated": {k: v.detach().cpu() for k, v in (replicated or {}).items()},
                          "rng": rng, "signature": self.signature}, os.path.join(sd, "replicated.pt"))
        if barrier is not None:
            barrier()
        if self.rank == 0:
            files = {}
            for f in sorted(x for x in os.listdir(sd) if x.endswith(".pt")):
                side = os.path.join(sd, f + ".sha256")
                files[f] = open(side).read().strip() if os.path.exists(side) else sha256_file(os.path.join(sd, f))
            man = {"step": step, "world": self.world, "signature": self.signature, "features": feats_digest,
                   "files": files}
            fd, tmp = tempfile.mkstemp(prefix=".manifest.", dir=sd)
            with os.fdopen(fd, "w") as f:
                json.dump(man, f, indent=1, sort_keys=True)
            os.replace(tmp, os.path.join(sd, "manifest.json"))
            self._prune()
        if barrier is not None:
            barrier()          # nobody goes back to the device before the manifest exists and old steps are pruned
        return sd

    def _prune(self) -> None:
        steps = sorted(d for d in os.listdir(self.dir) if d.startswith("step")
                       and os.path.exists(os.path.join(self.dir, d, "manifest.json")))
        for old in steps[:-self.keep] if self.keep > 0 else []:
            p = os.path.join(self.dir, old)
            for f in os.listdir(p):
                os.unlink(os.path.join(p, f))
            os.rmdir(p)

    def latest(self) -> Optional[int]:
        steps = sorted(int(d[4:]) for d in os.listdir(self.dir) if d.startswith("step")
                       and os.path.exists(os.path.join(self.dir, d, "manifest.json")))
        return steps[-1] if steps else None

    def load(self, step: int, feats_digest: str, rows: Tuple[int, int], dtype: torch.dtype, device="cpu"):
        sd = self._step_dir(step)
        try:
            man = json.load(open(os.path.join(sd, "manifest.json")))
        except (OSError, ValueError) as e:
            raise ResumeRefused(f"resume refused: manifest unreadable ({e})") from e
        if man["world"] != self.world:
            raise ResumeRefused(f"resume refused: world {man['world']} != {self.world}")
        if man["signature"] != self.signature:
            raise ResumeRefused("resume refused: numerics signature differs")
        if man["features"] != feats_digest:
            raise ResumeRefused("resume refused: features differ")
        name = f"z_rank{self.rank}.pt"
        for f in (name, "replicated.pt"):
            if man["files"].get(f) != sha256_file(os.path.join(sd, f)):
                raise ResumeRefused(f"resume refused: digest of {f} differs")
        mine = torch.load(os.path.join(sd, name), map_location="cpu")
        if tuple(mine["rows"]) != tuple(rows):
            raise ResumeRefused(f"resume refused: layout differs ({mine['rows']} != {tuple(rows)})")
        if mine["dtype"] != str(dtype):
            raise ResumeRefused(f"resume refused: dtype {mine['dtype']} != {dtype}")
        rep = torch.load(os.path.join(sd, "replicated.pt"), map_location="cpu")
        return mine["z"].to(device), {k: v.to(device) for k, v in rep["replicated"].items()}, rep["rng"]

    @staticmethod
    def restore_rng(rng) -> None:
        """Put the python / CPU / CUDA random states of a checkpoint back (older checkpoints hold the CPU state only)."""
        if isinstance(rng, torch.Tensor):
            torch.set_rng_state(rng)
            return
        import random
        torch.set_rng_state(rng["cpu"])
        if "python" in rng:
            random.setstate(rng["python"])
        if "cuda" in rng and torch.cuda.is_available() and len(rng["cuda"]) == torch.cuda.device_count():
            torch.cuda.set_rng_state_all(rng["cuda"])
