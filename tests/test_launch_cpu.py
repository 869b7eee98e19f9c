"""Launcher: rank processes on CPU (gloo), fail-fast teardown, RankFailed with the log tail."""
import os
import sys
import textwrap
import time

import pytest

from uplifting_biomolecular_modeling_b200.parallel import launch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _script(tmp_path, body):
    p = tmp_path / "w.py"
    p.write_text("import os, sys, time\nsys.path.insert(0, %r)\n" % ROOT + textwrap.dedent(body))
    return [sys.executable, str(p)]


def test_ranks_run_and_gather_over_gloo(tmp_path):
    argv = _script(tmp_path, """
        import torch
        from uplifting_biomolecular_modeling_b200.parallel import launch
        comm = launch.init_from_env(timeout_s=60)
        t = torch.full((comm.rank + 1, 2), float(comm.rank))
        full = comm.all_gather_rows(t)
        assert full.shape[0] == sum(range(1, comm.world + 1)), full.shape
        parts = [torch.full((1,), float(comm.rank * 10 + q)) for q in range(comm.world)]
        got = comm.all_to_all(parts)
        assert [int(x.item()) for x in got] == [q * 10 + comm.rank for q in range(comm.world)]
        assert comm.all_reduce_scalar(comm.rank, "max") == comm.world - 1
        comm.host_signal(f"done{comm.rank}")
        comm.host_wait("done0", 30)
        print("RANK-OK", comm.rank)
    """)
    assert launch.run_rank_processes(3, argv, cpu=True, run_timeout_s=120, log_dir=str(tmp_path),
                                     echo_rank0=False) == [0, 0, 0]
    assert "RANK-OK 2" in (tmp_path / "rank2.log").read_text()


def test_failing_rank_tears_the_others_down(tmp_path):
    argv = _script(tmp_path, """
        r = int(os.environ["ROWPAIR_RANK"])
        if r == 1:
            print("about to fail")
            raise SystemExit(7)
        time.sleep(60)
    """)
    t0 = time.time()
    with pytest.raises(launch.RankFailed) as ei:
        launch.run_rank_processes(3, argv, cpu=True, run_timeout_s=50, kill_grace_s=2, log_dir=str(tmp_path),
                                  echo_rank0=False)
    assert ei.value.rank == 1 and ei.value.rc == 7 and "about to fail" in ei.value.tail
    assert time.time() - t0 < 30


def test_stuck_run_times_out(tmp_path):
    argv = _script(tmp_path, "time.sleep(60)\n")
    with pytest.raises(launch.RankFailed) as ei:
        launch.run_rank_processes(2, argv, cpu=True, run_timeout_s=2, kill_grace_s=1, log_dir=str(tmp_path),
                                  echo_rank0=False)
    assert ei.value.rc == 124
