"""The benchmark prints its one JSON line exactly once, whatever the optional second measurement does: returns,
raises, or never comes back (the time-limit path leaves the process, so it runs in a child)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    sys.path.insert(0, ROOT)
    import importlib
    return importlib.import_module("bench")


def test_line_carries_the_second_metric_or_its_error(capsys):
    bench = _bench()
    assert bench.second_metric_then_line({"metric": "m"}, lambda: {"ms": 1.0}, 0, 5.0) == {"ms": 1.0}
    assert json.loads(capsys.readouterr().out) == {"metric": "m", "big_mode": {"ms": 1.0}}

    def boom():
        raise RuntimeError("peer gone")
    got = bench.second_metric_then_line({"metric": "m"}, boom, 0, 5.0)
    assert got["error"].startswith("RuntimeError: peer gone")
    assert json.loads(capsys.readouterr().out)["big_mode"] == got
    bench.second_metric_then_line({"metric": "m"}, None, 0, 0.0)
    assert json.loads(capsys.readouterr().out) == {"metric": "m", "big_mode": None}
    bench.second_metric_then_line({"metric": "m"}, lambda: 1, 3, 5.0)          # other ranks print nothing
    assert capsys.readouterr().out == ""


def test_a_measurement_that_never_returns_still_leaves_one_line():
    code = ("import sys, time; sys.path.insert(0, %r); import bench; "
            "bench.second_metric_then_line({'metric': 'm', 'value': 7}, lambda: time.sleep(60), 0, 0.5)") % ROOT
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["value"] == 7 and "abandoned" in line["big_mode"]["error"]
