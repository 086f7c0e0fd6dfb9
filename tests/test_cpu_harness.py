"""Experiment harness: grid expansion, completion marker, resume, time limit, box lock."""
import json
import os
import sys

import pytest

from recstore_b200.exp import Experiment, box_lock, expand_grid, log_succeeded


def test_expand_grid_order_fixed_and_exclude():
    g = expand_grid({"a": [1, 2], "b": ["x", "y"]}, fixed={"c": 0}, exclude=[{"a": 2, "b": "x"}])
    assert g == [{"c": 0, "a": 1, "b": "x"}, {"c": 0, "a": 1, "b": "y"}, {"c": 0, "a": 2, "b": "y"}]
    assert expand_grid({}, fixed={"z": 1}) == [{"z": 1}]
    assert len(expand_grid({"a": [1, 2, 3]}, keep=lambda c: c["a"] != 2)) == 2


def test_runs_marker_resume_and_timeout(tmp_path):
    script = tmp_path / "job.py"
    script.write_text(
        "import sys, time\n"
        "a = dict(zip(sys.argv[1::2], sys.argv[2::2]))\n"
        "mode = a['--mode']\n"
        "print('mode', mode, flush=True)\n"
        "if mode == 'hang': time.sleep(60)\n"
        "if mode == 'crash': sys.exit(3)\n"
        "print('Successfully xmh')\n")
    exp = Experiment("t", f"{sys.executable} {script}", {"mode": ["good", "crash", "hang"]}, fixed={"n": 1},
                     log_root=str(tmp_path / "runs"), timeout_s=1.5)
    res = exp.run()
    assert [r.status for r in res] == ["ok", "failed", "deadlock?"]
    assert res[1].returncode == 3 and res[2].seconds < 20
    assert log_succeeded(os.path.join(res[0].directory, "log"))
    cfg = json.load(open(os.path.join(res[0].directory, "config.json")))
    assert cfg["config"] == {"n": 1, "mode": "good"} and "mode=good" in res[0].directory
    exp2 = Experiment("t", f"{sys.executable} {script}", {"mode": ["good"]}, fixed={"n": 1}, log_root=str(tmp_path / "runs"))
    assert [r.status for r in exp2.run()] == ["skipped"]          # finished runs are not repeated
    assert os.path.exists(tmp_path / "runs" / "t" / "summary.json")


def test_box_lock_is_exclusive(tmp_path):
    p = str(tmp_path / "box.lock")
    with box_lock(p):
        with pytest.raises(TimeoutError):
            with box_lock(p, timeout_s=0.0):
                pass
    with box_lock(p):
        pass
