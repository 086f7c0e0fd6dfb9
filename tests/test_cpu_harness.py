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


def test_clean_unsuccessful_removes_only_failed_runs(tmp_path):
    import json
    from recstore_b200.exp import harness as H
    for name, text, cfg in (("run_a=1", "all good\n" + H.MARKER + "\n", True), ("run_a=2", "crashed\n", True), ("notes", "x", False)):
        d = tmp_path / name
        d.mkdir()
        (d / "log").write_text(text)
        if cfg:
            (d / "config.json").write_text(json.dumps({}))
    assert [p.split("/")[-1] for p in H.clean_unsuccessful(str(tmp_path), dry=True)] == ["run_a=2"] and (tmp_path / "run_a=2").exists()
    assert len(H.clean_unsuccessful(str(tmp_path))) == 1
    assert (tmp_path / "run_a=1").exists() and not (tmp_path / "run_a=2").exists() and (tmp_path / "notes").exists()


def test_determinism_recorder_and_driver_flag(tmp_path):
    """First run records, an identical run passes, a run with another seed is caught."""
    import pytest
    import torch
    from recstore_b200.utils.determinism import DeterminismError, RunRecorder
    rec = RunRecorder(str(tmp_path / "d"))
    rec.diff_objs(torch.arange(5), "x"); rec.diff_objs({"a": 1}, "cfg")
    rec2 = RunRecorder(str(tmp_path / "d"))
    rec2.diff_objs(torch.arange(5), "x"); rec2.diff_objs({"a": 1}, "cfg")
    assert rec.recorded == 2 and rec2.compared == 2
    with pytest.raises(DeterminismError):
        rec2.diff_objs(torch.arange(5) + 1, "x")
    RunRecorder(None).diff_objs(torch.zeros(1), "ignored")
    from recstore_b200.cli import kge_main
    base = ["--max_step", "6", "--n_entities", "200", "--n_triples", "2000", "--hidden_dim", "8", "--batch_size", "32",
            "--neg_sample_size", "8", "--log_interval", "1000", "--determinism_dir", str(tmp_path / "kg")]
    kge_main.main(base)
    kge_main.main(base)
    with pytest.raises(DeterminismError):
        kge_main.main(base + ["--seed", "7"])
