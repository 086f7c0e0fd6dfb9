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


def test_bindings_vary_options_together():
    """Sub-grids of a binding group are expanded one by one and concatenated, groups are multiplied with each other and
    with the grid (GenBinding / PreprocessConfig of src/kg/scripts/bench_util.py)."""
    from recstore_b200.exp.harness import expand_bindings
    groups = [[{"model": ["TransE_l2"], "gamma": [12.0]}, {"model": ["DistMult"], "gamma": [100.0, 140.0]}],
              [{"bs": [256], "lr": [0.1]}, {"bs": [1024], "lr": [0.4]}]]
    b = expand_bindings(groups)
    assert len(b) == 3 * 2 and b[0] == {"model": "TransE_l2", "gamma": 12.0, "bs": 256, "lr": 0.1}
    assert {"model": "DistMult", "gamma": 140.0, "bs": 1024, "lr": 0.4} in b
    assert not any(c["model"] == "TransE_l2" and c["gamma"] != 12.0 for c in b)
    g = expand_grid({"gpus": [1, 2]}, fixed={"steps": 5}, bindings=groups, exclude=[{"gpus": 2, "bs": 256}])
    assert len(g) == 2 * 6 - 3 and all(c["steps"] == 5 for c in g)
    assert expand_bindings(None) == [{}] and expand_grid({"a": [1]}, bindings=[]) == [{"a": 1}]
    with pytest.raises(ValueError):
        expand_grid({"bs": [1]}, bindings=groups)                       # an option cannot be in both
    with pytest.raises(ValueError):
        expand_bindings([[{"x": [1]}], [{"x": [2]}]])                   # nor in two groups


def test_client_server_runs_hooks_and_server_failure(tmp_path):
    """Servers come up first (ready marker), the client talks to them, they are stopped after the run; hooks run around
    it; a server that never gets ready fails the run without starting the client (bench_base.py CSExperiment)."""
    server = tmp_path / "server.py"
    server.write_text(
        "import socket, sys, time\n"
        "port, mode = int(sys.argv[1]), sys.argv[2]\n"
        "if mode == 'broken': sys.exit(5)\n"
        "s = socket.socket(); s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)\n"
        "s.bind(('127.0.0.1', port)); s.listen(4)\n"
        "print('listening', port, flush=True)\n"
        "while True:\n"
        "    c, _ = s.accept(); c.sendall(b'pong'); c.close()\n")
    client = tmp_path / "client.py"
    client.write_text(
        "import socket, sys\n"
        "a = dict(zip(sys.argv[1::2], sys.argv[2::2]))\n"
        "c = socket.create_connection(('127.0.0.1', int(a['--port'])), timeout=10)\n"
        "assert c.recv(4) == b'pong'\n"
        "print('Successfully xmh')\n")
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    exp = Experiment("cs", f"{sys.executable} {client}", {"mode": ["fine", "broken"]}, fixed={"port": port},
                     log_root=str(tmp_path / "runs"), timeout_s=30,
                     servers=[{"command": f"{sys.executable} {server} {{port}} {{mode}}", "ready_marker": "listening", "ready_timeout_s": 20}],
                     pre_run="echo before {mode} > {run_dir}/pre.txt", post_run="echo after {mode} > {run_dir}/post.txt")
    res = exp.run()
    assert [r.status for r in res] == ["ok", "failed"]
    d0, d1 = res[0].directory, res[1].directory
    assert "listening" in open(os.path.join(d0, "server_0.log")).read()
    assert open(os.path.join(d0, "pre.txt")).read().strip() == "before fine" and open(os.path.join(d0, "post.txt")).read().strip() == "after fine"
    assert "did not print" in open(os.path.join(d1, "log")).read()
    with pytest.raises(OSError):                                       # the first run's server is gone: nobody listens any more
        socket.create_connection(("127.0.0.1", port), timeout=2)


def test_runs_on_hosts_go_through_ssh_and_need_every_marker(tmp_path, monkeypatch):
    """With `hosts` the command runs once per host through `ssh` (here a stand-in on PATH that runs it locally and can
    fail one host); the run counts only if every host printed the marker."""
    from recstore_b200.exp.harness import ssh_argv
    assert ssh_argv("box7", ["python", "-c", "print('a b')"], cwd="/w d")[-2:] == ["box7", "cd '/w d' && python -c 'print('\"'\"'a b'\"'\"')'"]
    fake = tmp_path / "bin"
    fake.mkdir()
    (fake / "ssh").write_text("#!/bin/sh\n# stand-in: drop the options, note the host, run the command here\n"
                              "while [ \"$1\" = \"-o\" ]; do shift 2; done\nhost=$1; shift\n"
                              "if [ \"$host\" = \"bad\" ]; then echo no route; exit 255; fi\necho on $host; exec sh -c \"$1\"\n")
    (fake / "ssh").chmod(0o755)
    monkeypatch.setenv("PATH", f"{fake}:{os.environ['PATH']}")
    job = tmp_path / "job.py"
    job.write_text("print('Successfully xmh')\n")
    ok = Experiment("h", f"{sys.executable} {job}", {"x": [1]}, log_root=str(tmp_path / "runs"), hosts=["n1", "n2"], timeout_s=30).run()
    assert [r.status for r in ok] == ["ok"]
    text = open(os.path.join(ok[0].directory, "log")).read()
    assert "===== n1 =====" in text and "on n2" in text and text.count("Successfully xmh") == 2
    bad = Experiment("h2", f"{sys.executable} {job}", {"x": [1]}, log_root=str(tmp_path / "runs"), hosts=["n1", "bad"], timeout_s=30).run()
    assert [r.status for r in bad] == ["failed"] and bad[0].returncode == 255
    assert "no route" in open(os.path.join(bad[0].directory, "log")).read()


def test_sweep_of_the_ps_client_benchmark_against_stand_alone_servers(tmp_path):
    """The pieces together, as the reference's PS experiments run them: for every configuration the harness starts a
    server process, waits for its ready line, runs the client benchmark against it and stops the server."""
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    py = sys.executable
    exp = Experiment("ps_sweep", f"{py} -m recstore_b200.bench.ps_client --host 127.0.0.1 --seconds 0.4 --key-space 5000 --batch 64",
                     {"threads": [1, 2]}, fixed={"port": port, "dim": 8}, log_root=str(tmp_path / "runs"), timeout_s=120,
                     marker='"keys_per_s"',
                     servers=[{"command": f"{py} -m recstore_b200.ps.server --port {{port}} --dim {{dim}} --capacity 20000 --load_fake 5000 --workers 2",
                               "ready_marker": "listening on", "ready_timeout_s": 60}],
                     env={"PYTHONPATH": os.path.dirname(os.path.dirname(os.path.abspath(__file__)))})
    res = exp.run()
    assert [r.status for r in res] == ["ok", "ok"], [open(os.path.join(r.directory, "log")).read()[-500:] for r in res]
    out = json.loads(open(os.path.join(res[1].directory, "log")).read().strip().splitlines()[-1])
    assert out["threads"] == 2 and out["keys_per_s"] > 1000
    assert "listening on" in open(os.path.join(res[0].directory, "server_0.log")).read()
