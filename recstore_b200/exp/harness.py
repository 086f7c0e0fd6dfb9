"""Runs a command over the cartesian product of its options and keeps one directory per run.

    python -m recstore_b200.exp.harness --spec spec.json

``spec.json``: ``{"name": "emb_sweep", "command": "python -m recstore_b200.cli.perf_emb", "log_root": "runs",
"timeout_s": 3600, "grid": {"num_workers": [2, 4], "cache_ratio": [0.05, 0.1], "backwardMode": ["CppSync",
"CppAsyncV2"]}, "fixed": {"run_steps": 200}, "exclude": [{"num_workers": 4, "backwardMode": "CppSync"}]}``.

What it keeps from the reference's harness (src/kg/scripts/exp_config.py, bench_base.py, bench_util.py): the grid
expansion, a log directory per run named after its options, the rule that a run counts as finished only if its log
contains the completion marker ``Successfully xmh`` (exp_config.py:119-139; anything else after the time limit is
reported as a suspected deadlock), skipping of finished runs on restart, and an exclusive lock so that two sweeps
do not share the GPUs of one box (the reference used memcached / file locks).
"""
from __future__ import annotations

import argparse
import contextlib
import fcntl
import itertools
import json
import os
import shlex
import subprocess
import sys
import time
from dataclasses import asdict, dataclass
from typing import Callable, Dict, Iterator, List, Optional, Sequence

MARKER = "Successfully xmh"


def expand_grid(grid: Dict[str, Sequence], fixed: Optional[dict] = None, exclude: Optional[Sequence[dict]] = None,
                keep: Optional[Callable[[dict], bool]] = None) -> List[dict]:
    """Cartesian product of ``grid`` (insertion order, last key fastest) merged over ``fixed``; drops every
    configuration that contains all key/value pairs of an ``exclude`` entry or fails ``keep``."""
    keys = list(grid)
    out = []
    for vals in itertools.product(*(grid[k] for k in keys)):
        cfg = dict(fixed or {})
        cfg.update(zip(keys, vals))
        if any(all(cfg.get(k) == v for k, v in ex.items()) for ex in (exclude or [])):
            continue
        if keep is not None and not keep(cfg):
            continue
        out.append(cfg)
    return out


def run_dir_name(index: int, cfg: dict, varying: Sequence[str]) -> str:
    parts = [f"{k}={cfg[k]}" for k in varying]
    name = "run" + ("_" + "_".join(parts) if parts else f"_{index:03d}")   # named by its options: stable across re-runs
    return "".join(c if c.isalnum() or c in "=_.-" else "-" for c in name)[:200]


def log_succeeded(path: str, marker: str = MARKER) -> bool:
    try:
        with open(path, errors="replace") as f:
            return marker in f.read()
    except OSError:
        return False


def clean_unsuccessful(root: str, marker: str = MARKER, dry: bool = False) -> List[str]:
    """Removes the run directories under ``root`` whose log lacks the success marker, so that the next sweep runs them
    again from a clean directory (the reference's clean_unsuccess_log.py); returns the directories concerned.  Only
    directories that look like runs of this harness (a ``config.json`` beside the log) are touched."""
    import shutil
    gone = []
    for name in sorted(os.listdir(root)) if os.path.isdir(root) else []:
        d = os.path.join(root, name)
        if not (os.path.isdir(d) and os.path.exists(os.path.join(d, "config.json"))):
            continue
        if log_succeeded(os.path.join(d, "log"), marker):
            continue
        gone.append(d)
        if not dry:
            shutil.rmtree(d)
    return gone


@contextlib.contextmanager
def box_lock(path: str, timeout_s: float = 0.0, poll_s: float = 1.0) -> Iterator[None]:
    """Exclusive advisory lock on ``path``; waits up to ``timeout_s`` (0 = fail at once if it is taken)."""
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    f = open(path, "a+")
    t0 = time.time()
    while True:
        try:
            fcntl.flock(f, fcntl.LOCK_EX | fcntl.LOCK_NB)
            break
        except BlockingIOError:
            if time.time() - t0 >= timeout_s:
                f.close()
                raise TimeoutError(f"{path} is held by another sweep")
            time.sleep(poll_s)
    try:
        f.seek(0); f.truncate(); f.write(f"{os.getpid()}\n"); f.flush()
        yield
    finally:
        fcntl.flock(f, fcntl.LOCK_UN)
        f.close()


@dataclass
class RunResult:
    index: int
    config: dict
    directory: str
    status: str            # "ok", "failed", "deadlock?", "skipped"
    seconds: float
    returncode: Optional[int]


class Experiment:
    def __init__(self, name: str, command: str, grid: Dict[str, Sequence], fixed: Optional[dict] = None,
                 exclude: Optional[Sequence[dict]] = None, log_root: str = "runs", timeout_s: float = 3600.0,
                 marker: str = MARKER, env: Optional[dict] = None):
        self.name, self.command, self.grid, self.fixed = name, command, grid, dict(fixed or {})
        self.configs = expand_grid(grid, fixed, exclude)
        self.root = os.path.join(log_root, name)
        self.timeout_s, self.marker, self.env = timeout_s, marker, env

    def argv(self, cfg: dict) -> List[str]:
        args = shlex.split(self.command)
        for k, v in cfg.items():
            if isinstance(v, bool):
                if v:
                    args.append(f"--{k}")
            else:
                args += [f"--{k}", str(v)]
        return args

    def run(self, rerun: bool = False, dry: bool = False) -> List[RunResult]:
        os.makedirs(self.root, exist_ok=True)
        results = []
        varying = list(self.grid)             # every grid key names the directory, so a narrower re-run finds its runs
        for i, cfg in enumerate(self.configs):
            d = os.path.join(self.root, run_dir_name(i, cfg, varying))
            log = os.path.join(d, "log")
            if not rerun and log_succeeded(log, self.marker):
                results.append(RunResult(i, cfg, d, "skipped", 0.0, 0))
                continue
            os.makedirs(d, exist_ok=True)
            with open(os.path.join(d, "config.json"), "w") as f:
                json.dump({"command": self.argv(cfg), "config": cfg}, f, indent=1)
            if dry:
                results.append(RunResult(i, cfg, d, "dry", 0.0, None))
                continue
            t0 = time.time()
            env = dict(os.environ)
            env.update(self.env or {})
            with open(log, "w") as lf:
                p = subprocess.Popen(self.argv(cfg), stdout=lf, stderr=subprocess.STDOUT, env=env, start_new_session=True)
                try:
                    rc = p.wait(timeout=self.timeout_s)
                    timed_out = False
                except subprocess.TimeoutExpired:
                    timed_out = True
                    os.killpg(p.pid, 15)            # the run's own process group, nobody else's
                    try:
                        rc = p.wait(timeout=10)
                    except subprocess.TimeoutExpired:
                        os.killpg(p.pid, 9)
                        rc = p.wait()
            ok = log_succeeded(log, self.marker)
            status = "ok" if ok else ("deadlock?" if timed_out else "failed")
            results.append(RunResult(i, cfg, d, status, time.time() - t0, rc))
        with open(os.path.join(self.root, "summary.json"), "w") as f:
            json.dump([asdict(r) for r in results], f, indent=1)
        return results


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--spec", required=True, help="JSON file: name, command, grid, fixed, exclude, log_root, timeout_s")
    ap.add_argument("--rerun", action="store_true", help="run configurations again even if their log has the marker")
    ap.add_argument("--dry", action="store_true", help="only create the run directories and print the commands")
    ap.add_argument("--clean", action="store_true", help="remove the run directories without the success marker, then exit")
    ap.add_argument("--lock", default=None, help="lock file shared by every sweep on this box")
    ap.add_argument("--lock-timeout", type=float, default=0.0)
    a = ap.parse_args(argv)
    with open(a.spec) as f:
        spec = json.load(f)
    exp = Experiment(spec["name"], spec["command"], spec.get("grid", {}), spec.get("fixed"), spec.get("exclude"),
                     spec.get("log_root", "runs"), spec.get("timeout_s", 3600.0), spec.get("marker", MARKER), spec.get("env"))
    if a.clean:
        for d in clean_unsuccessful(exp.root, exp.marker, dry=a.dry):
            print(("would remove " if a.dry else "removed ") + d)
        sys.exit(0)
    ctx = box_lock(a.lock, a.lock_timeout) if a.lock else contextlib.nullcontext()
    with ctx:
        res = exp.run(rerun=a.rerun, dry=a.dry)
    for r in res:
        print(f"{r.status:10s} {r.seconds:8.1f}s  {r.directory}")
    bad = [r for r in res if r.status in ("failed", "deadlock?")]
    sys.exit(1 if bad else 0)


if __name__ == "__main__":
    main()
