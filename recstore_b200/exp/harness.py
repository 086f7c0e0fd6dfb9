"""Runs a command over the cartesian product of its options and keeps one directory per run.

    python -m recstore_b200.exp.harness --spec spec.json

``spec.json``: ``{"name": "emb_sweep", "command": "python -m recstore_b200.cli.perf_emb", "log_root": "runs",
"timeout_s": 3600, "grid": {"num_workers": [2, 4], "cache_ratio": [0.05, 0.1], "backwardMode": ["CppSync",
"CppAsyncV2"]}, "fixed": {"run_steps": 200}, "exclude": [{"num_workers": 4, "backwardMode": "CppSync"}]}``.

Optional keys: ``"bindings"``: options that vary TOGETHER -- a list of groups, each group a list of sub-grids whose
expansions are concatenated, e.g. ``[[{"model": ["TransE_l2"], "gamma": [12.0]}, {"model": ["DistMult"], "gamma":
[100.0, 140.0]}]]`` gives three (model, gamma) pairs, multiplied with the grid (bench_util.py ``GenBinding`` /
``PreprocessConfig``); ``"servers"``: commands started before every run and stopped after it (client / server
experiments such as PS benchmarks: ``[{"command": "...", "ready_marker": "listening", "ready_timeout_s": 60}]``; their
options may use ``{key}`` placeholders of the run's configuration); ``"pre_run"`` / ``"post_run"``: shell commands
around every run; ``"hosts"``: run the command on these machines over ``ssh`` at once (one log per host) instead of
locally.

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


def expand_bindings(groups: Optional[Sequence[Sequence[Dict[str, Sequence]]]]) -> List[dict]:
    """Every combination of one entry per group, where a group's entries are the concatenated expansions of its
    sub-grids: options that only make sense together vary together instead of being multiplied out."""
    per_group = []
    for group in groups or []:
        entries: List[dict] = []
        for sub in group:
            keys = list(sub)
            entries += [dict(zip(keys, vals)) for vals in itertools.product(*(sub[k] for k in keys))]
        per_group.append(entries)
    out = []
    for combo in itertools.product(*per_group):
        merged: dict = {}
        for c in combo:
            clash = set(merged) & set(c)
            if clash:
                raise ValueError(f"option(s) {sorted(clash)} appear in two binding groups")
            merged.update(c)
        out.append(merged)
    return out


def expand_grid(grid: Dict[str, Sequence], fixed: Optional[dict] = None, exclude: Optional[Sequence[dict]] = None,
                keep: Optional[Callable[[dict], bool]] = None,
                bindings: Optional[Sequence[Sequence[Dict[str, Sequence]]]] = None) -> List[dict]:
    """Cartesian product of ``grid`` (insertion order, last key fastest), times the bound option sets of ``bindings``,
    merged over ``fixed``; drops every configuration that contains all key/value pairs of an ``exclude`` entry or
    fails ``keep``."""
    keys = list(grid)
    bound = expand_bindings(bindings)
    if any(set(b) & set(keys) for b in bound):
        raise ValueError("an option is both in the grid and in a binding")
    out = []
    for vals, b in itertools.product(itertools.product(*(grid[k] for k in keys)), bound):
        cfg = dict(fixed or {})
        cfg.update(zip(keys, vals))
        cfg.update(b)
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


def ssh_argv(host: str, command: Sequence[str], cwd: Optional[str] = None) -> List[str]:
    """The ``ssh`` command line that runs ``command`` on ``host`` (in ``cwd``), every word quoted for the remote shell."""
    remote = " ".join(shlex.quote(c) for c in command)
    if cwd:
        remote = f"cd {shlex.quote(cwd)} && {remote}"
    return ["ssh", "-o", "StrictHostKeyChecking=no", "-o", "BatchMode=yes", host, remote]


def _stop_group(p: subprocess.Popen, grace_s: float = 10.0) -> Optional[int]:
    """Ends the process group that ``p`` leads (only what this harness started)."""
    if p.poll() is None:
        try:
            os.killpg(p.pid, 15)
        except ProcessLookupError:
            pass
        try:
            return p.wait(timeout=grace_s)
        except subprocess.TimeoutExpired:
            try:
                os.killpg(p.pid, 9)
            except ProcessLookupError:
                pass
            return p.wait()
    return p.returncode


class Experiment:
    def __init__(self, name: str, command: str, grid: Dict[str, Sequence], fixed: Optional[dict] = None,
                 exclude: Optional[Sequence[dict]] = None, log_root: str = "runs", timeout_s: float = 3600.0,
                 marker: str = MARKER, env: Optional[dict] = None,
                 bindings: Optional[Sequence[Sequence[Dict[str, Sequence]]]] = None, servers: Optional[Sequence[dict]] = None,
                 pre_run: Optional[str] = None, post_run: Optional[str] = None, hosts: Optional[Sequence[str]] = None,
                 remote_cwd: Optional[str] = None):
        self.name, self.command, self.grid, self.fixed = name, command, grid, dict(fixed or {})
        self.configs = expand_grid(grid, fixed, exclude, bindings=bindings)
        self.varying = list(grid) + [k for k in (expand_bindings(bindings)[0] if bindings else {})]
        self.root = os.path.join(log_root, name)
        self.timeout_s, self.marker, self.env = timeout_s, marker, env
        self.servers, self.pre_run, self.post_run = list(servers or []), pre_run, post_run
        self.hosts, self.remote_cwd = list(hosts or []), remote_cwd

    # ---- client / server runs (bench_base.py CSExperiment: servers first, clients once they are up) ----
    def _start_servers(self, cfg: dict, d: str, env: dict) -> List[subprocess.Popen]:
        procs = []
        for i, spec in enumerate(self.servers):
            argv = [a.format(**cfg) for a in shlex.split(spec["command"])]
            log = os.path.join(d, f"server_{i}.log")
            lf = open(log, "w")
            p = subprocess.Popen(argv, stdout=lf, stderr=subprocess.STDOUT, env=env, start_new_session=True)
            lf.close()
            procs.append(p)
            marker, limit = spec.get("ready_marker"), float(spec.get("ready_timeout_s", 60.0))
            t0 = time.time()
            while marker:
                if log_succeeded(log, marker):
                    break
                if p.poll() is not None or time.time() - t0 > limit:
                    for q in procs:
                        _stop_group(q)
                    raise RuntimeError(f"server {i} ({argv[0]} ...) did not print {marker!r}: see {log}")
                time.sleep(0.05)
            if not marker:
                time.sleep(float(spec.get("settle_s", 0.5)))
        return procs

    def _hook(self, command: Optional[str], cfg: dict, d: str, env: dict, tag: str) -> None:
        if not command:
            return
        with open(os.path.join(d, f"{tag}.log"), "w") as lf:
            subprocess.run(command.format(run_dir=d, **cfg), shell=True, stdout=lf, stderr=subprocess.STDOUT, env=env,
                           timeout=self.timeout_s, check=False)

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
        varying = self.varying                # every grid / bound key names the directory, so a narrower re-run finds its runs
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
            self._hook(self.pre_run, cfg, d, env, "pre_run")
            try:
                servers = self._start_servers(cfg, d, env)
            except RuntimeError as e:
                with open(log, "w") as lf:
                    lf.write(f"{e}\n")
                results.append(RunResult(i, cfg, d, "failed", time.time() - t0, None))
                continue
            try:
                rc, timed_out = self._run_clients(cfg, d, log, env)
            finally:
                for sp in servers:
                    _stop_group(sp)
                self._hook(self.post_run, cfg, d, env, "post_run")
            ok = log_succeeded(log, self.marker)
            status = "ok" if ok else ("deadlock?" if timed_out else "failed")
            results.append(RunResult(i, cfg, d, status, time.time() - t0, rc))
        with open(os.path.join(self.root, "summary.json"), "w") as f:
            json.dump([asdict(r) for r in results], f, indent=1)
        return results

    def _run_clients(self, cfg: dict, d: str, log: str, env: dict):
        """The run's command, locally or on every host at once; (return code, timed out).  With hosts the per-host
        outputs go to ``log.<host>`` and are joined into ``log`` at the end, so the marker rule reads one file; the
        run succeeds only if every host printed the marker."""
        targets = [(None, self.argv(cfg), log)] if not self.hosts else \
            [(h, ssh_argv(h, self.argv(cfg), self.remote_cwd), f"{log}.{h}") for h in self.hosts]
        procs = []
        for _, argv, path in targets:
            lf = open(path, "w")
            procs.append(subprocess.Popen(argv, stdout=lf, stderr=subprocess.STDOUT, env=env, start_new_session=True))
            lf.close()
        deadline = time.time() + self.timeout_s
        rcs, timed_out = [], False
        for p in procs:
            try:
                rcs.append(p.wait(timeout=max(0.0, deadline - time.time())))
            except subprocess.TimeoutExpired:
                timed_out = True
                rcs.append(_stop_group(p))          # the run's own process group, nobody else's
        if self.hosts:
            all_ok = all(log_succeeded(path, self.marker) for _, _, path in targets)
            with open(log, "w") as out:
                for h, _, path in targets:
                    out.write(f"===== {h} =====\n")
                    with open(path, errors="replace") as f:
                        text = f.read()
                    out.write(text if all_ok else text.replace(self.marker, "(marker of one host)"))
        rc = next((r for r in rcs if r not in (0, None)), rcs[0] if rcs else None)
        return rc, timed_out


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
                     spec.get("log_root", "runs"), spec.get("timeout_s", 3600.0), spec.get("marker", MARKER), spec.get("env"),
                     bindings=spec.get("bindings"), servers=spec.get("servers"), pre_run=spec.get("pre_run"),
                     post_run=spec.get("post_run"), hosts=spec.get("hosts"), remote_cwd=spec.get("remote_cwd"))
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
