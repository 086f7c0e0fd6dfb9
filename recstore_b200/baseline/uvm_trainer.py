"""Unified-memory baseline: a plain PyTorch embedding trainer run under the cudaMalloc -> cudaMallocManaged interposer.

This is the "let the driver page it" alternative to an embedding store: the table is an ordinary ``nn.Embedding`` on
the GPU, every device allocation of the process is turned into managed memory by the ``LD_PRELOAD`` shim
(``csrc/preload/uvm_intercept.cpp``), so a table larger than HBM still trains, page-faulting its rows in.  Same role
and same model as the reference's libtorch program (src/executable/uvm/uvm_libtorch.cc:17-130: one embedding table,
``loss = sum(embedding(indices))``, SGD lr 0.001, optionally data-parallel over several GPUs).

    python -m recstore_b200.baseline.uvm_trainer --vocab_size 100000000 --embed_size 32 --batch_size 26624 --sample_number 100

The module re-executes itself with the shim preloaded (``--no_uvm`` runs it on ordinary device memory for
comparison) and prints one JSON line: ms / step, keys / s, and how many allocations the shim redirected.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import time


def parse_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("--nr_gpus", type=int, default=1, help="replicas of torch.nn.parallel.data_parallel (the reference uses 4)")
    p.add_argument("--batch_size", type=int, default=26 * 1024)
    p.add_argument("--vocab_size", type=int, default=10000)
    p.add_argument("--embed_size", type=int, default=32)
    p.add_argument("--sample_number", type=int, default=100, help="steps")
    p.add_argument("--zipf_alpha", type=float, default=0.0, help="0: uniform ids")
    p.add_argument("--lr", type=float, default=0.001)
    p.add_argument("--device", choices=["cuda", "cpu"], default=None, help="default: cuda if there is one")
    p.add_argument("--no_uvm", action="store_true", help="do not preload the interposer (ordinary device memory)")
    p.add_argument("--min_bytes", type=int, default=0, help="only allocations of at least this size become managed")
    return p.parse_args(argv)


def shim_path() -> str:
    from ..build import UVM_SHIM_PATH, build_preload_shims
    if not UVM_SHIM_PATH.exists():
        build_preload_shims()
    return str(UVM_SHIM_PATH)


def _shim_stats():
    """(calls, redirected, bytes) if the interposer is loaded in this process, else None."""
    try:
        lib = ctypes.CDLL(None)
        fn = lib.rs_uvm_intercept_stats
    except (OSError, AttributeError):
        return None
    out = (ctypes.c_ulonglong * 3)()
    fn(out)
    return int(out[0]), int(out[1]), int(out[2])


def train(args) -> dict:
    import torch
    from ..utils.data import zipf_ids
    import numpy as np
    dev = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    torch.manual_seed(0)
    model = torch.nn.Embedding(args.vocab_size, args.embed_size).to(dev)
    opt = torch.optim.SGD(model.parameters(), lr=args.lr)
    rng = np.random.default_rng(0)
    devices = list(range(args.nr_gpus)) if dev.type == "cuda" and args.nr_gpus > 1 else None
    losses, t0 = [], None
    for step in range(args.sample_number + 1):
        if step == 1:                                  # the first step pays for context and allocator set-up
            if dev.type == "cuda":
                torch.cuda.synchronize()
            t0 = time.time()
        ids = torch.from_numpy(zipf_ids(args.batch_size, args.vocab_size, args.zipf_alpha, rng)).to(dev)
        opt.zero_grad()
        out = torch.nn.parallel.data_parallel(model, ids, devices, dev) if devices else model(ids)
        loss = out.sum()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    if dev.type == "cuda":
        torch.cuda.synchronize()
    el = time.time() - (t0 or time.time())
    steps = max(1, args.sample_number)
    st = _shim_stats()
    return {"device": str(dev), "uvm": st is not None, "ms_per_step": el / steps * 1e3,
            "keys_per_s": args.batch_size * steps / max(el, 1e-9), "first_loss": losses[0], "last_loss": losses[-1],
            "intercepted": None if st is None else {"cudaMalloc_calls": st[0], "made_managed": st[1], "bytes": st[2]}}


def main(argv=None) -> dict:
    args = parse_args(argv)
    child = os.environ.get("RECSTORE_UVM_CHILD") == "1"
    if args.no_uvm or child:
        res = train(args)
        print(json.dumps(res), flush=True)
        return res
    env = dict(os.environ, RECSTORE_UVM_CHILD="1", RECSTORE_UVM_MIN_BYTES=str(args.min_bytes))
    pkg_parent = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    env["PYTHONPATH"] = pkg_parent + (os.pathsep + env["PYTHONPATH"] if env.get("PYTHONPATH") else "")
    env["LD_PRELOAD"] = shim_path() + (":" + env["LD_PRELOAD"] if env.get("LD_PRELOAD") else "")
    cmd = [sys.executable, "-m", "recstore_b200.baseline.uvm_trainer"] + (list(argv) if argv is not None else sys.argv[1:])
    p = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    sys.stdout.write(p.stdout)
    if p.returncode != 0:
        raise RuntimeError(f"the preloaded trainer exited with {p.returncode}")
    last = [ln for ln in p.stdout.splitlines() if ln.startswith("{")]
    return json.loads(last[-1]) if last else {}


if __name__ == "__main__":
    main()
