"""Bandwidth probes of one box: PCIe / C2C copies, HBM copies, UVA reads of pinned host memory, NVLink peer traffic.

    python -m recstore_b200.bench.bandwidth --mb 256
    python -m recstore_b200.bench.bandwidth --p2p          # every ordered pair of visible GPUs

Native probes in ``csrc/tools/bandwidth.cu`` (CUDA-event timed, warm-up first); one JSON line per probe in GB/s.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

from .. import _lib
from .._lib import f64, i32, sz

_lib.register_signatures({
    "rs_probe_bandwidth": (i32, [i32, sz, i32, i32, C.POINTER(f64)]),
    "rs_probe_p2p": (i32, [i32, i32, sz, i32, i32, C.POINTER(f64), C.POINTER(i32)]),
})

KINDS = {"h2d": 0, "d2h": 1, "d2d": 2, "copy_kernel": 3, "uva_read": 4}


def probe(kind: str, nbytes: int, iters: int = 10, pinned: bool = True) -> float:
    g = f64()
    _lib.call("rs_probe_bandwidth", KINDS[kind], int(nbytes), iters, 1 if pinned else 0, C.byref(g))
    return g.value


def probe_p2p(src: int, dst: int, nbytes: int, iters: int = 10, kernel_read: bool = False):
    g, ok = f64(), i32()
    _lib.call("rs_probe_p2p", src, dst, int(nbytes), iters, 1 if kernel_read else 0, C.byref(g), C.byref(ok))
    return g.value, bool(ok.value)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--mb", type=int, default=256, help="buffer size in MiB (use more than the 126 MB L2 for HBM figures)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--p2p", action="store_true")
    a = ap.parse_args(argv)
    n = a.mb << 20
    for k in KINDS:
        for pinned in ((True, False) if k in ("h2d", "d2h") else (True,)):
            print(json.dumps({"probe": k, "pinned": pinned, "mib": a.mb, "gbs": round(probe(k, n, a.iters, pinned), 1)}), flush=True)
    if a.p2p:
        import torch
        nd = torch.cuda.device_count()
        for s in range(nd):
            for d in range(nd):
                if s != d:
                    for kr in (False, True):
                        g, ok = probe_p2p(s, d, n, a.iters, kr)
                        print(json.dumps({"probe": "p2p_kernel_read" if kr else "p2p_copy", "src": s, "dst": d,
                                          "peer_access": ok, "mib": a.mb, "gbs": round(g, 1)}), flush=True)


if __name__ == "__main__":
    main()
