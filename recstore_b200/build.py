"""In-tree native build of ``librecstore_b200.so``.

Every ``.cu`` under ``csrc/`` is compiled by ``nvcc`` for exactly one target,
``sm_100a`` (Blackwell B200), every ``.cpp`` by ``g++``; the objects are linked
into ``recstore_b200/lib/librecstore_b200.so``.  The library exposes a C ABI
(``extern "C"``) that ``recstore_b200._lib`` binds through ``ctypes``; it does
not include any libtorch header, so a full rebuild takes well under a minute
and the same binary works with any PyTorch build.  Tensors cross the boundary
as raw device/host pointers plus a ``cudaStream_t``.

Usage::

    python -m recstore_b200.build            # incremental
    python -m recstore_b200.build --force    # rebuild everything
    python -m recstore_b200.build --ptxas-v  # print registers / spills / smem

A CPU-only host can build and import the library (nvcc cross-compiles); the
CUDA runtime is linked dynamically and only touched when a GPU entry point is
actually called.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "lib" / "obj"
LIB_PATH = PKG_DIR / "lib" / "librecstore_b200.so"

GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _cuda_home() -> Path:
    for env in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(env):
            return Path(os.environ[env])
    nvcc = shutil.which("nvcc")
    if nvcc:
        return Path(nvcc).resolve().parent.parent
    return Path("/usr/local/cuda")


PRELOAD_DIR = CSRC / "preload"          # LD_PRELOAD shims: one small library each, never part of the main one
STRESS_DIR = CSRC / "stress"            # stand-alone drivers (their own main), built on demand with a sanitizer
UVM_SHIM_PATH = PKG_DIR / "lib" / "librecstore_uvm_intercept.so"


def _sources():
    skip = (PRELOAD_DIR, STRESS_DIR)
    cu = sorted(p for p in CSRC.rglob("*.cu") if not any(d in p.parents for d in skip))
    cpp = sorted(p for p in CSRC.rglob("*.cpp") if not any(d in p.parents for d in skip))
    return cu, cpp


def build_host_stress(sanitize: str = "thread", out_dir: Path | None = None, verbose: bool = False) -> Path:
    """Builds ``csrc/stress/host_stress.cpp`` together with the host runtime (``csrc/runtime``, ``csrc/common``: no
    CUDA kernels) into one executable under ``-fsanitize=<sanitize>`` ("thread", "address" or "" for none).  The CUDA
    runtime is linked for the symbols the allocator files name; the driver never calls into it."""
    cuda = _cuda_home()
    cxx = os.environ.get("CXX", "g++")
    if sanitize:                     # not every toolchain ships the sanitizer runtimes: take the first compiler that has this one
        rt = {"thread": "libtsan.so", "address": "libasan.so", "undefined": "libubsan.so"}.get(sanitize)
        for cand in dict.fromkeys([cxx, "g++", "/usr/bin/g++"]):
            if shutil.which(cand) is None:
                continue
            found = subprocess.run([cand, "-print-file-name=" + (rt or "libc.so")], stdout=subprocess.PIPE, text=True).stdout.strip()
            if rt is None or os.path.isabs(found):
                cxx = cand
                break
        else:
            raise RuntimeError(f"no compiler with the {sanitize} sanitizer runtime was found")
    out_dir = Path(out_dir) if out_dir is not None else PKG_DIR / "lib"
    out_dir.mkdir(parents=True, exist_ok=True)
    exe = out_dir / ("host_stress_" + (sanitize or "plain"))
    srcs = sorted((CSRC / "runtime").glob("*.cpp")) + sorted((CSRC / "common").glob("*.cpp")) + [STRESS_DIR / "host_stress.cpp"]
    cmd = [cxx, "-O1", "-g", "-std=c++17", "-pthread", "-fno-omit-frame-pointer", "-I", str(CSRC), "-I", str(cuda / "include")]
    if sanitize:
        cmd += ["-fsanitize=" + sanitize]
    cmd += [str(s) for s in srcs] + ["-o", str(exe), "-L", str(cuda / "lib64"), "-lcudart", "-lrt", "-ldl",
                                     "-Wl,-rpath," + str(cuda / "lib64")]
    rc, out = _run(cmd, verbose)
    if rc != 0:
        print(out, file=sys.stderr)
        raise RuntimeError("building the host stress driver failed")
    return exe


def build_preload_shims(verbose: bool = False) -> Path:
    """Builds the cudaMalloc -> cudaMallocManaged interposer (no CUDA needed at build time)."""
    src = PRELOAD_DIR / "uvm_intercept.cpp"
    UVM_SHIM_PATH.parent.mkdir(parents=True, exist_ok=True)
    if not UVM_SHIM_PATH.exists() or UVM_SHIM_PATH.stat().st_mtime < src.stat().st_mtime:
        rc, out = _run([os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
                        str(src), "-o", str(UVM_SHIM_PATH), "-ldl"], verbose)
        if rc != 0:
            print(out, file=sys.stderr)
            raise RuntimeError("building the UVM interposer failed")
    return UVM_SHIM_PATH


def _headers_digest() -> str:
    h = hashlib.sha1()
    for p in sorted(list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.hpp"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _obj_for(src: Path) -> Path:
    rel = src.relative_to(CSRC)
    return OBJ_DIR / ("_".join(rel.parts) + ".o")


def _stamp_for(obj: Path) -> Path:
    return obj.with_suffix(".stamp")


def _needs_build(src: Path, obj: Path, hdr_digest: str, flags: str) -> bool:
    stamp = _stamp_for(obj)
    if not obj.exists() or not stamp.exists():
        return True
    want = hashlib.sha1(src.read_bytes() + hdr_digest.encode() + flags.encode()).hexdigest()
    return stamp.read_text().strip() != want


def _write_stamp(src: Path, obj: Path, hdr_digest: str, flags: str) -> None:
    want = hashlib.sha1(src.read_bytes() + hdr_digest.encode() + flags.encode()).hexdigest()
    _stamp_for(obj).write_text(want)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    return p.returncode, p.stdout


def build(force: bool = False, verbose: bool = False, ptxas_v: bool = False, jobs: int | None = None) -> Path:
    """Compile and link the native library; returns the path of the ``.so``."""
    cuda = _cuda_home()
    nvcc = str(cuda / "bin" / "nvcc")
    cxx = os.environ.get("CXX", "g++")
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    cu, cpp = _sources()
    hdr = _headers_digest()
    inc = ["-I", str(CSRC)]
    nvcc_flags = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC,-O3",
                  "--expt-relaxed-constexpr", "-DRS_BOUNDS_CHECK=1"] + GENCODE
    if ptxas_v:
        nvcc_flags += ["-Xptxas", "-v"]
    cxx_flags = ["-O3", "-std=c++17", "-fPIC", "-pthread", "-Wall", "-Wno-unused-function",
                 "-I", str(cuda / "include")]
    if os.environ.get("RS_SANITIZE"):  # host-side TSAN/ASAN builds of the C++ runtime
        cxx_flags += ["-g", "-fsanitize=" + os.environ["RS_SANITIZE"]]

    tasks = []
    for s in cu:
        o = _obj_for(s)
        fl = " ".join(nvcc_flags)
        if force or ptxas_v or _needs_build(s, o, hdr, fl):
            tasks.append((s, o, [nvcc] + nvcc_flags + inc + ["-c", str(s), "-o", str(o)], fl))
    for s in cpp:
        o = _obj_for(s)
        fl = " ".join(cxx_flags)
        if force or _needs_build(s, o, hdr, fl):
            tasks.append((s, o, [cxx] + cxx_flags + inc + ["-c", str(s), "-o", str(o)], fl))

    failed = []
    if tasks:
        with cf.ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as ex:
            futs = {ex.submit(_run, cmd, verbose): (s, o, fl) for (s, o, cmd, fl) in tasks}
            for f in cf.as_completed(futs):
                s, o, fl = futs[f]
                rc, out = f.result()
                if rc != 0:
                    failed.append((s, out))
                else:
                    _write_stamp(s, o, hdr, fl)
                    if out.strip() and (verbose or ptxas_v or "warning" in out):
                        print(f"--- {s.relative_to(CSRC)}\n{out}", flush=True)
    if failed:
        for s, out in failed:
            print(f"*** build failed: {s}\n{out}", file=sys.stderr, flush=True)
        raise RuntimeError("native build failed: " + ", ".join(str(s.name) for s, _ in failed))

    objs = [str(_obj_for(s)) for s in cu + cpp]
    relink = force or bool(tasks) or not LIB_PATH.exists()
    if relink:
        # Only the C ABI (rs_*) is exported.  The C++ runtime may be linked in statically, and its symbols must not be
        # visible to other extension modules of the process: a module loaded later would bind its iostream calls to
        # this library's private copy, whose locale state that module never initialised.
        vs = OBJ_DIR / "exports.map"
        vs.write_text("{ global: rs_*; local: *; };\n")
        link = [cxx, "-shared", "-o", str(LIB_PATH)] + objs + [
            "-L", str(cuda / "lib64"), "-lcudart_static", "-lpthread", "-lrt", "-ldl",
            "-Wl,-rpath," + str(cuda / "lib64"), "-Wl,--version-script=" + str(vs), "-Wl,--exclude-libs,ALL"]
        if os.environ.get("RS_SANITIZE"):
            link += ["-fsanitize=" + os.environ["RS_SANITIZE"]]
        rc, out = _run(link, verbose)
        if rc != 0:
            print(out, file=sys.stderr)
            raise RuntimeError("link failed")
    build_preload_shims(verbose)
    return LIB_PATH


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-v", action="store_true")
    ap.add_argument("-j", "--jobs", type=int, default=None)
    a = ap.parse_args(argv)
    p = build(force=a.force, verbose=a.verbose, ptxas_v=a.ptxas_v, jobs=a.jobs)
    print(p)


if __name__ == "__main__":
    main()
