"""ctypes binding of ``librecstore_b200.so`` (the native C++/CUDA half of the package).

The library is built in-tree by :mod:`recstore_b200.build`.  Loading never falls back
silently: if the shared object is missing, :func:`lib` builds it when a compiler is present and
otherwise raises, so a GPU run can never end up on a pure-PyTorch path by accident.

Calling convention: every native function returns an ``int`` status (0 = ok); :func:`check`
turns a failure into :class:`RecStoreError` carrying the native message.  Tensors are passed as
raw pointers (``tensor.data_ptr()``), streams as the ``cudaStream_t`` integer of
``torch.cuda.current_stream()``.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "librecstore_b200.so"
_lock = threading.Lock()
_lib = None


class RecStoreError(RuntimeError):
    """A native call failed; ``code`` is the RsStatus value."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"[recstore_b200 native error {code}] {msg}")
        self.code = code


class DeviceStatusError(RecStoreError):
    """A kernel recorded a device-side error (bounds check, bounded wait ran out)."""


# RsStatus
OK, ERR_INVALID, ERR_CUDA, ERR_TIMEOUT, ERR_CAPACITY, ERR_NOTFOUND, ERR_IO, ERR_STATE = range(8)
# RsDevErr bits
DEV_OOB_ROW, DEV_OOB_SLOT, DEV_OOB_PEER, DEV_WAIT_TIMEOUT, DEV_TABLE_FULL, DEV_BAD_ARG = (1 << i for i in range(6))

vp = C.c_void_p
i32 = C.c_int
i64 = C.c_longlong
u32 = C.c_uint
u64 = C.c_ulonglong
f32 = C.c_float
f64 = C.c_double
sz = C.c_size_t
cstr = C.c_char_p


class HashTableView(C.Structure):
    """Mirror of ``rs::HashTableView`` (device pointers of one HBM hash-table shard)."""

    _fields_ = [("keys", vp), ("rows", vp), ("mask", u64), ("next_row", vp), ("free_rows", vp),
                ("free_top", vp), ("size", vp), ("max_rows", i32)]


_SIGNATURES = {
    "rs_last_error": (cstr, []),
    "rs_abi_version": (i32, []),
    # ops/gemm_tcgen05.cu
    "rs_gemm_bf16": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp]),
    # ops/embedding.cu
    "rs_emb_forward": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, i64, vp, i32, vp, vp, vp, vp, vp]),
    "rs_emb_backward": (i32, [vp, vp, i64, vp, vp, i64, vp, vp, i64, vp, i32, i32, i32, i32, vp, f32, f32, i32, vp, vp]),
    "rs_emb_forward_ex": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, i64, vp, i32, vp, vp, vp,
                                vp, i32, i32, vp, vp, vp, u64, i32, vp, vp, i32, i32, i32, vp]),
    "rs_emb_backward_ex": (i32, [vp, vp, i64, vp, vp, i64, vp, vp, i64, vp, i32, i32, i32, i32, f32, f32, i32, vp,
                                 vp, vp, vp, u64, i32, i32, vp]),
    # comm/emb_exchange.cu
    "rs_push_rows": (i32, [vp, i64, i32, i32, i32, i32, vp, vp, vp, i64, i64, vp, i32, vp, vp, vp, i32, i32, vp]),
    "rs_rw_push_keys": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, i32, vp]),
    "rs_rw_reduce_partials": (i32, [vp, vp, vp, i64, i32, i32, i32, i32, vp, vp, u64, i32, vp, vp]),
    "rs_interaction_forward_ex": (i32, [vp, i32, i32, i32, vp, i32, vp, vp, u64, i32, i32, vp, vp]),
    "rs_peer_wait_own": (i32, [vp, i32, i32, vp, u64, vp, vp]),
    "rs_rows_gather": (i32, [vp, vp, i64, i32, vp, vp]),
    "rs_rows_scatter": (i32, [vp, vp, i64, i32, vp, vp]),
    # ops/interaction.cu
    "rs_interaction_forward": (i32, [vp, i32, i32, i32, vp, i32, vp]),
    "rs_interaction_dx": (i32, [vp, vp, i32, i32, i32, i32, vp, i32, i32, vp]),
    "rs_interaction_backward": (i32, [vp, vp, i32, i32, i32, i32, vp, i32, vp, vp, vp, i64, i64, i32, vp, i32, i32, vp]),
    # ops/dense.cu
    "rs_head_bce": (i32, [vp, i32, i32, i32, vp, vp, vp, f32, vp, vp, vp, i32, vp, vp, vp]),
    "rs_colsum_bf16": (i32, [vp, i32, i32, i32, vp, vp]),
    "rs_dense_sgd": (i32, [vp, vp, i32, i32, f32, vp, i32, vp, i32, i32, vp]),
    "rs_vec_sgd": (i32, [vp, vp, i32, f32, i32, vp]),
    "rs_dense_sgd_multi": (i32, [vp, vp, i32, i32, vp, vp, i32, f32, i32, i64, i32, vp]),
    "rs_pad_cast_bf16": (i32, [vp, i32, i32, i32, vp, i32, vp]),
    "rs_mse_fwd_bwd": (i32, [vp, vp, i32, f32, vp, vp, vp]),
    "rs_cross_fwd": (i32, [vp, vp, vp, vp, i64, vp]),
    "rs_cross_bwd": (i32, [vp, vp, vp, vp, vp, i64, i32, vp]),
    "rs_push_feature_grads": (i32, [vp, vp, vp, i32, i32, i32, vp, i32, vp, vp, vp, i64, i64, i32, vp, i32, vp, i32, i32, vp]),
    "rs_proj_inter_fwd": (i32, [vp, i32, vp, vp, i32, i32, i32, i32, vp, i32, i32, vp]),
    "rs_proj_inter_bwd": (i32, [vp, i32, i32, vp, vp, i32, i32, i32, i32, vp, vp, vp]),
    # comm/peer.cu
    "rs_device_count": (i32, [C.POINTER(i32)]),
    "rs_peer_alloc": (i32, [sz, C.POINTER(vp)]),
    "rs_peer_free": (i32, [vp]),
    "rs_ipc_get_handle": (i32, [vp, vp]),
    "rs_ipc_open": (i32, [vp, C.POINTER(vp)]),
    "rs_ipc_close": (i32, [vp]),
    "rs_peer_signal": (i32, [vp, i32, i32, i32, vp, vp]),
    "rs_peer_wait": (i32, [vp, i32, i32, vp, u64, vp, vp]),
    "rs_peer_sync": (i32, [vp, vp, i32, i32, i32, vp, vp, u64, vp, vp]),
    "rs_allreduce_push": (i32, [vp, vp, i32, i32, i64, i64, f32, vp]),
    "rs_memset_async": (i32, [vp, i32, sz, vp]),
    "rs_stamp_time": (i32, [vp, vp]),
    "rs_read_status": (i32, [vp, C.POINTER(u64), i32]),
}


def register_signatures(sigs: dict) -> None:
    """Lets sub-modules declare the native functions they bind (applied on load)."""
    _SIGNATURES.update(sigs)
    if _lib is not None:
        _apply(_lib, sigs)


def _apply(lib, sigs):
    for name, (res, args) in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:  # stale binary
            raise RecStoreError(ERR_STATE, f"native symbol {name} missing from {_LIB_PATH}; rebuild with "
                                           f"`python -m recstore_b200.build --force`") from e
        fn.restype = res
        fn.argtypes = args


def lib():
    """Returns the loaded native library, building it first if the binary is absent."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = os.environ.get("RECSTORE_B200_LIB")   # an alternative build of the same ABI (A/B timing of kernels)
        if path is None:
            if not _LIB_PATH.exists() or os.environ.get("RECSTORE_B200_REBUILD"):
                from . import build as _build
                _build.build()
            path = str(_LIB_PATH)
        l = C.CDLL(path)       # RTLD_LOCAL: nothing of this library may interpose on other extension modules
        _apply(l, _SIGNATURES)
        _lib = l
    return _lib


def lib_path() -> str:
    """File the native library is (or will be) loaded from: ``RECSTORE_B200_LIB`` when set, else the in-tree build."""
    return os.environ.get("RECSTORE_B200_LIB") or str(_LIB_PATH)


def check(rc: int) -> None:
    if rc != 0:
        msg = lib().rs_last_error()
        raise RecStoreError(rc, msg.decode(errors="replace") if msg else "unknown error")


def call(name: str, *args):
    """``check(lib().<name>(*args))`` with ``None`` mapped to a null pointer."""
    check(getattr(lib(), name)(*args))


def ptr(t) -> int | None:
    """Device/host address of a tensor (``None`` stays ``None``)."""
    if t is None:
        return None
    return t.data_ptr()


def stream_ptr(stream=None) -> int:
    import torch
    if stream is None:
        stream = torch.cuda.current_stream()
    return stream.cuda_stream


def decode_status(word: int) -> str:
    names = ["oob_row", "oob_slot", "oob_peer", "wait_timeout", "table_full", "bad_arg"]
    bits = [n for i, n in enumerate(names) if word & (1 << i)]
    extra = ""
    if word & DEV_WAIT_TIMEOUT:
        extra = f" (waiting for rank {(word >> 32) & 0xFFFF}, channel {(word >> 48) & 0xFFFF})"
    return "|".join(bits) + extra
