"""The allocation-free unique() entry point, called through its exported C symbol.

Some users of the library cannot obtain device memory when they need a result (all HBM already given to
another allocator, allocation forbidden on their thread, or no tolerance for the device-wide stall of
cudaMalloc).  ``rs_unique_keys_noalloc`` serves them from a fixed 3 MiB array inside the library.  This
test checks it against the ordinary entry point (``rs_unique_keys``, scratch from the caller) on two calls
in a row -- the second call must not be disturbed by what the first one left in the shared array -- and
checks that an oversized batch is refused with a clear error.  The file is named so that pytest collects
it last.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_KEYS = 1 << 17


def _load():
    # The package's loader builds the library when it is missing and honours RECSTORE_B200_LIB; the symbols are then
    # looked up on a plain ctypes handle of that same file, so the call goes through the exported C symbol.
    from recstore_b200 import _lib
    _lib.lib()
    lib = C.CDLL(str(_lib.lib_path()))
    vp, i64, u64 = C.c_void_p, C.c_longlong, C.c_ulonglong
    lib.rs_unique_keys_noalloc.restype = C.c_int
    lib.rs_unique_keys_noalloc.argtypes = [vp, i64, vp, vp, vp, vp, vp]
    lib.rs_unique_keys.restype = C.c_int
    lib.rs_unique_keys.argtypes = [vp, i64, vp, vp, u64, vp, vp, vp, vp, vp]
    lib.rs_last_error.restype = C.c_char_p
    return lib


def _run_noalloc(lib, keys):
    n, dev = keys.numel(), keys.device
    uniq = torch.full((max(n, 1),), -7, dtype=torch.int64, device=dev)
    inv = torch.full((max(n, 1),), -7, dtype=torch.int32, device=dev)
    cnt = torch.full((1,), -7, dtype=torch.int32, device=dev)
    st = torch.zeros(1, dtype=torch.int64, device=dev)
    rc = lib.rs_unique_keys_noalloc(keys.data_ptr(), n, uniq.data_ptr(), inv.data_ptr(), cnt.data_ptr(), st.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.rs_last_error()
    torch.cuda.synchronize()
    assert st.item() == 0
    u = int(cnt.item())
    return uniq[:u], inv[:n].long()


def _run_reference_entry(lib, keys):
    n, dev = keys.numel(), keys.device
    nslots = 2
    while nslots < 2 * max(n, 1):
        nslots <<= 1
    sk = torch.empty(nslots, dtype=torch.int64, device=dev)
    si = torch.empty(nslots, dtype=torch.int32, device=dev)
    uniq = torch.empty(max(n, 1), dtype=torch.int64, device=dev)
    inv = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
    cnt = torch.zeros(1, dtype=torch.int32, device=dev)
    st = torch.zeros(1, dtype=torch.int64, device=dev)
    rc = lib.rs_unique_keys(keys.data_ptr(), n, sk.data_ptr(), si.data_ptr(), nslots, uniq.data_ptr(), inv.data_ptr(), cnt.data_ptr(),
                            st.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.rs_last_error()
    torch.cuda.synchronize()
    u = int(cnt.item())
    return uniq[:u], inv[:n].long()


def test_noalloc_unique_matches_allocating_entry_point_twice_in_a_row():
    lib = _load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(123)
    # first call: a large batch that fills a big part of the shared array with keys
    # second call: a smaller batch from a DIFFERENT key range, whose slots overlap the ones used before
    batches = [torch.randint(0, 40_000, (MAX_KEYS,), device=dev, generator=g),
               torch.randint(1_000_000, 1_003_000, (50_000,), device=dev, generator=g)]
    for keys in batches:
        u_new, inv_new = _run_noalloc(lib, keys)
        u_old, inv_old = _run_reference_entry(lib, keys)
        # the order of the unique list is arbitrary for both entry points: compare as sets, and check the mapping
        assert u_new.numel() == u_old.numel()
        assert torch.equal(torch.sort(u_new).values, torch.sort(u_old).values)
        assert torch.equal(torch.sort(u_new).values, torch.unique(keys))
        assert torch.equal(u_new[inv_new], keys) and torch.equal(u_old[inv_old], keys)
    # empty batch: count is reset, nothing else happens
    empty = torch.empty(0, dtype=torch.int64, device=dev)
    u, inv = _run_noalloc(lib, empty)
    assert u.numel() == 0 and inv.numel() == 0


def test_noalloc_unique_rejects_oversized_batches():
    lib = _load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    keys = torch.zeros(MAX_KEYS + 1, dtype=torch.int64, device=dev)
    out = torch.empty_like(keys)
    cnt = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = lib.rs_unique_keys_noalloc(keys.data_ptr(), keys.numel(), out.data_ptr(), None, cnt.data_ptr(), None,
                                    torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = lib.rs_last_error().decode()
    assert "exceed" in msg and str(MAX_KEYS) in msg
    torch.cuda.synchronize()
