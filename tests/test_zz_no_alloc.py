"""The allocation-free weight-gradient entry point against the regular one, through the C ABI.

`aprnet_conv111_backward_weights_static` serves hosts that cannot allocate device memory at the point
where they call the library (an arena that owns the whole GPU, a fixed start-up budget, a loop that must
not trigger an allocation's device-wide synchronisation).  Its block-partial sums live in a fixed array
inside the library instead of a caller workspace, and that array keeps the previous call's contents —
so the check runs two different problems back to back and compares each with the regular entry point
(same float32 tolerance as the other parity tests: relative error <= 1e-5).

This file is named so that pytest collects it last.
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    lib = C.CDLL(os.path.join(ROOT, "apr-cnn_b200", "libaprnet_b200.so"))
    lib.aprnet_last_error.restype = C.c_char_p
    lib.aprnet_conv111_partial_elems.restype = C.c_int64
    lib.aprnet_number_parts.restype = C.c_int64
    lib.aprnet_static_scratch_bytes.restype = C.c_int64
    return lib


def _create(lib, a):
    h = C.c_void_p()
    dims = np.ascontiguousarray(np.array(a.dims, dtype=np.int32).reshape(-1))
    rp = np.ascontiguousarray(a.row_ptr, dtype=np.int64); y = np.ascontiguousarray(a.y, dtype=np.uint16)
    trp = np.ascontiguousarray(a.tree_row_ptr, dtype=np.int64); ty = np.ascontiguousarray(a.tree_y, dtype=np.uint16)
    vp = lambda arr: arr.ctypes.data_as(C.c_void_p)
    rc = lib.aprnet_apr_create(C.byref(h), int(a.level_min), int(a.level_max), vp(dims), vp(rp), vp(y), vp(trp), vp(ty), 0)
    assert rc == 0, lib.aprnet_last_error()
    return h


def test_static_workspace_matches_regular_entry_point_twice():
    assert torch.cuda.is_available()
    lib = _lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    a = H.blob_arrays()
    h = _create(lib, a)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: C.c_void_p(t.data_ptr())
    try:
        # two different problems in a row: the second must not see anything of the first
        for call, (dl, cin, cout, nst) in enumerate([(0, 24, 40, 3), (1, 7, 5, 2)]):
            n = int(lib.aprnet_number_parts(h, dl))
            g = torch.Generator(device="cpu").manual_seed(100 + call)
            x = torch.randn(cin, n, generator=g).to(dev)
            go = torch.randn(cout, n, generator=g).to(dev)
            gw_ref = torch.zeros(nst, cout, cin, device=dev)
            gw_new = torch.zeros(nst, cout, cin, device=dev)
            partial = torch.empty(int(lib.aprnet_conv111_partial_elems(cin, cout)), device=dev)
            rc = lib.aprnet_conv111_backward_weights(h, dl, 0, cin, cout, nst, ptr(x), C.c_int64(n), ptr(go), C.c_int64(n),
                                                     ptr(gw_ref), ptr(partial), stream)
            assert rc == 0, lib.aprnet_last_error()
            rc = lib.aprnet_conv111_backward_weights_static(h, dl, cin, cout, nst, ptr(x), C.c_int64(n), ptr(go), C.c_int64(n),
                                                            ptr(gw_new), stream)
            assert rc == 0, lib.aprnet_last_error()
            torch.cuda.synchronize()
            assert H.rel_err(gw_new.cpu().numpy(), gw_ref.cpu().numpy()) <= 1e-5, (call, dl)
            assert float(gw_ref.abs().max()) > 0

        # sizes beyond the built-in workspace are refused with a clear message, nothing is launched
        big = 1024
        rc = lib.aprnet_conv111_backward_weights_static(h, dl, big, big, 1, ptr(x), C.c_int64(n), ptr(go), C.c_int64(n), ptr(gw_new), stream)
        assert rc == -3
        assert b"exceeds the built-in workspace" in lib.aprnet_last_error()
        assert lib.aprnet_static_scratch_bytes() == 4 << 20
    finally:
        torch.cuda.synchronize()
        lib.aprnet_apr_destroy(h)
