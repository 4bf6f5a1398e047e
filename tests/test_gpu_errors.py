"""Error paths on the GPU that need no fault: a bounded wait that runs out sets the error flag, the tensor-core
entry points refuse further work until the flag is reset, and a handle used from another device is an argument
error (checked before anything is launched)."""
import ctypes

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu


def _layer(C, apr, a):
    from _pyaprwrapper.data_containers import APRPtrVector
    dev = torch.device("cuda:0")
    L = a.level_max - a.level_min + 1
    x = torch.rand(1, 16, a.n_particles, device=dev)
    w = torch.randn(L, 16, 16, 3, 3, 3, device=dev)
    return C.conv333_forward(APRPtrVector([apr]), x, w, torch.zeros(1, dtype=torch.int32))


def test_bounded_wait_runs_out_and_the_flag_can_be_reset():
    import pyapr
    from _pyaprwrapper.aprnet import cuda as C
    a = H.blob_arrays()
    apr = pyapr.apr_from_arrays(a)
    apr.init_cuda()
    C.set_conv_precision("bf16")
    try:
        C.tc_error_reset()
        assert C.tc_error_flag() == 0
        ref = _layer(C, apr, a)
        C.tc_selftest_wait_timeout(2000)            # a kernel waits on a barrier nothing arrives at, gives up and returns
        assert C.tc_error_flag() == 1
        with pytest.raises(RuntimeError, match="gave up waiting"):
            _layer(C, apr, a)
        C.tc_error_reset()
        assert C.tc_error_flag() == 0
        out = _layer(C, apr, a)                       # the context is intact: the same call works again
        assert out.shape == ref.shape and torch.isfinite(out).all()
    finally:
        C.tc_error_reset()
        C.set_conv_precision("fp32")


def test_handle_on_another_device_is_an_argument_error():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import pyapr
    from _pyaprwrapper.aprnet import cuda as C
    from _pyaprwrapper.data_containers import APRPtrVector
    a = H.blob_arrays()
    apr = pyapr.apr_from_arrays(a)
    with torch.cuda.device(0):
        apr.init_cuda()
    assert torch.cuda.current_device() == 0
    x = torch.rand(1, 2, a.n_particles, device="cuda:1")
    with pytest.raises(RuntimeError, match="lives on cuda:0"):
        C.maxpool_forward_cuda(APRPtrVector([apr]), x, torch.zeros(1, dtype=torch.int32))
    # the C ABI itself: current device 1, handle on device 0 -> status code, nothing launched
    import os
    lib = ctypes.CDLL(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "apr-cnn_b200", "libaprnet_b200.so"))
    lib.aprnet_last_error.restype = ctypes.c_char_p
    with torch.cuda.device(1):
        torch.cuda.current_stream().synchronize()
        # plan() switches to the APR's device by itself
        apr.plan(0)
        assert torch.cuda.current_device() == 1
    del apr
    assert torch.cuda.current_device() == 0           # destroying an APR leaves the current device alone
