"""Tensor-core (bf16 operands, fp32 accumulation) 3x3x3 convolution against the CPU oracle.

Inputs and weights are chosen bf16-representable, so the only differences from the float64 oracle are
fp32 accumulation order and the bf16 rounding of the tree means: the check is much tighter (5e-3) than
the bound the bf16 path has to meet for arbitrary inputs (relative error <= 2e-2), which is checked
separately with unrounded inputs.
"""
import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu


def bf16_round(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).to(torch.float32).numpy()


@pytest.fixture()
def bf16_mode():
    from _pyaprwrapper.aprnet import cuda as C
    C.set_conv_precision("bf16")
    yield C
    C.set_conv_precision("fp32")
    assert C.tc_error_flag() == 0, "a tensor-core kernel gave up waiting on a barrier"


CHANNELS = [(3, 4, 2), (32, 32, 2), (33, 33, 3), (64, 48, 1), (16, 136, 2), (1, 32, 2), (72, 260, 1)]


@pytest.mark.parametrize("cin,cout,nst", CHANNELS)
@pytest.mark.parametrize("name", ["blob", "odd", "ref_shape"])
def test_conv333_tensor_core_path(name, cin, cout, nst, oracle, bf16_mode):
    import pyapr
    from _pyaprwrapper.data_containers import APRPtrVector
    C = bf16_mode
    dev = torch.device("cuda:0")
    a = H.arrays(name) if name in H.APR_CASES else H.blob_arrays()
    apr = pyapr.apr_from_arrays(a, name)
    apr.init_cuda()
    o = oracle.OracleAPR(a)
    L = a.level_max - a.level_min + 1
    rng = np.random.RandomState(3)
    for dl in range(0, min(H.max_dl(a), 2) + 1):
        n = o.number_parts(dl)
        ld = torch.full((1,), dl, dtype=torch.int32)
        for exact_inputs in (True, False):
            x = rng.rand(cin, n).astype(np.float32)
            w = (rng.randn(L, cout, cin, 3, 3, 3) / np.sqrt(27 * cin)).astype(np.float32)
            go = rng.randn(cout, n).astype(np.float32)
            if exact_inputs:
                x, w, go = bf16_round(x), bf16_round(w), bf16_round(go)
            xt = torch.from_numpy(x).to(dev)[None].contiguous()
            wt = torch.from_numpy(w).to(dev)
            got = torch.from_numpy(go).to(dev)[None].contiguous()
            out = C.conv333_forward(APRPtrVector([apr]), xt, wt, ld)
            gi, gw = C.conv333_backward(APRPtrVector([apr]), xt, wt, got, ld)
            want = o.conv333_forward(x.astype(np.float64), w.astype(np.float64), dl)
            gi_ref, gw_ref = o.conv333_backward(x.astype(np.float64), w.astype(np.float64), go.astype(np.float64), dl)
            # inputs that are exact in bf16 leave only the fp32 accumulation order (outputs: 27 * cin terms) and, for the input
            # gradient, the bf16 rounding of the per-(target, tap) sums of grad_output rows of the cross-level part
            tol_out, tol_gi = (5e-3, 5e-3) if exact_inputs else (2e-2, 2e-2)
            assert H.rel_err(H.t2n(out[0]), want) <= tol_out, (name, dl, exact_inputs)
            assert H.rel_err(H.t2n(gi[0]), gi_ref) <= tol_gi, (name, dl, exact_inputs)
            assert H.rel_err(H.t2n(gw), gw_ref) <= tol_out, (name, dl, exact_inputs)


@pytest.mark.parametrize("taps,wps,tma_taps", [(1, 1, 0), (3, 1, 0), (3, 2, 0), (3, 4, 0), (2, 4, 0), (9, 4, 0), (3, 2, 1), (2, 2, 1)])
def test_conv333_stage_shape_variants(taps, wps, tma_taps, oracle, bf16_mode):
    """Every compiled stage shape of the gather kernel (taps per stage, producer warps per stage, taps fetched by the TMA
    unit) gives the same parity; shapes that do not exist for a tile geometry fall back to the automatic choice."""
    import pyapr
    from _pyaprwrapper.data_containers import APRPtrVector
    C = bf16_mode
    dev = torch.device("cuda:0")
    a = H.blob_arrays((48, 64, 64), 8, 5)
    apr = pyapr.apr_from_arrays(a)
    apr.init_cuda()
    o = oracle.OracleAPR(a)
    L = a.level_max - a.level_min + 1
    rng = np.random.RandomState(5)
    C.tc_set_option("taps", taps); C.tc_set_option("wps", wps); C.tc_set_option("tma_taps", tma_taps)
    try:
        for cin, cout, dl in [(32, 32, 0), (64, 64, 0), (64, 32, 1), (16, 48, 0), (128, 130, 1)]:
            n = o.number_parts(dl)
            x = bf16_round(rng.rand(cin, n)); w = bf16_round(rng.randn(L, cout, cin, 3, 3, 3) / np.sqrt(27 * cin)); go = bf16_round(rng.randn(cout, n))
            ld = torch.full((1,), dl, dtype=torch.int32)
            xt = torch.from_numpy(x).to(dev)[None].contiguous()
            wt = torch.from_numpy(w).to(dev)
            got = torch.from_numpy(go).to(dev)[None].contiguous()
            out = C.conv333_forward(APRPtrVector([apr]), xt, wt, ld)
            gi, gw = C.conv333_backward(APRPtrVector([apr]), xt, wt, got, ld)
            want = o.conv333_forward(x.astype(np.float64), w.astype(np.float64), dl)
            gi_ref, gw_ref = o.conv333_backward(x.astype(np.float64), w.astype(np.float64), go.astype(np.float64), dl)
            assert H.rel_err(H.t2n(out[0]), want) <= 5e-3, (taps, wps, cin, cout, dl)
            assert H.rel_err(H.t2n(gi[0]), gi_ref) <= 5e-3, (taps, wps, cin, cout, dl)
            assert H.rel_err(H.t2n(gw), gw_ref) <= 5e-3, (taps, wps, cin, cout, dl)
    finally:
        C.tc_set_option("taps", 0); C.tc_set_option("wps", 0); C.tc_set_option("tma_taps", 0)


@pytest.mark.parametrize("cin,cout,nst", [(64, 32, 2), (32, 2, 2), (2, 32, 1), (40, 19, 6), (256, 128, 2), (128, 256, 1), (72, 130, 3), (1, 1, 1)])
@pytest.mark.parametrize("name", ["blob", "odd", "multi_tile"])
def test_conv111_tensor_core_path(name, cin, cout, nst, oracle, bf16_mode):
    """1x1x1 convolution on the tensor cores (forward, input gradient and weight gradient) against the float64 oracle:
    bf16-exact operands leave only the fp32 accumulation order."""
    import pyapr
    from _pyaprwrapper.data_containers import APRPtrVector
    C = bf16_mode
    dev = torch.device("cuda:0")
    a = H.blob_arrays((64, 128, 128), 40, 11) if name == "multi_tile" else (H.arrays(name) if name in H.APR_CASES else H.blob_arrays())
    apr = pyapr.apr_from_arrays(a, name)
    apr.init_cuda()
    o = oracle.OracleAPR(a)
    rng = np.random.RandomState(17)
    for dl in range(0, min(H.max_dl(a), 2) + 1):
        n = o.number_parts(dl)
        ld = torch.full((1,), dl, dtype=torch.int32)
        for exact_inputs in (True, False):
            x = rng.rand(cin, n).astype(np.float32)
            w = (rng.randn(nst, cout, cin, 1, 1, 1) / np.sqrt(cin)).astype(np.float32)
            go = rng.randn(cout, n).astype(np.float32)
            if exact_inputs:
                x, w, go = bf16_round(x), bf16_round(w), bf16_round(go)
            xt = torch.from_numpy(x).to(dev)[None].contiguous()
            wt = torch.from_numpy(w).to(dev)
            got = torch.from_numpy(go).to(dev)[None].contiguous()
            C.profile_read(); C.profile_enable(True)
            out = C.conv111_forward(APRPtrVector([apr]), xt, wt, ld)
            gi, gw = C.conv111_backward(APRPtrVector([apr]), xt, wt, got, ld)
            torch.cuda.synchronize()
            C.profile_enable(False)
            names = set(k.split(":")[0] for k in C.profile_read())
            # the tensor-core kernel ran unless the layer is narrower than 8 channels on either side (those stay on the CUDA cores)
            assert ("conv111_tc" in names) == (min(cin, cout) >= 8), names
            want = o.conv111_forward(x.astype(np.float64), w.astype(np.float64), dl)
            gi_ref, gw_ref = o.conv111_backward(x.astype(np.float64), w.astype(np.float64), go.astype(np.float64), dl)
            tol = 2e-5 if (exact_inputs or min(cin, cout) < 8) else 2e-2
            assert H.rel_err(H.t2n(out[0]), want) <= tol, (name, dl, exact_inputs)
            assert H.rel_err(H.t2n(gi[0]), gi_ref) <= tol, (name, dl, exact_inputs)
            assert H.rel_err(H.t2n(gw), gw_ref) <= (2e-5 if exact_inputs else 2e-2), (name, dl, exact_inputs)
            assert "conv111_tc_dw" in names, names            # the weight gradient takes the tensor cores at every width
            # an explicit per-call precision overrides the process-wide setting
            out32 = C.conv111_forward(APRPtrVector([apr]), xt, wt, ld, "fp32")
            assert H.rel_err(H.t2n(out32[0]), want) <= 1e-5
