"""GPU parity: every operator of the hot path against the CPU oracle on identical seeded inputs.

Bit-exact for integer structure (neighbour / child tables, particle counts, pooling argmax);
relative error (max |a-b| / max |b|) <= 1e-12 for float64 and <= 1e-5 for float32 values.
All calls go through the Python operator functions, which dispatch into the C ABI of
libaprnet_b200.
"""
import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

TOL = {torch.float64: 1e-12, torch.float32: 1e-5}
NP = {torch.float64: np.float64, torch.float32: np.float32}


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


def make(name, oracle):
    import pyapr
    a = H.arrays(name) if name in H.APR_CASES else H.blob_arrays()
    apr = pyapr.apr_from_arrays(a, name)
    apr.init_cuda()
    return a, apr, oracle.OracleAPR(a)


CASES = list(H.APR_CASES) + ["blob"]


@pytest.mark.parametrize("name", CASES)
def test_structure_tables_bit_exact(name, oracle, dev):
    from _pyaprwrapper.aprnet import cuda as C
    from pyapr import aprnet
    a, apr, o = make(name, oracle)
    assert np.array_equal(C.child_table(apr), o.child_table())
    for dl in range(0, H.max_dl(a) + 1):
        assert aprnet.utils.number_particles(apr, dl) == o.number_parts(dl)
        assert np.array_equal(C.plan_nbr_table(apr, dl), o.nbr_table(dl)), (name, dl)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("name", CASES)
def test_fill_tree_mean(name, dtype, oracle, dev):
    from _pyaprwrapper.aprnet import cuda as C
    a, apr, o = make(name, oracle)
    rng = np.random.RandomState(0)
    for dl in range(0, H.max_dl(a) + 1):
        n = o.number_parts(dl)
        x = rng.rand(3, n).astype(NP[dtype])
        got = C.fill_tree_mean(apr, torch.from_numpy(x).to(dev), dl)
        assert H.rel_err(H.t2n(got), o.fill_tree_mean(x.astype(np.float64), dl)) <= TOL[dtype]
        gt = rng.rand(3, o.tree_size(dl)).astype(NP[dtype])
        gi = rng.rand(3, n).astype(NP[dtype])
        got = C.fill_tree_mean_backward(apr, torch.from_numpy(gi).to(dev), torch.from_numpy(gt).to(dev), dl)
        want = o.fill_tree_mean_backward(gi.astype(np.float64), gt.astype(np.float64), dl)
        assert H.rel_err(H.t2n(got), want) <= TOL[dtype]


@pytest.mark.parametrize("name", CASES)
def test_fill_tree_full_mean_and_max(name, oracle, dev):
    import pyapr
    a, apr, o = make(name, oracle)
    x = np.random.RandomState(1).rand(a.n_particles)
    xt = torch.from_numpy(x).to(dev)
    assert H.rel_err(H.t2n(pyapr.tree.fill_tree_mean(apr, xt)), o.fill_tree_mean(x[None], 0)[0]) <= 1e-12
    got = H.t2n(pyapr.tree.fill_tree_max(apr, xt))
    assert np.array_equal(got, o.fill_tree_max(x))
    assert got[0] == x.max()          # root holds the global maximum (pyapr/tests/test_tree.py:39-40)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("cin,cout,nst", [(3, 4, 2), (33, 33, 3), (1, 16, 1)])
@pytest.mark.parametrize("name", CASES)
def test_conv333(name, cin, cout, nst, dtype, oracle, dev):
    from _pyaprwrapper.aprnet import cuda as C
    from _pyaprwrapper.data_containers import APRPtrVector
    a, apr, o = make(name, oracle)
    if cin == 33 and name not in ("odd", "blob"):
        pytest.skip("wide case on two structures only")
    L = a.level_max - a.level_min + 1
    rng = np.random.RandomState(7)
    for dl in range(0, H.max_dl(a) + 1):
        n = o.number_parts(dl)
        x = rng.rand(cin, n).astype(NP[dtype])
        w = (rng.randn(nst, cout, cin, 3, 3, 3) / np.sqrt(27 * cin)).astype(NP[dtype])
        go = rng.randn(cout, n).astype(NP[dtype])
        ld = torch.full((1,), dl, dtype=torch.int32)
        wt = torch.from_numpy(w).to(dev)
        we = C.restrict_kernel333_forward(wt, L)
        we_ref = oracle.restrict333_forward(w.astype(np.float64), L)
        assert H.rel_err(H.t2n(we), we_ref) <= TOL[dtype]
        xt = torch.from_numpy(x).to(dev)[None].contiguous()
        out = C.conv333_forward(APRPtrVector([apr]), xt, we, ld)
        want = o.conv333_forward(x.astype(np.float64), we_ref, dl)
        assert H.rel_err(H.t2n(out[0]), want) <= TOL[dtype], (name, dl)
        gi, gw = C.conv333_backward(APRPtrVector([apr]), xt, we, torch.from_numpy(go).to(dev)[None].contiguous(), ld)
        gi_ref, gw_ref = o.conv333_backward(x.astype(np.float64), we_ref, go.astype(np.float64), dl)
        assert H.rel_err(H.t2n(gi[0]), gi_ref) <= TOL[dtype], (name, dl)
        assert H.rel_err(H.t2n(gw), gw_ref) <= TOL[dtype], (name, dl)
        gws = C.restrict_kernel333_backward(gw, nst)
        assert H.rel_err(H.t2n(gws), oracle.restrict333_backward(gw_ref, nst)) <= TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("cin,cout,nst", [(3, 4, 2), (40, 19, 6), (1, 2, 1)])
@pytest.mark.parametrize("name", CASES)
def test_conv111(name, cin, cout, nst, dtype, oracle, dev):
    from _pyaprwrapper.aprnet import cuda as C
    from _pyaprwrapper.data_containers import APRPtrVector
    a, apr, o = make(name, oracle)
    rng = np.random.RandomState(8)
    for dl in range(0, H.max_dl(a) + 1):
        n = o.number_parts(dl)
        x = rng.rand(cin, n).astype(NP[dtype])
        w = (rng.randn(nst, cout, cin, 1, 1, 1) / np.sqrt(cin)).astype(NP[dtype])
        go = rng.randn(cout, n).astype(NP[dtype])
        ld = torch.full((1,), dl, dtype=torch.int32)
        xt = torch.from_numpy(x).to(dev)[None].contiguous()
        wt = torch.from_numpy(w).to(dev)
        out = C.conv111_forward(APRPtrVector([apr]), xt, wt, ld)
        assert H.rel_err(H.t2n(out[0]), o.conv111_forward(x.astype(np.float64), w.astype(np.float64), dl)) <= TOL[dtype]
        gi, gw = C.conv111_backward(APRPtrVector([apr]), xt, wt, torch.from_numpy(go).to(dev)[None].contiguous(), ld)
        gi_ref, gw_ref = o.conv111_backward(x.astype(np.float64), w.astype(np.float64), go.astype(np.float64), dl)
        assert H.rel_err(H.t2n(gi[0]), gi_ref) <= TOL[dtype]
        assert H.rel_err(H.t2n(gw), gw_ref) <= TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("name", CASES)
def test_maxpool_upsample(name, dtype, oracle, dev):
    from _pyaprwrapper.aprnet import cuda as C
    from _pyaprwrapper.data_containers import APRPtrVector
    a, apr, o = make(name, oracle)
    rng = np.random.RandomState(9)
    for dl in range(0, H.max_dl(a, need=2) + 1):
        n = o.number_parts(dl)
        x = (np.round(rng.rand(5, n) * 4) / 4).astype(NP[dtype])          # many exact ties
        x[0] = 0
        ld = torch.full((1,), dl, dtype=torch.int32)
        xt = torch.from_numpy(x).to(dev)[None].contiguous()
        out, idx = C.maxpool_forward_cuda(APRPtrVector([apr]), xt, ld)
        want, widx = o.maxpool_forward(x, dl)
        assert np.array_equal(H.t2n(out[0]), want)
        assert np.array_equal(H.t2n(idx[0]), widx), (name, dl)            # argmax bit-exact incl. ties
        go = rng.randn(*want.shape).astype(NP[dtype])
        gi = C.maxpool_backward_cuda(APRPtrVector([apr]), torch.from_numpy(go).to(dev)[None].contiguous(), idx, ld)
        assert np.array_equal(H.t2n(gi[0]), o.maxpool_backward(go, widx, dl))
        if dl > 0:
            up = C.upsample_const_forward(APRPtrVector([apr]), xt, ld)
            assert np.array_equal(H.t2n(up[0]), o.upsample_forward(x, dl))
            gu = rng.randn(5, o.number_parts(dl - 1)).astype(NP[dtype])
            gin = C.upsample_const_backward(APRPtrVector([apr]), torch.from_numpy(gu).to(dev)[None].contiguous(), ld)
            assert H.rel_err(H.t2n(gin[0]), o.upsample_backward(gu.astype(np.float64), dl)) <= TOL[dtype]


def test_conv333_fp32_input_gradient_is_deterministic(oracle, dev):
    """The CUDA-core path pulls the cross-level part of the input gradient over the cached edge plan (no atomic adds
    between locations): two calls give bit-identical results, and they agree with the oracle."""
    from _pyaprwrapper.aprnet import cuda as C
    from _pyaprwrapper.data_containers import APRPtrVector
    a, apr, o = make("blob", oracle)
    rng = np.random.RandomState(21)
    cin, cout = 19, 24
    L = a.level_max - a.level_min + 1
    for dl in range(0, H.max_dl(a) + 1):
        n = o.number_parts(dl)
        x = rng.rand(cin, n).astype(np.float32)
        w = (rng.randn(L, cout, cin, 3, 3, 3) / np.sqrt(27 * cin)).astype(np.float32)
        go = rng.randn(cout, n).astype(np.float32)
        ld = torch.full((1,), dl, dtype=torch.int32)
        xt = torch.from_numpy(x).to(dev)[None].contiguous()
        wt = torch.from_numpy(w).to(dev)
        got = torch.from_numpy(go).to(dev)[None].contiguous()
        C.profile_read(); C.profile_enable(True)
        gi1, gw1 = C.conv333_backward(APRPtrVector([apr]), xt, wt, got, ld)
        gi2, gw2 = C.conv333_backward(APRPtrVector([apr]), xt, wt, got, ld)
        torch.cuda.synchronize()
        C.profile_enable(False)
        names = set(k.split(":")[0] for k in C.profile_read())
        assert "conv333_bwd_cross_pull" in names or dl > 0, (dl, names)      # (coarse level deltas of this small APR may have one level only)
        assert torch.equal(gi1, gi2) and torch.equal(gw1, gw2), dl
        gi_ref, _ = o.conv333_backward(x.astype(np.float64), w.astype(np.float64), go.astype(np.float64), dl)
        assert H.rel_err(H.t2n(gi1[0]), gi_ref) <= 1e-5, dl
