"""Tensor-core 3x3x3 convolution against the CPU oracle at sizes where every persistent block of the
gather kernels walks through many 128-row tiles (accumulator rotation, source-row ring and barrier
parities wrap many times), plus cross-checks of the tensor-core path against the fp32 CUDA-core path
on a multi-million-particle APR where the oracle would take minutes.

APRs: the 128^3 / 200-blob image of the single-layer CPU configuration (about 0.48 M particles, 25 tiles
per block on 148 SMs), a 128x256x256 / 800-blob image (about 1.9 M particles, 100 tiles per block) and
the 256x512x512 / 625-blob image of the block-stack configuration (about 3.3 M particles).

Tolerances (max |a - b| / max |b|): fp32 path 1e-5; tensor-core path 2e-2 for arbitrary inputs.  With
inputs, weights and output gradients that are exact in bf16 the output of a location whose stencil
reads no tree mean (every location of the finest level of the tensor) differs from the float64 oracle
only by the fp32 accumulation order: 2e-5.  Locations next to finer cells read bf16-rounded tree
means (5e-3), the input gradient contains bf16-rounded partial sums (5e-3), and the weight gradient
averages those roundings over all locations (1e-3).
"""
import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu


def bf16_round(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).to(torch.float32).numpy()


@pytest.fixture()
def modes():
    from _pyaprwrapper.aprnet import cuda as C
    yield C
    C.set_conv_precision("fp32")
    assert C.tc_error_flag() == 0, "a tensor-core kernel gave up waiting on a barrier"


def _apr(shape, blobs, seed):
    import pyapr
    a = H.blob_arrays(shape, blobs, seed)
    apr = pyapr.apr_from_arrays(a)
    apr.init_cuda()
    return a, apr


def _finest_rows(a, o, dl):
    """Index range of the locations at the current maximum level (particles and upgraded tree nodes)."""
    cml = a.level_max - dl
    rows_before = 0
    for l in range(a.level_min, cml):
        rows_before += a.dims[l][0] * a.dims[l][1]
    return int(a.row_ptr[rows_before]), o.number_parts(dl)


def _layer_inputs(a, n, cin, cout, seed, exact):
    L = a.level_max - a.level_min + 1
    rng = np.random.RandomState(seed)
    x = rng.rand(cin, n).astype(np.float32)
    w = (rng.randn(L, cout, cin, 3, 3, 3) / np.sqrt(27 * cin)).astype(np.float32)
    go = rng.randn(cout, n).astype(np.float32)
    if exact:
        x, w, go = bf16_round(x), bf16_round(w), bf16_round(go)
    return x, w, go


def _run(C, apr, x, w, go, dl, mode):
    from _pyaprwrapper.data_containers import APRPtrVector
    dev = torch.device("cuda:0")
    C.set_conv_precision(mode)
    ld = torch.full((1,), dl, dtype=torch.int32)
    xt = torch.from_numpy(x).to(dev)[None].contiguous()
    wt = torch.from_numpy(w).to(dev)
    got = torch.from_numpy(go).to(dev)[None].contiguous()
    out = C.conv333_forward(APRPtrVector([apr]), xt, wt, ld)
    gi, gw = C.conv333_backward(APRPtrVector([apr]), xt, wt, got, ld)
    torch.cuda.synchronize()
    return H.t2n(out[0]), H.t2n(gi[0]), H.t2n(gw)


@pytest.mark.parametrize("cin,cout,dl", [(32, 32, 0), (64, 32, 0), (64, 64, 1)])
def test_conv333_against_oracle_many_tiles_per_block(cin, cout, dl, oracle, modes):
    C = modes
    a, apr = _apr((128, 128, 128), 200, 1000)
    o = oracle.OracleAPR(a)
    n = o.number_parts(dl)
    assert n >= 8 * 128 * 148 or dl > 0, "every persistent block must run several tiles"
    x, w, go = _layer_inputs(a, n, cin, cout, 11 + cin + dl, exact=True)
    want = o.conv333_forward(x.astype(np.float64), w.astype(np.float64), dl)
    gi_ref, gw_ref = o.conv333_backward(x.astype(np.float64), w.astype(np.float64), go.astype(np.float64), dl)
    # exact CUDA-core path
    out, gi, gw = _run(C, apr, x, w, go, dl, "fp32")
    assert H.rel_err(out, want) <= 1e-5 and H.rel_err(gi, gi_ref) <= 1e-5 and H.rel_err(gw, gw_ref) <= 1e-5
    # tensor-core path, bf16-exact operands
    out, gi, gw = _run(C, apr, x, w, go, dl, "bf16")
    f0, f1 = _finest_rows(a, o, dl)
    scale = np.abs(want).max()
    assert np.abs(out[:, f0:f1] - want[:, f0:f1]).max() <= 2e-5 * scale, "locations that read no tree mean"
    assert H.rel_err(out, want) <= 5e-3
    assert H.rel_err(gi, gi_ref) <= 5e-3
    assert H.rel_err(gw, gw_ref) <= 1e-3
    # tensor-core path, arbitrary fp32 operands: the bound the bf16 mode has to meet
    x, w, go = _layer_inputs(a, n, cin, cout, 5 + cout, exact=False)
    want = o.conv333_forward(x.astype(np.float64), w.astype(np.float64), dl)
    gi_ref, gw_ref = o.conv333_backward(x.astype(np.float64), w.astype(np.float64), go.astype(np.float64), dl)
    out, gi, gw = _run(C, apr, x, w, go, dl, "bf16")
    assert H.rel_err(out, want) <= 2e-2 and H.rel_err(gi, gi_ref) <= 2e-2 and H.rel_err(gw, gw_ref) <= 2e-2


def test_conv333_against_oracle_two_million_locations(oracle, modes):
    C = modes
    a, apr = _apr((128, 256, 256), 800, 1001)
    o = oracle.OracleAPR(a)
    n = o.number_parts(0)
    assert n >= 1_000_000
    x, w, go = _layer_inputs(a, n, 32, 32, 21, exact=True)
    want = o.conv333_forward(x.astype(np.float64), w.astype(np.float64), 0)
    gi_ref, gw_ref = o.conv333_backward(x.astype(np.float64), w.astype(np.float64), go.astype(np.float64), 0)
    out, gi, gw = _run(C, apr, x, w, go, 0, "bf16")
    f0, f1 = _finest_rows(a, o, 0)
    assert np.abs(out[:, f0:f1] - want[:, f0:f1]).max() <= 2e-5 * np.abs(want).max()
    assert H.rel_err(out, want) <= 5e-3 and H.rel_err(gi, gi_ref) <= 5e-3 and H.rel_err(gw, gw_ref) <= 1e-3
    out, gi, gw = _run(C, apr, x, w, go, 0, "fp32")
    assert H.rel_err(out, want) <= 1e-5 and H.rel_err(gi, gi_ref) <= 1e-5 and H.rel_err(gw, gw_ref) <= 1e-5


@pytest.mark.parametrize("cin,cout,dl", [(32, 32, 0), (64, 32, 0), (64, 64, 1), (128, 128, 2), (256, 128, 2), (128, 256, 3), (16, 16, 0)])
def test_tensor_core_path_matches_fp32_path_at_block_stack_size(cin, cout, dl, modes):
    """Two independent implementations (per-location CUDA-core gather, tile-wise tcgen05 gather GEMM) on the
    APR of the 256x512x512 configuration; bf16-exact operands, so they agree far inside the bf16 bound."""
    C = modes
    a, apr = _apr((256, 512, 512), 625, 2000)
    n = int(apr_number_parts(apr, dl))
    if dl == 0:
        assert n >= 3_000_000
    x, w, go = _layer_inputs(a, n, cin, cout, 31 + cin + cout, exact=True)
    ref = _run(C, apr, x, w, go, dl, "fp32")
    got = _run(C, apr, x, w, go, dl, "bf16")
    assert H.rel_err(got[0], ref[0]) <= 5e-3
    assert H.rel_err(got[1], ref[1]) <= 5e-3
    assert H.rel_err(got[2], ref[2]) <= 1e-3


def apr_number_parts(apr, dl):
    import pyapr
    return pyapr.aprnet.utils.number_particles(apr, dl)


def test_unet_step_bf16_against_fp32_on_config1_apr(modes):
    """One U-Net training step on the 128^3 APR in both modes: loss to 1e-3, gradients of the layers next to
    the loss to 1e-2 (the deep layers of a randomly initialised network amplify any perturbation of the
    activations, bf16 rounding included, so they are compared in direction only)."""
    import pyapr
    from pyapr.aprnet import cuda as ops
    from apr_unet import APRUNet
    C = modes
    a, apr = _apr((128, 128, 128), 200, 1000)
    dev = torch.device("cuda:0")
    n = a.n_particles
    torch.manual_seed(0)
    x = torch.rand(1, 1, n, device=dev)
    y = (torch.rand(1, n, device=dev) > 0.5).long()
    losses, grads = {}, {}
    for mode in ("fp32", "bf16"):
        C.set_conv_precision(mode)
        torch.manual_seed(3)
        net = APRUNet(ops, 1, 2, depth=3, n_filters_base=32).to(dev)
        ld = torch.zeros(1, dtype=torch.int32)
        out = net(x, [apr], ld)
        loss = torch.nn.functional.cross_entropy(out, y)
        loss.backward()
        losses[mode] = float(loss.detach())
        grads[mode] = {k: p.grad.clone() for k, p in net.named_parameters()}
        assert all(torch.isfinite(g).all() for g in grads[mode].values())
        del net, out, loss
    C.set_conv_precision("fp32")
    assert abs(losses["fp32"] - losses["bf16"]) <= 1e-3 * abs(losses["fp32"])
    rel = lambda k: float((grads["fp32"][k] - grads["bf16"][k]).norm() / grads["fp32"][k].norm())
    assert rel("head.weight") <= 1e-2 and rel("head.bias") <= 1e-2
    assert rel("dec.2.blocks.1.conv.weight") <= 5e-2 and rel("dec.2.blocks.0.conv.weight") <= 5e-2
    f32 = torch.cat([g.reshape(-1) for g in grads["fp32"].values()])
    b16 = torch.cat([g.reshape(-1) for g in grads["bf16"].values()])
    assert float(torch.dot(f32, b16) / (f32.norm() * b16.norm())) >= 0.9
