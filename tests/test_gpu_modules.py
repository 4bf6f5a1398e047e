"""The nn.Module / autograd layer on the GPU: numerical gradient checks in float64 (the relations the
reference's own test-suite pins, pyapr/tests/test_aprnet.py:183-245), batches of two APRs at different
level deltas, and a U-Net training step in both arithmetic modes."""
import numpy as np
import pytest
import torch
from torch.autograd import gradcheck

import helpers as H

pytestmark = pytest.mark.gpu


def _batch(names_dls, channels, dtype=torch.float64):
    import pyapr
    aprs, sizes = [], []
    for name, dl in names_dls:
        a = H.arrays(name)
        apr = pyapr.apr_from_arrays(a, name)
        apr.init_cuda()
        aprs.append(apr)
        sizes.append(int(pyapr.aprnet.utils.number_particles(apr, dl)))
    x = torch.rand(len(aprs), channels, max(sizes), dtype=dtype)
    for i, n in enumerate(sizes):
        x[i, :, n:] = 0
    ld = torch.tensor([dl for _, dl in names_dls], dtype=torch.int32)
    return x.cuda().requires_grad_(True), aprs, ld


CASES = [[("odd", 0)], [("cube16", 1)], [("odd", 2), ("cube16", 2)], [("odd2", 0), ("odd", 1)]]


@pytest.mark.parametrize("case", CASES)
def test_conv333_gradcheck(case):
    from pyapr.aprnet import cuda as aprnet
    x, aprs, ld = _batch(case, 2)
    model = aprnet.APRConv(2, 1, kernel_size=(3, 3, 3), nstencils=2).double().cuda()
    assert gradcheck(lambda t: model(t, aprs, ld), (x,), eps=1e-5)
    w = model.weight.detach().clone().requires_grad_(True)
    assert gradcheck(lambda ww: aprnet.conv.Conv333Function.apply(x.detach(), ww, None, aprs, ld), (w,), eps=1e-5)


@pytest.mark.parametrize("case", CASES)
def test_conv111_gradcheck(case):
    from pyapr.aprnet import cuda as aprnet
    x, aprs, ld = _batch(case, 2)
    model = aprnet.APRConv(2, 1, kernel_size=(1, 1, 1), nstencils=6).double().cuda()
    assert gradcheck(lambda t: model(t, aprs, ld), (x,), eps=1e-5)
    w = model.weight.detach().clone().requires_grad_(True)
    assert gradcheck(lambda ww: aprnet.conv.Conv111Function.apply(x.detach(), ww, None, aprs, ld), (w,), eps=1e-5)


@pytest.mark.parametrize("case", CASES[:3])
def test_maxpool_gradcheck(case):
    from pyapr.aprnet import cuda as aprnet
    x, aprs, ld = _batch(case, 2)
    with torch.no_grad():
        x += 10 * torch.arange(x.shape[2], device=x.device, dtype=x.dtype)      # distinct values: no argmax ties
    model = aprnet.MaxPool()
    model.increment_level_deltas = False
    assert gradcheck(lambda t: model(t, aprs, ld), (x,), eps=1e-3)


@pytest.mark.parametrize("case", [[("cube16", 1)], [("odd", 1), ("cube16", 2)]])
def test_upsample_gradcheck(case):
    from pyapr.aprnet import cuda as aprnet
    x, aprs, ld = _batch(case, 2)
    model = aprnet.UpSampleConst()
    model.decrement_level_deltas = False
    assert gradcheck(lambda t: model(t, aprs, ld), (x,), eps=1e-3)


def test_level_deltas_are_shared_state():
    from pyapr.aprnet import cuda as aprnet
    x, aprs, ld = _batch([("cube16", 0)], 3, torch.float32)
    y = aprnet.MaxPool()(x, aprs, ld)
    assert ld.tolist() == [1]
    z = aprnet.UpSampleConst()(y, aprs, ld)
    assert ld.tolist() == [0] and z.shape == x.shape
    with pytest.raises(RuntimeError):
        aprnet.UpSampleConst()(x, aprs, ld)          # level_delta 0 cannot be up-sampled


def test_unet_step_fp32_and_bf16_agree():
    """One forward/backward of the 4-level U-Net in both arithmetic modes.

    At random initialisation with random labels the gradients of the deep layers are extremely sensitive
    to perturbations (an fp32 run whose conv inputs are merely rounded to bf16 moves them by 30-40 %, the
    same as the tensor-core path does), so element-wise agreement is only asserted where the problem is
    well conditioned: the loss, and the gradients of the layers next to the loss.  Deeper layers are
    checked for direction (cosine similarity)."""
    import pyapr
    from pyapr.aprnet import cuda as ops
    from _pyaprwrapper.aprnet import cuda as C
    from apr_unet import APRUNet
    a = H.blob_arrays((48, 64, 64), 8, 5)
    apr = pyapr.apr_from_arrays(a)
    apr.init_cuda()
    dev = torch.device("cuda:0")
    n = a.n_particles
    torch.manual_seed(0)
    x = torch.rand(1, 1, n, device=dev)
    y = (torch.rand(1, n, device=dev) > 0.5).long()
    losses, grads = {}, {}
    for mode in ("fp32", "bf16"):
        C.set_conv_precision(mode)
        try:
            torch.manual_seed(3)
            net = APRUNet(ops, 1, 2, depth=3, n_filters_base=8).to(dev)
            ld = torch.zeros(1, dtype=torch.int32)
            out = net(x, [apr], ld)
            loss = torch.nn.functional.cross_entropy(out, y)
            loss.backward()
            assert ld.tolist() == [0]
            losses[mode] = float(loss.detach())
            grads[mode] = {k: p.grad.clone() for k, p in net.named_parameters()}
            assert all(torch.isfinite(g).all() for g in grads[mode].values())
        finally:
            C.set_conv_precision("fp32")
    assert C.tc_error_flag() == 0
    assert abs(losses["fp32"] - losses["bf16"]) <= 1e-3 * abs(losses["fp32"])
    rel = lambda k: float((grads["fp32"][k] - grads["bf16"][k]).norm() / grads["fp32"][k].norm())
    assert rel("head.weight") <= 1e-2 and rel("head.bias") <= 1e-2
    assert rel("dec.2.blocks.1.conv.weight") <= 1e-1 and rel("dec.2.blocks.0.conv.weight") <= 1e-1
    f32 = torch.cat([g.reshape(-1) for g in grads["fp32"].values()])
    b16 = torch.cat([g.reshape(-1) for g in grads["bf16"].values()])
    assert float(torch.dot(f32, b16) / (f32.norm() * b16.norm())) >= 0.85


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-10), (torch.float32, 2e-5)])
@pytest.mark.parametrize("b,c,g,n", [(1, 8, 8, 5000), (2, 12, 4, 3001), (1, 32, 32, 70001), (3, 6, 1, 777)])
def test_groupnorm_relu_matches_torch(b, c, g, n, dtype, tol):
    """Fused GroupNorm + ReLU against torch.nn.GroupNorm followed by ReLU: output and all gradients."""
    from pyapr.aprnet import cuda as aprnet
    dev = torch.device("cuda:0")
    torch.manual_seed(1)
    x = (torch.randn(b, c, n, dtype=dtype, device=dev) * 3 + 1).requires_grad_(True)
    ref = torch.nn.GroupNorm(g, c).to(dev, dtype)
    mine = aprnet.GroupNormReLU(g, c).to(dev, dtype)
    with torch.no_grad():
        ref.weight.uniform_(0.5, 1.5); ref.bias.uniform_(-0.5, 0.5)
        mine.weight.copy_(ref.weight); mine.bias.copy_(ref.bias)
    go = torch.randn(b, c, n, dtype=dtype, device=dev)
    y_ref = torch.relu(ref(x)); y_ref.backward(go)
    gx_ref, gw_ref, gb_ref = x.grad.clone(), ref.weight.grad.clone(), ref.bias.grad.clone()
    x.grad = None
    y = mine(x); y.backward(go)
    rel = lambda p, q: float((p - q).abs().max() / q.abs().max().clamp_min(1e-30))
    assert rel(y, y_ref) <= tol
    assert rel(x.grad, gx_ref) <= tol * 20
    assert rel(mine.weight.grad, gw_ref) <= tol * 20 and rel(mine.bias.grad, gb_ref) <= tol * 20


def test_groupnorm_relu_gradcheck():
    from pyapr.aprnet import cuda as aprnet
    dev = torch.device("cuda:0")
    torch.manual_seed(2)
    x = (torch.randn(2, 4, 50, dtype=torch.float64, device=dev) + 0.3).requires_grad_(True)
    m = aprnet.GroupNormReLU(2, 4).double().to(dev)
    assert gradcheck(lambda t: m(t), (x,), eps=1e-6, atol=1e-6)


def test_precision_is_a_per_module_option():
    """`APRConv(precision=...)` overrides the process-wide setting for that layer only, forward and backward."""
    import pyapr
    from pyapr.aprnet import cuda as aprnet
    from _pyaprwrapper.aprnet import cuda as C
    a = H.blob_arrays()
    apr = pyapr.apr_from_arrays(a)
    apr.init_cuda()
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    x = torch.rand(1, 16, a.n_particles, device=dev)
    go = torch.randn(1, 24, a.n_particles, device=dev)
    ld = torch.zeros(1, dtype=torch.int32)
    convs = {p: aprnet.APRConv(16, 24, nstencils=2, precision=p).to(dev) for p in (None, "fp32", "bf16")}
    for c in convs.values():
        c.load_state_dict(convs[None].state_dict())
    res = {}
    assert C.get_conv_precision() == "fp32"
    for mode in ("fp32", "bf16"):
        C.set_conv_precision(mode)
        try:
            for p, c in convs.items():
                c.zero_grad(set_to_none=True)
                xi = x.clone().requires_grad_(True)
                c(xi, [apr], ld).backward(go)
                res[(mode, p)] = (xi.grad.clone(), c.weight.grad.clone())
        finally:
            C.set_conv_precision("fp32")
    same = lambda u, v: all(torch.equal(s, t) for s, t in zip(u, v))
    # the fp32 input gradient scatters its cross-level part with atomic adds: equal up to the summation order
    close = lambda u, v: all(float((s - t).abs().max()) <= 1e-5 * float(t.abs().max()) for s, t in zip(u, v))
    assert close(res[("fp32", "fp32")], res[("bf16", "fp32")]) and close(res[("fp32", None)], res[("fp32", "fp32")])       # pinned to fp32
    assert same(res[("fp32", "bf16")], res[("bf16", "bf16")]) and same(res[("bf16", None)], res[("bf16", "bf16")])       # pinned to bf16
    assert not close(res[("fp32", "fp32")], res[("fp32", "bf16")])
    rel = float((res[("fp32", "fp32")][1] - res[("fp32", "bf16")][1]).abs().max() / res[("fp32", "fp32")][1].abs().max())
    assert rel <= 2e-2
    assert C.tc_error_flag() == 0
