"""Reconstruct / SampleParticles (particles <-> dense image) on the GPU against the numpy restatement,
plus the reference's own relational pins: gradcheck and sample(reconstruct(x)) == x
(pyapr/tests/test_aprnet.py:248-285)."""
import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def oracle():
    import apr_oracle
    apr_oracle.build()
    return apr_oracle


def _apr(name):
    import pyapr
    a = H.arrays(name) if name in H.APR_CASES else H.blob_arrays()
    apr = pyapr.apr_from_arrays(a, name)
    apr.init_cuda()
    return a, apr


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-13), (torch.float32, 1e-6)])
@pytest.mark.parametrize("name", ["blob", "odd", "odd2", "plane", "ref_shape"])
def test_image_ops_match_oracle(name, dtype, tol, oracle):
    from _pyaprwrapper.data_containers import APRPtrVector
    from _pyaprwrapper.aprnet import cuda as C
    a, apr = _apr(name)
    o = oracle.OracleAPR(a)
    dev = torch.device("cuda:0")
    rng = np.random.RandomState(1)
    for dl in range(0, H.max_dl(a) + 1):
        n = o.number_parts(dl)
        ld = torch.full((1,), dl, dtype=torch.int32)
        x = rng.rand(3, n)
        xt = torch.from_numpy(x).to(dev, dtype)[None].contiguous()
        img = C.reconstruct_forward(APRPtrVector([apr]), xt, ld)
        want = oracle.reconstruct_forward(a, x, dl)
        assert tuple(img.shape[2:]) == want.shape[1:]
        assert H.rel_err(H.t2n(img[0]), want) <= tol, (name, dl)
        g = rng.randn(*want.shape)
        gt = torch.from_numpy(g).to(dev, dtype)[None].contiguous()
        assert H.rel_err(H.t2n(C.reconstruct_backward(APRPtrVector([apr]), gt, ld)[0]), oracle.reconstruct_backward(a, g, dl, n)) <= tol * 64
        assert H.rel_err(H.t2n(C.sample_particles_forward(APRPtrVector([apr]), gt, ld)[0]), oracle.sample_particles_forward(a, g, dl, n)) <= tol * 64
        assert H.rel_err(H.t2n(C.sample_particles_backward(APRPtrVector([apr]), xt, ld)[0]), oracle.sample_particles_backward(a, x, dl)) <= tol


@pytest.mark.parametrize("name", ["blob", "odd", "ref_shape"])
def test_sample_of_reconstruction_is_identity(name):
    from pyapr.aprnet import cuda as aprnet
    a, apr = _apr(name)
    dev = torch.device("cuda:0")
    recon, sample = aprnet.Reconstruct(), aprnet.SampleParticles()
    for dl in range(0, H.max_dl(a) + 1):
        n = int(apr.number_parts(dl)) if hasattr(apr, "number_parts") else None
        import pyapr
        n = int(pyapr.aprnet.utils.number_particles(apr, dl))
        x = torch.rand(2, 4, n, device=dev, dtype=torch.float64)
        ld = torch.full((2,), dl, dtype=torch.int32)
        y = sample(recon(x, [apr, apr], ld), [apr, apr], ld)
        assert torch.allclose(x, y, rtol=0, atol=1e-13)


@pytest.mark.parametrize("name", ["odd", "cube16"])
def test_image_ops_gradcheck(name):
    import pyapr
    from pyapr.aprnet import cuda as aprnet
    from torch.autograd import gradcheck
    a, apr = _apr(name)
    dev = torch.device("cuda:0")
    dl = min(1, H.max_dl(a))
    n = int(pyapr.aprnet.utils.number_particles(apr, dl))
    ld = torch.full((1,), dl, dtype=torch.int32)
    x = torch.rand(1, 2, n, device=dev, dtype=torch.float64, requires_grad=True)
    assert gradcheck(lambda t: aprnet.Reconstruct()(t, [apr], ld.clone()), (x,), eps=1e-6, atol=1e-7)
    img = aprnet.Reconstruct()(x.detach(), [apr], ld.clone())
    im = torch.rand_like(img).requires_grad_(True)
    assert gradcheck(lambda t: aprnet.SampleParticles()(t, [apr], ld.clone()), (im,), eps=1e-6, atol=1e-7)
