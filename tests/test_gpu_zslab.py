"""One APR cut into two z-slabs on two GPUs: a U-Net training step over the slab modules (halo exchange over NCCL
point-to-point, GroupNorm sums and weight gradients all-reduced) equals the step on the whole APR on one GPU.

Needs two CUDA devices; skipped otherwise.  The ranks are child processes; NVLS is switched off for them."""
import os
import sys

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHAPE, BLOBS, SEED = (64, 96, 80), 14, 33


def _rank(rank, world, port, mode, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    for p in (os.path.join(ROOT, "apr-cnn_b200"), os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import pyapr
        from _pyaprwrapper.aprnet import cuda as C
        from pyapr.sharding import zslab_plan, allreduce_gradients
        from pyapr.aprnet.cuda.sharded import Shard, make_ops, sharded_cross_entropy
        from apr_unet import APRUNet
        C.set_conv_precision(mode)
        a = H.blob_arrays(SHAPE, BLOBS, SEED)
        plan = zslab_plan(a, rank, world, max_level_delta=3)
        apr = pyapr.apr_from_arrays(plan.local)
        apr.init_cuda()
        shard = Shard(plan, dev)
        rng = np.random.RandomState(1)
        xg = rng.rand(a.n_particles).astype(np.float32)
        yg = (rng.rand(a.n_particles) > 0.5).astype(np.int64)
        x = torch.from_numpy(xg[plan.l2g_particles])[None, None].contiguous().to(dev)
        y = torch.from_numpy(yg[plan.l2g_particles])[None].to(dev)
        torch.manual_seed(3)
        net = APRUNet(make_ops(shard), 1, 2, depth=3, n_filters_base=8).to(dev)
        state = {k: v.detach().cpu().clone() for k, v in net.state_dict().items()}
        out = net(x, [apr])
        loss, total = sharded_cross_entropy(out, y, shard)
        loss.backward()
        params = list(net.parameters())
        allreduce_gradients(params, world, average=False)
        torch.cuda.synchronize()
        owned = torch.from_numpy(plan.owned_particles)
        q.put((rank, dict(loss=float(total), grads={k: p.grad.detach().cpu().numpy() for k, p in net.named_parameters()},
                          out=out.detach().cpu()[0][:, owned].numpy(), l2g=plan.l2g_particles[plan.owned_particles],
                          state=state if rank == 0 else None, err=C.tc_error_flag())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,tol_out,tol_grad", [("fp32", 2e-4, 2e-3), ("bf16", 5e-2, None)])
def test_two_slab_unet_step_equals_single_gpu_step(mode, tol_out, tol_grad):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + (os.getpid() % 1000)
    procs = [ctx.Process(target=_rank, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=900) for _ in procs)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    import pyapr
    from pyapr.aprnet import cuda as ops
    from _pyaprwrapper.aprnet import cuda as C
    from apr_unet import APRUNet
    dev = torch.device("cuda:0")
    a = H.blob_arrays(SHAPE, BLOBS, SEED)
    apr = pyapr.apr_from_arrays(a)
    apr.init_cuda()
    rng = np.random.RandomState(1)
    xg = rng.rand(a.n_particles).astype(np.float32)
    yg = (rng.rand(a.n_particles) > 0.5).astype(np.int64)
    C.set_conv_precision(mode)
    try:
        net = APRUNet(ops, 1, 2, depth=3, n_filters_base=8).to(dev)
        net.load_state_dict(got[0]["state"])
        out = net(torch.from_numpy(xg)[None, None].to(dev), [apr])
        loss = torch.nn.functional.cross_entropy(out, torch.from_numpy(yg)[None].to(dev))
        loss.backward()
    finally:
        C.set_conv_precision("fp32")
    ref_out = out.detach().cpu().numpy()[0]
    for r in range(2):
        assert got[r]["err"] == 0
        assert H.rel_err(got[r]["out"], ref_out[:, got[r]["l2g"]]) <= tol_out, (mode, r)
        assert abs(got[r]["loss"] - float(loss)) <= (1e-5 if mode == "fp32" else 2e-3) * abs(float(loss))
    if tol_grad is not None:
        for k, p in net.named_parameters():
            g = p.grad.detach().cpu().numpy()
            assert H.rel_err(got[0]["grads"][k], g) <= tol_grad, k
            assert np.array_equal(got[0]["grads"][k], got[1]["grads"][k])        # the all-reduce leaves the same sums on both ranks
