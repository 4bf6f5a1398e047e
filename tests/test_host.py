"""Host-side logic that needs no GPU: the APR container, particle counting, pickling, the error
behaviour of the operator functions for bad inputs, and the multi-rank helpers (gloo, world size 2)."""
import os
import pickle
import sys

import numpy as np
import pytest
import torch

import helpers as H


def test_apr_container_and_counts(oracle):
    import pyapr
    for name in H.APR_CASES:
        a = H.arrays(name)
        apr = pyapr.apr_from_arrays(a, name)
        o = oracle.OracleAPR(a)
        assert apr.total_number_particles() == a.n_particles
        assert apr.total_number_tree_particles() == a.n_tree
        assert apr.level_max() == a.level_max and apr.level_min() == a.level_min
        assert apr.shape() == tuple(a.shape)
        assert (apr.org_dims(0), apr.org_dims(1), apr.org_dims(2)) == (a.shape[2], a.shape[1], a.shape[0])
        for l in range(a.level_max + 1):
            assert (apr.z_num(l), apr.x_num(l), apr.y_num(l)) == tuple(a.dims[l])
        for dl in range(0, a.level_max - a.level_min + 1):
            assert pyapr.aprnet.utils.number_particles(apr, dl) == o.number_parts(dl)
            assert pyapr.aprnet.utils.number_parts(apr, dl) == o.number_parts(dl)
            if dl > 0:
                assert pyapr.aprnet.utils.number_particles_after_upsampling(apr, dl) == o.number_parts(dl - 1)
            if dl < a.level_max - a.level_min:
                assert pyapr.aprnet.utils.number_particles_after_pooling(apr, dl) == o.number_parts(dl + 1)


def test_apr_pickle_roundtrip():
    import pyapr
    a = H.arrays("odd")
    apr = pyapr.apr_from_arrays(a, "pickled")
    b = pickle.loads(pickle.dumps(apr))
    assert b.name == "pickled" and b.total_number_particles() == a.n_particles
    assert b.shape() == apr.shape() and b.level_max() == apr.level_max()
    assert pyapr.aprnet.utils.number_particles(b, 1) == pyapr.aprnet.utils.number_particles(apr, 1)


def test_bad_arrays_are_rejected():
    import pyapr
    a = H.arrays("odd")
    apr = pyapr.APR()
    with pytest.raises(ValueError):
        apr.init_from_arrays(13, 9, 21, a.row_ptr[:-1], a.y, a.tree_row_ptr, a.tree_y)
    with pytest.raises(ValueError):
        apr.init_from_arrays(13, 9, 21, a.row_ptr, a.y[:-1], a.tree_row_ptr, a.tree_y)


def test_operator_errors_without_gpu():
    """Same conditions and exception type as the reference wrappers (pyapr/aprnet/cuda/src/common.hpp:14-17)."""
    import pyapr
    from pyapr.aprnet import cuda as aprnet
    a = H.arrays("odd")
    apr = pyapr.apr_from_arrays(a)
    x = torch.rand(1, 2, a.n_particles)
    ld = torch.zeros(1, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        aprnet.APRConv(2, 3)(x, [apr], ld)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        aprnet.APRConv(2, 3, kernel_size=(1, 1, 1))(x, [apr], ld)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        aprnet.MaxPool()(x, [apr], ld)
    with pytest.raises(RuntimeError):
        aprnet.UpSampleConst()(x, [apr], ld)
    with pytest.raises(AssertionError):
        aprnet.APRConv(2, 3, kernel_size=(5, 5, 5))
    m = aprnet.APRConv(4, 6, nstencils=3)
    assert tuple(m.weight.shape) == (3, 6, 4, 3, 3, 3) and tuple(m.bias.shape) == (6,)


def test_reference_unet_builds_on_these_modules():
    """The reference's own U-Net source files construct unchanged on top of pyapr.aprnet.cuda.

    The files are loaded directly (the package __init__ also pulls in the stardist models, which need
    the absent `stardist` dependency)."""
    import build_ref
    base = os.path.join(build_ref.reference_root(), "apr_models", "apr_models", "unet")
    if not os.path.isdir(base):
        pytest.skip("reference checkout not present")
    import importlib.util
    import types
    import pyapr  # noqa: F401
    pkg = types.ModuleType("_ref_unet_pkg")
    pkg.__path__ = [base]
    sys.modules["_ref_unet_pkg"] = pkg
    try:
        for name in ("unet_parts", "unet_model"):
            spec = importlib.util.spec_from_file_location("_ref_unet_pkg." + name, os.path.join(base, name + ".py"))
            mod = importlib.util.module_from_spec(spec)
            sys.modules["_ref_unet_pkg." + name] = mod
            spec.loader.exec_module(mod)
        net = sys.modules["_ref_unet_pkg.unet_model"].APRUNet(1, 2, depth=3, n_filters_base=8)
    finally:
        for k in [k for k in sys.modules if k.startswith("_ref_unet_pkg")]:
            del sys.modules[k]
    from apr_unet import APRUNet as Mine
    from pyapr.aprnet import cuda as ops
    mine = Mine(ops, 1, 2, depth=3, n_filters_base=8)
    assert sum(p.numel() for p in net.parameters()) == sum(p.numel() for p in mine.parameters())
    assert sorted(tuple(p.shape) for p in net.parameters()) == sorted(tuple(p.shape) for p in mine.parameters())


def test_shard_indices_partition_and_balance():
    from pyapr.sharding import shard_indices
    n, world = 64, 8
    seen = sorted(i for r in range(world) for i in shard_indices(n, r, world))
    assert seen == list(range(n))
    w = list(np.random.RandomState(0).randint(50, 400, size=n))
    parts = [shard_indices(n, r, world, w) for r in range(world)]
    assert sorted(i for p in parts for i in p) == list(range(n))
    loads = [sum(w[i] for i in p) for p in parts]
    assert max(loads) - min(loads) <= max(w)


def _gloo_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "apr-cnn_b200", "pyapr"))
    import sharding
    torch.manual_seed(0)
    lin = torch.nn.Linear(5, 3)
    x = torch.full((4, 5), float(rank + 1))
    lin(x).sum().backward()
    local = [p.grad.clone() for p in lin.parameters()]
    sharding.allreduce_gradients(list(lin.parameters()), world)
    q.put((rank, [g.tolist() for g in local], [p.grad.tolist() for p in lin.parameters()],
           sharding.shard_indices(5, rank, world)))
    dist.destroy_process_group()


def test_gradient_allreduce_two_ranks_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, l0, a0, s0), (r1, l1, a1, s1) = res
    assert s0 == [0, 2, 4] and s1 == [1, 3]
    for g0, g1, m0, m1 in zip(l0, l1, a0, a1):
        want = (np.array(g0) + np.array(g1)) / 2
        assert np.allclose(m0, want) and np.allclose(m1, want)


def test_apr_file_round_trip_and_libapr_conversion(tmp_path):
    """write_apr / read_apr keep the access arrays bit for bit; the LibAPR-layout conversion reproduces them."""
    import pyapr
    from pyapr import io
    a = H.arrays("odd2")
    feat = np.random.RandomState(0).rand(3, a.n_particles).astype(np.float32)
    path = str(tmp_path / "odd2.npz")
    io.write_apr(path, a, name="odd2", particle_data=feat)
    b, name, data = io.read_apr(path)
    assert name == "odd2" and b.shape == a.shape and b.level_max == a.level_max and b.dims == a.dims
    for f in ("row_ptr", "y", "tree_row_ptr", "tree_y"):
        assert np.array_equal(getattr(a, f), getattr(b, f))
    assert np.array_equal(data, feat)
    apr = pyapr.apr_from_arrays(b)
    assert apr.total_number_particles() == a.n_particles
    # LibAPR layout: rows of ALL levels from 0 (empty below level_min), row ends instead of CSR pointers
    rows_below = sum(a.dims[l][0] * a.dims[l][1] for l in range(0, a.level_min))
    level_xz, off = [], 0
    for l in range(a.level_max + 1):
        level_xz.append(off)
        off += a.dims[l][0] * a.dims[l][1]
    xz_end = np.concatenate([np.zeros(rows_below, dtype=np.int64), a.row_ptr[1:]])
    c = io.from_libapr_arrays(a.shape, a.level_min, a.level_max, level_xz, xz_end, a.y, level_xz, a.tree_row_ptr[1:], a.tree_y)
    for f in ("row_ptr", "y", "tree_row_ptr", "tree_y"):
        assert np.array_equal(getattr(a, f), getattr(c, f))
    bad = io.AprArrays(shape=a.shape, level_max=a.level_max, level_min=a.level_min, dims=a.dims, row_ptr=a.row_ptr[:-1], y=a.y,
                       tree_row_ptr=a.tree_row_ptr, tree_y=a.tree_y)
    with pytest.raises(ValueError):
        io.check_arrays(bad)
