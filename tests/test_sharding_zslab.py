"""One APR cut into z-slabs: the partitioner, the halo lists and the sharded layer logic, on CPU ranks.

The structure checks compare each slab's own access structure (built by `pyapr.sharding.zslab_plan`) with the
whole APR through the oracle's neighbour tables.  The operator checks run the sharded 3x3x3 convolution /
GroupNorm Functions of `pyapr.aprnet.cuda.sharded` on `gloo` ranks over a numpy backend that is first pinned
to the oracle's convolution, and compare outputs and gradients with the unsharded oracle on the whole APR.
"""
import os
import sys

import numpy as np
import pytest
import torch

import helpers as H

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _arrays():
    return H.blob_arrays((64, 64, 48), 10, 21)


def _plans(a, world, mld=1):
    from pyapr.sharding import zslab_plan
    return [zslab_plan(a, r, world, max_level_delta=mld) for r in range(world)]


@pytest.mark.parametrize("world", [2, 3, 4])
def test_slabs_partition_the_particles_and_halo_lists_pair_up(world):
    a = _arrays()
    plans = _plans(a, world)
    owned = np.concatenate([p.l2g_particles[p.owned_particles] for p in plans])
    assert np.array_equal(np.sort(owned), np.arange(a.n_particles))              # every particle has exactly one owner
    assert all(c % plans[0].align == 0 for c in plans[0].cuts[1:-1])
    for dl in plans[0].lists:
        assert sum(len(p.lists[dl].ghost_x) == 0 for p in plans) == 0 or world == 1
        n_owned = sum(p.lists[dl].n_local - len(p.lists[dl].ghost_x) for p in plans)
        assert n_owned == plans[0].lists[dl].n_global
        for r, p in enumerate(plans):
            for q in p.neighbours:
                L, M = p.lists[dl], plans[q].lists[dl]
                assert len(L.send_x[q]) == len(M.recv_x[r]) and len(L.send_t[q]) == len(M.recv_t[r])
                if dl == 0:      # the feature vector is the particle vector: the two sides name the same global particles
                    assert np.array_equal(p.l2g_particles[L.send_x[q]], plans[q].l2g_particles[M.recv_x[r]])
                assert np.array_equal(p.l2g_tree[L.send_t[q]], plans[q].l2g_tree[M.recv_t[r]])


@pytest.mark.parametrize("world", [2, 3])
def test_slab_structure_reproduces_the_global_neighbourhoods(world, oracle):
    """For every owned location the 27 neighbour entries of the slab's own table name the same global particles /
    tree nodes as the table of the whole APR."""
    a = _arrays()
    og = oracle.OracleAPR(a)
    for dl in (0, 1):
        gtab = og.nbr_table(dl)
        n_part_g = a.n_particles if dl == 0 else None
        for p in _plans(a, world):
            ol = oracle.OracleAPR(p.local)
            L = p.lists[dl]
            assert ol.number_parts(dl) == L.n_local and ol.tree_size(dl) == L.t_local
            ltab = ol.nbr_table(dl)
            # local feature index -> global feature index
            cml = a.level_max - dl
            n_part_l = L.n_local if dl == 0 else L.n_local - (ol.number_parts(dl) - _particles_upto(p.local, cml))
            l2g_x = np.empty(L.n_local, dtype=np.int64)
            l2g_x[:n_part_l] = p.l2g_particles[:n_part_l]
            if dl > 0:
                t0 = ol.tree_size(dl)                           # first local tree node of level cml
                l2g_x[n_part_l:] = p.l2g_tree[t0:t0 + (L.n_local - n_part_l)] + og.tree_offset(cml)
            owned = np.ones(L.n_local, dtype=bool)
            owned[L.ghost_x] = False
            loc = ltab[:, owned]
            glo = gtab[:, l2g_x[owned]]
            mapped = np.full(loc.shape, -1, dtype=np.int64)
            pos = loc >= 0
            mapped[pos] = l2g_x[loc[pos]]
            tre = loc <= -2
            mapped[tre] = -2 - p.l2g_tree[-2 - loc[tre]]
            assert np.array_equal(mapped, glo.astype(np.int64)), (world, dl, p.rank)


def _particles_upto(a, level):
    rows = 0
    for l in range(a.level_min, level + 1):
        rows += a.dims[l][0] * a.dims[l][1]
    return int(a.row_ptr[rows])


# ---- numpy operator backend over the oracle's tables -------------------------------------------------------
class _CpuApr:
    def __init__(self, arrays, oracle):
        self.arrays, self.o = arrays, oracle.OracleAPR(arrays)

    def level_max(self):
        return self.arrays.level_max

    def level_min(self):
        return self.arrays.level_min


class NumpyBackend:
    """3x3x3 convolution with given tree means, from the neighbour table: out[:, p] = sum_tap W[slot(p)][:, :, tap] v[:, nbr[tap, p]]."""

    def __init__(self, oracle):
        self.oracle = oracle

    def _slots(self, apr, dl, num_slots):
        a, o = apr.arrays, apr.o
        cml = a.level_max - dl
        n = o.number_parts(dl)
        slot = np.zeros(n, dtype=np.int64)
        for l in range(a.level_min, cml + 1):
            b, e = _particles_upto(a, l - 1) if l > a.level_min else 0, _particles_upto(a, l)
            slot[b:e] = min(cml - l, num_slots - 1)
        return slot

    def _vals_index(self, apr, dl, n, t):
        tab = apr.o.nbr_table(dl).astype(np.int64)
        idx = np.where(tab >= 0, tab, np.where(tab == -1, n + t, n + (-2 - tab)))
        return idx

    def restrict_forward(self, w, L):
        return torch.from_numpy(self.oracle.restrict333_forward(w.detach().numpy(), L))

    def restrict_backward(self, gw, S):
        return torch.from_numpy(self.oracle.restrict333_backward(gw.numpy(), S))

    def fill_tree(self, aprs, x, ld):
        return torch.from_numpy(aprs[0].o.fill_tree_mean(x[0].detach().numpy(), int(ld[0])))[None].contiguous()

    def conv_forward(self, aprs, x, tree, w, ld):
        dl = int(ld[0]); apr = aprs[0]
        xn, tn, wn = x[0].detach().numpy(), tree[0].numpy(), w.detach().numpy().reshape(w.shape[0], w.shape[1], w.shape[2], 27)
        n, t = xn.shape[1], tn.shape[1]
        vals = np.concatenate([xn, tn, np.zeros((xn.shape[0], 1))], axis=1)
        idx, slot = self._vals_index(apr, dl, n, t), self._slots(apr, dl, w.shape[0])
        out = np.zeros((w.shape[1], n))
        for s in np.unique(slot):
            m = slot == s
            for tap in range(27):
                out[:, m] += wn[s, :, :, tap] @ vals[:, idx[tap, m]]
        return torch.from_numpy(out)[None], torch.empty(0, dtype=torch.uint8)

    def conv_backward(self, aprs, x, tree, kept, w, go, ld, need_gi):
        dl = int(ld[0]); apr = aprs[0]
        xn, tn, gon = x[0].detach().numpy(), tree[0].numpy(), go[0].numpy()
        wn = w.detach().numpy().reshape(w.shape[0], w.shape[1], w.shape[2], 27)
        n, t = xn.shape[1], tn.shape[1]
        vals = np.concatenate([xn, tn, np.zeros((xn.shape[0], 1))], axis=1)
        idx, slot = self._vals_index(apr, dl, n, t), self._slots(apr, dl, w.shape[0])
        gvals = np.zeros_like(vals)
        gw = np.zeros_like(wn)
        for s in np.unique(slot):
            m = np.nonzero(slot == s)[0]
            for tap in range(27):
                gw[s, :, :, tap] += gon[:, m] @ vals[:, idx[tap, m]].T
                np.add.at(gvals, (slice(None), idx[tap, m]), wn[s, :, :, tap].T @ gon[:, m])
        gi = torch.from_numpy(gvals[:, :n].copy())[None]
        gt = torch.from_numpy(gvals[:, n:n + t].copy())[None]
        return gi, gt, torch.from_numpy(gw.reshape(w.shape))

    def tree_adjoint_(self, aprs, gi, gtree, ld):
        r = aprs[0].o.fill_tree_mean_backward(gi[0].numpy(), gtree[0].numpy(), int(ld[0]))
        gi[0].copy_(torch.from_numpy(r))

    def gn_row_sums(self, x):
        v = x[0].double()
        return torch.stack([v.sum(1), (v * v).sum(1)], dim=1)

    def gn_apply(self, x, gamma, beta, mean, rstd, groups, relu):
        C = x.shape[1]
        mu, rs = mean.repeat_interleave(C // groups)[None, :, None], rstd.repeat_interleave(C // groups)[None, :, None]
        y = (x - mu) * rs * gamma[None, :, None] + beta[None, :, None]
        return torch.relu(y) if relu else y

    def _dy_eff(self, x, gy, gamma, beta, mean, rstd, groups, relu):
        C = x.shape[1]
        mu, rs = mean.repeat_interleave(C // groups)[None, :, None], rstd.repeat_interleave(C // groups)[None, :, None]
        xh = (x - mu) * rs
        d = gy.clone()
        if relu:
            d[(xh * gamma[None, :, None] + beta[None, :, None]) <= 0] = 0
        return d, xh, rs

    def gn_backward_row_sums(self, x, gy, gamma, beta, mean, rstd, groups, relu):
        d, xh, _ = self._dy_eff(x, gy, gamma, beta, mean, rstd, groups, relu)
        return torch.stack([d[0].double().sum(1), (d[0].double() * xh[0].double()).sum(1)], dim=1)

    def gn_backward_apply(self, x, gy, gamma, beta, mean, rstd, terms, groups, relu):
        C = x.shape[1]
        d, xh, rs = self._dy_eff(x, gy, gamma, beta, mean, rstd, groups, relu)
        mA = terms[:, 0].repeat_interleave(C // groups)[None, :, None]
        mB = terms[:, 1].repeat_interleave(C // groups)[None, :, None]
        return rs * (d * gamma[None, :, None] - mA - xh * mB)


def test_numpy_backend_is_the_oracle_convolution(oracle):
    """The table-driven numpy convolution used by the rank tests equals the oracle's operator (forward, both gradients)."""
    a = _arrays()
    apr = _CpuApr(a, oracle)
    B = NumpyBackend(oracle)
    rng = np.random.RandomState(0)
    L = a.level_max - a.level_min + 1
    for dl in (0, 1):
        n = apr.o.number_parts(dl)
        x = torch.from_numpy(rng.rand(1, 3, n)); w = torch.from_numpy(rng.randn(L, 4, 3, 3, 3, 3)); go = torch.from_numpy(rng.randn(1, 4, n))
        ld = torch.tensor([dl], dtype=torch.int32)
        tree = B.fill_tree([apr], x, ld)
        out, _ = B.conv_forward([apr], x, tree, w, ld)
        assert H.rel_err(out[0].numpy(), apr.o.conv333_forward(x[0].numpy(), w.numpy(), dl)) <= 1e-12
        gi, gt, gw = B.conv_backward([apr], x, tree, None, w, go, ld, True)
        B.tree_adjoint_([apr], gi, gt, ld)
        gi_ref, gw_ref = apr.o.conv333_backward(x[0].numpy(), w.numpy(), go[0].numpy(), dl)
        assert H.rel_err(gi[0].numpy(), gi_ref) <= 1e-12 and H.rel_err(gw.numpy(), gw_ref) <= 1e-12


def _rank_main(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    for p in (os.path.join(ROOT, "apr-cnn_b200"), os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import apr_oracle
        apr_oracle.build()
        import pyapr  # noqa: F401
        from pyapr.sharding import zslab_plan, allreduce_gradients
        from pyapr.aprnet.cuda.sharded import Shard, ShardedConv333Function, ShardedGroupNormReLUFunction
        a = _arrays()
        plan = zslab_plan(a, rank, world, max_level_delta=1)
        shard = Shard(plan, torch.device("cpu"), backend=NumpyBackend(apr_oracle))
        apr = _CpuApr(plan.local, apr_oracle)
        rng = np.random.RandomState(5)
        L = a.level_max - a.level_min + 1
        res = {}
        for dl in (0, 1):
            Lst = plan.lists[dl]
            og = apr_oracle.OracleAPR(a)
            ng = og.number_parts(dl)
            xg = rng.rand(1, 3, ng)
            w1 = torch.from_numpy(rng.randn(2, 4, 3, 3, 3, 3) / 9).requires_grad_(True)
            w2 = torch.from_numpy(rng.randn(2, 2, 4, 3, 3, 3) / 9).requires_grad_(True)
            gam = torch.from_numpy(rng.rand(4) + 0.5).requires_grad_(True)
            bet = torch.from_numpy(rng.rand(4) - 0.5).requires_grad_(True)
            target = rng.randn(1, 2, ng)
            # local feature index -> global feature index (particles, then the pooled tree nodes)
            n_part_l = _particles_upto(plan.local, a.level_max - dl)
            l2g = np.empty(Lst.n_local, dtype=np.int64)
            l2g[:n_part_l] = plan.l2g_particles[:n_part_l]
            if dl > 0:
                t0 = apr.o.tree_size(dl)
                l2g[n_part_l:] = plan.l2g_tree[t0:t0 + Lst.n_local - n_part_l] + og.tree_offset(a.level_max - dl)
            owned = np.ones(Lst.n_local, dtype=bool); owned[Lst.ghost_x] = False
            x = torch.from_numpy(xg[:, :, l2g].copy())
            x[:, :, torch.from_numpy(~owned)] = 777.0            # halo entries start with junk: the exchange must fix them
            x.requires_grad_(True)
            ld = torch.tensor([dl], dtype=torch.int32)
            h = ShardedConv333Function.apply(x, w1, None, [apr], ld, shard)
            h = ShardedGroupNormReLUFunction.apply(h, gam, bet, 2, 1e-5, True, shard)
            y = ShardedConv333Function.apply(h, w2, None, [apr], ld, shard)
            tl = torch.from_numpy(target[:, :, l2g].copy())
            loss = (((y - tl) ** 2) * torch.from_numpy(owned)[None, None, :]).sum()
            loss.backward()
            params = [w1, w2, gam, bet]
            allreduce_gradients(params, world, average=False)
            tot = loss.detach().clone(); dist.all_reduce(tot)
            res[dl] = dict(l2g=l2g[owned], y=y.detach().numpy()[0][:, owned], gx=x.grad.numpy()[0][:, owned], loss=float(tot),
                           grads=[p.grad.numpy().copy() for p in params], xg=xg, target=target,
                           params=[p.detach().numpy().copy() for p in params], halo_gx=float(np.abs(x.grad.numpy()[0][:, ~owned]).max()))
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_layers_match_the_whole_apr_on_gloo_ranks(world, oracle):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() % 2000) + world
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=600) for _ in procs)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    a = _arrays()
    apr = _CpuApr(a, oracle)
    B = NumpyBackend(oracle)
    for dl in (0, 1):
        r0 = got[0][dl]
        w1, w2, gam, bet = [torch.from_numpy(v).requires_grad_(True) for v in r0["params"]]
        x = torch.from_numpy(r0["xg"]).requires_grad_(True)
        ld = torch.tensor([dl], dtype=torch.int32)
        L = a.level_max - a.level_min + 1

        class Conv(torch.autograd.Function):                  # the unsharded operator: the oracle on the whole APR
            @staticmethod
            def forward(ctx, xx, ww):
                we = oracle.restrict333_forward(ww.detach().numpy(), L)
                ctx.save_for_backward(xx, ww); ctx.we = we
                return torch.from_numpy(apr.o.conv333_forward(xx[0].detach().numpy(), we, dl))[None]

            @staticmethod
            def backward(ctx, go):
                xx, ww = ctx.saved_tensors
                gi, gwe = apr.o.conv333_backward(xx[0].detach().numpy(), ctx.we, go[0].numpy(), dl)
                return torch.from_numpy(gi)[None], torch.from_numpy(oracle.restrict333_backward(gwe, ww.shape[0]))

        h = torch.relu(torch.nn.functional.group_norm(Conv.apply(x, w1), 2, gam, bet, 1e-5))
        y = Conv.apply(h, w2)
        loss = ((y - torch.from_numpy(r0["target"])) ** 2).sum()
        loss.backward()
        for r in range(world):
            res = got[r][dl]
            assert H.rel_err(res["y"], y.detach().numpy()[0][:, res["l2g"]]) <= 1e-10, (world, dl, r)
            assert H.rel_err(res["gx"], x.grad.numpy()[0][:, res["l2g"]]) <= 1e-9, (world, dl, r)
            assert res["halo_gx"] == 0.0
            assert abs(res["loss"] - float(loss)) <= 1e-10 * abs(float(loss))
            for g, p in zip(res["grads"], (w1, w2, gam, bet)):
                assert H.rel_err(g, p.grad.numpy()) <= 1e-9, (world, dl, r)


def test_gradient_allreduce_tolerates_a_rank_without_gradients():
    """A rank whose parameters have no gradient contributes zeros (same flat length on every rank)."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29400 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_allreduce_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[0] == got[1] and got[0][0] == [0.5, 0.5, 0.5] and got[0][1] == [1.0]


def _allreduce_rank(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, os.path.join(ROOT, "apr-cnn_b200", "pyapr"))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import sharding
    a, b = torch.nn.Parameter(torch.zeros(3)), torch.nn.Parameter(torch.zeros(1))
    if rank == 0:
        a.grad = torch.ones(3)             # rank 1 has no gradient for `a`; rank 0 none for `b`
    else:
        b.grad = torch.full((1,), 2.0)
    sharding.allreduce_gradients([a, b], world)
    q.put((rank, (a.grad.tolist(), b.grad.tolist())))
    dist.destroy_process_group()
