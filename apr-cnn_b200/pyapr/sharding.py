"""Splitting work over GPUs.

The reference has no multi-GPU support (its batch is a sequential host loop on one device,
pyapr/aprnet/cuda/src/wrap_conv_gpu.hpp:23-28).  Two forms are provided here, both with one process per GPU
over any initialised torch.distributed backend (NCCL on GPUs, gloo in CPU tests):

* independent APRs (`shard_indices`, `allreduce_gradients`): APRs are dealt to ranks, every rank runs the
  operators on its own APRs, nothing of the data path is exchanged; only the (small) weight gradients are
  all-reduced when training;
* ONE APR cut into z-slabs (`zslab_plan`, `HaloExchange`): every rank holds the particles of its slab plus one
  halo row of cells per level on each inner side -- the reach of the 3x3x3 stencil, which reads z +- 1 at the
  level of the output particle, the covering particle one level coarser and the tree node of the cell
  (pyapr/aprnet/cuda/src/conv333_gpu.cu:65-72,239-246).  Before each 3x3x3 layer the owners send the halo
  values (particles, pooled tree nodes, tree means) to their neighbours with point-to-point messages; in the
  backward pass the halo parts of the input gradient travel back and are added by the owner.  Everything else
  (1x1x1 convolution, pooling, up-sampling, tree fill) is local to a slab because cells nest: with slab
  boundaries on multiples of the coarsest cell size that occurs, a cell and all of its descendants have the
  same owner.

This module holds the host-side logic (numpy / torch.distributed) and imports nothing of the extension, so
that it can be exercised on CPU ranks.
"""
import math
from dataclasses import dataclass, field

import numpy as np
import torch


def shard_indices(n_items, rank, world, weights=None):
    """Indices of the items owned by `rank`.

    Without weights: round-robin (item i -> rank i mod world, the split named for batches of APRs).
    With weights (e.g. particle counts): greedy longest-processing-time assignment so that the ranks'
    total weights are balanced; deterministic, every rank computes the same partition."""
    if weights is None:
        return list(range(rank, n_items, world))
    order = sorted(range(n_items), key=lambda i: (-weights[i], i))
    loads = [0] * world
    owner = [0] * n_items
    for i in order:
        r = min(range(world), key=lambda k: (loads[k], k))
        owner[i] = r
        loads[r] += weights[i]
    return [i for i in range(n_items) if owner[i] == rank]


def allreduce_gradients(params, world, average=True):
    """Sum (or average) the gradients of `params` over all ranks with one flat all-reduce.

    Every rank must pass the same parameters in the same order.  A parameter without a gradient on this rank
    (a rank that received no items, a layer that was skipped) contributes zeros and receives the reduced
    gradient, so the flat buffers have the same length everywhere and the collective cannot mismatch."""
    import torch.distributed as dist
    params = list(params)
    if world <= 1 or not params:
        return
    flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in params])
    dist.all_reduce(flat)
    if average:
        flat /= world
    off = 0
    for p in params:
        g = flat[off:off + p.numel()].view_as(p)
        if p.grad is None:
            p.grad = g.clone()
        else:
            p.grad.copy_(g)
        off += p.numel()


# ---------------------------------------------------------------------------------------------------
# z-slabs of one APR
# ---------------------------------------------------------------------------------------------------

@dataclass
class _Lists:
    """Index lists of one level delta, all positions in this rank's local vectors (int64 arrays)."""
    n_local: int = 0                 # length of the local feature vector N(dl)
    t_local: int = 0                 # length of the local tree-mean vector T(dl)
    n_global: int = 0                # owned entries over all ranks = N(dl) of the whole APR
    ghost_x: np.ndarray = None       # halo entries of the feature vector
    ghost_t: np.ndarray = None       # halo entries of the tree-mean vector
    # per neighbour (rank - 1, rank + 1): entries to send (owned here, halo there) and to receive
    send_x: dict = field(default_factory=dict)
    recv_x: dict = field(default_factory=dict)
    send_t: dict = field(default_factory=dict)
    recv_t: dict = field(default_factory=dict)


@dataclass
class SlabPlan:
    rank: int
    world: int
    cuts: list                        # slab boundaries in voxels, len world + 1
    align: int                        # boundaries are multiples of this many voxels
    local: object                     # AprArrays-like record of this rank's slab (+ halo rows)
    l2g_particles: np.ndarray         # global particle index of every local particle
    l2g_tree: np.ndarray              # global tree index of every local tree node
    owned_particles: np.ndarray       # bool per local particle
    n_particles_global: int
    lists: dict                       # level delta -> _Lists
    tree_level_min: int               # coarsest tree level kept in the slabs

    @property
    def neighbours(self):
        return [q for q in (self.rank - 1, self.rank + 1) if 0 <= q < self.world]


class _Local:
    """Minimal stand-in for pyapr.synthetic.AprArrays (same fields), so that this module does not import it."""

    def __init__(self, shape, level_max, level_min, dims, row_ptr, y, tree_row_ptr, tree_y):
        self.shape, self.level_max, self.level_min, self.dims = shape, level_max, level_min, dims
        self.row_ptr, self.y, self.tree_row_ptr, self.tree_y = row_ptr, y, tree_row_ptr, tree_y

    @property
    def n_particles(self):
        return int(self.y.shape[0])

    @property
    def n_tree(self):
        return int(self.tree_y.shape[0])


def _row_offsets(a):
    """First row of every level in the particle arrays (levels level_min..level_max) and the tree arrays
    (levels 0..level_max-1), as the access structure numbers them."""
    ro, to = [0] * (a.level_max + 2), [0] * (a.level_max + 2)
    for l in range(a.level_max + 1):
        rows = a.dims[l][0] * a.dims[l][1]
        ro[l + 1] = ro[l] + (rows if l >= a.level_min else 0)
        to[l + 1] = to[l] + (rows if l <= a.level_max - 1 else 0)
    return ro, to


def choose_cuts(unit_weights, world):
    """Boundaries (in units) of `world` contiguous, non-empty groups of units with balanced total weight."""
    n = len(unit_weights)
    if n < world:
        raise ValueError("cannot cut %d aligned z-units into %d slabs" % (n, world))
    cum = np.concatenate([[0], np.cumsum(np.asarray(unit_weights, dtype=np.float64))])
    cuts = [0]
    for k in range(1, world):
        target = cum[-1] * k / world
        c = int(np.searchsorted(cum, target, side="left"))
        if c > 0 and abs(cum[c - 1] - target) <= abs(cum[min(c, n)] - target):
            c -= 1
        c = max(c, cuts[-1] + 1)              # every slab keeps at least one unit ...
        c = min(c, n - (world - k))           # ... and leaves one for each slab after it
        cuts.append(c)
    cuts.append(n)
    return cuts


def zslab_plan(a, rank, world, max_level_delta=3, cuts=None):
    """Cut the APR `a` (an AprArrays record) into `world` z-slabs and build rank `rank`'s part.

    Slab boundaries are multiples of `align` = the cell size of level la = min(coarsest occupied particle
    level - 1, level_max - max_level_delta - 1): every particle cell, and every tree node that pooling down to
    max_level_delta turns into a feature location, then lies inside one slab.  Tree levels coarser than la are
    left out of the slabs (nothing on the path reads them).  Cuts balance the particle counts.

    The local structure is a valid access structure over the box [z0 - align, z1 + align) (clipped to the
    volume) that contains, per level, the rows of the slab and one halo row of cells on each inner side; the
    other rows of the box are empty.  Every rank can compute every other rank's lists, so the plans need no
    communication."""
    lmax, lmin = int(a.level_max), int(a.level_min)
    Z = int(a.shape[0])
    ro, to = _row_offsets(a)
    rp, trp = np.asarray(a.row_ptr, dtype=np.int64), np.asarray(a.tree_row_ptr, dtype=np.int64)
    counts = [int(rp[ro[l + 1]] - rp[ro[l]]) for l in range(lmax + 1)]
    occupied = [l for l in range(lmin, lmax + 1) if counts[l] > 0]
    if not occupied:
        raise ValueError("APR without particles")
    la = max(0, min(occupied[0] - 1, lmax - max_level_delta - 1))
    align = 2 ** (lmax - la)
    units = (Z + align - 1) // align
    if cuts is None:
        w = np.zeros(units, dtype=np.int64)
        for l in occupied:
            s = 2 ** (lmax - l)
            zn, xn = a.dims[l][0], a.dims[l][1]
            per_z = np.diff(rp[ro[l] + np.arange(zn + 1) * xn])
            np.add.at(w, (np.arange(zn) * s) // align, per_z)
        cuts = [c * align for c in choose_cuts(w, world)]
        cuts[-1] = Z
    cuts = [int(c) for c in cuts]
    assert len(cuts) == world + 1 and cuts[0] == 0 and cuts[-1] == Z
    for c in cuts[1:-1]:
        if c % align:
            raise ValueError("slab boundaries must be multiples of %d voxels" % align)
    z0, z1 = cuts[rank], cuts[rank + 1]
    lo_halo, hi_halo = rank > 0, rank < world - 1
    zb0 = z0 - align if lo_halo else 0
    zb1 = min(z1 + align, Z) if hi_halo else Z
    shape = (zb1 - zb0, int(a.shape[1]), int(a.shape[2]))
    if max(int(math.ceil(math.log2(max(shape)))), 1) != lmax:
        raise ValueError("a slab must keep the level range of the APR: the z extent may not be the only largest dimension")
    dims = [tuple(int(math.ceil(s / 2 ** (lmax - l))) for s in shape) for l in range(lmax + 1)]

    def rows_of(l):
        """Global z rows [g0, g1) stored locally at level l, the owned part [o0, o1) and the local row of g0."""
        s = 2 ** (lmax - l)
        zn = a.dims[l][0]
        o0, o1 = z0 // s, min((z1 + s - 1) // s, zn)
        g0, g1 = max(o0 - (1 if lo_halo else 0), 0), min(o1 + (1 if hi_halo else 0), zn)
        return g0, g1, o0, o1, g0 - zb0 // s

    def extract(levels, row_first, ptr, yv, keep):
        """Local CSR arrays of the given levels: per level the global rows rows_of(l), other rows empty."""
        cnt, ys, l2g, owned, spans = [], [], [], [], {}
        pos = 0
        for l in levels:
            xn = a.dims[l][1]
            local_rows = dims[l][0] * dims[l][1]
            c = np.zeros(local_rows, dtype=np.int64)
            if keep(l):
                g0, g1, o0, o1, lz = rows_of(l)
                if 2 ** (lmax - l) > align and ptr[row_first[l] + g1 * xn] > ptr[row_first[l] + g0 * xn]:
                    raise ValueError("level %d holds cells larger than the slab alignment" % l)
                r0, r1 = row_first[l] + g0 * xn, row_first[l] + g1 * xn
                c[lz * xn:(lz + g1 - g0) * xn] = np.diff(ptr[r0:r1 + 1])
                b, e = int(ptr[r0]), int(ptr[r1])
                ys.append(yv[b:e])
                l2g.append(np.arange(b, e, dtype=np.int64))
                ob, oe = int(ptr[row_first[l] + o0 * xn]), int(ptr[row_first[l] + o1 * xn])
                own = np.zeros(e - b, dtype=bool)
                own[ob - b:oe - b] = True
                owned.append(own)
                # first / last owned row of the level (what the neighbours hold as halo), as local positions
                fb, fe = ob, int(ptr[row_first[l] + min(o0 + 1, o1) * xn])
                lb, le = int(ptr[row_first[l] + max(o1 - 1, o0) * xn]), oe
                spans[l] = dict(begin=pos, end=pos + (e - b), ghost_lo=(pos, pos + (ob - b)), ghost_hi=(pos + (oe - b), pos + (e - b)),
                                first=(pos + (fb - b), pos + (fe - b)), last=(pos + (lb - b), pos + (le - b)))
                pos += e - b
            else:
                spans[l] = dict(begin=pos, end=pos, ghost_lo=(pos, pos), ghost_hi=(pos, pos), first=(pos, pos), last=(pos, pos))
            cnt.append(c)
        cnt = np.concatenate(cnt) if cnt else np.zeros(0, dtype=np.int64)
        row_ptr = np.concatenate([[0], np.cumsum(cnt)]).astype(np.int64)
        cat = lambda xs, dt: np.concatenate(xs) if xs else np.zeros(0, dtype=dt)
        return row_ptr, cat(ys, np.uint16).astype(np.uint16), cat(l2g, np.int64), cat(owned, bool), spans

    yv, tyv = np.asarray(a.y), np.asarray(a.tree_y)
    p_ptr, p_y, l2g_p, own_p, p_spans = extract(range(lmin, lmax + 1), ro, rp, yv, lambda l: counts[l] > 0)
    t_ptr, t_y, l2g_t, own_t, t_spans = extract(range(0, lmax), to, trp, tyv, lambda l: l >= la)
    local = _Local(shape, lmax, lmin, dims, p_ptr, p_y, t_ptr, t_y)
    n_glob = int(yv.shape[0])

    def rng(spans, levels, key):
        parts = [np.arange(*spans[l][key], dtype=np.int64) for l in levels]
        return np.concatenate(parts) if parts else np.zeros(0, dtype=np.int64)

    lists = {}
    for dl in range(0, max_level_delta + 1):
        cml = lmax - dl
        if cml < lmin:
            break
        L = _Lists()
        plev = list(range(lmin, cml + 1))
        n_part_local = p_spans[cml]["end"]
        up = cml <= lmax - 1                    # pooled tree nodes of level cml ride behind the particles
        # the local positions of the level-cml tree nodes inside the feature vector
        shift = n_part_local - t_spans[cml]["begin"] if up else 0
        L.n_local = n_part_local + ((t_spans[cml]["end"] - t_spans[cml]["begin"]) if up else 0)
        L.t_local = t_spans[cml]["begin"] if cml <= lmax - 1 else int(t_y.shape[0])
        L.n_global = int(rp[ro[cml + 1]]) + (int(trp[to[cml + 1]] - trp[to[cml]]) if up else 0)
        tlev = list(range(0, cml))              # tree-mean vector: levels below cml

        def xlist(key):
            v = rng(p_spans, plev, key)
            return np.concatenate([v, rng(t_spans, [cml], key) + shift]) if up else v

        L.ghost_x = np.concatenate([xlist("ghost_lo"), xlist("ghost_hi")])
        L.ghost_t = np.concatenate([rng(t_spans, tlev, "ghost_lo"), rng(t_spans, tlev, "ghost_hi")])
        if lo_halo:
            q = rank - 1
            L.recv_x[q], L.send_x[q] = xlist("ghost_lo"), xlist("first")
            L.recv_t[q], L.send_t[q] = rng(t_spans, tlev, "ghost_lo"), rng(t_spans, tlev, "first")
        if hi_halo:
            q = rank + 1
            L.recv_x[q], L.send_x[q] = xlist("ghost_hi"), xlist("last")
            L.recv_t[q], L.send_t[q] = rng(t_spans, tlev, "ghost_hi"), rng(t_spans, tlev, "last")
        lists[dl] = L
    return SlabPlan(rank=rank, world=world, cuts=cuts, align=align, local=local, l2g_particles=l2g_p, l2g_tree=l2g_t,
                    owned_particles=own_p, n_particles_global=n_glob, lists=lists, tree_level_min=la)


class HaloExchange:
    """Point-to-point exchange of the halo entries of a feature tensor (1, C, N(dl)) and a tree-mean tensor
    (1, C, T(dl)) between neighbouring slabs.  Both directions are in place.  A message carries the feature part
    and the tree part of one neighbour; sends and receives of both neighbours are posted together
    (torch.distributed.batch_isend_irecv: grouped ncclSend / ncclRecv on GPUs).  Sizes are known on both sides
    from the plan; a mismatch (a rank with another plan) raises before anything is posted."""

    def __init__(self, plan, device, group=None):
        self.plan, self.device, self.group = plan, device, group
        self._idx = {}
        for dl, L in plan.lists.items():
            t = lambda v: torch.from_numpy(np.ascontiguousarray(v)).to(device)
            self._idx[dl] = dict(ghost_x=t(L.ghost_x), ghost_t=t(L.ghost_t),
                                 send_x={q: t(v) for q, v in L.send_x.items()}, recv_x={q: t(v) for q, v in L.recv_x.items()},
                                 send_t={q: t(v) for q, v in L.send_t.items()}, recv_t={q: t(v) for q, v in L.recv_t.items()})

    def ghost_index(self, dl):
        return self._idx[dl]["ghost_x"]

    def _run(self, dl, x, tree, out_key_x, out_key_t, in_key_x, in_key_t, add):
        import torch.distributed as dist
        I = self._idx[dl]
        assert x.dim() == 3 and x.shape[0] == 1 and (tree is None or (tree.dim() == 3 and tree.shape[0] == 1)), \
            "one APR per rank: tensors are (1, channels, entries)"
        L = self.plan.lists[dl]
        if x.shape[2] < L.n_local or (tree is not None and tree.shape[2] < L.t_local):
            raise RuntimeError("halo exchange: tensor has %d entries, the slab plan expects %d" % (x.shape[2], L.n_local))
        xs, ts = x.data[0], (tree.data[0] if tree is not None else None)
        C = xs.shape[0]
        ops, recvs = [], []
        for q in self.plan.neighbours:
            ox, ot = I[out_key_x][q], I[out_key_t][q]
            parts = [xs.index_select(1, ox).reshape(-1)]
            if ts is not None:
                parts.append(ts.index_select(1, ot).reshape(-1))
            sbuf = torch.cat(parts) if len(parts) > 1 else parts[0]
            ix, it = I[in_key_x][q], I[in_key_t][q]
            rbuf = torch.empty(C * (ix.numel() + (it.numel() if ts is not None else 0)), dtype=xs.dtype, device=xs.device)
            if sbuf.numel():
                ops.append(dist.P2POp(dist.isend, sbuf, q, group=self.group))
            if rbuf.numel():
                ops.append(dist.P2POp(dist.irecv, rbuf, q, group=self.group))
            recvs.append((q, rbuf, ix, it))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        for q, rbuf, ix, it in recvs:
            nx = C * ix.numel()
            if add:
                xs.index_add_(1, ix, rbuf[:nx].view(C, -1))
                if ts is not None:
                    ts.index_add_(1, it, rbuf[nx:].view(C, -1))
            else:
                xs.index_copy_(1, ix, rbuf[:nx].view(C, -1))
                if ts is not None:
                    ts.index_copy_(1, it, rbuf[nx:].view(C, -1))

    def forward(self, dl, x, tree=None):
        """Owners -> halos: afterwards every halo entry holds its owner's value."""
        self._run(dl, x, tree, "send_x", "send_t", "recv_x", "recv_t", add=False)

    def reverse(self, dl, gx, gtree=None):
        """Halos -> owners: the halo entries are added to their owners' entries and then cleared."""
        self._run(dl, gx, gtree, "recv_x", "recv_t", "send_x", "send_t", add=True)
        I = self._idx[dl]
        gx.data[0].index_fill_(1, I["ghost_x"], 0)
        if gtree is not None:
            gtree.data[0].index_fill_(1, I["ghost_t"], 0)

    def zero_halo(self, dl, x):
        x.data[0].index_fill_(1, self._idx[dl]["ghost_x"], 0)
