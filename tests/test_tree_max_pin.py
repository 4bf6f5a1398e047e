"""Pins the oracle's fill_tree_max on every interior node: the value of a tree node equals the maximum of the
piecewise-constant reconstruction over the node's block, the relation the reference's own test uses for the mean
(pyapr/tests/test_tree.py:14-25; its max test only looks at the root, :39-40).  The CUDA fill_tree_max is compared
with the oracle bit for bit in the GPU parity tests, so this closes the chain for interior nodes."""
import numpy as np
import pytest

import helpers as H


def _cells(a, row_ptr, yv, levels):
    """(level, z, x, y) of every entry of a row-major sparse array."""
    out = []
    row = 0
    for l in levels:
        zn, xn = a.dims[l][0], a.dims[l][1]
        for z in range(zn):
            for x in range(xn):
                for i in range(int(row_ptr[row]), int(row_ptr[row + 1])):
                    out.append((l, z, x, int(yv[i])))
                row += 1
    return out


@pytest.mark.parametrize("name", ["cube16", "odd", "odd2", "plane"])
def test_tree_max_equals_block_max_of_the_reconstruction(name, oracle):
    a = H.arrays(name)
    o = oracle.OracleAPR(a)
    rng = np.random.RandomState(2)
    vals = rng.rand(a.n_particles)
    img = np.full(a.shape, -np.inf)
    lmax = a.level_max
    for (l, z, x, y), v in zip(_cells(a, a.row_ptr, a.y, range(a.level_min, lmax + 1)), vals):
        s = 2 ** (lmax - l)
        img[z * s:(z + 1) * s, x * s:(x + 1) * s, y * s:(y + 1) * s] = v
    assert np.isfinite(img).all()                      # the particle cells tile the volume
    tree = o.fill_tree_max(vals)
    nodes = _cells(a, a.tree_row_ptr, a.tree_y, range(0, lmax))
    assert len(nodes) == tree.shape[0]
    for (l, z, x, y), t in zip(nodes, tree):
        s = 2 ** (lmax - l)
        assert t == img[z * s:(z + 1) * s, x * s:(x + 1) * s, y * s:(y + 1) * s].max(), (l, z, x, y)
    if any(d & (d - 1) for d in a.shape):
        return          # at odd borders the tree mean is the mean over the existing CHILDREN, not over the clipped block's voxels
    mean = o.fill_tree_mean(vals[None], 0)[0]
    for (l, z, x, y), t in zip(nodes, mean):          # the same relation for the mean, as the reference's test has it
        s = 2 ** (lmax - l)
        assert abs(t - img[z * s:(z + 1) * s, x * s:(x + 1) * s, y * s:(y + 1) * s].mean()) <= 1e-12, (l, z, x, y)
