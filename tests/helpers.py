"""Shared test inputs: small seeded APR structures (incl. odd extents) and comparison helpers."""
import numpy as np
import torch

from pyapr import synthetic

# (shape_zxy, seed, density): odd extents exercise the boundary scale factors of the tree mean and the
# zero padding of the stencil; (65, 61, 63) / (1, 63, 63) are the shapes of the reference's own fixtures
# (pyapr/tests/test_io.py:5-9).
APR_CASES = {
    "cube16": ((16, 16, 16), 1, 0.03),
    "odd": ((13, 9, 21), 3, 0.05),
    "odd2": ((20, 11, 12), 9, 0.2),
    "plane": ((1, 33, 31), 5, 0.1),
    "cube32": ((32, 32, 32), 2, 0.01),
    "ref_shape": ((65, 61, 63), 11, 0.004),
}

_cache = {}


def arrays(name):
    if name not in _cache:
        shape, seed, dens = APR_CASES[name]
        _cache[name] = synthetic.random_apr(shape, seed, density=dens)
    return _cache[name]


def blob_arrays(shape=(32, 32, 32), n_blobs=6, seed=4):
    key = ("blob", shape, n_blobs, seed)
    if key not in _cache:
        img = synthetic.blob_image(shape, n_blobs, seed)
        _cache[key] = synthetic.apr_from_image(img)
    return _cache[key]


def max_dl(a, need=1):
    """Largest level delta with at least `need` levels left below it (and x extent > 1 at that level)."""
    dl = 0
    while a.level_max - (dl + 1) >= a.level_min + need - 1 and a.dims[a.level_max - (dl + 1)][1] > 1 and dl < 3:
        dl += 1
    return dl


def rel_err(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    if a.size == 0:
        return 0.0
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-300))


def t2n(t):
    return t.detach().cpu().numpy()
