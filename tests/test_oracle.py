"""The CPU restatement (oracle/apr_oracle.cpp) pinned against the reference's own CPU operators.

1. Committed golden vectors (tests/golden/*.npz, produced by tests/golden/make_golden.py from the
   reference code compiled unmodified): every operator, level deltas 0..2, float64, <= 1e-12 relative;
   integer outputs bit-exact.
2. When the compiled reference module is present (oracle/_ref), a live cross-check on further random
   structures.
3. Known-answer relations that follow from the reference code.
"""
import glob
import os
from types import SimpleNamespace

import numpy as np
import pytest

import helpers as H

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))
TOL = 1e-12


def _arrays_from_npz(g):
    return SimpleNamespace(shape=tuple(int(v) for v in g["shape"]), level_min=int(g["level_min"]), level_max=int(g["level_max"]),
                           dims=[tuple(int(v) for v in d) for d in g["dims"]], row_ptr=g["row_ptr"], y=g["y"],
                           tree_row_ptr=g["tree_row_ptr"], tree_y=g["tree_y"])


def test_golden_files_present():
    assert len(GOLDEN) >= 4


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_oracle_matches_reference_golden(path, oracle):
    g = np.load(path)
    a = _arrays_from_npz(g)
    o = oracle.OracleAPR(a)
    L = a.level_max - a.level_min + 1
    for dl in g["dls"]:
        dl = int(dl)
        k = "dl%d_" % dl
        assert o.number_parts(dl) == int(g[k + "n"])
        x, w, w1, go = g[k + "x"], g[k + "w"], g[k + "w1"], g[k + "go"]
        we = oracle.restrict333_forward(w, L)
        assert H.rel_err(we, g[k + "w_expanded"]) <= TOL
        assert H.rel_err(o.fill_tree_mean(x, dl), g[k + "tree"]) <= TOL
        assert H.rel_err(o.fill_tree_mean_backward(x, g[k + "gt"], dl), g[k + "tree_bwd"]) <= TOL
        assert H.rel_err(o.conv333_forward(x, we, dl), g[k + "conv333"]) <= TOL, (path, dl)
        gi, gw = o.conv333_backward(x, we, go, dl)
        assert H.rel_err(gi, g[k + "conv333_gi"]) <= TOL
        assert H.rel_err(gw, g[k + "conv333_gw"]) <= TOL
        assert H.rel_err(oracle.restrict333_backward(gw, w.shape[0]), g[k + "restrict_bwd"]) <= TOL
        assert H.rel_err(o.conv111_forward(x, w1, dl), g[k + "conv111"]) <= TOL
        gi, gw = o.conv111_backward(x, w1, go, dl)
        assert H.rel_err(gi, g[k + "conv111_gi"]) <= TOL
        assert H.rel_err(gw, g[k + "conv111_gw"]) <= TOL
        po, pi = o.maxpool_forward(g[k + "xr"], dl)
        assert np.array_equal(po, g[k + "pool"]) and np.array_equal(pi, g[k + "pool_idx"])
        assert np.array_equal(o.maxpool_backward(g[k + "gpo"], pi, dl), g[k + "pool_bwd"])
        if dl > 0:
            assert np.array_equal(o.upsample_forward(x, dl), g[k + "up"])
            assert H.rel_err(o.upsample_backward(g[k + "gu"], dl), g[k + "up_bwd"]) <= TOL


def test_oracle_matches_live_reference(oracle):
    import ref
    import torch
    m = ref.load()
    if m is None:
        pytest.skip("oracle/_ref not built (needs the reference checkout)")
    for name in ("ref_shape", "cube32"):
        a = H.arrays(name)
        apr, o = ref.make_apr(m, a), oracle.OracleAPR(a)
        L = a.level_max - a.level_min + 1
        rng = np.random.RandomState(5)
        for dl in range(0, 3):
            n = o.number_parts(dl)
            assert n == m.number_parts(apr, dl)
            x, w, go = rng.rand(2, n), rng.randn(3, 3, 2, 3, 3, 3), rng.randn(3, n)
            ld = torch.full((1,), dl, dtype=torch.int32)
            wc = torch.from_numpy(w).permute(2, 0, 1, 3, 4, 5).contiguous()
            we_ref = m.restrict_kernel333_forward(wc, L)
            we = oracle.restrict333_forward(w, L)
            out_ref = m.convolve333_forward([apr], torch.from_numpy(x)[None], we_ref, ld)[0].numpy()
            assert H.rel_err(o.conv333_forward(x, we, dl), out_ref) <= TOL
            gi_ref, gw_ref = m.convolve333_backward([apr], torch.from_numpy(x)[None], we_ref, torch.from_numpy(go)[None], ld)
            gi, gw = o.conv333_backward(x, we, go, dl)
            assert H.rel_err(gi, gi_ref[0].numpy()) <= TOL
            assert H.rel_err(gw, gw_ref.permute(1, 2, 0, 3, 4, 5).numpy()) <= TOL


def test_restriction_preserves_stencil_sum_and_first_slots(oracle):
    # pyapr/aprnet/src/kernel.hpp:71-123: the first S slots are copied, box-averaging keeps the sum
    w = np.random.RandomState(0).randn(2, 3, 2, 3, 3, 3)
    we = oracle.restrict333_forward(w, 6)
    assert np.array_equal(we[:2], w)
    s_last = w[1].reshape(3, 2, 27).sum(-1)
    for k in range(2, 6):
        assert np.allclose(we[k].reshape(3, 2, 27).sum(-1), s_last, rtol=1e-12)


@pytest.mark.parametrize("name", ["cube16", "odd", "cube32"])
def test_constant_input_relations(name, oracle):
    a = H.arrays(name)
    o = oracle.OracleAPR(a)
    n = o.number_parts(0)
    ones = np.ones((1, n))
    # tree mean of a constant is the constant, including odd borders (helpers.hpp:133-153)
    assert np.allclose(o.fill_tree_mean(ones, 0), 1.0, rtol=0, atol=1e-15)
    # all-ones stencil on constant input counts the in-domain neighbour cells: 27 for interior particles
    L = a.level_max - a.level_min + 1
    out = o.conv333_forward(ones, np.ones((L, 1, 1, 3, 3, 3)), 0)[0]
    nb = o.nbr_table(0)
    inside = (nb != -1).sum(0)
    assert np.array_equal(np.round(out).astype(np.int64), inside)
    assert out.max() == 27 or a.shape[0] < 3
    # centre-only stencil scales every particle by its level's weight
    w = np.zeros((L, 1, 1, 27)); w[:, 0, 0, 13] = np.arange(1, L + 1)
    x = np.random.RandomState(1).rand(1, n)
    out = o.conv333_forward(x, w.reshape(L, 1, 1, 3, 3, 3), 0)[0]
    ro = 0
    for l in range(a.level_min, a.level_max + 1):
        nr = a.dims[l][0] * a.dims[l][1]
        b, e = int(a.row_ptr[ro]), int(a.row_ptr[ro + nr]); ro += nr
        assert np.allclose(out[b:e], (a.level_max - l + 1) * x[0, b:e], rtol=1e-14)


@pytest.mark.parametrize("name", ["cube16", "odd", "ref_shape"])
def test_upsample_then_maxpool_is_identity_on_pooled_values(name, oracle):
    a = H.arrays(name)
    o = oracle.OracleAPR(a)
    x = np.random.RandomState(2).rand(2, o.number_parts(1))
    up = o.upsample_forward(x, 1)
    back, _ = o.maxpool_forward(up, 0)
    assert np.array_equal(back, x)


@pytest.mark.parametrize("name", list(H.APR_CASES))
def test_generated_structures_are_valid(name, oracle):
    """Particles tile the volume once, and every in-domain neighbour cell of every output resolves
    (2:1 balance in the 26-neighbourhood) for all level deltas used by the tests."""
    a = H.arrays(name)
    o = oracle.OracleAPR(a)
    vol = 0
    ro = 0
    for l in range(a.level_min, a.level_max + 1):
        nr = a.dims[l][0] * a.dims[l][1]
        zs = np.repeat(np.arange(nr) // a.dims[l][1], np.diff(a.row_ptr[ro:ro + nr + 1]))
        xs = np.repeat(np.arange(nr) % a.dims[l][1], np.diff(a.row_ptr[ro:ro + nr + 1]))
        ys = a.y[int(a.row_ptr[ro]):int(a.row_ptr[ro + nr])].astype(np.int64)
        s = 2 ** (a.level_max - l)
        ext = lambda c, full: np.minimum((c + 1) * s, full) - c * s
        vol += int((ext(zs, a.shape[0]) * ext(xs, a.shape[1]) * ext(ys, a.shape[2])).sum())
        ro += nr
    assert vol == a.shape[0] * a.shape[1] * a.shape[2]
    for dl in range(0, H.max_dl(a) + 1):
        nb = o.nbr_table(dl)
        ct = o.child_table()
        assert nb.shape == (27, o.number_parts(dl))
        assert (nb[13] == np.arange(nb.shape[1])).all()          # the centre tap is the location itself
        assert ct.shape[0] == 8


def test_image_ops_restatement_round_trip_and_adjoint():
    """numpy restatement of Reconstruct / SampleParticles: the reconstruction covers every voxel once,
    sample(reconstruct(x)) == x (pyapr/tests/test_aprnet.py:272-285) and backward is the adjoint of forward."""
    import apr_oracle
    a = H.arrays("odd")
    o = apr_oracle.OracleAPR(a)
    rng = np.random.RandomState(0)
    for dl in range(0, H.max_dl(a) + 1):
        n = o.number_parts(dl)
        x = rng.rand(2, n)
        img = apr_oracle.reconstruct_forward(a, x, dl)
        ones = apr_oracle.reconstruct_forward(a, np.ones((1, n)), dl)
        assert (ones == 1).all()
        assert np.abs(apr_oracle.sample_particles_forward(a, img, dl, n) - x).max() < 1e-14
        g = rng.randn(*img.shape)
        assert abs((img * g).sum() - (x * apr_oracle.reconstruct_backward(a, g, dl, n)).sum()) < 1e-9
        s = apr_oracle.sample_particles_forward(a, g, dl, n)
        assert abs((s * x).sum() - (g * apr_oracle.sample_particles_backward(a, x, dl)).sum()) < 1e-9
