"""TEST INFRASTRUCTURE ONLY — ctypes front end of the restated CPU oracle (apr_oracle.cpp).

Only tests/, the smoke check and the benchmark's CPU-baseline leg may import this module.  It is the
checker for the CUDA operators; nothing in the product path depends on it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force=False):
    src = os.path.join(HERE, "apr_oracle.cpp")
    out = os.path.join(HERE, "libapr_oracle.so")
    if force or not os.path.isfile(out) or os.path.getmtime(out) < os.path.getmtime(src):
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-fopenmp", "-shared", "-fPIC", src, "-o", out])
    return out


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
        for name in ("orc_number_parts", "orc_tree_size", "orc_tree_offset"):
            getattr(_LIB, name).restype = C.c_int64
        _LIB.orc_apr_create.restype = C.c_void_p
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


_SFX = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64"}


class OracleAPR:
    """Handle on one APR structure inside the oracle library (copies the access arrays)."""

    def __init__(self, a):
        self.arrays = a
        self.level_min, self.level_max = int(a.level_min), int(a.level_max)
        dims = np.ascontiguousarray(np.array(a.dims, dtype=np.int32).reshape(-1))
        rp = np.ascontiguousarray(a.row_ptr, dtype=np.int64)
        y = np.ascontiguousarray(a.y, dtype=np.uint16)
        trp = np.ascontiguousarray(a.tree_row_ptr, dtype=np.int64)
        ty = np.ascontiguousarray(a.tree_y, dtype=np.uint16)
        self.h = C.c_void_p(lib().orc_apr_create(self.level_min, self.level_max, _p(dims), _p(rp),
                                                 C.c_int64(rp.size - 1), _p(y), C.c_int64(y.size), _p(trp),
                                                 C.c_int64(trp.size - 1), _p(ty), C.c_int64(ty.size)))
        self.n_tree_total = int(ty.size)

    def __del__(self):
        try:
            lib().orc_apr_destroy(self.h)
        except Exception:
            pass

    def number_parts(self, dl):
        return int(lib().orc_number_parts(self.h, int(dl)))

    def tree_size(self, dl):
        return int(lib().orc_tree_size(self.h, int(dl)))

    def tree_offset(self, level):
        return int(lib().orc_tree_offset(self.h, int(level)))

    def nbr_table(self, dl):
        out = np.empty((27, self.number_parts(dl)), dtype=np.int32)
        lib().orc_nbr_table(self.h, int(dl), _p(out))
        return out

    def child_table(self):
        out = np.empty((8, self.n_tree_total), dtype=np.int32)
        lib().orc_child_table(self.h, _p(out))
        return out

    # ---- single-APR operators on (C, N) arrays -------------------------------------------------
    def _f(self, name, dtype):
        return getattr(lib(), "orc_%s_%s" % (name, _SFX[np.dtype(dtype)]))

    def fill_tree_mean(self, x, dl):
        x = np.ascontiguousarray(x)
        out = np.zeros((x.shape[0], self.tree_size(dl)), dtype=x.dtype)
        self._f("fill_tree_mean", x.dtype)(self.h, int(dl), x.shape[0], _p(x), _p(out))
        return out

    def fill_tree_mean_backward(self, grad_in, grad_tree, dl):
        g = np.array(grad_in, copy=True, order="C")
        t = np.array(grad_tree, copy=True, order="C")
        self._f("fill_tree_mean_backward", g.dtype)(self.h, int(dl), g.shape[0], _p(g), _p(t))
        return g

    def fill_tree_max(self, x):
        x = np.ascontiguousarray(x)
        out = np.zeros(self.n_tree_total, dtype=x.dtype)
        self._f("fill_tree_max", x.dtype)(self.h, _p(x), _p(out))
        return out

    def conv333_forward(self, x, w, dl):
        """x (Cin, N); w (L, Cout, Cin, 3, 3, 3) already expanded to L level slots."""
        x = np.ascontiguousarray(x); w = np.ascontiguousarray(w, dtype=x.dtype)
        out = np.zeros((w.shape[1], x.shape[1]), dtype=x.dtype)
        self._f("conv333_forward", x.dtype)(self.h, int(dl), x.shape[0], w.shape[1], w.shape[0], _p(x), _p(w), _p(out))
        return out

    def conv333_backward(self, x, w, gout, dl):
        x = np.ascontiguousarray(x); w = np.ascontiguousarray(w, dtype=x.dtype)
        gout = np.ascontiguousarray(gout, dtype=x.dtype)
        gin = np.zeros_like(x); gw = np.zeros_like(w)
        self._f("conv333_backward", x.dtype)(self.h, int(dl), x.shape[0], w.shape[1], w.shape[0], _p(x), _p(w),
                                             _p(gout), _p(gin), _p(gw))
        return gin, gw

    def conv111_forward(self, x, w, dl):
        x = np.ascontiguousarray(x); w = np.ascontiguousarray(w, dtype=x.dtype)
        out = np.zeros((w.shape[1], x.shape[1]), dtype=x.dtype)
        self._f("conv111_forward", x.dtype)(self.h, int(dl), x.shape[0], w.shape[1], w.shape[0], _p(x), _p(w), _p(out))
        return out

    def conv111_backward(self, x, w, gout, dl):
        x = np.ascontiguousarray(x); w = np.ascontiguousarray(w, dtype=x.dtype)
        gout = np.ascontiguousarray(gout, dtype=x.dtype)
        gin = np.zeros_like(x); gw = np.zeros_like(w)
        self._f("conv111_backward", x.dtype)(self.h, int(dl), x.shape[0], w.shape[1], w.shape[0], _p(x), _p(w),
                                             _p(gout), _p(gin), _p(gw))
        return gin, gw

    def maxpool_forward(self, x, dl):
        x = np.ascontiguousarray(x)
        m = self.number_parts(dl + 1)
        out = np.zeros((x.shape[0], m), dtype=x.dtype); idx = np.zeros((x.shape[0], m), dtype=np.int64)
        self._f("maxpool_forward", x.dtype)(self.h, int(dl), x.shape[0], _p(x), _p(out), _p(idx))
        return out, idx

    def maxpool_backward(self, gout, idx, dl):
        gout = np.ascontiguousarray(gout); idx = np.ascontiguousarray(idx, dtype=np.int64)
        gin = np.zeros((gout.shape[0], self.number_parts(dl)), dtype=gout.dtype)
        self._f("maxpool_backward", gout.dtype)(self.h, int(dl), gout.shape[0], _p(gout), _p(idx), _p(gin))
        return gin

    def upsample_forward(self, x, dl):
        x = np.ascontiguousarray(x)
        out = np.zeros((x.shape[0], self.number_parts(dl - 1)), dtype=x.dtype)
        self._f("upsample_forward", x.dtype)(self.h, int(dl), x.shape[0], _p(x), _p(out))
        return out

    def upsample_backward(self, gout, dl):
        gout = np.ascontiguousarray(gout)
        gin = np.zeros((gout.shape[0], self.number_parts(dl)), dtype=gout.dtype)
        self._f("upsample_backward", gout.dtype)(self.h, int(dl), gout.shape[0], _p(gout), _p(gin))
        return gin


def restrict333_forward(w, num_levels):
    """w (S, Cout, Cin, 3, 3, 3) -> (L, Cout, Cin, 3, 3, 3)."""
    w = np.ascontiguousarray(w)
    out = np.zeros((num_levels,) + w.shape[1:], dtype=w.dtype)
    fn = getattr(lib(), "orc_restrict333_forward_" + _SFX[w.dtype])
    fn(w.shape[0], int(num_levels), C.c_int64(w.shape[1] * w.shape[2]), _p(w), _p(out))
    return out


def restrict333_backward(gw, num_stencils):
    gw = np.ascontiguousarray(gw)
    out = np.zeros((num_stencils,) + gw.shape[1:], dtype=gw.dtype)
    fn = getattr(lib(), "orc_restrict333_backward_" + _SFX[gw.dtype])
    fn(int(num_stencils), gw.shape[0], C.c_int64(gw.shape[1] * gw.shape[2]), _p(gw), _p(out))
    return out


# ---------------------------------------------------------------------------------------------
# particles <-> dense image (numpy restatement; the reference has only CUDA code for these:
# pyapr/aprnet/cuda/src/reconstruct_gpu.cu:5-157, sample_particles_gpu.cu:5-170).  Pinned relationally
# like the reference's own tests (gradcheck and sample(reconstruct(x)) == x, pyapr/tests/test_aprnet.py:248-285).
# ---------------------------------------------------------------------------------------------
def _cells(a, dl):
    """Yield (feature index array, z0, x0, y0, edge) per particle / upgraded node for level_delta dl."""
    cml = a.level_max - dl
    row_off, tree_row_off = {}, {}
    r = 0
    for l in range(a.level_min, a.level_max + 1):
        row_off[l] = r
        r += a.dims[l][0] * a.dims[l][1]
    r = 0
    for l in range(0, a.level_max):
        tree_row_off[l] = r
        r += a.dims[l][0] * a.dims[l][1]
    out = []

    def level_cells(row_ptr, y, off, l, edge, index_offset):
        zn, xn, _ = a.dims[l]
        rp = row_ptr[off:off + zn * xn + 1]
        counts = np.diff(rp)
        rows = np.repeat(np.arange(zn * xn), counts)
        idx = np.arange(rp[0], rp[-1])
        return idx + index_offset, (rows // xn) * edge, (rows % xn) * edge, y[rp[0]:rp[-1]].astype(np.int64) * edge, edge

    for l in range(a.level_min, cml + 1):
        out.append(level_cells(a.row_ptr, a.y, row_off[l], l, 1 << (cml - l), 0))
    if dl > 0:
        n_le = int(a.row_ptr[row_off[cml] + a.dims[cml][0] * a.dims[cml][1]])                # particles of levels <= cml
        t_begin = int(a.tree_row_ptr[tree_row_off[cml]])
        out.append(level_cells(a.tree_row_ptr, a.tree_y, tree_row_off[cml], cml, 1, n_le - t_begin))
    return out, a.dims[cml]


def reconstruct_forward(a, x, dl):
    """x (C, N) -> image (C, Z, X, Y)."""
    cells, (Z, X, Y) = _cells(a, dl)
    img = np.zeros((x.shape[0], Z, X, Y), dtype=x.dtype)
    for idx, z0, x0, y0, e in cells:
        for dz in range(e):
            for dx in range(e):
                for dy in range(e):
                    ok = (z0 + dz < Z) & (x0 + dx < X) & (y0 + dy < Y)
                    img[:, z0[ok] + dz, x0[ok] + dx, y0[ok] + dy] = x[:, idx[ok]]
    return img


def reconstruct_backward(a, gimg, dl, n):
    """image gradient (C, Z, X, Y) -> (C, n)."""
    cells, (Z, X, Y) = _cells(a, dl)
    g = np.zeros((gimg.shape[0], n), dtype=gimg.dtype)
    for idx, z0, x0, y0, e in cells:
        for dz in range(e):
            for dx in range(e):
                for dy in range(e):
                    ok = (z0 + dz < Z) & (x0 + dx < X) & (y0 + dy < Y)
                    g[:, idx[ok]] += gimg[:, z0[ok] + dz, x0[ok] + dx, y0[ok] + dy]
    return g


def _cell_volume(z0, x0, y0, e, Z, X, Y):
    return (np.minimum(z0 + e, Z) - z0) * (np.minimum(x0 + e, X) - x0) * (np.minimum(y0 + e, Y) - y0)


def sample_particles_forward(a, img, dl, n):
    out = reconstruct_backward(a, img, dl, n)
    cells, (Z, X, Y) = _cells(a, dl)
    for idx, z0, x0, y0, e in cells:
        out[:, idx] /= _cell_volume(z0, x0, y0, e, Z, X, Y)
    return out


def sample_particles_backward(a, g, dl):
    cells, (Z, X, Y) = _cells(a, dl)
    scaled = g.copy()
    for idx, z0, x0, y0, e in cells:
        scaled[:, idx] /= _cell_volume(z0, x0, y0, e, Z, X, Y)
    return reconstruct_forward(a, scaled, dl)
