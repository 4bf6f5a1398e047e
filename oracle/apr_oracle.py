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
