"""Reading and writing APR access structures (reference: pyapr/io, LibAPR's APRFile on HDF5).

LibAPR and HDF5 are not part of this package, so APRs are stored in numpy's `.npz` container with the
fields of the reference's pickle state (pyapr/data_containers/src/BindAPR.hpp:66-131): the original
dimensions, a name, and the linear access arrays of particles and tree (row ends per (level, z, x) and the
y coordinate of every particle).  `from_libapr_arrays` converts the arrays LibAPR's linear access holds
(`level_xz_vec`, `xz_end_vec`, `y_vec`; usage evidenced at pyapr/aprnet/cuda/src/conv333_gpu.cu:65-67,82)
into this package's row-pointer form.
"""
import numpy as np

from .synthetic import AprArrays, level_dims

FORMAT = "aprnet-b200-apr-1"


def write_apr(path, arrays, name="", particle_data=None):
    """Store an `AprArrays` record (and optionally per-particle features, (C, N) or (N,)) in `path` (.npz)."""
    fields = dict(format=np.array(FORMAT), shape=np.asarray(arrays.shape, dtype=np.int64), name=np.array(name),
                  level_min=np.int64(arrays.level_min), level_max=np.int64(arrays.level_max),
                  row_ptr=np.asarray(arrays.row_ptr, dtype=np.int64), y=np.asarray(arrays.y, dtype=np.uint16),
                  tree_row_ptr=np.asarray(arrays.tree_row_ptr, dtype=np.int64), tree_y=np.asarray(arrays.tree_y, dtype=np.uint16))
    if particle_data is not None:
        fields["particle_data"] = np.asarray(particle_data)
    np.savez_compressed(path, **fields)


def read_apr(path):
    """Inverse of `write_apr`: returns (AprArrays, name, particle_data or None); validates the array lengths."""
    with np.load(path, allow_pickle=False) as f:
        if str(f["format"]) != FORMAT:
            raise ValueError("not an APR file of this package: format %r" % (str(f["format"]),))
        shape = tuple(int(v) for v in f["shape"])
        level_max, level_min = int(f["level_max"]), int(f["level_min"])
        a = AprArrays(shape=shape, level_max=level_max, level_min=level_min, dims=level_dims(shape, level_max),
                      row_ptr=f["row_ptr"].copy(), y=f["y"].copy(), tree_row_ptr=f["tree_row_ptr"].copy(), tree_y=f["tree_y"].copy())
        data = f["particle_data"].copy() if "particle_data" in f.files else None
        name = str(f["name"])
    check_arrays(a)
    return a, name, data


def check_arrays(a):
    """Raise ValueError unless the row pointers are monotone, cover the y arrays and have one entry per row."""
    rows = sum(a.dims[l][0] * a.dims[l][1] for l in range(a.level_min, a.level_max + 1))
    trows = sum(a.dims[l][0] * a.dims[l][1] for l in range(0, a.level_max))
    for ptr, yv, n, what in ((a.row_ptr, a.y, rows, "particle"), (a.tree_row_ptr, a.tree_y, trows, "tree")):
        ptr = np.asarray(ptr)
        if ptr.shape[0] != n + 1 or ptr[0] != 0 or ptr[-1] != np.asarray(yv).shape[0] or np.any(np.diff(ptr) < 0):
            raise ValueError("inconsistent %s access arrays" % what)


def from_libapr_arrays(shape_zxy, level_min, level_max, level_xz_vec, xz_end_vec, y_vec,
                       tree_level_xz_vec, tree_xz_end_vec, tree_y_vec):
    """LibAPR linear access -> AprArrays.

    LibAPR numbers row (l, z, x) as `level_xz_vec[l] + z * x_num(l) + x` and stores in `xz_end_vec[r]` the index one
    past the row's last particle (row r spans [xz_end_vec[r - 1], xz_end_vec[r])); this package keeps the same rows
    from `level_min` (tree: from level 0) as a CSR pointer array with a leading zero."""
    shape = tuple(int(s) for s in shape_zxy)
    dims = level_dims(shape, int(level_max))

    def csr(level_xz, ends, first_level, last_level):
        ends = np.asarray(ends, dtype=np.int64)
        r0 = int(level_xz[first_level])
        n = sum(dims[l][0] * dims[l][1] for l in range(first_level, last_level + 1))
        seg = ends[r0:r0 + n]
        base = int(ends[r0 - 1]) if r0 > 0 else 0
        return np.concatenate([[0], seg - base]).astype(np.int64), base

    row_ptr, pbase = csr(level_xz_vec, xz_end_vec, int(level_min), int(level_max))
    trp, tbase = csr(tree_level_xz_vec, tree_xz_end_vec, 0, int(level_max) - 1)
    y = np.asarray(y_vec, dtype=np.uint16)[pbase:pbase + int(row_ptr[-1])]
    ty = np.asarray(tree_y_vec, dtype=np.uint16)[tbase:tbase + int(trp[-1])]
    a = AprArrays(shape=shape, level_max=int(level_max), level_min=int(level_min), dims=dims, row_ptr=row_ptr, y=y, tree_row_ptr=trp, tree_y=ty)
    check_arrays(a)
    return a
