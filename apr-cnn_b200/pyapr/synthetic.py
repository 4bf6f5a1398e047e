"""Seeded synthetic APR inputs: blob images and the particle/tree access arrays built from them.

The reference obtains an APR from LibAPR's converter (pyapr/converter/converter_methods.py:11-71),
which is a third-party library that this package does not ship.  The operators on the hot path only
need a *valid* APR: a 2:1-balanced octree whose leaves ("particles") tile the volume once, stored as
sparse rows in level-major, then z, then x, then ascending-y order, plus the set of all strict
ancestors (the "tree").  This module builds such a structure from a seeded image with plain tensor
operations so that it runs unchanged on the CPU (tests) or on a GPU (large benchmark volumes).

The per-voxel level follows the formula the reference itself evaluates
(pyapr/converter/src/BindConverter.hpp:131-157):

    level = min(floor(log2(2^level_max / rel_error * grad / lis)), level_max)

with grad < grad_th -> 0, lis < sigma_th -> sigma_th and intensity < Ip_th -> grad = 0.  Gradient and
local intensity scale are computed on the 2x-downsampled image (the resolution of level_max - 1,
whose cells own the finest particles).  The level map is then turned into a balanced tree bottom-up:
a cell is subdivided when the map asks for it or when a 26-neighbour of one of its children is
subdivided, which guarantees that touching particles differ by at most one level.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np
import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------------
# images
# --------------------------------------------------------------------------------------------

def blob_image(shape_zxy, n_blobs, seed, device="cpu", background=100.0,
               sigma_range=(2.0, 8.0), amp_range=(500.0, 2000.0), noise=True,
               return_blobs=False):
    """uint16-valued image (stored as float32) of Gaussian blobs on a flat background plus Poisson noise.

    Blob centres are uniform in the volume, sigma ~ U[sigma_range] voxels (isotropic),
    amplitude ~ U[amp_range].  Blob parameters come from numpy's seeded generator so that they
    do not depend on the device; the Poisson draw uses a torch generator seeded on `device`.
    """
    z_num, x_num, y_num = (int(s) for s in shape_zxy)
    rng = np.random.RandomState(seed)
    cz = rng.uniform(0, z_num, n_blobs)
    cx = rng.uniform(0, x_num, n_blobs)
    cy = rng.uniform(0, y_num, n_blobs)
    sg = rng.uniform(sigma_range[0], sigma_range[1], n_blobs)
    am = rng.uniform(amp_range[0], amp_range[1], n_blobs)

    img = torch.full((z_num, x_num, y_num), float(background), dtype=torch.float32, device=device)
    for b in range(n_blobs):
        r = int(math.ceil(4.0 * sg[b]))
        z0, z1 = max(int(cz[b]) - r, 0), min(int(cz[b]) + r + 1, z_num)
        x0, x1 = max(int(cx[b]) - r, 0), min(int(cx[b]) + r + 1, x_num)
        y0, y1 = max(int(cy[b]) - r, 0), min(int(cy[b]) + r + 1, y_num)
        if z0 >= z1 or x0 >= x1 or y0 >= y1:
            continue
        inv = -0.5 / (sg[b] * sg[b])
        gz = torch.exp(inv * (torch.arange(z0, z1, device=device, dtype=torch.float32) + 0.5 - cz[b]) ** 2)
        gx = torch.exp(inv * (torch.arange(x0, x1, device=device, dtype=torch.float32) + 0.5 - cx[b]) ** 2)
        gy = torch.exp(inv * (torch.arange(y0, y1, device=device, dtype=torch.float32) + 0.5 - cy[b]) ** 2)
        img[z0:z1, x0:x1, y0:y1] += float(am[b]) * gz[:, None, None] * gx[None, :, None] * gy[None, None, :]

    if noise:
        gen = torch.Generator(device=device)
        gen.manual_seed(int(seed) + 7919)
        # Poisson noise on the summed intensity, slab by slab to bound the temporary
        step = max(1, (1 << 26) // max(1, x_num * y_num))
        for z0 in range(0, z_num, step):
            img[z0:z0 + step] = torch.poisson(img[z0:z0 + step], generator=gen)
    img.clamp_(0, 65535)
    if return_blobs:
        return img, dict(cz=cz, cx=cx, cy=cy, sigma=sg, amp=am)
    return img


# --------------------------------------------------------------------------------------------
# level map -> balanced tree -> linear access arrays
# --------------------------------------------------------------------------------------------

def _ceil_half(n):
    return (n + 1) // 2


def level_dims(shape_zxy, level_max):
    """Per-level (z, x, y) extents: ceil(dim / 2^(level_max - l)) for l = 0..level_max."""
    return [tuple(int(math.ceil(s / 2 ** (level_max - l))) for s in shape_zxy) for l in range(level_max + 1)]


def _pool2(t, mode):
    """2x down-sampling of a (z, x, y) tensor with ceil semantics at odd borders."""
    pz, px, py = (s % 2 for s in t.shape)
    v = t[None, None]
    if pz or px or py:
        v = F.pad(v, (0, py, 0, px, 0, pz), mode="replicate")
    if mode == "max":
        return F.max_pool3d(v, 2)[0, 0]
    return F.avg_pool3d(v, 2)[0, 0]


def _box3(t, mode):
    v = F.pad(t[None, None], (1, 1, 1, 1, 1, 1), mode="replicate")
    if mode == "max":
        return F.max_pool3d(v, 3, stride=1)[0, 0]
    return F.avg_pool3d(v, 3, stride=1)[0, 0]


def local_level_map(img, level_max, rel_error=0.1, sigma_th=50.0, grad_th=10.0, Ip_th=120.0):
    """Desired particle level per cell of level_max-1 (integer tensor, values 0..level_max)."""
    d = _pool2(img.float(), "avg")                       # resolution of level_max - 1
    s = _box3(d, "avg")                                  # light smoothing against shot noise
    p = F.pad(s[None, None], (1, 1, 1, 1, 1, 1), mode="replicate")[0, 0]
    # central differences; the cell spacing at this resolution is 2 voxels
    gz = (p[2:, 1:-1, 1:-1] - p[:-2, 1:-1, 1:-1]) * 0.25
    gx = (p[1:-1, 2:, 1:-1] - p[1:-1, :-2, 1:-1]) * 0.25
    gy = (p[1:-1, 1:-1, 2:] - p[1:-1, 1:-1, :-2]) * 0.25
    grad = torch.sqrt(gz * gz + gx * gx + gy * gy)
    del gz, gx, gy, p
    v5 = F.pad(s[None, None], (2, 2, 2, 2, 2, 2), mode="replicate")
    lis = (F.max_pool3d(v5, 5, stride=1) + F.max_pool3d(-v5, 5, stride=1))[0, 0]   # local range
    del v5
    grad = torch.where(grad < grad_th, torch.zeros_like(grad), grad)
    grad = torch.where(s < Ip_th, torch.zeros_like(grad), grad)
    lis = lis.clamp_min(sigma_th)
    arg = (2.0 ** level_max / rel_error) * grad / lis
    lvl = torch.floor(torch.log2(arg.clamp_min(1.0)))
    lvl = torch.where(grad > 0, lvl, torch.zeros_like(lvl)).clamp_(0, level_max)
    return lvl.to(torch.int16)


@dataclass
class AprArrays:
    """Host-side linear access arrays of one APR.

    Rows are numbered level-major: row(l, z, x) = row_off[l] + z * x_num(l) + x for
    l = level_min..level_max; particles of row r are [row_ptr[r], row_ptr[r+1]) and `y` holds their
    ascending y coordinates.  The tree uses the same scheme for levels 0..level_max-1.
    """
    shape: tuple                      # original image extents (z, x, y)
    level_max: int
    level_min: int
    dims: list                        # dims[l] = (z_num, x_num, y_num) for l = 0..level_max
    row_ptr: np.ndarray = field(repr=False, default=None)        # int64, n_rows + 1
    y: np.ndarray = field(repr=False, default=None)              # uint16, N
    tree_row_ptr: np.ndarray = field(repr=False, default=None)   # int64
    tree_y: np.ndarray = field(repr=False, default=None)         # uint16, T

    @property
    def n_particles(self):
        return int(self.y.shape[0])

    @property
    def n_tree(self):
        return int(self.tree_y.shape[0])


def _rows_from_masks(masks):
    """Concatenate per-level boolean (z, x, y) masks into CSR row pointers + y coordinates."""
    counts, ys = [], []
    for m in masks:
        counts.append(m.sum(dim=2, dtype=torch.int64).reshape(-1))
        ys.append(torch.nonzero(m)[:, 2].to(torch.int32))
    counts = torch.cat(counts) if counts else torch.zeros(0, dtype=torch.int64)
    row_ptr = torch.zeros(counts.numel() + 1, dtype=torch.int64, device=counts.device)
    torch.cumsum(counts, 0, out=row_ptr[1:])
    y = torch.cat(ys) if ys else torch.zeros(0, dtype=torch.int32)
    return row_ptr.cpu().numpy(), y.cpu().numpy().astype(np.uint16)


def apr_from_level_map(level_map, shape_zxy):
    """Balanced tree + particle set from a desired-level map given at the resolution of level_max-1."""
    shape_zxy = tuple(int(s) for s in shape_zxy)
    level_max = max(int(math.ceil(math.log2(max(shape_zxy)))), 1)
    dims = level_dims(shape_zxy, level_max)
    assert tuple(level_map.shape) == dims[level_max - 1], (tuple(level_map.shape), dims[level_max - 1])

    # req[l]: cells of level l that the map wants subdivided (some cell inside asks for > l)
    sub = [None] * level_max            # sub[l] = boolean mask of subdivided cells (= tree nodes) at level l
    m = level_map
    req = [None] * level_max
    for l in range(level_max - 1, -1, -1):
        req[l] = m >= (l + 1)
        if l > 0:
            m = _pool2(m.float(), "max").to(level_map.dtype)
            assert tuple(m.shape) == dims[l - 1]
    sub[level_max - 1] = req[level_max - 1]
    for l in range(level_max - 2, -1, -1):
        grown = _box3(sub[l + 1].float(), "max")
        sub[l] = req[l] | (_pool2(grown, "max") > 0)
    sub[0] = torch.ones_like(sub[0])    # the root is always a tree node

    def up2(mask, target):
        u = mask.repeat_interleave(2, 0).repeat_interleave(2, 1).repeat_interleave(2, 2)
        return u[:target[0], :target[1], :target[2]]

    part_masks = []
    for l in range(1, level_max + 1):
        exists = up2(sub[l - 1], dims[l])
        part_masks.append(exists & ~sub[l] if l < level_max else exists)
    # a tree node exists only if its parent does (closure holds by construction; keep it explicit)
    tree_masks = [sub[0]]
    for l in range(1, level_max):
        tree_masks.append(sub[l] & up2(sub[l - 1], dims[l]))

    row_ptr, y = _rows_from_masks(part_masks)
    tree_row_ptr, tree_y = _rows_from_masks(tree_masks)
    return AprArrays(shape=shape_zxy, level_max=level_max, level_min=1, dims=dims,
                     row_ptr=row_ptr, y=y, tree_row_ptr=tree_row_ptr, tree_y=tree_y)


def apr_from_image(img, rel_error=0.1, sigma_th=50.0, grad_th=10.0, Ip_th=120.0):
    shape = tuple(int(s) for s in img.shape)
    level_max = max(int(math.ceil(math.log2(max(shape)))), 1)
    lm = local_level_map(img, level_max, rel_error, sigma_th, grad_th, Ip_th)
    return apr_from_level_map(lm, shape)


def random_apr(shape_zxy, seed, density=0.02, device="cpu"):
    """Small irregular APR for tests: random seeds of fine resolution instead of an image."""
    shape_zxy = tuple(int(s) for s in shape_zxy)
    level_max = max(int(math.ceil(math.log2(max(shape_zxy)))), 1)
    dims = level_dims(shape_zxy, level_max)
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    u = torch.rand(dims[level_max - 1], generator=gen)
    lv = torch.randint(0, level_max + 1, dims[level_max - 1], generator=gen)
    lm = torch.where(u < density, lv, torch.zeros_like(lv)).to(torch.int16).to(device)
    return apr_from_level_map(lm, shape_zxy)


def sample_particles_from_image(img, apr: AprArrays):
    """Mean image intensity over each particle's cell (float32, N) — the input feature channel."""
    out = np.empty(apr.n_particles, dtype=np.float32)
    cur = img.float()
    rows_before = [0] * (apr.level_max + 2)
    for l in range(apr.level_min, apr.level_max + 1):
        rows_before[l + 1] = rows_before[l] + apr.dims[l][0] * apr.dims[l][1]
    pyramid = {apr.level_max: cur}
    for l in range(apr.level_max - 1, apr.level_min - 1, -1):
        cur = _pool2(cur, "avg")
        pyramid[l] = cur
    for l in range(apr.level_min, apr.level_max + 1):
        r0, r1 = rows_before[l], rows_before[l + 1]
        b, e = int(apr.row_ptr[r0]), int(apr.row_ptr[r1])
        if e == b:
            continue
        counts = np.diff(apr.row_ptr[r0:r1 + 1])
        rows = np.repeat(np.arange(r1 - r0), counts)
        z = torch.from_numpy(rows // apr.dims[l][1]).to(img.device)
        x = torch.from_numpy(rows % apr.dims[l][1]).to(img.device)
        y = torch.from_numpy(apr.y[b:e].astype(np.int64)).to(img.device)
        out[b:e] = pyramid[l][z, x, y].cpu().numpy()
    return out
