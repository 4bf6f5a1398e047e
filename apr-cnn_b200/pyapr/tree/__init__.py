"""Tree fill on the GPU (reference: pyapr/tree/fill_tree.py:20-71).

The reference fills LibAPR `ParticleData` containers on the CPU; here both functions take and return
CUDA tensors: `parts` is (channels, particles) or (particles,), the result holds one value per
interior tree node in tree-linear order (level-major, root first).
"""
from _pyaprwrapper import tree as _tree


def _as_2d(parts):
    return (parts[None], True) if parts.dim() == 1 else (parts, False)


def fill_tree_mean(apr, parts):
    """Every tree node = mean of its children (exact mean over existing children at odd borders)."""
    p, squeeze = _as_2d(parts.contiguous())
    out = _tree.fill_tree_mean(apr, p)
    return out[0] if squeeze else out


def fill_tree_max(apr, parts):
    """Every tree node = maximum over its descendants."""
    p, squeeze = _as_2d(parts.contiguous())
    out = _tree.fill_tree_max(apr, p)
    return out[0] if squeeze else out
