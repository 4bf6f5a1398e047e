"""TEST INFRASTRUCTURE ONLY.  Loader for `oracle/_ref/_apr_ref` (the reference's CPU operators
compiled unmodified against a LibAPR stand-in; see build_ref.py).  Returns None when the module has
not been built, so callers can fall back to the restated oracle (apr_oracle.py)."""
import glob
import importlib.util
import os

HERE = os.path.dirname(os.path.abspath(__file__))
_mod = None


def load():
    global _mod
    if _mod is not None:
        return _mod
    hits = glob.glob(os.path.join(HERE, "_ref", "_apr_ref*.so"))
    if not hits:
        return None
    import torch  # noqa: F401  (libtorch must be loaded first)
    spec = importlib.util.spec_from_file_location("_apr_ref", hits[0])
    try:
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    except Exception:
        return None
    _mod = mod
    return mod


def make_apr(mod, a):
    """Build the stand-in APR object from an AprArrays-like object (see pyapr/synthetic.py)."""
    return mod.APR(list(a.shape), int(a.level_min), int(a.level_max), [list(d) for d in a.dims],
                   a.row_ptr, a.y, a.tree_row_ptr, a.tree_y)
