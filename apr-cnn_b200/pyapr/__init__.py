"""pyapr — host-side mirror of the part of the reference package that the particle-domain CNN path needs.

Only the pieces on that path exist here: the `APR` container and `APRPtrVector`
(`pyapr.data_containers`), the CUDA operator modules (`pyapr.aprnet.cuda`), the tree-fill helpers
(`pyapr.tree`) and a synthetic-APR generator (`pyapr.synthetic`).  Everything computes on the GPU
through the `_pyaprwrapper` extension; there is no CPU implementation behind these classes.
"""
import os as _os
import sys as _sys

_pkg_root = _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__)))
if _pkg_root not in _sys.path:
    _sys.path.insert(0, _pkg_root)

import torch as _torch  # noqa: F401,E402  (libtorch must be loaded before the extension)

try:
    import _pyaprwrapper  # noqa: E402
except ImportError as _e:  # fail loudly: there is no fallback implementation
    raise ImportError(
        "pyapr: the native extension `_pyaprwrapper` (and libaprnet_b200.so) is missing or failed to load; "
        "build it with `python apr-cnn_b200/build.py`. Original error: %s" % (_e,)) from _e

from _pyaprwrapper import __cuda_build__, __version__  # noqa: E402
from . import data_containers  # noqa: E402
from .data_containers import APR, APRPtrVector, apr_from_arrays  # noqa: E402
from . import aprnet  # noqa: E402
from . import tree  # noqa: E402
from . import synthetic  # noqa: E402
from . import sharding  # noqa: E402
from . import io  # noqa: E402


def cuda_enabled() -> bool:
    """True when the extension was built with CUDA support (always, for this package)."""
    return bool(__cuda_build__)
