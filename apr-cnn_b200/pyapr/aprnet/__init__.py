"""Particle-domain CNN modules (reference: pyapr/aprnet/__init__.py).

The reference also ships CPU twins of these modules (pyapr/aprnet/{conv,pool,upsample}.py); this
package has no CPU path, so the top-level names resolve to the CUDA modules.
"""
from _pyaprwrapper.aprnet import utils
from . import cuda
from .cuda import APRConv, MaxPool, UpSampleConst

__all__ = ["utils", "cuda", "APRConv", "MaxPool", "UpSampleConst"]
