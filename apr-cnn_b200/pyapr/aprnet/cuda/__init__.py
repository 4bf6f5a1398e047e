"""CUDA modules of the particle-domain CNN operators (names as in the reference package)."""
from .conv import APRConv
from .maxpool import MaxPool
from .norm import GroupNormReLU
from .upsample import UpSampleConst
from .utils import Reconstruct, SampleParticles

__all__ = ["APRConv", "MaxPool", "UpSampleConst", "GroupNormReLU", "Reconstruct", "SampleParticles"]
