from .maxpool import MaxPool
from .conv import APRConv
from .upsample import UpSampleConst
from .norm import GroupNormReLU
from .utils import Reconstruct, SampleParticles

__all__ = ["MaxPool", "APRConv", "UpSampleConst", "GroupNormReLU", "Reconstruct", "SampleParticles"]
