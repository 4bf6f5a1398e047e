from .maxpool import MaxPool
from .conv import APRConv
from .upsample import UpSampleConst
from .norm import GroupNormReLU

__all__ = ["MaxPool", "APRConv", "UpSampleConst", "GroupNormReLU"]
