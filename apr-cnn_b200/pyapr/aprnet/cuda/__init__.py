from .maxpool import MaxPool
from .conv import APRConv
from .upsample import UpSampleConst

__all__ = ["MaxPool", "APRConv", "UpSampleConst"]
