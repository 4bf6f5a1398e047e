"""`APR` and `APRPtrVector` (reference: pyapr/data_containers/src/BindAPR.hpp:44-133)."""
import numpy as np
from _pyaprwrapper.data_containers import APR, APRPtrVector

__all__ = ["APR", "APRPtrVector", "apr_from_arrays"]


def apr_from_arrays(arrays, name=""):
    """Wrap linear access arrays (see `pyapr.synthetic.AprArrays`) into an `APR` object."""
    apr = APR()
    z, x, y = (int(s) for s in arrays.shape)
    apr.init_from_arrays(z, x, y, np.ascontiguousarray(arrays.row_ptr, dtype=np.int64),
                         np.ascontiguousarray(arrays.y, dtype=np.uint16),
                         np.ascontiguousarray(arrays.tree_row_ptr, dtype=np.int64),
                         np.ascontiguousarray(arrays.tree_y, dtype=np.uint16))
    apr.name = name
    assert apr.level_max() == arrays.level_max and apr.level_min() == arrays.level_min
    return apr
