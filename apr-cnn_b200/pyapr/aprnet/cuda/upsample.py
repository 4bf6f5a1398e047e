"""`UpSampleConst`: the inverse move of `MaxPool` — features of level delta d are carried to d - 1, every
particle and node of the restored level taking the value of its parent node
(reference module: pyapr/aprnet/cuda/upsample.py:8-38)."""
from torch import nn
from torch.autograd import Function

from _pyaprwrapper import aprnet as _ext
from _pyaprwrapper.data_containers import APRPtrVector


class _NearestParent(Function):
    """Forward copies parent values down; backward sums the children's gradients into the parent."""

    @staticmethod
    def forward(ctx, coarse, apr_list, deltas, step_deltas):
        ctx.apr_list = apr_list
        ctx.deltas_at_call = deltas.clone()               # the shared tensor is changed below
        fine = _ext.cuda.upsample_const_forward(APRPtrVector(apr_list), coarse, deltas)
        if step_deltas:
            deltas.sub_(1)                                # callers thread one level_deltas tensor through the network
        return fine

    @staticmethod
    def backward(ctx, grad_fine):
        grad_coarse = _ext.cuda.upsample_const_backward(APRPtrVector(ctx.apr_list), grad_fine.contiguous(), ctx.deltas_at_call)
        return grad_coarse, None, None, None


class UpSampleConst(nn.Module):
    def __init__(self):
        super().__init__()
        # the shared level_deltas tensor is decremented after the call unless this is cleared (see MaxPool)
        self.decrement_level_deltas = True

    def forward(self, input_features, aprs, level_deltas):
        return _NearestParent.apply(input_features, aprs, level_deltas, self.decrement_level_deltas)
