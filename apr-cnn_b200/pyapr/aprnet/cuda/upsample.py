"""`UpSampleConst`: restore the next finer level by nearest-parent copy
(reference: pyapr/aprnet/cuda/upsample.py:8-38)."""
from torch import nn
from torch.autograd import Function

from _pyaprwrapper.data_containers import APRPtrVector
from _pyaprwrapper.aprnet.cuda import upsample_const_backward, upsample_const_forward


class UpsampleConstFunction(Function):
    @staticmethod
    def forward(ctx, inputs, aprs, level_deltas, decrement_level_deltas):
        ctx.aprs = aprs
        ctx.save_for_backward(level_deltas.clone())
        output = upsample_const_forward(APRPtrVector(aprs), inputs, level_deltas)
        if decrement_level_deltas:
            level_deltas.sub_(1)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        level_deltas, = ctx.saved_tensors
        grad_input = upsample_const_backward(APRPtrVector(ctx.aprs), grad_output.contiguous(), level_deltas)
        return grad_input, None, None, None


class UpSampleConst(nn.Module):
    def __init__(self):
        super().__init__()
        # When True the shared level_deltas tensor is decremented after the call (see MaxPool).
        self.decrement_level_deltas = True

    def forward(self, input_features, aprs, level_deltas):
        return UpsampleConstFunction.apply(input_features, aprs, level_deltas, self.decrement_level_deltas)
