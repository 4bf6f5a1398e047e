"""`MaxPool`: drop the current finest level (reference: pyapr/aprnet/cuda/maxpool.py:8-40)."""
from torch import nn
from torch.autograd import Function

from _pyaprwrapper.data_containers import APRPtrVector
from _pyaprwrapper.aprnet.cuda import maxpool_backward_cuda, maxpool_forward_cuda


class MaxPoolFunction(Function):
    @staticmethod
    def forward(ctx, inputs, aprs, level_deltas, increment_level_deltas):
        output, max_indices = maxpool_forward_cuda(APRPtrVector(aprs), inputs, level_deltas)
        ctx.aprs = aprs
        ctx.save_for_backward(max_indices, level_deltas.clone())
        if increment_level_deltas:
            level_deltas.add_(1)        # shared state: later layers see the pooled resolution
        return output

    @staticmethod
    def backward(ctx, grad_output):
        max_indices, level_deltas = ctx.saved_tensors
        grad_input = maxpool_backward_cuda(APRPtrVector(ctx.aprs), grad_output.contiguous(), max_indices, level_deltas)
        return grad_input, None, None, None


class MaxPool(nn.Module):
    def __init__(self):
        super().__init__()
        # When True the shared level_deltas tensor is incremented after the call.  Set to False when the
        # module is called repeatedly on the same input (e.g. numerical gradient checks).
        self.increment_level_deltas = True

    def forward(self, input_features, aprs, level_deltas):
        return MaxPoolFunction.apply(input_features, aprs, level_deltas, self.increment_level_deltas)
