"""`APRConv` with 3x3x3 and 1x1x1 stencils (reference: pyapr/aprnet/cuda/conv.py:12-94).

Same constructor, parameter shapes (`weight`: (nstencils, out, in, k, k, k), `bias`: (out,)),
initialisation and forward signature `(features, aprs, level_deltas)` as the reference module, so
checkpoints and calling code interchange.
"""
import math

import torch
from torch import nn
from torch.autograd import Function
from torch.nn import init

from _pyaprwrapper.data_containers import APRPtrVector
from _pyaprwrapper.aprnet.cuda import (conv111_backward, conv111_forward, conv333_backward_with_rows, conv333_backward_with_tree,
                                       conv333_forward_keep_rows, conv333_forward_keep_tree, get_conv_precision,
                                       restrict_kernel333_backward, restrict_kernel333_forward)


class Conv333Function(Function):
    """3x3x3 stencil: the given stencils are expanded to one per level, then applied per level."""

    @staticmethod
    def forward(ctx, inputs, weights, bias, aprs, level_deltas, precision=None):
        num_levels = max(a.level_max() - a.level_min() + 1 for a in aprs)
        expanded = restrict_kernel333_forward(weights, num_levels)
        ctx.aprs = aprs
        ctx.num_stencils = weights.shape[0]
        # arithmetic of this layer: the module's own setting, else the process-wide one
        ctx.packed = (precision or get_conv_precision()) == "bf16" and inputs.dtype == torch.float32
        if ctx.packed:
            # tensor-core path: the backward pass works from the packed bf16 rows of the input (particles + tree
            # means) that the forward pass produced anyway; they replace the fp32 input among the saved tensors
            # (half the bytes) and spare the backward pass the tree fill and the packing
            out, rows = conv333_forward_keep_rows(APRPtrVector(aprs), inputs, expanded, level_deltas)
            ctx.save_for_backward(expanded, bias, level_deltas.clone(), rows)
        else:
            # the tree means computed by the forward pass are kept (1/7 of the input's size) so that the
            # backward pass does not have to fill the tree again
            out, tree = conv333_forward_keep_tree(APRPtrVector(aprs), inputs, expanded, level_deltas, "fp32")
            ctx.save_for_backward(inputs, expanded, bias, level_deltas.clone(), tree)
        if bias is not None:
            out = out + bias.view(1, -1, 1)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        grad_output = grad_output.contiguous()
        if ctx.packed:
            expanded, bias, level_deltas, rows = ctx.saved_tensors
            grad_input, grad_expanded = conv333_backward_with_rows(APRPtrVector(ctx.aprs), rows, expanded, grad_output, level_deltas,
                                                                   bool(ctx.needs_input_grad[0]))
            grad_weights = restrict_kernel333_backward(grad_expanded, ctx.num_stencils)
            grad_bias = grad_output.sum(dim=(0, 2)) if bias is not None else None
            return grad_input, grad_weights, grad_bias, None, None, None
        inputs, expanded, bias, level_deltas, tree = ctx.saved_tensors
        # the input gradient of a first layer (features that do not require grad) is not computed
        grad_input, grad_expanded = conv333_backward_with_tree(APRPtrVector(ctx.aprs), inputs, expanded, grad_output, level_deltas, tree,
                                                               bool(ctx.needs_input_grad[0]), "fp32")
        grad_weights = restrict_kernel333_backward(grad_expanded, ctx.num_stencils)
        grad_bias = grad_output.sum(dim=(0, 2)) if bias is not None else None
        return grad_input, grad_weights, grad_bias, None, None, None


class Conv111Function(Function):
    """1x1x1 stencil: a per-level channel mix, no neighbour access and no stencil expansion."""

    @staticmethod
    def forward(ctx, inputs, weights, bias, aprs, level_deltas, precision=None):
        ctx.aprs = aprs
        ctx.precision = precision or ""
        ctx.save_for_backward(inputs, weights, bias, level_deltas.clone())
        out = conv111_forward(APRPtrVector(aprs), inputs, weights, level_deltas, ctx.precision)
        if bias is not None:
            out = out + bias.view(1, -1, 1)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        inputs, weights, bias, level_deltas = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        grad_input, grad_weights = conv111_backward(APRPtrVector(ctx.aprs), inputs, weights, grad_output, level_deltas, ctx.precision)
        grad_bias = grad_output.sum(dim=(0, 2)) if bias is not None else None
        return grad_input, grad_weights, grad_bias, None, None, None


_FUNCTIONS = {(1, 1, 1): Conv111Function, (3, 3, 3): Conv333Function}


class APRConv(nn.Module):
    """`precision` (not in the reference): arithmetic of the layer on float32 tensors, "fp32" (CUDA-core kernels,
    exact) or "bf16" (tensor cores, bf16 operands with fp32 accumulation); None follows the process-wide setting
    (`set_conv_precision`)."""

    def __init__(self, in_channels, out_channels, nstencils=1, kernel_size=(3, 3, 3), bias=True, precision=None):
        super().__init__()
        assert precision in (None, "fp32", "bf16")
        self.precision = precision
        kernel_size = tuple(kernel_size)
        assert kernel_size in _FUNCTIONS, \
            'aprnet.cuda.APRConv currently only supports kernels of size (1, 1, 1) and (3, 3, 3)'
        self._function = _FUNCTIONS[kernel_size]
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.nstencils = nstencils
        self.kernel_size = kernel_size
        self.weight = nn.Parameter(torch.empty(nstencils, out_channels, in_channels, *kernel_size))
        self.bias = nn.Parameter(torch.empty(out_channels)) if bias else None
        self.reset_parameters()

    def extra_repr(self):
        return '{}, {}, kernel_size={}, nstencils={}, bias={}'.format(
            self.in_channels, self.out_channels, self.kernel_size, self.nstencils, self.bias is not None)

    def reset_parameters(self):
        init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            fan_in, _ = init._calculate_fan_in_and_fan_out(self.weight)
            bound = 1 / math.sqrt(fan_in)
            init.uniform_(self.bias, -bound, bound)

    def forward(self, input_features, aprs, level_deltas):
        return self._function.apply(input_features, self.weight, self.bias, aprs, level_deltas, self.precision)
