"""Fused GroupNorm + ReLU for (batch, channels, particles) feature tensors.

Not part of the reference's `aprnet` API: its network blocks apply `torch.nn.GroupNorm` and `nn.ReLU`
after every convolution (apr_models/apr_models/unet/unet_parts.py:18-26).  `GroupNormReLU` computes the
same function (parameters `weight` / `bias` like `nn.GroupNorm`, so state dicts interchange) with
kernels sized for tens of millions of particles per row; the ReLU mask is recomputed in the backward
pass, so only the input and the per-group statistics are kept for it.
"""
import torch
from torch import nn
from torch.autograd import Function

from _pyaprwrapper.aprnet.cuda import groupnorm_relu_backward, groupnorm_relu_forward


class GroupNormReLUFunction(Function):
    @staticmethod
    def forward(ctx, x, weight, bias, groups, eps, relu):
        x = x.contiguous()
        y, mean, rstd = groupnorm_relu_forward(x, weight, bias, groups, eps, relu)
        ctx.save_for_backward(x, weight, bias, mean, rstd)
        ctx.groups, ctx.relu = groups, relu
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, weight, bias, mean, rstd = ctx.saved_tensors
        dx, dgamma, dbeta = groupnorm_relu_backward(x, grad_y.contiguous(), weight, bias, mean, rstd, ctx.groups, ctx.relu)
        return dx, (dgamma if weight is not None else None), (dbeta if bias is not None else None), None, None, None


class GroupNormReLU(nn.Module):
    def __init__(self, num_groups, num_channels, eps=1e-5, affine=True, relu=True):
        super().__init__()
        assert num_channels % num_groups == 0
        self.num_groups, self.num_channels, self.eps, self.relu = num_groups, num_channels, eps, relu
        self.weight = nn.Parameter(torch.ones(num_channels)) if affine else None
        self.bias = nn.Parameter(torch.zeros(num_channels)) if affine else None

    def extra_repr(self):
        return '{}, {}, eps={}, relu={}'.format(self.num_groups, self.num_channels, self.eps, self.relu)

    def forward(self, x):
        return GroupNormReLUFunction.apply(x, self.weight, self.bias, self.num_groups, self.eps, self.relu)
