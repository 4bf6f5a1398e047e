"""Dense-image bridges of the particle representation: `Reconstruct` paints every particle's cell into an
image at the resolution of level_max - level_delta, `SampleParticles` averages an image back onto the
cells (reference modules of the same names: pyapr/aprnet/cuda/utils.py:10-55)."""
import torch
from torch import nn
from torch.autograd import Function

from _pyaprwrapper import aprnet as _ext
from _pyaprwrapper.data_containers import APRPtrVector


class _ImageBridge(Function):
    """One autograd node for both directions.  `kind` selects the pair of extension calls: the backward of
    "reconstruct" sums the image gradient over each cell, the backward of "sample_particles" spreads
    value / cell volume over the cell."""

    @staticmethod
    def forward(ctx, features, apr_list, deltas, kind):
        ctx.kind, ctx.apr_list = kind, apr_list
        ctx.deltas = deltas.clone()
        return getattr(_ext.cuda, kind + "_forward")(APRPtrVector(apr_list), features, deltas)

    @staticmethod
    def backward(ctx, upstream):
        grad = getattr(_ext.cuda, ctx.kind + "_backward")(APRPtrVector(ctx.apr_list), upstream.contiguous(), ctx.deltas)
        return grad, None, None, None


def _default_deltas(apr_list, deltas):
    return deltas if deltas is not None else torch.zeros(len(apr_list), dtype=torch.int32)


class Reconstruct(nn.Module):
    """(B, C, N) particle features -> (B, C, Z, X, Y) piecewise-constant image."""

    def forward(self, input_features, aprs, level_deltas=None):
        return _ImageBridge.apply(input_features, aprs, _default_deltas(aprs, level_deltas), "reconstruct")


class SampleParticles(nn.Module):
    """(B, C, Z, X, Y) image -> (B, C, N) cell means."""

    def forward(self, input_features, aprs, level_deltas=None):
        return _ImageBridge.apply(input_features, aprs, _default_deltas(aprs, level_deltas), "sample_particles")
