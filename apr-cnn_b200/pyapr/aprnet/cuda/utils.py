"""`Reconstruct` and `SampleParticles`: particle features <-> dense image at the resolution of
level_max - level_delta (reference: pyapr/aprnet/cuda/utils.py:10-55)."""
import torch
from torch import nn
from torch.autograd import Function

from _pyaprwrapper.data_containers import APRPtrVector
from _pyaprwrapper.aprnet.cuda import (reconstruct_backward, reconstruct_forward, sample_particles_backward,
                                       sample_particles_forward)


class ReconstructFunction(Function):
    """Piecewise-constant image from particle values; the adjoint sums the image gradient over each cell."""

    @staticmethod
    def forward(ctx, inputs, aprs, level_deltas):
        ctx.aprs = aprs
        ctx.save_for_backward(level_deltas.clone())
        return reconstruct_forward(APRPtrVector(aprs), inputs, level_deltas)

    @staticmethod
    def backward(ctx, grad_output):
        level_deltas, = ctx.saved_tensors
        return reconstruct_backward(APRPtrVector(ctx.aprs), grad_output.contiguous(), level_deltas), None, None


class Reconstruct(nn.Module):
    def forward(self, input_features, aprs, level_deltas=None):
        level_deltas = torch.zeros(len(aprs), dtype=torch.int32) if level_deltas is None else level_deltas
        return ReconstructFunction.apply(input_features, aprs, level_deltas)


class SampleParticlesFunction(Function):
    """Mean of the image over each particle's cell; the adjoint spreads value / cell volume over the cell."""

    @staticmethod
    def forward(ctx, inputs, aprs, level_deltas):
        ctx.aprs = aprs
        ctx.save_for_backward(level_deltas.clone())
        return sample_particles_forward(APRPtrVector(aprs), inputs, level_deltas)

    @staticmethod
    def backward(ctx, grad_output):
        level_deltas, = ctx.saved_tensors
        return sample_particles_backward(APRPtrVector(ctx.aprs), grad_output.contiguous(), level_deltas), None, None


class SampleParticles(nn.Module):
    def forward(self, input_features, aprs, level_deltas=None):
        level_deltas = torch.zeros(len(aprs), dtype=torch.int32) if level_deltas is None else level_deltas
        return SampleParticlesFunction.apply(input_features, aprs, level_deltas)
