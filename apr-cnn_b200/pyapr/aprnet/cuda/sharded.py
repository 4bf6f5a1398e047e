"""Operator modules for ONE APR cut into z-slabs, one slab per GPU (`pyapr.sharding.zslab_plan`).

The reference has no multi-GPU path.  These modules keep the reference's module interface
(`APRConv(in, out, nstencils, kernel_size, bias)(features, aprs, level_deltas)` etc., pyapr/aprnet/cuda/conv.py:66-94)
so that the same network code runs on a slab: `make_ops(shard)` returns a namespace to build the network from.

What differs from the single-GPU modules:

* `APRConv` with the 3x3x3 stencil: local tree fill -> halo exchange of features and tree means (owners to
  halos) -> gather convolution -> halo outputs cleared.  Backward: direct input gradient and tree gradient ->
  reverse exchange (halo parts added at their owners) -> tree adjoint.  The weight gradient of a rank covers
  the locations it owns; the ranks' gradients are SUMMED afterwards (`pyapr.sharding.allreduce_gradients`
  with average=False).
* `GroupNormReLU`: per-channel sums over the owned locations, one small all-reduce, then the same fused
  apply kernels; likewise in the backward pass.
* 1x1x1 convolution, max-pooling and up-sampling are the single-GPU modules: they never read across a slab
  boundary (halo entries carry values that the next exchange overwrites).

Invariants the modules keep: halo entries of every 3x3x3 convolution output and of every GroupNorm input are
zero; halo entries of every activation gradient are cleared in place when a module of this file receives it,
and the gradients these modules return are zero at halo entries (so the unchanged modules between them -- 1x1x1
convolution, pooling, up-sampling, concatenation -- never see a contribution from a location the rank does not own).
"""
import types

import torch
from torch import nn
from torch.autograd import Function


class GpuBackend:
    """The operator calls of this package (extension module `_pyaprwrapper.aprnet.cuda`)."""

    def __init__(self):
        from _pyaprwrapper.aprnet import cuda as C
        from _pyaprwrapper.data_containers import APRPtrVector
        self.C, self.vec = C, APRPtrVector

    def restrict_forward(self, w, num_levels):
        return self.C.restrict_kernel333_forward(w, num_levels)

    def restrict_backward(self, gw, num_stencils):
        return self.C.restrict_kernel333_backward(gw, num_stencils)

    def fill_tree(self, aprs, x, ld):
        return self.C.fill_tree_mean_batch(self.vec(aprs), x, ld)

    def conv_forward(self, aprs, x, tree, w, ld, precision=None):
        return self.C.conv333_forward_pretree(self.vec(aprs), x, tree, w, ld, precision or "")

    def conv_backward(self, aprs, x, tree, kept, w, go, ld, need_grad_input):
        return self.C.conv333_backward_pretree(self.vec(aprs), x, tree, kept, w, go, ld, need_grad_input)

    def tree_adjoint_(self, aprs, gi, gtree, ld):
        self.C.fill_tree_mean_backward_inplace(self.vec(aprs), gi, gtree, ld)

    def gn_row_sums(self, x):
        return self.C.groupnorm_row_sums(x)

    def gn_apply(self, x, gamma, beta, mean, rstd, groups, relu):
        return self.C.groupnorm_relu_apply(x, gamma, beta, mean, rstd, groups, relu)

    def gn_backward_row_sums(self, x, gy, gamma, beta, mean, rstd, groups, relu):
        return self.C.groupnorm_backward_row_sums(x, gy, gamma, beta, mean, rstd, groups, relu)

    def gn_backward_apply(self, x, gy, gamma, beta, mean, rstd, terms, groups, relu):
        return self.C.groupnorm_backward_apply(x, gy, gamma, beta, mean, rstd, terms, groups, relu)


class Shard:
    """One rank's slab: the plan, the halo exchange on a device and the operator backend."""

    def __init__(self, plan, device, backend=None, group=None):
        from pyapr.sharding import HaloExchange
        self.plan, self.device, self.group = plan, device, group
        self.halo = HaloExchange(plan, device, group)
        self.backend = backend if backend is not None else GpuBackend()
        self._by_len = {L.n_local: dl for dl, L in plan.lists.items()}
        if len(self._by_len) != len(plan.lists):
            raise ValueError("two level deltas of this slab have feature vectors of the same length")

    def level_delta_of(self, n):
        """Level delta of a feature tensor from its length (each level delta has its own length)."""
        if n not in self._by_len:
            raise RuntimeError("a feature tensor of length %d matches no level delta of the slab plan" % n)
        return self._by_len[n]

    def n_global(self, dl):
        return self.plan.lists[dl].n_global

    def all_reduce(self, t):
        import torch.distributed as dist
        if self.plan.world > 1:
            dist.all_reduce(t, group=self.group)
        return t


class ShardedConv333Function(Function):
    @staticmethod
    def forward(ctx, inputs, weights, bias, aprs, level_deltas, shard, precision=None):
        B = shard.backend
        assert len(aprs) == 1 and inputs.shape[0] == 1, "one APR (slab) per rank"
        dl = int(level_deltas[0])
        num_levels = max(a.level_max() - a.level_min() + 1 for a in aprs)
        expanded = B.restrict_forward(weights, num_levels)
        inputs = inputs.contiguous()
        tree = B.fill_tree(aprs, inputs, level_deltas)
        shard.halo.forward(dl, inputs, tree)                 # halo entries of input and tree now hold their owners' values
        out, kept = B.conv_forward(aprs, inputs, tree, expanded, level_deltas) if precision is None else \
            B.conv_forward(aprs, inputs, tree, expanded, level_deltas, precision)
        if bias is not None:
            out = out + bias.view(1, -1, 1)
        shard.halo.zero_halo(dl, out)
        ctx.aprs, ctx.shard, ctx.dl, ctx.num_stencils = aprs, shard, dl, weights.shape[0]
        ctx.packed = kept.numel() > 0
        ctx.tree_shape = tuple(tree.shape)
        if ctx.packed:          # the packed rows hold input and tree means; neither is needed again
            ctx.save_for_backward(kept, expanded, bias, level_deltas.clone())
        else:
            ctx.save_for_backward(inputs, tree, expanded, bias, level_deltas.clone())
        return out

    @staticmethod
    def backward(ctx, grad_output):
        shard, B, dl = ctx.shard, ctx.shard.backend, ctx.dl
        grad_output = grad_output.contiguous()
        shard.halo.zero_halo(dl, grad_output)                # outputs at halo locations belong to the neighbour
        need_gi = bool(ctx.needs_input_grad[0])
        if ctx.packed:
            kept, expanded, bias, ld = ctx.saved_tensors
            inputs = kept.new_empty((0,))
            tree = grad_output.new_empty(ctx.tree_shape)     # shape only: the packed rows carry the values
        else:
            inputs, tree, expanded, bias, ld = ctx.saved_tensors
            kept = inputs.new_empty((0,), dtype=torch.uint8)
        gi, gtree, gwe = B.conv_backward(ctx.aprs, inputs, tree, kept, expanded, grad_output, ld, need_gi)
        if need_gi:
            shard.halo.reverse(dl, gi, gtree)                # halo parts go to their owners
            B.tree_adjoint_(ctx.aprs, gi, gtree, ld)
        else:
            gi = None
        gw = B.restrict_backward(gwe, ctx.num_stencils)
        gb = grad_output.sum(dim=(0, 2)) if bias is not None else None
        return gi, gw, gb, None, None, None, None


class ShardedGroupNormReLUFunction(Function):
    @staticmethod
    def forward(ctx, x, weight, bias, groups, eps, relu, shard):
        B = shard.backend
        x = x.contiguous()
        assert x.shape[0] == 1, "one APR (slab) per rank"
        C = x.shape[1]
        dl = shard.level_delta_of(x.shape[2])
        shard.halo.zero_halo(dl, x)                          # halo entries must not count (a 1x1x1 convolution leaves values there)
        sums = B.gn_row_sums(x).view(groups, C // groups, 2).sum(dim=1)          # (G, 2) float64, owned locations only
        shard.all_reduce(sums)
        m = float(C // groups) * float(shard.n_global(dl))
        mean = sums[:, 0] / m
        var = (sums[:, 1] / m - mean * mean).clamp_min(0.0)
        rstd = torch.rsqrt(var + eps)
        mean, rstd = mean.to(x.dtype).contiguous(), rstd.to(x.dtype).contiguous()
        y = B.gn_apply(x, weight, bias, mean, rstd, groups, relu)
        ctx.save_for_backward(x, weight, bias, mean, rstd)
        ctx.groups, ctx.relu, ctx.shard, ctx.dl, ctx.m = groups, relu, shard, dl, m
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, weight, bias, mean, rstd = ctx.saved_tensors
        shard, B, groups = ctx.shard, ctx.shard.backend, ctx.groups
        grad_y = grad_y.contiguous()
        shard.halo.zero_halo(ctx.dl, grad_y)
        C = x.shape[1]
        rs = B.gn_backward_row_sums(x, grad_y, weight, bias, mean, rstd, groups, ctx.relu)      # (C, 2): sum dy, sum dy * xhat
        gamma = weight.double() if weight is not None else torch.ones(C, dtype=torch.float64, device=x.device)
        terms = (rs * gamma[:, None]).view(groups, C // groups, 2).sum(dim=1)
        shard.all_reduce(terms)
        terms = (terms / ctx.m).to(x.dtype).contiguous()
        dx = B.gn_backward_apply(x, grad_y, weight, bias, mean, rstd, terms, groups, ctx.relu)
        shard.halo.zero_halo(ctx.dl, dx)                     # the mean terms are non-zero everywhere; halo gradients must stay zero
        dgamma = rs[:, 1].to(x.dtype) if weight is not None else None
        dbeta = rs[:, 0].to(x.dtype) if bias is not None else None
        return dx, dgamma, dbeta, None, None, None, None


def sharded_cross_entropy(logits, labels, shard):
    """Mean cross-entropy over the particles of the WHOLE APR: this rank's part of the sum (halo entries
    excluded) divided by the global particle count.  Returns (local loss for backward, all-reduced value)."""
    owned = torch.from_numpy(shard.plan.owned_particles).to(logits.device)
    per = torch.nn.functional.cross_entropy(logits, labels, reduction="none")        # (1, N)
    local = (per[0] * owned).sum() / float(shard.plan.n_particles_global)
    total = shard.all_reduce(local.detach().clone())
    return local, total


def make_ops(shard):
    """Namespace with the module classes to build a network for one slab."""
    from . import conv as _conv
    from .maxpool import MaxPool
    from .upsample import UpSampleConst

    class APRConv(_conv.APRConv):
        def forward(self, input_features, aprs, level_deltas):
            if self.kernel_size == (3, 3, 3):
                return ShardedConv333Function.apply(input_features, self.weight, self.bias, aprs, level_deltas, shard, self.precision)
            return super().forward(input_features, aprs, level_deltas)

    class GroupNormReLU(nn.Module):
        def __init__(self, num_groups, num_channels, eps=1e-5, affine=True, relu=True):
            super().__init__()
            assert num_channels % num_groups == 0
            self.num_groups, self.num_channels, self.eps, self.relu = num_groups, num_channels, eps, relu
            self.weight = nn.Parameter(torch.ones(num_channels)) if affine else None
            self.bias = nn.Parameter(torch.zeros(num_channels)) if affine else None

        def forward(self, x):
            return ShardedGroupNormReLUFunction.apply(x, self.weight, self.bias, self.num_groups, self.eps, self.relu, shard)

    return types.SimpleNamespace(APRConv=APRConv, MaxPool=MaxPool, UpSampleConst=UpSampleConst, GroupNormReLU=GroupNormReLU)
