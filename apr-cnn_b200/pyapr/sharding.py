"""Splitting work over GPUs: independent APRs are dealt to ranks, weight gradients are averaged.

The reference has no multi-GPU support (its batch is a sequential host loop on one device,
pyapr/aprnet/cuda/src/wrap_conv_gpu.hpp:23-28).  Independent APRs need no data-path collective: each
rank runs the operators on its own APRs; only the (small) weight gradients are all-reduced when
training.  Works with any initialised torch.distributed backend (NCCL on GPUs, gloo in CPU tests).
"""
import torch


def shard_indices(n_items, rank, world, weights=None):
    """Indices of the items owned by `rank`.

    Without weights: round-robin (item i -> rank i mod world, the split named for batches of APRs).
    With weights (e.g. particle counts): greedy longest-processing-time assignment so that the ranks'
    total weights are balanced; deterministic, every rank computes the same partition."""
    if weights is None:
        return list(range(rank, n_items, world))
    order = sorted(range(n_items), key=lambda i: (-weights[i], i))
    loads = [0] * world
    owner = [0] * n_items
    for i in order:
        r = min(range(world), key=lambda k: (loads[k], k))
        owner[i] = r
        loads[r] += weights[i]
    return [i for i in range(n_items) if owner[i] == rank]


def allreduce_gradients(params, world):
    """Average the gradients of `params` over all ranks with one flat all-reduce."""
    import torch.distributed as dist
    grads = [p.grad for p in params if p.grad is not None]
    if world <= 1 or not grads:
        return
    flat = torch.cat([g.reshape(-1) for g in grads])
    dist.all_reduce(flat)
    flat /= world
    off = 0
    for g in grads:
        g.copy_(flat[off:off + g.numel()].view_as(g))
        off += g.numel()
