"""Multi-GPU use of the operator: one process per GPU, (batch x head) streams sharded.

The streams are independent (each touches only its own slices of every tensor), so a rank runs
the operator on its own shard with no traffic on the per-stream path.  The single exchange is the
sum over batch shards of the per-head norm gradients, which the operator emits as one row per
batch element ([B, H, 1, 64]; kernels/ttt_backward/ttt.cu:1437-1438 of the reference, summed by
the caller at kernels/ttt_backward/matching.py:522-523).
"""
import torch
import torch.distributed as dist


def shard_bounds(n, rank, world):
    """Contiguous block [lo, hi) of `n` items for `rank` of `world` (sizes differ by at most 1)."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_batch(tensors, rank, world, batch_keys=None):
    """Slice every tensor that has a batch dimension (dim 0 of size B) to this rank's batch shard.
    Per-head tensors of shape [1, H, ...] (norm weight / bias) are shared by all ranks."""
    B = tensors["XQ"].shape[0]
    lo, hi = shard_bounds(B, rank, world)
    out = {}
    for k, v in tensors.items():
        shared = v.shape[0] == 1 and B != 1 if batch_keys is None else k not in batch_keys
        out[k] = v if shared else v[lo:hi].contiguous()
    return out


def reduce_norm_grads(grad_weight, grad_bias, group=None):
    """Sum the per-batch-element rows locally, then across ranks with ONE all-reduce of a packed
    [2, H, 64] buffer.  Returns (grad_weight, grad_bias) with shape [1, H, 1, 64]."""
    H = grad_weight.shape[1]
    packed = torch.stack([grad_weight.sum(dim=0).reshape(H, 64), grad_bias.sum(dim=0).reshape(H, 64)])
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
    return packed[0].reshape(1, H, 1, 64), packed[1].reshape(1, H, 1, 64)
