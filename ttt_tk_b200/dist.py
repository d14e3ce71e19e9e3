"""Multi-GPU use of the operator: one process per GPU, the (batch x head) streams of ONE problem
partitioned across the ranks.

The streams are independent (each touches only its own slices of every tensor; the reference's grid
index is (b, h): kernels/ttt/ttt.cu:106-107), so a rank runs the operator on its own streams with no
traffic on the per-stream path.  The flattened B*H streams are cut into `world` contiguous blocks of
whole heads: `world` = gb * gh, the batch elements are split gb ways and, inside each batch block,
the heads gh ways.  A rank's block is then a rectangle [b0:b1, h0:h1] of every [B, H, ...] tensor,
which the operator takes as a contiguous [B', H', ...] problem of its own.

The single exchange is the sum over ranks of the per-head norm gradients, which the operator emits as
one row per batch element ([B, H, 1, 64]; kernels/ttt_backward/ttt.cu:1437-1438 of the reference,
summed by the caller at kernels/ttt_backward/matching.py:522-523): every rank adds its rows into its
own heads of a zero-filled [2, H, 64] buffer and ONE all-reduce sums the buffers.  Ranks that share a
head (batch split) are summed by it, ranks that own different heads (head split) are merged by it.
"""

import torch
import torch.distributed as dist


def shard_bounds(n, rank, world):
    """Contiguous block [lo, hi) of `n` items for `rank` of `world` (sizes differ by at most 1)."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def stream_grid(B, H, world):
    """(gb, gh) with gb * gh == world: the batch axis is cut gb ways, the head axis gh ways.  The batch
    axis is cut first (ranks that own whole heads of whole batch elements need nothing else); the
    heads are cut only when there are more ranks than batch elements can feed."""
    if world < 1:
        raise ValueError("world must be >= 1")
    best = None
    for gb in range(min(B, world), 0, -1):
        if world % gb:
            continue
        gh = world // gb
        if gh > H:
            continue
        # prefer even blocks; among those the widest batch split
        uneven = (B % gb != 0) + (H % gh != 0)
        key = (uneven, -gb)
        if best is None or key < best[0]:
            best = (key, gb, gh)
    if best is None:
        raise ValueError(f"cannot place {world} ranks on B={B} x H={H} streams (more ranks than streams?)")
    return best[1], best[2]


def shard_streams(B, H, rank, world):
    """This rank's rectangle (b0, b1, h0, h1) of the (batch x head) streams of one problem."""
    gb, gh = stream_grid(B, H, world)
    rb, rh = divmod(rank, gh)
    b0, b1 = shard_bounds(B, rb, gb)
    h0, h1 = shard_bounds(H, rh, gh)
    return b0, b1, h0, h1


def shard_tensors(tensors, rank, world):
    """Slice every tensor of one problem to this rank's streams.  Tensors with a batch dimension
    ([B, H, ...]) are cut to [b0:b1, h0:h1]; per-head tensors ([1, H, ...], the norm weight / bias) to
    [:, h0:h1].  Returns (shard dict of contiguous tensors, (b0, b1, h0, h1))."""
    B, H = tensors["XQ"].shape[:2]
    b0, b1, h0, h1 = shard_streams(B, H, rank, world)
    out = {}
    for k, v in tensors.items():
        if v.dim() >= 2 and v.shape[1] == H and v.shape[0] in (1, B):
            per_head_only = k.startswith("ttt_norm")       # [1, H, 1, 64]: shared by all batch elements
            out[k] = (v[:, h0:h1] if per_head_only else v[b0:b1, h0:h1]).contiguous()
        else:
            out[k] = v
    return out, (b0, b1, h0, h1)


def shard_batch(tensors, rank, world, batch_keys=None):
    """Batch-only split (every rank keeps all heads): slice every tensor that has a batch dimension
    (dim 0 of size B) to this rank's batch block.  Per-head tensors [1, H, ...] are shared."""
    B = tensors["XQ"].shape[0]
    lo, hi = shard_bounds(B, rank, world)
    out = {}
    for k, v in tensors.items():
        shared = v.shape[0] == 1 and B != 1 if batch_keys is None else k not in batch_keys
        out[k] = v if shared else v[lo:hi].contiguous()
    return out


def reduce_norm_grads(grad_weight, grad_bias, group=None, heads=None, total_heads=None):
    """Sum the per-batch-element rows locally, then across ranks with ONE all-reduce of a packed
    [2, H, 64] buffer.  `heads` = (h0, h1) and `total_heads` = H place a rank that owns only some of the
    heads (its tensors are [B', h1 - h0, 1, 64]); by default the rank owns all heads.
    Returns (grad_weight, grad_bias) of the whole problem, shape [1, H, 1, 64], on every rank."""
    Hl = grad_weight.shape[1]
    h0, h1 = (0, Hl) if heads is None else heads
    H = Hl if total_heads is None else total_heads
    if h1 - h0 != Hl or h1 > H:
        raise ValueError("heads do not match the gradient tensors")
    local = torch.stack([grad_weight.sum(dim=0).reshape(Hl, 64), grad_bias.sum(dim=0).reshape(Hl, 64)])
    if Hl == H:
        packed = local
    else:
        packed = torch.zeros(2, H, 64, dtype=local.dtype, device=local.device)
        packed[:, h0:h1] = local
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
    return packed[0].reshape(1, H, 1, 64), packed[1].reshape(1, H, 1, 64)
