"""Column-parallel sharding of a quantized linear layer over the ranks of one node.

Only the output-feature dimension shards (rows of W[out,in], a contiguous slab of the packed
buffer: crates/nsl-runtime/src/tensor_parallel/sharding.rs:18-58 of NSL).  x and its
quantisation are replicated, so every rank's int32 accumulators equal the unsharded ones; the
one exchange step is an all-gather of the [M, N/G] outputs
(crates/nsl-runtime/src/tensor_parallel/collective.rs:1061).
"""
import torch
import torch.distributed as dist

from .ops import shard_rows


def shard_weight_rows(weight_rows, world, rank):
    """Rows [row0, row0+rows) of a per-output-row tensor (packed weight, scales, zero points)."""
    r0, n = shard_rows(weight_rows.shape[0], world, rank)
    return weight_rows[r0:r0 + n].contiguous()


def gather_buffer(M, n_local, world, dtype, device):
    return torch.empty(world, M, n_local, dtype=dtype, device=device)


def all_gather_columns(y_local, gathered=None, group=None):
    """All-gathers [M, N/G] shards.  Returns the [G, M, N/G] buffer: for M == 1 its memory is
    already y[N]; `assemble` gives the [M, N] view/copy for M > 1."""
    world = dist.get_world_size(group)
    if gathered is None:
        gathered = gather_buffer(y_local.shape[0], y_local.shape[1], world, y_local.dtype, y_local.device)
    # concatenation along dim 0 of the [M, N/G] shards is exactly the [G, M, N/G] buffer
    dist.all_gather_into_tensor(gathered.view(world * y_local.shape[0], y_local.shape[1]), y_local, group=group)
    return gathered


def assemble(gathered):
    """[G, M, N/G] -> [M, N] (a view when M == 1)."""
    G, M, n = gathered.shape
    if M == 1:
        return gathered.reshape(1, G * n)
    return gathered.permute(1, 0, 2).reshape(M, G * n)
