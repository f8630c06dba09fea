"""Multi-GPU partitioning of the two kernels (one process per GPU).

Neither kernel exchanges data while it computes.  The GEMM is split by
N-column blocks: B is stored N x K, so a rank's block of columns is a
contiguous block of B's rows, A is replicated, and in the reference's
column-major output layout (python/mlir/dialects/wave_matmul.py:1040,
offset = n*M + m) the rank's block of C is contiguous too.  Attention is
split by (batch, head): contiguous slabs of the [B*H][S][D] layout
(python/mlir/dialects/wave_flash_attention.py:242-254).  A collective
(all-gather) is used only when the caller wants the whole output on every rank.
"""
from __future__ import annotations


def column_shard(n_total: int, world: int, rank: int, align: int = 16) -> tuple[int, int]:
    """[begin, end) of the N columns owned by `rank`: as equal as possible in
    units of `align` columns (the kernels need multiples of 16)."""
    if n_total % align:
        raise ValueError(f"N must be a multiple of {align}; got {n_total}")
    if not 0 <= rank < world:
        raise ValueError(f"rank must be in [0, {world}); got {rank}")
    units = n_total // align
    q, r = divmod(units, world)
    begin = rank * q + min(rank, r)
    end = begin + q + (1 if rank < r else 0)
    return begin * align, end * align


def head_shard(batch_heads: int, world: int, rank: int) -> tuple[int, int]:
    """[begin, end) of the (batch*head) slabs owned by `rank`."""
    if not 0 <= rank < world:
        raise ValueError(f"rank must be in [0, {world}); got {rank}")
    q, r = divmod(batch_heads, world)
    begin = rank * q + min(rank, r)
    return begin, begin + q + (1 if rank < r else 0)


def all_gather_shards(local, dist, group=None):
    """Gathers equally sized contiguous shards (column-major C blocks, or O
    slabs) from every rank into one tensor ordered by rank.  `dist` is
    torch.distributed; works with nccl (GPU tensors) and gloo (CPU tensors)."""
    import torch
    world = dist.get_world_size(group)
    local = local.contiguous()
    flat = torch.empty(world * local.numel(), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, local.reshape(-1), group=group)
    return flat.reshape((world,) + tuple(local.shape))
