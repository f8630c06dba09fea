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


def row_shard(m_total: int, world: int, rank: int, align: int = 16) -> tuple[int, int]:
    """[begin, end) of the rows of the replicated A that `rank` brings to the
    device from its host before the ranks exchange them (same split as
    column_shard)."""
    return column_shard(m_total, world, rank, align)


def gather_replicated_rows(a_full_dev, a_host, dist, rank: int, world: int, group=None):
    """Fills `a_full_dev` (device, [M, K]) with the replicated operand A, of
    which every rank holds a host copy `a_host` (pinned, [M, K]): each rank
    copies only its M/world rows over PCIe and the ranks exchange them with
    one all-gather over NVLink, so that the host links carry A once in total
    instead of once per GPU.  With one rank it is a plain copy."""
    if world == 1:
        a_full_dev.copy_(a_host, non_blocking=True)
        return
    m_total = a_full_dev.shape[0]
    if m_total % (16 * world):
        raise ValueError(f"M must be a multiple of {16 * world} for an even row exchange; got {m_total}")
    r0, r1 = row_shard(m_total, world, rank)
    a_full_dev[r0:r1].copy_(a_host[r0:r1], non_blocking=True)
    # bytes, so that 16-bit patterns held in any torch dtype travel (NCCL has no int16)
    import torch
    dist.all_gather_into_tensor(a_full_dev.reshape(-1).view(torch.uint8), a_full_dev[r0:r1].reshape(-1).view(torch.uint8),
                                group=group)


def sharded_gemm_host(wc, desc_shard, a_full_dev, a_host, b_host_shard, c_host_shard, dist, rank: int, world: int,
                      stream: int, group=None) -> None:
    """One rank's part of C = A * B^T with B and C split by N-column blocks and
    every operand starting and ending in (pinned) host memory: A reaches the
    device by gather_replicated_rows, the rank's B block and C block travel
    through the library's host-buffer call.  `desc_shard` describes the rank's
    block (N = its columns; column-major C makes the block contiguous,
    python/mlir/dialects/wave_matmul.py:1040)."""
    gather_replicated_rows(a_full_dev, a_host, dist, rank, world, group)
    wc.gemm_host_a_resident(desc_shard, a_full_dev.data_ptr(), b_host_shard.data_ptr(), c_host_shard.data_ptr(),
                            stream)


class PeerMappedOutput:
    """Every rank's copy of a full output tensor, allocated so that each rank
    can address all of them (torch's symmetric memory: the ranks' buffers are
    mapped into one another's address space over NVLink).  It is what
    wave_cuda_gemm_multi_output writes the column blocks into: rank r passes
    `block_targets(r, offset)` -- the place of ITS block inside every rank's
    copy, its own copy first -- and the all-gather happens inside the GEMM
    kernel.  `settle(stream_tensor)` is the barrier after which a rank may read
    its copy: a one-element all-reduce ordered on the current stream behind the
    kernel (no host synchronisation)."""

    def __init__(self, shape, dtype, dist, rank: int, world: int, device=None):
        import torch
        import torch.distributed._symmetric_memory as symm
        self.dist, self.rank, self.world = dist, rank, world
        self.local = symm.empty(*tuple(shape), dtype=dtype,
                                device=device or torch.device("cuda", torch.cuda.current_device()))
        self.handle = symm.rendezvous(self.local, dist.group.WORLD)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(self.ptrs) != world or self.ptrs[rank] != self.local.data_ptr():
            raise RuntimeError("symmetric memory returned an unexpected set of buffer addresses")
        # 0 where the system has no NVLink multicast (NVLS) for this group
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self._token = torch.zeros(1, device=self.local.device, dtype=torch.float32)

    def block_targets(self, offset_bytes: int) -> list[int]:
        """Addresses `offset_bytes` into every rank's copy, this rank's first."""
        order = [self.rank] + [r for r in range(self.world) if r != self.rank]
        return [self.ptrs[r] + offset_bytes for r in order]

    def settle(self) -> None:
        self.dist.all_reduce(self._token)
