"""How the operators shard over the GPUs of one node (one process per GPU, torch.distributed).

Every operator of the path splits into independent units, so ranks exchange nothing on the data path except
where the operator itself reduces over the split dimension:

* GEMM: B and C are split by columns (N), A is replicated; epilogue vectors (bias, column scales) follow the
  columns. A gathered C is an optional all-gather.
* convolution forward / backward data: the batch is split; the filter is replicated.
* convolution backward weight: the batch is split, every rank reduces its own images into a full-size partial
  filter gradient, and the partials are summed with one all-reduce (the only collective of the path).
* attention and GEMM+GEMM: the groups (batch x heads) are split.

The reference has no multi-GPU path (one kernel, one device: mlir/tools/rocmlir-gen/rocmlir-gen.cpp:2094-2124
emits single-device kernels); this module defines the partitioning a client needs to use N devices.

Functions take an explicit process group so they run under NCCL on GPUs and under gloo in CPU tests.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Shard:
    """Half-open range [begin, end) of a split dimension owned by one rank."""
    begin: int
    end: int

    @property
    def size(self) -> int:
        return self.end - self.begin


def shard_range(total: int, rank: int, world: int, granule: int = 1) -> Shard:
    """Contiguous, balanced split of `total` units in multiples of `granule` (the last rank takes the ragged
    rest). Ranks past the end of the data get an empty range."""
    if total < 0 or world <= 0 or not (0 <= rank < world) or granule <= 0:
        raise ValueError("shard_range: bad arguments")
    chunks = -(-total // granule)
    base, extra = divmod(chunks, world)
    first = rank * base + min(rank, extra)
    count = base + (1 if rank < extra else 0)
    begin = min(first * granule, total)
    end = min((first + count) * granule, total)
    return Shard(begin, end)


def gemm_column_shard(n: int, rank: int, world: int) -> Shard:
    """Columns of B and C owned by `rank`; multiples of 8 columns keep every 16-bit row pitch TMA-aligned."""
    return shard_range(n, rank, world, granule=8)


def conv_batch_shard(batch: int, rank: int, world: int) -> Shard:
    return shard_range(batch, rank, world)


def attention_group_shard(groups: int, rank: int, world: int) -> Shard:
    return shard_range(groups, rank, world)


def job_time_ms(local_ms: float, group: Optional[dist.ProcessGroup] = None, device=None) -> float:
    """A multi-rank job takes as long as its slowest rank: MAX over ranks of the device-timed duration."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(local_ms)
    t = torch.tensor([float(local_ms)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def allreduce_weight_gradient(partial: torch.Tensor, group: Optional[dist.ProcessGroup] = None, async_op: bool = False):
    """Sums the per-rank partial filter gradients of a batch-split backward-weight convolution in place.
    The partials should be f32 so that the sum over ranks rounds once at the caller's final conversion.
    With `async_op` the collective runs on the communication stream while the caller launches the next layer's
    kernels; the returned handle's wait() orders the caller's stream after it (None when there is nothing to do)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        work = dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
        return work if async_op else partial
    return None if async_op else partial


def gather_columns(c_local: torch.Tensor, n: int, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gathers a column-split C ([..., M, n_local] per rank) into [..., M, n] on every rank."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return c_local
    world = dist.get_world_size(group)
    shards = [gemm_column_shard(n, r, world) for r in range(world)]
    widest = max(s.size for s in shards)
    # all_gather wants equal shapes: pad the column dimension of the narrower shards
    padded = c_local.new_zeros(*c_local.shape[:-1], widest)
    padded[..., : c_local.shape[-1]] = c_local
    parts: List[torch.Tensor] = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded.contiguous(), group=group)
    return torch.cat([parts[r][..., : shards[r].size] for r in range(world)], dim=-1)


def covers_exactly(total: int, world: int, granule: int = 1) -> Tuple[bool, List[Shard]]:
    """True when the ranks' ranges tile [0, total) without gap or overlap (used by the tests and by callers
    that want to assert their split)."""
    shards = [shard_range(total, r, world, granule) for r in range(world)]
    pos = 0
    for s in shards:
        if s.begin != pos or s.end < s.begin:
            return False, shards
        pos = s.end
    return pos == total, shards
