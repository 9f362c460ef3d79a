"""Batch sharding of the window path across the GPUs of one box.

Rows (training) and streams (serving) are independent inside a window: state, tape, decisions and
the reverse sweep are per row (the reference runs one block per row, ``kernels/cuda/hsn_window.cu``;
it has no distributed code at all). So each rank runs the window entry points on a contiguous
slice of the rows with replicated weights, and the only exchange is the training-gradient
all-reduce after each window backward plus two tiny reductions for the batch statistics the tape
reports per position (``refreshed`` is a mean over rows, ``state_abs_max`` a maximum;
``python/hsn/train/compile.py:1211-1212``). One process per GPU; NCCL on GPUs, gloo on CPU.
"""

from __future__ import annotations

from collections.abc import Iterable, Sequence

import torch
import torch.distributed as dist
from torch import Tensor

__all__ = ["shard_rows", "all_reduce_gradients", "reduce_window_stats"]


def shard_rows(n_rows: int, world_size: int, rank: int) -> slice:
    """The contiguous slice of ``n_rows`` rows that ``rank`` owns: the first ``n_rows %
    world_size`` ranks take one row more, no row is owned twice, none is left out."""
    if not (0 <= rank < world_size) or n_rows < 0:
        raise ValueError(f"invalid shard: rank {rank} of {world_size}, {n_rows} rows")
    base, extra = divmod(n_rows, world_size)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def all_reduce_gradients(grads: Iterable[Tensor | None], group: dist.ProcessGroup | None = None,
                         average: bool = True) -> None:  # fmt: skip
    """Sum (or average) the parameter gradients over the ranks, in place: one flat bucket per
    dtype, one collective each (the model is a few MB, so the exchange is latency bound and a
    single bucket is the cheapest shape)."""
    if not dist.is_available() or not dist.is_initialized():
        return
    world = dist.get_world_size(group)
    if world == 1:
        return
    by_dtype: dict[torch.dtype, list[Tensor]] = {}
    for g in grads:
        if g is not None:
            by_dtype.setdefault(g.dtype, []).append(g)
    for tensors in by_dtype.values():
        flat = torch.cat([t.reshape(-1) for t in tensors])
        dist.all_reduce(flat, group=group)
        if average:
            flat /= world
        offset = 0
        for t in tensors:
            n = t.numel()
            t.copy_(flat[offset : offset + n].view_as(t))
            offset += n


def reduce_window_stats(refreshed: Tensor, state_abs_max: Tensor, rows: Sequence[int],
                        group: dist.ProcessGroup | None = None) -> tuple[Tensor, Tensor]:  # fmt: skip
    """The tape's per-position batch statistics over all ranks: ``refreshed [T]`` is each rank's
    mean over its rows (``rows[r]`` rows on rank ``r``) and becomes the mean over all rows;
    ``state_abs_max [T]`` becomes the maximum (a maximum of absolute values: a rank that owns no rows
    contributes zeros, whatever it passes in)."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return refreshed, state_abs_max
    rank = dist.get_rank(group)
    total = float(sum(rows))
    if rows[rank] > 0:
        weighted = refreshed * (rows[rank] / total)
        peak = state_abs_max.clone()
    else:
        # a rank without rows (fewer rows than ranks): its mean over nothing is NaN and would poison the sum
        weighted = torch.zeros_like(refreshed)
        peak = torch.zeros_like(state_abs_max)
    dist.all_reduce(weighted, group=group)
    dist.all_reduce(peak, op=dist.ReduceOp.MAX, group=group)
    return weighted, peak
