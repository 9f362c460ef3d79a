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

import ctypes
import os
from collections.abc import Iterable, Sequence

import torch
import torch.distributed as dist
from torch import Tensor

__all__ = ["shard_rows", "all_reduce_gradients", "reduce_window_stats", "shard_elements", "ShardedAdamW"]


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


def shard_elements(n_elements: int, world_size: int) -> int:
    """Elements per rank of a flat vector of ``n_elements`` cut into ``world_size`` equal shards of whole
    16-byte groups: the vector is padded to ``world_size * shard``."""
    if n_elements < 1 or world_size < 1:
        raise ValueError(f"invalid shards: {n_elements} elements over {world_size} ranks")
    per = -(-n_elements // world_size)
    return -(-per // 4) * 4


class ShardedAdamW:
    """The training-gradient exchange fused with the optimiser step (``hsnw_exchange_adamw``): every rank keeps the
    flat parameter vector and its flat gradients in buffers that the other ranks of the box can address (peer
    memory over NVLink; allocated and exchanged with ``torch.distributed._symmetric_memory``, multicast off), and
    owns the AdamW moments of one shard. :meth:`step` is one kernel per rank: read every rank's gradients of the
    shard, sum in rank order, average, AdamW, write the new parameters to every rank. Around it two one-element
    all-reduces on the stream order the ranks (gradients complete before; parameters complete after), so nothing
    in the kernel waits and there is no host synchronisation.

    ``params`` and ``grads`` are the flat views a model's tensors should alias (``[world * shard]`` float32, the
    tail beyond ``n_elements`` is padding). Replaces ``all_reduce_gradients`` + an optimiser step on replicated
    state; the moments take ``1 / world`` of the memory."""

    def __init__(self, n_elements: int, *, lr: float, betas: tuple[float, float] = (0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.0, average: bool = True, group: dist.ProcessGroup | None = None,
                 device: torch.device | None = None, buffers: tuple[Sequence[Tensor], Sequence[Tensor]] | None = None,
                 rank: int | None = None) -> None:  # fmt: skip
        from . import _lib

        self.lr, self.betas, self.eps, self.weight_decay, self.average = float(lr), (float(betas[0]), float(betas[1])), float(eps), float(weight_decay), bool(average)
        self.group, self.steps, self._lib = group, 0, _lib
        if buffers is not None:
            # every rank's buffers given outright (one process holding several ranks' buffers on one device: tests)
            grads, params = buffers
            self.world, self.rank = len(grads), int(rank or 0)
            self.shard = shard_elements(n_elements, self.world)
            self.grads, self.params = grads[self.rank], params[self.rank]
            grad_ptrs, param_ptrs = [t.data_ptr() for t in grads], [t.data_ptr() for t in params]
            self._barrier = False
        else:
            import torch.distributed._symmetric_memory as symm

            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer loads and stores only
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
            self.shard = shard_elements(n_elements, self.world)
            device = device or torch.device("cuda", torch.cuda.current_device())
            which = group if group is not None else dist.group.WORLD
            self.grads = symm.empty(self.world * self.shard, dtype=torch.float32, device=device)
            self.params = symm.empty(self.world * self.shard, dtype=torch.float32, device=device)
            self._handles = (symm.rendezvous(self.grads, which), symm.rendezvous(self.params, which))
            grad_ptrs, param_ptrs = list(self._handles[0].buffer_ptrs), list(self._handles[1].buffer_ptrs)
            self.grads.zero_()
            self.params.zero_()
            self._barrier = self.world > 1
            self._token = torch.zeros(1, device=device)
        if not 1 <= self.world <= 8:
            raise ValueError("the fused exchange takes 1 to 8 ranks of one box")
        self.n_elements = int(n_elements)
        dev = self.params.device
        self.exp_avg = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        x = _lib.HsnwExchange()
        x.world, x.rank, x.average, x.weight_decay_on, x.shard = self.world, self.rank, int(self.average), int(self.weight_decay != 0), self.shard
        for k in range(self.world):
            x.grads[k], x.params[k] = grad_ptrs[k], param_ptrs[k]
        x.exp_avg, x.exp_avg_sq = self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr()
        self._x = x
        lib = _lib.library()
        index = dev.index if dev.index is not None else torch.cuda.current_device()
        if not lib.hsnw_prepared(index):
            _lib.check(lib.hsnw_prepare(index))

    def _order(self) -> None:
        if self._barrier:
            dist.all_reduce(self._token, group=self.group)   # on the stream: completes when every rank's earlier work has

    def step(self) -> None:
        """One optimiser step on the gradients every rank has written into its ``grads``."""
        self.steps += 1
        beta1, beta2 = self.betas
        x = self._x
        scalars = (1 - self.lr * self.weight_decay, 1 - beta1, beta2, 1 - beta2, 1.0 / (1 - beta2**self.steps) ** 0.5, self.eps,
                   -(self.lr / (1 - beta1**self.steps)))  # fmt: skip
        for k, v in enumerate(scalars):
            x.f[k] = v
        dev = self.params.device
        self._order()
        with torch.cuda.device(dev):
            stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
            self._lib.check(self._lib.library().hsnw_exchange_adamw(ctypes.byref(x), stream))
        self._order()
