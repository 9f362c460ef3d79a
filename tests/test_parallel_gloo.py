"""The N > 1 path on CPU: two gloo ranks shard the rows, exchange gradients and batch statistics."""

from __future__ import annotations

import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hsn_b200.parallel import all_reduce_gradients, reduce_window_stats, shard_rows


def test_shards_cover_every_row_once() -> None:
    for n_rows in (0, 1, 7, 32, 255, 4096):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for rank in range(world):
                s = shard_rows(n_rows, world, rank)
                seen.extend(range(s.start, s.stop))
            assert seen == list(range(n_rows))
            sizes = [shard_rows(n_rows, world, r).stop - shard_rows(n_rows, world, r).start for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_rows(8, 2, 2)


def _worker(rank: int, world: int, port: int, out) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows = [shard_rows(5, world, r) for r in range(world)]
        mine = rows[rank]
        g = torch.Generator().manual_seed(3)
        full = [torch.randn(5, 4, 3, generator=g), torch.randn(5, 7, generator=g)]
        # each rank's "gradient" is the sum over its rows: the all-reduce must give the sum over all
        grads = [t[mine].sum(dim=0) for t in full] + [None]
        all_reduce_gradients(grads, average=False)
        ok = all(torch.allclose(got, t.sum(dim=0), atol=1e-6) for got, t in zip(grads, full))
        per_row = torch.randn(5, 6, generator=g).abs()
        refreshed, peak = reduce_window_stats(
            per_row[mine].mean(dim=0), per_row[mine].amax(dim=0), [r.stop - r.start for r in rows]
        )
        ok = ok and torch.allclose(refreshed, per_row.mean(dim=0), atol=1e-6) and torch.equal(peak, per_row.amax(dim=0))
        out.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_two_ranks_exchange_gradients_and_statistics() -> None:
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + int(np.random.default_rng().integers(0, 2000))
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == [(0, True), (1, True)]
