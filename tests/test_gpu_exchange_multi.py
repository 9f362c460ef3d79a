"""The fused gradient exchange + AdamW across real GPUs of one box (``hsn_b200.parallel.ShardedAdamW``): one
process per GPU over NCCL, the buffers in symmetric memory. Needs at least two GPUs (skipped otherwise; the same
kernel runs with every rank's buffers on one device in ``tests/test_trainer_kernels.py``)."""

from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

N = 250_003
HYPER = dict(lr=2.5e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01)


def _gradients(rank: int, step: int, size: int) -> np.ndarray:
    return (np.random.default_rng(100 * step + rank).standard_normal(size) * (1e-3, 1.0, 30.0)[step - 1]).astype(np.float32)


def _rank(rank: int, world: int, port: int, out_dir: str) -> None:
    import torch.distributed as dist

    from hsn_b200.parallel import ShardedAdamW

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        opt = ShardedAdamW(N, lr=HYPER["lr"], betas=(HYPER["beta1"], HYPER["beta2"]), eps=HYPER["eps"],
                           weight_decay=HYPER["weight_decay"])  # fmt: skip
        size = world * opt.shard
        p0 = np.zeros(size, np.float32)
        p0[:N] = (np.random.default_rng(1).standard_normal(N) * 0.1).astype(np.float32)
        opt.params.copy_(torch.from_numpy(p0))
        for step in range(1, 4):
            opt.grads.copy_(torch.from_numpy(_gradients(rank, step, size)))
            opt.step()
        torch.cuda.synchronize()
        np.save(os.path.join(out_dir, f"params_{rank}.npy"), opt.params.cpu().numpy())
        np.save(os.path.join(out_dir, f"m_{rank}.npy"), opt.exp_avg.cpu().numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_fused_exchange_across_gpus(world: int, tmp_path) -> None:
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    from oracle import trainer_oracle as TO

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_rank, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    got = [np.load(tmp_path / f"params_{r}.npy") for r in range(world)]
    size = got[0].size
    p = np.zeros(size, np.float32)
    p[:N] = (np.random.default_rng(1).standard_normal(N) * 0.1).astype(np.float32)
    m, v = np.zeros_like(p), np.zeros_like(p)
    for step in range(1, 4):
        p, m, v = TO.exchange_adamw([_gradients(r, step, size) for r in range(world)], p, m, v, step=step, **HYPER)
    for r in range(world):
        assert np.array_equal(got[r].view(np.uint32), p.view(np.uint32)), r   # every rank: the oracle's bits
    assert np.array_equal(np.concatenate([np.load(tmp_path / f"m_{r}.npy") for r in range(world)]).view(np.uint32), m.view(np.uint32))
