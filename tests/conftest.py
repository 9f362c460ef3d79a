"""Shared test plumbing: the ``gpu`` marker, paths, and the fixtures' loader."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
GOLDEN = ROOT / "tests" / "golden"
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config: pytest.Config, items: list[pytest.Item]) -> None:
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str):
    return np.load(GOLDEN / f"{name}.npz")


SWEEP_SETS = ["plain_f32", "fast_bf16", "fast2_bf16", "relu_f32"]
SWEEP_WRITTEN = ("A", "R", "dc", "db", "op1", "op1_fast", "op2", "op2_fast", "sigma")
SWEEP_READ = (
    "c", "b", "h_old", "y", "gate_pre", "mv", "rms", "hidden", "cells", "units", "valid", "reset",
    "d_q_pre", "d_q_post", "d_h_sel", "d_h_fast", "cand_gain", "gate_bias", "b1", "out_tgt", "out_w",
)  # fmt: skip


def sweep_fixture(name: str):
    """A ``sweep_*.npz`` fixture as ``(z, sizes, buffers)``: the file, the eleven sizes of the
    sweep's shape in its order, and the buffers at the start (copies, by the sweep's names)."""
    z = load_golden(f"sweep_{name}")
    sizes = [int(v) for v in z["shape"]]
    buffers = {key: np.array(z[key]) for key in SWEEP_READ}
    buffers.update({key: np.array(z[f"start_{key}"]) for key in SWEEP_WRITTEN})
    return z, sizes, buffers


def settled(logits: np.ndarray, cells: np.ndarray, valid: np.ndarray, margin) -> np.ndarray:
    """Rows x positions that are safe to compare when two sweeps' logits differ in the last place
    (the reference's protocol for discrete routing, its tests/kernels/test_p2_10c_window.py:380-440):
    a position is risky when the gap between the last selected and the first unselected cell
    score, or between the two best units of a selected cell, is within ``margin`` (a number, or an
    array ``[B, T]``). ``logits [B, T, N, M]`` are one sweep's own."""
    B, T, N, M = logits.shape
    margin = np.broadcast_to(np.asarray(margin, dtype=np.float64), (B, T))
    score = logits.max(axis=-1)
    order = np.sort(score, axis=-1)[..., ::-1]
    K = cells.shape[-1]
    gap = order[..., K - 1] - order[..., K] if N > K else np.full((B, T), np.inf)
    risky = gap <= margin
    if M > 1:
        two = np.sort(logits, axis=-1)[..., ::-1]
        unit_gap = two[..., 0] - two[..., 1]  # [B,T,N]
        picked = np.take_along_axis(unit_gap, cells, axis=-1)
        risky |= (np.where(valid, picked, np.inf) <= margin[..., None]).any(axis=-1)
    return ~risky


def alive_rows(*pairs) -> np.ndarray:
    """``[B, T]``: True up to (not including) a row's first position where any pair ``(got, want)`` of
    decision arrays ``[B, T, ...]`` differs. With bfloat16 logits a margin cannot separate safe from
    risky positions (exact ties between 8-bit-mantissa scores are everywhere and both sweeps break them
    the same way); what can differ is one logit whose float32 sum sat on a rounding boundary, about one
    position in a thousand. So two bf16 sweeps are compared directly and a row counts up to its first
    difference; the callers bound how many positions may be lost that way."""
    same = None
    for got, want in pairs:
        eq = (np.asarray(got) == np.asarray(want)).reshape(got.shape[0], got.shape[1], -1).all(axis=-1)
        same = eq if same is None else same & eq
    return np.logical_and.accumulate(same, axis=1)


def dev(a, dtype=None):
    """A numpy array as a CUDA tensor."""
    import torch

    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def synthetic_window(rng, B, T, N, d, K, H, M, D, p_reset, age_max=1 << 30, S=9, score_scale=40.0):
    """Seeded weights of the reference's shapes (the oracle's ``WindowWeights.random``) with the scorer
    scaled so that scores spread well beyond a tie margin, and a window's inputs: ``(W, z, ctx,
    scalars, reset, (h, q, age, pos))`` as numpy arrays, every row starting from a reset."""
    from oracle import window_oracle as O

    W = O.WindowWeights.random(rng, N=N, d=d, K=K, H=H, M=M, D=D, S=S, age_max=age_max)
    W.score_w = (W.score_w * score_scale).astype(np.float32)
    z = rng.standard_normal((B, T, d)).astype(np.float32)
    ctx = (rng.standard_normal((B, T, d)) * 0.02).astype(np.float32)
    scalars = rng.random((B, T, N, S)).astype(np.float32)
    reset = rng.random((B, T)) < p_reset
    reset[:, 0] = True
    state = (np.zeros((B, N, d), np.float32), np.zeros((B, d), np.float32), np.zeros((B, N), np.int64), np.zeros(B, np.int64))
    return W, z, ctx, scalars, reset, state


def to_np(t):
    """A device tensor as a numpy array (bfloat16, which numpy lacks, as float32: exact)."""
    import torch

    return t.float().cpu().numpy() if t.dtype == torch.bfloat16 else t.cpu().numpy()
