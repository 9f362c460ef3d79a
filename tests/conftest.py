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
