"""The stand-in for the reference's pybind launcher (``hsn_window_py``): kernels launched by name with
the reference's descriptors through ``launch``, ``launch_views`` and ``loop``."""

from __future__ import annotations

import numpy as np
import pytest
import torch
from conftest import dev

from oracle import window_oracle as O

pytestmark = pytest.mark.gpu


def _case(rng, B=5, N=48, M=4, K=6, T=7):
    logits = (np.round(rng.standard_normal((B, N, M)) * 2) / 2).astype(np.float32)  # ties on purpose
    ages = (rng.integers(0, 12, (B, T, N)) // 3 * 3).astype(np.int64)
    cost = np.linspace(0.01, 0.04, M).astype(np.float32)
    params = dict(k=K, age_max=5, probes=True, lambda_cost=0.25, cell_overhead=0.02, shared_cost=0.05, limit=0.3)
    return logits, ages, cost, params


def _outputs(B, T, K):
    return (torch.full((B, T, K), -7, dtype=torch.int64, device="cuda"), torch.full((B, T, K), -7, dtype=torch.int64, device="cuda"),
            torch.zeros((B, T, K), dtype=torch.bool, device="cuda"), torch.full((B, T), -7.0, device="cuda"),
            torch.zeros((B, T, K), dtype=torch.bool, device="cuda"))  # fmt: skip


def test_launch_and_loop_run_the_kernels_by_name() -> None:
    """``hsn_win_select`` in its tape form (record ``t`` of the outputs from record ``t`` of the ages;
    the record index is descriptor int 6): one ``launch`` per position, and one ``loop`` over the
    positions (``hsnw_loop``), both equal to the router's decision; nothing but the records is touched."""
    from hsn_b200.kernels import hsn_window_py as ext

    rng = np.random.default_rng(21)
    logits, ages, cost, p = _case(rng)
    B, T, N = ages.shape
    M, K = logits.shape[2], p["k"]
    ext.prepare("unused.fatbin", 0)
    tensors = lambda outs: [dev(logits), dev(ages), dev(cost), *outs]  # noqa: E731
    ints = lambda t: [B, N, M, K, p["age_max"], 1, t, T, T, 0, 0, 0, 0]  # noqa: E731
    floats = [p["lambda_cost"], p["cell_overhead"], p["shared_cost"], p["limit"]]
    one = _outputs(B, T, K)
    for t in range(T):
        ext.launch("hsn_win_select", B, 256, 0, tensors(one), ints(t), floats)
    many = _outputs(B, T, K)
    ext.loop(["hsn_win_select"], [B], [256], [0], tensors(many), ints(0), floats, T, 6)
    views = _outputs(B, T, K)
    ext.launch_views("hsn_win_select", B, 256, 0, tensors(views), [], ints(2), floats)
    for t in range(T):
        want = O.select(logits, ages[:, t], cost, **p)
        for got in (one, many):
            assert np.array_equal(got[0][:, t].cpu().numpy(), want[0]) and np.array_equal(got[1][:, t].cpu().numpy(), want[1])
            assert np.array_equal(got[2][:, t].cpu().numpy(), want[2]) and np.array_equal(got[3][:, t].cpu().numpy(), want[3])
            assert np.array_equal(got[4][:, t].cpu().numpy(), want[4])
    assert torch.equal(views[0][:, 2], one[0][:, 2]) and bool((views[0][:, 3] == -7).all())  # only record 2 was written
    # grid <= 0 launches nothing; unknown names, too many operands and wrong devices raise as the reference does
    untouched = _outputs(B, T, K)
    ext.launch("hsn_win_select", 0, 256, 0, tensors(untouched), ints(0), floats)
    assert bool((untouched[0] == -7).all())
    with pytest.raises(RuntimeError):
        ext.launch("hsn_win_nothing", B, 256, 0, tensors(untouched), ints(0), floats)
    with pytest.raises(RuntimeError):
        ext.launch("hsn_win_select", B, 256, 0, tensors(untouched), list(range(40)), floats)
    with pytest.raises(RuntimeError):
        ext.launch("hsn_win_select", B, 256, 0, [torch.zeros(3)], ints(0), floats)
    with pytest.raises(RuntimeError):
        ext.loop(["hsn_win_select"], [B], [256], [0], tensors(untouched), ints(0), floats, T, 40)
    # the trainer's kernels by name through the same module (tests/test_trainer_kernels.py checks their values)
    a, b = torch.zeros(3, device="cuda"), torch.ones(3, device="cuda")
    assert ext.launch_table("hsn_tr_copy", 256, [[a], [b]], 2, [], [], [], []) is True and torch.equal(a, b)
    assert ext.launch_table("hsn_tr_copy", 256, [[torch.zeros(3)], [torch.ones(3)]], 2, [], [], [], []) is False   # CPU tensors
