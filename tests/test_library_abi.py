"""The C-ABI library without a GPU: it builds, loads and exports every symbol the header
declares; the ctypes structures have the header's sizes; calls that need a device fail loudly."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from hsn_b200 import _lib, build

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "hsn_window_b200.h"


@pytest.fixture(scope="module")
def lib() -> ctypes.CDLL:
    build.build()
    return _lib.library()


def test_every_declared_symbol_is_exported(lib: ctypes.CDLL) -> None:
    text = "".join((HEADER.parent / name).read_text() for name in ("hsn_window_b200.h", "hsn_trainer_b200.h", "hsn_units_b200.h", "hsn_scorer_b200.h", "hsn_tail_b200.h", "hsn_gate_b200.h", "hsn_messages_b200.h"))
    declared = set(re.findall(r"\b(hsnw_[a-z_]+)\s*\(", text))
    assert declared, "no entry points found in the header"
    assert declared == set(_lib.SYMBOLS), declared ^ set(_lib.SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name


def test_structures_match_the_header() -> None:
    assert ctypes.sizeof(_lib.HsnWinArgs) == 8 * 48 + 4 * 32 + 4 * 8  # the reference's 544 bytes
    assert ctypes.sizeof(_lib.HsnTrainArgs) == 8 * 4 * 40 + 8 * 40 + 8 * 2 + 4 * 8 + 4 * 8 + 4 * 6 * 64  # its 3760
    assert _lib.HsnTrainArgs.end.offset == 1280 and _lib.HsnTrainArgs.u.offset == 1280 + 320 + 16 + 32 + 32
    assert ctypes.sizeof(_lib.HsnwModel) == 12 * 4 + 6 * 4 + 29 * 8
    assert ctypes.sizeof(_lib.HsnwForward) == 4 * 4 + 30 * 8 + 8
    assert ctypes.sizeof(_lib.HsnwBackward) == 4 * 4 + 20 * 8 + 8
    assert ctypes.sizeof(_lib.HsnwUnits) == 6 * 4 + 4 * 8 and _lib.HsnwUnits.w1.offset == 24
    assert ctypes.sizeof(_lib.HsnwScorer) == 6 * 4 + 2 * 8 and _lib.HsnwScorer.weight.offset == 24
    assert ctypes.sizeof(_lib.HsnwTail) == 4 * 4 + 2 * 8 and _lib.HsnwTail.w_out.offset == 16
    assert ctypes.sizeof(_lib.HsnwGate) == 4 * 4 + 3 * 8 and _lib.HsnwGate.norm_weight.offset == 16
    assert ctypes.sizeof(_lib.HsnwMessages) == 6 * 4 + 3 * 8 and _lib.HsnwMessages.v_w.offset == 24


def test_version_and_errors_without_a_device(lib: ctypes.CDLL) -> None:
    assert lib.hsnw_version() >= 100
    assert lib.hsnw_prepared(0) in (0, 1)
    args = _lib.HsnWinArgs()
    table = _lib.HsnTrainArgs()
    assert lib.hsnw_launch_table(b"hsn_tr_adamw", ctypes.byref(table), None) == _lib.E_ARG   # no tensors
    table.i[0], table.end[0] = 1, 16
    assert lib.hsnw_launch_table(b"no_such_kernel", ctypes.byref(table), None) == _lib.E_NAME
    assert lib.hsnw_launch_table(b"hsn_tr_copy", ctypes.byref(table), None) == _lib.E_ARG    # null rows
    assert lib.hsnw_launch(b"no_such_kernel", ctypes.byref(args), 1, 64, 0, None) == _lib.E_NAME
    assert b"no kernel" in lib.hsnw_last_error()
    grid, block, shared = ctypes.c_int64(), ctypes.c_int(), ctypes.c_int()
    args.i[0], args.i[1], args.i[2], args.i[3] = 4, 256, 8, 8
    assert lib.hsnw_launch_shape(b"hsn_win_select", ctypes.byref(args), ctypes.byref(grid), ctypes.byref(block), ctypes.byref(shared)) == 0
    assert (grid.value, block.value, shared.value) == (4, 256, 2048)
    args.i[3] = 65  # more slots than the kernel takes
    assert lib.hsnw_launch_shape(b"hsn_win_select", ctypes.byref(args), ctypes.byref(grid), ctypes.byref(block), ctypes.byref(shared)) == _lib.E_UNSUPPORTED


def test_no_gpu_means_a_loud_failure_not_a_fallback(lib: ctypes.CDLL) -> None:
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from hsn_b200.window import WindowModel

    with pytest.raises(RuntimeError):
        WindowModel.build({}, k=1, device="cpu")
    args = _lib.HsnWinArgs()
    code = lib.hsnw_launch(b"hsn_win_select", ctypes.byref(args), 1, 64, 0, None)
    assert code == _lib.E_STATE
    from hsn_b200.kernels.units import grouped_forward

    with pytest.raises(RuntimeError):   # the grouped unit pass has no CPU path either
        grouped_forward(torch.zeros(4, 32), torch.zeros(4, dtype=torch.int64), torch.zeros(2, 32, 16), torch.zeros(2, 16),
                        torch.zeros(2, 16, 8), torch.zeros(2, 8))
    from hsn_b200.kernels.gate import norm_gate_forward
    from hsn_b200.kernels.messages import messages_forward
    from hsn_b200.kernels.scorer import scorer_logits_forward
    from hsn_b200.kernels.tail import tail_forward

    z = torch.zeros
    with pytest.raises(RuntimeError):   # nor have the other pieces of the replay
        tail_forward(z(4, 16), torch.ones(4), z(16, 16), torch.ones(16))
    with pytest.raises(RuntimeError):
        norm_gate_forward(z(4, 64), torch.ones(64), z(16, 64), z(16))
    with pytest.raises(RuntimeError):
        messages_forward(z(2, 16), z(2, 16), z(2, 8, 16), z(2, 1, dtype=torch.int64), z(8, 2, dtype=torch.int64), z(8, 2), z(16, 16))
    with pytest.raises(RuntimeError):
        scorer_logits_forward(z(2, 3 * 16 + 1 + 2), z(2), z(3, 16), z(3, 16), z(3, 5, 16), z(3, 5, dtype=torch.int64), z(3, 5, 2), age_max=10.0)


def test_python_interface_keeps_the_reference_names() -> None:
    from hsn_b200.kernels import window

    for name in (
        "available", "prepare", "prepared", "recurrence_backward", "dense_recurrence_backward",
        "cell_round_error", "cell_round", "select", "select_tape", "select_fold", "select_unsupported",
        "cell_update", "update_tape", "update_fold", "cell_update_unsupported", "select_op",
        "select_tape_op", "select_fold_op", "cell_update_op", "update_tape_op", "update_fold_op",
    ):  # fmt: skip
        assert callable(getattr(window, name)), name
    import torch

    ns = getattr(torch.ops, window._NAMESPACE)
    for op in ("window_select", "window_select_tape", "window_select_fold", "window_cell_update",
               "window_update_tape", "window_update_fold"):  # fmt: skip
        assert hasattr(ns, op), op
    assert window.select_unsupported(4096, 16, 8) is None
    assert window.select_unsupported(8, 16) is not None


def test_synthetic_weights_are_the_oracles_random_weights() -> None:
    """The package's seeded benchmark weights and the oracle's: the same arrays from the same seed,
    so the benchmark's CPU leg and its GPU leg run one model."""
    import numpy as np

    from hsn_b200.window import synthetic_weights
    from oracle.window_oracle import WindowWeights

    sizes = dict(N=24, d=8, K=3, H=32, M=3, D=2, S=5, age_max=77)
    mine = synthetic_weights(np.random.default_rng(4), **sizes)
    theirs = WindowWeights.random(np.random.default_rng(4), **sizes)
    for key, want in vars(theirs).items():
        got = getattr(mine, key)
        assert np.array_equal(got, want) if isinstance(want, np.ndarray) else got == want, key
    WindowWeights(**vars(mine))
