"""GPU parity of the reverse sweep's three by-name glue kernels (hsn_win_back_head / _mid / _tail)
against the reference's own PyTorch steps (fixtures) and, at larger sizes, against the oracle.
Every call goes through the C ABI."""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch
from conftest import SWEEP_READ, SWEEP_SETS, SWEEP_WRITTEN, sweep_fixture

from oracle import window_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def window():
    from hsn_b200.kernels import window as w

    assert w.available(), "the CUDA library is not built (python -m hsn_b200.build)"
    w.prepare(0)
    return w


def _put(target: torch.Tensor, values: np.ndarray) -> None:
    target.copy_(torch.as_tensor(np.ascontiguousarray(values)).to(target.dtype))


def _get(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy() if t.dtype == torch.bfloat16 else t.detach().cpu().numpy()


def _buffers(window, sizes, buf, *, half, activation, cand_norm, cand_eps, cell_norm):
    sweep = window.SweepBuffers(
        window.SweepShape(*sizes), device=torch.device("cuda", 0),
        product_dtype=torch.bfloat16 if half else torch.float32, activation=activation,
        cand_norm=cand_norm, cand_eps=cand_eps, cell_norm=cell_norm,
    )  # fmt: skip
    for key in (*SWEEP_READ, *SWEEP_WRITTEN):
        _put(getattr(sweep, key), buf[key])
    return sweep


def _check(sweep, want, stage: str, half: bool) -> None:
    """fp32 values to 1e-5 of the buffer's scale (the sums' order differs from torch's); bf16
    operands within one bf16 step, and all but 2 % of them to the bit."""
    for key in SWEEP_WRITTEN:
        got, ref = _get(getattr(sweep, key)), want(key)
        scale = max(1.0, float(np.abs(ref).max()))
        if half and key.startswith("op"):
            assert np.mean(got != ref) < 0.02, (stage, key)
            assert np.abs(got - ref).max() <= 2.0**-7 * scale, (stage, key)
        else:
            assert np.abs(got - ref).max() <= 1e-5 * scale, (stage, key)


@pytest.mark.parametrize("name", SWEEP_SETS)
def test_sweep_kernels_equal_the_references_steps(window, name: str) -> None:
    """Two positions in sweep order on the reference's buffers: after every kernel every buffer it
    may write equals the reference's, so nothing outside its own blocks is touched either (the
    operands start from random values)."""
    z, sizes, buf = sweep_fixture(name)
    half = bool(z["half"])
    sweep = _buffers(window, sizes, buf, half=half, activation=str(z["activation"]),
                     cand_norm=bool(z["cand_norm"]), cand_eps=float(z["cand_eps"]),
                     cell_norm=bool(z["cell_norm"]))  # fmt: skip
    assert window.back_unsupported(sweep.shape) is None
    T = sizes[1]
    for t in (T - 1, T - 2):
        window.back_head(sweep, t)
        _check(sweep, lambda key: z[f"head{t}_{key}"], f"head{t}", half)
        _put(sweep.act_r, z[f"mid{t}_act_r"])
        _put(sweep.act_f, z[f"mid{t}_act_f"])
        window.back_mid(sweep, t)
        _check(sweep, lambda key: z[f"mid{t}_{key}"], f"mid{t}", half)
        _put(sweep.dv_r, z[f"tail{t}_dv_r"])
        _put(sweep.dv_f, z[f"tail{t}_dv_f"])
        window.back_tail(sweep, t)
        _check(sweep, lambda key: z[f"tail{t}_{key}"], f"tail{t}", half)


def _random_buffers(sizes, half: bool, seed: int):
    B, T, K, N, d, H, M, F, n_read, _, d_out = sizes
    rng = np.random.default_rng(seed)
    f32 = np.float32
    rows = B * (K - F)

    def normal(*shape):
        v = rng.standard_normal(shape).astype(f32)
        return v

    def operand(*shape):
        v = normal(*shape)
        return O.bf16_round(v) if half else v

    buf = {key: normal(B, T, K, d) for key in ("h_old", "y", "gate_pre", "mv", "d_h_sel", "dc", "db")}
    buf["c"] = np.tanh(normal(B, T, K, d))
    buf["b"] = O.sigmoid(normal(B, T, K, d))
    buf["rms"] = (rng.random((B, T, K)) + 0.5).astype(f32)
    buf["hidden"] = operand(B, T, K, H)
    buf["cells"] = np.stack([np.stack([rng.permutation(N)[:K] for _ in range(T)]) for _ in range(B)]).astype(np.int64)
    buf["units"] = rng.integers(0, M, (B, T, K)).astype(np.int64)
    buf["valid"] = rng.random((B, T, K)) < 0.8
    buf["cells"][~buf["valid"]] = 0
    buf["units"][~buf["valid"]] = 0
    buf["reset"] = rng.random((B, T)) < 0.25
    buf["d_q_pre"], buf["d_q_post"] = normal(B, T, d), normal(B, T, d)
    buf["d_h_fast"] = normal(B, T, max(n_read, 1), d)
    buf["cand_gain"] = (1.0 + 0.1 * normal(d)).astype(f32)
    buf["gate_bias"], buf["b1"] = normal(d), normal(M, H)
    pad_src = rng.integers(0, N, (N, d_out))
    pad_mask = rng.random((N, d_out)) < 0.7
    out_tgt, _ = O.out_adjacency(pad_src, pad_mask)
    width = out_tgt.shape[1]
    buf["out_tgt"] = out_tgt.astype(np.int32)
    buf["out_w"] = (normal(N, width) * (out_tgt >= 0)).astype(f32)
    buf["A"], buf["R"], buf["sigma"] = normal(B, N, d), normal(B, d), normal(B, K)
    buf["op1"], buf["op2"] = operand(rows, M * d), operand(rows, M * H + d)
    buf["op1_fast"], buf["op2_fast"] = operand(max(F, 1), B, d), operand(max(F, 1), B, H + d)
    return buf, width, rng


@pytest.mark.parametrize(
    "sizes, half, activation",
    [
        ((32, 3, 8, 256, 64, 512, 8, 0, 0, 256), True, "gelu"),  # the benchmark's cell
        ((5, 4, 8, 96, 32, 96, 3, 2, 4, 128), True, "silu"),
        ((3, 3, 40, 700, 24, 40, 5, 1, 3, 72), False, "tanh"),  # more than 32 slots, odd widths
        ((4, 1, 6, 40, 16, 48, 3, 5, 0, 64), False, "relu"),    # one position, a single routed slot
    ],
)
def test_sweep_kernels_equal_the_oracle_at_larger_sizes(window, sizes, half: bool, activation: str) -> None:
    buf, width, rng = _random_buffers((*sizes, 6), half, seed=sizes[0])
    sizes = (*sizes, width)
    s = O.SweepSizes(*sizes)
    sweep = _buffers(window, sizes, buf, half=half, activation=activation, cand_norm=True, cand_eps=1e-5,
                     cell_norm=True)  # fmt: skip
    assert window.back_unsupported(sweep.shape) is None
    rows = s.B * (s.K - s.n_fast)
    for t in range(s.T - 1, -1, -1):
        window.back_head(sweep, t)
        O.sweep_head(s, buf, t, cand_norm=True, cand_eps=1e-5, half=half)
        _check(sweep, lambda key: buf[key], f"head{t}", half)
        for key, shape in (("act_r", (rows, s.H)), ("act_f", (max(s.n_fast, 1), s.B, s.H))):
            v = rng.standard_normal(shape).astype(np.float32)
            buf[key] = O.bf16_round(v) if half else v
            _put(getattr(sweep, key), buf[key])
        window.back_mid(sweep, t)
        O.sweep_middle(s, buf, t, activation=activation, half=half)
        _check(sweep, lambda key: buf[key], f"mid{t}", half)
        for key, shape in (("dv_r", (rows, 2 * s.d)), ("dv_f", (max(s.n_fast, 1), s.B, 2 * s.d))):
            v = rng.standard_normal(shape).astype(np.float32)
            buf[key] = O.bf16_round(v) if half else v
            _put(getattr(sweep, key), buf[key])
        window.back_tail(sweep, t)
        O.sweep_tail(s, buf, t, cell_norm=True)
        _check(sweep, lambda key: buf[key], f"tail{t}", half)


def test_sweep_kernels_take_the_references_launch_shape(window) -> None:
    """The reference's wrappers launch 512 threads with their own shared-memory sizes
    (reference python/hsn/kernels/window.py:1151-1163): the kernels give the same results under
    that launch as under the library's own."""
    from hsn_b200 import _lib

    z, sizes, buf = sweep_fixture("fast2_bf16")
    B, T, K, N, d, H, M, F, n_read, in_dim, d_out = sizes
    sweep = _buffers(window, sizes, buf, half=True, activation=str(z["activation"]), cand_norm=True,
                     cand_eps=float(z["cand_eps"]), cell_norm=True)  # fmt: skip
    t = T - 1
    shared = 4 * (2 * d + 5 * K + 2 * K * d + 3 * ((K * d + 31) // 32))
    tensors = [sweep.A, sweep.R, sweep.c, sweep.b, sweep.h_old, sweep.y, sweep.cells, sweep.units, sweep.valid,
               sweep.d_q_post, sweep.d_h_sel, sweep.d_h_fast, sweep.cand_gain, sweep.gate_pre, sweep.gate_bias,
               sweep.dc, sweep.db, sweep.op1, sweep.op1_fast, sweep.op2, sweep.op2_fast, sweep.sigma]  # fmt: skip
    args = _lib.HsnWinArgs()
    for k, tensor in enumerate(tensors):
        args.p[k] = tensor.data_ptr()
    for k, v in enumerate([B, T, K, d, N, M, H, F, t, n_read, 1, 1]):
        args.i[k] = v
    args.f[0] = float(z["cand_eps"])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(_lib.library().hsnw_launch(b"hsn_win_back_head", ctypes.byref(args), B, 512, shared, stream))
    _check(sweep, lambda key: z[f"head{t}_{key}"], "head", True)


def test_sweep_kernels_decline_what_they_cannot_take(window) -> None:
    assert "routed slot" in window.back_unsupported(window.SweepShape(2, 2, 4, 16, 8, 16, 2, 4, 0, 32, 2))
    assert "shared memory" in window.back_unsupported(window.SweepShape(2, 2, 8, 100000, 64, 16, 2, 0, 0, 256, 2))
    sweep = window.SweepBuffers(window.SweepShape(2, 2, 4, 16, 8, 16, 2, 0, 0, 32, 2), device=torch.device("cuda", 0))
    with pytest.raises(ValueError):
        window.back_head(sweep, 2)
