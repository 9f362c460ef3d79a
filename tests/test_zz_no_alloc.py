"""The reverse sweep for callers that cannot allocate (``hsnw_window_backward_static``).

Some hosts only pass on buffers they were given, or run inside a pool that already owns the free
device memory; they cannot produce a scratch buffer for ``hsnw_window_backward``. This entry point
brings its own, a fixed array inside the library. The test drives both entry points through the
C ABI on the same inputs, twice in a row (the second call meets the first call's leftovers in the
shared array), and expects the same cotangents; it also checks that a window too large for the
array is refused, not truncated. Collected last, so a failure here stops no other test.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from oracle import window_oracle as O

pytestmark = pytest.mark.gpu


def _case(B: int, T: int, seed: int):
    from hsn_b200.window import WindowModel, window_forward

    rng = np.random.default_rng(seed)
    N, d, K, H, M, D, S = 64, 32, 4, 96, 4, 3, 9
    W = O.WindowWeights.random(rng, N=N, d=d, K=K, H=H, M=M, D=D, S=S)
    for key in ("w1", "w2", "gate_w", "v_w", "wout_w", "score_w"):
        setattr(W, key, (getattr(W, key) * 8).astype(np.float32))
    model = WindowModel.from_oracle_weights(W, device="cuda")
    cuda = lambda a: torch.as_tensor(a).cuda()  # noqa: E731
    reset = rng.random((B, T)) < 0.1
    reset[:, 0] = True
    state = (torch.zeros((B, N, d)), torch.zeros((B, d)), torch.zeros((B, N), dtype=torch.int64),
             torch.zeros(B, dtype=torch.int64))  # fmt: skip
    tape = window_forward(
        model, cuda(rng.standard_normal((B, T, d)).astype(np.float32)),
        cuda((rng.standard_normal((B, T, d)) * 0.02).astype(np.float32)),
        cuda(rng.random((B, T, N, S)).astype(np.float32)), cuda(reset), tuple(s.cuda() for s in state),
    )  # fmt: skip
    cots = [cuda(rng.standard_normal(s).astype(np.float32)) for s in ((B, T, d), (B, T, d), (B, T, K, d))]
    return model, tape, cuda(reset), cots, (B, T, N, d, K)


def _io(model, tape, reset, cots, dims, A, R, dc, db, scratch):
    from hsn_b200 import _lib

    B, T, N, d, K = dims
    io = _lib.HsnwBackward()
    io.B, io.T, io.full_cut = B, T, 0
    for field, t in (
        ("c", tape["rec_c"]), ("b", tape["rec_b"]), ("h_old", tape["rec_h_old"]), ("y", tape["rec_y"]),
        ("gate_pre", tape["rec_gate_pre"]), ("m", tape["rec_m"]), ("rms", tape["rec_rms"]),
        ("hidden", tape["rec_hidden"]), ("cells", tape["sel_cell_idx"]), ("units", tape["sel_unit_idx"]),
        ("valid", tape["sel_valid"]), ("reset", reset), ("d_q_pre", cots[0]), ("d_q_post", cots[1]),
        ("d_h_sel", cots[2]), ("dc", dc), ("db", db), ("A", A), ("R", R),
    ):  # fmt: skip
        setattr(io, field, t.data_ptr())
    if scratch is not None:
        io.scratch, io.scratch_bytes = scratch.data_ptr(), scratch.numel()
    return io


def test_static_scratch_entry_point_matches_the_allocating_one() -> None:
    from hsn_b200 import _lib

    lib = _lib.library()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (B, T, seed) in enumerate(((5, 9, 21), (3, 6, 22))):  # two calls in a row, other sizes
        model, tape, reset, cots, dims = _case(B, T, seed)
        _, _, N, d, K = dims
        need = int(lib.hsnw_backward_scratch_bytes(ctypes.byref(model.struct), B, T))
        assert need <= int(lib.hsnw_static_scratch_bytes())
        scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
        start_A = torch.randn((B, N, d), device="cuda")
        start_R = torch.randn((B, d), device="cuda")
        results = []
        for static in (False, True):
            A, R = start_A.clone(), start_R.clone()
            dc = torch.full((B, T, K, d), float("nan"), device="cuda")
            db = torch.full((B, T, K, d), float("nan"), device="cuda")
            io = _io(model, tape, reset, cots, dims, A, R, dc, db, None if static else scratch)
            fn = lib.hsnw_window_backward_static if static else lib.hsnw_window_backward
            _lib.check(fn(ctypes.byref(model.struct), ctypes.byref(io), stream))
            torch.cuda.synchronize()
            results.append((dc, db, A, R))
        for got, want in zip(results[1], results[0]):
            assert bool(torch.isfinite(want).all()), call
            scale = max(1.0, float(want.abs().max()))
            assert float((got - want).abs().max()) <= 1e-5 * scale, call


def test_static_scratch_entry_point_refuses_what_does_not_fit() -> None:
    from hsn_b200 import _lib
    from hsn_b200.window import WindowModel

    lib = _lib.library()
    rng = np.random.default_rng(3)
    W = O.WindowWeights.random(rng, N=64, d=64, K=8, H=512, M=8, D=4)
    model = WindowModel.from_oracle_weights(W, device="cuda")
    B = 4096  # 32768 pairs: far beyond the built-in array
    assert int(lib.hsnw_backward_scratch_bytes(ctypes.byref(model.struct), B, 1)) > int(lib.hsnw_static_scratch_bytes())
    io = _lib.HsnwBackward()
    io.B, io.T = B, 1
    code = lib.hsnw_window_backward_static(ctypes.byref(model.struct), ctypes.byref(io), None)
    assert code == _lib.E_UNSUPPORTED
    assert b"built-in array" in lib.hsnw_last_error()
