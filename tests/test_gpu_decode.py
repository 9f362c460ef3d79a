"""The window's epilogue on the device (``hsnw_window_decode``) and the forward sweeps' ``us`` output it reads:
against the reference's fixtures (``tests/golden/decode_*.npz``: ``HSN._decode`` on the CPU, float32 and under
bf16 autocast) and against the oracle at the benchmark's sizes."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import dev, load_golden, synthetic_window, to_np
from oracle import window_oracle as O

pytestmark = pytest.mark.gpu

KEYS = ("dec_w1", "dec_b1", "dec_w2", "dec_b2")


def _decoder(P, d_q, prod):
    from hsn_b200.window import WindowDecoder

    return WindowDecoder.build(P["dec_w1"], P["dec_b1"], P["dec_w2"], P["dec_b2"], d_q=d_q, device="cuda", prod=prod)


@pytest.mark.parametrize("name", ["f32", "bf16"])
def test_decode_equals_the_reference(name: str) -> None:
    from hsn_b200.window import window_decode

    z = load_golden(f"decode_{name}")
    bf = name == "bf16"
    dec = _decoder({k: z[k] for k in KEYS}, z["qs"].shape[-1], "bf16" if bf else "fp32")
    out: dict = {}
    got = window_decode(dec, dev(z["qs"]), dev(z["us"]), out=out)
    assert int(out["decode_status"][0]) == 0 and tuple(got.shape) == z["logits"].shape
    scale = float(np.abs(z["logits"]).max())
    tol = 2e-2 if bf else 1e-5
    np.testing.assert_allclose(to_np(got), z["logits"], rtol=tol, atol=tol * scale)
    if bf:   # bfloat16 logits: all but a few equal the reference's to the bit (a float32 sum on a rounding boundary)
        assert float(np.mean(to_np(got) == z["logits"])) > 0.97
    again = window_decode(dec, dev(z["qs"]), dev(z["us"]), out=out)
    assert again.data_ptr() == got.data_ptr()


@pytest.mark.parametrize("prod", ["bf16", "fp32"])
@pytest.mark.parametrize("rows,d,H,V", [((32, 256), 64, 512, 256), ((5,), 64, 512, 256), ((3, 7), 16, 200, 130)])
def test_decode_equals_the_oracle(prod: str, rows, d: int, H: int, V: int) -> None:
    """The benchmark's decoder over a whole window's 8192 rows, a serving step's handful, and widths that are
    no multiples of a tile."""
    from hsn_b200.window import window_decode

    rng = np.random.default_rng(5)
    f = lambda *s: (rng.standard_normal(s) * 0.2).astype(np.float32)  # noqa: E731
    P = dict(dec_w1=f(H, 2 * d), dec_b1=f(H), dec_w2=f(V, H), dec_b2=f(V))
    if prod == "bf16":
        P = {k: O.bf16_round(v) for k, v in P.items()}
    qs, us = f(*rows, d), f(*rows, d)
    want = O.window_decode(P, qs, us, bf16=prod == "bf16")
    got = to_np(window_decode(_decoder(P, d, prod), dev(qs), dev(us)))
    scale = float(np.abs(want).max())
    tol = 2e-2 if prod == "bf16" else 1e-5
    np.testing.assert_allclose(got, want, rtol=tol, atol=tol * scale)
    if prod == "bf16":
        assert float(np.mean(got == want)) > 0.97


@pytest.mark.parametrize("prod,row_clusters", [("bf16", True), ("bf16", False), ("fp32", False)])
def test_forward_sweeps_return_u(prod: str, row_clusters: bool) -> None:
    """``want_us``: the shared path's output at every position, by the row kernels and by the phases, against
    the oracle with the same decisions."""
    from hsn_b200.window import WindowModel, window_forward

    rng = np.random.default_rng(8)
    B, T, N, d, K, H, M, D = 4, 6, 64, 32, 4, 128, 3, 2
    W, z, ctx, scalars, reset, state = synthetic_window(rng, B, T, N, d, K, H, M, D, 0.2)
    if prod == "bf16":
        for key in ("w1", "w2", "gate_w", "v_w", "wout_w"):
            setattr(W, key, O.bf16_round(getattr(W, key)))
    model = WindowModel.from_oracle_weights(W, device="cuda", prod=prod, row_clusters=row_clusters)
    tape = window_forward(model, dev(z), dev(ctx), dev(scalars), dev(reset), tuple(dev(s) for s in state), want_us=True)
    assert tape["path"] == ("rows" if row_clusters else "phases") and int(tape["status"]) == 0
    forced = tuple(to_np(tape[k]) for k in ("sel_cell_idx", "sel_unit_idx", "sel_valid"))
    want = O.window_forward(W, z, ctx, scalars, reset, *state, bf16=prod == "bf16", forced=forced)
    tol = 2e-2 if prod == "bf16" else 1e-5
    scale = float(np.abs(want["us"]).max())
    np.testing.assert_allclose(to_np(tape["us"]), want["us"], rtol=tol, atol=tol * scale)
    np.testing.assert_allclose(to_np(tape["qs"]), want["qs"], rtol=tol, atol=tol * float(np.abs(want["qs"]).max()))
    assert "us" not in window_forward(model, dev(z), dev(ctx), dev(scalars), dev(reset), tuple(dev(s) for s in state))


def test_decode_refuses_what_it_cannot_take() -> None:
    from hsn_b200._lib import WindowKernelError
    from hsn_b200.window import window_decode

    rng = np.random.default_rng(6)
    f = lambda *s: rng.standard_normal(s).astype(np.float32)  # noqa: E731
    P = dict(dec_w1=f(24, 20), dec_b1=f(24), dec_w2=f(9, 24), dec_b2=f(9))
    dec = _decoder(P, 10, "bf16")   # widths that are no multiples of 8: bf16 products decline by name
    with pytest.raises(WindowKernelError, match="multiples of 8"):
        window_decode(dec, dev(f(3, 10)), dev(f(3, 10)))
    fp = _decoder(P, 10, "fp32")
    got = to_np(window_decode(fp, dev(f(3, 10)), dev(f(3, 10))))
    assert got.shape == (3, 9) and np.isfinite(got).all()
    with pytest.raises(ValueError):
        window_decode(fp, dev(f(3, 10)), None)
    with pytest.raises(ValueError):
        window_decode(fp, dev(f(3, 11)), dev(f(3, 10)))


def test_serving_step_with_logits() -> None:
    """The reference's serving step returns logits: two streamed positions (the second carried) and the decoder
    on each step's ``qs`` and ``us``, against the oracle's step and decoder."""
    from hsn_b200.window import WindowModel, stream_step, window_decode

    rng = np.random.default_rng(10)
    B, N, d, K, H, M, D = 6, 64, 32, 4, 128, 3, 2
    W, z, ctx, scalars, reset, state = synthetic_window(rng, B, 2, N, d, K, H, M, D, 0.0)
    reset[:, 0] = False
    f = lambda *s: (rng.standard_normal(s) * 0.2).astype(np.float32)  # noqa: E731
    P = dict(dec_w1=f(96, 2 * d), dec_b1=f(96), dec_w2=f(256, 96), dec_b2=f(256))
    model = WindowModel.from_oracle_weights(W, device="cuda", prod="fp32")
    dec = _decoder(P, d, "fp32")
    live = tuple(dev(s) for s in state)
    h, q, age, pos = state
    step = None
    for t in range(2):
        step = stream_step(model, dev(z[:, t]), dev(ctx[:, t]), dev(scalars[:, t]), dev(reset[:, t]), live, out=step,
                           carried=t > 0, want_us=True)  # fmt: skip
        logits = window_decode(dec, step["qs"][:, 0], step["us"][:, 0])
        p = O.stream_step(W, z[:, t], ctx[:, t], scalars[:, t], reset[:, t], h, q, age, pos)
        h, q, age, pos = p["h"], p["q"], p["age"], p["pos"]
        want = O.window_decode(P, p["q"], p["u"])
        assert tuple(logits.shape) == (B, 256)
        np.testing.assert_allclose(to_np(logits), want, rtol=1e-5, atol=1e-5 * float(np.abs(want).max()))
