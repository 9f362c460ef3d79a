"""GPU parity of the window's prologue (token and context ids to z, context embeddings, positions and
the scorer's scalars) against the reference's fixtures and the oracle, through the C ABI."""

from __future__ import annotations

import numpy as np
import pytest
import torch
from conftest import dev, load_golden

from oracle import window_oracle as O

pytestmark = pytest.mark.gpu

_TABLES = ("byte_emb", "enc_w1", "enc_b1", "enc_w2", "enc_b2", "ctx_emb", "byte_codes", "cell_addresses",
           "ema_utility", "ema_selected")  # fmt: skip


def _build(tables: dict, prod: str, numbers, position: str):
    from hsn_b200.window import WindowPrologue

    budget, round_frac, n_context, unroll = (float(v) for v in numbers)
    return WindowPrologue.build(tables, device="cuda", prod=prod, budget_frac=budget, round_frac=round_frac,
                                n_context=n_context, unroll=unroll, position=position, bos=O.BOS)  # fmt: skip


@pytest.mark.parametrize("name", ["fresh_f32", "carried_f32", "fresh_bf16"])
def test_prologue_equals_the_reference(name: str) -> None:
    from hsn_b200.window import window_prologue

    z = load_golden(f"prologue_{name}")
    bf = name.endswith("bf16")
    pro = _build({k: z[k] for k in _TABLES}, "bf16" if bf else "fp32", z["numbers"], str(z["position"]))
    prev = dev(z["prev_tokens"]) if "prev_tokens" in z.files else None
    got = window_prologue(pro, dev(z["tokens"]), dev(z["ctx_ids"]), dev(z["reset"].astype(bool)), dev(z["pos0"]), prev)
    tol = 2e-2 if bf else 1e-5
    scale = float(np.abs(z["z"]).max())
    np.testing.assert_allclose(got["z"].cpu().numpy(), z["z"], rtol=tol, atol=tol * scale)
    assert np.array_equal(got["ctx"].cpu().numpy(), z["context"])
    np.testing.assert_allclose(got["scalars"].cpu().numpy(), z["scalars"], rtol=1e-5, atol=1e-5)
    want = O.window_positions(z["pos0"], z["reset"])
    assert np.array_equal(got["positions"].cpu().numpy(), want)


@pytest.mark.parametrize("position", ["document", "clamp", "wrap"])
def test_prologue_equals_the_oracle_at_the_reference_shape(position: str) -> None:
    """B8 T64 N256 d64 H512 with per-row running averages, carried positions beyond the unroll and a
    carried previous byte: every output against the oracle's restatement."""
    from hsn_b200.window import window_prologue

    rng = np.random.default_rng(3)
    B, T, N, d, H, V = 8, 64, 256, 64, 512, 256
    f = lambda *s: (rng.standard_normal(s) * 0.3).astype(np.float32)  # noqa: E731
    P = dict(byte_emb=f(V, d), enc_w1=f(H, d), enc_b1=f(H), enc_w2=f(d, H), enc_b2=f(d), ctx_emb=f(16, d),
             byte_codes=f(V, d), cell_addresses=f(N, d), ema_utility=rng.random((B, N)).astype(np.float32),
             ema_selected=rng.random((B, N)).astype(np.float32))  # fmt: skip
    numbers = (0.75, 0.0, 16.0, 48.0)
    tokens = rng.integers(0, V, (B, T))
    ctx_ids = rng.integers(0, 16, (B, T))
    reset = rng.random((B, T)) < 0.05
    pos0 = rng.integers(0, 300, B)
    prev = rng.integers(0, V, B)
    want = O.window_prologue(dict(P, budget_frac=numbers[0], round_frac=numbers[1], n_context=numbers[2], unroll=numbers[3],
                                  position=position), tokens, ctx_ids, reset, pos0, prev)  # fmt: skip
    pro = _build(P, "fp32", numbers, position)
    got = window_prologue(pro, dev(tokens), dev(ctx_ids), dev(reset), dev(pos0), dev(prev))
    scale = float(np.abs(want["z"]).max())
    np.testing.assert_allclose(got["z"].cpu().numpy(), want["z"], rtol=1e-5, atol=1e-5 * scale)
    assert np.array_equal(got["ctx"].cpu().numpy(), want["ctx"])
    assert np.array_equal(got["positions"].cpu().numpy(), want["positions"])
    np.testing.assert_allclose(got["scalars"].cpu().numpy(), want["scalars"], rtol=1e-5, atol=1e-5)
    # the buffers of a result are reused by the next call of the same size
    again = window_prologue(pro, dev(tokens), dev(ctx_ids), dev(reset), dev(pos0), dev(prev), out=got)
    assert again["scalars"].data_ptr() == got["scalars"].data_ptr()
    with pytest.raises(ValueError):
        window_prologue(pro, dev(tokens[:4]), dev(ctx_ids[:4]), dev(reset[:4]), dev(pos0[:4]))  # per-row averages of 8 rows


def test_prologue_with_more_cells_than_one_staging_tile() -> None:
    """N 2304: the scalars of a row leave in tiles of 1024 cells, the last one of 256 (the scaling
    configuration has 4096 cells)."""
    from hsn_b200.window import window_prologue

    rng = np.random.default_rng(9)
    B, T, N, d, H, V = 2, 5, 2304, 16, 32, 256
    f = lambda *s: (rng.standard_normal(s) * 0.3).astype(np.float32)  # noqa: E731
    P = dict(byte_emb=f(V, d), enc_w1=f(H, d), enc_b1=f(H), enc_w2=f(d, H), enc_b2=f(d), ctx_emb=f(16, d),
             byte_codes=f(V, d), cell_addresses=f(N, d), ema_utility=rng.random(N).astype(np.float32),
             ema_selected=rng.random(N).astype(np.float32))  # fmt: skip
    numbers = (0.5, 0.25, 16.0, 8.0)
    tokens, ctx_ids = rng.integers(0, V, (B, T)), rng.integers(0, 16, (B, T))
    reset = rng.random((B, T)) < 0.3
    pos0 = rng.integers(0, 20, B)
    want = O.window_prologue(dict(P, budget_frac=numbers[0], round_frac=numbers[1], n_context=numbers[2], unroll=numbers[3],
                                  position="wrap"), tokens, ctx_ids, reset, pos0, None)  # fmt: skip
    got = window_prologue(_build(P, "fp32", numbers, "wrap"), dev(tokens), dev(ctx_ids), dev(reset), dev(pos0))
    np.testing.assert_allclose(got["scalars"].cpu().numpy(), want["scalars"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(got["z"].cpu().numpy(), want["z"], rtol=1e-5, atol=1e-5 * float(np.abs(want["z"]).max()))
