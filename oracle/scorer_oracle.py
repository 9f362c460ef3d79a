"""TEST INFRASTRUCTURE ONLY: a numpy restatement of the replay's scorer logits and of the gradients of the scorer's
weight and bias.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU legs may import this module; the product path
never does.

What is restated (reference ``python/hsn/train/split.py:305-342``, ``_scorer_logits``, for the linear scorer without
an address gate and without excluded features): for ``R`` window positions and ``N`` cells the logits ``[R, N, M]`` of
the features ``[u; eps; h_i; age_i / age_max; scalars_i]`` without building them — the product is taken per feature
block: ``row = [u; eps] W[:, :2d]^T`` once per position, ``cells = h W[:, 2d:3d]^T`` and ``tail = [age / age_max;
scalars] W[:, 3d:]^T + b`` per cell, ``out = (cells + tail) + row``. The features are constants of the replay (``h``
is the recorded state, ``u`` and ``eps`` are detached): autograd's backward gives ``d W`` and ``d b`` only.

``bf16=True`` is the pass under ``torch.autocast(dtype=bfloat16)``: each of the three linear maps reads bfloat16
operands (the bias too), sums in float32 and rounds its output to bfloat16; the three outputs are added in float32.
In the backward the cotangent reaches each map rounded to bfloat16 (the row map's after its float32 sum over the
cells), and every weight-gradient block and the bias gradient are rounded to bfloat16 before they are widened.

Pinned by ``tests/golden/scorer_*.npz`` (``tests/golden/make_golden.py --only scorer``: the reference's function in
float64, float32 and under CPU autocast).
"""

from __future__ import annotations

import numpy as np

from .window_oracle import bf16_round

__all__ = ["scorer_logits", "scorer_logits_backward"]


def _r(x: np.ndarray, bf16: bool) -> np.ndarray:
    return bf16_round(x.astype(np.float32)) if bf16 else x


def _tail(age, scalars, age_max, dtype):
    return np.concatenate([(age.astype(dtype) / dtype.type(age_max))[..., None], scalars], axis=-1)


def scorer_logits(weight, bias, u, eps, h, age, scalars, age_max, *, bf16: bool = False):
    """``[R, N, M]`` in ``h``'s dtype. ``weight [M, 3d + 1 + S]``, ``bias [M]``, ``u, eps [R, d]``, ``h [R, N, d]``,
    ``age [R, N]`` int64, ``scalars [R, N, S]``."""
    d = h.shape[-1]
    dtype = h.dtype
    x = np.concatenate([u, eps], axis=-1)
    row = _r(_r(x, bf16) @ _r(weight[:, : 2 * d], bf16).T, bf16)
    cells = _r(_r(h, bf16) @ _r(weight[:, 2 * d : 3 * d], bf16).T, bf16)
    tail = _tail(age, scalars, age_max, dtype)
    part = _r(_r(tail, bf16) @ _r(weight[:, 3 * d :], bf16).T + _r(bias, bf16), bf16)
    return ((cells + part) + row[:, None, :]).astype(dtype)


def scorer_logits_backward(weight, u, eps, h, age, scalars, age_max, d_out, *, bf16: bool = False):
    """``(d_weight [M, 3d + 1 + S], d_bias [M])`` for the cotangent ``d_out [R, N, M]``."""
    d = h.shape[-1]
    dtype = h.dtype
    M = weight.shape[0]
    g = _r(d_out, bf16).reshape(-1, M)
    g_row = _r(d_out.sum(axis=1), bf16)   # the broadcast's backward: summed over the cells, then the map's dtype
    x = _r(np.concatenate([u, eps], axis=-1), bf16)
    tail = _r(_tail(age, scalars, age_max, dtype), bf16).reshape(g.shape[0], -1)
    d_weight = np.concatenate(
        [_r(g_row.T @ x, bf16), _r(g.T @ _r(h, bf16).reshape(-1, d), bf16), _r(g.T @ tail, bf16)], axis=1
    ).astype(weight.dtype)
    return d_weight, _r(g.sum(axis=0), bf16).astype(weight.dtype)
