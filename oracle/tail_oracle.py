"""TEST INFRASTRUCTURE ONLY: a numpy restatement of the end of the replay's cell pass and its backward.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU legs may import this module; the product path
never does.

What is restated (reference ``python/hsn/model/cell.py:719-721``, the branch of ``PDGCell.replay_sparse`` with the
candidate norm on): for ``P`` slots ``y = W_out(unit_out)`` without bias, cast to the state's float32,
``pre = RMSNorm_g(y)`` (``cell.py:210-211``: ``eps = 1e-6``) and ``c = tanh(alpha * pre)`` with ``alpha`` the slot's
weight; ``record["y"] = y`` (``cell.py:723``). Its backward is autograd's of those operations:
``dz = d_c (1 - c^2)``, ``d_alpha = sum_j dz pre``, ``d_pre = alpha dz``, ``d_g = sum_p d_pre y rho``,
``d_y = rho (g d_pre) - rho^3 y mean_j(y g d_pre)`` with ``rho = 1 / sqrt(mean(y^2) + eps)``,
``d_unit_out = d_y W_out``, ``d_W_out = d_y^T unit_out``.

``bf16=True`` is the pass under ``torch.autocast(dtype=bfloat16)``: the linear reads ``unit_out`` and ``W_out`` as
bfloat16, sums in float32 and rounds ``y`` to bfloat16; the norm and the ``tanh`` stay in float32. In the backward
``d_y`` is rounded to bfloat16 where it crosses the cast, and both of the linear's products are rounded to bfloat16.

Pinned by ``tests/golden/replay_*.npz`` (made by ``tests/golden/make_golden.py --only replay`` from the reference's
own ``replay_sparse`` inside a split window, float32 and under CPU autocast).
"""

from __future__ import annotations

import numpy as np

from .window_oracle import bf16_round

__all__ = ["forward_tail", "backward_tail"]


def _r(x: np.ndarray, bf16: bool) -> np.ndarray:
    return bf16_round(x.astype(np.float32)) if bf16 else x


def _rho(y: np.ndarray, eps: float) -> np.ndarray:
    return 1.0 / np.sqrt((y * y).mean(axis=-1, keepdims=True) + y.dtype.type(eps))


def forward_tail(unit_out, alpha, w_out, cand_w, *, cand_eps: float = 1e-6, bf16: bool = False):
    """``(c [P, d], y [P, d])`` for ``unit_out [P, d]``, ``alpha [P]``, ``w_out [d, d]`` (``nn.Linear``'s
    ``[out, in]``) and the norm's gain ``cand_w [d]``."""
    x = np.asarray(unit_out)
    y = _r(_r(x, bf16) @ _r(w_out, bf16).T, bf16).astype(x.dtype)
    pre = y * _rho(y, cand_eps) * cand_w.astype(x.dtype)
    c = np.tanh(np.asarray(alpha, dtype=x.dtype)[:, None] * pre).astype(x.dtype)
    return c, y


def backward_tail(unit_out, alpha, w_out, cand_w, y, d_c, *, cand_eps: float = 1e-6, bf16: bool = False):
    """``(d_unit_out [P, d], d_alpha [P], d_w_out [d, d], d_cand_w [d])`` for the cotangent ``d_c`` of
    :func:`forward_tail`'s ``c``, with ``y`` its record."""
    x = np.asarray(unit_out)
    dtype = x.dtype
    a = np.asarray(alpha, dtype=dtype)[:, None]
    g = cand_w.astype(dtype)
    rho = _rho(y, cand_eps)
    pre = y * rho * g
    c = np.tanh(a * pre)
    dz = np.asarray(d_c, dtype=dtype) * (1 - c * c)
    d_alpha = (dz * pre).sum(axis=-1)
    d_pre = a * dz
    d_cand_w = (d_pre * y * rho).sum(axis=0)
    scaled = d_pre * g
    d_y = rho * scaled - rho * rho * rho * y * (y * scaled).mean(axis=-1, keepdims=True)
    d_yb = _r(d_y, bf16)
    d_unit_out = _r(d_yb @ _r(w_out, bf16), bf16).astype(dtype)
    d_w_out = _r(d_yb.T @ _r(x, bf16), bf16).astype(dtype)
    return d_unit_out, d_alpha.astype(dtype), d_w_out, d_cand_w.astype(dtype)
