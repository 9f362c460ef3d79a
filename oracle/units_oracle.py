"""TEST INFRASTRUCTURE ONLY: a numpy restatement of the replay's grouped unit pass and its backward.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU legs may import this module; the product path
never does.

What is restated (reference ``python/hsn/model/units.py:356-414``, ``UnitBank.forward_grouped``): for ``P`` pairs
``(v_p [4d], unit_p)`` the chosen unit's two-layer perceptron ``out_p = act(v_p W1[u] + b1[u]) W2[u] + b2[u]`` with
``act`` the exact-erf GELU, the pairs of a unit taken together as one ``addmm`` per layer, and ``record["hidden"]``
= the first layer's pre-activation in the input order. Its backward is autograd's of those operations: per unit
``d_hidden = d_out W2ᵀ``, ``d_W2 = hiddenᵀ d_out``, ``d_b2 = Σ_p d_out``, ``d_pre = d_hidden · act'(pre)``,
``d_v = d_pre W1ᵀ``, ``d_W1 = vᵀ d_pre``, ``d_b1 = Σ_p d_pre``.

``bf16=True`` is the pass under ``torch.autocast(dtype=bfloat16)``: every ``addmm`` reads its three operands as
bfloat16, sums in float32 and rounds its output to bfloat16, the activation and its derivative are evaluated in
float32 on bfloat16 values and rounded, and in the backward every product (the weight gradients too) and every bias
sum is rounded to bfloat16 before it is widened to the parameter's float32.

Pinned by ``tests/golden/units_*.npz`` (made by ``tests/golden/make_golden.py --only units`` from the reference's own
module in float64, float32 and under CPU autocast).
"""

from __future__ import annotations

import numpy as np

from .window_oracle import bf16_round, gelu, gelu_grad

__all__ = ["forward_grouped", "backward_grouped"]


def _r(x: np.ndarray, bf16: bool) -> np.ndarray:
    return bf16_round(x.astype(np.float32)) if bf16 else x


def forward_grouped(v, unit_idx, W1, b1, W2, b2, *, bf16: bool = False):
    """``(out [P, d], pre [P, H])``: the pass and its record. float64 inputs stay float64; ``bf16`` wants float32."""
    v = np.asarray(v)
    P, M = v.shape[0], W1.shape[0]
    idx = np.asarray(unit_idx, dtype=np.int64)
    if P and (idx.min() < 0 or idx.max() >= M):
        raise IndexError(f"unit_idx values must lie in [0, {M})")
    out = np.zeros((P, W2.shape[2]), dtype=v.dtype)
    pre = np.zeros((P, W1.shape[2]), dtype=v.dtype)
    for j in range(M):
        rows = np.nonzero(idx == j)[0]
        if rows.size == 0:
            continue
        x = _r(v[rows], bf16)
        pre[rows] = _r(x @ _r(W1[j], bf16) + _r(b1[j], bf16), bf16)
        hid = _r(gelu(pre[rows]), bf16)
        out[rows] = _r(hid @ _r(W2[j], bf16) + _r(b2[j], bf16), bf16)
    return out, pre


def backward_grouped(v, unit_idx, W1, b1, W2, b2, pre, d_out, *, bf16: bool = False):
    """``(d_v, d_W1, d_b1, d_W2, d_b2)`` for the cotangent ``d_out [P, d]`` of :func:`forward_grouped`'s ``out``,
    with ``pre`` its record. A unit no pair chose gets zero gradients."""
    v = np.asarray(v)
    idx = np.asarray(unit_idx, dtype=np.int64)
    d_v = np.zeros_like(v)
    d_W1, d_b1, d_W2, d_b2 = (np.zeros_like(a) for a in (W1, b1, W2, b2))
    for j in range(W1.shape[0]):
        rows = np.nonzero(idx == j)[0]
        if rows.size == 0:
            continue
        x = _r(v[rows], bf16)
        g = _r(d_out[rows], bf16)
        hid = _r(gelu(pre[rows]), bf16)
        d_hid = _r(g @ _r(W2[j], bf16).T, bf16)
        d_W2[j] = _r(hid.T @ g, bf16)
        d_b2[j] = _r(g.sum(axis=0), bf16)
        d_pre = _r(d_hid * gelu_grad(pre[rows]), bf16)
        d_v[rows] = _r(d_pre @ _r(W1[j], bf16).T, bf16)
        d_W1[j] = _r(x.T @ d_pre, bf16)
        d_b1[j] = _r(d_pre.sum(axis=0), bf16)
    return d_v, d_W1, d_b1, d_W2, d_b2
