"""TEST INFRASTRUCTURE ONLY: a numpy restatement of the cell norm and the gate of the replay's cell pass, with their
backward.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU legs may import this module; the product path
never does.

What is restated (reference ``python/hsn/model/cell.py:707-709`` in ``PDGCell.replay_sparse``): for ``P`` slots with
the gathered inputs ``v_raw [P, 4d]``, ``v = RMSNorm_w(v_raw)`` (the unit pass's and the gate's input),
``gate_pre = gate(v)`` (``nn.Linear(4d, d)`` with bias) cast to the state's float32, ``b = sigmoid(gate_pre)``, and the
record's ``rms = 1 / sqrt(mean(v_raw^2) + eps)`` (``cell.py:727-733``). Its backward is autograd's: ``d_gate_pre =
d_b b (1 - b)``, ``d_v = d_v_units + d_gate_pre W_gate`` (``d_v_units`` is what the unit pass's backward returns),
``d_W_gate = d_gate_pre^T v``, ``d_b_gate = sum_p d_gate_pre``, then the norm's: ``d_w = sum_p d_v v_raw rms``,
``d_v_raw = rms (w d_v) - rms^3 v_raw mean_j(v_raw w d_v)``.

``bf16=True`` is the pass under ``torch.autocast(dtype=bfloat16)``: the norm stays in float32; the gate reads ``v``,
its weight and bias as bfloat16, sums in float32 and rounds to bfloat16; in the backward ``d_gate_pre`` is rounded to
bfloat16 where it crosses the cast and the linear's two products and the bias sum are rounded to bfloat16.

Pinned by ``tests/golden/replay_*.npz`` (made by ``tests/golden/make_golden.py --only replay`` from the reference's
own ``replay_sparse`` inside a split window, float32 and under CPU autocast).
"""

from __future__ import annotations

import numpy as np

from .window_oracle import bf16_round, sigmoid

__all__ = ["forward_norm_gate", "backward_norm_gate"]


def _r(x: np.ndarray, bf16: bool) -> np.ndarray:
    return bf16_round(x.astype(np.float32)) if bf16 else x


def forward_norm_gate(v_raw, norm_w, gate_w, gate_b, *, norm_eps: float, bf16: bool = False):
    """``(v [P, 4d], rms [P], gate_pre [P, d], b [P, d])`` for ``v_raw [P, 4d]``, the norm's gain ``norm_w [4d]``,
    ``gate_w [d, 4d]`` and ``gate_b [d]``."""
    x = np.asarray(v_raw)
    dtype = x.dtype
    rms = 1.0 / np.sqrt((x * x).mean(axis=-1) + dtype.type(norm_eps))
    v = x * rms[:, None] * norm_w.astype(dtype)
    gate_pre = _r(_r(v, bf16) @ _r(gate_w, bf16).T + _r(gate_b, bf16), bf16).astype(dtype)
    return v, rms, gate_pre, sigmoid(gate_pre)


def backward_norm_gate(v_raw, norm_w, gate_w, gate_b, d_v_units, d_b, *, norm_eps: float, bf16: bool = False):
    """``(d_v_raw [P, 4d], d_norm_w [4d], d_gate_w [d, 4d], d_gate_b [d])`` for the cotangents ``d_v_units`` of
    ``v`` (from the unit pass) and ``d_b`` of ``b``."""
    x = np.asarray(v_raw)
    dtype = x.dtype
    v, rms, _, b = forward_norm_gate(x, norm_w, gate_w, gate_b, norm_eps=norm_eps, bf16=bf16)
    d_gp = _r(np.asarray(d_b, dtype=dtype) * b * (1 - b), bf16)
    d_gate_w = _r(d_gp.T @ _r(v, bf16), bf16).astype(dtype)
    d_gate_b = _r(d_gp.sum(axis=0), bf16).astype(dtype)
    d_v = np.asarray(d_v_units, dtype=dtype) + _r(d_gp @ _r(gate_w, bf16), bf16).astype(dtype)
    r = rms[:, None]
    d_norm_w = (d_v * x * r).sum(axis=0)
    scaled = d_v * norm_w.astype(dtype)
    d_v_raw = r * scaled - r * r * r * x * (x * scaled).mean(axis=-1, keepdims=True)
    return d_v_raw.astype(dtype), d_norm_w.astype(dtype), d_gate_w, d_gate_b
