"""TEST INFRASTRUCTURE ONLY: a numpy restatement of the messages and the gathered inputs of the replay's cell pass, with
their backward.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU legs may import this module; the product path
never does.

What is restated (reference ``python/hsn/model/cell.py:698-705`` in ``PDGCell.replay_sparse``, with
``python/hsn/kernels/native.py:113-157`` ``gather_concat``): for the ``K`` selected cells of each of ``R`` rows, with
``src = pad_src[cell]`` the cell's ``D`` in-neighbours and ``w = edge_w[cell]`` their weights (zero on padding),
``sources_j = V(h[src_j])``, ``m = sum_j w_j sources_j`` and ``v_raw = [u ; eps ; h[cell] ; m]``. The state is a
constant there, so the backward gives ``d_u = sum_k d_v_raw[:, k, :d]``, ``d_eps`` likewise, ``d_edge_w[n, j] = sum
over the slots of cell n of <d_m, sources_j>`` and ``d_V = sum_{slots, j} (w_j d_m)^T h[src_j]``.

``bf16=True`` is the pass under ``torch.autocast(dtype=bfloat16)``: ``V`` reads bfloat16 operands, sums in float32 and
rounds to bfloat16; the weights are cast to bfloat16, each product ``w_j sources_j`` is a bfloat16 value and their sum
over ``j`` is rounded once; the concatenation is float32. In the backward ``d_m`` is rounded to bfloat16, the products
``w_j d_m`` and ``d_m sources_j`` are bfloat16 values, the sum over the features of the latter is rounded to bfloat16,
and ``d_V`` is a bfloat16 product. The reference adds the slots' shares of ``d_edge_w`` one by one into a bfloat16
tensor; here they are summed in float32 and rounded once (the same value while a cell has a few slots).

Pinned by ``tests/golden/replay_*.npz`` (made by ``tests/golden/make_golden.py --only replay``).
"""

from __future__ import annotations

import numpy as np

from .window_oracle import bf16_round

__all__ = ["forward_messages", "backward_messages"]


def _r(x: np.ndarray, bf16: bool) -> np.ndarray:
    return bf16_round(x.astype(np.float32)) if bf16 else x


def _sources(h, cells, pad_src, v_w, bf16):
    R = h.shape[0]
    src = pad_src[cells]                                            # [R, K, D]
    h_src = h[np.arange(R)[:, None, None], src]                     # [R, K, D, d]
    return h_src, _r(_r(h_src, bf16) @ _r(v_w, bf16).T, bf16)


def forward_messages(u, eps, h, cells, pad_src, edge_w, v_w, *, bf16: bool = False):
    """``v_raw [R, K, 4d]`` for ``u, eps [R, d]``, ``h [R, N, d]``, ``cells [R, K]`` (padded slots hold cell 0),
    ``pad_src [N, D]``, ``edge_w [N, D]`` and ``v_w [d, d]`` (``nn.Linear``'s ``[out, in]``)."""
    h = np.asarray(h)
    R, K = cells.shape
    d = h.shape[-1]
    _, sources = _sources(h, cells, pad_src, v_w, bf16)
    w = _r(edge_w, bf16)[cells]                                     # [R, K, D]
    m = _r(_r(sources * w[..., None], bf16).sum(axis=2), bf16).astype(h.dtype)
    rows = np.arange(R)[:, None]
    return np.concatenate([np.broadcast_to(u[:, None], (R, K, d)), np.broadcast_to(eps[:, None], (R, K, d)), h[rows, cells], m], axis=-1)


def backward_messages(h, cells, pad_src, edge_w, v_w, d_v_raw, *, bf16: bool = False):
    """``(d_u [R, d], d_eps [R, d], d_edge_w [N, D], d_v_w [d, d])`` for the cotangent ``d_v_raw [R, K, 4d]``."""
    h = np.asarray(h)
    d = h.shape[-1]
    dtype = h.dtype
    d_u = d_v_raw[..., :d].sum(axis=1).astype(dtype)
    d_eps = d_v_raw[..., d : 2 * d].sum(axis=1).astype(dtype)
    h_src, sources = _sources(h, cells, pad_src, v_w, bf16)
    w = _r(edge_w, bf16)[cells]
    d_m = _r(d_v_raw[..., 3 * d :], bf16)                           # [R, K, d]
    d_w_slots = _r(_r(d_m[:, :, None, :] * sources, bf16).sum(axis=-1), bf16)   # [R, K, D]
    d_edge_w = np.zeros(edge_w.shape, dtype=np.float64)
    np.add.at(d_edge_w, cells, d_w_slots.astype(np.float64))
    d_sources = _r(d_m[:, :, None, :] * w[..., None], bf16)         # [R, K, D, d]
    flat = d_sources.reshape(-1, d)
    d_v_w = _r(flat.T @ _r(h_src, bf16).reshape(-1, d), bf16)
    return d_u, d_eps, _r(d_edge_w.astype(dtype), bf16), d_v_w.astype(dtype)
