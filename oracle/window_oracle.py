"""CPU oracle of the HSN window path. TEST INFRASTRUCTURE ONLY.

A numpy restatement of the reference's algorithm for the TBPTT window (forward sweep, full-cut
and state-gradient backward recurrences, streaming step). Only the tests, the smoke check and the
benchmark's CPU-baseline leg may import this module; the product path (``hsn_b200``) never does
and fails loudly when its CUDA library is missing.

Parity is pinned: ``tests/test_oracle_golden.py`` checks every function here against fixtures
produced by running the reference's own CPU code (``tests/golden/make_golden.py``), among them the
reference tests' tie-heavy selection trials and its float64 recurrences.

Every function cites the reference file:line it follows (paths inside the reference project).
All arrays are numpy; ``dtype`` is the state dtype (float32, or float64 for the tight checks).
Weights are in torch's layouts (``nn.Linear.weight`` is ``[out, in]``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

try:  # scipy's vectorised erf; the fallback is exact too, only slower
    from scipy.special import erf as _erf
except Exception:  # pragma: no cover
    _erf = np.vectorize(math.erf, otypes=[np.float64])

_SQRT1_2 = 0.7071067811865475244
_INV_SQRT_2PI = 0.3989422804014326779


# --------------------------------------------------------------------------------------------------
# Small numerics
# --------------------------------------------------------------------------------------------------


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round float32 values to bfloat16 (nearest, ties to even) and return them as float32: the
    cast torch makes (reference ``kernels/cuda/hsn_window.cu:34-38`` states the same rule)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    nan = (bits & 0x7FFFFFFF) > 0x7F800000
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    rounded = np.where(nan, ((bits >> 16) | 0x40) << 16, rounded)
    return (rounded & 0xFFFFFFFF).astype(np.uint32).view(np.float32).reshape(x.shape)


def gelu(x: np.ndarray) -> np.ndarray:
    """Exact (erf) GELU, the reference's ``model.activation = gelu``
    (``python/hsn/model/encoder.py`` ACTIVATIONS; ``kernels/cuda/hsn_window.cu:189-191``)."""
    return (0.5 * x * (1.0 + _erf(x * _SQRT1_2))).astype(x.dtype)


def gelu_grad(x: np.ndarray) -> np.ndarray:
    """``python/hsn/train/state_gradient.py:192-197``."""
    cdf = 0.5 * (1.0 + _erf(x * _SQRT1_2))
    return (cdf + x * np.exp(-0.5 * x * x) * _INV_SQRT_2PI).astype(x.dtype)


def sigmoid(x: np.ndarray) -> np.ndarray:
    return (1.0 / (1.0 + np.exp(-x))).astype(x.dtype)


# --------------------------------------------------------------------------------------------------
# The router's hard decision
# --------------------------------------------------------------------------------------------------


def select(
    logits: np.ndarray,
    age: np.ndarray | None,
    cost: np.ndarray,
    *,
    k: int,
    age_max: int,
    probes: bool,
    lambda_cost: float,
    cell_overhead: float,
    shared_cost: float,
    limit: float,
    reserved: int = 0,
    reserved_units: bool = False,
):
    """``Router.select`` with mode ``topk``, the hard decision, no exploration
    (``python/hsn/model/router.py:1263-1417``): ``_topk`` ``:1640-1648`` (stable descending sort:
    equal scores keep index order; the unit is the first maximiser), ``_truncate`` ``:1650-1657``
    (longest prefix inside the budget; padded slots hold cell 0 and unit 0), ``_ste_threshold``
    ``:1771-1786`` and the refresh probes of ``_post_process`` ``:1788-1850``.

    ``logits [B, N, M]`` float32, ``age [B, N]`` int64, ``cost [M]`` float32. Returns ``(cells,
    units [B, k] int64, valid [B, k] bool, theta [B] float32, refreshed [B, k] bool)``."""
    logits = np.asarray(logits, dtype=np.float32)
    cost = np.asarray(cost, dtype=np.float32)
    B, N, M = logits.shape
    f32 = np.float32
    scores = logits
    if lambda_cost > 0.0:
        scores = logits - f32(lambda_cost) * cost  # router.py:1246-1252
    cell_scores = scores.max(axis=2)
    unit_argmax = scores.argmax(axis=2)  # the first maximiser
    key = cell_scores.copy()
    if reserved:
        key[:, :reserved] = np.inf
    order = np.argsort(-key, axis=1, kind="stable")[:, :k]
    units = np.take_along_axis(unit_argmax, order, axis=1)
    if reserved and reserved_units:
        units[:, :reserved] = np.arange(reserved) % M
    cells = order
    per_slot = (f32(cell_overhead) + cost[units]).astype(f32)
    cumulative = f32(shared_cost) + np.cumsum(per_slot, axis=1, dtype=f32)
    valid = cumulative <= f32(limit)
    cells = np.where(valid, cells, 0)
    units = np.where(valid, units, 0)
    rows = np.arange(B)[:, None]

    def selected_mask(c: np.ndarray) -> np.ndarray:
        counts = np.zeros((B, N), dtype=np.int64)
        np.add.at(counts, (np.broadcast_to(rows, c.shape), c), valid.astype(np.int64))
        return counts > 0

    chosen = selected_mask(cells)
    lowest_in = np.where(chosen, cell_scores, f32(np.inf))
    if reserved:
        lowest_in[:, :reserved] = np.inf
    highest_out = np.where(chosen, f32(-np.inf), cell_scores)
    with np.errstate(invalid="ignore"):
        theta = (f32(0.5) * (lowest_in.min(axis=1) + highest_out.max(axis=1))).astype(f32)
    refreshed = np.zeros((B, k), dtype=bool)
    if probes and age is not None:
        age = np.asarray(age, dtype=np.int64)
        cells0, units0 = cells, units
        n_valid = valid.sum(axis=1)
        slots = np.arange(k)[None, :]
        stale = (age > age_max) & ~chosen
        n_force = np.minimum(stale.sum(axis=1), np.clip(n_valid - reserved, 0, None))
        stale_key = np.where(stale, age, -1).astype(np.float32)
        by_age = np.argsort(-stale_key, axis=1, kind="stable")  # stalest first, ties by index
        j = n_valid[:, None] - 1 - slots
        replace = (j >= 0) & (j < n_force[:, None])
        new_cells = np.take_along_axis(by_age, np.clip(j, 0, N - 1), axis=1)
        cells = np.where(replace, new_cells, cells)
        units = np.where(replace, np.take_along_axis(unit_argmax, new_cells, axis=1), units)
        refreshed = replace
        spent = ((f32(cell_overhead) + cost[units]) * valid.astype(f32)).astype(f32)
        over = (f32(shared_cost) + spent.sum(axis=1, dtype=f32)) > f32(limit)
        cells = np.where(over[:, None], cells0, cells)
        units = np.where(over[:, None], units0, units)
        refreshed = refreshed & ~over[:, None]
    return cells.astype(np.int64), units.astype(np.int64), valid, theta, refreshed


# --------------------------------------------------------------------------------------------------
# The end of a position's round
# --------------------------------------------------------------------------------------------------


def cell_update(y, gate, h, q, age, pos, cells, valid, cand_w, *, cand_norm: bool, cand_eps: float):
    """The candidate, the gate, the gated write and the tick of one position
    (``python/hsn/model/cell.py:478-487``; ``python/hsn/kernels/native.py:244-303``
    ``gated_delta_update``; ``python/hsn/model/state.py:316-324`` ``tick``; the contract of
    ``hsn_win_cell_update``, ``kernels/cuda/hsn_window.cu:751-791``).

    ``y``, ``gate`` ``[B, K, d]``; ``h [B, N, d]``, ``q [B, d]``, ``age [B, N]``, ``pos [B]``.
    Returns ``(h', q', age', pos', h_sel [B, K, d], h_max [B], c, b)``: padded slots write nothing
    and read cell 0 (after the update) in ``h_sel``."""
    dtype = h.dtype
    B, N, d = h.shape
    K = cells.shape[1]
    y = y.astype(dtype)
    gate = gate.astype(dtype)
    if cand_norm:
        scale = 1.0 / np.sqrt((y * y).mean(axis=-1, keepdims=True) + dtype.type(cand_eps))
        pre = y * scale * cand_w.astype(dtype)
    else:
        pre = y
    c = np.tanh(pre).astype(dtype)
    b = sigmoid(gate)
    safe = np.where(valid, cells, 0)
    rows = np.arange(B)[:, None]
    h_old = h[rows, safe]  # [B, K, d]
    gated = (1 - b) * h_old + b * c
    h_new = np.where(valid[..., None], gated, h_old).astype(dtype)
    h_next = h.copy()
    for r in range(B):
        for s in range(K):
            if valid[r, s]:
                h_next[r, cells[r, s]] = h_new[r, s]
    delta = np.where(valid[..., None], h_new - h_old, 0).astype(dtype)
    total = np.zeros((B, d), dtype=dtype)
    for s in range(K):  # slot order (hsn_window.cu:892-895)
        total = total + delta[:, s]
    q_next = (q + total / dtype.type(N)).astype(dtype)
    written = np.zeros((B, N), dtype=bool)
    for r in range(B):
        written[r, cells[r][valid[r]]] = True
    age_next = np.where(written, 0, age + 1).astype(np.int64)
    h_sel = h_next[rows, safe]
    with np.errstate(invalid="ignore"):
        h_max = np.abs(h_next).reshape(B, -1).max(axis=1)
    return h_next, q_next, age_next, pos + 1, h_sel, h_max, c, b


# --------------------------------------------------------------------------------------------------
# The window's weights
# --------------------------------------------------------------------------------------------------


@dataclass
class WindowWeights:
    """Every weight a window reads (torch layouts), as the golden fixtures store them:
    ``shared`` / ``predictor`` (``python/hsn/model/encoder.py:128-198``, two-layer MLPs), the linear
    scorer (``python/hsn/model/router.py:319-321``), the cell (``python/hsn/model/cell.py:180-220``),
    the unit bank (``python/hsn/model/units.py``), the padded cell graph and the router's
    scalars."""

    s_w1: np.ndarray
    s_b1: np.ndarray
    s_w2: np.ndarray
    s_b2: np.ndarray
    p_w1: np.ndarray
    p_b1: np.ndarray
    p_w2: np.ndarray
    p_b2: np.ndarray
    score_w: np.ndarray
    score_b: np.ndarray
    v_w: np.ndarray
    wout_w: np.ndarray
    gate_w: np.ndarray
    gate_b: np.ndarray
    norm_w: np.ndarray
    cand_w: np.ndarray
    w1: np.ndarray
    b1: np.ndarray
    w2: np.ndarray
    b2: np.ndarray
    pad_src: np.ndarray
    edge_w: np.ndarray
    cost: np.ndarray
    age_max: int = 64
    lambda_cost: float = 0.0
    cell_overhead: float = 0.0
    shared_cost: float = 0.0
    limit: float = 1.00001
    norm_eps: float = 1e-6
    cand_eps: float = 1e-6
    k: int = 1
    probes: bool = True

    @staticmethod
    def from_npz(z, k: int, dtype=np.float32, prefix: str = "w_") -> "WindowWeights":
        names = (
            "s_w1 s_b1 s_w2 s_b2 p_w1 p_b1 p_w2 p_b2 score_w score_b v_w wout_w gate_w gate_b "
            "norm_w cand_w w1 b1 w2 b2 edge_w"
        ).split()
        fields = {n: np.asarray(z[prefix + n], dtype=dtype) for n in names}
        scal = z[prefix + "scalars_f"]
        return WindowWeights(
            **fields,
            pad_src=np.asarray(z[prefix + "pad_src"], dtype=np.int64),
            cost=np.asarray(z[prefix + "cost"], dtype=np.float32),
            age_max=int(scal[0]),
            lambda_cost=float(scal[1]),
            cell_overhead=float(scal[2]),
            shared_cost=float(scal[3]),
            limit=float(scal[4]),
            norm_eps=float(scal[5]),
            cand_eps=float(scal[6]),
            k=k,
        )

    @staticmethod
    def random(rng: np.random.Generator, *, N, d, K, H, M, D, S=9, dc=None, std=0.02,
               age_max=1 << 30, dtype=np.float32) -> "WindowWeights":  # fmt: skip
        """Seeded N(0, std) weights of the reference's shapes (biases zero, the gate's bias −3,
        gains one), a ring-like padded graph with softmax edge weights: the benchmark's synthetic
        model."""
        dc = d if dc is None else dc

        def w(*shape):
            return (rng.standard_normal(shape) * std).astype(dtype)

        src = np.stack([(np.arange(N) + 1 + e * 7) % N for e in range(D)], axis=1).astype(np.int64)
        logit = rng.standard_normal((N, D))
        edge = np.exp(logit) / np.exp(logit).sum(axis=1, keepdims=True)
        in_s = 2 * d + dc
        feat = 3 * d + 1 + S
        return WindowWeights(
            s_w1=w(H, in_s), s_b1=np.zeros(H, dtype), s_w2=w(d, H), s_b2=np.zeros(d, dtype),
            p_w1=w(H, d), p_b1=np.zeros(H, dtype), p_w2=w(d, H), p_b2=np.zeros(d, dtype),
            score_w=w(M, feat), score_b=np.zeros(M, dtype),
            v_w=w(d, d), wout_w=w(d, d), gate_w=w(d, 4 * d), gate_b=np.full(d, -3.0, dtype),
            norm_w=np.ones(4 * d, dtype), cand_w=np.ones(d, dtype),
            w1=w(M, 4 * d, H), b1=np.zeros((M, H), dtype), w2=w(M, H, d), b2=np.zeros((M, d), dtype),
            pad_src=src, edge_w=edge.astype(dtype), cost=np.full(M, 1.0 / (8 * N), np.float32),
            age_max=age_max, limit=1.00001, k=K,
        )  # fmt: skip


# --------------------------------------------------------------------------------------------------
# One position, and the forward sweep
# --------------------------------------------------------------------------------------------------


def _lin(x, w, b=None, bf16=False):
    """``F.linear``; with ``bf16`` the operands are rounded to bfloat16, the sum is taken in
    float32 and the result is rounded to bfloat16 (a matmul under bf16 autocast)."""
    if bf16:
        out = bf16_round(x).astype(np.float32) @ bf16_round(w).astype(np.float32).T
        if b is not None:
            out = out + bf16_round(b)
        return bf16_round(out)
    out = x @ w.T
    return out if b is None else out + b


def position(W: WindowWeights, h, q, age, z_t, ctx_t, scalars_t, *, bf16: bool = False,
             forced=None):  # fmt: skip
    """One position of the forward sweep for every row: ``HSN._position``
    (``python/hsn/model/hsn.py:1903-1980``) with the capturable sparse round
    ``PDGCell.step_sparse(static=True)`` (``python/hsn/model/cell.py:349-505``), i.e. the body of
    ``_tape_block``'s loop (``python/hsn/train/compile.py:1311-1344``) after the reset.

    Returns a dict with the decision, the round's intermediate values (what the replay records for
    the state-gradient sweep, ``cell.py:722-733``) and the state after the position.
    ``bf16=True`` rounds the matrix products as the folded sweep under bf16 autocast does
    (``compile.py:1117-1193``): operands and outputs of every product are bfloat16, sums float32,
    state and norms float32. ``forced = (cells, units, valid)`` replays a recorded decision."""
    dtype = h.dtype
    B, N, d = h.shape
    K = W.k
    M = W.cost.shape[0]
    rows = np.arange(B)[:, None]
    # the shared path: P reads q, S reads [z; q; ctx]  (hsn.py:1941-1945)
    x = np.concatenate([z_t, q, ctx_t], axis=-1)
    act = (lambda v: bf16_round(gelu(v))) if bf16 else gelu
    u = _lin(act(_lin(x, W.s_w1, W.s_b1, bf16)), W.s_w2, W.s_b2, bf16)
    z_hat = _lin(act(_lin(q, W.p_w1, W.p_b1, bf16)), W.p_w2, W.p_b2, bf16)
    u = u.astype(dtype)
    eps = (z_t - z_hat).astype(dtype)
    # the scorer: [u; eps; h_i; age_i / age_max; scalars_i] -> M logits  (router.py:767-796)
    feats = np.concatenate(
        [
            np.broadcast_to(u[:, None, :], (B, N, d)),
            np.broadcast_to(eps[:, None, :], (B, N, d)),
            h,
            (age.astype(dtype) / dtype.type(W.age_max))[:, :, None],
            scalars_t,
        ],
        axis=-1,
    )
    logits = _lin(feats, W.score_w, W.score_b, bf16).astype(np.float32)
    theta = refreshed = None
    if forced is None:
        cells, units, valid, theta, refreshed = select(
            logits, age, W.cost, k=K, age_max=W.age_max, probes=W.probes,
            lambda_cost=W.lambda_cost, cell_overhead=W.cell_overhead,
            shared_cost=W.shared_cost, limit=W.limit,
        )  # fmt: skip
    else:
        cells, units, valid = forced
    safe = np.where(valid, cells, 0)
    safe_units = np.where(valid, units, 0)
    # messages of the selected cells  (graph.py:294-333)
    vh = _lin(h, W.v_w, None, bf16)
    src = W.pad_src[safe]  # [B, K, D]
    sources = vh[rows[:, :, None], src]  # [B, K, D, d]
    edge = W.edge_w[safe]
    if bf16:
        m = bf16_round((sources * bf16_round(edge)[..., None]).sum(axis=2))
    else:
        m = (sources * edge[..., None]).sum(axis=2)
    h_old = h[rows, safe]
    v_raw = np.concatenate(
        [np.broadcast_to(u[:, None], (B, K, d)), np.broadcast_to(eps[:, None], (B, K, d)),
         h_old, m.astype(dtype)], axis=-1,
    )  # fmt: skip  (native.py:113-157)
    rms = 1.0 / np.sqrt((v_raw * v_raw).mean(axis=-1) + dtype.type(W.norm_eps))
    v = v_raw * rms[..., None] * W.norm_w
    # the executed unit's two layers, the gate, W_out  (units.py:530-572, cell.py:644-652)
    hidden = np.empty((B, K, W.w1.shape[2]), dtype=dtype)
    f_out = np.empty((B, K, d), dtype=dtype)
    for j in range(M):
        pick = safe_units == j
        if not pick.any():
            continue
        vj = v[pick]
        if bf16:
            hid = bf16_round(bf16_round(vj) @ bf16_round(W.w1[j]) + bf16_round(W.b1[j]))
            out = bf16_round(bf16_round(gelu(hid)) @ bf16_round(W.w2[j]) + bf16_round(W.b2[j]))
        else:
            hid = vj @ W.w1[j] + W.b1[j]
            out = gelu(hid) @ W.w2[j] + W.b2[j]
        hidden[pick] = hid
        f_out[pick] = out
    gate_pre = _lin(v, W.gate_w, W.gate_b, bf16).astype(dtype)
    y = _lin(f_out, W.wout_w, None, bf16).astype(dtype)
    pos = np.zeros(B, dtype=np.int64)
    h2, q2, age2, _, h_sel, h_max, c, b = cell_update(
        y, gate_pre, h, q, age, pos, cells, valid, W.cand_w, cand_norm=True, cand_eps=W.cand_eps
    )
    return dict(
        cells=cells, units=units, valid=valid, theta=theta, refreshed=refreshed, logits=logits,
        u=u, eps=eps, z_hat=z_hat, m=m.astype(dtype), rms=rms, hidden=hidden, gate_pre=gate_pre,
        y=y, c=c, b=b, h_old=h_old, h=h2, q=q2, age=age2, h_sel=h_sel, h_max=h_max,
    )  # fmt: skip


def window_forward(W: WindowWeights, z, ctx, scalars, reset, h, q, age, pos, *, bf16=False,
                   forced=None):  # fmt: skip
    """The forward sweep of a split window: ``run_tape`` / ``_tape_block``
    (``python/hsn/train/compile.py:1773-1845``, ``:1296-1362``). Per position: the column's reset
    (``python/hsn/model/state.py:267-283``), the pre-round record, the position, the decision and
    the post-round record. Returns the reference's tape (``TAPE_KEYS``, ``compile.py:1218-1231``,
    with the final state) plus ``rec_*``: the round's values per slot as the replay records them.
    ``forced``: recorded ``(cells, units, valid)`` ``[B, T, K]`` to replay instead of deciding."""
    B, T = reset.shape
    dtype = h.dtype
    reset = reset.astype(bool)
    keys = ("tape_h tape_q tape_age tape_hsel tape_theta qs sel_cell_idx sel_unit_idx sel_valid "
            "sel_refreshed h_max rec_c rec_b rec_h_old rec_y rec_gate_pre rec_m rec_rms rec_hidden "
            "logits us").split()  # fmt: skip
    out: dict[str, list] = {k: [] for k in keys}
    pos = pos.copy()
    for t in range(T):
        r = reset[:, t]
        h = np.where(r[:, None, None], 0, h).astype(dtype)
        q = np.where(r[:, None], 0, q).astype(dtype)
        age = np.where(r[:, None], 0, age)
        pos = np.where(r, 0, pos)
        out["tape_h"].append(h)
        out["tape_q"].append(q)
        out["tape_age"].append(age)
        f = None if forced is None else tuple(a[:, t] for a in forced)
        p = position(W, h, q, age, z[:, t], ctx[:, t], scalars[:, t], bf16=bf16, forced=f)
        h, q, age = p["h"], p["q"], p["age"]
        pos = pos + 1
        out["tape_hsel"].append(p["h_sel"])
        out["tape_theta"].append(p["theta"] if p["theta"] is not None else np.zeros(B, np.float32))
        out["qs"].append(q)
        out["sel_cell_idx"].append(p["cells"])
        out["sel_unit_idx"].append(p["units"])
        out["sel_valid"].append(p["valid"])
        out["sel_refreshed"].append(
            p["refreshed"] if p["refreshed"] is not None else np.zeros_like(p["valid"])
        )
        out["h_max"].append(p["h_max"])
        for name in ("c", "b", "h_old", "y", "gate_pre", "m", "rms", "hidden"):
            out["rec_" + name].append(p[name])
        out["logits"].append(p["logits"])
        out["us"].append(p["u"])
    tape = {k: np.stack(v, axis=1) for k, v in out.items()}
    tape.update(h=h, q=q, age=age, pos=pos)
    tape["refreshed"] = tape["sel_refreshed"].astype(np.float32).sum(axis=2).mean(axis=0)
    with np.errstate(invalid="ignore"):
        tape["state_abs_max"] = tape["h_max"].max(axis=0)
    return tape


def stream_step(W: WindowWeights, z_t, ctx_t, scalars_t, reset_t, h, q, age, pos, *, bf16=False):
    """One position of the serving step on a resident state: ``ServingStep`` / ``HSN._step_impl``
    in evaluation mode (``python/hsn/train/compile.py:1913-2006``, ``python/hsn/model/hsn.py:920``):
    the hard top-K decision with the probes on, the state updated and returned."""
    r = reset_t.astype(bool)
    h = np.where(r[:, None, None], 0, h).astype(h.dtype)
    q = np.where(r[:, None], 0, q).astype(q.dtype)
    age = np.where(r[:, None], 0, age)
    pos = np.where(r, 0, pos)
    p = position(W, h, q, age, z_t, ctx_t, scalars_t, bf16=bf16)
    p["pos"] = pos + 1
    return p


# --------------------------------------------------------------------------------------------------
# The backward recurrences
# --------------------------------------------------------------------------------------------------


def recurrence_backward(c, b, h_old, cells, valid, reset, n_cells, d_q_pre, d_q_post, d_h_sel,
                        initial=None, final=None):  # fmt: skip
    """The full-cut backward state recurrence (``python/hsn/train/split.py:128-174``; the kernel
    ``hsn_win_recurrence``, ``kernels/cuda/hsn_window.cu:59-115``). ``final``: a dict that receives
    the cotangent ``(A, R)`` of the state the window started from."""
    B, T, K, d = c.shape
    N = int(n_cells)
    dtype = c.dtype
    A = np.zeros((B, N + 1, d), dtype=dtype)  # row N: the padded slots' dummy cell
    R = np.zeros((B, d), dtype=dtype)
    if initial is not None:
        A[:, :N] = initial[0]
        R = initial[1].astype(dtype).copy()
    dc = np.zeros_like(c)
    db = np.zeros_like(b)
    rows = np.arange(B)[:, None]
    valid = valid.astype(bool)
    reset = reset.astype(bool)
    for t in range(T - 1, -1, -1):
        ok = valid[:, t, :, None]
        index = np.where(valid[:, t], cells[:, t], N)
        if d_q_post is not None:
            R = R + d_q_post[:, t]
        if d_h_sel is not None:
            np.add.at(A, (np.broadcast_to(rows, index.shape), index), np.where(ok, d_h_sel[:, t], 0))
        carried = A[rows, index]
        share = (R / dtype.type(N))[:, None, :]
        g = carried + share
        b_t = b[:, t]
        dc[:, t] = np.where(ok, b_t * g, 0)
        db[:, t] = np.where(ok, (c[:, t] - h_old[:, t]) * g, 0)
        A[rows, index] = np.where(ok, (1 - b_t) * carried - b_t * share, 0)
        A[:, N] = 0
        if d_q_pre is not None:
            R = R + d_q_pre[:, t]
        if final is not None and t == 0:
            final["A"], final["R"] = A[:, :N].copy(), R.copy()
        row = reset[:, t]
        A = np.where(row[:, None, None], 0, A)
        R = np.where(row[:, None], 0, R)
    return dc, db


def dense_recurrence_backward(c, b, h_old, reset, n_cells, d_q_pre, d_q_post):
    """The recurrence of the rows that ran the dense round
    (``python/hsn/train/split.py:177-209``; ``hsn_win_recurrence_dense``,
    ``kernels/cuda/hsn_window.cu:124-163``)."""
    Bd, T, N, d = c.shape
    dtype = c.dtype
    A = np.zeros((Bd, N, d), dtype=dtype)
    R = np.zeros((Bd, d), dtype=dtype)
    dc = np.zeros_like(c)
    db = np.zeros_like(b)
    reset = reset.astype(bool)
    for t in range(T - 1, -1, -1):
        if d_q_post is not None:
            R = R + d_q_post[:, t]
        g = A + (R / dtype.type(N))[:, None, :]
        dc[:, t] = b[:, t] * g
        db[:, t] = (c[:, t] - h_old[:, t]) * g
        A = (1 - b[:, t]) * g
        R = np.zeros_like(R) if d_q_pre is None else d_q_pre[:, t].copy()
        row = reset[:, t]
        A = np.where(row[:, None, None], 0, A)
        R = np.where(row[:, None], 0, R)
    return dc, db


def cell_state_vjp(W: WindowWeights, dc, db, *, c, b, h_old, units, y, hidden, gate_pre, m, rms):
    """The vector-Jacobian product of the selected cells' candidate and gate with respect to the
    state they read: ``(dh, dvm)`` (``python/hsn/train/state_gradient.py:288-354``; hard slots:
    ``alpha = 1``; candidate norm and cell norm on)."""
    dtype = c.dtype
    d = c.shape[-1]
    n = W.norm_w.shape[0]
    M = W.w1.shape[0]
    dz = dc * (1.0 - c * c)
    scaled = W.cand_w * dz
    rho = 1.0 / np.sqrt((y * y).mean(axis=-1, keepdims=True) + dtype.type(W.cand_eps))
    dy = rho * scaled - rho**3 * y * (y * scaled).mean(axis=-1, keepdims=True)
    d_unit = dy @ W.wout_w
    hid = hidden.astype(dtype)
    d_gate = db * b * (1.0 - b)
    w1_state = W.w1[:, n - 2 * d :, :]  # [M, 2d, H]
    d_hid = np.zeros_like(hid)
    dv = np.zeros((*c.shape[:-1], 2 * d), dtype=dtype)
    for j in range(M):
        pick = units == j
        if not pick.any():
            continue
        d_act = d_unit[pick] @ W.w2[j].T
        dh_j = d_act * gelu_grad(hid[pick])
        d_hid[pick] = dh_j
        dv[pick] = dh_j @ w1_state[j].T
    dv = dv + d_gate @ W.gate_w[:, n - 2 * d :]
    sigma = (d_hid * (hid - W.b1[units])).sum(axis=-1)
    sigma = sigma + (d_gate * (gate_pre - W.gate_b)).sum(axis=-1)
    state = np.concatenate([h_old, m], axis=-1)
    r = rms.astype(dtype)[..., None]
    ds = r * (W.norm_w[n - 2 * d :] * dv) - (r * r / n) * state * sigma[..., None]
    return ds[..., :d], ds[..., d:] @ W.v_w


def state_gradient_backward(W: WindowWeights, c, b, h_old, cells, units, valid, reset, n_cells,
                            d_q_pre, d_q_post, d_h_sel, record, initial=None, trace=None):  # fmt: skip
    """The reverse sweep of the window with the state gradient
    (``python/hsn/train/state_gradient.py:357-485``; its kernels ``hsn_win_back_head/mid/tail``,
    ``kernels/cuda/hsn_window.cu:1014-1427``). ``record``: ``y``, ``hidden``, ``gate_pre``, ``m``,
    ``rms`` per slot. ``trace`` receives ``A [B, T, N, d]`` and ``R [B, T, d]``: the cotangent of the
    state every position reads (before the zeroing of the rows that reset); ``trace["A"][:, 0]`` is
    the cotangent of the window's start state, the ``initial`` of the window before."""
    B, T, K, d = c.shape
    N = int(n_cells)
    D = W.pad_src.shape[1]
    dtype = c.dtype
    A = np.zeros((B, N + 1, d), dtype=dtype)
    R = np.zeros((B, d), dtype=dtype)
    if initial is not None:
        A[:, :N] = initial[0]
        R = initial[1].astype(dtype).copy()
    dc = np.zeros_like(c)
    db = np.zeros_like(b)
    rows = np.arange(B)[:, None]
    valid = valid.astype(bool)
    reset = reset.astype(bool)
    steps_A, steps_R, steps_dh, steps_dvm = [], [], [], []
    for t in range(T - 1, -1, -1):
        ok = valid[:, t, :, None]
        safe = np.where(valid[:, t], cells[:, t], 0)
        index = np.where(valid[:, t], cells[:, t], N)
        if d_q_post is not None:
            R = R + d_q_post[:, t]
        if d_h_sel is not None:
            np.add.at(A, (np.broadcast_to(rows, index.shape), index), np.where(ok, d_h_sel[:, t], 0))
        carried = A[rows, index]
        share = (R / dtype.type(N))[:, None, :]
        g = carried + share
        b_t, c_t, h_t = b[:, t], c[:, t], h_old[:, t]
        dc_t = np.where(ok, b_t * g, 0).astype(dtype)
        db_t = np.where(ok, (c_t - h_t) * g, 0).astype(dtype)
        dc[:, t], db[:, t] = dc_t, db_t
        dh, dvm = cell_state_vjp(
            W, dc_t, db_t, c=c_t, b=b_t, h_old=h_t, units=np.where(valid[:, t], units[:, t], 0),
            y=record["y"][:, t], hidden=record["hidden"][:, t], gate_pre=record["gate_pre"][:, t],
            m=record["m"][:, t], rms=record["rms"][:, t],
        )  # fmt: skip
        dh = np.where(ok, dh, 0)
        dvm = np.where(ok, dvm, 0)
        A[rows, index] = np.where(ok, (1 - b_t) * carried - b_t * share + dh, 0)
        A[:, N] = 0
        source = W.pad_src[safe].reshape(B, K * D)
        weighted = (W.edge_w[safe][..., None] * dvm[:, :, None, :]).reshape(B, K * D, d)
        np.add.at(A, (np.broadcast_to(rows, source.shape), source), weighted)
        if d_q_pre is not None:
            R = R + d_q_pre[:, t]
        steps_A.append(A[:, :N].copy())
        steps_R.append(R.copy())
        steps_dh.append(dh)
        steps_dvm.append(dvm)
        row = reset[:, t]
        A = np.where(row[:, None, None], 0, A)
        R = np.where(row[:, None], 0, R)
    if trace is not None:
        trace["A"] = np.stack(steps_A[::-1], axis=1)
        trace["R"] = np.stack(steps_R[::-1], axis=1)
        trace["dh"] = np.stack(steps_dh[::-1], axis=1)
        trace["dvm"] = np.stack(steps_dvm[::-1], axis=1)
    return dc, db


def out_adjacency(pad_src: np.ndarray, pad_mask: np.ndarray):
    """The message graph by source (``python/hsn/train/state_sweep.py:89-109``): row ``n`` lists
    the edges out of cell ``n`` ordered by target cell, then by the target's slot. Returns
    ``(out_tgt [N, D_out] int64, −1 on padding; out_edge [N, D_out] int64: target * D + slot)``."""
    N, D = pad_src.shape
    target, slot = np.nonzero(pad_mask)
    source = pad_src[target, slot]
    order = np.argsort(source, kind="stable")
    source, target, flat = source[order], target[order], (target * D + slot)[order]
    counts = np.bincount(source, minlength=N)
    d_out = max(int(counts.max()) if counts.size else 0, 1)
    start = np.cumsum(counts) - counts
    position_ = np.arange(source.size) - start[source]
    out_tgt = np.full((N, d_out), -1, dtype=np.int64)
    out_edge = np.zeros((N, d_out), dtype=np.int64)
    out_tgt[source, position_] = target
    out_edge[source, position_] = flat
    return out_tgt, out_edge


# --------------------------------------------------------------------------------------------------
# The reverse sweep's glue steps between its two products (the by-name kernels' contract)
# --------------------------------------------------------------------------------------------------


def activation_grad(name: str, x: np.ndarray) -> np.ndarray:
    """``python/hsn/train/state_gradient.py:192-205``."""
    if name == "gelu":
        return gelu_grad(x)
    if name == "relu":
        return (x > 0).astype(x.dtype)
    if name == "silu":
        s = sigmoid(x)
        return (s * (1.0 + x * (1.0 - s))).astype(x.dtype)
    if name == "tanh":
        return (1.0 - np.tanh(x) ** 2).astype(x.dtype)
    raise ValueError(name)


@dataclass
class SweepSizes:
    """``SweepShape`` (``python/hsn/train/state_sweep.py:70-86``)."""

    B: int
    T: int
    K: int
    N: int
    d: int
    H: int
    M: int
    n_fast: int
    n_read: int
    in_dim: int
    d_out: int


def _operand(x: np.ndarray, half: bool) -> np.ndarray:
    return bf16_round(x) if half else x.astype(np.float32)


def _sweep_write_blocks(s: SweepSizes, buf: dict, operand: str, fast: str, values, t: int, width: int,
                        half: bool) -> None:
    """``ReverseSweep._write_blocks`` (``state_sweep.py:424-439``): a routed slot's values into its
    unit's block of its row of the operand, after the block position ``t + 1`` used is cleared; a
    fixed slot's into the fast operand ``[F, B, ·]``."""
    F, routed = s.n_fast, s.K - s.n_fast
    for b in range(s.B):
        for k in range(F, s.K):
            row = b * routed + (k - F)
            if t + 1 < s.T:
                before = int(buf["units"][b, t + 1, k])
                buf[operand][row, before * width:(before + 1) * width] = 0
        for k in range(F, s.K):
            row = b * routed + (k - F)
            now = int(buf["units"][b, t, k])
            buf[operand][row, now * width:(now + 1) * width] = _operand(values[b, k], half)
        for k in range(F):
            buf[fast][k, b, :width] = _operand(values[b, k], half)


def sweep_head(s: SweepSizes, buf: dict, t: int, *, cand_norm: bool, cand_eps: float, half: bool) -> None:
    """``ReverseSweep.head_reference`` (``state_sweep.py:441-477``) in place on ``buf`` (arrays by
    the sweep's buffer names; fp32 state, operands bf16-valued when ``half``)."""
    f32 = np.float32
    F, d = s.n_fast, s.d
    R = (buf["R"] + buf["d_q_post"][:, t]).astype(f32)
    buf["R"][...] = R
    d_unit = np.zeros((s.B, s.K, d), f32)
    d_gate = np.zeros((s.B, s.K, d), f32)
    for b in range(s.B):
        A = buf["A"][b]
        if s.n_read:
            A[: s.n_read] += buf["d_h_fast"][b, t, : s.n_read]
        share = (R[b] / f32(s.N)).astype(f32)
        for k in range(s.K):
            if not buf["valid"][b, t, k]:
                buf["dc"][b, t, k] = 0
                buf["db"][b, t, k] = 0
                continue
            n = int(buf["cells"][b, t, k])
            carried = (A[n] + buf["d_h_sel"][b, t, k]).astype(f32)
            g = carried + share
            gate, c = buf["b"][b, t, k], buf["c"][b, t, k]
            dc = (gate * g).astype(f32)
            db = ((c - buf["h_old"][b, t, k]) * g).astype(f32)
            buf["dc"][b, t, k], buf["db"][b, t, k] = dc, db
            A[n] = ((f32(1) - gate) * carried - gate * share).astype(f32)
            dz = (dc * (f32(1) - c * c)).astype(f32)
            if cand_norm:
                y = buf["y"][b, t, k]
                scaled = (buf["cand_gain"] * dz).astype(f32)
                rho = f32(1) / np.sqrt(np.mean(y * y, dtype=f32) + f32(cand_eps), dtype=f32)
                dz = (rho * scaled - rho * rho * rho * y * np.mean(y * scaled, dtype=f32)).astype(f32)
            d_unit[b, k] = dz
            d_gate[b, k] = db * gate * (f32(1) - gate)
    buf["sigma"][...] = (d_gate * (buf["gate_pre"][:, t] - buf["gate_bias"])).sum(axis=-1, dtype=f32)
    _sweep_write_blocks(s, buf, "op1", "op1_fast", d_unit, t, d, half)
    routed = s.K - F
    buf["op2"][:, s.M * s.H:] = _operand(d_gate[:, F:].reshape(s.B * routed, d), half)
    if F:
        buf["op2_fast"][:, :, s.H:] = _operand(d_gate[:, :F].transpose(1, 0, 2), half)


def _sweep_per_slot(s: SweepSizes, routed: np.ndarray, fast: np.ndarray) -> np.ndarray:
    """``ReverseSweep._per_slot`` (``state_sweep.py:479-485``)."""
    out = routed.reshape(s.B, s.K - s.n_fast, -1)
    if s.n_fast:
        out = np.concatenate([fast.transpose(1, 0, 2), out], axis=1)
    return out.astype(np.float32)


def sweep_middle(s: SweepSizes, buf: dict, t: int, *, activation: str, half: bool) -> None:
    """``ReverseSweep.middle_reference`` (``state_sweep.py:487-495``)."""
    f32 = np.float32
    ok = buf["valid"][:, t].astype(bool)[:, :, None]
    hidden = buf["hidden"][:, t].astype(f32)
    d_act = _sweep_per_slot(s, buf["act_r"], buf["act_f"])
    d_hid = np.where(ok, d_act * activation_grad(activation, hidden), f32(0)).astype(f32)
    units = buf["units"][:, t]
    buf["sigma"] += (d_hid * (hidden - buf["b1"][units])).sum(axis=-1, dtype=f32)
    _sweep_write_blocks(s, buf, "op2", "op2_fast", d_hid, t, s.H, half)


def sweep_tail(s: SweepSizes, buf: dict, t: int, *, cell_norm: bool) -> None:
    """``ReverseSweep.tail_reference`` (``state_sweep.py:497-533``, no row limit)."""
    f32 = np.float32
    d = s.d
    prod = _sweep_per_slot(s, buf["dv_r"], buf["dv_f"])
    for b in range(s.B):
        ds = np.zeros((s.K, 2 * d), f32)
        slot_of = np.full(s.N, -1, np.int64)
        for k in range(s.K):
            if not buf["valid"][b, t, k]:
                continue
            if cell_norm:
                r = buf["rms"][b, t, k]
                back = (r * r / f32(s.in_dim)) * buf["sigma"][b, k]
                state = np.concatenate([buf["h_old"][b, t, k], buf["mv"][b, t, k]])
                ds[k] = (r * prod[b, k] - back * state).astype(f32)
            else:
                ds[k] = prod[b, k]
            slot_of[int(buf["cells"][b, t, k])] = k
        A = buf["A"][b]
        for k in range(s.K):
            if buf["valid"][b, t, k]:
                A[int(buf["cells"][b, t, k])] += ds[k, :d]
        for j in range(s.d_out):
            for n in range(s.N):
                target = int(buf["out_tgt"][n, j])
                if target >= 0 and slot_of[target] >= 0:
                    A[n] += buf["out_w"][n, j] * ds[slot_of[target], d:]
        buf["R"][b] += buf["d_q_pre"][b, t]
        if buf["reset"][b, t]:
            A[...] = 0
            buf["R"][b] = 0


# --------------------------------------------------------------------------------------------------
# The window's prologue: what the sweep reads per position, from the token and context ids
# --------------------------------------------------------------------------------------------------

def window_decode(P: dict, qs, us, *, bf16: bool = False):
    """The window's epilogue without its diagnostics: ``HSN._decode`` in evaluation mode, no selected
    readout (``python/hsn/model/hsn.py:2374-2390``): ``D([q_t; u_t])`` with ``D`` the two-layer ``MLP2``
    ``2d -> H -> V`` (``python/hsn/model/encoder.py:74-126``, ``:175-182``). ``P``: ``dec_w1 [H, 2d]``,
    ``dec_b1``, ``dec_w2 [V, H]``, ``dec_b2``. With ``bf16`` each linear runs as under autocast."""
    x = np.concatenate([np.asarray(qs), np.asarray(us)], axis=-1)
    act = (lambda v: bf16_round(gelu(v))) if bf16 else gelu
    return _lin(act(_lin(x, P["dec_w1"], P["dec_b1"], bf16)), P["dec_w2"], P["dec_b2"], bf16)


BOS = 1  # the byte that stands for "no previous byte" (python/hsn/data/synthetic.py:117)


def window_positions(pos: np.ndarray, reset: np.ndarray) -> np.ndarray:
    """``_window_positions`` (``python/hsn/model/hsn.py:347-355``): the session position before each
    step, int64 ``[B, T]``: ``t - s`` after the row's last reset ``s <= t``, ``pos + t`` without one."""
    B, T = reset.shape
    steps = np.arange(T, dtype=np.int64)
    last = np.maximum.accumulate(np.where(reset.astype(bool), steps, -1), axis=1)
    return np.where(last >= 0, steps - last, pos[:, None] + steps)


def window_prologue(P: dict, tokens, ctx_ids, reset, pos0, prev_tokens=None, *, bf16: bool = False):
    """The part of ``HSN._window_prologue`` (``python/hsn/model/hsn.py:1707-1860``) that the forward
    sweep reads, with ``model.key_address`` on, one address byte, no reader, no word addresses:

    * ``z = E(byte_emb(x))`` ``[B, T, d]`` (``:1741-1742``; ``MLP2``, ``python/hsn/model/encoder.py:74``),
    * ``context = ctx_emb(ctx)`` ``[B, T, dc]`` (``:1744``),
    * ``positions`` (``:1772``), the previous byte of each position, BOS at resets (``:1787-1789``),
    * ``scalars [B, T, N, 9]`` = ``Scorer.window_scalars`` (``python/hsn/model/router.py:597-640``):
      budget, round, context id / n_context, the two running averages, position / unroll, one
      (``_scalars``, ``:727-765``), then ``a_cur, a_prev = sqrt(d) <byte_codes[x], cell_addresses[n]>``
      for the current and the previous byte in float32 (``address_features``, ``:653-725``).

    ``P``: ``byte_emb [V, d]``, ``enc_w1 [H, d]``, ``enc_b1``, ``enc_w2 [d, H]``, ``enc_b2``, ``ctx_emb
    [n_context, dc]``, ``byte_codes [V, d]``, ``cell_addresses [N, d]``, ``ema_utility``, ``ema_selected``
    (``[N]`` or ``[B, N]``) and the numbers ``budget_frac, round_frac, n_context, unroll, position``
    (``model.scorer_position``: ``"document" | "clamp" | "wrap"``). ``bf16``: the encoder's two linears as under bf16 autocast.
    Returns ``dict(z, ctx, scalars, positions, previous)``."""
    tokens = np.asarray(tokens)
    B, T = tokens.shape
    f32 = np.float32
    emb = P["byte_emb"][tokens]
    act = (lambda v: bf16_round(gelu(v))) if bf16 else gelu
    z = _lin(act(_lin(emb, P["enc_w1"], P["enc_b1"], bf16)), P["enc_w2"], P["enc_b2"], bf16)
    context = P["ctx_emb"][np.asarray(ctx_ids)]
    reset = np.asarray(reset).astype(bool)
    positions = window_positions(np.asarray(pos0, dtype=np.int64), reset)
    first = np.full(B, BOS, dtype=tokens.dtype) if prev_tokens is None else np.asarray(prev_tokens, dtype=tokens.dtype)
    previous = np.where(reset, BOS, np.concatenate([first[:, None], tokens[:, :-1]], axis=1))
    N, d = P["cell_addresses"].shape
    dtype = z.dtype if z.dtype == np.float64 else f32
    pos = positions
    if P["position"] == "clamp":
        pos = np.minimum(pos, int(P["unroll"]) - 1)
    elif P["position"] == "wrap":
        pos = np.remainder(pos, int(P["unroll"]))

    def per_cell(x):  # [N] or [B, N] -> [B, T, N]
        x = np.asarray(x, dtype=dtype)
        x = np.broadcast_to(x, (B, N)) if x.ndim == 1 else x
        return np.broadcast_to(x[:, None, :], (B, T, N))

    def per_step(x):  # [B, T] -> [B, T, N]
        return np.broadcast_to(np.asarray(x, dtype=dtype)[:, :, None], (B, T, N))

    ones = np.ones((B, T, N), dtype=dtype)
    parts = [
        ones * dtype(P["budget_frac"]), ones * dtype(P["round_frac"]),
        per_step(np.asarray(ctx_ids).astype(dtype) / dtype(P["n_context"])),
        per_cell(P["ema_utility"]), per_cell(P["ema_selected"]),
        per_step(pos.astype(dtype) / dtype(P["unroll"])), ones,
    ]  # fmt: skip
    addresses = P["cell_addresses"].astype(f32).T  # the two products run in float32, outside autocast
    root = f32(np.sqrt(f32(d)))
    for ids in (tokens, previous):
        parts.append(((P["byte_codes"].astype(f32)[ids] @ addresses) * root).astype(dtype))
    scalars = np.stack(parts, axis=-1)
    return dict(z=z, ctx=context, scalars=scalars, positions=positions, previous=previous)
