"""Parity of the bf16 path that the benchmark times, through the C ABI: the per-row cluster kernels'
own routing against the oracle's select on the kernels' own logits (bit for bit), the kernels against
windows the reference itself ran under bf16 autocast, and the larger configurations' models in bf16
against the oracle."""

from __future__ import annotations

import numpy as np
import pytest
import torch
from conftest import dev, load_golden, synthetic_window, to_np

from oracle import window_oracle as O

pytestmark = pytest.mark.gpu

F32 = torch.float32


def _select_every_position(W, logits: np.ndarray, age: np.ndarray):
    """``O.select`` on recorded logits ``[B, T, N, M]`` and pre-round ages ``[B, T, N]``."""
    outs = [
        O.select(logits[:, t], age[:, t], W.cost, k=W.k, age_max=W.age_max, probes=W.probes,
                 lambda_cost=W.lambda_cost, cell_overhead=W.cell_overhead, shared_cost=W.shared_cost, limit=W.limit)
        for t in range(logits.shape[1])
    ]  # fmt: skip
    return tuple(np.stack([o[i] for o in outs], axis=1) for i in range(5))


def _assert_decisions_follow_the_logits(W, out) -> dict[str, int]:
    """The decision a sweep recorded equals the reference router's decision on the logits the same
    sweep recorded, at every row and position: cells, units, valid, refreshed bit for bit, theta
    exactly (the select boundary of the reference's tests/kernels/test_p2_10_window.py:316-379)."""
    logits = out["logits"].cpu().numpy()
    age = out["tape_age"].cpu().numpy()
    cells, units, valid, theta, refreshed = _select_every_position(W, logits, age)
    assert np.array_equal(out["sel_valid"].cpu().numpy(), valid)
    assert np.array_equal(out["sel_cell_idx"].cpu().numpy(), cells)
    assert np.array_equal(out["sel_unit_idx"].cpu().numpy(), units)
    assert np.array_equal(out["sel_refreshed"].cpu().numpy(), refreshed)
    assert np.array_equal(out["tape_theta"].cpu().numpy(), theta)
    score = logits.max(axis=-1)
    top = np.sort(score, axis=-1)[..., ::-1]
    K = cells.shape[-1]
    return dict(refreshed=int(refreshed.sum()), padded=int((~valid).sum()),
                ties_at_the_cut=int((top[..., K - 1] == top[..., K]).sum()))  # fmt: skip


BOUNDARY_CASES = {
    # the benchmark's model (N 256: every warp sorts its keys), the refresh probes firing
    "c2_probes": dict(B=32, T=64, N=256, d=64, K=8, H=512, M=8, D=4, p_reset=0.03, age_max=3),
    # a budget that pads two slots, probes on the slots that remain
    "c2_budget": dict(B=8, T=48, N=256, d=64, K=8, H=512, M=8, D=4, p_reset=0.05, age_max=2, overhead=0.16),
    # exact ties: every cell gets the same scalars and the scorer is small, so the bf16 scores collide
    "c2_ties": dict(B=8, T=48, N=256, d=64, K=8, H=512, M=8, D=4, p_reset=0.1, age_max=1 << 30, flat=True, score_scale=2.0),
    # more cells than threads (configuration 3: a thread per cell counts against all keys; 1024 cells of
    # width 32 still fit a cluster's shared memory, configuration 5's 1024 x 64 do not)
    "c3": dict(B=6, T=24, N=512, d=64, K=8, H=512, M=8, D=4, p_reset=0.05, age_max=64),
    "n1024": dict(B=4, T=16, N=1024, d=32, K=8, H=512, M=8, D=4, p_reset=0.05, age_max=8),
    # a cost term: the scores are float32 differences (64-bit keys)
    "cost_256": dict(B=6, T=24, N=256, d=64, K=8, H=512, M=8, D=4, p_reset=0.05, age_max=4, lambda_cost=0.5),
    "cost_512": dict(B=4, T=16, N=512, d=32, K=5, H=256, M=6, D=3, p_reset=0.05, age_max=4, lambda_cost=0.5),
}


@pytest.mark.parametrize("name", list(BOUNDARY_CASES))
def test_row_cluster_routing_is_the_routers_decision_on_its_own_logits(name: str) -> None:
    """The free-running per-row cluster kernel (bf16 products), which ranks cells with its own
    code, against the oracle's select fed the kernel's recorded logits and ages: identical
    everywhere, ties to the lowest cell index, budget prefix, threshold, probes."""
    from hsn_b200.window import WindowModel, window_forward

    case = dict(BOUNDARY_CASES[name])
    overhead, flat = case.pop("overhead", 0.0), case.pop("flat", False)
    lambda_cost = case.pop("lambda_cost", 0.0)
    rng = np.random.default_rng(sum(map(ord, name)))
    W, z, ctx, scalars, reset, state = synthetic_window(rng, **case)
    W.cell_overhead = overhead
    if lambda_cost:
        W.lambda_cost = lambda_cost
        W.cost = np.linspace(0.0, 3.0, W.cost.shape[0]).astype(np.float32)[::-1].copy()
        W.limit = 1e9
    if flat:
        scalars[:] = scalars[:, :, :1]
    model = WindowModel.from_oracle_weights(W, device="cuda", prod="bf16")
    out = window_forward(model, dev(z), dev(ctx), dev(scalars), dev(reset), tuple(dev(s) for s in state),
                         want_logits=True)  # fmt: skip
    assert out["path"] == "rows" and int(out["status"]) == 0
    seen = _assert_decisions_follow_the_logits(W, out)
    if "probes" in name or "budget" in name:
        assert seen["refreshed"] > 0
    if "budget" in name:
        assert seen["padded"] > 0
    if "ties" in name:
        assert seen["ties_at_the_cut"] > 0


@pytest.mark.parametrize("name,reverse_path", [("bf16_a", "rows"), ("bf16_b", "phases")])
def test_row_clusters_reproduce_the_reference_under_bf16_autocast(name: str, reverse_path: str) -> None:
    """The per-row cluster kernels against windows the reference ran on the CPU under bf16 autocast
    (its ``train.precision=bf16``). Values with the reference's decision replayed: 2e-2 of each
    array's scale. Decisions position by position from the reference's own pre-round states (one
    launch of B T one-position rows): equal, or different only among cells whose scores lie within
    one bfloat16 unit of the last selected score. The reverse sweep on the reference's record."""
    from hsn_b200.window import WindowModel, window_backward, window_forward

    z = load_golden(f"window_{name}")
    K = z["tape_sel_cell_idx"].shape[-1]
    W = O.WindowWeights.from_npz(z, K, np.dtype(np.float32))
    model = WindowModel.from_oracle_weights(W, device="cuda", prod="bf16")
    valid = z["tape_sel_valid"].astype(bool)
    args = (dev(z["z"], F32), dev(z["ctx"], F32), dev(z["scalars"], F32), dev(z["reset"].astype(bool)))
    state = (dev(z["h0"], F32), dev(z["q0"], F32), dev(z["age0"]), dev(z["pos0"]))
    forced = (dev(z["tape_sel_cell_idx"]), dev(z["tape_sel_unit_idx"]), dev(valid))
    got = window_forward(model, *args, state, forced=forced)
    assert got["path"] == "rows" and int(got["status"]) == 0
    tol = 2e-2
    for mine, ref in (("tape_h", "tape_tape_h"), ("tape_q", "tape_tape_q"), ("tape_hsel", "tape_tape_hsel"),
                      ("qs", "tape_qs"), ("h", "tape_h"), ("q", "tape_q")):  # fmt: skip
        scale = float(np.abs(z[ref]).max())
        np.testing.assert_allclose(got[mine].cpu().numpy(), z[ref], rtol=tol, atol=tol * scale, err_msg=mine)
    assert np.array_equal(got["tape_age"].cpu().numpy(), z["tape_tape_age"])
    for key, ref in (("y", "rec_y"), ("gate_pre", "rec_gate_pre"), ("m", "rec_m"), ("rms", "rec_rms"),
                     ("hidden", "rec_hidden"), ("c", "bw_c"), ("b", "bw_b"), ("h_old", "bw_h_old")):  # fmt: skip
        want = z[ref][valid]
        scale = float(np.abs(want).max())
        np.testing.assert_allclose(to_np(got["rec_" + key])[valid], want, rtol=tol, atol=tol * scale, err_msg=key)
    # every position on its own: B T rows of one position, each from the reference's pre-round state
    B, T = valid.shape[:2]
    flat = lambda a: np.ascontiguousarray(a.reshape((B * T, 1) + a.shape[2:]))  # noqa: E731
    one = window_forward(
        model, dev(flat(z["z"]), F32), dev(flat(z["ctx"]), F32), dev(flat(z["scalars"]), F32),
        dev(np.zeros((B * T, 1), dtype=bool)),
        (dev(z["tape_tape_h"].reshape((B * T,) + z["h0"].shape[1:]), F32), dev(z["tape_tape_q"].reshape(B * T, -1), F32),
         dev(z["tape_tape_age"].reshape(B * T, -1)), dev(np.zeros(B * T, np.int64))),
        want_logits=True, record=False,
    )  # fmt: skip
    assert one["path"] == "rows"
    score = one["logits"][:, 0].cpu().numpy().max(axis=-1).reshape(B, T, -1)
    cells = one["sel_cell_idx"][:, 0].cpu().numpy().reshape(B, T, K)
    units = one["sel_unit_idx"][:, 0].cpu().numpy().reshape(B, T, K)
    assert np.array_equal(one["sel_valid"][:, 0].cpu().numpy().reshape(B, T, K), valid)
    same = (cells == z["tape_sel_cell_idx"]).all(axis=-1) & (units == z["tape_sel_unit_idx"]).all(axis=-1)
    for b, t in zip(*np.nonzero(~same)):
        mine, theirs = set(cells[b, t][valid[b, t]].tolist()), set(z["tape_sel_cell_idx"][b, t][valid[b, t]].tolist())
        moved = sorted(mine ^ theirs) or sorted(mine)
        last = np.sort(score[b, t])[::-1][K - 1]
        assert np.abs(score[b, t][moved] - last).max() <= abs(last) * 2.0**-7, (b, t, moved)
    assert same.mean() >= 0.9
    # the reverse sweep by the per-row cluster kernel on the reference's own record
    record = {k: dev(z["rec_" + k], F32) for k in ("y", "hidden", "gate_pre", "m", "rms")}
    cot = lambda k: dev(z[k], F32) if k in z.files else None  # noqa: E731
    info: dict = {}
    dc, db, (A, R) = window_backward(
        model, dev(z["bw_c"], F32), dev(z["bw_b"], F32), dev(z["bw_h_old"], F32), dev(z["bw_cells"]),
        dev(z["bw_units"]), dev(z["bw_valid"].astype(bool)), args[3],
        cot("bw_d_q_pre"), cot("bw_d_q_post"), cot("bw_d_h_sel"), record, info=info,
    )  # fmt: skip
    assert info["path"] == reverse_path and int(info["status"]) == 0
    scale = max(float(np.abs(z["bw_dc"]).max()), float(np.abs(z["bw_A"]).max()))
    keep = ~z["reset"][:, 0].astype(bool)
    np.testing.assert_allclose(dc.cpu().numpy(), z["bw_dc"], rtol=tol, atol=tol * scale)
    np.testing.assert_allclose(db.cpu().numpy(), z["bw_db"], rtol=tol, atol=tol * scale)
    np.testing.assert_allclose(A.cpu().numpy(), z["bw_A"][:, 0] * keep[:, None, None], rtol=tol, atol=tol * scale)
    np.testing.assert_allclose(R.cpu().numpy(), z["bw_R"][:, 0] * keep[:, None], rtol=tol, atol=tol * scale)


LARGER = {
    # the model, the kernels that serve its forward sweep, those of its reverse sweep (whose resident
    # cotangent is a third of the forward's resident state and still fits at 1024 cells)
    "c3": (dict(N=512, d=64, K=8, H=512, M=8, D=4), "rows", "rows"),
    "c4": (dict(N=4096, d=128, K=16, H=1024, M=8, D=4), "phases", "phases"),
    "c5": (dict(N=1024, d=64, K=8, H=512, M=8, D=4), "phases", "rows"),
}


@pytest.mark.parametrize("name", list(LARGER))
def test_larger_configurations_in_bf16_equal_the_oracle(name: str) -> None:
    """Configurations 3, 4 and 5's models with bf16 products at a reduced batch (B2, T3), by the
    kernels the benchmark times for them (per-row clusters for 3; for 4 and 5, whose state does not
    fit a cluster's shared memory, the phases with the tensor-core unit kernels): values with the oracle's decisions
    forced within 2e-2 of the oracle's bf16 mode, the free-running routing equal to the router's
    decision on the kernels' own logits, the reverse sweep within 2e-2 of the float64 oracle."""
    from hsn_b200.window import WindowModel, window_backward, window_forward

    shape, path, reverse_path = LARGER[name]
    rng = np.random.default_rng(shape["N"] + 1)
    B, T = 2, 3
    W, z, ctx, scalars, reset, state = synthetic_window(rng, B, T, p_reset=0.2, age_max=64, **shape)
    for key in ("w1", "w2", "gate_w", "v_w", "wout_w"):
        setattr(W, key, (getattr(W, key) * 4).astype(np.float32))
    h0 = (rng.standard_normal(state[0].shape) * 0.3).astype(np.float32)
    reset[:, 0] = False
    state = (h0, h0.mean(axis=1), rng.integers(0, 200, state[2].shape), state[3])
    want = O.window_forward(W, z, ctx, scalars, reset, *state, bf16=True)
    model = WindowModel.from_oracle_weights(W, device="cuda", prod="bf16")
    args = (dev(z), dev(ctx), dev(scalars), dev(reset))
    forced = (dev(want["sel_cell_idx"]), dev(want["sel_unit_idx"]), dev(want["sel_valid"]))
    got = window_forward(model, *args, tuple(dev(s) for s in state), forced=forced, want_logits=True)
    assert got["path"] == path and int(got["status"]) == 0
    tol = 2e-2
    for key in ("tape_h", "tape_q", "qs", "tape_hsel", "h", "q", "rec_c", "rec_b", "rec_y", "rec_gate_pre", "rec_m",
                "rec_rms", "rec_hidden", "logits"):  # fmt: skip
        w = want[key].astype(np.float64)
        scale = max(1e-3, float(np.abs(w).max()))
        np.testing.assert_allclose(to_np(got[key]), w, rtol=tol, atol=tol * scale, err_msg=key)
    assert np.array_equal(got["tape_age"].cpu().numpy(), want["tape_age"])
    free = window_forward(model, *args, tuple(dev(s) for s in state), want_logits=True)
    assert free["path"] == path
    _assert_decisions_follow_the_logits(W, free)
    # the reverse sweep on the forced sweep's own record, bf16 products, against the float64 oracle
    N, d, K = shape["N"], shape["d"], shape["K"]
    post = rng.standard_normal((B, T, d)).astype(np.float32)
    sel = rng.standard_normal((B, T, K, d)).astype(np.float32)
    cpu = {k: to_np(v) for k, v in got.items() if isinstance(v, torch.Tensor)}
    rec = {k: cpu["rec_" + k].astype(np.float64) for k in ("y", "hidden", "gate_pre", "m", "rms")}
    W64 = O.WindowWeights(**{k: (O.bf16_round(v).astype(np.float64) if isinstance(v, np.ndarray) and v.dtype == np.float32 else v)
                             for k, v in W.__dict__.items()})  # fmt: skip
    valid = cpu["sel_valid"]
    cells, units = np.where(valid, cpu["sel_cell_idx"], 0), np.where(valid, cpu["sel_unit_idx"], 0)
    trace: dict = {}
    want_dc, want_db = O.state_gradient_backward(
        W64, cpu["rec_c"].astype(np.float64), cpu["rec_b"].astype(np.float64), cpu["rec_h_old"].astype(np.float64),
        cells, units, valid, reset, N, None, post.astype(np.float64), sel.astype(np.float64), rec, trace=trace,
    )  # fmt: skip
    info: dict = {}
    dc, db, (A, R) = window_backward(
        model, got["rec_c"], got["rec_b"], got["rec_h_old"], dev(cells), dev(units), got["sel_valid"], dev(reset),
        None, dev(post), dev(sel), {k: got["rec_" + k] for k in rec}, info=info,
    )  # fmt: skip
    assert info["path"] == reverse_path and int(info["status"]) == 0
    scale = max(1.0, float(np.abs(want_dc).max()), float(np.abs(trace["A"]).max()))
    keep = ~reset[:, 0]
    np.testing.assert_allclose(dc.cpu().numpy(), want_dc, rtol=tol, atol=tol * scale)
    np.testing.assert_allclose(db.cpu().numpy(), want_db, rtol=tol, atol=tol * scale)
    np.testing.assert_allclose(A.cpu().numpy(), trace["A"][:, 0] * keep[:, None, None], rtol=tol, atol=tol * scale)
    np.testing.assert_allclose(R.cpu().numpy(), trace["R"][:, 0] * keep[:, None], rtol=tol, atol=tol * scale)
