"""GPU parity of the whole-window entry points (forward sweep, reverse sweep, streaming step,
carried state) against the reference's fixtures and the oracle, through the C ABI."""

from __future__ import annotations

import numpy as np
import pytest
import torch
from conftest import load_golden, to_np

from oracle import window_oracle as O

pytestmark = pytest.mark.gpu

F32 = torch.float32


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def _model(z, K, prod="fp32"):
    from hsn_b200.window import WindowModel

    W = O.WindowWeights.from_npz(z, K, np.dtype(np.float32))
    return W, WindowModel.from_oracle_weights(W, device="cuda", prod=prod)


def _inputs(z):
    return (
        dev(z["z"], F32), dev(z["ctx"], F32), dev(z["scalars"], F32), dev(z["reset"].astype(bool)),
        (dev(z["h0"], F32), dev(z["q0"], F32), dev(z["age0"]), dev(z["pos0"])),
    )  # fmt: skip


WINDOWS = ["c1_f32", "c1_f64", "c1p_f64", "c1p_f32", "probes_f64", "budget_f64", "odd_f64", "cut_f64", "mid_f32"]


def _settled(tape_ref_logits: np.ndarray, cells: np.ndarray, valid: np.ndarray, margin: float) -> np.ndarray:
    """Rows x positions that are safe to compare when two sweeps' logits differ in the last place
    (the reference's protocol for discrete routing, its tests/kernels/test_p2_10c_window.py:380-440):
    a position is risky when the gap between the last selected and the first unselected cell
    score, or between the two best units of a selected cell, is within ``margin``."""
    B, T, N, M = tape_ref_logits.shape
    score = tape_ref_logits.max(axis=-1)
    order = np.sort(score, axis=-1)[..., ::-1]
    K = cells.shape[-1]
    gap = order[..., K - 1] - order[..., K] if N > K else np.full((B, T), np.inf)
    risky = gap <= margin
    if M > 1:
        two = np.sort(tape_ref_logits, axis=-1)[..., ::-1]
        unit_gap = two[..., 0] - two[..., 1]  # [B,T,N]
        picked = np.take_along_axis(unit_gap, cells, axis=-1)
        risky |= (np.where(valid, picked, np.inf) <= margin).any(axis=-1)
    return ~risky


@pytest.mark.parametrize("name", WINDOWS + ["chain_f64"])
def test_forward_sweep_reproduces_the_reference_tape(name: str) -> None:
    """fp32 products against the reference's CPU sweep: routing bit for bit, state and tape within
    1e-5 relative. (A fixture made in float64 is compared where its decision is not within 1e-4
    of a tie, the reference's own rule; none of these fixtures has such a position.)"""
    from hsn_b200.window import window_forward

    z = load_golden(name if name.startswith("chain") else f"window_{name}")
    K = z["tape_sel_cell_idx"].shape[-1]
    W, model = _model(z, K)
    zz, ctx, scalars, reset, state = _inputs(z)
    start = [t.clone() for t in state]
    out = window_forward(model, zz, ctx, scalars, reset, state, want_logits=True)
    for a, b in zip(state, start):
        assert torch.equal(a, b)  # the carried state is the caller's: not modified
    ok = _settled(out["logits"].cpu().numpy(), z["tape_sel_cell_idx"], z["tape_sel_valid"].astype(bool), 1e-4)
    good = np.logical_and.accumulate(ok, axis=1)  # a row counts up to its first near tie
    assert good.mean() > 0.6, "fixture has too many near ties: regenerate it with another seed"
    assert np.array_equal(out["sel_valid"].cpu().numpy()[good], z["tape_sel_valid"].astype(bool)[good])
    assert np.array_equal(out["sel_cell_idx"].cpu().numpy()[good], z["tape_sel_cell_idx"][good])
    assert np.array_equal(out["sel_unit_idx"].cpu().numpy()[good], z["tape_sel_unit_idx"][good])
    assert np.array_equal(out["tape_age"].cpu().numpy()[good], z["tape_tape_age"][good])
    whole = good.all(axis=1)  # rows without a near tie: their final state too
    assert np.array_equal(out["age"].cpu().numpy()[whole], z["tape_age"][whole])
    assert np.array_equal(out["pos"].cpu().numpy(), z["tape_pos"])
    tol = 1e-5
    for mine, ref in (
        ("tape_h", "tape_tape_h"), ("tape_q", "tape_tape_q"), ("tape_hsel", "tape_tape_hsel"),
        ("qs", "tape_qs"), ("tape_theta", "tape_tape_theta"),
    ):  # fmt: skip
        want = z[ref].astype(np.float64)
        scale = max(1.0, float(np.abs(want).max()))
        np.testing.assert_allclose(out[mine].cpu().numpy()[good], want[good], rtol=tol, atol=tol * scale, err_msg=mine)
    for mine, ref in (("h", "tape_h"), ("q", "tape_q")):
        np.testing.assert_allclose(out[mine].cpu().numpy()[whole], z[ref][whole], rtol=tol, atol=tol, err_msg=mine)
    if whole.all():
        for mine, ref in (("state_abs_max", "tape_state_abs_max"), ("refreshed", "tape_refreshed")):
            np.testing.assert_allclose(out[mine].cpu().numpy(), z[ref], rtol=tol, atol=tol, err_msg=mine)
    if "rec_y" in z.files:
        mask = z["tape_sel_valid"].astype(bool) & good[..., None]
        for key, ref in (("y", "rec_y"), ("gate_pre", "rec_gate_pre"), ("m", "rec_m"), ("rms", "rec_rms"),
                         ("hidden", "rec_hidden"), ("c", "bw_c"), ("b", "bw_b"), ("h_old", "bw_h_old")):  # fmt: skip
            want = z[ref].astype(np.float64)[mask]
            scale = max(1.0, float(np.abs(want).max()))
            np.testing.assert_allclose(out["rec_" + key].cpu().numpy()[mask], want, rtol=1e-4, atol=2e-5 * scale, err_msg=key)


@pytest.mark.parametrize("name", [w for w in WINDOWS if w != "cut_f64"] + ["chain_f64"])
def test_reverse_sweep_equals_the_reference(name: str) -> None:
    """The state-gradient sweep on the reference's own record: dc, db and the cotangent of the
    start state within 1e-5 relative of the float64 / float32 CPU sweep."""
    from hsn_b200.window import window_backward

    z = load_golden(name if name.startswith("chain") else f"window_{name}")
    K = z["bw_cells"].shape[-1]
    _, model = _model(z, K)
    record = {k: dev(z["rec_" + k], F32) for k in ("y", "hidden", "gate_pre", "m", "rms")}
    cot = lambda k: dev(z[k], F32) if k in z.files else None  # noqa: E731
    dc, db, (A, R) = window_backward(
        model, dev(z["bw_c"], F32), dev(z["bw_b"], F32), dev(z["bw_h_old"], F32), dev(z["bw_cells"]),
        dev(z["bw_units"]), dev(z["bw_valid"].astype(bool)), dev(z["reset"].astype(bool)),
        cot("bw_d_q_pre"), cot("bw_d_q_post"), cot("bw_d_h_sel"), record,
    )  # fmt: skip
    scale = max(1.0, float(np.abs(z["bw_dc"]).max()), float(np.abs(z["bw_A"]).max()))
    tol = 2e-5 * scale
    np.testing.assert_allclose(dc.cpu().numpy(), z["bw_dc"], rtol=1e-4, atol=tol)
    np.testing.assert_allclose(db.cpu().numpy(), z["bw_db"], rtol=1e-4, atol=tol)
    keep = ~z["reset"][:, 0].astype(bool)
    np.testing.assert_allclose(A.cpu().numpy(), z["bw_A"][:, 0] * keep[:, None, None], rtol=1e-4, atol=tol)
    np.testing.assert_allclose(R.cpu().numpy(), z["bw_R"][:, 0] * keep[:, None], rtol=1e-4, atol=tol)
    assert bool((dc[~dev(z["bw_valid"].astype(bool))] == 0).all())


def test_full_cut_window_equals_the_reference() -> None:
    from hsn_b200.window import window_backward

    z = load_golden("window_cut_f64")
    K = z["bw_cells"].shape[-1]
    _, model = _model(z, K)
    cot = lambda k: dev(z[k], F32) if k in z.files else None  # noqa: E731
    dc, db, _ = window_backward(
        model, dev(z["bw_c"], F32), dev(z["bw_b"], F32), dev(z["bw_h_old"], F32), dev(z["bw_cells"]), None,
        dev(z["bw_valid"].astype(bool)), dev(z["reset"].astype(bool)), cot("bw_d_q_pre"),
        cot("bw_d_q_post"), cot("bw_d_h_sel"), None, full_cut=True,
    )  # fmt: skip
    scale = max(1.0, float(np.abs(z["bw_dc"]).max()))
    np.testing.assert_allclose(dc.cpu().numpy(), z["bw_dc"], rtol=1e-4, atol=2e-5 * scale)
    np.testing.assert_allclose(db.cpu().numpy(), z["bw_db"], rtol=1e-4, atol=2e-5 * scale)


def test_chained_windows_equal_the_unsplit_window() -> None:
    """Split-window TBPTT with the state-gradient carry: two windows of T positions, the state
    handed forward and (A, R) handed back, against the reference's unsplit window of 2T."""
    from hsn_b200.window import window_backward, window_forward

    z = load_golden("chain_f64")
    K = z["bw_cells"].shape[-1]
    _, model = _model(z, K)
    zz, ctx, scalars, reset, state = _inputs(z)
    T2 = reset.shape[1]
    T = T2 // 2
    first = window_forward(model, zz[:, :T], ctx[:, :T], scalars[:, :T], reset[:, :T], state)
    carried = (first["h"].clone(), first["q"].clone(), first["age"].clone(), first["pos"].clone())
    second = window_forward(model, zz[:, T:], ctx[:, T:], scalars[:, T:], reset[:, T:], carried)
    joined = torch.cat([first["sel_cell_idx"], second["sel_cell_idx"]], dim=1)
    assert np.array_equal(joined.cpu().numpy(), z["tape_sel_cell_idx"])
    for key in ("tape_h", "tape_q", "qs", "tape_hsel"):
        got = torch.cat([first[key], second[key]], dim=1).cpu().numpy()
        np.testing.assert_allclose(got, z["tape_" + key], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(second["h"].cpu().numpy(), z["tape_h"], rtol=1e-5, atol=1e-5)
    assert np.array_equal(second["pos"].cpu().numpy(), z["tape_pos"])
    # backward on the sweeps' own record: the second window first, its (A, R) into the first
    carry = None
    halves = {}
    for lo, tape in ((T, second), (0, first)):
        s = slice(lo, lo + T)
        rec = {k: tape["rec_" + k] for k in ("y", "hidden", "gate_pre", "m", "rms")}
        cot = lambda k: dev(z[k][:, s], F32) if k in z.files else None  # noqa: E731, B023
        dc, db, carry = window_backward(
            model, tape["rec_c"], tape["rec_b"], tape["rec_h_old"],
            torch.where(tape["sel_valid"], tape["sel_cell_idx"], 0),
            torch.where(tape["sel_valid"], tape["sel_unit_idx"], 0), tape["sel_valid"], reset[:, s].contiguous(),
            cot("bw_d_q_pre"), cot("bw_d_q_post"), cot("bw_d_h_sel"), rec, initial=carry,
        )  # fmt: skip
        halves[lo] = (dc, db)
    dc = torch.cat([halves[0][0], halves[T][0]], dim=1).cpu().numpy()
    db = torch.cat([halves[0][1], halves[T][1]], dim=1).cpu().numpy()
    scale = max(1.0, float(np.abs(z["bw_dc"]).max()))
    np.testing.assert_allclose(dc, z["bw_dc"], rtol=1e-3, atol=5e-5 * scale)
    np.testing.assert_allclose(db, z["bw_db"], rtol=1e-3, atol=5e-5 * scale)
    keep = ~z["reset"][:, 0].astype(bool)
    np.testing.assert_allclose(carry[0].cpu().numpy(), z["bw_A"][:, 0] * keep[:, None, None], rtol=1e-3, atol=5e-5 * scale)


def _synthetic(rng, B, T, N, d, K, H, M, D, p_reset, age_max=1 << 30, S=9, score_scale=40.0):
    W = O.WindowWeights.random(rng, N=N, d=d, K=K, H=H, M=M, D=D, S=S, age_max=age_max)
    W.score_w = (W.score_w * score_scale).astype(np.float32)  # scores spread well beyond the tie margin
    z = rng.standard_normal((B, T, d)).astype(np.float32)
    ctx = (rng.standard_normal((B, T, d)) * 0.02).astype(np.float32)
    scalars = rng.random((B, T, N, S)).astype(np.float32)
    reset = rng.random((B, T)) < p_reset
    reset[:, 0] = True
    h = np.zeros((B, N, d), np.float32)
    q = np.zeros((B, d), np.float32)
    age = np.zeros((B, N), np.int64)
    pos = np.zeros(B, np.int64)
    return W, z, ctx, scalars, reset, (h, q, age, pos)


@pytest.mark.parametrize("prod", ["fp32", "bf16"])
def test_forward_sweep_equals_the_oracle_on_a_slice_of_the_reference_shape(prod: str) -> None:
    """N256 d64 K8 H512 M8 D4 (the benchmark's model) at B4 T12 with the probes on: teacher-forced
    values within tolerance (fp32 1e-5 relative; bf16 products 2e-2), and the free-running fp32
    decisions bit for bit wherever the oracle's decision is not within 1e-4 of a tie."""
    from hsn_b200.window import WindowModel, window_forward

    rng = np.random.default_rng(7)
    W, z, ctx, scalars, reset, state = _synthetic(rng, 4, 12, 256, 64, 8, 512, 8, 4, 0.1, age_max=4)
    bf = prod == "bf16"
    want = O.window_forward(W, z, ctx, scalars, reset, *state, bf16=bf)
    model = WindowModel.from_oracle_weights(W, device="cuda", prod=prod)
    args = (dev(z), dev(ctx), dev(scalars), dev(reset), tuple(dev(s) for s in state))
    forced = (dev(want["sel_cell_idx"]), dev(want["sel_unit_idx"]), dev(want["sel_valid"]))
    got = window_forward(model, *args, forced=forced, want_logits=True)
    tol = 2e-2 if bf else 1e-5
    for key in ("tape_h", "tape_q", "qs", "tape_hsel", "h", "q", "rec_c", "rec_b", "rec_y", "rec_gate_pre",
                "rec_m", "rec_rms", "rec_hidden", "logits"):  # fmt: skip
        w = want[key].astype(np.float64)
        scale = max(1e-3, float(np.abs(w).max()))
        np.testing.assert_allclose(to_np(got[key]), w, rtol=tol, atol=tol * scale, err_msg=key)
    assert np.array_equal(got["tape_age"].cpu().numpy(), want["tape_age"])
    if not bf:
        free = window_forward(model, *args)
        ok = _settled(want["logits"], want["sel_cell_idx"], want["sel_valid"], 1e-4)
        # a row is compared up to its first risky position
        good = np.logical_and.accumulate(ok, axis=1)
        assert good.mean() > 0.9
        assert np.array_equal(free["sel_cell_idx"].cpu().numpy()[good], want["sel_cell_idx"][good])
        assert np.array_equal(free["sel_unit_idx"].cpu().numpy()[good], want["sel_unit_idx"][good])
        assert np.array_equal(free["sel_refreshed"].cpu().numpy()[good], want["sel_refreshed"][good])
        assert int(free["sel_refreshed"].sum()) > 0


def test_reverse_sweep_equals_the_oracle_on_a_slice_of_the_reference_shape() -> None:
    from hsn_b200.window import WindowModel, window_backward, window_forward

    rng = np.random.default_rng(8)
    B, T, N, d, K = 3, 10, 256, 64, 8
    W, z, ctx, scalars, reset, state = _synthetic(rng, B, T, N, d, K, 512, 8, 4, 0.1)
    # weights away from the tiny init so that every path of the backward is live
    for key in ("w1", "w2", "gate_w", "v_w", "wout_w"):
        setattr(W, key, (getattr(W, key) * 6).astype(np.float32))
    model = WindowModel.from_oracle_weights(W, device="cuda")
    tape = window_forward(model, dev(z), dev(ctx), dev(scalars), dev(reset), tuple(dev(s) for s in state))
    pre, post = rng.standard_normal((B, T, d)).astype(np.float32), rng.standard_normal((B, T, d)).astype(np.float32)
    sel = rng.standard_normal((B, T, K, d)).astype(np.float32)
    A0, R0 = rng.standard_normal((B, N, d)).astype(np.float32), rng.standard_normal((B, d)).astype(np.float32)
    cpu = {k: v.cpu().numpy() for k, v in tape.items() if isinstance(v, torch.Tensor)}
    valid = cpu["sel_valid"]
    cells = np.where(valid, cpu["sel_cell_idx"], 0)
    units = np.where(valid, cpu["sel_unit_idx"], 0)
    rec = {k: cpu["rec_" + k].astype(np.float64) for k in ("y", "hidden", "gate_pre", "m", "rms")}
    W64 = O.WindowWeights(**{k: (v.astype(np.float64) if isinstance(v, np.ndarray) and v.dtype == np.float32 else v)
                             for k, v in W.__dict__.items()})  # fmt: skip
    trace: dict = {}
    want_dc, want_db = O.state_gradient_backward(
        W64, cpu["rec_c"].astype(np.float64), cpu["rec_b"].astype(np.float64), cpu["rec_h_old"].astype(np.float64),
        cells, units, valid, reset, N, pre.astype(np.float64), post.astype(np.float64), sel.astype(np.float64), rec,
        initial=(A0.astype(np.float64), R0.astype(np.float64)), trace=trace,
    )  # fmt: skip
    dc, db, (A, R) = window_backward(
        model, tape["rec_c"], tape["rec_b"], tape["rec_h_old"], dev(cells), dev(units), tape["sel_valid"],
        dev(reset), dev(pre), dev(post), dev(sel), {k: tape["rec_" + k] for k in rec}, initial=(dev(A0), dev(R0)),
    )  # fmt: skip
    scale = max(1.0, float(np.abs(want_dc).max()), float(np.abs(trace["A"]).max()))
    np.testing.assert_allclose(dc.cpu().numpy(), want_dc, rtol=1e-4, atol=1e-5 * scale)
    np.testing.assert_allclose(db.cpu().numpy(), want_db, rtol=1e-4, atol=1e-5 * scale)
    keep = ~reset[:, 0]
    np.testing.assert_allclose(A.cpu().numpy(), trace["A"][:, 0] * keep[:, None, None], rtol=1e-4, atol=1e-5 * scale)
    np.testing.assert_allclose(R.cpu().numpy(), trace["R"][:, 0] * keep[:, None], rtol=1e-4, atol=1e-5 * scale)


def test_stream_step_updates_a_resident_state_in_place() -> None:
    """The serving step (N1024 d64 K8 H512, the streaming configuration's model) for a few steps
    on a resident state against the oracle, resets included."""
    from hsn_b200.window import WindowModel, stream_step

    rng = np.random.default_rng(9)
    B, steps, N, d = 6, 5, 1024, 64
    W, z, ctx, scalars, reset, state = _synthetic(rng, B, steps, N, d, 8, 512, 8, 4, 0.2, age_max=64)
    reset[:, 0] = False
    h = (rng.standard_normal((B, N, d)) * 0.3).astype(np.float32)
    st = (h, h.mean(axis=1), rng.integers(0, 200, (B, N)), np.arange(B, dtype=np.int64))
    model = WindowModel.from_oracle_weights(W, device="cuda")
    gpu = tuple(dev(s) for s in st)
    cur = st
    alive = np.ones(B, dtype=bool)  # rows whose decisions were never within 1e-4 of a tie
    for t in range(steps):
        want = O.stream_step(W, z[:, t], ctx[:, t], scalars[:, t], reset[:, t], *cur)
        got = stream_step(model, dev(z[:, t]), dev(ctx[:, t]), dev(scalars[:, t]), dev(reset[:, t]), gpu)
        alive &= _settled(want["logits"][:, None], want["cells"][:, None], want["valid"][:, None], 1e-4)[:, 0]
        assert np.array_equal(got["sel_cell_idx"][:, 0].cpu().numpy()[alive], want["cells"][alive])
        assert np.array_equal(got["sel_unit_idx"][:, 0].cpu().numpy()[alive], want["units"][alive])
        np.testing.assert_allclose(gpu[0].cpu().numpy()[alive], want["h"][alive], rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(gpu[1].cpu().numpy()[alive], want["q"][alive], rtol=1e-5, atol=1e-5)
        assert np.array_equal(gpu[2].cpu().numpy()[alive], want["age"][alive])
        assert np.array_equal(gpu[3].cpu().numpy(), want["pos"])
        cur = (want["h"], want["q"], want["age"], want["pos"])
    assert alive.sum() >= B - 1


@pytest.mark.parametrize("prod", ["fp32", "bf16"])
def test_carried_stream_steps_equal_one_resident_window(prod: str) -> None:
    """Serving steps that carry the cells' derived values from step to step (no pass over the whole
    state after the first) against the same positions as one resident window of the batch-synchronous
    kernels: the same arithmetic, so to the bit, resets included; and against steps that recompute
    the derived values every time."""
    from hsn_b200.window import WindowModel, stream_step, window_forward

    rng = np.random.default_rng(31)
    B, steps, N, d, K = 7, 6, 1024, 64, 8
    W, z, ctx, scalars, reset, state = _synthetic(rng, B, steps, N, d, K, 512, 8, 4, 0.25, age_max=64)
    reset[:, 0] = rng.random(B) < 0.3
    h = (rng.standard_normal((B, N, d)) * 0.3).astype(np.float32)
    start = (h, h.mean(axis=1), rng.integers(0, 200, (B, N)), np.arange(B, dtype=np.int64))
    model = WindowModel.from_oracle_weights(W, device="cuda", prod=prod, row_clusters=False)
    args = tuple(dev(a) for a in (z, ctx, scalars, reset))
    whole = tuple(dev(s) for s in start)
    want = window_forward(model, *args, whole, record=False, tape_state=False)
    carried, fresh = tuple(dev(s) for s in start), tuple(dev(s) for s in start)
    out = None
    for t in range(steps):
        now = tuple(a[:, t].contiguous() for a in args)
        out = stream_step(model, *now, carried, out=out, carried=t > 0)
        assert int(out["status"]) == 0
        for key in ("sel_cell_idx", "sel_unit_idx", "sel_valid", "qs", "tape_hsel"):
            assert torch.equal(out[key][:, 0], want[key][:, t]), (t, key)
        other = stream_step(model, *now, fresh)
        assert torch.equal(other["sel_cell_idx"], out["sel_cell_idx"])
        torch.testing.assert_close(other["qs"], out["qs"], rtol=1e-5, atol=1e-6)
    for got, ref in zip(carried, whole):
        assert torch.equal(got, ref)
    torch.testing.assert_close(fresh[0], whole[0], rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        stream_step(model, *now, carried, carried=True)
    # chunks of three positions, the second continuing the first
    chunked = tuple(dev(s) for s in start)
    res = None
    for half in range(2):
        part = tuple(a[:, 3 * half : 3 * half + 3].contiguous() for a in args)
        res = window_forward(model, *part, chunked, record=False, tape_state=False, out=res, carried=half > 0)
        assert torch.equal(res["qs"], want["qs"][:, 3 * half : 3 * half + 3])
        assert torch.equal(res["sel_cell_idx"], want["sel_cell_idx"][:, 3 * half : 3 * half + 3])
    for got, ref in zip(chunked, whole):
        assert torch.equal(got, ref)


def test_full_size_window_properties() -> None:
    """The benchmark's configuration 2 (B32 T256 N256 d64 K8 H512, bf16 products) at full size:
    size-independent properties. Two runs are bitwise equal (fixed reduction orders, no atomics);
    replaying the recorded decision reproduces the tape bit for bit; valid slots name distinct
    cells; the summary is the running mean of the state; ages restart at written cells; the
    backward of a window split in two equals the backward of the whole bit for bit."""
    from hsn_b200.window import WindowModel, window_backward, window_forward

    rng = np.random.default_rng(2)
    B, T, N, d, K = 32, 256, 256, 64, 8
    W, z, ctx, scalars, reset, state = _synthetic(rng, B, T, N, d, K, 512, 8, 4, 1 / 1024)
    model = WindowModel.from_oracle_weights(W, device="cuda", prod="bf16")
    args = (dev(z), dev(ctx), dev(scalars), dev(reset), tuple(dev(s) for s in state))
    one = window_forward(model, *args)
    assert int(one["status"]) == 0  # no bounded wait of the staging ran out
    two = window_forward(model, *args)
    for key in ("tape_h", "qs", "sel_cell_idx", "sel_unit_idx", "tape_theta", "rec_c", "rec_hidden"):
        assert torch.equal(one[key], two[key]), key
    replay = window_forward(model, *args, forced=(one["sel_cell_idx"], one["sel_unit_idx"], one["sel_valid"]))
    for key in ("tape_h", "qs", "rec_c", "rec_b"):
        assert torch.equal(one[key], replay[key]), key
    cells = one["sel_cell_idx"]
    assert bool(one["sel_valid"].all())  # budget 1.0: every slot fits
    assert int((cells.sort(dim=-1).values.diff(dim=-1) == 0).sum()) == 0
    mean = one["tape_h"].double().mean(dim=2)
    assert float((one["tape_q"].double() - mean).abs().max()) < 1e-5
    written = torch.zeros((B, T, N), dtype=torch.bool, device="cuda").scatter_(2, cells, True)
    assert bool((one["_tape_age"][:, 1:][written] == 0).all())
    cot = [dev(rng.standard_normal(s).astype(np.float32)) for s in ((B, T, d), (B, T, d), (B, T, K, d))]
    rec = {k: one["rec_" + k] for k in ("y", "hidden", "gate_pre", "m", "rms")}
    base = (one["rec_c"], one["rec_b"], one["rec_h_old"], cells, one["sel_unit_idx"], one["sel_valid"], args[3])
    dc, db, (A, R) = window_backward(model, *base, *cot, rec)
    assert bool(torch.isfinite(dc).all()) and bool(torch.isfinite(A).all())
    half = T // 2
    carry = None
    parts = []
    for s in (slice(half, T), slice(0, half)):
        sub = tuple(t[:, s].contiguous() for t in base)
        dcs, dbs, carry = window_backward(model, *sub, *(c[:, s].contiguous() for c in cot),
                                          {k: v[:, s].contiguous() for k, v in rec.items()}, initial=carry)  # fmt: skip
        parts.append((dcs, dbs))
    assert torch.equal(torch.cat([parts[1][0], parts[0][0]], dim=1), dc)
    assert torch.equal(torch.cat([parts[1][1], parts[0][1]], dim=1), db)
    assert torch.equal(carry[0], A) and torch.equal(carry[1], R)


def test_entry_points_refuse_what_they_do_not_take() -> None:
    from hsn_b200 import _lib
    from hsn_b200.window import WindowModel, window_forward

    rng = np.random.default_rng(1)
    W, z, ctx, scalars, reset, state = _synthetic(rng, 2, 3, 16, 32, 2, 32, 2, 2, 0.1)
    model = WindowModel.from_oracle_weights(W, device="cuda")
    args = [dev(z), dev(ctx), dev(scalars), dev(reset), tuple(dev(s) for s in state)]
    with pytest.raises(ValueError):
        window_forward(model, args[0].double(), *args[1:])
    with pytest.raises(ValueError):
        window_forward(model, args[0][:, :2], *args[1:])
    with pytest.raises(ValueError):
        window_forward(model, *args, scratch=torch.empty(16, dtype=torch.uint8, device="cuda"))
    W.w1 = np.zeros((17, W.w1.shape[1], W.w1.shape[2]), np.float32)  # more units than the kernels take
    W.b1, W.w2, W.b2 = np.zeros((17, 32), np.float32), np.zeros((17, 32, 32), np.float32), np.zeros((17, 32), np.float32)
    W.score_w, W.score_b, W.cost = np.zeros((17, W.score_w.shape[1]), np.float32), np.zeros(17, np.float32), np.ones(17, np.float32)
    big = WindowModel.from_oracle_weights(W, device="cuda")
    with pytest.raises(_lib.WindowKernelError) as err:
        window_forward(big, *args)
    assert err.value.code == _lib.E_UNSUPPORTED


@pytest.mark.parametrize(
    "shape",
    [
        dict(N=512, d=64, K=8, H=512, M=8, D=4),     # the split-window chain's model
        dict(N=4096, d=128, K=16, H=1024, M=8, D=4),  # the scaled sparse-routing model
        dict(N=1024, d=64, K=8, H=512, M=8, D=4),    # the streaming model
    ],
)
def test_models_of_the_larger_configurations(shape) -> None:
    """The other benchmark configurations' models at a reduced batch (B2, T3): forward values with
    the oracle's decisions forced, free-running decisions where not within 1e-4 of a tie, and the
    reverse sweep against the float64 oracle, state tape on and off."""
    from hsn_b200.window import WindowModel, window_backward, window_forward

    rng = np.random.default_rng(shape["N"])
    B, T = 2, 3
    W, z, ctx, scalars, reset, state = _synthetic(rng, B, T, p_reset=0.2, age_max=64, **shape)
    for key in ("w1", "w2", "gate_w", "v_w", "wout_w"):
        setattr(W, key, (getattr(W, key) * 4).astype(np.float32))
    h0 = (rng.standard_normal(state[0].shape) * 0.3).astype(np.float32)
    reset[:, 0] = False
    state = (h0, h0.mean(axis=1), rng.integers(0, 200, state[2].shape), state[3])
    want = O.window_forward(W, z, ctx, scalars, reset, *state)
    model = WindowModel.from_oracle_weights(W, device="cuda")
    args = (dev(z), dev(ctx), dev(scalars), dev(reset))
    forced = (dev(want["sel_cell_idx"]), dev(want["sel_unit_idx"]), dev(want["sel_valid"]))
    got = window_forward(model, *args, tuple(dev(s) for s in state), forced=forced)
    assert int(got["status"]) == 0
    for key in ("tape_h", "tape_q", "qs", "tape_hsel", "h", "q", "rec_c", "rec_b", "rec_y", "rec_m", "rec_hidden"):
        w = want[key].astype(np.float64)
        scale = max(1e-3, float(np.abs(w).max()))
        np.testing.assert_allclose(got[key].cpu().numpy(), w, rtol=1e-5, atol=1e-5 * scale, err_msg=key)
    assert np.array_equal(got["tape_age"].cpu().numpy(), want["tape_age"])
    good = np.logical_and.accumulate(_settled(want["logits"], want["sel_cell_idx"], want["sel_valid"], 1e-4), axis=1)
    free = window_forward(model, *args, tuple(dev(s) for s in state))
    assert good.mean() > 0.6
    assert np.array_equal(free["sel_cell_idx"].cpu().numpy()[good], want["sel_cell_idx"][good])
    assert np.array_equal(free["sel_refreshed"].cpu().numpy()[good], want["sel_refreshed"][good])
    # the resident form: no state tape, the state updated in place
    resident = tuple(dev(s) for s in state)
    res = window_forward(model, *args, resident, forced=forced, tape_state=False)
    np.testing.assert_allclose(resident[0].cpu().numpy(), want["h"], rtol=1e-5, atol=1e-5)
    assert np.array_equal(resident[2].cpu().numpy(), want["age"])
    np.testing.assert_allclose(res["qs"].cpu().numpy(), want["qs"], rtol=1e-5, atol=1e-5)
    # the reverse sweep on the sweep's own record
    N, d, K = shape["N"], shape["d"], shape["K"]
    post = rng.standard_normal((B, T, d)).astype(np.float32)
    sel = rng.standard_normal((B, T, K, d)).astype(np.float32)
    cpu = {k: v.cpu().numpy() for k, v in got.items() if isinstance(v, torch.Tensor)}
    rec = {k: cpu["rec_" + k].astype(np.float64) for k in ("y", "hidden", "gate_pre", "m", "rms")}
    W64 = O.WindowWeights(**{k: (v.astype(np.float64) if isinstance(v, np.ndarray) and v.dtype == np.float32 else v)
                             for k, v in W.__dict__.items()})  # fmt: skip
    valid = cpu["sel_valid"]
    cells, units = np.where(valid, cpu["sel_cell_idx"], 0), np.where(valid, cpu["sel_unit_idx"], 0)
    trace: dict = {}
    want_dc, want_db = O.state_gradient_backward(
        W64, cpu["rec_c"].astype(np.float64), cpu["rec_b"].astype(np.float64), cpu["rec_h_old"].astype(np.float64),
        cells, units, valid, reset, N, None, post.astype(np.float64), sel.astype(np.float64), rec, trace=trace,
    )  # fmt: skip
    dc, db, (A, R) = window_backward(
        model, got["rec_c"], got["rec_b"], got["rec_h_old"], dev(cells), dev(units), got["sel_valid"], dev(reset),
        None, dev(post), dev(sel), {k: got["rec_" + k] for k in rec},
    )  # fmt: skip
    scale = max(1.0, float(np.abs(want_dc).max()), float(np.abs(trace["A"]).max()))
    np.testing.assert_allclose(dc.cpu().numpy(), want_dc, rtol=1e-4, atol=1e-5 * scale)
    np.testing.assert_allclose(db.cpu().numpy(), want_db, rtol=1e-4, atol=1e-5 * scale)
    keep = ~reset[:, 0]
    np.testing.assert_allclose(A.cpu().numpy(), trace["A"][:, 0] * keep[:, None, None], rtol=1e-4, atol=1e-5 * scale)


@pytest.mark.parametrize("dims", [dict(N=256, d=64, K=8, H=512, M=8, D=4), dict(N=16, d=12, K=2, H=20, M=3, D=2),
                                  dict(N=32, d=128, K=4, H=1024, M=8, D=4)])  # fmt: skip
@pytest.mark.parametrize("prod", ["bf16", "fp32"])
def test_front_projection_equals_a_plain_product(dims, prod: str) -> None:
    """The window-invariant projection ([z; ctx] W + b for every position): tensor-core tiles with
    bf16 products, CUDA cores with fp32 products, against torch on the same (rounded) operands;
    rows and columns that are not multiples of the tile, several tiles in both directions."""
    from hsn_b200.window import WindowModel, front_projection

    rng = np.random.default_rng(5)
    W = O.WindowWeights.random(rng, std=0.2, **dims)
    W.s_b1 = rng.standard_normal(W.s_b1.shape).astype(np.float32)
    model = WindowModel.from_oracle_weights(W, device="cuda", prod=prod)
    d = dims["d"]
    for rows in (1, 130, 1000):
        z = dev(rng.standard_normal((rows, d)).astype(np.float32))
        ctx = dev(rng.standard_normal((rows, d)).astype(np.float32))
        got = front_projection(model, z, ctx)
        x = torch.cat([z, ctx], dim=1)
        w = torch.cat([dev(W.s_w1[:, :d]), dev(W.s_w1[:, 2 * d :])], dim=1)
        b = dev(W.s_b1)
        if prod == "bf16":
            x, w, b = (t.to(torch.bfloat16).double() for t in (x, w, b))
        want = (x.double() @ w.double().t() + b.double()).float()
        scale = float(want.abs().max())
        assert float((got - want).abs().max()) <= 2e-5 * scale, (rows, prod)


def _both_ways(rng, B, T, N, d, K, H, M, D, mult, path="rows"):
    """The same bf16 model twice: the kernels under test (``path``: "rows" = the per-row cluster
    kernels where the shape fits them, "phases" = the batch-synchronous tensor-core kernels), and
    the CUDA-core phases with the same roundings; a forward record by the first and the reverse
    sweep's inputs."""
    from hsn_b200.window import WindowModel, window_forward

    W, z, ctx, scalars, reset, state = _synthetic(rng, B, T, N, d, K, H, M, D, 0.1)
    for key in ("w1", "w2", "gate_w", "v_w", "wout_w"):
        setattr(W, key, O.bf16_round(getattr(W, key) * mult))
    tc = WindowModel.from_oracle_weights(W, device="cuda", prod="bf16", row_clusters=path == "rows")
    cc = WindowModel.from_oracle_weights(W, device="cuda", prod="bf16", tensor_cores=False, row_clusters=False)
    args = (dev(z), dev(ctx), dev(scalars), dev(reset), tuple(dev(s) for s in state))
    tape = window_forward(tc, *args)
    cots = [dev(rng.standard_normal(s).astype(np.float32)) for s in ((B, T, d), (B, T, d), (B, T, K, d))]
    rec = {k: tape["rec_" + k] for k in ("y", "hidden", "gate_pre", "m", "rms")}
    base = (tape["rec_c"], tape["rec_b"], tape["rec_h_old"], tape["sel_cell_idx"], tape["sel_unit_idx"],
            tape["sel_valid"], dev(reset))  # fmt: skip
    return W, tc, cc, args, tape, base, cots, rec


@pytest.mark.parametrize("path", ["rows", "phases"])
@pytest.mark.parametrize(
    "B,T,N,d,K,H,M,D,mult",
    [
        (6, 9, 256, 64, 8, 512, 8, 4, 1.0),    # the benchmark's model
        (6, 9, 256, 64, 8, 512, 8, 4, 6.0),    # large weights: the recurrence amplifies any difference
        (40, 3, 64, 64, 8, 200, 2, 2, 1.0),    # 160 pairs a unit: several batches of 32 and pair tiles; H % 128 != 0
        (5, 4, 96, 32, 4, 128, 3, 2, 1.0),     # d 32: half a state tile; one block a row
        (3, 3, 64, 128, 4, 256, 4, 2, 1.0),    # d 128: two state tiles
        (3, 7, 64, 16, 5, 256, 5, 3, 1.0),     # d 16, two blocks a row, K not a multiple of the blocks
        (2, 5, 512, 64, 8, 1024, 8, 4, 1.0),   # eight blocks a row
        (3, 6, 512, 64, 8, 512, 8, 4, 1.0),    # 128 cells a block: the forward ring has two slots
        (160, 2, 64, 64, 8, 256, 3, 2, 1.0),   # 1280 pairs a position: 512-pair tiles, batches of 64 pairs
        (270, 2, 64, 32, 4, 128, 3, 2, 1.0),   # 270 rows: front tiles of 32 rows, the last one of 14
    ],
)
def test_tensor_core_kernels_equal_the_cuda_core_kernels_with_the_same_roundings(path, B, T, N, d, K, H, M, D, mult) -> None:
    """The per-row cluster kernels and the tcgen05 phase kernels (unit layers forward, transposed
    unit layers in the reverse sweep) against the CUDA-core phase kernels on the same bf16 operands:
    the products are exact in fp32 and only the order of the sums differs, so 5e-3 of the scale at
    the 99.9th percentile forward (teacher-forced; a bf16 rounding may flip on a last-bit difference)
    and 1e-3 for the reverse sweep over T positions."""
    from hsn_b200.window import window_backward, window_forward

    rng = np.random.default_rng(12)
    W, tc, cc, args, tape, base, cots, rec = _both_ways(rng, B, T, N, d, K, H, M, D, mult, path)
    forced = (tape["sel_cell_idx"], tape["sel_unit_idx"], tape["sel_valid"])
    other = window_forward(cc, *args, forced=forced)
    assert int(tape["status"]) == 0
    for key in ("rec_hidden", "rec_y", "rec_gate_pre", "rec_c", "rec_b", "tape_h", "tape_q", "h", "q", "tape_hsel",
                "qs", "h_max", "rec_m", "rec_h_old", "rec_rms"):  # fmt: skip
        g, w = tape[key], other[key]
        if key == "rec_hidden":   # only the slots that ran are recorded
            ok = tape["sel_valid"].unsqueeze(-1)
            g, w = g * ok, w * ok
        scale = max(1e-3, float(w.abs().max()))
        diff = (g - w).abs().flatten()
        assert float(diff.max()) <= 2e-2 * scale, (key, float(diff.max()), scale)
        assert float(torch.quantile(diff[: 1 << 24].float(), 0.999)) <= 5e-3 * scale, key
    assert torch.equal(tape["tape_age"], other["tape_age"]) and torch.equal(tape["pos"], other["pos"])
    got = window_backward(tc, *base, *cots, rec)
    want = window_backward(cc, *base, *cots, rec)
    for name, g, w in zip(("dc", "db", "A", "R"), (got[0], got[1], got[2][0], got[2][1]),
                          (want[0], want[1], want[2][0], want[2][1])):  # fmt: skip
        scale = max(1e-6, float(w.abs().max()))
        worst = float((g - w).abs().max())
        assert worst <= 1e-3 * scale, (name, worst, scale)
    again = window_backward(tc, *base, *cots, rec)
    assert torch.equal(again[0], got[0]) and torch.equal(again[2][0], got[2][0])  # run to run: bit for bit
    # a carried cotangent and a reset in the middle of the window
    A0 = dev(rng.standard_normal((B, N, d)).astype(np.float32))
    R0 = dev(rng.standard_normal((B, d)).astype(np.float32))
    g2 = window_backward(tc, *base, *cots, rec, initial=(A0.clone(), R0.clone()))
    w2 = window_backward(cc, *base, *cots, rec, initial=(A0.clone(), R0.clone()))
    for g, w in ((g2[0], w2[0]), (g2[2][0], w2[2][0]), (g2[2][1], w2[2][1])):
        assert float((g - w).abs().max()) <= 1e-3 * max(1e-6, float(w.abs().max()))


@pytest.mark.parametrize("N,H", [(1024, 512), (256, 512)])
def test_row_clusters_on_a_resident_state_equal_the_phases(N: int, H: int) -> None:
    """The serving form (no state tape, the state updated in place, no record) on the streaming
    model's shape by the per-row cluster kernel, two calls in a row on the same state, against the
    CUDA-core phases with the decisions forced: the state, the summaries and the ages."""
    from hsn_b200.window import WindowModel, window_forward

    rng = np.random.default_rng(N)
    B, T, d, K = 5, 4, 64, 8
    W, z, ctx, scalars, reset, state = _synthetic(rng, B, 2 * T, N, d, K, H, 8, 4, 0.1)
    for key in ("w1", "w2", "gate_w", "v_w", "wout_w"):
        setattr(W, key, O.bf16_round(getattr(W, key)))
    reset[:, 0] = False
    h0 = (rng.standard_normal(state[0].shape) * 0.3).astype(np.float32)
    start = (h0, h0.mean(axis=1), rng.integers(0, 50, state[2].shape), state[3])
    rows = WindowModel.from_oracle_weights(W, device="cuda", prod="bf16")
    phases = WindowModel.from_oracle_weights(W, device="cuda", prod="bf16", tensor_cores=False, row_clusters=False)
    mine, theirs = tuple(dev(s) for s in start), tuple(dev(s) for s in start)
    for half in range(2):
        cut = slice(half * T, (half + 1) * T)
        args = tuple(dev(np.ascontiguousarray(a[:, cut])) for a in (z, ctx, scalars, reset))
        got = window_forward(rows, *args, mine, record=False, tape_state=False)
        assert int(got["status"]) == 0
        forced = (got["sel_cell_idx"], got["sel_unit_idx"], got["sel_valid"])
        want = window_forward(phases, *args, theirs, record=False, tape_state=False, forced=forced)
        for name, g, w in (("h", mine[0], theirs[0]), ("q", mine[1], theirs[1]), ("qs", got["qs"], want["qs"]),
                           ("hsel", got["tape_hsel"], want["tape_hsel"])):  # fmt: skip
            scale = max(1e-3, float(w.abs().max()))
            diff = (g - w).abs().flatten()
            assert float(diff.max()) <= 2e-2 * scale, (half, name)
            assert float(torch.quantile(diff.float(), 0.999)) <= 5e-3 * scale, (half, name)
        assert torch.equal(mine[2], theirs[2]) and torch.equal(mine[3], theirs[3])
    # a continuation asked of a scratch that the row kernel used (it keeps no derived values there):
    # the library notices and recomputes them, so the result is the plain call's
    again = tuple(t.clone() for t in mine)
    plain = window_forward(rows, *args, mine, record=False, tape_state=False, forced=forced)
    cont = window_forward(rows, *args, again, record=False, tape_state=False, forced=forced, out=got, carried=True)
    for g, w in ((again[0], mine[0]), (again[1], mine[1]), (cont["qs"], plain["qs"])):
        scale = max(1e-3, float(w.abs().max()))
        assert float((g - w).abs().max()) <= 2e-2 * scale
    assert torch.equal(again[2], mine[2])


def test_reverse_sweep_with_bf16_products_stays_within_bf16_tolerance() -> None:
    """The reverse sweep with bf16 products (tensor cores) against the sweep with fp32 products on
    the same weights and record: 2e-2 of the scale."""
    from hsn_b200.window import WindowModel, window_backward

    rng = np.random.default_rng(13)
    W, tc, _, _, _, base, cots, rec = _both_ways(rng, 6, 9, 256, 64, 8, 512, 8, 4, 1.0)
    full = WindowModel.from_oracle_weights(W, device="cuda", prod="fp32")
    got = window_backward(tc, *base, *cots, rec)
    want = window_backward(full, *base, *cots, rec)
    for name, g, w in zip(("dc", "db", "A", "R"), (got[0], got[1], got[2][0], got[2][1]),
                          (want[0], want[1], want[2][0], want[2][1])):  # fmt: skip
        scale = float(w.abs().max())
        worst = float((g - w).abs().max())
        assert worst <= 2e-2 * scale, (name, worst, scale)
