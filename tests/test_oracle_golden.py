"""The oracle against the fixtures the reference itself produced (tests/golden/make_golden.py)."""

from __future__ import annotations

import numpy as np
import pytest
from conftest import SWEEP_SETS, SWEEP_WRITTEN, load_golden, sweep_fixture

from oracle import window_oracle as O

SELECT_SETS = ["plain", "probes", "budget", "probes_budget", "cost", "reserved"]


@pytest.mark.parametrize("name", SELECT_SETS)
def test_select_takes_the_routers_decision(name: str) -> None:
    z = load_golden(f"select_{name}")
    p = z["params"]
    reserved = int(p[6]) if len(p) > 6 else 0
    fired = 0
    for i in range(int(z["n"])):
        pre = f"t{i}_"
        cells, units, valid, theta, refreshed = O.select(
            z[pre + "logits"], z[pre + "age"], z["cost"], k=int(p[0]), age_max=int(p[1]),
            probes=bool(z[pre + "probes"]), lambda_cost=float(p[2]), cell_overhead=float(p[3]),
            shared_cost=float(p[4]), limit=float(p[5]), reserved=reserved,
            reserved_units=bool(z[pre + "fixed_units"]) if reserved else False,
        )  # fmt: skip
        assert np.array_equal(valid, z[pre + "valid"].astype(bool))
        assert np.array_equal(cells, z[pre + "cells"])
        assert np.array_equal(units, z[pre + "units"])
        assert np.array_equal(refreshed, z[pre + "refreshed"].astype(bool))
        assert np.array_equal(theta, z[pre + "theta"])
        fired += int(refreshed.sum())
    if "probes" in name or name in ("cost", "reserved"):
        assert fired > 0


@pytest.mark.parametrize("name", ["rms", "none", "budget"])
def test_cell_update_equals_the_native_round(name: str) -> None:
    z = load_golden(f"update_{name}")
    padded = 0
    for i in range(int(z["n"])):
        s = f"s{i}_"
        valid = z[s + "valid"].astype(bool)
        h, q, age, pos, h_sel, h_max, _, _ = O.cell_update(
            z[s + "y"], z[s + "gate"], z[s + "h"], z[s + "q"], z[s + "age"], z[s + "pos"],
            z[s + "cells"], valid, z["cand_w"], cand_norm=bool(z["cand_norm"]),
            cand_eps=float(z["cand_eps"]),
        )  # fmt: skip
        assert np.abs(h - z[s + "h_next"]).max() <= 2e-6
        assert np.abs(q - z[s + "q_next"]).max() <= 2e-6
        assert np.array_equal(age, z[s + "age_next"]) and np.array_equal(pos, z[s + "pos_next"])
        assert np.array_equal(h_max, np.abs(h).reshape(h.shape[0], -1).max(axis=1))
        padded += int((~valid).sum())
    if name == "budget":
        assert padded > 0


@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_recurrence_equals_the_reference(name: str) -> None:
    z = load_golden(f"recurrence_{name}")
    N = int(z["N"])
    base = (z["c"], z["b"], z["h_old"], z["cells"], z["valid"], z["reset"], N)
    for tag in ("111", "010", "101"):
        cots = [z[k] if on == "1" else None for k, on in zip(("pre", "post", "sel"), tag)]
        dc, db = O.recurrence_backward(*base, *cots)
        np.testing.assert_allclose(dc, z[f"dc_{tag}"], rtol=1e-12, atol=1e-13)
        np.testing.assert_allclose(db, z[f"db_{tag}"], rtol=1e-12, atol=1e-13)
        assert (dc[~z["valid"].astype(bool)] == 0).all()
    dc, db = O.dense_recurrence_backward(
        z["dense_c"], z["dense_b"], z["dense_h"], z["reset"], N, z["pre"], z["post"]
    )
    np.testing.assert_allclose(dc, z["dense_dc"], rtol=1e-12, atol=1e-13)
    np.testing.assert_allclose(db, z["dense_db"], rtol=1e-12, atol=1e-13)


WINDOWS = ["c1_f32", "c1_f64", "c1p_f64", "c1p_f32", "probes_f64", "budget_f64", "odd_f64",
           "cut_f64", "mid_f32", ]  # fmt: skip


def _forward(z, dtype):
    K = z["tape_sel_cell_idx"].shape[-1]
    W = O.WindowWeights.from_npz(z, K, dtype)
    cast = lambda a: np.asarray(a, dtype=dtype)  # noqa: E731
    tape = O.window_forward(
        W, cast(z["z"]), cast(z["ctx"]), cast(z["scalars"]), z["reset"], cast(z["h0"]),
        cast(z["q0"]), z["age0"], z["pos0"],
    )  # fmt: skip
    return W, tape


@pytest.mark.parametrize("name", WINDOWS + ["chain_f64"])
def test_forward_sweep_reproduces_the_reference_tape(name: str) -> None:
    z = load_golden(name if name.startswith("chain") else f"window_{name}")
    f64 = z["h0"].dtype == np.float64
    dtype = np.float64 if f64 else np.float32
    _, tape = _forward(z, np.dtype(dtype))
    tol = 1e-9 if f64 else 2e-5
    # routing: bit-exact
    assert np.array_equal(tape["sel_valid"], z["tape_sel_valid"].astype(bool))
    assert np.array_equal(tape["sel_cell_idx"], z["tape_sel_cell_idx"])
    assert np.array_equal(tape["sel_unit_idx"], z["tape_sel_unit_idx"])
    assert np.array_equal(tape["tape_age"], z["tape_tape_age"])
    assert np.array_equal(tape["age"], z["tape_age"]) and np.array_equal(tape["pos"], z["tape_pos"])
    for mine, ref in (
        ("tape_h", "tape_tape_h"), ("tape_q", "tape_tape_q"), ("tape_hsel", "tape_tape_hsel"),
        ("qs", "tape_qs"), ("h", "tape_h"), ("q", "tape_q"), ("state_abs_max", "tape_state_abs_max"),
        ("refreshed", "tape_refreshed"),
    ):  # fmt: skip
        np.testing.assert_allclose(tape[mine], z[ref], rtol=tol, atol=tol, err_msg=mine)
    np.testing.assert_allclose(tape["tape_theta"], z["tape_tape_theta"], rtol=1e-5, atol=1e-6)
    if name.startswith("probes"):
        assert tape["sel_refreshed"].sum() > 0
    if name.startswith("budget"):
        assert (~tape["sel_valid"]).sum() > 0
    if "rec_y" in z.files:
        # the sweep's own values of the round against the replay's record (batched matmuls)
        for key in ("y", "gate_pre", "m", "rms", "hidden"):
            got, want = tape["rec_" + key], z["rec_" + key]
            mask = tape["sel_valid"]
            np.testing.assert_allclose(got[mask], want[mask], rtol=10 * tol, atol=10 * tol, err_msg=key)
        mask = tape["sel_valid"]
        np.testing.assert_allclose(tape["rec_c"][mask], z["bw_c"][mask], rtol=10 * tol, atol=10 * tol)
        np.testing.assert_allclose(tape["rec_b"][mask], z["bw_b"][mask], rtol=10 * tol, atol=10 * tol)


@pytest.mark.parametrize("name", [w for w in WINDOWS if w != "cut_f64"] + ["chain_f64"])
def test_state_gradient_sweep_equals_the_reference(name: str) -> None:
    z = load_golden(name if name.startswith("chain") else f"window_{name}")
    f64 = z["h0"].dtype == np.float64
    dtype = np.dtype(np.float64 if f64 else np.float32)
    K = z["bw_cells"].shape[-1]
    W = O.WindowWeights.from_npz(z, K, dtype)
    N = z["h0"].shape[1]
    record = {k: z["rec_" + k] for k in ("y", "hidden", "gate_pre", "m", "rms")}
    cot = lambda k: z[k] if k in z.files else None  # noqa: E731
    trace: dict = {}
    dc, db = O.state_gradient_backward(
        W, z["bw_c"], z["bw_b"], z["bw_h_old"], z["bw_cells"], z["bw_units"], z["bw_valid"],
        z["reset"], N, cot("bw_d_q_pre"), cot("bw_d_q_post"), cot("bw_d_h_sel"), record, trace=trace,
    )  # fmt: skip
    tol = 1e-10 if f64 else 2e-5
    scale = max(1.0, float(np.abs(z["bw_dc"]).max()))
    np.testing.assert_allclose(dc, z["bw_dc"], rtol=tol, atol=tol * scale)
    np.testing.assert_allclose(db, z["bw_db"], rtol=tol, atol=tol * scale)
    np.testing.assert_allclose(trace["A"], z["bw_A"], rtol=tol, atol=tol * scale)
    np.testing.assert_allclose(trace["R"], z["bw_R"], rtol=tol, atol=tol * scale)
    np.testing.assert_allclose(trace["dh"], z["bw_dh"], rtol=tol, atol=tol * scale)
    np.testing.assert_allclose(trace["dvm"], z["bw_dvm"], rtol=tol, atol=tol * scale)


@pytest.mark.parametrize("name", ["bf16_a", "bf16_b"])
def test_bf16_mode_reproduces_the_reference_under_autocast(name: str) -> None:
    """The oracle's ``bf16=True`` against the reference's CPU sweep under bf16 autocast (its
    ``train.precision=bf16``): the decisions of every position, then state, tape and the round's
    record within 2e-2 of each array's scale with the reference's decision replayed."""
    z = load_golden(f"window_{name}")
    K = z["tape_sel_cell_idx"].shape[-1]
    W = O.WindowWeights.from_npz(z, K, np.dtype(np.float32))
    args = (z["z"], z["ctx"], z["scalars"], z["reset"].astype(bool), z["h0"], z["q0"], z["age0"], z["pos0"])
    valid = z["tape_sel_valid"].astype(bool)
    ref_cells, ref_units = z["tape_sel_cell_idx"], z["tape_sel_unit_idx"]
    B, T = valid.shape[:2]
    # decisions, position by position from the reference's own pre-round state (so one flipped
    # decision does not cost the rest of its row): equal, or different only among cells whose scores
    # are within one bfloat16 unit of the last selected score (a float32 sum on a rounding boundary:
    # bf16_a has one, its reference score lies half a unit from the oracle's)
    same = np.zeros((B, T), dtype=bool)
    fired = 0
    for t in range(T):
        p = O.position(W, z["tape_tape_h"][:, t], z["tape_tape_q"][:, t], z["tape_tape_age"][:, t],
                       z["z"][:, t], z["ctx"][:, t], z["scalars"][:, t], bf16=True)  # fmt: skip
        fired += int(p["refreshed"].sum())
        score = p["logits"].max(axis=-1)
        for b in range(B):
            same[b, t] = (np.array_equal(p["cells"][b], ref_cells[b, t]) and np.array_equal(p["units"][b], ref_units[b, t])
                          and np.array_equal(p["valid"][b], valid[b, t]))  # fmt: skip
            if not same[b, t]:
                assert np.array_equal(p["valid"][b], valid[b, t])
                mine, theirs = set(p["cells"][b][valid[b, t]].tolist()), set(ref_cells[b, t][valid[b, t]].tolist())
                moved = sorted(mine ^ theirs) or sorted(mine)
                last = np.sort(score[b])[::-1][K - 1]
                assert np.abs(score[b][moved] - last).max() <= abs(last) * 2.0**-7, (b, t, moved)
    assert same.mean() >= 0.9, same
    if name == "bf16_a":
        assert fired > 0
    # values with the reference's decision replayed: every row and position counts
    tape = O.window_forward(W, *args, bf16=True, forced=(z["tape_sel_cell_idx"], z["tape_sel_unit_idx"], valid))
    tol = 2e-2
    for mine, ref in (
        ("tape_h", "tape_tape_h"), ("tape_q", "tape_tape_q"), ("tape_hsel", "tape_tape_hsel"),
        ("qs", "tape_qs"), ("h", "tape_h"), ("q", "tape_q"),
    ):  # fmt: skip
        scale = float(np.abs(z[ref]).max())
        np.testing.assert_allclose(tape[mine], z[ref], rtol=tol, atol=tol * scale, err_msg=mine)
    for key, ref in (("y", "rec_y"), ("gate_pre", "rec_gate_pre"), ("m", "rec_m"), ("rms", "rec_rms"),
                     ("hidden", "rec_hidden"), ("c", "bw_c"), ("b", "bw_b"), ("h_old", "bw_h_old")):  # fmt: skip
        got, want = tape["rec_" + key][valid], z[ref][valid]
        scale = float(np.abs(want).max())
        np.testing.assert_allclose(got, want, rtol=tol, atol=tol * scale, err_msg=key)
    # the reverse sweep on the reference's own record: the oracle in float32 against the reference's
    # sweep (whose two transposed products ran under the same autocast)
    N = z["h0"].shape[1]
    record = {k: z["rec_" + k] for k in ("y", "hidden", "gate_pre", "m", "rms")}
    cot = lambda k: z[k] if k in z.files else None  # noqa: E731
    trace: dict = {}
    dc, db = O.state_gradient_backward(
        W, z["bw_c"], z["bw_b"], z["bw_h_old"], z["bw_cells"], z["bw_units"], z["bw_valid"],
        z["reset"], N, cot("bw_d_q_pre"), cot("bw_d_q_post"), cot("bw_d_h_sel"), record, trace=trace,
    )  # fmt: skip
    scale = max(float(np.abs(z["bw_dc"]).max()), float(np.abs(z["bw_A"]).max()))
    np.testing.assert_allclose(dc, z["bw_dc"], rtol=tol, atol=tol * scale)
    np.testing.assert_allclose(db, z["bw_db"], rtol=tol, atol=tol * scale)
    np.testing.assert_allclose(trace["A"], z["bw_A"], rtol=tol, atol=tol * scale)
    np.testing.assert_allclose(trace["R"], z["bw_R"], rtol=tol, atol=tol * scale)


def test_full_cut_window_equals_the_reference() -> None:
    z = load_golden("window_cut_f64")
    N = z["h0"].shape[1]
    cot = lambda k: z[k] if k in z.files else None  # noqa: E731
    dc, db = O.recurrence_backward(
        z["bw_c"], z["bw_b"], z["bw_h_old"], z["bw_cells"], z["bw_valid"], z["reset"], N,
        cot("bw_d_q_pre"), cot("bw_d_q_post"), cot("bw_d_h_sel"),
    )  # fmt: skip
    np.testing.assert_allclose(dc, z["bw_dc"], rtol=1e-12, atol=1e-14)
    np.testing.assert_allclose(db, z["bw_db"], rtol=1e-12, atol=1e-14)


def test_chained_windows_equal_the_unsplit_window() -> None:
    """Two windows of T positions with the state carried forward and (A, R) carried back are the
    window of 2T positions (fixture: the reference's unsplit window and its sweep's trace)."""
    z = load_golden("chain_f64")
    dtype = np.dtype(np.float64)
    K = z["bw_cells"].shape[-1]
    W = O.WindowWeights.from_npz(z, K, dtype)
    N = z["h0"].shape[1]
    T2 = z["reset"].shape[1]
    T = T2 // 2
    # forward: window 1, then window 2 from its final state
    first = O.window_forward(W, z["z"][:, :T], z["ctx"][:, :T], z["scalars"][:, :T], z["reset"][:, :T],
                             z["h0"], z["q0"], z["age0"], z["pos0"])  # fmt: skip
    second = O.window_forward(W, z["z"][:, T:], z["ctx"][:, T:], z["scalars"][:, T:], z["reset"][:, T:],
                              first["h"], first["q"], first["age"], first["pos"])  # fmt: skip
    for key in ("tape_h", "tape_q", "qs", "tape_hsel"):
        joined = np.concatenate([first[key], second[key]], axis=1)
        np.testing.assert_allclose(joined, z["tape_" + key], rtol=1e-9, atol=1e-10)
    assert np.array_equal(np.concatenate([first["sel_cell_idx"], second["sel_cell_idx"]], 1), z["tape_sel_cell_idx"])
    np.testing.assert_allclose(second["h"], z["tape_h"], rtol=1e-9, atol=1e-10)
    assert np.array_equal(second["pos"], z["tape_pos"])
    # backward: window 2's sweep, its (A, R) into window 1's sweep
    record = {k: z["rec_" + k] for k in ("y", "hidden", "gate_pre", "m", "rms")}
    part = lambda a, s: None if a is None else a[:, s]  # noqa: E731
    cot = lambda k: z[k] if k in z.files else None  # noqa: E731
    halves = {}
    carry = None
    for s in (slice(T, T2), slice(0, T)):
        trace: dict = {}
        dc, db = O.state_gradient_backward(
            W, z["bw_c"][:, s], z["bw_b"][:, s], z["bw_h_old"][:, s], z["bw_cells"][:, s],
            z["bw_units"][:, s], z["bw_valid"][:, s], z["reset"][:, s], N,
            part(cot("bw_d_q_pre"), s), part(cot("bw_d_q_post"), s), part(cot("bw_d_h_sel"), s),
            {k: v[:, s] for k, v in record.items()}, initial=carry, trace=trace,
        )  # fmt: skip
        halves[s.start] = (dc, db)
        reset0 = z["reset"][:, s.start].astype(bool)
        carry = (np.where(reset0[:, None, None], 0, trace["A"][:, 0]),
                 np.where(reset0[:, None], 0, trace["R"][:, 0]))  # fmt: skip
    dc = np.concatenate([halves[0][0], halves[T][0]], axis=1)
    db = np.concatenate([halves[0][1], halves[T][1]], axis=1)
    np.testing.assert_allclose(dc, z["bw_dc"], rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(db, z["bw_db"], rtol=1e-10, atol=1e-12)


def test_out_adjacency_lists_every_edge_by_source() -> None:
    rng = np.random.default_rng(0)
    N, D = 9, 3
    pad_src = rng.integers(0, N, (N, D))
    mask = rng.random((N, D)) > 0.2
    tgt, edge = O.out_adjacency(pad_src, mask)
    seen = set()
    for n in range(N):
        for j in range(tgt.shape[1]):
            if tgt[n, j] >= 0:
                t, s = divmod(int(edge[n, j]), D)
                assert t == tgt[n, j] and pad_src[t, s] == n and mask[t, s]
                seen.add((t, s))
    assert len(seen) == int(mask.sum())


def test_bf16_rounding_is_nearest_even() -> None:
    import torch

    x = torch.randn(4096, generator=torch.Generator().manual_seed(0)) * 3
    x[:4] = torch.tensor([1.00390625, 1.01171875, float("inf"), -0.0])
    want = x.to(torch.bfloat16).float().numpy()
    assert np.array_equal(O.bf16_round(x.numpy()), want)


@pytest.mark.parametrize("name", SWEEP_SETS)
def test_sweep_glue_steps_equal_the_reference(name: str) -> None:
    """The head, middle and tail of two positions in sweep order against the reference's own
    PyTorch steps on the same buffers: the operands (bf16 in two sets) to the bit where they are
    copies or single roundings of fp32 values within an ulp, the fp32 sums to 1e-5."""
    z, sizes, buf = sweep_fixture(name)
    s = O.SweepSizes(*sizes)
    half = bool(z["half"])

    def check(stage: str) -> None:
        for key in SWEEP_WRITTEN:
            want = z[f"{stage}_{key}"]
            tol = 1e-5 * max(1.0, float(np.abs(want).max()))
            if half and key.startswith("op"):
                tol = 2.0**-7 * max(1.0, float(np.abs(want).max()))  # one bf16 step at most
                assert np.mean(buf[key] != want) < 0.02, (stage, key)
            assert np.abs(buf[key] - want).max() <= tol, (stage, key)

    for t in (s.T - 1, s.T - 2):
        O.sweep_head(s, buf, t, cand_norm=bool(z["cand_norm"]), cand_eps=float(z["cand_eps"]), half=half)
        check(f"head{t}")
        buf["act_r"], buf["act_f"] = z[f"mid{t}_act_r"], z[f"mid{t}_act_f"]
        O.sweep_middle(s, buf, t, activation=str(z["activation"]), half=half)
        check(f"mid{t}")
        buf["dv_r"], buf["dv_f"] = z[f"tail{t}_dv_r"], z[f"tail{t}_dv_f"]
        O.sweep_tail(s, buf, t, cell_norm=bool(z["cell_norm"]))
        check(f"tail{t}")


def _prologue_tables(z) -> dict:
    budget, round_frac, n_context, unroll = (float(v) for v in z["numbers"])
    P = {k: z[k] for k in ("byte_emb", "enc_w1", "enc_b1", "enc_w2", "enc_b2", "ctx_emb", "byte_codes",
                           "cell_addresses", "ema_utility", "ema_selected")}  # fmt: skip
    P.update(budget_frac=budget, round_frac=round_frac, n_context=n_context, unroll=unroll, position=str(z["position"]))
    return P


@pytest.mark.parametrize("name", ["fresh_f32", "carried_f32", "fresh_bf16"])
def test_window_prologue_equals_the_reference(name: str) -> None:
    """Token and context ids to what the sweep reads (z, context embeddings, scorer scalars) against
    ``HSN._window_prologue`` on the CPU: a fresh stream, a carried position with carried previous
    bytes and non-zero running averages, and the encoder under bf16 autocast."""
    z = load_golden(f"prologue_{name}")
    prev = z["prev_tokens"] if "prev_tokens" in z.files else None
    bf = name.endswith("bf16")
    got = O.window_prologue(_prologue_tables(z), z["tokens"], z["ctx_ids"], z["reset"], z["pos0"], prev, bf16=bf)
    tol = 2e-2 if bf else 1e-5
    scale = float(np.abs(z["z"]).max())
    np.testing.assert_allclose(got["z"], z["z"], rtol=tol, atol=tol * scale)
    assert np.array_equal(got["ctx"], z["context"])
    np.testing.assert_allclose(got["scalars"], z["scalars"], rtol=1e-5, atol=1e-5)
    assert got["scalars"].shape[-1] == 9
    if name == "carried_f32":
        assert float(np.abs(got["scalars"][..., 3]).max()) > 0 and int(got["positions"].max()) > 100


@pytest.mark.parametrize("name,tol", [("f64", 1e-12), ("f32", 1e-5), ("bf16", 0.0)])
def test_window_decode_equals_the_reference(name: str, tol: float) -> None:
    """The decoder over ``[q; u]`` against ``HSN._decode`` on the CPU: float64, float32, and under bf16
    autocast, where the restatement reproduces the reference's bfloat16 logits exactly."""
    z = load_golden(f"decode_{name}")
    got = O.window_decode({k: z[k] for k in ("dec_w1", "dec_b1", "dec_w2", "dec_b2")}, z["qs"], z["us"], bf16=name == "bf16")
    assert got.shape == z["logits"].shape == z["qs"].shape[:-1] + (256,)
    if tol == 0.0:
        assert np.array_equal(got, z["logits"])
    else:
        np.testing.assert_allclose(got, z["logits"], rtol=tol, atol=tol * float(np.abs(z["logits"]).max()))


@pytest.mark.parametrize("case", ["a", "b"])
@pytest.mark.parametrize("name,tol", [("f64", 1e-12), ("f32", 1e-5), ("bf16", 1e-5)])
def test_grouped_units_equal_the_reference(case: str, name: str, tol: float) -> None:
    """The replay's grouped unit pass and its backward against ``UnitBank.forward_grouped`` with autograd on the
    CPU: float64, float32, and under bf16 autocast, where the restatement reproduces the reference's bfloat16
    values (the record to the bit, the gradients but for a rounding boundary of the activation's derivative)."""
    from oracle import units_oracle as U

    z = load_golden(f"units_{case}_{name}")
    bf = name == "bf16"
    bank = tuple(z[k] for k in ("W1", "b1", "W2", "b2"))
    out, pre = U.forward_grouped(z["v"], z["unit_idx"], *bank, bf16=bf)
    grads = U.backward_grouped(z["v"], z["unit_idx"], *bank, pre, z["cot"], bf16=bf)
    if bf:
        assert np.array_equal(pre, z["hidden"]) and np.array_equal(out, z["out"])
    got = dict(out=out, hidden=pre, **dict(zip(("d_v", "d_W1", "d_b1", "d_W2", "d_b2"), grads, strict=True)))
    for key, value in got.items():
        np.testing.assert_allclose(value, z[key], rtol=0, atol=tol * float(np.abs(z[key]).max()), err_msg=key)
    if case == "a":   # a unit no pair chose: zero gradients, as autograd leaves them
        assert not np.any(z["unit_idx"] == 3) and not np.any(grads[1][3]) and not np.any(grads[4][3])
    with pytest.raises(IndexError):
        U.forward_grouped(z["v"], np.full_like(z["unit_idx"], z["W1"].shape[0]), *bank)


@pytest.mark.parametrize("name,tol", [("f64", 1e-12), ("f32", 1e-5), ("bf16", 0.0)])
def test_scorer_logits_equal_the_reference(name: str, tol: float) -> None:
    """The replay's scorer logits and the gradients of the scorer's weight and bias against ``_scorer_logits`` with
    autograd on the CPU: float64, float32, and under bf16 autocast, where the restatement reproduces the reference's
    values to the bit."""
    from oracle import scorer_oracle as S

    z = load_golden(f"scorer_{name}")
    bf = name == "bf16"
    feats = tuple(z[k] for k in ("u", "eps", "h", "age", "scalars"))
    out = S.scorer_logits(z["weight"], z["bias"], *feats, float(z["age_max"]), bf16=bf)
    d_w, d_b = S.scorer_logits_backward(z["weight"], *feats, float(z["age_max"]), z["cot"], bf16=bf)
    for got, key in ((out, "logits"), (d_w, "d_weight"), (d_b, "d_bias")):
        assert got.shape == z[key].shape
        if tol == 0.0:
            assert np.array_equal(got, z[key]), key
        else:
            np.testing.assert_allclose(got, z[key], rtol=0, atol=tol * float(np.abs(z[key]).max()), err_msg=key)


def _tail_case(name: str):
    z = load_golden(f"replay_{name}")
    d = z["unit_out"].shape[-1]
    flat = lambda key: z[key].reshape(-1, d)  # noqa: E731
    args = (flat("unit_out"), z["alpha"].reshape(-1), z["w_W_out.weight"], z["w_cand_norm.weight"])
    want = dict(c=flat("c"), y=flat("rec_y"), d_unit_out=flat("d_unit_out"), d_alpha=z["d_alpha"].reshape(-1),
                d_w_out=z["g_W_out.weight"], d_cand_w=z["g_cand_norm.weight"])  # fmt: skip
    return z, args, flat("d_c"), want


@pytest.mark.parametrize("name", ["f32", "cut_f32", "bf16", "wide_bf16"])
def test_replay_tail_equals_the_reference(name: str) -> None:
    """``W_out``, the candidate norm and the weighted ``tanh`` of ``replay_sparse`` with autograd's gradients, on the
    values the reference's own replay held inside a split window: float32 (also with slots the budget cut, whose
    weight is zero) and under bf16 autocast, where ``y`` and the linear's two gradients equal the reference's to the
    bit and the float32 parts to rounding."""
    from oracle import tail_oracle as T

    z, args, d_c, want = _tail_case(name)
    bf = "bf16" in name
    eps = float(z["cand_eps"])
    c, y = T.forward_tail(*args, cand_eps=eps, bf16=bf)
    assert np.array_equal(y, want["y"])
    grads = T.backward_tail(*args, want["y"], d_c, cand_eps=eps, bf16=bf)
    got = dict(c=c, d_unit_out=grads[0], d_alpha=grads[1], d_w_out=grads[2], d_cand_w=grads[3])
    for key, value in got.items():
        assert value.shape == want[key].shape and value.dtype == np.float32, key
        np.testing.assert_allclose(value, want[key], rtol=0, atol=1e-6 * float(np.abs(want[key]).max()), err_msg=key)
    if bf:
        assert np.array_equal(got["d_unit_out"], want["d_unit_out"]) and np.array_equal(got["d_w_out"], want["d_w_out"])
    if name == "cut_f32":   # a slot the budget cut: weight 0, candidate 0, no gradient into the unit's output
        cut = ~z["valid"].reshape(-1)
        assert cut.any() and not np.any(args[1][cut]) and not np.any(c[cut]) and not np.any(grads[0][cut])


@pytest.mark.parametrize("name", ["f32", "cut_f32", "bf16", "wide_bf16"])
def test_replay_norm_and_gate_equal_the_reference(name: str) -> None:
    """The cell norm, the gate and the sigmoid of ``replay_sparse`` with autograd's gradients, on the values the
    reference's own replay held inside a split window (the norm's input and output taken by a forward hook, the unit
    pass's own gradient of ``v`` by wrapping ``forward_grouped``): float32 to rounding; under bf16 autocast the
    bfloat16-rounded results to one bfloat16 step."""
    from oracle import gate_oracle as G

    z = load_golden(f"replay_{name}")
    bf = "bf16" in name
    F = z["v_raw"].shape[-1]
    d = F // 4
    args = (z["v_raw"].reshape(-1, F), z["w_norm.weight"], z["w_gate.weight"], z["w_gate.bias"])
    eps = float(z["norm_eps"])
    v, rms, gate_pre, b = G.forward_norm_gate(*args, norm_eps=eps, bf16=bf)
    grads = G.backward_norm_gate(*args, z["d_v_units"].reshape(-1, F), z["d_b"].reshape(-1, d), norm_eps=eps, bf16=bf)
    step = 2.0**-7 if bf else 4e-6   # one bfloat16 step of the largest value, or float32 rounding of a sum
    for got, want, tol, what in (
        (v, z["v"].reshape(-1, F), 4e-6, "v"), (rms, z["rec_rms"].reshape(-1), 4e-6, "rms"),
        (gate_pre, z["rec_gate_pre"].reshape(-1, d), step, "gate_pre"), (b, z["b"].reshape(-1, d), step, "b"),
        (grads[0], z["d_v_raw"].reshape(-1, F), 1e-4 if bf else 4e-6, "d_v_raw"), (grads[1], z["g_norm.weight"], 4e-6, "d_norm_w"),
        (grads[2], z["g_gate.weight"], step, "d_gate_w"), (grads[3], z["g_gate.bias"], step, "d_gate_b"),
    ):  # fmt: skip
        assert got.shape == want.shape and got.dtype == np.float32, what
        np.testing.assert_allclose(got, want, rtol=0, atol=tol * float(np.abs(want).max()), err_msg=what)
    if name == "bf16":   # here nothing falls on a rounding boundary: the bfloat16 parts equal the reference's to the bit
        assert np.array_equal(gate_pre, z["rec_gate_pre"].reshape(-1, d)) and np.array_equal(grads[2], z["g_gate.weight"])


@pytest.mark.parametrize("name", ["f32", "cut_f32", "bf16", "wide_bf16"])
def test_replay_messages_equal_the_reference(name: str) -> None:
    """The gathered inputs ``v_raw = [u; eps; h[cell]; m]`` of ``replay_sparse`` with the messages ``m`` over the cell's
    in-neighbours, and autograd's gradients of ``u``, ``eps``, the padded edge weights and ``V``: under bf16 autocast to
    the bit but for the edge weights' gradient, which the reference accumulates slot by slot in bfloat16 (within one
    bfloat16 step); float32 to rounding."""
    from oracle import messages_oracle as M

    z = load_golden(f"replay_{name}")
    bf = "bf16" in name
    cells = np.where(z["valid"], z["cells"], 0)
    tables = (cells, z["pad_src"], z["edge_w"], z["w_V.weight"])
    v_raw = M.forward_messages(z["u"], z["eps"], z["h_read"], *tables, bf16=bf)
    grads = M.backward_messages(z["h_read"], *tables, z["d_v_raw"], bf16=bf)
    d = z["u"].shape[-1]
    assert v_raw.dtype == np.float32 and np.array_equal(v_raw[..., : 3 * d], z["v_raw"][..., : 3 * d])
    np.testing.assert_allclose(v_raw, z["v_raw"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(v_raw[..., 3 * d :], z["rec_m"], rtol=0, atol=1e-6)
    for got, key, tol in zip(grads, ("d_u", "d_eps", "d_edge_w", "g_V.weight"), (1e-6, 1e-6, 2.0**-7 if bf else 1e-6, 1e-6), strict=True):
        assert got.shape == z[key].shape and got.dtype == np.float32, key
        np.testing.assert_allclose(got, z[key], rtol=0, atol=tol * float(np.abs(z[key]).max()), err_msg=key)
    if bf:
        assert np.array_equal(v_raw, z["v_raw"]) and np.array_equal(grads[3], z["g_V.weight"])


def _numeric(fn, x, eps=1e-6):
    """Central differences of the scalar ``fn`` at ``x`` (float64), entry by entry."""
    g = np.zeros_like(x)
    it = np.nditer(x, flags=["multi_index"])
    for _ in it:
        i = it.multi_index
        keep = x[i]
        x[i] = keep + eps
        hi = fn()
        x[i] = keep - eps
        lo = fn()
        x[i] = keep
        g[i] = (hi - lo) / (2 * eps)
    return g


def test_the_replay_oracles_backwards_are_the_gradients_of_their_forwards() -> None:
    """Independent of the fixtures: in float64 the three restated backwards of ``replay_sparse``'s steps equal central
    differences of the restated forwards."""
    from oracle import gate_oracle as G
    from oracle import messages_oracle as M
    from oracle import tail_oracle as T

    rng = np.random.default_rng(7)
    f = lambda *s, scale=1.0: rng.standard_normal(s) * scale  # noqa: E731
    # the tail
    P, d = 5, 6
    x, alpha, w, g, cot = f(P, d), 1.0 + 0.3 * f(P), f(d, d, scale=0.5), 1.0 + 0.2 * f(d), f(P, d)
    loss = lambda: float((T.forward_tail(x, alpha, w, g)[0] * cot).sum())  # noqa: E731
    _, y = T.forward_tail(x, alpha, w, g)
    got = T.backward_tail(x, alpha, w, g, y, cot)
    for a, wrt in zip(got, (x, alpha, w, g), strict=True):
        np.testing.assert_allclose(a, _numeric(loss, wrt), rtol=1e-6, atol=1e-8)
    # the norm and the gate
    F = 4 * d
    vr, nw, gw, gb, dv, db = f(P, F), 1.0 + 0.2 * f(F), f(d, F, scale=0.3), f(d, scale=0.3), f(P, F), f(P, d)

    def loss2():
        v, _, _, b = G.forward_norm_gate(vr, nw, gw, gb, norm_eps=1e-6)
        return float((v * dv).sum() + (b * db).sum())

    got = G.backward_norm_gate(vr, nw, gw, gb, dv, db, norm_eps=1e-6)
    for a, wrt in zip(got, (vr, nw, gw, gb), strict=True):
        np.testing.assert_allclose(a, _numeric(loss2, wrt), rtol=1e-6, atol=1e-8)
    # the messages
    R, N, K, D = 3, 7, 2, 3
    u, e, h, vw, ew, cot3 = f(R, d), f(R, d), f(R, N, d), f(d, d, scale=0.5), rng.random((N, D)), f(R, K, 4 * d)
    cells, src = rng.integers(0, N, (R, K)), rng.integers(0, N, (N, D))
    loss3 = lambda: float((M.forward_messages(u, e, h, cells, src, ew, vw) * cot3).sum())  # noqa: E731
    got = M.backward_messages(h, cells, src, ew, vw, cot3)
    for a, wrt in zip(got, (u, e, ew, vw), strict=True):
        np.testing.assert_allclose(a, _numeric(loss3, wrt), rtol=1e-6, atol=1e-8)
