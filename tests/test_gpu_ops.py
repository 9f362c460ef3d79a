"""GPU parity of the kernels launched by name (select, cell update, recurrences) against the
reference's fixtures and the oracle. Every call goes through the C ABI."""

from __future__ import annotations

import numpy as np
import pytest
import torch
from conftest import load_golden

from oracle import window_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def window():
    from hsn_b200.kernels import window as w

    assert w.available(), "the CUDA library is not built (python -m hsn_b200.build)"
    w.prepare(0)
    return w


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


SELECT_SETS = ["plain", "probes", "budget", "probes_budget", "cost", "reserved"]


@pytest.mark.parametrize("name", SELECT_SETS)
def test_select_kernel_takes_the_routers_decision(window, name: str) -> None:
    """The reference's own trials (exact ties between cells and units, equal ages among the stale
    cells, budget cuts, cost penalties, reserved slots): bit for bit, theta included."""
    z = load_golden(f"select_{name}")
    p = z["params"]
    reserved = int(p[6]) if len(p) > 6 else 0
    cost = dev(z["cost"], torch.float32)
    for i in range(int(z["n"])):
        pre = f"t{i}_"
        cells, units, valid, theta, refreshed = window.select(
            dev(z[pre + "logits"], torch.float32), dev(z[pre + "age"]), cost, k=int(p[0]),
            age_max=int(p[1]), probes=bool(z[pre + "probes"]), lambda_cost=float(p[2]),
            cell_overhead=float(p[3]), shared_cost=float(p[4]), limit=float(p[5]), reserved=reserved,
            reserved_units=bool(z[pre + "fixed_units"]) if reserved else False,
        )  # fmt: skip
        assert np.array_equal(valid.cpu().numpy(), z[pre + "valid"].astype(bool)), (name, i)
        assert np.array_equal(cells.cpu().numpy(), z[pre + "cells"]), (name, i)
        assert np.array_equal(units.cpu().numpy(), z[pre + "units"]), (name, i)
        assert np.array_equal(refreshed.cpu().numpy(), z[pre + "refreshed"].astype(bool)), (name, i)
        assert np.array_equal(theta.cpu().numpy(), z[pre + "theta"]), (name, i)


@pytest.mark.parametrize("shape", [(32, 256, 8, 8), (4, 512, 8, 8), (3, 4096, 8, 16), (5, 1000, 3, 7), (2, 33, 5, 33)])
@pytest.mark.parametrize("ties", [False, True])
def test_select_kernel_equals_the_oracle_at_the_benchmark_sizes(window, shape, ties: bool) -> None:
    B, N, M, K = shape
    rng = np.random.default_rng(sum(shape) + int(ties))
    logits = rng.standard_normal((B, N, M)).astype(np.float32)
    if ties:
        logits = np.round(logits * 2) / 2
    age = rng.integers(0, 140, (B, N))
    if ties:
        age = (age // 3) * 3
    cost = np.full(M, 1.0 / (8 * N), np.float32)
    for probes, limit in ((True, 1.00001), (False, 1.00001), (True, 0.6 * K / (8 * N))):
        kw = dict(k=K, age_max=64, probes=probes, lambda_cost=0.0, cell_overhead=0.0, shared_cost=0.0,
                  limit=limit)  # fmt: skip
        want = O.select(logits, age, cost, **kw)
        got = window.select(dev(logits), dev(age), dev(cost), **kw)
        for g, w in zip(got, want):
            assert np.array_equal(g.cpu().numpy(), w)


def test_select_fold_reads_a_wider_bf16_product_in_place(window) -> None:
    rng = np.random.default_rng(3)
    B, N, M, K, W = 4, 64, 8, 6, 72
    scored = torch.as_tensor(rng.standard_normal((B * N, W)).astype(np.float32)).to(torch.bfloat16).cuda()
    age = dev(rng.integers(0, 100, (B, 3, N)))
    cost = dev(np.full(M, 0.001, np.float32))
    n = 2
    sentinel = -7
    cells = torch.full((B, n, K), sentinel, dtype=torch.int64, device="cuda")
    units = torch.full_like(cells, sentinel)
    valid = torch.zeros((B, n, K), dtype=torch.bool, device="cuda")
    refreshed = torch.zeros_like(valid)
    theta = torch.full((B, n), float(sentinel), device="cuda")
    kw = dict(age_max=64, probes=True, lambda_cost=0.0, cell_overhead=0.0, shared_cost=0.0, limit=1.0)
    window.select_fold(scored, age, cost, cells, units, valid, theta, refreshed, t=1, n_units=M, **kw)
    logits = scored.float().cpu().numpy().reshape(B, N, W)[:, :, :M]
    want = O.select(logits, age[:, 1].cpu().numpy(), cost.cpu().numpy(), k=K, **kw)
    assert np.array_equal(cells[:, 1].cpu().numpy(), want[0])
    assert np.array_equal(units[:, 1].cpu().numpy(), want[1])
    assert np.array_equal(theta[:, 1].cpu().numpy(), want[3])
    assert bool((cells[:, 0] == sentinel).all()) and bool((theta[:, 0] == sentinel).all())  # record 0 untouched


class _Cell:
    """The attributes of the reference's PDGCell that the wrappers read."""

    def __init__(self, cand_w, cand_norm: bool, eps: float) -> None:
        self.cand_norm_kind = "rms" if cand_norm else "none"
        self.cand_norm = torch.nn.RMSNorm(cand_w.shape[0], eps=eps if cand_norm else None)
        self.cand_norm.weight = torch.nn.Parameter(cand_w, requires_grad=False)
        self.norm = self.cand_norm


class _State:
    def __init__(self, h, q, age, pos) -> None:
        self.h, self.q, self.age, self.pos = h, q, age, pos

    @classmethod
    def _make(cls, h, q, age, pos):
        return cls(h, q, age, pos)


@pytest.mark.parametrize("name", ["rms", "none", "budget"])
def test_cell_update_kernel_equals_the_native_round(window, name: str) -> None:
    z = load_golden(f"update_{name}")
    cell = _Cell(dev(z["cand_w"], torch.float32), bool(z["cand_norm"]), float(z["cand_eps"]))
    for i in range(int(z["n"])):
        s = f"s{i}_"
        state = _State(dev(z[s + "h"]), dev(z[s + "q"]), dev(z[s + "age"]), dev(z[s + "pos"]))
        valid = dev(z[s + "valid"].astype(bool))
        got, h_sel, h_max = window.cell_update(cell, dev(z[s + "y"]), dev(z[s + "gate"]), state, dev(z[s + "cells"]), valid)
        assert float((got.h.cpu() - torch.as_tensor(z[s + "h_next"])).abs().max()) <= 2e-6
        assert float((got.q.cpu() - torch.as_tensor(z[s + "q_next"])).abs().max()) <= 2e-6
        assert np.array_equal(got.age.cpu().numpy(), z[s + "age_next"])
        assert np.array_equal(got.pos.cpu().numpy(), z[s + "pos_next"])
        safe = torch.where(valid, dev(z[s + "cells"]), 0)
        slots = got.h.gather(1, safe[:, :, None].expand(-1, -1, got.h.shape[2]))
        assert torch.equal(h_sel, slots)
        assert torch.equal(h_max, got.h.abs().amax(dim=(1, 2)))
        written = torch.zeros(got.h.shape[:2], dtype=torch.bool, device="cuda")
        written.scatter_(1, safe, valid)
        assert torch.equal(got.h[~written], state.h[~written])  # untouched cells: bit for bit


def test_tape_forms_write_only_their_own_records(window) -> None:
    """update_tape / update_fold over a block against the plain form and an explicit reset,
    position by position, on sentinel-filled tapes; bf16 products read in place; NaN row max."""
    rng = np.random.default_rng(5)
    B, n, N, d, K, dz, dcx = 3, 5, 12, 16, 3, 16, 8
    cell = _Cell(dev(rng.standard_normal(d).astype(np.float32)), True, 1e-6)
    sent = 123.0
    tape_h = torch.full((B, n + 1, N, d), sent, device="cuda")
    tape_q = torch.full((B, n + 1, d), sent, device="cuda")
    tape_age = torch.full((B, n + 1, N), 77, dtype=torch.int64, device="cuda")
    tape_h[:, 0] = dev(rng.standard_normal((B, N, d)).astype(np.float32))
    tape_q[:, 0] = tape_h[:, 0].mean(dim=1)
    tape_age[:, 0] = dev(rng.integers(0, 9, (B, N)))
    h_sel = torch.full((B, n, K, d), sent, device="cuda")
    h_max = torch.full((B, n), sent, device="cuda")
    qs = torch.full((B, n, d), sent, device="cuda")
    reset = torch.zeros((B, n), dtype=torch.bool, device="cuda")
    reset[0, 1] = reset[1, 2] = reset[1, 3] = reset[2, n - 1] = True
    x = torch.full((n, B, dz + d + dcx), sent, device="cuda", dtype=torch.bfloat16)
    zs = dev(rng.standard_normal((B, n, dz)).astype(np.float32)).to(torch.bfloat16)
    cs = dev(rng.standard_normal((B, n, dcx)).astype(np.float32))
    cells = torch.stack([torch.stack([torch.randperm(N)[:K] for _ in range(n)]) for _ in range(B)]).cuda()
    valid = torch.rand(B, n, K, device="cuda") > 0.2
    for t in range(n):
        y = dev(rng.standard_normal((B, K, d)).astype(np.float32)).to(torch.bfloat16)
        wide = dev(rng.standard_normal((B * K, d + 5)).astype(np.float32)).to(torch.bfloat16)
        gate = wide[:, 5:]  # a strided view of a wider product
        before = _State(tape_h[:, t].clone(), tape_q[:, t].clone(), tape_age[:, t].clone(),
                        torch.zeros(B, dtype=torch.int64, device="cuda"))  # fmt: skip
        want, want_sel, want_max = window.cell_update(cell, y.float(), gate.float().contiguous(), before, cells[:, t], valid[:, t])
        window.update_fold(cell, y, gate, tape_h, tape_q, tape_age, cells, valid, reset, h_sel, h_max, qs, x, zs, cs, t=t)
        clear = reset[:, t + 1] if t + 1 < n else torch.zeros(B, dtype=torch.bool, device="cuda")
        assert torch.equal(tape_h[:, t + 1], want.h.masked_fill(clear[:, None, None], 0))
        assert torch.equal(tape_q[:, t + 1], want.q.masked_fill(clear[:, None], 0))
        assert torch.equal(tape_age[:, t + 1], want.age.masked_fill(clear[:, None], 0))
        assert torch.equal(h_sel[:, t], want_sel) and torch.equal(h_max[:, t], want_max)
        assert torch.equal(qs[:, t], want.q)
        if t + 1 < n:
            row = torch.cat([zs[:, t + 1].float(), tape_q[:, t + 1], cs[:, t + 1]], dim=-1).to(torch.bfloat16)
            assert torch.equal(x[t + 1], row)
            assert bool((tape_h[:, t + 2 :] == sent).all()) and bool((x[t + 2 :] == sent).all())
            assert bool((h_sel[:, t + 1 :] == sent).all()) and bool((qs[:, t + 1 :] == sent).all())
    assert bool((x[0] == sent).all())  # position 0's row is the caller's
    # a NaN anywhere in the row makes the row's maximum NaN
    state = _State(tape_h[:, 0].clone(), tape_q[:, 0].clone(), tape_age[:, 0].clone(), torch.zeros(B, dtype=torch.int64, device="cuda"))
    state.h[1, 4, 2] = float("nan")
    y = torch.zeros((B, K, d), device="cuda")
    _, _, row_max = window.cell_update(cell, y, y.reshape(B * K, d), state, cells[:, 0], torch.zeros_like(valid[:, 0]))
    assert bool(torch.isnan(row_max[1])) and bool(torch.isfinite(row_max[0]))


@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_recurrence_kernel_equals_the_reference(window, name: str) -> None:
    z = load_golden(f"recurrence_{name}")
    N = int(z["N"])
    f32 = torch.float32
    base = (dev(z["c"], f32), dev(z["b"], f32), dev(z["h_old"], f32), dev(z["cells"]),
            dev(z["valid"].astype(bool)), dev(z["reset"].astype(bool)), N)  # fmt: skip
    for tag in ("111", "010", "101"):
        cots = [dev(z[k], f32) if on == "1" else None for k, on in zip(("pre", "post", "sel"), tag)]
        got = window.recurrence_backward(*base, *cots)
        assert got is not None
        for g, w in zip(got, (z[f"dc_{tag}"], z[f"db_{tag}"])):
            scale = max(1.0, float(np.abs(w).max()))
            assert float(np.abs(g.cpu().numpy().astype(np.float64) - w).max()) <= 2e-5 * scale
            assert bool((g[~base[4]] == 0).all())
    got = window.dense_recurrence_backward(
        dev(z["dense_c"], f32), dev(z["dense_b"], f32), dev(z["dense_h"], f32), base[5], N,
        dev(z["pre"], f32), dev(z["post"], f32),
    )  # fmt: skip
    assert got is not None
    for g, w in zip(got, (z["dense_dc"], z["dense_db"])):
        scale = max(1.0, float(np.abs(w).max()))
        assert float(np.abs(g.cpu().numpy().astype(np.float64) - w).max()) <= 2e-5 * scale


def test_recurrence_kernel_at_the_reference_shape_and_beyond_48k(window) -> None:
    """B32 T256 N256 d64 K8 needs 65 KB of cotangents per row: the reference kernel declines it."""
    rng = np.random.default_rng(11)
    B, T, N, K, d = 8, 64, 256, 8, 64
    cells = np.stack([np.stack([rng.permutation(N)[:K] for _ in range(T)]) for _ in range(B)])
    valid = rng.random((B, T, K)) > 0.1
    reset = rng.random((B, T)) < 0.03
    c = rng.uniform(-1, 1, (B, T, K, d)); b = rng.uniform(0, 1, (B, T, K, d)); h = rng.uniform(-1, 1, (B, T, K, d))
    pre, post = rng.standard_normal((B, T, d)), rng.standard_normal((B, T, d))
    sel = rng.standard_normal((B, T, K, d))
    cells = np.where(valid, cells, 0)
    final: dict = {}
    want = O.recurrence_backward(c, b, h, cells, valid, reset, N, pre, post, sel, final=final)
    f32 = torch.float32
    A = torch.zeros((B, N, d), device="cuda"); R = torch.zeros((B, d), device="cuda")
    got = window.recurrence_backward(dev(c, f32), dev(b, f32), dev(h, f32), dev(cells), dev(valid), dev(reset), N,
                                     dev(pre, f32), dev(post, f32), dev(sel, f32), initial=(A, R))  # fmt: skip
    assert got is not None
    for g, w in zip(got, want):
        scale = max(1.0, float(np.abs(w).max()))
        assert float(np.abs(g.cpu().numpy() - w).max()) <= 2e-5 * scale
    keep = ~reset[:, 0]
    scale = max(1.0, float(np.abs(final["A"]).max()))
    assert float(np.abs(A.cpu().numpy() - final["A"] * keep[:, None, None]).max()) <= 2e-5 * scale
    assert float(np.abs(R.cpu().numpy() - final["R"] * keep[:, None]).max()) <= 2e-5 * scale


def test_recurrence_kernel_keeps_a_padded_nan_out_and_declines_other_dtypes(window) -> None:
    rng = np.random.default_rng(3)
    B, T, N, K, d = 4, 16, 8, 3, 8
    f32 = torch.float32
    valid = dev(rng.random((B, T, K)) > 0.25)
    cells = torch.where(valid, dev(np.stack([np.stack([rng.permutation(N)[:K] for _ in range(T)]) for _ in range(B)])), 0)
    case = {k: dev(rng.standard_normal((B, T, K, d)), f32) for k in ("c", "b", "h_old", "sel")}
    for t in case.values():
        t[~valid] = float("nan")
    reset = dev(rng.random((B, T)) < 0.05)
    pre, post = dev(rng.standard_normal((B, T, d)), f32), dev(rng.standard_normal((B, T, d)), f32)
    got = window.recurrence_backward(case["c"], case["b"], case["h_old"], cells, valid, reset, N, pre, post, case["sel"])
    assert got is not None and bool(torch.isfinite(got[0]).all()) and bool(torch.isfinite(got[1]).all())
    assert window.recurrence_backward(case["c"].double(), case["b"].double(), case["h_old"].double(), cells, valid, reset, N, None, post.double(), None) is None
    assert window.recurrence_backward(case["c"].cpu(), case["b"].cpu(), case["h_old"].cpu(), cells.cpu(), valid.cpu(), reset.cpu(), N, None, None, None) is None


def test_a_wait_that_nothing_completes_runs_out_and_reports() -> None:
    """Every mbarrier wait of the window kernels is bounded. A small kernel waits on a barrier that
    nothing arrives at (no copy in flight, nothing faults): both kinds of wait give up after their
    limit and set their status word, a later wait of the same block returns at once, the kernel
    reaches its end, and the context still runs work afterwards."""
    from hsn_b200 import _lib
    from hsn_b200.window import prepare

    prepare(0)
    words = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    _lib.check(_lib.library().hsnw_selftest_wait_timeout(words.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert words.tolist() == [1, 1, 7, 0]
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0
