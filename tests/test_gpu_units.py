"""The replay's grouped unit pass on the device (``hsnw_units_forward`` / ``hsnw_units_backward`` through
``hsn_b200.kernels.units``): against the reference's fixtures (``tests/golden/units_*.npz``:
``UnitBank.forward_grouped`` with autograd on the CPU, float32 and under bf16 autocast), against the oracle at the
benchmark's widths, the edges (no pairs, a unit nobody chose, every pair on one unit, a bad index), and at the
benchmark's full size through what does not depend on the size: the pairs' order does not matter."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import dev, load_golden, to_np
from oracle import units_oracle as U
from oracle import window_oracle as O

pytestmark = pytest.mark.gpu

BANK = ("W1", "b1", "W2", "b2")
GRADS = ("d_v", "d_W1", "d_b1", "d_W2", "d_b2")


def _close(got, want, tol, what=""):
    np.testing.assert_allclose(got, want, rtol=0, atol=tol * max(float(np.abs(want).max()), 1e-30), err_msg=what)


@pytest.mark.parametrize("case", ["a", "b"])
@pytest.mark.parametrize("name", ["f32", "bf16"])
def test_grouped_units_equal_the_reference(case: str, name: str) -> None:
    """Through autograd, as the replay calls it: values, record and all five gradients."""
    from hsn_b200.kernels.units import forward_grouped

    z = load_golden(f"units_{case}_{name}")
    bf = name == "bf16"
    tol = 2e-2 if bf else 1e-5
    v = dev(z["v"]).requires_grad_(True)
    bank = [dev(z[k]).requires_grad_(True) for k in BANK]
    record: dict = {}
    out = forward_grouped(v, dev(z["unit_idx"]), *bank, record=record, prod="bf16" if bf else "fp32")
    assert out.dtype == (torch.bfloat16 if bf else torch.float32) and not record["hidden"].requires_grad
    got_out = to_np(out.detach().float())
    _close(got_out, z["out"], tol, "out")
    _close(to_np(record["hidden"].float()), z["hidden"], tol, "hidden")
    if bf:   # bfloat16 values: all but a few equal the reference's to the bit
        assert float(np.mean(got_out == z["out"])) > 0.97
        assert float(np.mean(to_np(record["hidden"].float()) == z["hidden"])) > 0.97
    (out.float() * dev(z["cot"])).sum().backward()
    for key, t in zip(GRADS, [v, *bank], strict=True):
        assert t.grad is not None and t.grad.dtype == torch.float32
        _close(to_np(t.grad), z[key], tol, key)


def _case(rng, P, M, d, H, bf, units=None):
    f = lambda *s, scale=1.0: (rng.standard_normal(s) * scale).astype(np.float32)  # noqa: E731
    bank = [f(M, 4 * d, H, scale=(4 * d) ** -0.5), f(M, H, scale=0.3), f(M, H, d, scale=H**-0.5), f(M, d, scale=0.3)]
    v, cot = f(P, 4 * d), f(P, d)
    idx = rng.integers(0, M, P) if units is None else np.asarray(units, dtype=np.int64)
    if bf:
        cot = O.bf16_round(cot)
    return v, idx.astype(np.int64), bank, cot


@pytest.mark.parametrize("prod", ["bf16", "fp32"])
@pytest.mark.parametrize("P,M,d,H", [(4099, 8, 64, 512), (1, 3, 16, 128), (700, 5, 32, 136), (300, 2, 128, 1024)])
def test_grouped_units_equal_the_oracle(prod: str, P: int, M: int, d: int, H: int) -> None:
    """The benchmark's widths on a count that is no multiple of a tile, one pair, a hidden width that is no
    multiple of a tile, the widest model's unit."""
    from hsn_b200.kernels.units import grouped_backward, grouped_forward

    bf = prod == "bf16"
    tol = 2e-2 if bf else 1e-5
    v, idx, bank, cot = _case(np.random.default_rng(P), P, M, d, H, bf)
    want_out, want_pre = U.forward_grouped(v, idx, *bank, bf16=bf)
    out, pre, status = grouped_forward(dev(v), dev(idx), *map(dev, bank), prod=prod)
    assert int(status) == 0
    _close(to_np(pre.float()), want_pre, tol, "pre")
    _close(to_np(out.float()), want_out, tol, "out")
    # the backward on the oracle's record, so that one rounding boundary of the forward does not travel
    want = U.backward_grouped(v, idx, *bank, want_pre, cot, bf16=bf)
    got = grouped_backward(dev(v), dev(idx), *map(dev, bank), dev(want_pre).to(pre.dtype), dev(cot).to(pre.dtype), prod=prod)
    for key, g, w in zip(GRADS, got, want, strict=True):
        _close(to_np(g), w, tol, key)


def test_edges() -> None:
    from hsn_b200.kernels.units import forward_grouped, grouped_backward, grouped_forward

    rng = np.random.default_rng(3)
    v, idx, bank, cot = _case(rng, 260, 4, 16, 64, True, units=np.full(260, 2))   # every pair on one unit
    out, pre, _ = grouped_forward(dev(v), dev(idx), *map(dev, bank))
    want_out, want_pre = U.forward_grouped(v, idx, *bank, bf16=True)
    _close(to_np(out.float()), want_out, 2e-2)
    got = grouped_backward(dev(v), dev(idx), *map(dev, bank), pre, dev(cot).bfloat16())
    want = U.backward_grouped(v, idx, *bank, to_np(pre.float()), cot, bf16=True)
    for key, g, w in zip(GRADS, got, want, strict=True):
        _close(to_np(g), w, 2e-2, key)
    for j in (0, 1, 3):   # the units nobody chose: zero gradients
        assert not to_np(got[1])[j].any() and not to_np(got[2])[j].any() and not to_np(got[3])[j].any() and not to_np(got[4])[j].any()
    # no pairs
    record: dict = {}
    empty = forward_grouped(dev(v[:0]), dev(idx[:0]), *map(dev, bank), record=record)
    assert tuple(empty.shape) == (0, 16) and tuple(record["hidden"].shape) == (0, 64)
    # an index outside [0, M): the reference's IndexError
    bad = idx.copy()
    bad[17] = 4
    with pytest.raises(IndexError):
        grouped_forward(dev(v), dev(bad), *map(dev, bank))
    bad[17] = -1
    with pytest.raises(IndexError):
        grouped_forward(dev(v), dev(bad), *map(dev, bank))
    # what the call refuses
    with pytest.raises(ValueError):
        grouped_forward(dev(v[:, :60]), dev(idx), *map(dev, bank))
    with pytest.raises(ValueError):
        grouped_forward(dev(v), dev(idx[:-1]), *map(dev, bank))
    with pytest.raises(RuntimeError):
        grouped_forward(torch.from_numpy(v), torch.from_numpy(idx), *map(torch.from_numpy, bank))


@pytest.mark.parametrize("prod", ["bf16", "fp32"])
def test_the_pairs_order_does_not_matter_at_full_size(prod: str) -> None:
    """The benchmark's window (32 rows x 256 positions x 8 slots = 65,536 pairs, 8 units, 256 -> 512 -> 64): a
    permutation of the pairs permutes ``out``, ``pre`` and ``d_v`` bit for bit (a pair's row of a product does
    not depend on its neighbours in the tile) and leaves the parameter gradients within the sums' rounding; two
    runs of the same call agree to the bit (the weight gradients' partial sums have a fixed order); and the
    cotangent enters linearly."""
    from hsn_b200.kernels.units import grouped_backward, grouped_forward

    bf = prod == "bf16"
    P, M, d, H = 32 * 256 * 8, 8, 64, 512
    rng = np.random.default_rng(11)
    v, idx, bank, cot = _case(rng, P, M, d, H, bf)
    idx[: P // 2] = rng.choice(M, P // 2, p=[0.5, 0.2, 0.1, 0.1, 0.05, 0.03, 0.02, 0.0])   # uneven, one unit rare
    tv, ti, tc = dev(v), dev(idx), dev(cot)
    tb = [dev(b) for b in bank]
    dt = torch.bfloat16 if bf else torch.float32
    out, pre, status = grouped_forward(tv, ti, *tb, prod=prod)
    grads = grouped_backward(tv, ti, *tb, pre, tc.to(dt), prod=prod)
    assert int(status) == 0 and bool(torch.isfinite(out.float()).all())
    perm = torch.from_numpy(rng.permutation(P)).cuda()
    out_p, pre_p, _ = grouped_forward(tv[perm], ti[perm], *tb, prod=prod)
    assert torch.equal(out_p, out[perm]) and torch.equal(pre_p, pre[perm])
    grads_p = grouped_backward(tv[perm], ti[perm], *tb, pre_p, tc[perm].to(dt), prod=prod)
    assert torch.equal(grads_p[0], grads[0][perm])
    tol = 2e-2 if bf else 1e-5
    for key, a, b in zip(GRADS[1:], grads_p[1:], grads[1:], strict=True):
        _close(to_np(a), to_np(b), tol, key)
    again = grouped_backward(tv, ti, *tb, pre, tc.to(dt), prod=prod)
    for a, b in zip(again, grads, strict=True):
        assert torch.equal(a, b)
    if not bf:   # linear in the cotangent (exact factors of two)
        twice = grouped_backward(tv, ti, *tb, pre, 2 * tc, prod=prod)
        for a, b in zip(twice, grads, strict=True):
            assert torch.equal(a, 2 * b)
    # a sample of pairs against the oracle
    rows = rng.choice(P, 257, replace=False)
    want_out, want_pre = U.forward_grouped(v[rows], idx[rows], *bank, bf16=bf)
    _close(to_np(out[rows].float()), want_out, tol, "out")
    _close(to_np(pre[rows].float()), want_pre, tol, "pre")


@pytest.mark.parametrize("prod", ["bf16", "fp32"])
def test_against_pytorch_on_the_device(prod: str) -> None:
    """The reference's own formulation run live on the GPU (pairs sorted by unit, one ``addmm`` per layer and present
    unit, under bf16 autocast or not, autograd's backward) against ``forward_grouped`` with the same leaves."""
    from hsn_b200.kernels.units import forward_grouped

    bf = prod == "bf16"
    P, M, d, H = 3000, 6, 32, 256
    v, idx, bank, cot = _case(np.random.default_rng(21), P, M, d, H, bf)
    idx[idx == 4] = 1   # a unit nobody chose

    def leaves():
        return dev(v).requires_grad_(True), [dev(b).requires_grad_(True) for b in bank]

    tv, tb = leaves()
    out = forward_grouped(tv, dev(idx), *tb, prod=prod)
    (out.float() * dev(cot)).sum().backward()
    rv, rb = leaves()
    order = torch.argsort(dev(idx), stable=True)
    counts = torch.bincount(dev(idx), minlength=M).tolist()
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=bf):
        sorted_v, outs, start = rv.index_select(0, order), [], 0
        for j, n in enumerate(counts):
            if n:
                hidden = torch.nn.functional.gelu(torch.addmm(rb[1][j], sorted_v[start:start + n], rb[0][j]))
                outs.append(torch.addmm(rb[3][j], hidden, rb[2][j]))
            start += n
        want = torch.empty_like(torch.cat(outs)).index_copy_(0, order, torch.cat(outs))
    (want.float() * dev(cot)).sum().backward()
    tol = 2e-2 if bf else 1e-5
    _close(to_np(out.detach().float()), to_np(want.detach().float()), tol, "out")
    for name, a, b in zip(GRADS, [tv, *tb], [rv, *rb], strict=True):
        want_grad = b.grad if b.grad is not None else torch.zeros_like(b)
        _close(to_np(a.grad), to_np(want_grad), tol, name)
