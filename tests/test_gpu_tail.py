"""The end of the replay's cell pass on the device (``hsnw_tail_forward`` / ``hsnw_tail_backward`` through
``hsn_b200.kernels.tail``): against the reference's fixtures (``tests/golden/replay_*.npz``: ``replay_sparse`` inside a
split window with autograd on the CPU, float32 and under bf16 autocast), against the oracle at the benchmark's sizes
and at ragged ones, and at the benchmark's full window through what does not depend on the size."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import dev, load_golden, to_np
from oracle import tail_oracle as TO

pytestmark = pytest.mark.gpu


def _close(got, want, tol, what=""):
    np.testing.assert_allclose(got, want, rtol=0, atol=tol * max(float(np.abs(want).max()), 1e-30), err_msg=what)


@pytest.mark.parametrize("name", ["f32", "cut_f32", "bf16", "wide_bf16"])
def test_tail_equals_the_reference(name: str) -> None:
    """Through autograd, in the replay's own shapes ``[R, K, d]``: the candidate, the record and the four gradients."""
    from hsn_b200.kernels.tail import candidate_tail

    z = load_golden(f"replay_{name}")
    bf = "bf16" in name
    tol = 2e-2 if bf else 1e-5
    x = dev(z["unit_out"])
    x = (x.to(torch.bfloat16) if bf else x).requires_grad_(True)
    alpha = dev(z["alpha"]).requires_grad_(True)
    w_out, cand_w = dev(z["w_W_out.weight"]).requires_grad_(True), dev(z["w_cand_norm.weight"]).requires_grad_(True)
    record: dict = {}
    c = candidate_tail(x, alpha, w_out, cand_w, eps=float(z["cand_eps"]), record=record, prod="bf16" if bf else "fp32")
    assert c.dtype == torch.float32 and tuple(c.shape) == z["c"].shape and not record["y"].requires_grad
    _close(to_np(record["y"]), z["rec_y"], tol, "y")
    _close(to_np(c.detach()), z["c"], tol, "c")
    if bf:   # one bfloat16 rounding of a float32 sum: all but a few equal the reference's to the bit
        assert float(np.mean(to_np(record["y"]) == z["rec_y"])) > 0.98
    (c * dev(z["d_c"])).sum().backward()
    assert x.grad.dtype == x.dtype
    _close(to_np(x.grad.float()), z["d_unit_out"], tol, "d_unit_out")
    _close(to_np(alpha.grad), z["d_alpha"], tol, "d_alpha")
    _close(to_np(w_out.grad), z["g_W_out.weight"], tol, "d_W_out")
    _close(to_np(cand_w.grad), z["g_cand_norm.weight"], tol, "d_cand_w")
    if name == "cut_f32":
        cut = ~z["valid"]
        assert cut.any() and not np.any(to_np(c.detach())[cut]) and not np.any(to_np(x.grad)[cut])


def _case(rng, P, d, bf):
    f = lambda *s, scale=1.0: (rng.standard_normal(s) * scale).astype(np.float32)  # noqa: E731
    x = f(P, d, scale=0.6)
    if bf:
        x = TO.bf16_round(x)
    alpha = np.where(rng.random(P) < 0.1, 0.0, 1.0 + 0.2 * rng.standard_normal(P)).astype(np.float32)
    return x, alpha, f(d, d, scale=1.0 / np.sqrt(d)), (1.0 + f(d, scale=0.2)), f(P, d)


@pytest.mark.parametrize("prod", ["bf16", "fp32"])
@pytest.mark.parametrize("P,d", [(8 * 41, 64), (1, 16), (67, 32), (200, 128), (64 * 300 + 5, 64)])
def test_tail_equals_the_oracle(prod: str, P: int, d: int) -> None:
    """The benchmark's width, one slot, a ragged last tile, the widest model, more tiles than resident blocks."""
    from hsn_b200.kernels.tail import tail_backward, tail_forward

    bf = prod == "bf16"
    tol = 2e-2 if bf else 1e-5
    x, alpha, w, g, d_c = _case(np.random.default_rng(P + d), P, d, bf)
    c, y = tail_forward(dev(x), dev(alpha), dev(w), dev(g), prod=prod)
    want_c, want_y = TO.forward_tail(x, alpha, w, g, bf16=bf)
    _close(to_np(y), want_y, tol, "y")
    _close(to_np(c), want_c, tol, "c")
    got = tail_backward(dev(x), dev(alpha), dev(w), dev(g), dev(want_y), dev(d_c), prod=prod)
    want = TO.backward_tail(x, alpha, w, g, want_y, d_c, bf16=bf)
    for a, b, what in zip(got, want, ("d_unit_out", "d_alpha", "d_w_out", "d_cand_w"), strict=True):
        _close(to_np(a.float()), b, tol, what)


def test_tail_against_pytorch_on_the_device() -> None:
    """The same three lines written with PyTorch's own modules under autocast on the GPU, at the benchmark's width."""
    from hsn_b200.kernels.tail import candidate_tail

    d, P = 64, 4096
    gen = torch.Generator(device="cuda").manual_seed(3)
    lin = torch.nn.Linear(d, d, bias=False, device="cuda")
    norm = torch.nn.RMSNorm(d, eps=1e-6, device="cuda")
    with torch.no_grad():
        norm.weight.add_(0.2 * torch.randn(d, device="cuda", generator=gen))
    x = (0.6 * torch.randn(P, d, device="cuda", generator=gen)).to(torch.bfloat16)
    alpha = 1.0 + 0.2 * torch.randn(P, device="cuda", generator=gen)
    d_c = torch.randn(P, d, device="cuda", generator=gen)
    xr, ar = x.clone().requires_grad_(True), alpha.clone().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = lin(xr).to(torch.float32)
    ref = torch.tanh(ar[:, None] * norm(y))
    (ref * d_c).sum().backward()
    xm, am = x.clone().requires_grad_(True), alpha.clone().requires_grad_(True)
    w, g = lin.weight.detach().clone().requires_grad_(True), norm.weight.detach().clone().requires_grad_(True)
    mine = candidate_tail(xm, am, w, g, prod="bf16")
    (mine * d_c).sum().backward()
    _close(to_np(mine.detach()), to_np(ref.detach()), 2e-2, "c")
    for a, b, what in ((xm.grad, xr.grad, "d_unit_out"), (am.grad, ar.grad, "d_alpha"), (w.grad, lin.weight.grad, "d_W_out"),
                       (g.grad, norm.weight.grad, "d_cand_w")):  # fmt: skip
        _close(to_np(a.float()), to_np(b.float()), 2e-2, what)


def test_tail_at_the_full_window() -> None:
    """The benchmark's 65,536 slots: the same bits on a second run, slots independent of their neighbours (a
    permutation of the slots permutes ``c``, ``y``, ``d_unit_out`` and ``d_alpha``), gradients linear in the cotangent."""
    from hsn_b200.kernels.tail import tail_backward, tail_forward

    P, d = 32 * 256 * 8, 64
    gen = torch.Generator(device="cuda").manual_seed(9)
    x = (0.6 * torch.randn(P, d, device="cuda", generator=gen)).to(torch.bfloat16)
    alpha = (torch.rand(P, device="cuda", generator=gen) > 0.1).float()
    w = torch.randn(d, d, device="cuda", generator=gen) / 8
    g = 1.0 + 0.2 * torch.randn(d, device="cuda", generator=gen)
    d_c = torch.randn(P, d, device="cuda", generator=gen)
    c, y = tail_forward(x, alpha, w, g)
    c2, y2 = tail_forward(x, alpha, w, g)
    assert torch.equal(c, c2) and torch.equal(y, y2) and bool(torch.isfinite(c).all())
    assert not bool(c[alpha == 0].any())
    grads = tail_backward(x, alpha, w, g, y, d_c)
    again = tail_backward(x, alpha, w, g, y, d_c)
    assert all(torch.equal(a, b) for a, b in zip(grads, again, strict=True))
    perm = torch.randperm(P, device="cuda", generator=gen)
    cp, yp = tail_forward(x[perm], alpha[perm], w, g)
    assert torch.equal(cp, c[perm]) and torch.equal(yp, y[perm])
    gp = tail_backward(x[perm], alpha[perm], w, g, y[perm], d_c[perm])
    assert torch.equal(gp[0], grads[0][perm]) and torch.equal(gp[1], grads[1][perm])
    _close(to_np(gp[2]), to_np(grads[2]), 2e-2, "d_W_out under a permutation")
    _close(to_np(gp[3]), to_np(grads[3]), 1e-4, "d_cand_w under a permutation")
    twice = tail_backward(x, alpha, w, g, y, 2 * d_c)
    assert torch.equal(twice[0].float(), 2 * grads[0].float()) and torch.equal(twice[1], 2 * grads[1])
    assert torch.equal(twice[2], 2 * grads[2]) and torch.equal(twice[3], 2 * grads[3])


def test_tail_refuses_what_it_does_not_take() -> None:
    from hsn_b200.kernels.tail import tail_forward

    x, a = torch.zeros(4, 24, device="cuda"), torch.ones(4, device="cuda")
    with pytest.raises(ValueError):
        tail_forward(x, a, torch.zeros(24, 24, device="cuda"), torch.ones(24, device="cuda"))
    with pytest.raises(ValueError):
        tail_forward(torch.zeros(4, 16, device="cuda"), torch.ones(5, device="cuda"), torch.zeros(16, 16, device="cuda"),
                     torch.ones(16, device="cuda"))  # fmt: skip
    with pytest.raises(RuntimeError):
        tail_forward(torch.zeros(4, 16), torch.ones(4), torch.zeros(16, 16), torch.ones(16))
