"""The replay's scorer logits on the device (``hsnw_scorer_logits`` / ``hsnw_scorer_logits_backward`` through
``hsn_b200.kernels.scorer``): against the reference's fixtures (``tests/golden/scorer_*.npz``: ``_scorer_logits`` with
autograd on the CPU, float32 and under bf16 autocast), against the oracle at the benchmark's sizes and at ragged
ones, and at the benchmark's full window through what does not depend on the size."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import dev, load_golden, to_np
from oracle import scorer_oracle as SO

pytestmark = pytest.mark.gpu

FEATURES = ("u", "eps", "h", "age", "scalars")


def _close(got, want, tol, what=""):
    np.testing.assert_allclose(got, want, rtol=0, atol=tol * max(float(np.abs(want).max()), 1e-30), err_msg=what)


@pytest.mark.parametrize("name", ["f32", "bf16"])
def test_scorer_logits_equal_the_reference(name: str) -> None:
    """Through autograd, as the replay calls it: the logits and the gradients of the weight and the bias."""
    from hsn_b200.kernels.scorer import scorer_logits

    z = load_golden(f"scorer_{name}")
    bf = name == "bf16"
    tol = 2e-2 if bf else 1e-5
    weight, bias = dev(z["weight"]).requires_grad_(True), dev(z["bias"]).requires_grad_(True)
    out = scorer_logits(weight, bias, *(dev(z[k]) for k in FEATURES), age_max=float(z["age_max"]), prod="bf16" if bf else "fp32")
    assert out.dtype == torch.float32 and tuple(out.shape) == z["logits"].shape
    _close(to_np(out.detach()), z["logits"], tol, "logits")
    if bf:   # sums of three bfloat16 values: all but a few equal the reference's to the bit
        assert float(np.mean(to_np(out.detach()) == z["logits"])) > 0.9
    (out * dev(z["cot"])).sum().backward()
    _close(to_np(weight.grad), z["d_weight"], tol, "d_weight")
    _close(to_np(bias.grad), z["d_bias"], tol, "d_bias")
    d = z["h"].shape[-1]
    for lo, hi, what in ((0, 2 * d, "row block"), (2 * d, 3 * d, "state block"), (3 * d, None, "tail block")):
        _close(to_np(weight.grad)[:, lo:hi], z["d_weight"][:, lo:hi], tol, what)


def _case(rng, R, N, d, M, S, bf):
    f = lambda *s, scale=1.0: (rng.standard_normal(s) * scale).astype(np.float32)  # noqa: E731
    weight, bias = f(M, 3 * d + 1 + S, scale=0.2), f(M, scale=0.3)
    feats = [f(R, d, scale=0.7), f(R, d, scale=0.4), f(R, N, d, scale=0.5), rng.integers(0, 300, (R, N)), f(R, N, S)]
    cot = f(R, N, M)
    return weight, bias, feats, cot


@pytest.mark.parametrize("prod", ["bf16", "fp32"])
@pytest.mark.parametrize("R,N,d,M,S", [(40, 256, 64, 8, 9), (3, 200, 32, 5, 11), (7, 1, 16, 1, 0), (2, 300, 128, 8, 9)])
def test_scorer_logits_equal_the_oracle(prod: str, R: int, N: int, d: int, M: int, S: int) -> None:
    """The benchmark's model, a ragged last tile with fewer units and more scalars, one cell and one unit and no
    scalars, the widest model's state."""
    from hsn_b200.kernels.scorer import scorer_logits_backward, scorer_logits_forward

    bf = prod == "bf16"
    tol = 2e-2 if bf else 1e-5
    weight, bias, feats, cot = _case(np.random.default_rng(R + N), R, N, d, M, S, bf)
    want = SO.scorer_logits(weight, bias, *feats, 100.0, bf16=bf)
    got = scorer_logits_forward(dev(weight), dev(bias), *map(dev, feats), age_max=100.0, prod=prod)
    _close(to_np(got), want, tol, "logits")
    want_w, want_b = SO.scorer_logits_backward(weight, *feats, 100.0, cot, bf16=bf)
    got_w, got_b = scorer_logits_backward(dev(weight), dev(bias), *map(dev, feats), dev(cot), age_max=100.0, prod=prod)
    _close(to_np(got_w), want_w, tol, "d_weight")
    _close(to_np(got_b), want_b, tol, "d_bias")
    assert want.shape == (R, N, M)


def test_edges_and_refusals() -> None:
    from hsn_b200.kernels.scorer import scorer_logits, scorer_logits_forward

    rng = np.random.default_rng(2)
    weight, bias, feats, _ = _case(rng, 4, 64, 32, 3, 9, True)
    with pytest.raises(ValueError):
        scorer_logits_forward(dev(weight[:, :-1]), dev(bias), *map(dev, feats), age_max=10.0)
    with pytest.raises(RuntimeError):
        scorer_logits_forward(*map(torch.from_numpy, (weight, bias, *feats)), age_max=10.0)
    u = dev(feats[0]).requires_grad_(True)   # a feature with a gradient: the replay detaches them, the function refuses
    out = scorer_logits(dev(weight).requires_grad_(True), dev(bias), u, *map(dev, feats[1:]), age_max=10.0)
    with pytest.raises(RuntimeError):
        out.sum().backward()


@pytest.mark.parametrize("prod", ["bf16", "fp32"])
def test_full_window(prod: str) -> None:
    """The benchmark's window (8192 positions x 256 cells, d 64, 8 units): a sample of positions against the oracle;
    the gradients are linear in the cotangent, additive over a split of the positions, and two runs give the same
    bits."""
    from hsn_b200.kernels.scorer import scorer_logits_backward, scorer_logits_forward

    bf = prod == "bf16"
    tol = 2e-2 if bf else 1e-5
    R, N, d, M, Sn = 32 * 256, 256, 64, 8, 9
    gen = torch.Generator(device="cuda").manual_seed(3)
    f = lambda *s, scale=1.0: torch.randn(*s, generator=gen, device="cuda") * scale  # noqa: E731
    weight, bias = f(M, 3 * d + 1 + Sn, scale=0.2), f(M, scale=0.3)
    feats = [f(R, d, scale=0.7), f(R, d, scale=0.4), f(R, N, d, scale=0.5),
             torch.randint(0, 300, (R, N), generator=gen, device="cuda"), f(R, N, Sn)]  # fmt: skip
    cot = f(R, N, M)
    out = scorer_logits_forward(weight, bias, *feats, age_max=100.0, prod=prod)
    rows = torch.tensor([0, 1, 4095, 8190, 8191], device="cuda")
    want = SO.scorer_logits(to_np(weight), to_np(bias), *(to_np(t[rows]) for t in feats), 100.0, bf16=bf)
    _close(to_np(out[rows]), want, tol, "logits")
    gw, gb = scorer_logits_backward(weight, bias, *feats, cot, age_max=100.0, prod=prod)
    again = scorer_logits_backward(weight, bias, *feats, cot, age_max=100.0, prod=prod)
    assert torch.equal(again[0], gw) and torch.equal(again[1], gb)
    half = R // 2
    a = scorer_logits_backward(weight, bias, *(t[:half] for t in feats), cot[:half], age_max=100.0, prod="fp32")
    b = scorer_logits_backward(weight, bias, *(t[half:] for t in feats), cot[half:], age_max=100.0, prod="fp32")
    whole = scorer_logits_backward(weight, bias, *feats, cot, age_max=100.0, prod="fp32")
    _close(to_np(a[0] + b[0]), to_np(whole[0]), 1e-4, "additive")
    twice = scorer_logits_backward(weight, bias, *feats, 2 * cot, age_max=100.0, prod="fp32")
    assert torch.equal(twice[0], 2 * whole[0]) and torch.equal(twice[1], 2 * whole[1])
    sample = SO.scorer_logits_backward(to_np(weight), *(to_np(t[:64]) for t in feats), 100.0, to_np(cot[:64]), bf16=bf)
    got = scorer_logits_backward(weight, bias, *(t[:64] for t in feats), cot[:64], age_max=100.0, prod=prod)
    _close(to_np(got[0]), sample[0], tol, "d_weight of 64 positions")
    _close(to_np(got[1]), sample[1], tol, "d_bias of 64 positions")
