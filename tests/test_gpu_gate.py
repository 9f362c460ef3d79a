"""The cell norm and the gate of the replay's cell pass on the device (``hsnw_gate_forward`` / ``hsnw_gate_backward``
through ``hsn_b200.kernels.gate``): against the reference's fixtures (``tests/golden/replay_*_bf16.npz``:
``replay_sparse`` inside a split window under bf16 autocast on the CPU), against the oracle at the benchmark's sizes and
at ragged ones, against PyTorch's own modules on the GPU, and at the benchmark's full window through what does not
depend on the size."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import dev, load_golden, to_np
from oracle import gate_oracle as GO

pytestmark = pytest.mark.gpu

TOL = 2e-2


def _close(got, want, tol, what=""):
    np.testing.assert_allclose(got, want, rtol=0, atol=tol * max(float(np.abs(want).max()), 1e-30), err_msg=what)


@pytest.mark.parametrize("name", ["bf16", "wide_bf16"])
def test_norm_and_gate_equal_the_reference(name: str) -> None:
    """Through autograd, in the replay's own shapes ``[R, K, 4d]``: ``v``, ``b``, the record and the four gradients for
    the cotangents the reference's own graph sent to ``v`` (the unit pass's) and to ``b``."""
    from hsn_b200.kernels.gate import norm_gate

    z = load_golden(f"replay_{name}")
    x = dev(z["v_raw"]).requires_grad_(True)
    nw, gw, gb = (dev(z[k]).requires_grad_(True) for k in ("w_norm.weight", "w_gate.weight", "w_gate.bias"))
    record: dict = {}
    v, b = norm_gate(x, nw, gw, gb, eps=float(z["norm_eps"]), record=record)
    assert v.dtype == torch.float32 and tuple(v.shape) == z["v"].shape and tuple(b.shape) == z["b"].shape
    _close(to_np(v.detach()), z["v"], 1e-5, "v")
    _close(to_np(record["rms"]), z["rec_rms"], 1e-5, "rms")
    _close(to_np(record["gate_pre"]), z["rec_gate_pre"], TOL, "gate_pre")
    _close(to_np(b.detach()), z["b"], TOL, "b")
    assert float(np.mean(to_np(record["gate_pre"]) == z["rec_gate_pre"])) > 0.95   # one bfloat16 rounding of a float32 sum
    ((v * dev(z["d_v_units"]).reshape(v.shape)).sum() + (b * dev(z["d_b"])).sum()).backward()   # (the unit pass saw v as [R K, 4d])
    _close(to_np(x.grad), z["d_v_raw"], TOL, "d_v_raw")
    _close(to_np(nw.grad), z["g_norm.weight"], TOL, "d_norm_w")
    _close(to_np(gw.grad), z["g_gate.weight"], TOL, "d_gate_w")
    _close(to_np(gb.grad), z["g_gate.bias"], TOL, "d_gate_b")


def _case(rng, P, d):
    f = lambda *s, scale=1.0: (rng.standard_normal(s) * scale).astype(np.float32)  # noqa: E731
    F = 4 * d
    return f(P, F, scale=0.8), 1.0 + f(F, scale=0.2), f(d, F, scale=F**-0.5), f(d, scale=0.3), f(P, F), f(P, d)


@pytest.mark.parametrize("P,d", [(8 * 41, 64), (1, 16), (67, 32), (128 * 150 + 5, 64), (128 * 300 + 77, 32)])
def test_norm_and_gate_equal_the_oracle(P: int, d: int) -> None:
    """The benchmark's width, one slot, a ragged last tile, more tiles than resident blocks at both block counts."""
    from hsn_b200.kernels.gate import norm_gate_backward, norm_gate_forward

    x, nw, gw, gb, d_v, d_b = _case(np.random.default_rng(P + d), P, d)
    v, rms, gp, b = norm_gate_forward(dev(x), dev(nw), dev(gw), dev(gb))
    want = GO.forward_norm_gate(x, nw, gw, gb, norm_eps=1e-6, bf16=True)
    for got, w, tol, what in zip((v, rms, gp, b), want, (1e-5, 1e-5, TOL, TOL), ("v", "rms", "gate_pre", "b"), strict=True):
        _close(to_np(got), w, tol, what)
    got = norm_gate_backward(dev(x), dev(nw), dev(gw), dev(gb), dev(want[2]), dev(d_v), dev(d_b))
    wantb = GO.backward_norm_gate(x, nw, gw, gb, d_v, d_b, norm_eps=1e-6, bf16=True)
    for a, w, what in zip(got, wantb, ("d_v_raw", "d_norm_w", "d_gate_w", "d_gate_b"), strict=True):
        _close(to_np(a), w, TOL, what)
    _close(to_np(got[0]), wantb[0], 1e-3, "d_v_raw (float32 but for the gate's bfloat16 share)")


def test_norm_and_gate_against_pytorch_on_the_device() -> None:
    """The same lines written with PyTorch's own modules under autocast on the GPU, at the benchmark's width."""
    from hsn_b200.kernels.gate import norm_gate

    d, P = 64, 4096
    F = 4 * d
    gen = torch.Generator(device="cuda").manual_seed(5)
    norm = torch.nn.RMSNorm(F, eps=1e-6, device="cuda")
    gate = torch.nn.Linear(F, d, device="cuda")
    with torch.no_grad():
        norm.weight.add_(0.2 * torch.randn(F, device="cuda", generator=gen))
    x = 0.8 * torch.randn(P, F, device="cuda", generator=gen)
    d_v, d_b = torch.randn(P, F, device="cuda", generator=gen), torch.randn(P, d, device="cuda", generator=gen)
    xr = x.clone().requires_grad_(True)
    vr = norm(xr)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        gp = gate(vr).to(torch.float32)
    br = torch.sigmoid(gp)
    ((vr * d_v).sum() + (br * d_b).sum()).backward()
    xm = x.clone().requires_grad_(True)
    nw, gw, gb = (t.detach().clone().requires_grad_(True) for t in (norm.weight, gate.weight, gate.bias))
    v, b = norm_gate(xm, nw, gw, gb)
    ((v * d_v).sum() + (b * d_b).sum()).backward()
    _close(to_np(v.detach()), to_np(vr.detach()), 1e-5, "v")
    _close(to_np(b.detach()), to_np(br.detach()), TOL, "b")
    for a, w, what in ((xm.grad, xr.grad, "d_v_raw"), (nw.grad, norm.weight.grad, "d_norm_w"), (gw.grad, gate.weight.grad, "d_gate_w"),
                       (gb.grad, gate.bias.grad, "d_gate_b")):  # fmt: skip
        _close(to_np(a), to_np(w), TOL, what)


def test_norm_and_gate_at_the_full_window() -> None:
    """The benchmark's 65,536 slots: the same bits on a second run, slots independent of their neighbours (a
    permutation of the slots permutes the per-slot results to the bit), gradients linear in the cotangents."""
    from hsn_b200.kernels.gate import norm_gate_backward, norm_gate_forward

    P, d = 32 * 256 * 8, 64
    F = 4 * d
    gen = torch.Generator(device="cuda").manual_seed(11)
    x = 0.8 * torch.randn(P, F, device="cuda", generator=gen)
    nw = 1.0 + 0.2 * torch.randn(F, device="cuda", generator=gen)
    gw, gb = torch.randn(d, F, device="cuda", generator=gen) / 16, 0.3 * torch.randn(d, device="cuda", generator=gen)
    d_v, d_b = torch.randn(P, F, device="cuda", generator=gen), torch.randn(P, d, device="cuda", generator=gen)
    out = norm_gate_forward(x, nw, gw, gb)
    again = norm_gate_forward(x, nw, gw, gb)
    assert all(torch.equal(a, b) for a, b in zip(out, again, strict=True)) and all(bool(torch.isfinite(t).all()) for t in out)
    grads = norm_gate_backward(x, nw, gw, gb, out[2], d_v, d_b)
    assert all(torch.equal(a, b) for a, b in zip(grads, norm_gate_backward(x, nw, gw, gb, out[2], d_v, d_b), strict=True))
    perm = torch.randperm(P, device="cuda", generator=gen)
    outp = norm_gate_forward(x[perm], nw, gw, gb)
    assert all(torch.equal(a, b[perm]) for a, b in zip(outp, out, strict=True))
    gp = norm_gate_backward(x[perm], nw, gw, gb, out[2][perm], d_v[perm], d_b[perm])
    assert torch.equal(gp[0], grads[0][perm])
    for a, b, what in zip(gp[1:], grads[1:], ("d_norm_w", "d_gate_w", "d_gate_b"), strict=True):
        _close(to_np(a), to_np(b), TOL, what + " under a permutation")
    twice = norm_gate_backward(x, nw, gw, gb, out[2], 2 * d_v, 2 * d_b)
    assert all(torch.equal(a, 2 * b) for a, b in zip(twice, grads, strict=True))


def test_norm_and_gate_refuse_what_they_do_not_take() -> None:
    from hsn_b200.kernels.gate import norm_gate_forward

    with pytest.raises(ValueError):   # the widest model keeps the reference's lines
        norm_gate_forward(torch.zeros(4, 512, device="cuda"), torch.ones(512, device="cuda"), torch.zeros(128, 512, device="cuda"),
                          torch.zeros(128, device="cuda"))  # fmt: skip
    with pytest.raises(ValueError):
        norm_gate_forward(torch.zeros(4, 60, device="cuda"), torch.ones(64, device="cuda"), torch.zeros(16, 64, device="cuda"),
                          torch.zeros(16, device="cuda"))  # fmt: skip
    with pytest.raises(RuntimeError):
        norm_gate_forward(torch.zeros(4, 64), torch.ones(64), torch.zeros(16, 64), torch.zeros(16))
