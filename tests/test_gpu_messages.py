"""The messages and the gathered inputs of the replay's cell pass on the device (``hsnw_messages_forward`` /
``hsnw_messages_backward`` through ``hsn_b200.kernels.messages``): against the reference's fixtures
(``tests/golden/replay_*_bf16.npz``), against the oracle at the benchmark's sizes and at ragged ones, and at the
benchmark's full window through what does not depend on the size."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import dev, load_golden, to_np
from oracle import messages_oracle as MO

pytestmark = pytest.mark.gpu

TOL = 2e-2


def _close(got, want, tol, what=""):
    np.testing.assert_allclose(got, want, rtol=0, atol=tol * max(float(np.abs(want).max()), 1e-30), err_msg=what)


@pytest.mark.parametrize("name", ["bf16", "wide_bf16"])
def test_messages_equal_the_reference(name: str) -> None:
    """Through autograd: ``v_raw`` (its first three blocks are copies: to the bit) and the gradients of ``u``, ``eps``,
    the padded edge weights and ``V`` for the cotangent the reference's own graph sent to ``v_raw``."""
    from hsn_b200.kernels.messages import gathered_inputs

    z = load_golden(f"replay_{name}")
    d = z["u"].shape[-1]
    u, eps, edge_w, v_w = (dev(z[k]).requires_grad_(True) for k in ("u", "eps", "edge_w", "w_V.weight"))
    cells = dev(np.where(z["valid"], z["cells"], 0))
    v_raw = gathered_inputs(u, eps, dev(z["h_read"]), cells, dev(z["pad_src"]), edge_w, v_w)
    got = to_np(v_raw.detach())
    assert got.shape == z["v_raw"].shape and np.array_equal(got[..., : 3 * d], z["v_raw"][..., : 3 * d])
    _close(got[..., 3 * d :], z["rec_m"], TOL, "m")
    assert float(np.mean(got[..., 3 * d :] == z["rec_m"])) > 0.95   # bfloat16 roundings of float32 sums
    (v_raw * dev(z["d_v_raw"])).sum().backward()
    _close(to_np(u.grad), z["d_u"], 1e-5, "d_u")
    _close(to_np(eps.grad), z["d_eps"], 1e-5, "d_eps")
    _close(to_np(edge_w.grad), z["d_edge_w"], TOL, "d_edge_w")
    _close(to_np(v_w.grad), z["g_V.weight"], TOL, "d_V")


def _case(rng, R, N, d, K, D):
    f = lambda *s, scale=1.0: (rng.standard_normal(s) * scale).astype(np.float32)  # noqa: E731
    cells = np.stack([rng.permutation(N)[:K] if K <= N else rng.integers(0, N, K) for _ in range(R)]).astype(np.int64)
    cells[rng.random((R, K)) < 0.1] = 0   # padded slots
    pad_src = rng.integers(0, N, (N, D)).astype(np.int64)
    edge_w = rng.random((N, D)).astype(np.float32)
    edge_w[rng.random((N, D)) < 0.15] = 0.0   # padding
    return f(R, d, scale=0.7), f(R, d, scale=0.4), f(R, N, d, scale=0.5), cells, pad_src, edge_w, f(d, d, scale=d**-0.5), f(R, K, 4 * d)


@pytest.mark.parametrize("R,N,d,K,D", [(40, 256, 64, 8, 4), (3, 7, 16, 1, 1), (5, 33, 32, 3, 3), (300, 64, 64, 8, 2), (3, 2100, 16, 6, 2)])
def test_messages_equal_the_oracle(R: int, N: int, d: int, K: int, D: int) -> None:
    """The benchmark's model, one slot and one neighbour, a ragged tile with three neighbours, more tiles than
    resident blocks, a graph too large for a block's table of edge sums (the scan per cell)."""
    from hsn_b200.kernels.messages import messages_backward, messages_forward

    u, eps, h, cells, pad_src, edge_w, v_w, d_v_raw = _case(np.random.default_rng(R + N + d), R, N, d, K, D)
    v_raw = to_np(messages_forward(dev(u), dev(eps), dev(h), dev(cells), dev(pad_src), dev(edge_w), dev(v_w)))
    want = MO.forward_messages(u, eps, h, cells, pad_src, edge_w, v_w, bf16=True)
    assert np.array_equal(v_raw[..., : 3 * d], want[..., : 3 * d])
    _close(v_raw[..., 3 * d :], want[..., 3 * d :], TOL, "m")
    got = messages_backward(dev(h), dev(cells), dev(pad_src), dev(edge_w), dev(v_w), dev(d_v_raw))
    wantb = MO.backward_messages(h, cells, pad_src, edge_w, v_w, d_v_raw, bf16=True)
    for a, w, tol, what in zip(got, wantb, (1e-5, 1e-5, TOL, TOL), ("d_u", "d_eps", "d_edge_w", "d_V"), strict=True):
        _close(to_np(a), w, tol, what)


def test_messages_at_the_full_window() -> None:
    """The benchmark's 8192 positions x 8 slots on a recorded state of 537 MB: the same bits on a second run, the
    gradients linear in the cotangent, a row's results independent of the other rows."""
    from hsn_b200.kernels.messages import messages_backward, messages_forward

    R, N, d, K, D = 32 * 256, 256, 64, 8, 4
    gen = torch.Generator(device="cuda").manual_seed(13)
    f = lambda *s, scale=1.0: torch.randn(*s, device="cuda", generator=gen) * scale  # noqa: E731
    u, eps, h = f(R, d, scale=0.7), f(R, d, scale=0.4), f(R, N, d, scale=0.5)
    cells = torch.rand(R, N, device="cuda", generator=gen).argsort(dim=1)[:, :K].contiguous()
    pad_src = torch.randint(0, N, (N, D), device="cuda", generator=gen)
    edge_w = torch.softmax(f(N, D), dim=1)
    v_w, d_v_raw = f(d, d, scale=d**-0.5), f(R, K, 4 * d)
    v_raw = messages_forward(u, eps, h, cells, pad_src, edge_w, v_w)
    assert torch.equal(v_raw, messages_forward(u, eps, h, cells, pad_src, edge_w, v_w)) and bool(torch.isfinite(v_raw).all())
    assert torch.equal(v_raw[:, :, :d], u[:, None].expand(R, K, d)) and torch.equal(v_raw[:, :, 2 * d : 3 * d], h.gather(1, cells[..., None].expand(R, K, d)))
    half = R // 2
    assert torch.equal(messages_forward(u[half:], eps[half:], h[half:], cells[half:], pad_src, edge_w, v_w), v_raw[half:])
    grads = messages_backward(h, cells, pad_src, edge_w, v_w, d_v_raw)
    assert all(torch.equal(a, b) for a, b in zip(grads, messages_backward(h, cells, pad_src, edge_w, v_w, d_v_raw), strict=True))
    twice = messages_backward(h, cells, pad_src, edge_w, v_w, 2 * d_v_raw)
    assert all(torch.equal(a, 2 * b) for a, b in zip(twice, grads, strict=True))


def test_messages_refuse_what_they_do_not_take() -> None:
    from hsn_b200.kernels.messages import messages_forward

    z = torch.zeros
    with pytest.raises(ValueError):   # five in-neighbours
        messages_forward(z(2, 16, device="cuda"), z(2, 16, device="cuda"), z(2, 8, 16, device="cuda"), z(2, 1, dtype=torch.int64, device="cuda"),
                         z(8, 5, dtype=torch.int64, device="cuda"), z(8, 5, device="cuda"), z(16, 16, device="cuda"))  # fmt: skip
    with pytest.raises(ValueError):   # the widest model
        messages_forward(z(2, 128, device="cuda"), z(2, 128, device="cuda"), z(2, 8, 128, device="cuda"), z(2, 1, dtype=torch.int64, device="cuda"),
                         z(8, 2, dtype=torch.int64, device="cuda"), z(8, 2, device="cuda"), z(128, 128, device="cuda"))  # fmt: skip
    with pytest.raises(RuntimeError):
        messages_forward(z(2, 16), z(2, 16), z(2, 8, 16), z(2, 1, dtype=torch.int64), z(8, 2, dtype=torch.int64), z(8, 2), z(16, 16))
