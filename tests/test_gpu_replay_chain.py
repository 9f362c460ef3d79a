"""``PDGCell.replay_sparse`` composed of this library's four autograd functions (``gathered_inputs`` -> ``norm_gate``
-> ``forward_grouped`` -> ``candidate_tail``), against the reference's own call inside a split window under bf16
autocast (``tests/golden/replay_*_bf16.npz``): the results ``(c, b)``, the record, and for the reference's cotangents of
``(c, b)`` the gradients of ``u``, ``eps``, the slot weights, the padded edge weights and every parameter of the cell."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import dev, load_golden, to_np

pytestmark = pytest.mark.gpu

TOL = 2e-2


def _close(got, want, tol, what=""):
    np.testing.assert_allclose(got, want, rtol=0, atol=tol * max(float(np.abs(want).max()), 1e-30), err_msg=what)


@pytest.mark.parametrize("name", ["bf16", "wide_bf16"])
def test_the_cell_pass_from_its_gathered_inputs_equals_the_reference(name: str) -> None:
    from hsn_b200.kernels.gate import norm_gate
    from hsn_b200.kernels.tail import candidate_tail
    from hsn_b200.kernels.units import forward_grouped

    z = load_golden(f"replay_{name}")
    R, K, F = z["v_raw"].shape
    d = F // 4
    names = ("norm.weight", "gate.weight", "gate.bias", "units.W1", "units.b1", "units.W2", "units.b2", "W_out.weight", "cand_norm.weight")
    w = {k: dev(z["w_" + k]).requires_grad_(True) for k in names}
    v_raw = dev(z["v_raw"]).requires_grad_(True)
    alpha = dev(z["alpha"]).requires_grad_(True)
    units = dev(np.where(z["valid"], z["units"], 0))
    record: dict = {}
    # cell.py:707-721 with this library's functions in place of the modules
    v, b = norm_gate(v_raw, w["norm.weight"], w["gate.weight"], w["gate.bias"], eps=float(z["norm_eps"]), record=record)
    unit_out = forward_grouped(v.reshape(R * K, F), units.reshape(R * K), w["units.W1"], w["units.b1"], w["units.W2"], w["units.b2"],
                               record=record, prod="bf16").reshape(R, K, d)  # fmt: skip
    c = candidate_tail(unit_out, alpha, w["W_out.weight"], w["cand_norm.weight"], eps=float(z["cand_eps"]), record=record, prod="bf16")
    _close(to_np(c.detach()), z["c"], TOL, "c")
    _close(to_np(b.detach()), z["b"], TOL, "b")
    _close(to_np(unit_out.detach().float()), z["unit_out"], TOL, "unit_out")
    for key in ("y", "gate_pre", "rms", "hidden"):
        _close(to_np(record[key].float()).reshape(z["rec_" + key].shape), z["rec_" + key], TOL, "record " + key)
    ((c * dev(z["d_c"])).sum() + (b * dev(z["d_b"])).sum()).backward()
    _close(to_np(v_raw.grad), z["d_v_raw"], TOL, "d_v_raw")
    _close(to_np(alpha.grad), z["d_alpha"], TOL, "d_alpha")
    for k in names:
        _close(to_np(w[k].grad), z["g_" + k], TOL, "gradient of " + k)


@pytest.mark.parametrize("name", ["bf16", "wide_bf16"])
def test_the_whole_cell_pass_equals_the_reference(name: str) -> None:
    """``replay_sparse(u, eps, h_read, sel, record=record)`` (``cell.py:655-734``) from its arguments to ``(c, b)``."""
    from hsn_b200.kernels.gate import norm_gate
    from hsn_b200.kernels.messages import gathered_inputs
    from hsn_b200.kernels.tail import candidate_tail
    from hsn_b200.kernels.units import forward_grouped

    z = load_golden(f"replay_{name}")
    R, K, F = z["v_raw"].shape
    d = F // 4
    names = ("V.weight", "norm.weight", "gate.weight", "gate.bias", "units.W1", "units.b1", "units.W2", "units.b2", "W_out.weight",
             "cand_norm.weight")  # fmt: skip
    w = {k: dev(z["w_" + k]).requires_grad_(True) for k in names}
    u, eps, alpha, edge_w = (dev(z[k]).requires_grad_(True) for k in ("u", "eps", "alpha", "edge_w"))
    cells = dev(np.where(z["valid"], z["cells"], 0))
    units = dev(np.where(z["valid"], z["units"], 0))
    record: dict = {}
    v_raw = gathered_inputs(u, eps, dev(z["h_read"]), cells, dev(z["pad_src"]), edge_w, w["V.weight"])
    v, b = norm_gate(v_raw, w["norm.weight"], w["gate.weight"], w["gate.bias"], eps=float(z["norm_eps"]), record=record)
    unit_out = forward_grouped(v.reshape(R * K, F), units.reshape(R * K), w["units.W1"], w["units.b1"], w["units.W2"], w["units.b2"],
                               record=record, prod="bf16").reshape(R, K, d)  # fmt: skip
    c = candidate_tail(unit_out, alpha, w["W_out.weight"], w["cand_norm.weight"], eps=float(z["cand_eps"]), record=record, prod="bf16")
    record["m"] = v_raw.detach()[..., 3 * d :]
    _close(to_np(c.detach()), z["c"], TOL, "c")
    _close(to_np(b.detach()), z["b"], TOL, "b")
    for key in ("y", "gate_pre", "rms", "hidden", "m"):
        _close(to_np(record[key].float()).reshape(z["rec_" + key].shape), z["rec_" + key], TOL, "record " + key)
    ((c * dev(z["d_c"])).sum() + (b * dev(z["d_b"])).sum()).backward()
    for got, key in ((u.grad, "d_u"), (eps.grad, "d_eps"), (alpha.grad, "d_alpha"), (edge_w.grad, "d_edge_w")):
        _close(to_np(got), z[key], TOL, key)
    for k in names:
        _close(to_np(w[k].grad), z["g_" + k], TOL, "gradient of " + k)
