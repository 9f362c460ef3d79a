"""The cell norm and the gate of the replay's cell pass with their backward, one launch over every slot of a window:
``v = self.norm(v_raw)``, ``gate_pre = self.gate(v)``, ``b = sigmoid(gate_pre)`` of ``PDGCell.replay_sparse``
(reference ``python/hsn/model/cell.py:707-709``) over this library.

:func:`norm_gate` takes ``norm.weight``, ``gate.weight`` and ``gate.bias`` instead of the modules: ``v_raw [..., 4d]``
-> ``(v [..., 4d], b [..., d])`` float32, ``record["gate_pre"]`` and ``record["rms"]`` as the reference records them
(``cell.py:727-733``), detached. It is an autograd function: the gradients that reach ``v`` (the unit pass's) and ``b``
(the state recurrence's) give the gradients of ``v_raw`` and of the three weights with the values autograd gives the
reference's lines (``hsn_b200/csrc/gate.cu``).

The pass is the one under ``torch.autocast(dtype=torch.bfloat16)`` (the norm in float32, the gate's products in
bfloat16); float32 products and ``d = 128`` are not taken: the call raises and the caller keeps the reference's
lines. There is no CPU or PyTorch path here: without the built library or a CUDA device the call raises.
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch
from torch import Tensor

from .. import _lib

__all__ = ["norm_gate", "norm_gate_forward", "norm_gate_backward"]


def _prepare(device: torch.device) -> Any:
    if device.type != "cuda":
        raise RuntimeError(f"the replay's norm and gate run on a CUDA device, got tensors on {device}")
    lib = _lib.library()
    index = device.index if device.index is not None else torch.cuda.current_device()
    if not lib.hsnw_prepared(index):
        _lib.check(lib.hsnw_prepare(index))
    return lib


def _stream(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _weights(norm_w: Tensor, gate_w: Tensor, gate_b: Tensor, eps: float) -> tuple[_lib.HsnwGate, tuple[Tensor, ...]]:
    if gate_w.dim() != 2 or int(gate_w.shape[1]) != 4 * int(gate_w.shape[0]):
        raise ValueError(f"the gate's weight must be [d, 4d], got {tuple(gate_w.shape)}")
    d = int(gate_w.shape[0])
    if d not in (16, 32, 64):
        raise ValueError(f"the replay's norm and gate take d of 16, 32 or 64, got {d}")
    if tuple(norm_w.shape) != (4 * d,) or tuple(gate_b.shape) != (d,):
        raise ValueError(f"the norm's weight must be [{4 * d}] and the gate's bias [{d}], got {tuple(norm_w.shape)} and {tuple(gate_b.shape)}")
    if norm_w.device != gate_w.device or gate_b.device != gate_w.device:
        raise ValueError("the norm's and the gate's weights must share one device")
    held = tuple(t.detach().to(torch.float32).contiguous() for t in (norm_w, gate_w, gate_b))
    st = _lib.HsnwGate(d=d, prod_bf16=1, norm_eps=float(eps), reserved=0, norm_weight=held[0].data_ptr(), gate_w=held[1].data_ptr(),
                       gate_b=held[2].data_ptr())  # fmt: skip
    return st, held


def _rows(t: Tensor, width: int, name: str) -> Tensor:
    if t.dim() < 1 or int(t.shape[-1]) != width:
        raise ValueError(f"{name} must be [..., {width}], got shape {tuple(t.shape)}")
    return t.detach().to(torch.float32).reshape(-1, width).contiguous()


def norm_gate_forward(v_raw: Tensor, norm_w: Tensor, gate_w: Tensor, gate_b: Tensor, *, eps: float = 1e-6) -> tuple[Tensor, ...]:
    """``hsnw_gate_forward`` without autograd: ``(v [..., 4d], rms [...], gate_pre [..., d], b [..., d])``, float32."""
    st, held = _weights(norm_w, gate_w, gate_b, eps)
    x = _rows(v_raw, 4 * st.d, "v_raw")
    dev = x.device
    lib = _prepare(dev)
    P = int(x.shape[0])
    lead = tuple(v_raw.shape[:-1])
    f32 = torch.float32
    v, rms = torch.empty((P, 4 * st.d), dtype=f32, device=dev), torch.empty((P,), dtype=f32, device=dev)
    gate_pre, b = torch.empty((P, st.d), dtype=f32, device=dev), torch.empty((P, st.d), dtype=f32, device=dev)
    need = int(lib.hsnw_gate_scratch_bytes(ctypes.byref(st), P, 0))
    scratch = torch.empty((max(need, 256),), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.hsnw_gate_forward(ctypes.byref(st), x.data_ptr(), P, v.data_ptr(), rms.data_ptr(), gate_pre.data_ptr(), b.data_ptr(),
                                         scratch.data_ptr(), int(scratch.numel()), _stream(dev)))  # fmt: skip
    del held
    return v.reshape(*lead, 4 * st.d), rms.reshape(lead), gate_pre.reshape(*lead, st.d), b.reshape(*lead, st.d)


def norm_gate_backward(v_raw: Tensor, norm_w: Tensor, gate_w: Tensor, gate_b: Tensor, gate_pre: Tensor, d_v_units: Tensor, d_b: Tensor, *,
                       eps: float = 1e-6) -> tuple[Tensor, Tensor, Tensor, Tensor]:  # fmt: skip
    """``hsnw_gate_backward``: ``(d_v_raw, d_norm_w, d_gate_w, d_gate_b)`` for the cotangents ``d_v_units`` of ``v``
    and ``d_b`` of ``b``, with ``gate_pre`` :func:`norm_gate_forward`'s."""
    st, held = _weights(norm_w, gate_w, gate_b, eps)
    x = _rows(v_raw, 4 * st.d, "v_raw")
    dvu = _rows(d_v_units, 4 * st.d, "d_v_units")
    gp, db = _rows(gate_pre, st.d, "gate_pre"), _rows(d_b, st.d, "d_b")
    dev = x.device
    P = int(x.shape[0])
    for name, t in (("d_v_units", dvu), ("gate_pre", gp), ("d_b", db)):
        if int(t.shape[0]) != P or t.device != dev:
            raise ValueError(f"{name} must hold {P} slots on {dev}, got {int(t.shape[0])} on {t.device}")
    lib = _prepare(dev)
    f32 = torch.float32
    d_x = torch.empty_like(x)
    d_nw, d_gw, d_gb = (torch.empty(t.shape, dtype=f32, device=dev) for t in held)
    need = int(lib.hsnw_gate_scratch_bytes(ctypes.byref(st), P, 1))
    scratch = torch.empty((max(need, 256),), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.hsnw_gate_backward(ctypes.byref(st), x.data_ptr(), gp.data_ptr(), dvu.data_ptr(), db.data_ptr(), P, d_x.data_ptr(),
                                          d_nw.data_ptr(), d_gw.data_ptr(), d_gb.data_ptr(), scratch.data_ptr(), int(scratch.numel()),
                                          _stream(dev)))  # fmt: skip
    del held
    return d_x.reshape(v_raw.shape), d_nw, d_gw, d_gb


class _NormGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, v_raw: Tensor, norm_w: Tensor, gate_w: Tensor, gate_b: Tensor, eps: float) -> tuple[Tensor, ...]:
        v, rms, gate_pre, b = norm_gate_forward(v_raw, norm_w, gate_w, gate_b, eps=eps)
        ctx.save_for_backward(v_raw, norm_w, gate_w, gate_b, gate_pre)
        ctx.eps = eps
        ctx.mark_non_differentiable(rms, gate_pre)
        return v, b, rms, gate_pre

    @staticmethod
    def backward(ctx: Any, d_v: Tensor | None, d_b: Tensor | None, _d_rms: Any, _d_gp: Any) -> tuple[Tensor | None, ...]:
        v_raw, norm_w, gate_w, gate_b, gate_pre = ctx.saved_tensors
        if d_v is None:
            d_v = torch.zeros_like(v_raw, dtype=torch.float32)
        if d_b is None:
            d_b = torch.zeros_like(gate_pre)
        grads = norm_gate_backward(v_raw, norm_w, gate_w, gate_b, gate_pre, d_v, d_b, eps=ctx.eps)
        likes = (v_raw, norm_w, gate_w, gate_b)
        out = [g.to(like.dtype) if wanted else None for g, like, wanted in zip(grads, likes, ctx.needs_input_grad[:4], strict=True)]
        return out[0], out[1], out[2], out[3], None


def norm_gate(v_raw: Tensor, norm_w: Tensor, gate_w: Tensor, gate_b: Tensor, *, eps: float = 1e-6,
              record: dict[str, Tensor] | None = None) -> tuple[Tensor, Tensor]:  # fmt: skip
    """``(v, b)`` = ``(norm(v_raw), sigmoid(gate(norm(v_raw))))`` with autograd through ``v_raw`` and the three
    weights; ``record`` receives ``gate_pre`` and ``rms``."""
    if v_raw.numel() == 0:
        d = int(gate_w.shape[0])
        empty = v_raw.new_zeros((*v_raw.shape[:-1], d), dtype=torch.float32)
        if record is not None:
            record["gate_pre"], record["rms"] = empty, v_raw.new_zeros(v_raw.shape[:-1], dtype=torch.float32)
        return v_raw.new_zeros(v_raw.shape, dtype=torch.float32), empty
    v, b, rms, gate_pre = _NormGate.apply(v_raw, norm_w, gate_w, gate_b, float(eps))
    if record is not None:
        record["gate_pre"], record["rms"] = gate_pre, rms
    return v, b
