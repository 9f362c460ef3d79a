"""The replay's grouped unit pass with its backward, one launch per product over every unit's pairs:
``UnitBank.forward_grouped`` (reference ``python/hsn/model/units.py:356-414``) over this library.

:func:`forward_grouped` takes the unit bank's four stacked parameters instead of the module, otherwise the
reference's arguments and answers: ``v [P, d_in]``, ``unit_idx [P]`` -> ``out [P, d]`` in the input order,
``record["hidden"]`` the first layer's pre-activation of every pair's own unit, detached. It is an autograd
function: ``out.backward(...)`` fills the gradients of ``v``, ``W1``, ``b1``, ``W2``, ``b2`` with the values
autograd gives the reference's pass (``hsn_b200/csrc/units.cu``: the backward's six products and two column sums).

``prod="bf16"`` is the pass under ``torch.autocast(dtype=torch.bfloat16)`` (``out`` and ``record["hidden"]`` are
bfloat16, every product's output is rounded to bfloat16, the parameter gradients are bfloat16 values widened to
float32), ``prod="fp32"`` the pass without autocast. A unit index outside ``[0, M)`` raises ``IndexError`` as in
the reference: one host read of the call's status word, where the reference reads the unit histogram
(``check=False`` leaves the word in ``record["status"]`` unread). There is no CPU or PyTorch path here: without the
built library or a CUDA device the call raises.
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch
from torch import Tensor

from .. import _lib

__all__ = ["forward_grouped", "grouped_forward", "grouped_backward"]


def _prepare(device: torch.device) -> Any:
    if device.type != "cuda":
        raise RuntimeError(f"the grouped unit pass runs on a CUDA device, got tensors on {device}")
    lib = _lib.library()
    index = device.index if device.index is not None else torch.cuda.current_device()
    if not lib.hsnw_prepared(index):
        _lib.check(lib.hsnw_prepare(index))
    return lib


def _stream(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _bank(W1: Tensor, b1: Tensor, W2: Tensor, b2: Tensor, prod: str) -> tuple[_lib.HsnwUnits, tuple[Tensor, ...]]:
    if prod not in ("bf16", "fp32"):
        raise ValueError(f"prod must be 'bf16' or 'fp32', got {prod!r}")
    if W1.dim() != 3 or W2.dim() != 3:
        raise ValueError(f"W1 must be [M, d_in, H] and W2 [M, H, d], got {tuple(W1.shape)} and {tuple(W2.shape)}")
    M, d_in, H = (int(n) for n in W1.shape)
    d = int(W2.shape[2])
    want = {"b1": (b1, (M, H)), "W2": (W2, (M, H, d)), "b2": (b2, (M, d))}
    for name, (t, shape) in want.items():
        if tuple(t.shape) != shape:
            raise ValueError(f"{name} must have shape {shape}, got {tuple(t.shape)}")
    held = tuple(t.detach().to(torch.float32).contiguous() for t in (W1, b1, W2, b2))
    for t in held:
        if t.device != W1.device:
            raise ValueError("the unit bank's parameters must share one device")
    st = _lib.HsnwUnits(n_units=M, d_in=d_in, hidden=H, d_out=d, prod_bf16=int(prod == "bf16"), reserved=0,
                        w1=held[0].data_ptr(), b1=held[1].data_ptr(), w2=held[2].data_ptr(), b2=held[3].data_ptr())  # fmt: skip
    return st, held


def _pairs(st: _lib.HsnwUnits, v: Tensor, unit_idx: Tensor) -> tuple[Tensor, Tensor]:
    if v.dim() != 2 or int(v.shape[1]) != st.d_in:
        raise ValueError(f"forward_grouped expects v [P, {st.d_in}], got shape {tuple(v.shape)}")
    if unit_idx.dim() != 1 or int(unit_idx.shape[0]) != int(v.shape[0]):
        raise ValueError(f"unit_idx must be [P] with P = {int(v.shape[0])} rows of v, got shape {tuple(unit_idx.shape)}")
    if unit_idx.device != v.device:
        raise ValueError("v and unit_idx must share one device")
    return v.detach().to(torch.float32).contiguous(), unit_idx.to(torch.int64).contiguous()


def grouped_forward(v: Tensor, unit_idx: Tensor, W1: Tensor, b1: Tensor, W2: Tensor, b2: Tensor, *, prod: str = "bf16",
                    check: bool = True) -> tuple[Tensor, Tensor, Tensor]:  # fmt: skip
    """``hsnw_units_forward`` without autograd: ``(out [P, d], pre [P, H], status [1] int32)``."""
    st, held = _bank(W1, b1, W2, b2, prod)
    v32, idx = _pairs(st, v, unit_idx)
    dev = v32.device
    lib = _prepare(dev)
    P = int(v32.shape[0])
    dtype = torch.bfloat16 if st.prod_bf16 else torch.float32
    pre = torch.empty((P, st.hidden), dtype=dtype, device=dev)
    out = torch.empty((P, st.d_out), dtype=dtype, device=dev)
    need = int(lib.hsnw_units_scratch_bytes(ctypes.byref(st), P, 0))
    if need <= 0:
        raise ValueError("the grouped unit pass takes at most 256 units")
    scratch = torch.empty((need,), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.hsnw_units_forward(ctypes.byref(st), v32.data_ptr(), idx.data_ptr(), P, pre.data_ptr(), out.data_ptr(),
                                          scratch.data_ptr(), need, _stream(dev)))  # fmt: skip
    status = scratch[:4].view(torch.int32).clone()
    del held
    if check:
        _raise_on(status, st.n_units)
    return out, pre, status


def grouped_backward(v: Tensor, unit_idx: Tensor, W1: Tensor, b1: Tensor, W2: Tensor, b2: Tensor, pre: Tensor, d_out: Tensor, *,
                     prod: str = "bf16", check: bool = True) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:  # fmt: skip
    """``hsnw_units_backward``: ``(d_v, d_W1, d_b1, d_W2, d_b2)``, all float32, for the cotangent ``d_out`` of
    :func:`grouped_forward`'s ``out`` with ``pre`` that call's."""
    st, held = _bank(W1, b1, W2, b2, prod)
    v32, idx = _pairs(st, v, unit_idx)
    dev = v32.device
    lib = _prepare(dev)
    P = int(v32.shape[0])
    dtype = torch.bfloat16 if st.prod_bf16 else torch.float32
    for name, t, width in (("pre", pre, st.hidden), ("d_out", d_out, st.d_out)):
        if tuple(t.shape) != (P, width) or t.device != dev:
            raise ValueError(f"{name} must be [{P}, {width}] on {dev}, got {tuple(t.shape)} on {t.device}")
    pre = pre.detach().to(dtype).contiguous()
    d_out = d_out.detach().to(dtype).contiguous()
    d_v = torch.empty((P, st.d_in), dtype=torch.float32, device=dev)
    grads = tuple(torch.empty(t.shape, dtype=torch.float32, device=dev) for t in held)
    need = int(lib.hsnw_units_scratch_bytes(ctypes.byref(st), P, 1))
    if need <= 0:
        raise ValueError("the grouped unit pass takes at most 256 units")
    scratch = torch.empty((need,), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.hsnw_units_backward(ctypes.byref(st), v32.data_ptr(), idx.data_ptr(), P, pre.data_ptr(), d_out.data_ptr(),
                                           d_v.data_ptr(), *(g.data_ptr() for g in grads), scratch.data_ptr(), need, _stream(dev)))  # fmt: skip
    if check:
        _raise_on(scratch[:4].view(torch.int32), st.n_units)
    del held
    return (d_v, *grads)


def _raise_on(status: Tensor, n_units: int) -> None:
    word = int(status.item())
    if word == 2:
        raise IndexError(f"unit_idx values must lie in [0, {n_units})")
    if word:
        raise RuntimeError(f"the grouped unit pass gave up a bounded device-side wait (status {word}): results discarded")


class _GroupedUnits(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, v: Tensor, unit_idx: Tensor, W1: Tensor, b1: Tensor, W2: Tensor, b2: Tensor, prod: str,
                check: bool) -> tuple[Tensor, Tensor, Tensor]:  # fmt: skip
        out, pre, status = grouped_forward(v, unit_idx, W1, b1, W2, b2, prod=prod, check=check)
        ctx.save_for_backward(v, unit_idx, W1, b1, W2, b2, pre)
        ctx.prod, ctx.check = prod, check
        ctx.mark_non_differentiable(pre, status)
        return out, pre, status

    @staticmethod
    def backward(ctx: Any, d_out: Tensor, _d_pre: Tensor | None, _d_status: Tensor | None) -> tuple[Tensor | None, ...]:
        v, unit_idx, W1, b1, W2, b2, pre = ctx.saved_tensors
        d_v, d_w1, d_b1, d_w2, d_b2 = grouped_backward(v, unit_idx, W1, b1, W2, b2, pre, d_out, prod=ctx.prod, check=ctx.check)
        need = ctx.needs_input_grad
        cast = [(d_v, v), (d_w1, W1), (d_b1, b1), (d_w2, W2), (d_b2, b2)]
        grads = [g.to(like.dtype) if wanted else None for (g, like), wanted in zip(cast, (need[0], *need[2:6]), strict=True)]
        return grads[0], None, grads[1], grads[2], grads[3], grads[4], None, None


def forward_grouped(v: Tensor, unit_idx: Tensor, W1: Tensor, b1: Tensor, W2: Tensor, b2: Tensor, *,
                    record: dict[str, Tensor] | None = None, prod: str = "bf16", check: bool = True) -> Tensor:  # fmt: skip
    """``UnitBank.forward_grouped(v, unit_idx, record=record)`` for the bank ``(W1 [M, d_in, H], b1 [M, H],
    W2 [M, H, d], b2 [M, d])``: ``out [P, d]`` with autograd through ``v`` and the four parameters. ``record``
    receives ``hidden [P, H]`` (and ``status``, the call's status word on the device)."""
    if int(v.shape[0]) == 0 if v.dim() == 2 else False:
        H, d = int(W1.shape[2]), int(W2.shape[2])
        if record is not None:
            record["hidden"] = v.new_zeros((0, H))
        return v.new_zeros((0, d))
    out, pre, status = _GroupedUnits.apply(v, unit_idx, W1, b1, W2, b2, prod, check)
    if record is not None:
        record["hidden"] = pre
        record["status"] = status
    return out
