"""The end of the replay's cell pass with its backward, one launch over every slot of a window: ``W_out``, the
candidate norm and the weighted ``tanh`` of ``PDGCell.replay_sparse`` (reference ``python/hsn/model/cell.py:719-721``)
over this library.

:func:`candidate_tail` takes ``W_out.weight`` and ``cand_norm.weight`` instead of the modules, otherwise the
reference's operands: ``unit_out [..., d]`` (the grouped unit pass's output), ``alpha [...]`` (the slot weights)
-> ``c [..., d]`` float32, ``record["y"]`` ``W_out``'s output (``cell.py:723``), detached. It is an autograd function:
``c.backward(...)`` fills the gradients of ``unit_out``, ``alpha`` and the two weights with the values autograd gives
the reference's three lines (``hsn_b200/csrc/tail.cu``).

``prod="bf16"`` is the pass under ``torch.autocast(dtype=torch.bfloat16)`` (``unit_out`` is read as bfloat16, ``y`` is
a bfloat16 value held in float32, ``d_unit_out`` and ``d_W_out`` are bfloat16 values), ``prod="fp32"`` the pass
without autocast. There is no CPU or PyTorch path here: without the built library or a CUDA device the call raises.
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch
from torch import Tensor

from .. import _lib

__all__ = ["candidate_tail", "tail_forward", "tail_backward"]


def _prepare(device: torch.device) -> Any:
    if device.type != "cuda":
        raise RuntimeError(f"the replay's tail runs on a CUDA device, got tensors on {device}")
    lib = _lib.library()
    index = device.index if device.index is not None else torch.cuda.current_device()
    if not lib.hsnw_prepared(index):
        _lib.check(lib.hsnw_prepare(index))
    return lib


def _stream(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _weights(w_out: Tensor, cand_w: Tensor, eps: float, prod: str) -> tuple[_lib.HsnwTail, tuple[Tensor, Tensor]]:
    if prod not in ("bf16", "fp32"):
        raise ValueError(f"prod must be 'bf16' or 'fp32', got {prod!r}")
    if w_out.dim() != 2 or w_out.shape[0] != w_out.shape[1]:
        raise ValueError(f"W_out must be [d, d], got {tuple(w_out.shape)}")
    d = int(w_out.shape[0])
    if d not in (16, 32, 64, 128):
        raise ValueError(f"the replay's tail takes d of 16, 32, 64 or 128, got {d}")
    if tuple(cand_w.shape) != (d,):
        raise ValueError(f"the candidate norm's weight must be [{d}], got {tuple(cand_w.shape)}")
    if cand_w.device != w_out.device:
        raise ValueError("W_out and the candidate norm's weight must share one device")
    held = (w_out.detach().to(torch.float32).contiguous(), cand_w.detach().to(torch.float32).contiguous())
    st = _lib.HsnwTail(d=d, prod_bf16=int(prod == "bf16"), norm_eps=float(eps), reserved=0, w_out=held[0].data_ptr(),
                       norm_weight=held[1].data_ptr())  # fmt: skip
    return st, held


def _slots(st: _lib.HsnwTail, unit_out: Tensor, alpha: Tensor) -> tuple[Tensor, Tensor]:
    if unit_out.dim() < 1 or int(unit_out.shape[-1]) != st.d:
        raise ValueError(f"unit_out must be [..., {st.d}], got shape {tuple(unit_out.shape)}")
    if tuple(alpha.shape) != tuple(unit_out.shape[:-1]):
        raise ValueError(f"alpha must be {tuple(unit_out.shape[:-1])}, got {tuple(alpha.shape)}")
    if alpha.device != unit_out.device:
        raise ValueError("unit_out and alpha must share one device")
    dtype = torch.bfloat16 if st.prod_bf16 else torch.float32
    return unit_out.detach().to(dtype).reshape(-1, st.d).contiguous(), alpha.detach().to(torch.float32).reshape(-1).contiguous()


def tail_forward(unit_out: Tensor, alpha: Tensor, w_out: Tensor, cand_w: Tensor, *, eps: float = 1e-6,
                 prod: str = "bf16") -> tuple[Tensor, Tensor]:  # fmt: skip
    """``hsnw_tail_forward`` without autograd: ``(c, y)``, both float32 in ``unit_out``'s shape."""
    st, held = _weights(w_out, cand_w, eps, prod)
    x, a = _slots(st, unit_out, alpha)
    dev = x.device
    lib = _prepare(dev)
    P = int(x.shape[0])
    y = torch.empty((P, st.d), dtype=torch.float32, device=dev)
    c = torch.empty((P, st.d), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.hsnw_tail_forward(ctypes.byref(st), x.data_ptr(), a.data_ptr(), P, y.data_ptr(), c.data_ptr(), _stream(dev)))
    del held
    return c.reshape(unit_out.shape), y.reshape(unit_out.shape)


def tail_backward(unit_out: Tensor, alpha: Tensor, w_out: Tensor, cand_w: Tensor, y: Tensor, d_c: Tensor, *, eps: float = 1e-6,
                  prod: str = "bf16") -> tuple[Tensor, Tensor, Tensor, Tensor]:  # fmt: skip
    """``hsnw_tail_backward``: ``(d_unit_out, d_alpha, d_W_out, d_cand_w)`` for the cotangent ``d_c`` of
    :func:`tail_forward`'s ``c`` with ``y`` that call's; ``d_unit_out`` is bfloat16 under ``prod="bf16"``."""
    st, held = _weights(w_out, cand_w, eps, prod)
    x, a = _slots(st, unit_out, alpha)
    dev = x.device
    lib = _prepare(dev)
    P = int(x.shape[0])
    for name, t in (("y", y), ("d_c", d_c)):
        if tuple(t.shape) != tuple(unit_out.shape) or t.device != dev:
            raise ValueError(f"{name} must be {tuple(unit_out.shape)} on {dev}, got {tuple(t.shape)} on {t.device}")
    y32 = y.detach().to(torch.float32).reshape(-1, st.d).contiguous()
    dc32 = d_c.detach().to(torch.float32).reshape(-1, st.d).contiguous()
    d_x = torch.empty_like(x)
    d_a = torch.empty((P,), dtype=torch.float32, device=dev)
    d_w = torch.empty((st.d, st.d), dtype=torch.float32, device=dev)
    d_g = torch.empty((st.d,), dtype=torch.float32, device=dev)
    need = int(lib.hsnw_tail_scratch_bytes(ctypes.byref(st), P))
    scratch = torch.empty((max(need, 256),), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.hsnw_tail_backward(ctypes.byref(st), x.data_ptr(), a.data_ptr(), y32.data_ptr(), dc32.data_ptr(), P,
                                          d_x.data_ptr(), d_a.data_ptr(), d_w.data_ptr(), d_g.data_ptr(), scratch.data_ptr(),
                                          int(scratch.numel()), _stream(dev)))  # fmt: skip
    del held
    return d_x.reshape(unit_out.shape), d_a.reshape(alpha.shape), d_w, d_g


class _Tail(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, unit_out: Tensor, alpha: Tensor, w_out: Tensor, cand_w: Tensor, eps: float, prod: str) -> tuple[Tensor, Tensor]:
        c, y = tail_forward(unit_out, alpha, w_out, cand_w, eps=eps, prod=prod)
        ctx.save_for_backward(unit_out, alpha, w_out, cand_w, y)
        ctx.eps, ctx.prod = eps, prod
        ctx.mark_non_differentiable(y)
        return c, y

    @staticmethod
    def backward(ctx: Any, d_c: Tensor, _d_y: Tensor | None) -> tuple[Tensor | None, ...]:
        unit_out, alpha, w_out, cand_w, y = ctx.saved_tensors
        grads = tail_backward(unit_out, alpha, w_out, cand_w, y, d_c, eps=ctx.eps, prod=ctx.prod)
        likes = (unit_out, alpha, w_out, cand_w)
        out = [g.to(like.dtype) if wanted else None for g, like, wanted in zip(grads, likes, ctx.needs_input_grad[:4], strict=True)]
        return out[0], out[1], out[2], out[3], None, None


def candidate_tail(unit_out: Tensor, alpha: Tensor, w_out: Tensor, cand_w: Tensor, *, eps: float = 1e-6,
                   record: dict[str, Tensor] | None = None, prod: str = "bf16") -> Tensor:  # fmt: skip
    """``tanh(alpha[..., None] * cand_norm(W_out(unit_out)))`` with autograd through ``unit_out``, ``alpha`` and the
    two weights; ``record`` receives ``y`` (``W_out``'s output in float32)."""
    if unit_out.numel() == 0:
        if record is not None:
            record["y"] = unit_out.new_zeros(unit_out.shape, dtype=torch.float32)
        return unit_out.new_zeros(unit_out.shape, dtype=torch.float32)
    c, y = _Tail.apply(unit_out, alpha, w_out, cand_w, float(eps), prod)
    if record is not None:
        record["y"] = y
    return c
