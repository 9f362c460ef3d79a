"""The messages and the gathered inputs of the replay's cell pass with their backward, one launch over every slot of a
window: ``sources = V(h[src])``, ``m = sum_j w_j sources_j``, ``v_raw = [u; eps; h[cell]; m]`` of
``PDGCell.replay_sparse`` (reference ``python/hsn/model/cell.py:698-705``) over this library.

:func:`gathered_inputs` takes the graph's tables instead of the module: ``pad_src [N, D]`` (``graph._pad_src``) and
the padded edge weights ``edge_w [N, D]`` (``graph._padded_weights()``, which keeps its own autograd path back to
``graph.edge_logit``), ``V.weight``, and ``cells [R, K]`` with padded slots set to cell 0 as the reference does. It is an
autograd function through ``u``, ``eps``, ``edge_w`` and ``V.weight`` (the state is a constant of the replay).

The pass is the one under ``torch.autocast(dtype=torch.bfloat16)``; float32 products, ``d = 128`` and more than four
in-neighbours are not taken: the call raises and the caller keeps the reference's lines. There is no CPU or PyTorch
path here: without the built library or a CUDA device the call raises.
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch
from torch import Tensor

from .. import _lib

__all__ = ["gathered_inputs", "messages_forward", "messages_backward"]


def _prepare(device: torch.device) -> Any:
    if device.type != "cuda":
        raise RuntimeError(f"the replay's messages run on a CUDA device, got tensors on {device}")
    lib = _lib.library()
    index = device.index if device.index is not None else torch.cuda.current_device()
    if not lib.hsnw_prepared(index):
        _lib.check(lib.hsnw_prepare(index))
    return lib


def _stream(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _tables(h: Tensor, cells: Tensor, pad_src: Tensor, edge_w: Tensor, v_w: Tensor) -> tuple[_lib.HsnwMessages, tuple[Tensor, ...]]:
    if h.dim() != 3:
        raise ValueError(f"h must be [R, N, d], got {tuple(h.shape)}")
    R, N, d = (int(n) for n in h.shape)
    if d not in (16, 32, 64):
        raise ValueError(f"the replay's messages take d of 16, 32 or 64, got {d}")
    if cells.dim() != 2 or int(cells.shape[0]) != R or int(cells.shape[1]) < 1:
        raise ValueError(f"cells must be [R, K] with R = {R}, got {tuple(cells.shape)}")
    if pad_src.dim() != 2 or int(pad_src.shape[0]) != N or tuple(edge_w.shape) != tuple(pad_src.shape):
        raise ValueError(f"pad_src and edge_w must be [{N}, D], got {tuple(pad_src.shape)} and {tuple(edge_w.shape)}")
    D = int(pad_src.shape[1])
    if not 1 <= D <= 4:
        raise ValueError(f"the replay's messages take 1 to 4 in-neighbours a cell, got {D}")
    if tuple(v_w.shape) != (d, d):
        raise ValueError(f"V's weight must be [{d}, {d}], got {tuple(v_w.shape)}")
    for t in (cells, pad_src, edge_w, v_w):
        if t.device != h.device:
            raise ValueError("the state, the decision, the graph's tables and V must share one device")
    held = (h.detach().to(torch.float32).contiguous(), cells.to(torch.int64).contiguous(), pad_src.to(torch.int64).contiguous(),
            edge_w.detach().to(torch.float32).contiguous(), v_w.detach().to(torch.float32).contiguous())  # fmt: skip
    st = _lib.HsnwMessages(d=d, n_cells=N, degree=D, k=int(cells.shape[1]), prod_bf16=1, reserved=0, v_w=held[4].data_ptr(),
                           edge_w=held[3].data_ptr(), pad_src=held[2].data_ptr())  # fmt: skip
    return st, held


def messages_forward(u: Tensor, eps: Tensor, h: Tensor, cells: Tensor, pad_src: Tensor, edge_w: Tensor, v_w: Tensor) -> Tensor:
    """``hsnw_messages_forward`` without autograd: ``v_raw [R, K, 4d]`` float32."""
    st, held = _tables(h, cells, pad_src, edge_w, v_w)
    dev = held[0].device
    R = int(h.shape[0])
    rows = []
    for name, t in (("u", u), ("eps", eps)):
        if tuple(t.shape) != (R, st.d) or t.device != dev:
            raise ValueError(f"{name} must be [{R}, {st.d}] on {dev}, got {tuple(t.shape)} on {t.device}")
        rows.append(t.detach().to(torch.float32).contiguous())
    lib = _prepare(dev)
    v_raw = torch.empty((R, st.k, 4 * st.d), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.hsnw_messages_forward(ctypes.byref(st), rows[0].data_ptr(), rows[1].data_ptr(), held[0].data_ptr(), held[1].data_ptr(), R,
                                             v_raw.data_ptr(), _stream(dev)))  # fmt: skip
    del held
    return v_raw


def messages_backward(h: Tensor, cells: Tensor, pad_src: Tensor, edge_w: Tensor, v_w: Tensor, d_v_raw: Tensor) -> tuple[Tensor, ...]:
    """``hsnw_messages_backward``: ``(d_u [R, d], d_eps [R, d], d_edge_w [N, D], d_v_w [d, d])`` for the cotangent
    ``d_v_raw [R, K, 4d]``."""
    st, held = _tables(h, cells, pad_src, edge_w, v_w)
    dev = held[0].device
    R = int(h.shape[0])
    if tuple(d_v_raw.shape) != (R, st.k, 4 * st.d) or d_v_raw.device != dev:
        raise ValueError(f"d_v_raw must be [{R}, {st.k}, {4 * st.d}] on {dev}, got {tuple(d_v_raw.shape)} on {d_v_raw.device}")
    g = d_v_raw.detach().to(torch.float32).contiguous()
    lib = _prepare(dev)
    f32 = torch.float32
    d_u, d_eps = torch.empty((R, st.d), dtype=f32, device=dev), torch.empty((R, st.d), dtype=f32, device=dev)
    d_edge_w, d_v_w = torch.empty((st.n_cells, st.degree), dtype=f32, device=dev), torch.empty((st.d, st.d), dtype=f32, device=dev)
    need = int(lib.hsnw_messages_scratch_bytes(ctypes.byref(st), R))
    scratch = torch.empty((max(need, 256),), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.hsnw_messages_backward(ctypes.byref(st), held[0].data_ptr(), held[1].data_ptr(), g.data_ptr(), R, d_u.data_ptr(),
                                              d_eps.data_ptr(), d_edge_w.data_ptr(), d_v_w.data_ptr(), scratch.data_ptr(),
                                              int(scratch.numel()), _stream(dev)))  # fmt: skip
    del held
    return d_u, d_eps, d_edge_w, d_v_w


class _Gathered(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, u: Tensor, eps: Tensor, h: Tensor, cells: Tensor, pad_src: Tensor, edge_w: Tensor, v_w: Tensor) -> Tensor:
        v_raw = messages_forward(u, eps, h, cells, pad_src, edge_w, v_w)
        ctx.save_for_backward(h, cells, pad_src, edge_w, v_w)
        ctx.dtypes = (u.dtype, eps.dtype, edge_w.dtype, v_w.dtype)
        return v_raw

    @staticmethod
    def backward(ctx: Any, d_v_raw: Tensor) -> tuple[Tensor | None, ...]:
        h, cells, pad_src, edge_w, v_w = ctx.saved_tensors
        d_u, d_eps, d_edge_w, d_v_w = messages_backward(h, cells, pad_src, edge_w, v_w, d_v_raw)
        need = ctx.needs_input_grad
        dt = ctx.dtypes
        return (d_u.to(dt[0]) if need[0] else None, d_eps.to(dt[1]) if need[1] else None, None, None, None,
                d_edge_w.to(dt[2]) if need[5] else None, d_v_w.to(dt[3]) if need[6] else None)  # fmt: skip


def gathered_inputs(u: Tensor, eps: Tensor, h: Tensor, cells: Tensor, pad_src: Tensor, edge_w: Tensor, v_w: Tensor) -> Tensor:
    """``v_raw [R, K, 4d] = [u; eps; h[cells]; m]`` with autograd through ``u``, ``eps``, ``edge_w`` and ``v_w``; ``h`` is
    read as a constant. ``m = v_raw[..., 3d:]`` is what the reference records as ``record["m"]``."""
    if h.requires_grad:
        raise ValueError("the replay reads the recorded state as a constant: detach h")
    if cells.numel() == 0:
        return h.new_zeros((*cells.shape, 4 * int(h.shape[-1])), dtype=torch.float32)
    return _Gathered.apply(u, eps, h, cells, pad_src, edge_w, v_w)
