"""The replay's scorer logits over every cell of every window position, with the gradients of the scorer's weight and
bias: ``_scorer_logits`` (reference ``python/hsn/train/split.py:305-342``) over this library.

:func:`scorer_logits` takes the linear scorer's ``weight [M, 3d + 1 + S]`` and ``bias [M]`` in place of the module,
otherwise the reference's arguments: ``u, eps [R, d]``, ``h [R, N, d]`` (the recorded state), ``age [R, N]`` int64,
``scalars [R, N, S]`` -> ``[R, N, M]`` float32. It is an autograd function: the features are constants of the replay
(``h`` is recorded, the caller detaches ``u`` and ``eps``, ``split.py:628-631``), so ``backward`` fills the gradients
of ``weight`` and ``bias`` only, with the values autograd gives the reference's three linear maps
(``hsn_b200/csrc/scorer.cu``). ``prod="bf16"`` is the function under ``torch.autocast(dtype=torch.bfloat16)``,
``prod="fp32"`` without. The address gate (A12) and excluded features are not covered: the caller keeps the
reference's assembled path for those, as the reference's own fast path does. No CPU or PyTorch path: without the
built library or a CUDA device the call raises.
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch
from torch import Tensor

from .. import _lib

__all__ = ["scorer_logits", "scorer_logits_backward", "scorer_logits_forward"]


def _prepare(device: torch.device) -> Any:
    if device.type != "cuda":
        raise RuntimeError(f"the scorer logits run on a CUDA device, got tensors on {device}")
    lib = _lib.library()
    index = device.index if device.index is not None else torch.cuda.current_device()
    if not lib.hsnw_prepared(index):
        _lib.check(lib.hsnw_prepare(index))
    return lib


def _stream(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _inputs(weight: Tensor, bias: Tensor, u: Tensor, eps: Tensor, h: Tensor, age: Tensor, scalars: Tensor, age_max: float,
            prod: str) -> tuple[_lib.HsnwScorer, tuple[Tensor, ...]]:  # fmt: skip
    if prod not in ("bf16", "fp32"):
        raise ValueError(f"prod must be 'bf16' or 'fp32', got {prod!r}")
    if h.dim() != 3:
        raise ValueError(f"h must be [R, N, d], got {tuple(h.shape)}")
    R, N, d = (int(n) for n in h.shape)
    S = int(scalars.shape[-1]) if scalars.dim() == 3 else -1
    M = int(weight.shape[0]) if weight.dim() == 2 else -1
    want = {"u": (u, (R, d)), "eps": (eps, (R, d)), "age": (age, (R, N)), "scalars": (scalars, (R, N, S)),
            "weight": (weight, (M, 3 * d + 1 + S)), "bias": (bias, (M,))}  # fmt: skip
    for name, (t, shape) in want.items():
        if tuple(t.shape) != shape or min(shape, default=0) < 0:
            raise ValueError(f"{name} must have shape {shape}, got {tuple(t.shape)}")
        if t.device != h.device:
            raise ValueError(f"{name} must live on {h.device}, got {t.device}")
    f32 = lambda t: t.detach().to(torch.float32).contiguous()  # noqa: E731
    held = (f32(weight), f32(bias), f32(u), f32(eps), f32(h), age.to(torch.int64).contiguous(), f32(scalars))
    st = _lib.HsnwScorer(d=d, n_cells=N, n_units=M, n_scalars=S, prod_bf16=int(prod == "bf16"), age_max=float(age_max),
                         weight=held[0].data_ptr(), bias=held[1].data_ptr())  # fmt: skip
    return st, held


def _scratch(lib: Any, st: _lib.HsnwScorer, rows: int, backward: bool, device: torch.device) -> Tensor:
    need = int(lib.hsnw_scorer_scratch_bytes(ctypes.byref(st), rows, int(backward)))
    if need <= 0:
        raise ValueError("scorer_logits: sizes the library does not take")
    return torch.empty((need,), dtype=torch.uint8, device=device)


def _raise_on(status: Tensor) -> None:
    word = int(status.item())
    if word:
        raise RuntimeError(f"the scorer logits gave up a bounded device-side wait (status {word}): results discarded")


def scorer_logits_forward(weight: Tensor, bias: Tensor, u: Tensor, eps: Tensor, h: Tensor, age: Tensor, scalars: Tensor, *,
                          age_max: float, prod: str = "bf16", check: bool = True) -> Tensor:  # fmt: skip
    """``hsnw_scorer_logits`` without autograd: ``[R, N, M]`` float32."""
    st, held = _inputs(weight, bias, u, eps, h, age, scalars, age_max, prod)
    dev = held[4].device
    lib = _prepare(dev)
    rows = int(h.shape[0])
    out = torch.empty((rows, st.n_cells, st.n_units), dtype=torch.float32, device=dev)
    scratch = _scratch(lib, st, rows, False, dev)
    with torch.cuda.device(dev):
        _lib.check(lib.hsnw_scorer_logits(ctypes.byref(st), held[2].data_ptr(), held[3].data_ptr(), held[4].data_ptr(),
                                          held[5].data_ptr(), held[6].data_ptr(), rows, out.data_ptr(), scratch.data_ptr(),
                                          scratch.numel(), _stream(dev)))  # fmt: skip
    if check:
        _raise_on(scratch[:4].view(torch.int32))
    return out


def scorer_logits_backward(weight: Tensor, bias: Tensor, u: Tensor, eps: Tensor, h: Tensor, age: Tensor, scalars: Tensor,
                           d_logits: Tensor, *, age_max: float, prod: str = "bf16", check: bool = True) -> tuple[Tensor, Tensor]:  # fmt: skip
    """``hsnw_scorer_logits_backward``: ``(d_weight, d_bias)``, float32, for the cotangent ``d_logits [R, N, M]``."""
    st, held = _inputs(weight, bias, u, eps, h, age, scalars, age_max, prod)
    dev = held[4].device
    lib = _prepare(dev)
    rows = int(h.shape[0])
    if tuple(d_logits.shape) != (rows, st.n_cells, st.n_units) or d_logits.device != dev:
        raise ValueError(f"d_logits must be [{rows}, {st.n_cells}, {st.n_units}] on {dev}, got {tuple(d_logits.shape)}")
    g = d_logits.detach().to(torch.float32).contiguous()
    d_weight = torch.empty_like(held[0])
    d_bias = torch.empty_like(held[1])
    scratch = _scratch(lib, st, rows, True, dev)
    with torch.cuda.device(dev):
        _lib.check(lib.hsnw_scorer_logits_backward(ctypes.byref(st), held[2].data_ptr(), held[3].data_ptr(), held[4].data_ptr(),
                                                   held[5].data_ptr(), held[6].data_ptr(), rows, g.data_ptr(), d_weight.data_ptr(),
                                                   d_bias.data_ptr(), scratch.data_ptr(), scratch.numel(), _stream(dev)))  # fmt: skip
    if check:
        _raise_on(scratch[:4].view(torch.int32))
    return d_weight, d_bias


class _ScorerLogits(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, weight: Tensor, bias: Tensor, u: Tensor, eps: Tensor, h: Tensor, age: Tensor, scalars: Tensor,
                age_max: float, prod: str, check: bool) -> Tensor:  # fmt: skip
        ctx.save_for_backward(weight, bias, u, eps, h, age, scalars)
        ctx.age_max, ctx.prod, ctx.check = age_max, prod, check
        return scorer_logits_forward(weight, bias, u, eps, h, age, scalars, age_max=age_max, prod=prod, check=check)

    @staticmethod
    def backward(ctx: Any, d_logits: Tensor) -> tuple[Tensor | None, ...]:
        weight, bias, u, eps, h, age, scalars = ctx.saved_tensors
        if any(ctx.needs_input_grad[2:7]):
            raise RuntimeError("scorer_logits reads its features as constants (the replay detaches them): no gradient for "
                               "u, eps, h, age or scalars")  # fmt: skip
        d_weight, d_bias = scorer_logits_backward(weight, bias, u, eps, h, age, scalars, d_logits, age_max=ctx.age_max,
                                                  prod=ctx.prod, check=ctx.check)  # fmt: skip
        need = ctx.needs_input_grad
        return (d_weight.to(weight.dtype) if need[0] else None, d_bias.to(bias.dtype) if need[1] else None,
                None, None, None, None, None, None, None, None)  # fmt: skip


def scorer_logits(weight: Tensor, bias: Tensor, u: Tensor, eps: Tensor, h: Tensor, age: Tensor, scalars: Tensor, *,
                  age_max: float, prod: str = "bf16", check: bool = True) -> Tensor:  # fmt: skip
    """``_scorer_logits(scorer, u, eps, h, age, scalars)`` for the linear scorer ``(weight, bias)``, ``age_max`` the
    scorer's: ``[R, N, M]`` float32 with autograd through ``weight`` and ``bias``."""
    return _ScorerLogits.apply(weight, bias, u, eps, h, age, scalars, float(age_max), prod, check)
