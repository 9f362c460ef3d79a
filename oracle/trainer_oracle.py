"""CPU restatement (numpy) of the trainer's per-step passes, as PyTorch's CUDA kernels round them.

TEST INFRASTRUCTURE ONLY: imported by ``tests/`` to check ``hsn_b200/csrc/trainer.cu``; the product never
imports it.

Each pass is the sequence of PyTorch operations the reference's trainer runs on the device when its fused
kernels are off, one rounding per operation, with a fused multiply-add exactly where the CUDA kernels of
``lerp``, ``addcmul`` and ``addcdiv`` have one (reference ``kernels/cuda/hsn_trainer.cu:9-18`` names the
ATen sources; PyTorch's CPU kernels round ``addcmul``/``addcdiv`` differently, so the pin is to values
computed by the CUDA operations: ``tests/golden/trainer_*.npz``, written by
``tests/golden/make_trainer_golden.py`` on a GPU):

* :func:`adamw`        ``LazyAdamW._dense_steps``   (``python/hsn/train/lazy_adam.py:462-486``)
* :func:`adamw_units`  ``LazyAdamW._unit_step``     (``lazy_adam.py:573-627``)
* :func:`lerp`         ``WeightEMA.update``         (``python/hsn/train/weight_ema.py:76``)
* :func:`scale64`      ``clip_grad_norm_``          (``python/hsn/train/grad_norm.py:62-69``)
* :func:`limit_squares`, :func:`limit_project`  ``UpdateLimiter._apply_by_group``
  (``python/hsn/train/update_limit.py:164-194``)
"""

from __future__ import annotations

import functools

import numpy as np

f32, f64 = np.float32, np.float64


def _quiet(fn):
    """Overflow to infinity and inf * 0 = NaN are results here, as on the device: no warnings."""

    @functools.wraps(fn)
    def run(*args, **kwargs):
        with np.errstate(over="ignore", invalid="ignore", divide="ignore", under="ignore"):
            return fn(*args, **kwargs)

    return run


def fma(a, b, c):
    """``round_to_float32(a * b + c)`` with ONE rounding, for float32 arrays. The product of two float32
    values is exact in float64; the sum is taken with its exact error term (a two-sum), and the one case
    in which rounding the float64 sum to float32 would round twice (the sum lies exactly between two
    float32 values and the error term is not zero) is decided by the error term's sign."""
    a, b, c = (np.asarray(x, f32).astype(f64) for x in (a, b, c))
    with np.errstate(over="ignore", invalid="ignore"):
        p = a * b
        s = p + c
        bb = s - p
        err = (p - (s - bb)) + (c - bb)
        r = s.astype(f32)
        d = s - r.astype(f64)
        up = np.nextafter(r, f32(np.inf)).astype(f64) - r.astype(f64)
        down = r.astype(f64) - np.nextafter(r, f32(-np.inf)).astype(f64)
        finite = np.isfinite(s) & np.isfinite(r) & np.isfinite(err)
        tie_up = finite & (d > 0) & (d == up / 2) & (err > 0)     # the exact sum is nearer the upper neighbour
        tie_down = finite & (d < 0) & (-d == down / 2) & (err < 0)
    r = np.where(tie_up, np.nextafter(r, f32(np.inf)), r)
    r = np.where(tie_down, np.nextafter(r, f32(-np.inf)), r)
    return r.astype(f32)


@_quiet
def lerp(self_, end, w):
    """``torch.lerp`` on the device: ``fma(w, end - self, self)`` for ``|w| < 0.5``, else
    ``fma(-(end - self), 1 - w, end)``; ``w`` a scalar or an array."""
    self_, end = np.asarray(self_, f32), np.asarray(end, f32)
    w = np.broadcast_to(np.asarray(w, f32), self_.shape)
    diff = end - self_
    return np.where(np.abs(w) < f32(0.5), fma(w, diff, self_), fma(-diff, f32(1.0) - w, end)).astype(f32)


@_quiet
def addcmul(x, a, b, value):
    value = f32(value)
    return fma(a, b, x) if value == f32(1.0) else fma(np.full_like(x, value), np.asarray(a, f32) * np.asarray(b, f32), x)


@_quiet
def addcdiv(x, a, b, value):
    value = f32(value)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.asarray(a, f32) / np.asarray(b, f32)
    return (np.asarray(x, f32) + q).astype(f32) if value == f32(1.0) else fma(np.full_like(x, value), q, x)


@_quiet
def adamw(p, g, m, v, *, lr, beta1, beta2, eps, weight_decay, step):
    """One AdamW step of one tensor at the (already advanced) step count; returns ``(p, m, v)``. The scalars
    are Python floats rounded to float32 where a tensor operation takes them; torch divides a tensor list
    by a scalar as the product with its reciprocal."""
    p, g, m, v = (np.asarray(x, f32) for x in (p, g, m, v))
    if weight_decay != 0:
        p = p * f32(1 - lr * weight_decay)
    m = lerp(m, g, 1 - beta1)
    v = addcmul(v * f32(beta2), g, g, 1 - beta2)
    bias1, bias2 = 1 - beta1**step, 1 - beta2**step
    den = np.sqrt(v) * f32(1.0 / bias2**0.5) + f32(eps)
    return addcdiv(p, m, den, -(lr / bias1)), m, v


@_quiet
def adamw_units(p, g, m, v, *, active, lr, beta1, beta2, eps, weight_decay, steps):
    """The masked per-unit step of a stacked tensor ``[M, ...]``; ``steps [M]`` are the already advanced
    per-unit counts of the active units (anything for the others). Returns ``(p, m, v)``."""
    p, g, m, v = (np.asarray(x, f32) for x in (p, g, m, v))
    M = p.shape[0]
    view = (M,) + (1,) * (p.ndim - 1)
    on = np.asarray(active, bool).reshape(view)
    coef = lambda a, b: np.where(on, f32(a), f32(b)).astype(f32)  # noqa: E731
    g = np.where(on, g, f32(0.0))
    if weight_decay != 0:
        p = p * coef(1 - lr * weight_decay, 1.0)
    m = lerp(m, g, np.broadcast_to(coef(1 - beta1, 0.0), p.shape))
    v = addcmul(v * coef(beta2, 1.0), g, g, 1 - beta2)
    steps = np.asarray(steps, f64)
    with np.errstate(divide="ignore", invalid="ignore"):
        step_size = np.where(np.asarray(active, bool), lr / (1 - np.power(beta1, steps)), 0.0).astype(f32).reshape(view)
        root = np.where(np.asarray(active, bool), np.power(1 - np.power(beta2, steps), 0.5), 1.0).astype(f32).reshape(view)
    den = np.sqrt(v) / root + f32(eps)
    return addcdiv(p, (m * step_size).astype(f32), den, -1.0), m, v


@_quiet
def scale64(grad, coefficient):
    return (np.asarray(grad, f32).astype(f64) * f64(coefficient)).astype(f32)


@_quiet
def limit_squares(param, old):
    param, old = np.asarray(param, f32), np.asarray(old, f32)
    delta = param - old
    return old * old, delta * delta


@_quiet
def limit_project(param, old, scale, clipped):
    """``param' = old + (param - old) * scale`` where the group is clipped, ``param`` otherwise; and the
    squares of the applied step. Returns ``(param', applied ** 2)``."""
    param, old = np.asarray(param, f32), np.asarray(old, f32)
    if clipped:
        param = old + (param - old) * f32(scale)
    applied = param - old
    return param.astype(f32), (applied * applied).astype(f32)


@_quiet
def exchange_adamw(grads_by_rank, p, m, v, *, average=True, **hyper):
    """The fused exchange's arithmetic for a whole flat vector (``hsn_b200/csrc/trainer.cu: k_exchange_adamw``;
    no counterpart in the reference, which all-reduces and then steps): the ranks' gradients summed in rank order,
    multiplied by ``1 / world`` when averaging, then :func:`adamw`. Returns ``(p, m, v)``."""
    g = np.asarray(grads_by_rank[0], f32)
    for other in grads_by_rank[1:]:
        g = g + np.asarray(other, f32)
    if average:
        g = g * (f32(1.0) / f32(len(grads_by_rank)))
    return adamw(p, g, m, v, **hyper)
