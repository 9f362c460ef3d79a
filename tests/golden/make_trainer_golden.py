"""Generates ``trainer_*.npz`` on a machine with a CUDA device: the values PyTorch's CUDA kernels
compute for the trainer's per-step passes, which the reference's fused trainer kernels reproduce bit for
bit (``kernels/cuda/hsn_trainer.cu``). PyTorch's CPU kernels round ``addcmul`` and ``addcdiv``
differently, so these fixtures cannot be made without a GPU.

    python tests/golden/make_trainer_golden.py --out tests/golden

Each pass below is the reference's own sequence of torch operations (its path when the fused kernels are
off), with the file and lines it stands at; inputs are seeded and carry zeros of both signs, subnormals
and large magnitudes (reference ``tests/test_p2_10b_trainer_kernels.py:100-107``).
"""

from __future__ import annotations

import argparse
from pathlib import Path

import numpy as np
import torch

SHAPES = [(32, 48), (8, 101), (1, 128), (512,), (8,), (1,), (3, 5, 7), (129,), (1031,)]
UNIT_SHAPES = [(8, 16, 12), (8, 33), (8, 1), (8, 7, 3)]


def values(shape, scale, gen):
    x = torch.randn(*shape, generator=gen) * scale
    flat = x.view(-1)
    if flat.numel() >= 8:
        flat[:6] = torch.tensor([0.0, -0.0, 1e-42, -1e-40, 1e30, -3e-30])
    return x


def dense_steps(params, grads, exp_avgs, exp_avg_sqs, step, lr, beta1, beta2, eps, weight_decay):
    """``LazyAdamW._dense_steps`` (python/hsn/train/lazy_adam.py:462-486)."""
    if weight_decay != 0:
        torch._foreach_mul_(params, 1 - lr * weight_decay)
    torch._foreach_lerp_(exp_avgs, grads, 1 - beta1)
    torch._foreach_mul_(exp_avg_sqs, beta2)
    torch._foreach_addcmul_(exp_avg_sqs, grads, grads, value=1 - beta2)
    bias_correction1 = 1 - beta1**step
    bias_correction2 = 1 - beta2**step
    step_size = lr / bias_correction1
    denoms = torch._foreach_sqrt(exp_avg_sqs)
    torch._foreach_div_(denoms, bias_correction2**0.5)
    torch._foreach_add_(denoms, eps)
    torch._foreach_addcdiv_(params, exp_avgs, denoms, value=-step_size)


def unit_step(p, grad, exp_avg, exp_avg_sq, steps, active, lr, beta1, beta2, eps, weight_decay):
    """``LazyAdamW._unit_step`` (lazy_adam.py:573-627) with ``_unit_bias_terms`` (:508-523); ``steps`` are
    the already advanced per-unit counts (float64 on the host)."""
    M = p.shape[0]
    view = (M,) + (1,) * (p.ndim - 1)
    act = active.to(p.device).view(view)
    const = lambda v: torch.tensor(v, dtype=p.dtype, device=p.device)  # noqa: E731
    coef = lambda on, off: torch.where(act, const(on), const(off))  # noqa: E731
    g = torch.where(act, grad, const(0.0))
    if weight_decay != 0:
        p.mul_(coef(1 - lr * weight_decay, 1.0))
    exp_avg.lerp_(g, coef(1 - beta1, 0.0))
    exp_avg_sq.mul_(coef(beta2, 1.0)).addcmul_(g, g, value=1 - beta2)
    s64 = steps.to(torch.float64)
    zero, one = torch.zeros((), dtype=torch.float64), torch.ones((), dtype=torch.float64)
    step_size = torch.where(active, lr / (1 - torch.pow(beta1, s64)), zero).to(p.dtype).to(p.device)
    root = torch.where(active, (1 - torch.pow(beta2, s64)).pow(0.5), one).to(p.dtype).to(p.device)
    denom = exp_avg_sq.sqrt().div_(root.view(view)).add_(eps)
    p.addcdiv_(exp_avg.mul(step_size.view(view)), denom, value=-1.0)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--out", type=Path, required=True)
    args = parser.parse_args()
    dev = torch.device("cuda", 0)
    out: dict[str, np.ndarray] = {}
    gen = torch.Generator().manual_seed(0)
    n = lambda t: t.detach().cpu().numpy()  # noqa: E731

    # AdamW on ordinary tensors, three steps with gradients of very different scales
    for case, (betas, wd) in enumerate([((0.9, 0.95), 0.01), ((0.9, 0.999), 0.0), ((0.0, 0.5), 0.01), ((0.5, 0.0), 0.0)]):
        lr, eps = 2.5e-3, 1e-8
        ps = [values(s, 0.1, gen).to(dev) for s in SHAPES]
        ms = [torch.zeros_like(p) for p in ps]
        vs = [torch.zeros_like(p) for p in ps]
        out[f"adamw{case}_hyper"] = np.array([lr, betas[0], betas[1], eps, wd])
        for j, p in enumerate(ps):
            out[f"adamw{case}_p0_{j}"] = n(p)
        for step in range(1, 4):
            gs = [values(s, (1e-3, 1.0, 30.0)[step - 1], gen).to(dev) for s in SHAPES]
            dense_steps(ps, gs, ms, vs, step, lr, betas[0], betas[1], eps, wd)
            for j in range(len(SHAPES)):
                out[f"adamw{case}_g{step}_{j}"] = n(gs[j])
                out[f"adamw{case}_p{step}_{j}"] = n(ps[j])
                out[f"adamw{case}_m{step}_{j}"] = n(ms[j])
                out[f"adamw{case}_v{step}_{j}"] = n(vs[j])

    # AdamW on stacked unit tensors: two steps, different units active
    lr, beta1, beta2, eps = 1e-3, 0.9, 0.95, 1e-8
    for case, wd in enumerate([0.01, 0.0]):
        ps = [values(s, 0.1, gen).to(dev) for s in UNIT_SHAPES]
        ms = [values(s, 0.01, gen).to(dev) for s in UNIT_SHAPES]
        vs = [values(s, 0.01, gen).abs().to(dev) for s in UNIT_SHAPES]
        steps = torch.tensor([3, 0, 7, 1, 0, 40, 2, 9], dtype=torch.int64)
        out[f"units{case}_hyper"] = np.array([lr, beta1, beta2, eps, wd])
        for j in range(len(UNIT_SHAPES)):
            out[f"units{case}_p0_{j}"], out[f"units{case}_m0_{j}"], out[f"units{case}_v0_{j}"] = n(ps[j]), n(ms[j]), n(vs[j])
        for step, mask in enumerate([[1, 0, 1, 1, 0, 1, 0, 1], [0, 1, 1, 0, 0, 1, 1, 1]], start=1):
            active = torch.tensor(mask, dtype=torch.bool)
            steps = steps + active.to(torch.int64)
            out[f"units{case}_active{step}"], out[f"units{case}_steps{step}"] = n(active), n(steps)
            for j, s in enumerate(UNIT_SHAPES):
                g = values(s, (1e-2, 3.0)[step - 1], gen).to(dev)
                unit_step(ps[j], g, ms[j], vs[j], steps, active, lr, beta1, beta2, eps, wd)
                out[f"units{case}_g{step}_{j}"] = n(g)
                out[f"units{case}_p{step}_{j}"], out[f"units{case}_m{step}_{j}"], out[f"units{case}_v{step}_{j}"] = n(ps[j]), n(ms[j]), n(vs[j])

    # the weight average (python/hsn/train/weight_ema.py:76: torch._foreach_lerp_)
    for case, w in enumerate([1e-3, 0.3, 0.5, 0.999]):
        selfs = [values(s, 0.1, gen).to(dev) for s in SHAPES]
        ends = [values(s, 0.1, gen).to(dev) for s in SHAPES]
        out[f"lerp{case}_w"] = np.array(w)
        for j in range(len(SHAPES)):
            out[f"lerp{case}_self_{j}"], out[f"lerp{case}_end_{j}"] = n(selfs[j]), n(ends[j])
        torch._foreach_lerp_(selfs, ends, w)
        for j in range(len(SHAPES)):
            out[f"lerp{case}_out_{j}"] = n(selfs[j])

    # the float64 clip's scaling (python/hsn/train/grad_norm.py:62-69)
    for case, c in enumerate([0.37, 1e-12, 3e-41]):
        grads = [values(s, 10.0, gen).to(dev) for s in SHAPES]
        coefficient = torch.tensor(c, dtype=torch.float64, device=dev)
        out[f"scale{case}_c"] = np.array(c, dtype=np.float64)
        for j, g in enumerate(grads):
            out[f"scale{case}_in_{j}"] = n(g)
            out[f"scale{case}_out_{j}"] = n((g.double() * coefficient).float())

    # the update caps (python/hsn/train/update_limit.py:164-194), a clipped and an unclipped group
    for case, (scale, clipped) in enumerate([(0.25, True), (1.0, False), (1e-3, True)]):
        params = [values(s, 0.1, gen).to(dev) for s in SHAPES]
        olds = [values(s, 0.1, gen).to(dev) for s in SHAPES]
        out[f"limit{case}_decision"] = np.array([scale, float(clipped)], dtype=np.float32)
        deltas = torch._foreach_sub(params, olds)
        scale_t, clipped_t = torch.tensor(scale, device=dev), torch.tensor(clipped, device=dev)
        projected = torch._foreach_add(olds, list(torch._foreach_mul(deltas, scale_t)))
        new = [torch.where(clipped_t, a, p) for a, p in zip(projected, params)]
        for j in range(len(SHAPES)):
            out[f"limit{case}_param_{j}"], out[f"limit{case}_old_{j}"] = n(params[j]), n(olds[j])
            out[f"limit{case}_oldsq_{j}"] = n(olds[j] * olds[j])
            out[f"limit{case}_deltasq_{j}"] = n(deltas[j] * deltas[j])
            out[f"limit{case}_new_{j}"] = n(new[j])
            applied = new[j] - olds[j]
            out[f"limit{case}_appliedsq_{j}"] = n(applied * applied)
    np.savez_compressed(args.out / "trainer_passes.npz", **out)
    print("trainer_passes.npz", len(out), "arrays", sum(a.size for a in out.values()), "values, torch", torch.__version__)


if __name__ == "__main__":
    main()
