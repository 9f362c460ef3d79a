"""The trainer's per-step passes (``hsn_b200/csrc/trainer.cu`` behind ``hsn_b200/kernels/trainer.py``).

On the CPU the oracle's restatement of PyTorch's CUDA arithmetic (``oracle/trainer_oracle.py``) must
reproduce, bit for bit, values that PyTorch's CUDA kernels computed (``tests/golden/trainer_passes.npz``,
written on a GPU by ``tests/golden/make_trainer_golden.py``). On the GPU the kernels must reproduce those
values, the oracle's at other sizes, and the live sequences of torch operations they replace (the protocol
of the reference's ``tests/test_p2_10b_trainer_kernels.py``: equal bit patterns, -0.0 is not 0.0).
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import trainer_oracle as TO

N_SHAPES, N_UNIT_SHAPES = 9, 4


def same(a, b) -> bool:
    """Equal bit patterns (so -0.0 is not 0.0); a NaN equals a NaN whatever its payload (numpy's and the
    device's differ)."""
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    both_nan = np.isnan(a) & np.isnan(b)
    bits = {4: np.uint32, 8: np.uint64}[a.dtype.itemsize]
    return bool(np.all((a.view(bits) == b.view(bits)) | both_nan))


@pytest.fixture(scope="module")
def golden():
    return load_golden("trainer_passes")


def test_exact_fused_multiply_add() -> None:
    """The two-rounding trap: a * b + c exactly halfway between two float32 values in float64, off it exactly."""
    one, eps = np.float32(1.0), np.float32(2.0**-23)
    a = np.array([1.0 + 2.0**-12], np.float32)     # a * a = 1 + 2^-11 + 2^-24: the last term is half an ulp of 1 + 2^-11
    assert TO.fma(a, a, np.array([2.0**-60], np.float32))[0] == np.float32(1.0 + 2.0**-11) + eps   # just above: up
    assert TO.fma(a, a, np.array([-(2.0**-60)], np.float32))[0] == np.float32(1.0 + 2.0**-11)      # just below: down
    assert TO.fma(a, a, np.zeros(1, np.float32))[0] == np.float32(1.0 + 2.0**-11)                  # the tie: to even
    rng = np.random.default_rng(0)
    x, y, z = (rng.standard_normal(4096).astype(np.float32) for _ in range(3))
    exact = [float(np.float32(float(p) * float(q) + float(r))) for p, q, r in zip(x[:64], y[:64], z[:64])]
    assert np.allclose(TO.fma(x, y, z)[:64], exact, rtol=1e-7)
    assert TO.fma(one, one, -one) == 0


def test_oracle_equals_the_cuda_operations_adamw(golden) -> None:
    for case in range(4):
        lr, b1, b2, eps, wd = (float(v) for v in golden[f"adamw{case}_hyper"])
        for j in range(N_SHAPES):
            p = golden[f"adamw{case}_p0_{j}"]
            m, v = np.zeros_like(p), np.zeros_like(p)
            for step in range(1, 4):
                p, m, v = TO.adamw(p, golden[f"adamw{case}_g{step}_{j}"], m, v, lr=lr, beta1=b1, beta2=b2, eps=eps,
                                   weight_decay=wd, step=step)  # fmt: skip
                for name, got in (("p", p), ("m", m), ("v", v)):
                    assert same(got, golden[f"adamw{case}_{name}{step}_{j}"]), (case, j, step, name)


def test_oracle_equals_the_cuda_operations_unit_step(golden) -> None:
    for case in range(2):
        lr, b1, b2, eps, wd = (float(v) for v in golden[f"units{case}_hyper"])
        for j in range(N_UNIT_SHAPES):
            p, m, v = (golden[f"units{case}_{k}0_{j}"] for k in "pmv")
            for step in (1, 2):
                p, m, v = TO.adamw_units(p, golden[f"units{case}_g{step}_{j}"], m, v, active=golden[f"units{case}_active{step}"],
                                         lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=wd,
                                         steps=golden[f"units{case}_steps{step}"])  # fmt: skip
                for name, got in (("p", p), ("m", m), ("v", v)):
                    assert same(got, golden[f"units{case}_{name}{step}_{j}"]), (case, j, step, name)


def test_oracle_equals_the_cuda_operations_other_passes(golden) -> None:
    for j in range(N_SHAPES):
        for case in range(4):
            got = TO.lerp(golden[f"lerp{case}_self_{j}"], golden[f"lerp{case}_end_{j}"], float(golden[f"lerp{case}_w"]))
            assert same(got, golden[f"lerp{case}_out_{j}"]), ("lerp", case, j)
        for case in range(3):
            assert same(TO.scale64(golden[f"scale{case}_in_{j}"], golden[f"scale{case}_c"]), golden[f"scale{case}_out_{j}"])
            scale, clipped = golden[f"limit{case}_decision"]
            osq, dsq = TO.limit_squares(golden[f"limit{case}_param_{j}"], golden[f"limit{case}_old_{j}"])
            assert same(osq, golden[f"limit{case}_oldsq_{j}"]) and same(dsq, golden[f"limit{case}_deltasq_{j}"])
            new, asq = TO.limit_project(golden[f"limit{case}_param_{j}"], golden[f"limit{case}_old_{j}"], scale, clipped != 0)
            assert same(new, golden[f"limit{case}_new_{j}"]) and same(asq, golden[f"limit{case}_appliedsq_{j}"])


def test_kernels_decline_cpu_tensors_and_switch_off() -> None:
    from hsn_b200.kernels import trainer

    t = [torch.zeros(8)]
    assert trainer.lerp(t, t, 0.5) is False and trainer.copy(t, t) is False
    assert trainer.adamw(t, t, t, t, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, step=1) is False
    previous = trainer.set_enabled(False)
    try:
        assert trainer.enabled() is False and trainer.ready(torch.device("cpu")) is False
    finally:
        trainer.set_enabled(previous)


# ------------------------------------------------------------------------------------------------ GPU


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _np(t):
    return t.detach().cpu().numpy()


@pytest.mark.gpu
def test_kernels_equal_the_fixtures(golden) -> None:
    from hsn_b200.kernels import trainer

    for case in range(4):
        lr, b1, b2, eps, wd = (float(v) for v in golden[f"adamw{case}_hyper"])
        ps = [_dev(golden[f"adamw{case}_p0_{j}"]) for j in range(N_SHAPES)]
        ms, vs = [torch.zeros_like(p) for p in ps], [torch.zeros_like(p) for p in ps]
        for step in range(1, 4):
            gs = [_dev(golden[f"adamw{case}_g{step}_{j}"]) for j in range(N_SHAPES)]
            assert trainer.adamw(ps, gs, ms, vs, lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=wd, step=step)
            for j in range(N_SHAPES):
                for name, got in (("p", ps), ("m", ms), ("v", vs)):
                    assert same(_np(got[j]), golden[f"adamw{case}_{name}{step}_{j}"]), (case, j, step, name)
    for case in range(2):
        lr, b1, b2, eps, wd = (float(v) for v in golden[f"units{case}_hyper"])
        ps, ms, vs = ([_dev(golden[f"units{case}_{k}0_{j}"]) for j in range(N_UNIT_SHAPES)] for k in "pmv")
        for step in (1, 2):
            active = golden[f"units{case}_active{step}"].astype(bool)
            steps = golden[f"units{case}_steps{step}"].astype(np.float64)
            with np.errstate(divide="ignore", invalid="ignore"):
                size = np.where(active, lr / (1 - np.power(b1, steps)), 0.0).astype(np.float32)
                root = np.where(active, np.power(1 - np.power(b2, steps), 0.5), 1.0).astype(np.float32)
            gs = [_dev(golden[f"units{case}_g{step}_{j}"]) for j in range(N_UNIT_SHAPES)]
            assert trainer.adamw_units(ps, gs, ms, vs, n_units=8, active=active.tolist(),
                                       decay=[1 - lr * wd if on else 1.0 for on in active], lerp_weight=[1 - b1 if on else 0.0 for on in active],
                                       beta2_factor=[b2 if on else 1.0 for on in active], bias_correction2_sqrt=root.tolist(),
                                       step_size=size.tolist(), beta2=b2, eps=eps, weight_decay=wd)  # fmt: skip
            for j in range(N_UNIT_SHAPES):
                for name, got in (("p", ps), ("m", ms), ("v", vs)):
                    assert same(_np(got[j]), golden[f"units{case}_{name}{step}_{j}"]), (case, j, step, name)
    for case in range(4):
        selfs = [_dev(golden[f"lerp{case}_self_{j}"]) for j in range(N_SHAPES)]
        assert trainer.lerp(selfs, [_dev(golden[f"lerp{case}_end_{j}"]) for j in range(N_SHAPES)], float(golden[f"lerp{case}_w"]))
        assert all(same(_np(selfs[j]), golden[f"lerp{case}_out_{j}"]) for j in range(N_SHAPES))
    for case in range(3):
        grads = [_dev(golden[f"scale{case}_in_{j}"]) for j in range(N_SHAPES)]
        assert trainer.scale64(grads, torch.tensor(float(golden[f"scale{case}_c"]), dtype=torch.float64, device="cuda"))
        assert all(same(_np(grads[j]), golden[f"scale{case}_out_{j}"]) for j in range(N_SHAPES))
        params = [_dev(golden[f"limit{case}_param_{j}"]) for j in range(N_SHAPES)]
        olds = [_dev(golden[f"limit{case}_old_{j}"]) for j in range(N_SHAPES)]
        a, b = [torch.empty_like(p) for p in params], [torch.empty_like(p) for p in params]
        assert trainer.limit_squares(params, olds, a, b)
        assert all(same(_np(a[j]), golden[f"limit{case}_oldsq_{j}"]) and same(_np(b[j]), golden[f"limit{case}_deltasq_{j}"]) for j in range(N_SHAPES))
        group = _dev(golden[f"limit{case}_decision"])
        assert trainer.limit_project(params, olds, a, [group] * N_SHAPES)
        assert all(same(_np(params[j]), golden[f"limit{case}_new_{j}"]) and same(_np(a[j]), golden[f"limit{case}_appliedsq_{j}"]) for j in range(N_SHAPES))
        saved = [torch.empty_like(p) for p in params]
        assert trainer.copy(saved, params) and all(same(_np(s), _np(p)) for s, p in zip(saved, params))


@pytest.mark.gpu
@pytest.mark.parametrize("weight_decay", [0.0, 0.01])
def test_dense_step_equals_the_live_multi_tensor_step(weight_decay: float) -> None:
    """Forty steps of 53 tensors (more than one launch holds; odd sizes, a 70001-element tensor, views that do
    not start on a 16-byte boundary) against torch's multi-tensor operations on the same device."""
    from hsn_b200.kernels import trainer

    gen = torch.Generator().manual_seed(1)
    shapes = [(256, 64), (512, 192), (8, 202), (1, 128), (512,), (8,), (1,), (3, 5, 7), (129,), (70001,)] + [(17 + k,) for k in range(43)]

    def values(shape, scale):
        x = torch.randn(*shape, generator=gen) * scale
        if x.numel() >= 8:
            x.view(-1)[:6] = torch.tensor([0.0, -0.0, 1e-42, -1e-40, 1e30, -3e-30])
        return x

    def odd(t):   # the same values in storage that starts 4 bytes after a 16-byte boundary
        pad = torch.empty(t.numel() + 1, device="cuda")
        view = pad[1:].view(t.shape)
        view.copy_(t)
        return view

    ref = [values(s, 0.1).cuda() for s in shapes]
    fast = [odd(p) if k % 3 == 1 else p.clone() for k, p in enumerate(ref)]
    state_ref = [[torch.zeros_like(p) for p in ref] for _ in range(2)]
    state_fast = [[odd(torch.zeros_like(p)) if k % 3 == 2 else torch.zeros_like(p) for k, p in enumerate(ref)] for _ in range(2)]
    lr, b1, b2, eps = 2.5e-3, 0.9, 0.999, 1e-8
    for step in range(1, 41):
        grads = [values(s, (1e-3, 1.0, 30.0, 1e-9)[step % 4]).cuda() for s in shapes]
        if weight_decay != 0:
            torch._foreach_mul_(ref, 1 - lr * weight_decay)
        torch._foreach_lerp_(state_ref[0], grads, 1 - b1)
        torch._foreach_mul_(state_ref[1], b2)
        torch._foreach_addcmul_(state_ref[1], grads, grads, value=1 - b2)
        den = torch._foreach_sqrt(state_ref[1])
        torch._foreach_div_(den, (1 - b2**step) ** 0.5)
        torch._foreach_add_(den, eps)
        torch._foreach_addcdiv_(ref, state_ref[0], den, value=-(lr / (1 - b1**step)))
        assert trainer.adamw(fast, grads, state_fast[0], state_fast[1], lr=lr, beta1=b1, beta2=b2, eps=eps,
                             weight_decay=weight_decay, step=step)  # fmt: skip
        for k in range(len(shapes)):
            assert same(_np(fast[k]), _np(ref[k])), (step, k)
    for k in range(len(shapes)):
        assert same(_np(state_fast[0][k]), _np(state_ref[0][k])) and same(_np(state_fast[1][k]), _np(state_ref[1][k]))


@pytest.mark.gpu
def test_kernels_equal_the_oracle_at_other_sizes_and_decline_what_they_cannot_take() -> None:
    from hsn_b200.kernels import trainer

    rng = np.random.default_rng(2)
    shapes = [(5000,), (1023,), (1025,), (4, 300)]
    a = [rng.standard_normal(s).astype(np.float32) for s in shapes]
    b = [rng.standard_normal(s).astype(np.float32) for s in shapes]
    for w in (0.01, 0.75):
        selfs = [_dev(x) for x in a]
        assert trainer.lerp(selfs, [_dev(x) for x in b], w)
        assert all(same(_np(s), TO.lerp(x, y, w)) for s, x, y in zip(selfs, a, b))
    # non-contiguous, half precision, another element count: nothing is launched, nothing is touched
    wide = _dev(rng.standard_normal((8, 8)).astype(np.float32))
    before = wide.clone()
    assert trainer.lerp([wide.t()], [wide.t()], 0.5) is False
    assert trainer.lerp([wide.half()], [wide.half()], 0.5) is False
    assert trainer.lerp([wide], [wide[:4]], 0.5) is False
    assert trainer.scale64([wide], torch.tensor(0.5, device="cuda")) is False          # the coefficient must be float64
    assert trainer.limit_project([wide], [wide], [wide.clone()], [torch.zeros(3, device="cuda")]) is False
    assert torch.equal(wide, before)
    empty = torch.empty(0, device="cuda")
    assert trainer.copy([empty, wide.clone()], [empty, wide]) is True                  # tensors without elements are skipped


def test_shards_are_whole_16_byte_groups() -> None:
    from hsn_b200.parallel import shard_elements

    assert shard_elements(1, 1) == 4 and shard_elements(8, 2) == 4 and shard_elements(9, 2) == 8
    assert shard_elements(1000003, 8) == 125004 and 8 * shard_elements(1000003, 8) >= 1000003
    with pytest.raises(ValueError):
        shard_elements(0, 2)


@pytest.mark.gpu
@pytest.mark.parametrize("world", [1, 2, 4])
def test_fused_exchange_equals_the_oracle_with_every_rank_on_one_device(world: int) -> None:
    """The ranks' buffers side by side on one GPU, each rank's kernel launched in turn (nothing in the kernel
    waits for another rank): after three steps every rank's parameter buffer holds the same bits, those of the
    oracle's rank-ordered sum, average and AdamW step."""
    from hsn_b200.parallel import ShardedAdamW, shard_elements

    rng = np.random.default_rng(7)
    n = 10007
    shard = shard_elements(n, world)
    hyper = dict(lr=2.5e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01)
    p0 = np.zeros(world * shard, np.float32)
    p0[:n] = rng.standard_normal(n).astype(np.float32) * 0.1
    grads = [torch.zeros(world * shard, device="cuda") for _ in range(world)]
    params = [_dev(p0) for _ in range(world)]
    ranks = [ShardedAdamW(n, lr=hyper["lr"], betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01, buffers=(grads, params), rank=r)
             for r in range(world)]  # fmt: skip
    p, m, v = p0, np.zeros_like(p0), np.zeros_like(p0)
    for step in range(1, 4):
        gs = [rng.standard_normal(world * shard).astype(np.float32) * (1e-3, 1.0, 30.0)[step - 1] for _ in range(world)]
        for r in range(world):
            grads[r].copy_(_dev(gs[r]))
        for opt in ranks:
            opt.step()
        p, m, v = TO.exchange_adamw(gs, p, m, v, step=step, **hyper)
        for r in range(world):
            assert same(_np(params[r]), p), (step, r)
        moments = np.concatenate([_np(opt.exp_avg) for opt in ranks])
        assert same(moments, m)
