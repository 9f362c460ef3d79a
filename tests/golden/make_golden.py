"""Generates the golden fixtures of this folder from the reference implementation itself.

Run where the reference checkout is available (it is NOT needed to run the tests):

    python tests/golden/make_golden.py --reference /path/to/hsn

It imports the reference's own CPU code (``python/hsn``) and dumps, for small seeded cases, the
inputs and outputs of every function on the window path as ``.npz`` files:

* ``select_*.npz``      ``Router.select`` (``python/hsn/model/router.py:1263``): tie-heavy logits, stale
                        ages, budget cuts, cost penalties, reserved slots.
* ``update_*.npz``      ``PDGCell.step_sparse`` + ``CellGraphState.tick``
                        (``python/hsn/model/cell.py:349``, ``python/hsn/model/state.py:316``) on the
                        products of ``PDGCell.sparse_products`` (``cell.py:507``).
* ``recurrence_*.npz``  ``recurrence_backward`` (``python/hsn/train/split.py:128``).
* ``window_*.npz``      a whole split window: the prologue's inputs, every weight, the eager sweep's
                        tape (``python/hsn/train/compile.py:1234``), the replay's record, the arguments
                        and results of ``state_gradient_backward``
                        (``python/hsn/train/state_gradient.py:357``) with its ``A``/``R`` trace.
* ``sweep_*.npz``       the three glue steps of ``ReverseSweep`` between its two products
                        (``python/hsn/train/state_sweep.py:441`` head, ``:487`` middle, ``:497`` tail)
                        on seeded buffers, two positions in sweep order, every written buffer before
                        and after each step.
* ``window_bf16_*.npz`` the same split window run under ``torch.autocast("cpu", dtype=torch.bfloat16)``, what
                        ``train.precision=bf16`` (``python/hsn/config.py:1113``) turns on through
                        ``python/hsn/train/amp.py:30-39``: every linear's operands and output in bfloat16,
                        state and norms in float32. Pins the oracle's ``bf16=True`` mode.
* ``prologue_*.npz``    ``HSN._window_prologue`` (``python/hsn/model/hsn.py:1707``): token and context ids in, ``z``,
                        the context embeddings and the scorer's scalars out, with the tables it reads.
* ``decode_*.npz``      ``HSN._decode`` (``python/hsn/model/hsn.py:2374``): the decoder on seeded ``q``, ``u``.
* ``snapshot_*.npz``    ``CellGraphState.snapshot`` (``python/hsn/model/state.py:363``): seeded states, their metas
                        and the reference's digests.
* ``replay_*.npz``      ``PDGCell.replay_sparse`` (``python/hsn/model/cell.py:655-734``) as the split window's replay
                        calls it (``python/hsn/train/split.py:657``), on that call's own arguments: inputs, results,
                        the record, the values at the cuts between its steps (the cell norm's input and output and
                        ``W_out``'s input with their gradients, the unit pass's own gradient of its input), the
                        graph's tables with the padded edge weights and their gradient, and autograd's gradients of
                        the inputs and of every cell parameter for seeded cotangents of ``(c, b)``.
* ``chain_*.npz``       two chained windows against the unsplit window of twice the length: the
                        carried state forward, the state cotangent ``(A, R)`` backward.

Nothing here is read at test time except the ``.npz`` files it wrote.
"""

from __future__ import annotations

import argparse
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def _import_reference(root: Path) -> None:
    stub = Path(tempfile.mkdtemp()) / "hsn-0.1.0.dist-info"
    stub.mkdir(parents=True)
    (stub / "METADATA").write_text("Metadata-Version: 2.1\nName: hsn\nVersion: 0.1.0\n")
    sys.path[:0] = [str(stub.parent), str(root / "python"), str(root / "tests")]


def _np(x):
    import torch

    if isinstance(x, torch.Tensor):
        x = x.detach().cpu()
        if x.dtype == torch.bool:
            return x.numpy().astype(np.uint8)
        if x.dtype == torch.bfloat16:
            return x.float().numpy()
        return x.numpy()
    return np.asarray(x)


def _cfg(root: Path, *, B, T, N, d, K, H, M, D, fd, extra=(), precision="fp32"):
    from hsn.config import load_config

    return load_config(
        root / "configs" / "ref_a1.yaml",
        overrides=[
            "profile=cpu",
            f"model.d={d}",
            f"model.context_dim={d}",
            f"model.n_cells={N}",
            f"model.in_degree={D}",
            f"model.n_units={M}",
            f"model.k_select={K}",
            f"model.hidden={H}",
            "model.routing=topk",
            "train.gate_mode=ste",
            "model.key_address=true",
            "model.selected_readout=true",
            "model.cand_norm=rms",
            "model.budget=1.0",
            "model.lambda_cost=0",
            "model.init=trunc_normal_0.02",
            "model.state_init=trunc_normal_0.02",
            f"train.unroll={T}",
            f"train.batch={B}",
            f"train.micro_batch={B}",
            f"train.precision={precision}",
            f"train.feedback_detach={fd}",
            *extra,
        ],
    )


def _model(cfg, dtype, perturb: float):
    import torch
    from hsn.device import seed_everything
    from hsn.model.hsn import HSN

    seed_everything(0)
    model = HSN.from_config(cfg).to(dtype)
    if perturb:
        with torch.no_grad():
            for p in model.parameters():
                p.add_(perturb * torch.randn_like(p))
    return model.train()


def _weights(model) -> dict[str, np.ndarray]:
    """Every weight the window reads, in torch's own layouts (``nn.Linear``: ``[out, in]``)."""
    from hsn.model.router import BUDGET_SLACK

    cell, router = model.cell, model.router
    scorer = model.scorer
    with cell.window():
        edge_w = cell.graph._padded_weights().detach().clone()
    out = {
        "s_w1": model.shared.fc1.weight, "s_b1": model.shared.fc1.bias,
        "s_w2": model.shared.fc2.weight, "s_b2": model.shared.fc2.bias,
        "p_w1": model.predictor.fc1.weight, "p_b1": model.predictor.fc1.bias,
        "p_w2": model.predictor.fc2.weight, "p_b2": model.predictor.fc2.bias,
        "score_w": scorer.net.weight, "score_b": scorer.net.bias,
        "v_w": cell.V.weight, "wout_w": cell.W_out.weight,
        "gate_w": cell.gate.weight, "gate_b": cell.gate.bias,
        "norm_w": cell.norm.weight, "cand_w": cell.cand_norm.weight,
        "w1": cell.units.W1, "b1": cell.units.b1, "w2": cell.units.W2, "b2": cell.units.b2,
        "pad_src": cell.graph._pad_src, "edge_w": edge_w, "cost": router.cost_table,
    }  # fmt: skip
    out = {k: _np(v) for k, v in out.items()}
    out["scalars_f"] = np.array(
        [
            float(router.age_max),
            float(router.lambda_cost),
            float(router.cell_overhead),
            float(router.shared_cost),
            float(model.cfg.budget) * (1.0 + BUDGET_SLACK),
            float(cell.norm.eps),
            float(cell.cand_norm.eps),
        ],
        dtype=np.float64,
    )
    return out


# --------------------------------------------------------------------------------------------------


def make_select(root: Path) -> None:
    import torch
    from hsn.model.router import BUDGET_SLACK
    from test_a6_feedback_detach import A5, ALL, _cfg as ref_cfg, _model as ref_model

    sets = {
        "plain": (),
        "probes": ("model.age_max=2",),
        "budget": ("model.budget=0.1",),
        "probes_budget": ("model.age_max=2", "model.budget=0.1"),
        "cost": ("model.lambda_cost=0.05", "model.age_max=3"),
    }
    for name, overrides in sets.items():
        cfg = ref_cfg(*A5, ALL, "model.cand_norm=rms", *overrides)
        router = ref_model(cfg).router.to(dtype=torch.float32)
        N, M, K = cfg.model.n_cells, cfg.model.n_units, cfg.model.k_select
        g = torch.Generator().manual_seed(7)
        out: dict[str, np.ndarray] = {}
        n = 0
        for trial in range(40):
            B = 1 + trial % 5
            logits = torch.randn(B, N, M, generator=g)
            if trial % 2:
                logits = (logits * 2).round() / 2
            age = torch.randint(0, 2 * int(router.age_max) + 2, (B, N), generator=g)
            if trial % 3 == 0:
                age = (age // 3) * 3
            for probes in (True, False):
                want = router.select(
                    logits, cfg.model.budget, K, cfg.model.k_min, "topk", gate=None,
                    age=age if probes else None,
                )  # fmt: skip
                pre = f"t{n}_"
                out[pre + "logits"] = _np(logits)
                out[pre + "age"] = _np(age)
                out[pre + "probes"] = np.array(int(probes))
                out[pre + "cells"] = _np(want.cell_idx)
                out[pre + "units"] = _np(want.unit_idx)
                out[pre + "valid"] = _np(want.valid)
                out[pre + "theta"] = _np(want.threshold)
                out[pre + "refreshed"] = _np(want.refreshed)
                n += 1
        out["n"] = np.array(n)
        out["cost"] = _np(router.cost_table)
        out["params"] = np.array(
            [
                K,
                int(router.age_max),
                float(router.lambda_cost),
                float(router.cell_overhead),
                float(router.shared_cost),
                float(cfg.model.budget) * (1.0 + BUDGET_SLACK),
            ],
            dtype=np.float64,
        )
        np.savez_compressed(HERE / f"select_{name}.npz", **out)
    # amendment A8's reserved slots (router.py:1640-1648): a larger router, fixed and free units
    cfg = _cfg(root, B=2, T=4, N=12, d=8, K=5, H=8, M=4, D=2, fd="[summary,eps,state,router]",
               extra=("model.age_max=2",))  # fmt: skip
    router = _model(cfg, torch.float32, 0.3).router
    g = torch.Generator().manual_seed(9)
    out = {}
    n = 0
    for trial in range(16):
        logits = (torch.randn(3, 12, 4, generator=g) * 2).round() / 2
        age = torch.randint(0, 6, (3, 12), generator=g)
        for fixed_units in (False, True):
            want = router.select(
                logits, cfg.model.budget, 5, cfg.model.k_min, "topk", gate=None, age=age,
                reserved=2, reserved_units=fixed_units,
            )  # fmt: skip
            pre = f"t{n}_"
            out[pre + "logits"] = _np(logits)
            out[pre + "age"] = _np(age)
            out[pre + "probes"] = np.array(1)
            out[pre + "fixed_units"] = np.array(int(fixed_units))
            out[pre + "cells"] = _np(want.cell_idx)
            out[pre + "units"] = _np(want.unit_idx)
            out[pre + "valid"] = _np(want.valid)
            out[pre + "theta"] = _np(want.threshold)
            out[pre + "refreshed"] = _np(want.refreshed)
            n += 1
    out["n"] = np.array(n)
    out["cost"] = _np(router.cost_table)
    out["params"] = np.array(
        [5, int(router.age_max), float(router.lambda_cost), float(router.cell_overhead),
         float(router.shared_cost), float(cfg.model.budget) * (1.0 + BUDGET_SLACK), 2],
        dtype=np.float64,
    )  # fmt: skip
    np.savez_compressed(HERE / "select_reserved.npz", **out)


def make_update(root: Path) -> None:
    import torch
    from test_a6_feedback_detach import A5, ALL, _cfg as ref_cfg, _model as ref_model

    sets = {
        "rms": ("model.cand_norm=rms",),
        "none": ("model.cand_norm=none",),
        "budget": ("model.cand_norm=rms", "model.budget=0.1"),
    }
    for name, extra in sets.items():
        cfg = ref_cfg(*A5, ALL, *extra)
        model = ref_model(cfg).to(dtype=torch.float32)
        cell, router = model.cell, model.router
        N, d, K = cfg.model.n_cells, cfg.model.d, cfg.model.k_select
        g = torch.Generator().manual_seed(11)
        B = 5
        state = model.init_state(B)
        out: dict[str, np.ndarray] = {}
        with torch.no_grad(), cell.window():
            consts = cell.window_consts()
            for step in range(12):
                u = torch.randn(B, d, generator=g)
                eps = torch.randn(B, d, generator=g)
                logits = torch.randn(B, N, cfg.model.n_units, generator=g)
                sel = router.select(logits, cfg.model.budget, K, cfg.model.k_min, "topk", gate=None)
                _, info = cell.step_sparse(u, eps, state, sel, static=True, consts=consts)
                want = info["state"].tick(info["selected"])
                gate, y = cell.sparse_products(
                    u, eps, state, sel.cell_idx, sel.unit_idx, sel.valid, consts
                )
                pre = f"s{step}_"
                for key, value in (
                    ("y", y), ("gate", gate), ("h", state.h), ("q", state.q), ("age", state.age),
                    ("pos", state.pos), ("cells", sel.cell_idx), ("valid", sel.valid),
                    ("h_next", want.h), ("q_next", want.q), ("age_next", want.age),
                    ("pos_next", want.pos),
                ):  # fmt: skip
                    out[pre + key] = _np(value)
                state = want
        out["n"] = np.array(12)
        out["cand_w"] = _np(cell.cand_norm.weight if name != "none" else cell.norm.weight)
        out["cand_norm"] = np.array(int(name != "none"))
        out["cand_eps"] = np.array(float(cell.cand_norm.eps) if name != "none" else 0.0)
        np.savez_compressed(HERE / f"update_{name}.npz", **out)


def make_recurrence(root: Path) -> None:
    import torch
    from hsn.train.split import dense_recurrence_backward, recurrence_backward

    shapes = {"a": (3, 7, 5, 3, 4), "b": (1, 1, 2, 1, 1), "c": (3, 9, 9, 9, 37), "d": (2, 6, 40, 6, 20)}
    for name, (B, T, N, K, d) in shapes.items():
        g = torch.Generator().manual_seed(B + T + N + K + d)
        cells = torch.stack(
            [torch.stack([torch.randperm(N, generator=g)[:K] for _ in range(T)]) for _ in range(B)]
        )
        valid = torch.rand(B, T, K, generator=g) > 0.25
        reset = torch.rand(B, T, generator=g) < 0.05
        case = {
            "c": torch.rand(B, T, K, d, generator=g, dtype=torch.float64) * 2 - 1,
            "b": torch.rand(B, T, K, d, generator=g, dtype=torch.float64),
            "h_old": torch.rand(B, T, K, d, generator=g, dtype=torch.float64) * 2 - 1,
            "cells": torch.where(valid, cells, torch.zeros_like(cells)),
            "valid": valid,
            "reset": reset,
            "pre": torch.randn(B, T, d, generator=g, dtype=torch.float64),
            "post": torch.randn(B, T, d, generator=g, dtype=torch.float64),
            "sel": torch.randn(B, T, K, d, generator=g, dtype=torch.float64),
        }
        out = {k: _np(v) for k, v in case.items()}
        out["N"] = np.array(N)
        for tag, present in (("111", (1, 1, 1)), ("010", (0, 1, 0)), ("101", (1, 0, 1))):
            cots = [case[k] if on else None for k, on in zip(("pre", "post", "sel"), present)]
            dc, db = recurrence_backward(
                case["c"], case["b"], case["h_old"], case["cells"], valid, reset, N, *cots
            )
            out[f"dc_{tag}"], out[f"db_{tag}"] = _np(dc), _np(db)
        # the dense-fallback rows' recurrence (split.py:177): every cell is a slot
        cN = torch.rand(B, T, N, d, generator=g, dtype=torch.float64) * 2 - 1
        bN = torch.rand(B, T, N, d, generator=g, dtype=torch.float64)
        hN = torch.rand(B, T, N, d, generator=g, dtype=torch.float64) * 2 - 1
        dcN, dbN = dense_recurrence_backward(cN, bN, hN, reset, N, case["pre"], case["post"])
        out.update(dense_c=_np(cN), dense_b=_np(bN), dense_h=_np(hN), dense_dc=_np(dcN), dense_db=_np(dbN))
        np.savez_compressed(HERE / f"recurrence_{name}.npz", **out)


def _run_window(root, cfg, model, dtype, tokens, ctx, reset, state, *, initial=None, cot_seed=5):
    """One split window of the reference on the CPU, every intermediate captured."""
    import torch
    import hsn.train.split as split
    import hsn.train.state_gradient as sg
    from hsn.train.split import SplitWindow

    captured: dict[str, object] = {}
    real_tape, real_sweep, real_rec = split.run_tape, sg.state_gradient_backward, split.recurrence_backward
    real_prologue = model._window_prologue

    def tape_spy(*args, **kwargs):
        tape = real_tape(*args, **kwargs)
        captured["tape"] = {k: v.clone() for k, v in tape.items()}
        return tape

    def prologue_spy(*args, **kwargs):
        pro = real_prologue(*args, **kwargs)
        captured["pro"] = pro
        return pro

    def sweep_spy(*args, **kwargs):
        trace: dict[str, torch.Tensor] = {}
        kwargs = dict(kwargs, trace=trace, initial=initial)
        result = real_sweep(*args, **kwargs)
        captured["sweep_args"] = args
        captured["sweep_out"] = result
        captured["trace"] = trace
        return result

    def rec_spy(*args):
        result = real_rec(*args)
        captured["rec_args"] = args
        captured["rec_out"] = result
        return result

    split.run_tape, sg.state_gradient_backward, split.recurrence_backward = tape_spy, sweep_spy, rec_spy
    model._window_prologue = prologue_spy
    try:
        win = SplitWindow(model, cfg, None)
        logits, final, info = win(tokens, ctx, state, reset)
        g = torch.Generator().manual_seed(cot_seed)
        weight = torch.randn(logits.shape, generator=g, dtype=torch.float64).to(logits.dtype)
        loss = (logits * weight).sum() / logits.shape[0]
        model.zero_grad(set_to_none=True)
        loss.backward()
    finally:
        split.run_tape, sg.state_gradient_backward, split.recurrence_backward = real_tape, real_sweep, real_rec
        model._window_prologue = real_prologue
    captured["final"] = final
    captured["logits"] = logits.detach()
    return captured


def _dump_window(path: Path, model, cap, reset, state) -> None:
    pro = cap["pro"]
    out = {f"w_{k}": v for k, v in _weights(model).items()}
    out.update(
        z=_np(pro.z), ctx=_np(pro.context), scalars=_np(pro.scalars), reset=_np(reset),
        h0=_np(state.h), q0=_np(state.q), age0=_np(state.age), pos0=_np(state.pos),
    )  # fmt: skip
    for key, value in cap["tape"].items():
        out[f"tape_{key}"] = _np(value)
    if "sweep_args" in cap:
        (c, b, h_old, cells, units, valid, rst, n_cells, d_q_pre, d_q_post, d_h_sel, d_h_fast,
         record, consts) = cap["sweep_args"]  # fmt: skip
        out.update(
            bw_c=_np(c), bw_b=_np(b), bw_h_old=_np(h_old), bw_cells=_np(cells), bw_units=_np(units),
            bw_valid=_np(valid), bw_dc=_np(cap["sweep_out"][0]), bw_db=_np(cap["sweep_out"][1]),
            bw_A=_np(cap["trace"]["A"]), bw_R=_np(cap["trace"]["R"]),
            bw_dh=_np(cap["trace"]["dh"]), bw_dvm=_np(cap["trace"]["dvm"]),
        )  # fmt: skip
        for name, cot in (("d_q_pre", d_q_pre), ("d_q_post", d_q_post), ("d_h_sel", d_h_sel)):
            if cot is not None:
                out[f"bw_{name}"] = _np(cot)
        for key, value in record.items():
            out[f"rec_{key}"] = _np(value)
    if "rec_args" in cap:
        c, b, h_old, cells, valid, rst, n_cells, d_q_pre, d_q_post, d_h_sel = cap["rec_args"]
        out.update(
            bw_c=_np(c), bw_b=_np(b), bw_h_old=_np(h_old), bw_cells=_np(cells), bw_valid=_np(valid),
            bw_dc=_np(cap["rec_out"][0]), bw_db=_np(cap["rec_out"][1]),
        )  # fmt: skip
        for name, cot in (("d_q_pre", d_q_pre), ("d_q_post", d_q_post), ("d_h_sel", d_h_sel)):
            if cot is not None:
                out[f"bw_{name}"] = _np(cot)
    np.savez_compressed(path, **out)


def _inputs(cfg, B, T, p_reset, seed=1):
    import torch

    g = torch.Generator().manual_seed(seed)
    tokens = torch.randint(0, cfg.model.vocab_size, (B, T), generator=g)
    ctx = torch.randint(0, cfg.model.n_context, (B, T), generator=g)
    reset = torch.rand(B, T, generator=g) < p_reset
    reset[:, 0] = True
    return tokens, ctx, reset


def make_windows(root: Path) -> None:
    import torch

    SG, FULL = "[summary,eps,router]", "[summary,eps,state,router]"
    cases = {
        # config 1 of the benchmark contract: B2 T8 N16 d32 K2 H32, M2 D2, resets p=0.1
        "c1_f32": dict(shape=dict(B=2, T=8, N=16, d=32, K=2, H=32, M=2, D=2), fd=SG, dtype="f32", perturb=0.0, p=0.1),
        "c1_f64": dict(shape=dict(B=2, T=8, N=16, d=32, K=2, H=32, M=2, D=2), fd=SG, dtype="f64", perturb=0.0, p=0.1),
        # the same with every path live (weights away from their init), fp64 and fp32
        "c1p_f64": dict(shape=dict(B=2, T=8, N=16, d=32, K=2, H=32, M=2, D=2), fd=SG, dtype="f64", perturb=0.3, p=0.1),
        "c1p_f32": dict(shape=dict(B=2, T=8, N=16, d=32, K=2, H=32, M=2, D=2), fd=SG, dtype="f32", perturb=0.3, p=0.1),
        # the refresh probes fire (age_max 2) and the budget pads slots
        "probes_f64": dict(shape=dict(B=3, T=12, N=12, d=16, K=3, H=24, M=3, D=2), fd=SG, dtype="f64", perturb=0.3, p=0.15,
                           extra=("model.age_max=2",)),
        "budget_f64": dict(shape=dict(B=3, T=10, N=12, d=16, K=4, H=24, M=3, D=3), fd=SG, dtype="f64", perturb=0.3, p=0.1,
                           extra=("model.budget=0.06",)),
        # odd sizes: nothing a power of two
        "odd_f64": dict(shape=dict(B=3, T=7, N=11, d=12, K=3, H=20, M=3, D=2), fd=SG, dtype="f64", perturb=0.3, p=0.2),
        # the full feedback cut (the plain recurrence of split.py:128)
        "cut_f64": dict(shape=dict(B=2, T=8, N=16, d=32, K=2, H=32, M=2, D=2), fd=FULL, dtype="f64", perturb=0.3, p=0.1),
        # a mid-sized fp32 case closer to the reference shape's proportions
        "mid_f32": dict(shape=dict(B=2, T=12, N=64, d=32, K=8, H=64, M=8, D=4), fd=SG, dtype="f32", perturb=0.0, p=0.05,
                        extra=("model.age_max=1000000",)),
    }  # fmt: skip
    for name, case in cases.items():
        shape = case["shape"]
        dtype = torch.float64 if case["dtype"] == "f64" else torch.float32
        cfg = _cfg(root, **shape, fd=case["fd"], extra=case.get("extra", ()),
                   precision="fp64" if dtype == torch.float64 else "fp32")  # fmt: skip
        model = _model(cfg, dtype, case["perturb"])
        tokens, ctx, reset = _inputs(cfg, shape["B"], shape["T"], case["p"])
        state = model.init_state(shape["B"])
        cap = _run_window(root, cfg, model, dtype, tokens, ctx, reset, state)
        _dump_window(HERE / f"window_{name}.npz", model, cap, reset, state)
        print(name, "ok")


def make_windows_bf16(root: Path) -> None:
    """Windows under bf16 autocast on the CPU, at shapes the per-row cluster kernels take (hidden width
    a multiple of 128, state width 32 or 64): one block a row, and two blocks a row with the
    128-byte-swizzled operand tiles. The refresh probes fire in the first."""
    import torch

    SG = "[summary,eps,router]"
    cases = {
        "bf16_a": dict(shape=dict(B=3, T=8, N=64, d=32, K=4, H=128, M=4, D=3), perturb=0.3, p=0.15,
                       extra=("model.age_max=3",)),
        "bf16_b": dict(shape=dict(B=2, T=6, N=64, d=64, K=8, H=256, M=4, D=4), perturb=0.1, p=0.1,
                       extra=("model.age_max=1000000",)),
    }  # fmt: skip
    for name, case in cases.items():
        shape = case["shape"]
        cfg = _cfg(root, **shape, fd=SG, extra=case["extra"], precision="bf16")
        model = _model(cfg, torch.float32, case["perturb"])
        tokens, ctx, reset = _inputs(cfg, shape["B"], shape["T"], case["p"])
        state = model.init_state(shape["B"])
        with torch.autocast("cpu", dtype=torch.bfloat16):
            cap = _run_window(root, cfg, model, torch.float32, tokens, ctx, reset, state)
        _dump_window(HERE / f"window_{name}.npz", model, cap, reset, state)
        print(name, "ok")


def make_prologue(root: Path) -> None:
    """``HSN._window_prologue`` on seeded token and context ids: the weights and buffers it reads and
    what the sweep takes from it (``z``, the context embeddings, the scorer's scalars), for a fresh
    stream, for a carried position with carried previous bytes and non-zero running averages, and under
    bf16 autocast."""
    import torch
    from hsn.model.state import CellGraphState

    shape = dict(B=3, T=10, N=12, d=16, K=3, H=24, M=3, D=2)
    for name, precision, carried in (("fresh_f32", "fp32", False), ("carried_f32", "fp32", True), ("fresh_bf16", "bf16", False)):
        cfg = _cfg(root, **shape, fd="[summary,eps,router]", precision=precision)
        model = _model(cfg, torch.float32, 0.3)
        tokens, ctx, reset = _inputs(cfg, shape["B"], shape["T"], 0.2, seed=7)
        state = model.init_state(shape["B"])
        prev = None
        if carried:
            g = torch.Generator().manual_seed(11)
            reset[:, 0] = False
            state = CellGraphState._make(h=state.h, q=state.q, age=state.age,
                                         pos=torch.randint(0, 500, (shape["B"],), generator=g))  # fmt: skip
            prev = torch.randint(0, cfg.model.vocab_size, (shape["B"],), generator=g)
            with torch.no_grad():
                model.scorer.ema_utility.copy_(torch.rand(shape["N"], generator=g))
                model.scorer.ema_selected.copy_(torch.rand(shape["N"], generator=g))
        ctxm = torch.autocast("cpu", dtype=torch.bfloat16) if precision == "bf16" else torch.autocast("cpu", enabled=False)
        with torch.no_grad(), ctxm:
            pro = model._window_prologue(tokens, ctx, state, reset, "topk", reset_first=True, prev_tokens=prev, steps=False)
        sc = model.scorer
        out = dict(
            tokens=_np(tokens), ctx_ids=_np(ctx), reset=_np(reset), pos0=_np(state.pos),
            byte_emb=_np(model.byte_emb.weight if hasattr(model.byte_emb, "weight") else model.byte_emb.emb.weight),
            enc_w1=_np(model.encoder.fc1.weight), enc_b1=_np(model.encoder.fc1.bias),
            enc_w2=_np(model.encoder.fc2.weight), enc_b2=_np(model.encoder.fc2.bias),
            ctx_emb=_np(model.ctx_emb.weight if hasattr(model.ctx_emb, "weight") else model.ctx_emb.emb.weight),
            byte_codes=_np(sc.byte_codes), cell_addresses=_np(sc.cell_addresses),
            ema_utility=_np(sc.ema.utility), ema_selected=_np(sc.ema.selected),
            numbers=np.array([float(cfg.model.budget), 0.0 / sc.r_max, float(sc.n_context), float(sc.unroll)], dtype=np.float64),
            position=np.array(str(sc.position)),
            z=_np(pro.z), context=_np(pro.context), scalars=_np(pro.scalars),
        )  # fmt: skip
        if prev is not None:
            out["prev_tokens"] = _np(prev)
        np.savez_compressed(HERE / f"prologue_{name}.npz", **out)
        print("prologue", name, "ok")


def make_chain(root: Path) -> None:
    """Two chained windows of T positions against one window of 2T: the forward carry is the
    final state; the backward carry is the unsplit sweep's (A, R) at position T (what the second
    window's sweep ends with), given to the first window's sweep as ``initial``."""
    import torch
    from hsn.model.state import CellGraphState

    shape = dict(B=2, N=12, d=16, K=3, H=24, M=3, D=2)
    T = 6
    for name, dtype in (("f64", torch.float64),):
        cfg2 = _cfg(root, **shape, T=2 * T, fd="[summary,eps,router]", precision="fp64")
        model = _model(cfg2, dtype, 0.3)
        tokens, ctx, reset = _inputs(cfg2, shape["B"], 2 * T, 0.1)
        g = torch.Generator().manual_seed(2)
        zero = model.init_state(shape["B"])
        h = (0.5 * torch.rand(zero.h.shape, generator=g, dtype=torch.float64) - 0.25).to(dtype)
        reset[:, 0] = False  # a carried, non-zero start state
        start = CellGraphState._make(h=h, q=h.mean(dim=1), age=zero.age, pos=zero.pos)
        whole = _run_window(root, cfg2, model, dtype, tokens, ctx, reset, start)
        _dump_window(HERE / f"chain_{name}.npz", model, whole, reset, start)
        print("chain", name, "ok")


SWEEP_WRITTEN = ("A", "R", "dc", "db", "op1", "op1_fast", "op2", "op2_fast", "sigma")
SWEEP_READ = (
    "c", "b", "h_old", "y", "gate_pre", "mv", "rms", "hidden", "cells", "units", "valid", "reset",
    "d_q_pre", "d_q_post", "d_h_sel", "d_h_fast", "cand_gain", "gate_bias", "b1", "out_tgt", "out_w",
)  # fmt: skip


def make_sweep(root: Path) -> None:
    """The reverse sweep's glue steps on their own: a ``ReverseSweep`` on the CPU (its PyTorch
    steps are the kernels' contract), its buffers filled from a seed, then for the positions
    ``T - 1`` and ``T - 2``: head, middle (after new ``act_r``/``act_f``), tail (after new
    ``dv_r``/``dv_f``). Every written buffer is stored after every step."""
    import types

    import torch
    from hsn.train.state_sweep import ReverseSweep, SweepShape, out_adjacency

    cases = {
        # name: (B, T, K, N, d, H, M, n_fast, n_read, D, product dtype, cand norm, cell norm, act)
        "plain_f32": (3, 3, 4, 12, 8, 16, 3, 0, 0, 3, torch.float32, True, True, "gelu"),
        "fast_bf16": (2, 3, 5, 10, 8, 16, 2, 1, 2, 2, torch.bfloat16, False, False, "silu"),
        "fast2_bf16": (3, 2, 4, 9, 16, 32, 3, 2, 1, 4, torch.bfloat16, True, True, "tanh"),
        "relu_f32": (2, 3, 3, 7, 4, 8, 2, 0, 3, 2, torch.float32, True, False, "relu"),
    }
    for name, (B, T, K, N, d, H, M, F, n_read, D, pdt, cand, cell, act) in cases.items():
        gen = torch.Generator().manual_seed(len(name) * 7 + B)
        pad_src = torch.randint(0, N, (N, D), generator=gen)
        pad_mask = torch.rand(N, D, generator=gen) < 0.8
        out_tgt, out_edge = out_adjacency(pad_src, pad_mask)
        d_out = int(out_tgt.shape[1])
        shape = SweepShape(B, T, K, N, d, H, M, F, n_read, 4 * d, d_out)
        consts = types.SimpleNamespace(
            activation=act,
            cand_gain=torch.ones(d) if cand else None,
            cand_eps=1e-5,
            norm_gain_state=torch.ones(2 * d) if cell else None,
        )
        sweep = ReverseSweep(
            shape, consts, device=torch.device("cpu"), state_dtype=torch.float32,
            product_dtype=pdt, kernels=False,
        )  # fmt: skip

        def fill(t, scale=1.0):
            t.copy_((torch.randn(t.shape, generator=gen) * scale).to(t.dtype))

        for key in ("A", "R", "h_old", "y", "gate_pre", "mv", "hidden", "d_q_pre", "d_q_post",
                    "d_h_sel", "d_h_fast", "gate_bias", "b1", "op1", "op1_fast", "op2", "op2_fast",
                    "sigma", "dc", "db"):  # fmt: skip
            fill(getattr(sweep, key))
        sweep.c.copy_(torch.tanh(torch.randn(sweep.c.shape, generator=gen)))
        sweep.b.copy_(torch.sigmoid(torch.randn(sweep.b.shape, generator=gen)))
        sweep.rms.copy_(torch.rand(sweep.rms.shape, generator=gen) + 0.5)
        sweep.cand_gain.copy_(1.0 + 0.1 * torch.randn(d, generator=gen))
        for b in range(B):
            for t in range(T):
                sweep.cells[b, t] = torch.randperm(N, generator=gen)[:K]
        sweep.units.copy_(torch.randint(0, M, sweep.units.shape, generator=gen))
        sweep.valid.copy_(torch.rand(sweep.valid.shape, generator=gen) < 0.75)
        sweep.valid[0, T - 1] = True
        sweep.cells[~sweep.valid] = 0  # the tape's padded slots
        sweep.units[~sweep.valid] = 0
        sweep.reset.copy_(torch.rand(sweep.reset.shape, generator=gen) < 0.3)
        sweep.reset[0, T - 1] = False
        sweep.out_tgt.copy_(out_tgt.to(torch.int32))
        sweep.out_w.copy_(torch.randn(N, d_out, generator=gen) * (out_tgt >= 0))

        out: dict[str, np.ndarray] = {
            "shape": np.asarray(list(shape), dtype=np.int64),
            "half": np.asarray(int(pdt == torch.bfloat16)),
            "cand_norm": np.asarray(int(cand)), "cell_norm": np.asarray(int(cell)),
            "cand_eps": np.asarray(consts.cand_eps), "activation": np.asarray(act),
        }  # fmt: skip
        for key in SWEEP_READ:
            out[key] = np.array(_np(getattr(sweep, key)))
        for key in SWEEP_WRITTEN:
            out[f"start_{key}"] = np.array(_np(getattr(sweep, key)))
        for t in (T - 1, T - 2):
            sweep.head_reference(t)
            for key in SWEEP_WRITTEN:
                out[f"head{t}_{key}"] = np.array(_np(getattr(sweep, key)))
            fill(sweep.act_r)
            fill(sweep.act_f)
            out[f"mid{t}_act_r"], out[f"mid{t}_act_f"] = np.array(_np(sweep.act_r)), np.array(_np(sweep.act_f))
            sweep.middle_reference(t)
            for key in SWEEP_WRITTEN:
                out[f"mid{t}_{key}"] = np.array(_np(getattr(sweep, key)))
            fill(sweep.dv_r)
            fill(sweep.dv_f)
            out[f"tail{t}_dv_r"], out[f"tail{t}_dv_f"] = np.array(_np(sweep.dv_r)), np.array(_np(sweep.dv_f))
            sweep.tail_reference(t)
            for key in SWEEP_WRITTEN:
                out[f"tail{t}_{key}"] = np.array(_np(getattr(sweep, key)))
        np.savez_compressed(HERE / f"sweep_{name}.npz", **out)
        print("sweep", name, "ok", "d_out", d_out)


def make_decode(root: Path) -> None:
    """``HSN._decode`` (``python/hsn/model/hsn.py:2374``) in evaluation mode on seeded ``q``, ``u``: float64,
    float32 and under ``torch.autocast("cpu", dtype=torch.bfloat16)``, with the decoder's weights."""
    import torch

    B, T = 3, 5
    cfg = _cfg(root, B=B, T=T, N=12, d=16, K=3, H=40, M=3, D=2, fd="[summary,eps,state,router]",
               extra=("model.selected_readout=false",))
    for name, dtype, auto in (("f64", torch.float64, False), ("f32", torch.float32, False), ("bf16", torch.float32, True)):
        model = _model(cfg, dtype, 0.3)
        model.eval()
        gen = torch.Generator().manual_seed(21)
        d = cfg.model.d
        qs = (torch.randn(B, T, d, generator=gen) * 0.5).to(dtype)
        us = (torch.randn(B, T, d, generator=gen) * 0.8).to(dtype)
        with torch.no_grad():
            if auto:
                with torch.autocast("cpu", dtype=torch.bfloat16):
                    logits = model._decode(qs, us, None)
            else:
                logits = model._decode(qs, us, None)
        dec = model.decoder
        np.savez_compressed(
            HERE / f"decode_{name}.npz", qs=_np(qs), us=_np(us), logits=_np(logits.to(dtype)),
            dec_w1=_np(dec.fc1.weight), dec_b1=_np(dec.fc1.bias), dec_w2=_np(dec.fc2.weight), dec_b2=_np(dec.fc2.bias),
        )  # fmt: skip
        print("decode", name, tuple(logits.shape), logits.dtype)


def make_units(root: Path) -> None:
    """``UnitBank.forward_grouped`` (``python/hsn/model/units.py:356-414``) with its autograd backward on seeded
    pairs: float64, float32 and under ``torch.autocast("cpu", dtype=torch.bfloat16)``; a unit that no pair chose,
    a count that is no multiple of a tile, the ``record`` of the first layer's pre-activation."""
    import torch
    from hsn.model.units import UnitBank

    cases = {"a": dict(M=5, d=16, H=48, P=333, absent=(3,)), "b": dict(M=3, d=8, H=32, P=70, absent=())}
    for case, c in cases.items():
        for name, dtype, auto in (("f64", torch.float64, False), ("f32", torch.float32, False), ("bf16", torch.float32, True)):
            torch.manual_seed(31)
            bank = UnitBank(c["M"], c["d"], c["H"], "gelu", init="fan_in").to(dtype)
            gen = torch.Generator().manual_seed(32)
            with torch.no_grad():
                bank.b1.copy_((torch.randn(bank.b1.shape, generator=gen) * 0.3).to(dtype))
                bank.b2.copy_((torch.randn(bank.b2.shape, generator=gen) * 0.3).to(dtype))
            present = [j for j in range(c["M"]) if j not in c["absent"]]
            idx = torch.tensor(present)[torch.randint(0, len(present), (c["P"],), generator=gen)]
            v = torch.randn(c["P"], 4 * c["d"], generator=gen).to(dtype).requires_grad_(True)
            cot = torch.randn(c["P"], c["d"], generator=gen).to(dtype)
            record: dict = {}
            if auto:
                with torch.autocast("cpu", dtype=torch.bfloat16):
                    out = bank.forward_grouped(v, idx, record=record)
                    loss = (out.to(dtype) * cot).sum()   # the cotangent reaches the pass as bfloat16(cot)
            else:
                out = bank.forward_grouped(v, idx, record=record)
                loss = (out * cot).sum()
            loss.backward()
            np.savez_compressed(
                HERE / f"units_{case}_{name}.npz", v=_np(v), unit_idx=idx.numpy(), cot=_np(cot), out=_np(out.to(dtype)),
                hidden=_np(record["hidden"].to(dtype)), W1=_np(bank.W1), b1=_np(bank.b1), W2=_np(bank.W2), b2=_np(bank.b2),
                d_v=_np(v.grad), d_W1=_np(bank.W1.grad), d_b1=_np(bank.b1.grad), d_W2=_np(bank.W2.grad), d_b2=_np(bank.b2.grad),
            )  # fmt: skip
            print("units", case, name, tuple(out.shape), out.dtype, record["hidden"].dtype)


def make_scorer(root: Path) -> None:
    """The replay's scorer logits ``_scorer_logits`` (``python/hsn/train/split.py:305-342``) with autograd's gradients
    of the scorer's weight and bias for a seeded cotangent: float64, float32 and under
    ``torch.autocast("cpu", dtype=torch.bfloat16)``; features in the reference's layout (``u, eps, h, age, 7 scalars,
    a_cur, a_prev``), no address gate, no excluded features."""
    import torch
    from hsn.train.split import _scorer_logits

    R, N, d, M = 6, 20, 16, 5
    cfg = _cfg(root, B=2, T=3, N=N, d=d, K=3, H=40, M=M, D=2, fd="[summary,eps,state,router]")
    for name, dtype, auto in (("f64", torch.float64, False), ("f32", torch.float32, False), ("bf16", torch.float32, True)):
        model = _model(cfg, dtype, 0.3)
        scorer = model.scorer
        assert isinstance(scorer.net, torch.nn.Linear) and not scorer.exclude and scorer.address_gate is None
        S = scorer.in_features - 3 * d - 1
        gen = torch.Generator().manual_seed(41)
        u = (torch.randn(R, d, generator=gen) * 0.7).to(dtype)
        eps = (torch.randn(R, d, generator=gen) * 0.4).to(dtype)
        h = (torch.randn(R, N, d, generator=gen) * 0.5).to(dtype)
        age = torch.randint(0, 3 * int(scorer.age_max), (R, N), generator=gen)
        scalars = torch.randn(R, N, S, generator=gen).to(dtype)
        cot = torch.randn(R, N, M, generator=gen).to(dtype)
        scorer.zero_grad()
        if auto:
            with torch.autocast("cpu", dtype=torch.bfloat16):
                logits = _scorer_logits(scorer, u, eps, h, age, scalars)
        else:
            logits = _scorer_logits(scorer, u, eps, h, age, scalars)
        (logits * cot).sum().backward()
        np.savez_compressed(
            HERE / f"scorer_{name}.npz", u=_np(u), eps=_np(eps), h=_np(h), age=age.numpy(), scalars=_np(scalars), cot=_np(cot),
            weight=_np(scorer.net.weight), bias=_np(scorer.net.bias), age_max=np.array(float(scorer.age_max)),
            logits=_np(logits), d_weight=_np(scorer.net.weight.grad), d_bias=_np(scorer.net.bias.grad),
        )  # fmt: skip
        print("scorer", name, tuple(logits.shape), logits.dtype, "S", S)


def make_replay(root: Path) -> None:
    """``PDGCell.replay_sparse`` (``python/hsn/model/cell.py:655-734``) on the arguments the split window's replay
    gives it (``python/hsn/train/split.py:657``), taken by a wrapper around the bound method while a whole window runs:
    the call is made once more on leaf copies of ``u``, ``eps`` and the slot weights, with seeded cotangents of
    ``(c, b)``, so that the gradients written here are this function's alone. float32, float32 with slots the budget
    cut, and under ``torch.autocast("cpu", dtype=torch.bfloat16)``."""
    import dataclasses

    import torch

    SG = "[summary,eps,router]"
    cases = {
        "f32": dict(shape=dict(B=3, T=8, N=64, d=32, K=4, H=128, M=4, D=3), extra=("model.age_max=3",), precision="fp32"),
        "cut_f32": dict(shape=dict(B=3, T=10, N=12, d=16, K=4, H=24, M=3, D=3), extra=("model.budget=0.06",), precision="fp32"),
        "bf16": dict(shape=dict(B=3, T=8, N=64, d=32, K=4, H=128, M=4, D=3), extra=("model.age_max=3",), precision="bf16"),
        "wide_bf16": dict(shape=dict(B=2, T=6, N=32, d=64, K=8, H=128, M=2, D=4), extra=("model.age_max=1000000",), precision="bf16"),
    }  # fmt: skip
    for name, case in cases.items():
        shape = case["shape"]
        cfg = _cfg(root, **shape, fd=SG, extra=case["extra"], precision=case["precision"])
        model = _model(cfg, torch.float32, 0.3)
        tokens, ctx, reset = _inputs(cfg, shape["B"], shape["T"], 0.15)
        state = model.init_state(shape["B"])
        cell = model.cell
        real = cell.replay_sparse
        out: dict[str, np.ndarray] = {}

        def wrapper(u, eps, h_read, sel, *, record=None, real=real, cell=cell, out=out):
            leaves = [t.detach().clone().requires_grad_(True) for t in (u, eps, sel.alpha)]
            seen: dict[str, torch.Tensor] = {}
            hooks = [cell.W_out.register_forward_hook(lambda mod, inp, res: seen.update(unit_out=inp[0])),
                     cell.norm.register_forward_hook(lambda mod, inp, res: seen.update(v_raw=inp[0], v=res))]  # fmt: skip
            grouped = cell.units.forward_grouped

            def grouped_seen(v, idx, **kw):   # the view of v the unit pass reads: its gradient is the unit pass's alone
                seen["v_units"] = v
                return grouped(v, idx, **kw)

            cell.units.forward_grouped = grouped_seen
            try:
                rec: dict[str, torch.Tensor] = {}
                c, b = real(leaves[0], leaves[1], h_read, dataclasses.replace(sel, alpha=leaves[2]), record=rec)
            finally:
                for hook in hooks:
                    hook.remove()
                del cell.units.forward_grouped
            gen = torch.Generator().manual_seed(51)
            d_c = torch.randn(c.shape, generator=gen).to(c.dtype)
            d_b = torch.randn(b.shape, generator=gen).to(b.dtype)
            params = dict(cell.named_parameters())
            graph = cell.graph
            padded = graph._padded_weights()   # [N, D_max] float32, the window's cached tensor: the one the call used
            grads = torch.autograd.grad([c, b], [*leaves, seen["unit_out"], seen["v_raw"], seen["v_units"], padded, *params.values()], [d_c, d_b], allow_unused=True,
                                        retain_graph=True)   # the window caches casts of the weights: the real call below shares them
            f32 = torch.float32
            out.update(u=_np(u), eps=_np(eps), h_read=_np(h_read), cells=sel.cell_idx.numpy(), units=sel.unit_idx.numpy(),
                       valid=sel.valid.numpy(), alpha=_np(sel.alpha), c=_np(c), b=_np(b), d_c=_np(d_c), d_b=_np(d_b),
                       unit_out=_np(seen["unit_out"].to(f32)), d_u=_np(grads[0]), d_eps=_np(grads[1]), d_alpha=_np(grads[2]),
                       d_unit_out=_np(grads[3].to(f32)), cand_eps=np.array(float(cell.cand_norm.eps)),
                       v_raw=_np(seen["v_raw"]), v=_np(seen["v"].to(f32)), d_v_raw=_np(grads[4]), d_v_units=_np(grads[5].to(f32)),
                       norm_eps=np.array(float(cell.norm.eps if cell.norm.eps is not None else torch.finfo(torch.float32).eps)),
                       pad_src=graph._pad_src.numpy(), edge_w=_np(padded), d_edge_w=_np(grads[6]))  # fmt: skip
            print("   dtypes: v_raw", seen["v_raw"].dtype, "v", seen["v"].dtype, "v_units", seen["v_units"].dtype, "d_v_units", grads[5].dtype,
                  "gate_pre", rec["gate_pre"].dtype, "b", b.dtype)
            for key, value in rec.items():
                out["rec_" + key] = _np(value.to(f32))
            for (key, value), grad in zip(params.items(), grads[7:], strict=True):
                out["w_" + key] = _np(value)
                if grad is not None:
                    out["g_" + key] = _np(grad.to(f32))
            return real(u, eps, h_read, sel, record=record)

        cell.replay_sparse = wrapper
        try:
            if case["precision"] == "bf16":
                with torch.autocast("cpu", dtype=torch.bfloat16):
                    _run_window(root, cfg, model, torch.float32, tokens, ctx, reset, state)
            else:
                _run_window(root, cfg, model, torch.float32, tokens, ctx, reset, state)
        finally:
            del cell.replay_sparse
        assert out, "the window never reached the replay"
        np.savez_compressed(HERE / f"replay_{name}.npz", **out)
        print("replay", name, {k: v.shape for k, v in out.items() if k in ("unit_out", "c", "rec_y", "g_W_out.weight")},
              "valid", float(out["valid"].mean()))  # fmt: skip


def make_snapshot(root: Path) -> None:
    """``CellGraphState.snapshot`` (``python/hsn/model/state.py:363``) and ``pack_cell_state``
    (``python/hsn/train/checkpoint.py:260``): seeded states in float32 and bfloat16, their metas and the
    reference's digests. bfloat16 tensors are stored as their 16-bit patterns."""
    import torch
    from hsn.model.state import CellGraphState, StateMeta
    from hsn.train.checkpoint import pack_cell_state

    cases = {
        "f32": (torch.float32, StateMeta("hsn-test-r1", 1, "tenant-a", None)),
        "bf16": (torch.bfloat16, StateMeta("hsn-b200/é", 3, "tenant-ü", 4102444800.5)),
    }
    for name, (dtype, meta) in cases.items():
        gen = torch.Generator().manual_seed(11)
        B, N, d = 3, 7, 5
        h = torch.randn(B, N, d, generator=gen).to(dtype)
        state = CellGraphState(h=h, q=h.float().mean(dim=1).to(dtype), age=torch.randint(0, 90, (B, N), generator=gen),
                               pos=torch.randint(0, 4000, (B,), generator=gen))  # fmt: skip
        snap = state.snapshot(meta)
        packed = pack_cell_state(state)
        assert sorted(packed) == ["age", "h", "pos", "q"]
        bits = (lambda t: t.view(torch.int16).numpy()) if dtype == torch.bfloat16 else (lambda t: t.numpy())
        np.savez_compressed(
            HERE / f"snapshot_{name}.npz", h=bits(snap.h), q=bits(snap.q), age=snap.age.numpy(), pos=snap.pos.numpy(),
            dtype=np.array(str(dtype)), digest=np.array(snap.digest), meta_json=np.array(meta.to_bytes().decode("utf-8")),
            model_version=np.array(meta.model_version), state_schema_version=np.array(meta.state_schema_version),
            tenant_id=np.array(meta.tenant_id), expires_at=np.array(np.nan if meta.expires_at is None else meta.expires_at),
        )  # fmt: skip
        print("snapshot", name, snap.digest[:16])


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", type=Path, required=True)
    parser.add_argument("--only", default="")
    args = parser.parse_args()
    _import_reference(args.reference)
    import torch

    torch.set_num_threads(1)
    steps = {
        "select": make_select, "update": make_update, "recurrence": make_recurrence,
        "windows": make_windows, "bf16": make_windows_bf16, "prologue": make_prologue, "chain": make_chain,
        "sweep": make_sweep, "snapshot": make_snapshot, "decode": make_decode, "units": make_units, "scorer": make_scorer,
        "replay": make_replay,
    }  # fmt: skip
    for key, fn in steps.items():
        if not args.only or key in args.only.split(","):
            fn(args.reference)


if __name__ == "__main__":
    main()
