"""Benchmark of the HSN window path: window row-positions per second, forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c2|c3|c1]

A *step* is one TBPTT window (configuration 3: a chain of four) for the rank's rows, from the
window's token and context ids: the prologue (ids to encoder outputs ``z``, context embeddings and
scorer scalars), the forward sweep (tape + record) and the state-gradient reverse sweep with
synthetic cotangents. Uniform random bytes stand in for the reference's data set. One JSON line is
printed by rank 0. ``--impl reference`` times the CPU restatement of the reference's window
(``oracle/``) on the host cores instead, on a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

if "reference" in sys.argv and "OMP_NUM_THREADS" in os.environ:
    # the reference arm uses every host core; torchrun pins OMP_NUM_THREADS to 1 for its children
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)

import numpy as np  # noqa: E402

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

CONFIGS = {
    # name: B (per GPU), T, N, d, K, H, M, D, S, p_reset, windows
    "c1": dict(B=2, T=8, N=16, d=32, K=2, H=32, M=2, D=2, S=9, p=0.1, prod="fp32"),
    "c2": dict(B=32, T=256, N=256, d=64, K=8, H=512, M=8, D=4, S=9, p=1 / 1024, prod="bf16"),
    # four chained windows: the state carried forward, its cotangent (A, R) carried back across every boundary
    "c3": dict(B=64, T=512, N=512, d=64, K=8, H=512, M=8, D=4, S=9, p=1 / 1024, prod="bf16", windows=4),
    # the resident contract (no state tape; the state lives in HBM between calls). B is the GLOBAL batch:
    # `--gpus N` gives every rank 256 / N rows (strong scaling); on one GPU without --rows, one eighth of it
    "c4": dict(B=256, T=1024, N=4096, d=128, K=16, H=1024, M=8, D=4, S=9, p=1 / 1024, prod="bf16", resident=True,
               global_batch=True),
    "c5": dict(B=512, T=32, N=1024, d=64, K=8, H=512, M=8, D=4, S=9, p=1 / 4096, prod="bf16", resident=True,
               forward_only=True),
    # the same streams token by token: one hsnw_stream_step, then hsnw_stream_continue per position
    "c5s": dict(B=512, T=32, N=1024, d=64, K=8, H=512, M=8, D=4, S=9, p=1 / 4096, prod="bf16", resident=True,
                forward_only=True, stream=True),
}
# the trainer's AdamW pass (not the headline): forty tensors of a few million elements, one launch a step
CONFIGS["adamw"] = dict(tensors=40, elements=4_194_304 + 1031, trainer=True)
# the window's epilogue (not the headline): the decoder over the c2 window's 8192 rows
CONFIGS["decode"] = dict(rows=32 * 256, d=64, H=512, V=256, decoder=True)
# the replay's grouped unit pass (not the headline): every pair of the c2 window at once, forward and backward
CONFIGS["units"] = dict(pairs=32 * 256 * 8, M=8, d=64, H=512, units=True)
# the replay's scorer logits (not the headline): every cell of every position of the c2 window, forward and backward
CONFIGS["scorer"] = dict(R=32 * 256, N=256, d=64, M=8, S=9, scorer=True)
# the end of the replay's cell pass (not the headline): every slot of the c2 window, forward and backward
CONFIGS["tail"] = dict(slots=32 * 256 * 8, d=64, tail=True)
# the cell norm and the gate of the replay's cell pass (not the headline): every slot of the c2 window, forward and backward
CONFIGS["gate"] = dict(slots=32 * 256 * 8, d=64, gate=True)
# the messages and the gathered inputs of the replay's cell pass (not the headline): every slot of the c2 window
CONFIGS["messages"] = dict(R=32 * 256, N=256, d=64, K=8, D=4, messages=True)
WORKLOADS = {
    "messages": "the replay's messages + gathered inputs over a window's 8192 positions x 8 slots (N 256, d 64, 4 in-neighbours), bf16 products, forward + backward",
    "gate": "the replay's cell norm + gate + sigmoid over a window's 65,536 slots (4d 256 -> d 64), bf16 products, forward + backward",
    "tail": "the replay's W_out + candidate norm + weighted tanh over a window's 65,536 slots (d 64), bf16 products, forward + backward",
    "scorer": "the replay's scorer logits over a window's 8192 positions x 256 cells (d 64, 8 units, 9 scalars), bf16 products, forward + weight gradients",
    "units": "the replay's grouped unit pass over a window's 65,536 pairs: 8 units 256 -> 512 -> 64, bf16 products, forward + backward",
    "decode": "the decoder D([q; u]) over a window's 8192 rows: 128 -> 512 -> 256, bf16 products",
    "adamw": "the trainer's AdamW step over 40 fp32 tensors of 4,195,335 elements (671 MB of parameters), one launch",
    "c1": "tiny gradcheck-shape window B2 T8 N16 d32 K2 H32",
    "c2": "reference-shape window fwd+bwd: B32 T256 N256 d64 K8 H512 M8 D4, bf16 products, fp32 state, resets p=1/1024",
    "c3": "split-window chain: B64, 4 chained windows of T512 (state carried forward, its cotangent back), N512 d64 K8 H512, bf16 products",
    "c4": "scaled sparse routing, global B256 sharded over the ranks: T1024 N4096 d128 K16 H1024, resident state, fwd+bwd, gradient all-reduce",
    "c5s": "streaming token by token, one GPU's 512 streams of 4096: N1024 d64 K8 H512, one call per position (32 calls a step), derived values carried",
    "c5": "streaming, one GPU's 512 streams of 4096: N1024 d64 K8 H512, forward only on a resident state, 32 steps a call, each call continuing the last",
}


def bytes_per_row_position(c: dict) -> int:
    """Algorithmic HBM bytes of one row-position, forward (taped contract) + state-gradient
    backward: state = 4Nd + 4d + 8N per record; F = 2 state + 4(2d) + 4NS + (18K + 4) +
    (4Kd + 4d + 4); B = 4(6Kd + 2d) + 9K + 1 + 4(3Kd) + 4K + 2KH + 8K."""
    N, d, K, H, S = c["N"], c["d"], c["K"], c["H"], c["S"]
    state = 4 * N * d + 4 * d + 8 * N
    fwd = 2 * state + 4 * (2 * d) + 4 * N * S + (18 * K + 4) + (4 * K * d + 4 * d + 4)
    if c.get("resident"):  # read every cell, write the K written rows, q and the ages
        fwd = state + (4 * K * d + 4 * d + 8 * N) + 4 * (2 * d) + 4 * N * S + (18 * K + 4) + (4 * K * d + 4 * d + 4)
    full = 4 * (6 * K * d + 2 * d) + 9 * K + 1
    bwd = full + 4 * (3 * K * d) + 4 * K + 2 * K * H + 8 * K
    return fwd if c.get("forward_only") else fwd + bwd


def kernel_bytes_per_row_position(c: dict) -> dict[str, int]:
    """The same algorithmic bytes split by the kernel that moves them (per row and launch). The
    per-row cluster kernels ``rows_fwd`` / ``rows_bwd`` do a whole sweep in one launch; of the
    batch-synchronous phases ``front`` carries the state
    tape (read record t, write record t + 1) and the position's inputs, ``row`` the scorer scalars
    and the decision, ``update`` the selected rows and summaries, ``mid`` the recorded hidden
    pre-activations, ``tail_head`` the rest of the reverse sweep; ``unit`` works on chip."""
    N, d, K, H, S = c["N"], c["d"], c["K"], c["H"], c["S"]
    state = 4 * N * d + 4 * d + 8 * N
    full = 4 * (6 * K * d + 2 * d) + 9 * K + 1
    fwd = 2 * state + 4 * (2 * d) + 4 * N * S + 18 * K + 4 + 4 * K * d + 4 * d + 4
    bwd = full + 4 * (3 * K * d) + 4 * K + 2 * K * H + 8 * K
    return {
        "rows_fwd": fwd * c["T"],   # the per-row cluster kernels: one launch does every position
        "rows_bwd": bwd * c["T"],
        "front": 2 * state + 4 * (2 * d),
        "row": 4 * N * S + 18 * K + 4,
        "unit": 0,
        "update": 4 * K * d + 4 * d + 4,
        "mid": 2 * K * H,
        "tail_head": full + 4 * (3 * K * d) + 4 * K + 8 * K,
    }


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of each kernel of the c2
# workload, from the ncu captures summarised in profiles/rows_kernels_c2.md (the per-row cluster
# kernels) and profiles/phases_kernels_c2_dram.md (the phase kernels).
NCU_TRAFFIC_SOURCE = ("ncu capture of bench.py --steps 1 --warmup 3 at the kernels of commit 9acb6c0 "
                      "(profiles/rows_kernels_c2.md)")
NCU_TRAFFIC_PER_LAUNCH: dict[str, dict[str, float]] = {
    "c2": {"rows_fwd": 783.8e6, "rows_bwd": 227.0e6, "pre": 4.6e6, "front": 2.798e6, "row": 1.375e6, "unit": 3.419e6, "update": 0.526e6, "mid": 2.254e6, "tail_head": 1.703e6},
}


def synthetic_model(c: dict):
    """Seeded N(0, 0.02) weights of the configuration's shapes, and the tables the window's prologue
    reads (byte and context embeddings and the encoder at the same scale, the scorer's fixed byte codes
    and cell addresses N(0, 1) / sqrt(d) as the reference draws them, running averages at zero)."""
    from hsn_b200.window import synthetic_weights

    W = synthetic_weights(np.random.default_rng(0), N=c["N"], d=c["d"], K=c["K"], H=c["H"], M=c["M"],
                          D=c["D"], S=c["S"], age_max=2**31 - 1)  # fmt: skip
    rng = np.random.default_rng(5)
    N, d, H = c["N"], c["d"], c["H"]
    f = lambda *shape: (rng.standard_normal(shape) * 0.02).astype(np.float32)  # noqa: E731
    tables = dict(
        byte_emb=f(256, d), enc_w1=f(H, d), enc_b1=np.zeros(H, np.float32), enc_w2=f(d, H), enc_b2=np.zeros(d, np.float32),
        ctx_emb=f(16, d), byte_codes=(rng.standard_normal((256, d)) / np.sqrt(d)).astype(np.float32),
        cell_addresses=(rng.standard_normal((N, d)) / np.sqrt(d)).astype(np.float32),
        ema_utility=np.zeros(N, np.float32), ema_selected=np.zeros(N, np.float32),
        budget_frac=1.0, round_frac=0.0, n_context=16.0, unroll=float(c["T"]), position="document",
    )  # fmt: skip
    return W, tables


def synthetic_ids(c: dict, first_row: int, rows: int):
    """Seeded ids and cotangents for ``rows`` rows from global row ``first_row`` on, for every window of
    the configuration's chain: uniform bytes, uniform context ids, Bernoulli resets (column 0 of the
    first window starts every stream), N(0, 0.1) cotangents. A row's data depends on its global index
    only, so results do not depend on the number of GPUs. Returns a list over windows of
    ``(tokens, ctx_ids, reset, d_q_pre, d_q_post, d_h_sel)``."""
    T, d, K, W = c["T"], c["d"], c["K"], c.get("windows", 1)
    per_row = []
    for r in range(rows):
        rng = np.random.default_rng(1000 + first_row + r)
        tokens = rng.integers(0, 256, W * T)
        ctx_ids = rng.integers(0, 16, W * T)
        reset = rng.random(W * T) < c["p"]
        reset[0] = True
        cot = [(rng.standard_normal(shape) * 0.1).astype(np.float32) for shape in ((W * T, d), (W * T, d), (W * T, K, d))]
        per_row.append((tokens, ctx_ids, reset, *cot))
    whole = [np.stack([p[i] for p in per_row]) for i in range(6)]
    return [tuple(np.ascontiguousarray(a[:, w * T : (w + 1) * T]) for a in whole) for w in range(W)]


def synthetic(c: dict, rank: int, rows: int):
    """The weights and ONE window's direct inputs ``[z, ctx, scalars, reset, d_q_pre, d_q_post, d_h_sel]``
    (numpy): the ids of :func:`synthetic_ids` through the oracle's prologue. The CPU legs use it."""
    from oracle import window_oracle as O

    W, tables = synthetic_model(c)
    tokens, ctx_ids, reset, pre, post, sel = synthetic_ids(dict(c, windows=1), rank * rows, rows)[0]
    pro = O.window_prologue(tables, tokens, ctx_ids, reset, np.zeros(rows, np.int64))
    return W, [pro["z"], pro["ctx"].astype(np.float32), pro["scalars"].astype(np.float32), reset, pre, post, sel]


def sample_clocks(stop: threading.Event, out: list) -> None:
    cmd = ["nvidia-smi", "--query-gpu=index,clocks.sm,clocks.max.sm,clocks_event_reasons.active,"
           "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
           "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap",
           "--format=csv,noheader,nounits", "-lms", "200"]  # fmt: skip
    try:
        proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    except OSError:
        return
    try:
        while not stop.is_set():
            line = proc.stdout.readline()
            if not line:
                break
            out.append(line.strip())
    finally:
        proc.terminate()


def clocks_summary(lines: list, device: int) -> dict:
    sm, mx, reasons = [], 0.0, set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for line in lines:
        f = [x.strip() for x in line.split(",")]
        if len(f) < 8 or not f[0].isdigit() or int(f[0]) != device:
            continue
        try:
            sm.append(float(f[1]))
            mx = max(mx, float(f[2]))
        except ValueError:
            continue
        for name, v in zip(names, f[4:8]):
            if v.lower().startswith("active"):
                reasons.add(name)
    return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
            "samples": len(sm)}  # fmt: skip


def cpu_window(W, tables, ids, rows: int, positions: int):
    """The oracle's prologue, window forward and state-gradient backward on ``rows`` x ``positions``
    of the workload (the first window's first positions); returns seconds."""
    from oracle import window_oracle as O

    W = O.WindowWeights(**vars(W))   # the same weights in the oracle's container
    tokens, ctx_ids, reset, pre, post, sel = (a[:rows, :positions] for a in ids)
    N, d = W.pad_src.shape[0], pre.shape[-1]
    state = (np.zeros((rows, N, d), np.float32), np.zeros((rows, d), np.float32), np.zeros((rows, N), np.int64),
             np.zeros(rows, np.int64))  # fmt: skip
    t0 = time.perf_counter()
    pro = O.window_prologue(tables, tokens, ctx_ids, reset, state[3])
    tape = O.window_forward(W, pro["z"], pro["ctx"].astype(np.float32), pro["scalars"].astype(np.float32), reset, *state)
    valid = tape["sel_valid"]
    rec = {k: tape["rec_" + k] for k in ("y", "hidden", "gate_pre", "m", "rms")}
    O.state_gradient_backward(
        W, tape["rec_c"], tape["rec_b"], tape["rec_h_old"], np.where(valid, tape["sel_cell_idx"], 0),
        np.where(valid, tape["sel_unit_idx"], 0), valid, reset, N, pre, post, sel, rec,
    )  # fmt: skip
    return time.perf_counter() - t0


def blas_threads() -> int:
    try:
        from threadpoolctl import threadpool_info

        return int(max([p.get("num_threads", 1) for p in threadpool_info()] or [1]))
    except Exception:
        return os.cpu_count() or 1


def cpu_baseline(c: dict, W, tables, ids, budget_s: float = 12.0) -> dict:
    rows = min(c["B"], ids[0].shape[0])
    probe = min(2, c["T"])
    dt = cpu_window(W, tables, ids, rows, probe)
    positions = int(max(probe, min(c["T"], budget_s / max(dt / probe, 1e-6))))
    seconds = cpu_window(W, tables, ids, rows, positions)
    return {
        "value": rows * positions / seconds,
        "unit": "row-positions/s",
        "cores": blas_threads(),
        "kind": "port",
        "sample": f"{rows} rows x {positions} positions of the workload, fp32, numpy oracle (BLAS threads = cores), {seconds:.1f} s",
    }


def run_reference(args, c: dict, name: str) -> None:
    """The CPU arm: the reference's window as restated in oracle/ (the reference is Python and is
    not present on the benchmark machine; the restatement is pinned to it by tests/golden). A step is
    a sample of the workload: 8 rows x 32 positions (256 row-positions), prologue + forward + backward."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows, positions = min(c["B"], 8), min(c["T"], 32)
    c = dict(c, T=positions, windows=1)   # only the sampled positions are drawn
    W, tables = synthetic_model(c)
    ids = synthetic_ids(c, 0, rows)[0]
    for _ in range(args.warmup):
        cpu_window(W, tables, ids, rows, positions)
    times = [cpu_window(W, tables, ids, rows, positions) for _ in range(args.steps)]
    sec = float(np.mean(times))
    value = rows * positions / sec
    threads = blas_threads()
    line = {
        "impl": "reference", "metric": "window row-positions/s fwd+bwd", "value": value, "unit": "row-positions/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOADS[name], "sample": f"{rows} rows x {positions} positions per step"},
        "cpu_baseline": {"value": value, "unit": "row-positions/s", "cores": threads, "kind": "port",
                         "sample": f"{rows} rows x {positions} positions per step, numpy oracle"},
        "e2e": {"value": value, "unit": "row-positions/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }  # fmt: skip
    print(json.dumps(line), flush=True)


def run_side_reference(args, c: dict, name: str) -> None:
    """`--impl reference` for the side configurations `units`, `scorer`, `tail`, `gate` and `messages`: the numpy restatement of the pass
    (forward + backward, bf16 rounding emulated) on a sample of the workload, on the host's cores."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    rng = np.random.default_rng(0)
    f = lambda *shape, scale=1.0: (rng.standard_normal(shape) * scale).astype(np.float32)  # noqa: E731
    if name == "units":
        from oracle import units_oracle as U

        n, M, d, H = 4096, c["M"], c["d"], c["H"]
        bank = [f(M, 4 * d, H, scale=(4 * d) ** -0.5), f(M, H, scale=0.3), f(M, H, d, scale=H**-0.5), f(M, d, scale=0.3)]
        v, cot, idx = f(n, 4 * d), f(n, d), rng.integers(0, M, n)
        unit, sample = "pairs/s", f"{n} of the window's pairs per step"

        def step():
            _, pre = U.forward_grouped(v, idx, *bank, bf16=True)
            U.backward_grouped(v, idx, *bank, pre, cot, bf16=True)
            return n
    elif name == "messages":
        from oracle import messages_oracle as MO

        n, N, d, K, D = 128, c["N"], c["d"], c["K"], c["D"]
        mu, me, mh, mv, mdv = f(n, d), f(n, d), f(n, N, d, scale=0.5), f(d, d, scale=d**-0.5), f(n, K, 4 * d)
        mcells = np.stack([rng.permutation(N)[:K] for _ in range(n)]).astype(np.int64)
        msrc, mw = rng.integers(0, N, (N, D)).astype(np.int64), rng.random((N, D)).astype(np.float32)
        unit, sample = "slots/s", f"{n} of the window's positions ({n * K} slots) per step"

        def step():
            MO.forward_messages(mu, me, mh, mcells, msrc, mw, mv, bf16=True)
            MO.backward_messages(mh, mcells, msrc, mw, mv, mdv, bf16=True)
            return n * K
    elif name == "gate":
        from oracle import gate_oracle as GO

        n, d = 16384, c["d"]
        gx, gnw, ggw, ggb = f(n, 4 * d, scale=0.8), 1.0 + f(4 * d, scale=0.2), f(d, 4 * d, scale=(4 * d) ** -0.5), f(d, scale=0.3)
        gdv, gdb = f(n, 4 * d), f(n, d)
        unit, sample = "slots/s", f"{n} of the window's slots per step"

        def step():
            GO.forward_norm_gate(gx, gnw, ggw, ggb, norm_eps=1e-6, bf16=True)
            GO.backward_norm_gate(gx, gnw, ggw, ggb, gdv, gdb, norm_eps=1e-6, bf16=True)
            return n
    elif name == "tail":
        from oracle import tail_oracle as TO

        n, d = 16384, c["d"]
        x, alpha, w, g, cot = f(n, d, scale=0.6), np.ones(n, np.float32), f(d, d, scale=d**-0.5), 1.0 + f(d, scale=0.2), f(n, d)
        unit, sample = "slots/s", f"{n} of the window's slots per step"

        def step():
            _, y = TO.forward_tail(x, alpha, w, g, bf16=True)
            TO.backward_tail(x, alpha, w, g, y, cot, bf16=True)
            return n
    else:
        from oracle import scorer_oracle as SO

        n, N, d, M, S = 64, c["N"], c["d"], c["M"], c["S"]
        weight, bias = f(M, 3 * d + 1 + S, scale=0.2), f(M, scale=0.3)
        feats = [f(n, d), f(n, d), f(n, N, d), rng.integers(0, 300, (n, N)), f(n, N, S)]
        cot = f(n, N, M)
        unit, sample = "cells/s", f"{n} of the window's positions per step"

        def step():
            SO.scorer_logits(weight, bias, *feats, 100.0, bf16=True)
            SO.scorer_logits_backward(weight, *feats, 100.0, cot, bf16=True)
            return n * N
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    done = sum(step() for _ in range(args.steps))
    sec = time.perf_counter() - t0
    value = done / sec
    metric = {"units": "grouped unit pass pairs/s (forward + backward)", "tail": TAIL_METRIC, "gate": GATE_METRIC, "messages": MSG_METRIC}.get(name, "scorer logits cells/s (forward + weight gradients)")
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 with bf16 rounding emulated", "data": "synthetic", "config": {"workload": WORKLOADS[name], "sample": sample},
        "cpu_baseline": {"value": value, "unit": unit, "cores": blas_threads(), "kind": "port", "sample": sample + ", numpy oracle"},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}), flush=True)  # fmt: skip


def dist_setup():
    """(world, rank, local rank, device) with the NCCL process group up when launched by torchrun."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the window path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    return world, rank, local, dev


def n_parameters(c: dict) -> int:
    """The parameter count of the configuration's window model: the size of the training-gradient
    exchange after a window's backward (the gradients themselves come from the batched replay, which is
    outside this path; the benchmark exchanges a buffer of their size)."""
    d, H, M, S = c["d"], c["H"], c["M"], c["S"]
    shared = (3 * d) * H + H + H * d + d
    predictor = d * H + H + H * d + d
    scorer = M * (3 * d + 1 + S) + M
    cell = 2 * d * d + 4 * d * d + d + 4 * d + d
    units = M * (4 * d * H + H + H * d + d)
    return shared + predictor + scorer + cell + units


def timed_steps(step, steps: int, barrier):
    """``steps`` calls of ``step`` between two barriers, an event after every one: total milliseconds
    and the per-step times."""
    import torch

    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    barrier()
    marks[0].record()
    for i in range(steps):
        step(i)
        marks[i + 1].record()
    barrier()
    each = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]
    return marks[0].elapsed_time(marks[steps]), each


def spread(each: list) -> dict:
    return {"median": float(np.median(each)), "p95": float(np.percentile(each, 95)), "min": float(np.min(each)),
            "max": float(np.max(each)), "n": len(each)}  # fmt: skip


def run_resident(args, c: dict, name: str) -> None:
    """The configurations of the resident contract: inputs drawn on the device from a seed (their host
    copies would not fit a pinned buffer), the state updated in place from call to call. Configuration
    4 shards its GLOBAL batch over the ranks (strong scaling) and exchanges a gradient-sized buffer
    after every backward; the streaming configurations run one GPU's share. No end-to-end leg."""
    import torch
    import torch.distributed as dist

    from hsn_b200.window import WindowModel, launch_profile, synthetic_weights, window_backward, window_forward

    world, rank, local, dev = dist_setup()
    T, N, d, K, S = c["T"], c["N"], c["d"], c["K"], c["S"]
    global_rows = c["B"]
    if c.get("global_batch"):
        B = args.rows if args.rows > 0 else (global_rows // world if world > 1 else global_rows // 8)
        global_rows = B * world
    else:
        B = args.rows if args.rows > 0 else c["B"]
        global_rows = B * world
    W = synthetic_weights(np.random.default_rng(0), N=N, d=d, K=K, H=c["H"], M=c["M"], D=c["D"], S=S,
                          age_max=2**31 - 1)  # fmt: skip
    model = WindowModel.from_weights(W, device=dev, prod=c["prod"], row_clusters=not args.phases)
    gen = torch.Generator(device=dev).manual_seed(1 + rank)
    z = torch.randn((B, T, d), device=dev, generator=gen) * 0.5
    ctx = torch.randn((B, T, model.dims["dc"]), device=dev, generator=gen) * 0.02
    scalars = torch.rand((B, T, N, S), device=dev, generator=gen)
    reset = torch.rand((B, T), device=dev, generator=gen) < c["p"]
    cots = [torch.randn(shape, device=dev, generator=gen) * 0.1 for shape in ((B, T, d), (B, T, d), (B, T, K, d))]
    state = (torch.zeros((B, N, d), device=dev), torch.zeros((B, d), device=dev),
             torch.zeros((B, N), dtype=torch.int64, device=dev), torch.zeros(B, dtype=torch.int64, device=dev))  # fmt: skip
    forward_only = bool(c.get("forward_only"))
    grads = torch.zeros(n_parameters(c), device=dev)
    out: dict = {}
    info: dict = {}
    bw_scratch = None

    per_position = [tuple(a[:, t].contiguous() for a in (z, ctx, scalars, reset)) for t in range(T)] if c.get("stream") else []
    calls = [0]

    def step(_i=0, exchange=True):
        nonlocal bw_scratch
        if per_position:
            from hsn_b200.window import stream_step

            for now in per_position:
                stream_step(model, *now, state, out=out, carried=calls[0] > 0)
                calls[0] += 1
            return
        # a stream's next chunk continues the resident state: the cells' derived values carry over
        tape = window_forward(model, z, ctx, scalars, reset, state, record=not forward_only, tape_state=False, out=out,
                              carried=forward_only and calls[0] > 0)
        calls[0] += 1
        if forward_only:
            return
        rec = {k: tape["rec_" + k] for k in ("y", "hidden", "gate_pre", "m", "rms")}
        if bw_scratch is None:
            from hsn_b200 import _lib

            need = int(_lib.library().hsnw_backward_scratch_bytes(model.struct, B, T))
            bw_scratch = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
        window_backward(model, tape["rec_c"], tape["rec_b"], tape["rec_h_old"], tape["sel_cell_idx"],
                        tape["sel_unit_idx"], tape["sel_valid"], reset, cots[0], cots[1], cots[2], rec,
                        scratch=bw_scratch, info=info)  # fmt: skip
        if world > 1 and exchange:  # the training-gradient exchange after each window backward
            dist.all_reduce(grads)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    barrier()
    stop, lines = threading.Event(), []
    sampler = threading.Thread(target=sample_clocks, args=(stop, lines), daemon=True)
    sampler.start()
    time.sleep(0.3)
    total_ms, each = timed_steps(step, args.steps, barrier)
    stop.set()
    sampler.join(timeout=2)
    barrier()
    with launch_profile() as prof:   # (without the exchange: its wait for the other ranks would be charged to the launch before it)
        step(exchange=False)
    barrier()
    times = torch.tensor([total_ms / args.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms = float(times.cpu()[0])
    if rank == 0:
        peaks_file = ROOT / "MEASURED_PEAKS.json"
        peaks = json.loads(peaks_file.read_text()) if peaks_file.exists() else {}
        peak = float(peaks.get("hbm_gbs", 6650.0))
        per = bytes_per_row_position(c)
        achieved = per * B * T / (ms * 1e-3) / 1e9   # per GPU
        total_prof = sum(prof.ms.values()) or 1.0
        kernels = {k: {"launches_per_step": n, "us_per_launch": round(1e3 * prof.ms[k] / n, 3),
                       "share": round(prof.ms[k] / total_prof, 4)} for k, n in prof.launches.items() if n}  # fmt: skip
        paths = {"forward": out.get("path"), "backward": info.get("path")}
        line = {
            "metric": "window row-positions/s " + ("fwd" if forward_only else "fwd+bwd"),
            "value": global_rows * T / (ms * 1e-3), "unit": "row-positions/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms, "step_ms": spread(each), "higher_is_better": True,
            "scaling": "strong" if c.get("global_batch") and world > 1 and args.rows <= 0 else "weak", "vs_baseline": None,
            "dtype": "bf16 products, f32 state", "data": "synthetic (drawn on the device)",
            "config": {"workload": WORKLOADS[name], "rows_per_gpu": B, "global_rows": global_rows, "positions": T,
                       "kernels": paths, "l2": "state and inputs larger than L2",
                       "allreduce_floats_per_step": int(grads.numel()) if world > 1 and not forward_only else 0},
            "e2e": None, "gpu_launches": args.steps * sum(prof.launches.values()),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": "measured" if peaks else "fallback", "per": "GPU",
                         "bytes_per_row_position": per, "kernels": kernels},
            "clocks": clocks_summary(lines, local),
        }  # fmt: skip
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


class TapedJob:
    """One rank's windows of a taped configuration on the device: the prologue, the forward sweep of
    every window of the chain (state carried forward) and the reverse sweeps in reverse order (the state's
    cotangent carried back), from ids that already are on the device."""

    def __init__(self, c: dict, dev, rows: int, phases: bool) -> None:
        import torch

        from hsn_b200.window import WindowModel, WindowPrologue

        self.c, self.dev, self.rows = c, dev, rows
        W, tables = synthetic_model(c)
        numbers = {k: tables.pop(k) for k in ("budget_frac", "round_frac", "n_context", "unroll", "position")}
        self.model = WindowModel.from_weights(W, device=dev, prod=c["prod"], row_clusters=not phases)
        self.pro = WindowPrologue.build(tables, device=dev, prod=c["prod"], **numbers)
        self.windows = c.get("windows", 1)
        N, d = c["N"], c["d"]
        self.start = (torch.zeros((rows, N, d), device=dev), torch.zeros((rows, d), device=dev),
                      torch.zeros((rows, N), dtype=torch.int64, device=dev), torch.zeros(rows, dtype=torch.int64, device=dev))  # fmt: skip
        self.pro_out = [dict() for _ in range(self.windows)]
        self.fw_out = [dict() for _ in range(self.windows)]
        self.bw_scratch = None
        self.paths: dict = {}

    def step(self, ids):
        """``ids``: per window ``(tokens, ctx_ids, reset, d_q_pre, d_q_post, d_h_sel)`` on the device.
        Returns the tapes, ``[(dc, db)]`` per window and the start state's cotangent."""
        import torch

        from hsn_b200 import _lib
        from hsn_b200.window import window_backward, window_forward, window_prologue

        state, prev, tapes = self.start, None, []
        for w in range(self.windows):
            tokens, ctx_ids, reset = ids[w][:3]
            p = window_prologue(self.pro, tokens, ctx_ids, reset, state[3], prev, out=self.pro_out[w])
            tape = window_forward(self.model, p["z"], p["ctx"], p["scalars"], reset, state, out=self.fw_out[w])
            tapes.append(tape)
            state = (tape["h"], tape["q"], tape["age"], tape["pos"])
            prev = tokens[:, -1].contiguous()
        if self.bw_scratch is None:
            need = int(_lib.library().hsnw_backward_scratch_bytes(self.model.struct, self.rows, self.c["T"]))
            self.bw_scratch = torch.empty(max(need, 256), dtype=torch.uint8, device=self.dev)
        carry, grads, info = None, [None] * self.windows, {}
        for w in reversed(range(self.windows)):
            tape = tapes[w]
            rec = {k: tape["rec_" + k] for k in ("y", "hidden", "gate_pre", "m", "rms")}
            dc, db, carry = window_backward(
                self.model, tape["rec_c"], tape["rec_b"], tape["rec_h_old"], tape["sel_cell_idx"], tape["sel_unit_idx"],
                tape["sel_valid"], ids[w][2], ids[w][3], ids[w][4], ids[w][5], rec, initial=carry,
                scratch=self.bw_scratch, info=info,
            )  # fmt: skip
            grads[w] = (dc, db)
        self.paths = {"forward": tapes[0]["path"], "backward": info.get("path")}
        return tapes, grads, carry


def run_taped(args, c: dict, name: str) -> None:
    import torch
    import torch.distributed as dist

    from hsn_b200.window import launch_profile

    world, rank, local, dev = dist_setup()
    warmup = max(args.warmup, 3)
    B = args.rows if args.rows > 0 else c["B"]
    T, N, d, K, nW = c["T"], c["N"], c["d"], c["K"], c.get("windows", 1)
    job = TapedJob(c, dev, B, args.phases)
    host = synthetic_ids(c, rank * B, B)
    pinned = [[torch.from_numpy(a).pin_memory() for a in window] for window in host]
    ids = [[t.to(dev, non_blocking=True) for t in window] for window in pinned]
    grads = torch.zeros(n_parameters(c), device=dev)

    def step(on_device):
        out = job.step(on_device)
        if world > 1:  # the training-gradient exchange after the window's backward
            dist.all_reduce(grads)
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step(ids)
    barrier()
    stop, lines = threading.Event(), []
    sampler = threading.Thread(target=sample_clocks, args=(stop, lines), daemon=True)
    sampler.start()
    time.sleep(0.3)
    # device-resident steps: the ids are on the device
    total_ms, each = timed_steps(lambda i: step(ids), args.steps, barrier)
    ms = total_ms / args.steps
    # end to end: ids and cotangents from pinned host memory in, gradients and the final state back, every step
    out_shapes = {"dc": (nW, B, T, K, d), "db": (nW, B, T, K, d), "h": (B, N, d), "q": (B, d)}
    host_out = {k: torch.empty(shape, dtype=torch.float32).pin_memory() for k, shape in out_shapes.items()}
    # Two staging sets: step i + 1's inputs cross the bus on a copy stream while step i computes (what a
    # data loader does); every step's host-to-device copy and read-back is inside the timed region.
    staged = [[[torch.empty_like(t, device=dev) for t in window] for window in pinned] for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream(dev)
    landed = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def upload(i):
        buf = i & 1
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[buf])   # the step that last read this set is done with it
            for dst_w, src_w in zip(staged[buf], pinned):
                for dst, src in zip(dst_w, src_w):
                    dst.copy_(src, non_blocking=True)
            landed[buf].record(copy_stream)

    readback = torch.cuda.Stream(device=dev)
    computed = torch.cuda.Event()

    def e2e_step(i):
        buf = i & 1
        upload(i + 1)
        main_stream.wait_event(landed[buf])
        tapes, grad_list, _ = step(staged[buf])
        consumed[buf].record(main_stream)
        # the final state lives in the tape's static buffer, which the next step rewrites: read it back
        # in order; the gradients are this step's own tensors and cross the bus beside the next step
        host_out["h"].copy_(tapes[-1]["h"], non_blocking=True)
        host_out["q"].copy_(tapes[-1]["q"], non_blocking=True)
        computed.record(main_stream)
        with torch.cuda.stream(readback):
            readback.wait_event(computed)
            for w, (dc, db) in enumerate(grad_list):
                host_out["dc"][w].copy_(dc, non_blocking=True)
                host_out["db"][w].copy_(db, non_blocking=True)
        for dc, db in grad_list:
            dc.record_stream(readback)
            db.record_stream(readback)

    for ev in consumed:
        ev.record(main_stream)
    upload(0)
    e2e_step(0)   # untimed: fills the pipeline
    e2e_steps = max(3, min(args.steps, 20))

    def e2e_run(i):
        e2e_step(i + 1)
        if i + 1 == e2e_steps:
            main_stream.wait_stream(readback)   # the last step's read-back ends before the closing event

    total_e2e, _ = timed_steps(e2e_run, e2e_steps, barrier)
    ms_e2e = total_e2e / e2e_steps
    stop.set()
    sampler.join(timeout=2)
    # one more step, untimed, with an event before every launch: the per-kernel times and counts (without the
    # gradient exchange: its wait for the other ranks would be charged to the launch before it)
    barrier()
    with launch_profile() as prof:
        job.step(ids)
    barrier()
    # the same global batch spread over the ranks (strong scaling), when there are several
    strong = None
    if world > 1 and args.rows <= 0 and c["B"] % world == 0 and c["B"] // world >= 1:
        rows = c["B"] // world
        small = TapedJob(c, dev, rows, args.phases)
        small_ids = [[torch.from_numpy(a).to(dev) for a in window] for window in synthetic_ids(c, rank * rows, rows)]

        def small_step(_i):
            small.step(small_ids)
            dist.all_reduce(grads)

        for _ in range(3):
            small_step(0)
        n = max(3, min(args.steps, 20))
        total_small, _ = timed_steps(small_step, n, barrier)
        strong = [total_small / n, rows]
    times = torch.tensor([ms, ms_e2e, strong[0] if strong else 0.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, ms_e2e, ms_strong = (float(x) for x in times.cpu())
    if rank == 0:
        peaks_file = ROOT / "MEASURED_PEAKS.json"
        peaks = json.loads(peaks_file.read_text()) if peaks_file.exists() else {}
        peak = float(peaks.get("hbm_gbs", 6650.0))
        row_pos = B * T * nW
        per = bytes_per_row_position(c)
        achieved = per * row_pos / (ms * 1e-3) / 1e9
        # the step's kernels by measured time (the profiled step); the dominant one's roofline
        launches_per_step = sum(prof.launches.values())
        total_prof = sum(prof.ms.values()) or 1.0
        split = kernel_bytes_per_row_position(c)
        traffic = NCU_TRAFFIC_PER_LAUNCH.get(name, {}) if args.positions == 0 and args.rows <= 0 else {}
        kernels = {}
        for kind, n in prof.launches.items():
            if n:
                us = 1e3 * prof.ms[kind] / n
                alg = split.get(kind, 0) * B
                kernels[kind] = {"launches_per_step": n, "us_per_launch": round(us, 3),
                                 "share": round(prof.ms[kind] / total_prof, 4), "algorithmic_bytes_per_launch": alg,
                                 "achieved_gbs": round(alg / (us * 1e-6) / 1e9, 3) if us > 0 else None,
                                 "traffic": traffic.get(kind)}  # fmt: skip
        top = max(kernels, key=lambda k: kernels[k]["share"])
        roofline = {
            "bound": "hbm", "kernel": top, "achieved": kernels[top]["achieved_gbs"], "peak": peak, "unit": "GB/s",
            "frac": kernels[top]["achieved_gbs"] / peak, "traffic": kernels[top]["traffic"],
            "traffic_source": NCU_TRAFFIC_SOURCE if kernels[top]["traffic"] else None,
            "peak_source": "measured" if peaks else "fallback",
            "how": "algorithmic bytes of the kernel's launch / its mean event-to-event time in a profiled step",
            "step": {"achieved": achieved, "frac": achieved / peak, "bytes_per_row_position": per},
            "kernels": kernels,
        }  # fmt: skip
        h2d = sum(t.numel() * t.element_size() for window in pinned for t in window)
        d2h = sum(t.numel() * t.element_size() for t in host_out.values())
        line = {
            "metric": "window row-positions/s fwd+bwd", "value": world * row_pos / (ms * 1e-3),
            "unit": "row-positions/s", "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms,
            "step_ms": spread(each), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 products, f32 state" if c["prod"] == "bf16" else "f32", "data": "synthetic",
            "config": {"workload": WORKLOADS[name] + (f" [shortened to {T} positions]" if args.positions else ""),
                       "rows_per_gpu": B, "positions": T, "windows": nW, "kernels": job.paths,
                       "step": "prologue from ids + forward sweep(s) + reverse sweep(s)" + (" + gradient all-reduce" if world > 1 else ""),
                       "l2": "tape and scalars per step far larger than L2",
                       "allreduce_floats_per_step": int(grads.numel()) if world > 1 else 0},
            "e2e": {"value": world * row_pos / (ms_e2e * 1e-3), "unit": "row-positions/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "note": "token and context ids, resets and the cotangents come from pinned host memory on a copy stream while the previous step computes; the final state is read back on the compute stream, the gradients dc/db on a read-back stream beside the next step; every copy ends inside the timed region"},
            "gpu_launches": args.steps * launches_per_step,
            "roofline": roofline,
            "clocks": clocks_summary(lines, local),
        }  # fmt: skip
        if strong:
            line["strong"] = {"value": c["B"] * T * nW / (ms_strong * 1e-3), "unit": "row-positions/s", "ms_per_step": ms_strong,
                              "rows_per_gpu": strong[1], "global_rows": c["B"],
                              "note": "the same global batch spread over the ranks: a row's positions are sequential, so fewer rows per GPU do not shorten a step"}  # fmt: skip
        if not args.no_cpu_baseline and world == 1:
            W, tables = synthetic_model(c)
            line["cpu_baseline"] = cpu_baseline(c, W, tables, host[0])
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_trainer(args, c: dict, name: str) -> None:
    """One AdamW step a "step": `hsn_tr_adamw` over the configuration's tensors in one launch (parameters and
    moments far larger than L2), with torch's multi-tensor sequence it replaces timed beside it on the same
    device. 28 algorithmic bytes an element: p, g, m, v read, p, m, v written."""
    import torch

    from hsn_b200.kernels import trainer

    if args.impl == "reference":   # the reference's CPU path: torch's multi-tensor operations on the host cores
        if int(os.environ.get("RANK", "0")) != 0:
            return
        n, elements = 8, c["elements"]
        gen = torch.Generator().manual_seed(0)
        ps, gs = ([torch.randn(elements, generator=gen) * 0.1 for _ in range(n)] for _ in range(2))
        ms, vs = [torch.zeros_like(p) for p in ps], [torch.zeros_like(p) for p in ps]
        times = []
        for step in range(1, args.warmup + args.steps + 1):
            t0 = time.perf_counter()
            _torch_adamw(torch, ps, gs, ms, vs, step)
            if step > args.warmup:
                times.append(time.perf_counter() - t0)
        value = n * elements / float(np.mean(times))
        print(json.dumps({
            "impl": "reference", "metric": "trainer AdamW elements/s", "value": value, "unit": "elements/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * float(np.mean(times)), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOADS[name] + f" [sample: {n} of the tensors a step]"},
            "cpu_baseline": {"value": value, "unit": "elements/s", "cores": torch.get_num_threads(), "kind": "reference",
                             "sample": f"{n} tensors a step, torch multi-tensor operations on the host"},
            "e2e": {"value": value, "unit": "elements/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))  # fmt: skip
        return
    world, rank, local, dev = dist_setup()
    if world > 1:
        return run_trainer_sharded(args, c, name, world, rank, dev)
    n, elements = c["tensors"], c["elements"]
    gen = torch.Generator(device=dev).manual_seed(0)
    make = lambda scale: [torch.randn(elements, generator=gen, device=dev) * scale for _ in range(n)]  # noqa: E731
    ps, gs = make(0.1), make(1.0)
    ms, vs = [torch.zeros_like(p) for p in ps], [torch.zeros_like(p) for p in ps]
    hyper = dict(lr=2.5e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01)
    clock_lines: list = []
    stop = threading.Event()
    sampler = threading.Thread(target=sample_clocks, args=(stop, clock_lines), daemon=True)
    sampler.start()
    count = [0]

    def ours(i):
        count[0] += 1
        if not trainer.adamw(ps, gs, ms, vs, step=count[0], **hyper):
            raise RuntimeError("the trainer kernels declined fp32 CUDA tensors")

    for i in range(args.warmup):
        ours(i)
    torch.cuda.synchronize()
    ms_total, each = timed_steps(ours, args.steps, torch.cuda.synchronize)
    ps2, ms2, vs2 = [p.clone() for p in ps], [m.clone() for m in ms], [v.clone() for v in vs]
    for i in range(3):
        _torch_adamw(torch, ps2, gs, ms2, vs2, i + 1)
    torch.cuda.synchronize()
    torch_total, _ = timed_steps(lambda i: _torch_adamw(torch, ps2, gs, ms2, vs2, i + 4), max(3, args.steps // 4), torch.cuda.synchronize)
    stop.set()
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = float(peaks.get("hbm_gbs", 6650.0))
    step_ms = ms_total / args.steps
    achieved = 28.0 * n * elements / (step_ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "trainer AdamW elements/s", "value": n * elements / (step_ms * 1e-3), "unit": "elements/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "step_ms": spread(each), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOADS[name], "l2": "parameters, gradients and moments larger than L2",
                   "torch_multi_tensor_ms_per_step": torch_total / max(3, args.steps // 4)},
        "gpu_launches": args.steps,
        "roofline": {"bound": "hbm", "kernel": "hsn_tr_adamw", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": None, "peak_source": "measured" if peaks else "fallback",
                     "how": "28 bytes an element (p, g, m, v read; p, m, v written) / the step's mean event time"},
        "clocks": clocks_summary(clock_lines, 0)}))  # fmt: skip


def run_decoder(args, c: dict, name: str) -> None:
    """`--config decode`: `hsnw_window_decode` over the benchmark window's rows; a step = both layers."""
    import torch

    from hsn_b200.window import WindowDecoder, launch_profile, window_decode

    world, rank, local, dev = dist_setup()
    rows, d, H, V = c["rows"], c["d"], c["H"], c["V"]
    gen = torch.Generator(device=dev).manual_seed(0)
    f = lambda *shape: torch.randn(*shape, generator=gen, device=dev) * 0.2  # noqa: E731
    dec = WindowDecoder.build(f(H, 2 * d), f(H), f(V, H), f(V), d_q=d, device=dev, prod="bf16")
    qs, us = f(rows, d), f(rows, d)
    out: dict = {}
    for _ in range(max(3, args.warmup)):
        window_decode(dec, qs, us, out=out)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step(i):
        flush.zero_()   # (the operands are smaller than L2: written over between the steps)
        window_decode(dec, qs, us, out=out)

    with launch_profile() as prof:
        step(0)
    ms_total, each = timed_steps(step, args.steps, torch.cuda.synchronize)
    kernel_ms = prof.ms.get("decode", 0.0)
    flops = 2.0 * rows * (2 * d * H + H * V)
    print(json.dumps({
        "metric": "decoder rows/s", "value": rows / (kernel_ms * 1e-3), "unit": "rows/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": kernel_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 products", "data": "synthetic",
        "config": {"workload": WORKLOADS[name], "l2": "a 256 MB buffer is written between the steps",
                   "step_with_flush_ms": ms_total / args.steps},
        "gpu_launches": 2 * args.steps,
        "roofline": {"bound": "tensor", "kernel": "k_linear_tc", "achieved": flops / (kernel_ms * 1e-3) / 1e12, "peak": 1590.0,
                     "unit": "TFLOP/s", "frac": flops / (kernel_ms * 1e-3) / 1e12 / 1590.0, "traffic": None,
                     "how": "the two layers' 2 M N K flops / the two launches' event time in a profiled step; 3.2 GFLOP: the kernels are latency bound at this size"}}))  # fmt: skip


def run_units(args, c: dict, name: str) -> None:
    """`--config units`: `hsnw_units_forward` + `hsnw_units_backward` over every pair of the benchmark window; a step =
    the pass and its backward (sort, packing, eight tile products, reductions). Beside it the CPU restatement on a
    sample of the pairs, and PyTorch's own grouped bf16 products on the same device."""
    import torch

    from hsn_b200.kernels.units import grouped_backward, grouped_forward
    from hsn_b200.window import launch_profile

    world, rank, local, dev = dist_setup()
    P, M, d, H = c["pairs"], c["M"], c["d"], c["H"]
    gen = torch.Generator(device=dev).manual_seed(0)
    f = lambda *shape, scale=1.0: torch.randn(*shape, generator=gen, device=dev) * scale  # noqa: E731
    bank = [f(M, 4 * d, H, scale=(4 * d) ** -0.5), f(M, H, scale=0.3), f(M, H, d, scale=H**-0.5), f(M, d, scale=0.3)]
    v, cot = f(P, 4 * d), f(P, d).bfloat16()
    idx = torch.randint(0, M, (P,), generator=gen, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    kept: dict = {}

    def step(i):
        flush.zero_()   # (the window's operands are about the size of L2: written over between the steps)
        out, pre, _ = grouped_forward(v, idx, *bank, check=False)
        kept["grads"] = grouped_backward(v, idx, *bank, pre, cot, check=False)
        kept["out"] = out

    for i in range(max(3, args.warmup)):
        step(i)
    clock_lines: list = []
    stop = threading.Event()
    threading.Thread(target=sample_clocks, args=(stop, clock_lines), daemon=True).start()
    with launch_profile() as prof:
        step(0)
    ms_total, each = timed_steps(step, args.steps, torch.cuda.synchronize)
    stop.set()
    fwd_ms, bwd_ms = prof.ms.get("units_fwd", 0.0), prof.ms.get("units_bwd", 0.0)
    # PyTorch's own: pairs sorted by unit, bf16 addmm per unit and layer, autograd backward
    order = torch.argsort(idx, stable=True)
    counts = torch.bincount(idx, minlength=M).tolist()
    leaves = [b.clone().requires_grad_(True) for b in bank]

    def torch_step(i):
        vs = v.index_select(0, order).requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            outs, start = [], 0
            for j, n in enumerate(counts):
                hidden = torch.nn.functional.gelu(torch.addmm(leaves[1][j], vs[start:start + n], leaves[0][j]))
                outs.append(torch.addmm(leaves[3][j], hidden, leaves[2][j]))
                start += n
            out = torch.cat(outs)
        out.backward(cot.index_select(0, order))
        for leaf in leaves:
            leaf.grad = None

    for i in range(3):
        torch_step(i)
    torch_total, _ = timed_steps(torch_step, max(3, args.steps // 4), torch.cuda.synchronize)
    cpu = None
    if not args.no_cpu_baseline:
        from oracle import units_oracle as U

        n = 4096   # a sample of the pairs: about a second of numpy
        hv, hi, hc = v[:n].cpu().numpy(), idx[:n].cpu().numpy(), cot[:n].float().cpu().numpy()
        hb = [b.cpu().numpy() for b in bank]
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 10.0:
            _, hp = U.forward_grouped(hv, hi, *hb, bf16=True)
            U.backward_grouped(hv, hi, *hb, hp, hc, bf16=True)
            reps += 1
        cpu = {"value": reps * n / (time.perf_counter() - t0), "unit": "pairs/s", "cores": 1, "kind": "port",
               "sample": f"{reps} passes of forward + backward over {n} of the window's pairs (numpy restatement, bf16 rounding emulated)"}
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    kernel_ms = fwd_ms + bwd_ms
    flops = 3 * 2.0 * P * (4 * d * H + H * d)   # forward once, backward twice (inputs and weights)
    achieved = flops / (kernel_ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": "grouped unit pass pairs/s (forward + backward)", "value": P / (kernel_ms * 1e-3), "unit": "pairs/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": kernel_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 products", "data": "synthetic",
        "config": {"workload": WORKLOADS[name], "l2": "a 256 MB buffer is written between the steps",
                   "forward_ms": fwd_ms, "backward_ms": bwd_ms, "step_with_flush_ms": spread(each),
                   "torch_grouped_bf16_addmm_autograd_ms": torch_total / max(3, args.steps // 4)},
        "gpu_launches": 23 * args.steps,
        "roofline": {"bound": "tensor", "kernel": "k_units_tc", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak, "traffic": None, "peak_source": "measured (sustained)" if peaks else "fallback",
                     "how": "3 x 2 P (4d H + H d) flops (forward, and the backward's input and weight products) / the two calls' event time in a profiled step"},
        "cpu_baseline": cpu, "clocks": clocks_summary(clock_lines, 0)}))  # fmt: skip


def run_scorer(args, c: dict, name: str) -> None:
    """`--config scorer`: `hsnw_scorer_logits` + `hsnw_scorer_logits_backward` over the benchmark window's recorded
    state; a step = both (each one read of the state, 0.5 GB). Beside it the CPU restatement on a sample of the
    positions, and the reference's own formulation in PyTorch on the same device."""
    import torch

    from hsn_b200.kernels.scorer import scorer_logits_backward, scorer_logits_forward
    from hsn_b200.window import launch_profile

    world, rank, local, dev = dist_setup()
    R, N, d, M, S = c["R"], c["N"], c["d"], c["M"], c["S"]
    gen = torch.Generator(device=dev).manual_seed(0)
    f = lambda *shape, scale=1.0: torch.randn(*shape, generator=gen, device=dev) * scale  # noqa: E731
    weight, bias = f(M, 3 * d + 1 + S, scale=0.2), f(M, scale=0.3)
    feats = [f(R, d, scale=0.7), f(R, d, scale=0.4), f(R, N, d, scale=0.5), torch.randint(0, 300, (R, N), generator=gen, device=dev),
             f(R, N, S)]  # fmt: skip
    cot = f(R, N, M)
    kept: dict = {}

    def step(i):   # (the state alone is four times L2: nothing of one pass survives to the next)
        kept["out"] = scorer_logits_forward(weight, bias, *feats, age_max=100.0, check=False)
        kept["grads"] = scorer_logits_backward(weight, bias, *feats, cot, age_max=100.0, check=False)

    for i in range(max(3, args.warmup)):
        step(i)
    clock_lines: list = []
    stop = threading.Event()
    threading.Thread(target=sample_clocks, args=(stop, clock_lines), daemon=True).start()
    with launch_profile() as prof:
        step(0)
    ms_total, each = timed_steps(step, args.steps, torch.cuda.synchronize)
    stop.set()
    fwd_ms, bwd_ms = prof.ms.get("scorer_fwd", 0.0), prof.ms.get("scorer_bwd", 0.0)
    # the reference's formulation live: three linear maps under autocast, autograd's backward
    lw, lb = weight.clone().requires_grad_(True), bias.clone().requires_grad_(True)

    def torch_step(i):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            row = torch.nn.functional.linear(torch.cat(feats[:2], dim=-1), lw[:, : 2 * d])
            tail = torch.cat([(feats[3].float() / 100.0)[:, :, None], feats[4]], dim=-1)
            cells = torch.nn.functional.linear(feats[2], lw[:, 2 * d : 3 * d]).float()
            cells = cells + torch.nn.functional.linear(tail, lw[:, 3 * d :], lb).float()
            out = cells + row.float()[:, None, :]
        (out * cot).sum().backward()
        lw.grad = lb.grad = None

    for i in range(3):
        torch_step(i)
    torch_total, _ = timed_steps(torch_step, max(3, args.steps // 4), torch.cuda.synchronize)
    cpu = None
    if not args.no_cpu_baseline:
        from oracle import scorer_oracle as SO

        n = 64   # a sample of the positions
        host = [t[:n].cpu().numpy() for t in feats]
        hw, hb, hc = weight.cpu().numpy(), bias.cpu().numpy(), cot[:n].cpu().numpy()
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 10.0:
            SO.scorer_logits(hw, hb, *host, 100.0, bf16=True)
            SO.scorer_logits_backward(hw, *host, 100.0, hc, bf16=True)
            reps += 1
        cpu = {"value": reps * n * N / (time.perf_counter() - t0), "unit": "cells/s", "cores": 1, "kind": "port",
               "sample": f"{reps} passes of forward + backward over {n} of the window's positions (numpy restatement, bf16 rounding emulated)"}
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = float(peaks.get("hbm_gbs", 6650.0))
    cells = float(R) * N
    fwd_bytes = cells * (4 * d + 8 + 4 * S + 4 * M)   # state, age, scalars read; logits written
    bwd_bytes = cells * (4 * d + 8 + 4 * S + 4 * M)   # state, age, scalars and the cotangent read
    kernel_ms = fwd_ms + bwd_ms
    achieved = (fwd_bytes + bwd_bytes) / (kernel_ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "scorer logits cells/s (forward + weight gradients)", "value": cells / (kernel_ms * 1e-3), "unit": "cells/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": kernel_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 products, f32 tensors", "data": "synthetic",
        "config": {"workload": WORKLOADS[name], "l2": "the recorded state (537 MB) is larger than L2",
                   "forward_ms": fwd_ms, "backward_ms": bwd_ms, "step_ms": spread(each),
                   "torch_three_linear_maps_autocast_autograd_ms": torch_total / max(3, args.steps // 4)},
        "gpu_launches": 5 * args.steps,
        "roofline": {"bound": "hbm", "kernel": "k_scorer_fwd_tc + k_scorer_bwd_tc", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": 686.4e6 + 697.1e6,
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of the two kernels at this size (profiles/scorer_c2.md)", "peak_source": "measured" if peaks else "fallback",
                     "forward": {"achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9, "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak},
                     "backward": {"achieved": bwd_bytes / (bwd_ms * 1e-3) / 1e9, "frac": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / peak},
                     "how": "per cell 4 d + 8 + 4 S + 4 M bytes each way (state, age, scalars, and logits written or cotangent read) / the calls' event time in a profiled step"},
        "cpu_baseline": cpu, "clocks": clocks_summary(clock_lines, 0)}))  # fmt: skip


TAIL_METRIC = "replay tail slots/s (forward + backward)"


def run_tail(args, c: dict, name: str) -> None:
    """`--config tail`: `hsnw_tail_forward` + `hsnw_tail_backward` over the benchmark window's slots; a step = both.
    Beside it the CPU restatement on a sample of the slots, and the reference's three lines in PyTorch on the same
    device."""
    import torch

    from hsn_b200.kernels.tail import tail_backward, tail_forward
    from hsn_b200.window import launch_profile

    world, rank, local, dev = dist_setup()
    P, d = c["slots"], c["d"]
    gen = torch.Generator(device=dev).manual_seed(0)
    f = lambda *shape, scale=1.0: torch.randn(*shape, generator=gen, device=dev) * scale  # noqa: E731
    x = f(P, d, scale=0.6).to(torch.bfloat16)
    alpha = (torch.rand(P, generator=gen, device=dev) > 0.05).float()
    w, g, cot = f(d, d, scale=d**-0.5), 1.0 + f(d, scale=0.2), f(P, d)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # the pass's tensors (76 MB) fit L2: flushed between steps

    class flush:   # written, then read: the read pushes the write's dirty lines out, so the timed kernels do not pay for them
        @staticmethod
        def zero_():
            flush_buf.zero_()
            flush_buf.view(torch.int64).sum()

    # the two entry points straight through the C ABI on buffers made once (what a caller that holds its buffers
    # pays); the Python wrappers' answers are the check
    import ctypes

    from hsn_b200 import _lib

    lib = _lib.library()
    if not lib.hsnw_prepared(local):
        _lib.check(lib.hsnw_prepare(local))
    st = _lib.HsnwTail(d=d, prod_bf16=1, norm_eps=1e-6, reserved=0, w_out=w.data_ptr(), norm_weight=g.data_ptr())
    y, cand = torch.empty(P, d, device=dev), torch.empty(P, d, device=dev)
    d_x, d_a = torch.empty_like(x), torch.empty(P, device=dev)
    d_w, d_g = torch.empty(d, d, device=dev), torch.empty(d, device=dev)
    need = int(lib.hsnw_tail_scratch_bytes(ctypes.byref(st), P))
    scratch = torch.empty(need, dtype=torch.uint8, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    def step(i):
        flush.zero_()
        _lib.check(lib.hsnw_tail_forward(ctypes.byref(st), x.data_ptr(), alpha.data_ptr(), P, y.data_ptr(), cand.data_ptr(), stream))
        _lib.check(lib.hsnw_tail_backward(ctypes.byref(st), x.data_ptr(), alpha.data_ptr(), y.data_ptr(), cot.data_ptr(), P, d_x.data_ptr(),
                                          d_a.data_ptr(), d_w.data_ptr(), d_g.data_ptr(), scratch.data_ptr(), need, stream))  # fmt: skip

    for i in range(max(3, args.warmup)):
        step(i)
    want_c, want_y = tail_forward(x, alpha, w, g)
    want = tail_backward(x, alpha, w, g, want_y, cot)
    if not (torch.equal(cand, want_c) and torch.equal(y, want_y) and all(torch.equal(a, b) for a, b in zip((d_x, d_a, d_w, d_g), want, strict=True))):
        raise SystemExit("bench.py --config tail: the direct calls and the Python wrappers disagree")
    clock_lines: list = []
    stop = threading.Event()
    threading.Thread(target=sample_clocks, args=(stop, clock_lines), daemon=True).start()
    fwd_ms = bwd_ms = 0.0
    for i in range(5):   # the calls are tens of microseconds: the mean of five profiled steps
        with launch_profile() as prof:
            step(i)
        fwd_ms += prof.ms.get("tail_fwd", 0.0) / 5
        bwd_ms += prof.ms.get("tail_bwd", 0.0) / 5
    ms_total, each = timed_steps(step, args.steps, torch.cuda.synchronize)
    stop.set()
    lin = torch.nn.Linear(d, d, bias=False, device=dev)
    norm = torch.nn.RMSNorm(d, eps=1e-6, device=dev)

    def torch_step(i):
        flush.zero_()
        xr, ar = x.clone().requires_grad_(True), alpha.clone().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = lin(xr).to(torch.float32)
        torch.tanh(ar[:, None] * norm(y)).backward(cot)
        lin.weight.grad = norm.weight.grad = None

    for i in range(3):
        torch_step(i)
    torch_total, torch_each = timed_steps(torch_step, max(3, args.steps // 4), torch.cuda.synchronize)
    cpu = None
    if not args.no_cpu_baseline:
        from oracle import tail_oracle as TO

        n = 16384
        hx, ha, hw, hg, hc = (t.float().cpu().numpy() for t in (x[:n], alpha[:n], w, g, cot[:n]))
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 10.0:
            _, hy = TO.forward_tail(hx, ha, hw, hg, bf16=True)
            TO.backward_tail(hx, ha, hw, hg, hy, hc, bf16=True)
            reps += 1
        cpu = {"value": reps * n / (time.perf_counter() - t0), "unit": "slots/s", "cores": blas_threads(), "kind": "port",
               "sample": f"{reps} passes of forward + backward over {n} of the window's slots (numpy restatement, bf16 rounding emulated)"}
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = float(peaks.get("hbm_gbs", 6650.0))
    fwd_bytes = float(P) * (2 * d + 4 + 8 * d)            # unit_out (bf16), alpha read; y, c written
    bwd_bytes = float(P) * (2 * d + 4 + 8 * d + 2 * d + 4)   # unit_out, alpha, y, d_c read; d_unit_out (bf16), d_alpha written
    kernel_ms = fwd_ms + bwd_ms
    achieved = (fwd_bytes + bwd_bytes) / (kernel_ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": TAIL_METRIC, "value": P / (kernel_ms * 1e-3), "unit": "slots/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": kernel_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 products, f32 norm and tanh", "data": "synthetic",
        "config": {"workload": WORKLOADS[name], "l2": "256 MB written, then read, between steps (the pass's tensors fit L2; the read leaves no dirty lines for the timed kernels to evict)",
                   "forward_ms": fwd_ms, "backward_ms": bwd_ms, "step_ms_with_flush_and_host": spread(each),
                   "torch_linear_rmsnorm_tanh_autocast_autograd_ms_with_flush": spread(torch_each)},
        "gpu_launches": 3 * args.steps,
        "roofline": {"bound": "hbm", "kernel": "k_tail_fwd + k_tail_bwd", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": None, "peak_source": "measured" if peaks else "fallback",
                     "forward": {"achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9, "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak},
                     "backward": {"achieved": bwd_bytes / (bwd_ms * 1e-3) / 1e9, "frac": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / peak},
                     "how": "per slot 10 d + 4 bytes forward (unit_out as bf16, alpha, y and c written) and 12 d + 8 backward / the calls' event time, mean of five profiled steps"},
        "cpu_baseline": cpu, "clocks": clocks_summary(clock_lines, 0)}))  # fmt: skip


GATE_METRIC = "replay norm + gate slots/s (forward + backward)"


def run_gate(args, c: dict, name: str) -> None:
    """`--config gate`: `hsnw_gate_forward` + `hsnw_gate_backward` over the benchmark window's slots through the C ABI on
    buffers made once; a step = both. Beside it the CPU restatement on a sample of the slots, and the reference's lines
    in PyTorch on the same device."""
    import ctypes

    import torch

    from hsn_b200 import _lib
    from hsn_b200.kernels.gate import norm_gate_backward, norm_gate_forward
    from hsn_b200.window import launch_profile

    world, rank, local, dev = dist_setup()
    P, d = c["slots"], c["d"]
    F = 4 * d
    gen = torch.Generator(device=dev).manual_seed(0)
    f = lambda *shape, scale=1.0: torch.randn(*shape, generator=gen, device=dev) * scale  # noqa: E731
    x, nw, gw, gb = f(P, F, scale=0.8), 1.0 + f(F, scale=0.2), f(d, F, scale=F**-0.5), f(d, scale=0.3)
    d_v, d_b = f(P, F), f(P, d)
    lib = _lib.library()
    if not lib.hsnw_prepared(local):
        _lib.check(lib.hsnw_prepare(local))
    st = _lib.HsnwGate(d=d, prod_bf16=1, norm_eps=1e-6, reserved=0, norm_weight=nw.data_ptr(), gate_w=gw.data_ptr(), gate_b=gb.data_ptr())
    v, rms, gp, b = torch.empty(P, F, device=dev), torch.empty(P, device=dev), torch.empty(P, d, device=dev), torch.empty(P, d, device=dev)
    d_x, d_nw, d_gw, d_gb = torch.empty(P, F, device=dev), torch.empty(F, device=dev), torch.empty(d, F, device=dev), torch.empty(d, device=dev)
    need_f = int(lib.hsnw_gate_scratch_bytes(ctypes.byref(st), P, 0))
    need_b = int(lib.hsnw_gate_scratch_bytes(ctypes.byref(st), P, 1))
    scr_f, scr_b = torch.empty(need_f, dtype=torch.uint8, device=dev), torch.empty(need_b, dtype=torch.uint8, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    def step(i):   # (the pass's tensors, 300 MB, are more than twice L2: nothing of one pass survives to the next)
        _lib.check(lib.hsnw_gate_forward(ctypes.byref(st), x.data_ptr(), P, v.data_ptr(), rms.data_ptr(), gp.data_ptr(), b.data_ptr(),
                                         scr_f.data_ptr(), need_f, stream))  # fmt: skip
        _lib.check(lib.hsnw_gate_backward(ctypes.byref(st), x.data_ptr(), gp.data_ptr(), d_v.data_ptr(), d_b.data_ptr(), P, d_x.data_ptr(),
                                          d_nw.data_ptr(), d_gw.data_ptr(), d_gb.data_ptr(), scr_b.data_ptr(), need_b, stream))  # fmt: skip

    for i in range(max(3, args.warmup)):
        step(i)
    want = norm_gate_forward(x, nw, gw, gb)
    wantb = norm_gate_backward(x, nw, gw, gb, want[2], d_v, d_b)
    if not (all(torch.equal(a, w) for a, w in zip((v, rms, gp, b), want, strict=True))
            and all(torch.equal(a, w) for a, w in zip((d_x, d_nw, d_gw, d_gb), wantb, strict=True))):
        raise SystemExit("bench.py --config gate: the direct calls and the Python wrappers disagree")
    clock_lines: list = []
    stop = threading.Event()
    threading.Thread(target=sample_clocks, args=(stop, clock_lines), daemon=True).start()
    fwd_ms = bwd_ms = 0.0
    for i in range(5):
        with launch_profile() as prof:
            step(i)
        fwd_ms += prof.ms.get("gate_fwd", 0.0) / 5
        bwd_ms += prof.ms.get("gate_bwd", 0.0) / 5
    ms_total, each = timed_steps(step, args.steps, torch.cuda.synchronize)
    stop.set()
    norm = torch.nn.RMSNorm(F, eps=1e-6, device=dev)
    gate = torch.nn.Linear(F, d, device=dev)

    def torch_step(i):
        xr = x.clone().requires_grad_(True)
        vr = norm(xr)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            pre = gate(vr).to(torch.float32)
        torch.autograd.backward([vr, torch.sigmoid(pre)], [d_v, d_b])
        norm.weight.grad = gate.weight.grad = gate.bias.grad = None

    for i in range(3):
        torch_step(i)
    torch_total, torch_each = timed_steps(torch_step, max(3, args.steps // 4), torch.cuda.synchronize)
    cpu = None
    if not args.no_cpu_baseline:
        from oracle import gate_oracle as GO

        n = 16384
        hx, hnw, hgw, hgb, hdv, hdb = (t.cpu().numpy() for t in (x[:n], nw, gw, gb, d_v[:n], d_b[:n]))
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 10.0:
            GO.forward_norm_gate(hx, hnw, hgw, hgb, norm_eps=1e-6, bf16=True)
            GO.backward_norm_gate(hx, hnw, hgw, hgb, hdv, hdb, norm_eps=1e-6, bf16=True)
            reps += 1
        cpu = {"value": reps * n / (time.perf_counter() - t0), "unit": "slots/s", "cores": blas_threads(), "kind": "port",
               "sample": f"{reps} passes of forward + backward over {n} of the window's slots (numpy restatement, bf16 rounding emulated)"}
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = float(peaks.get("hbm_gbs", 6650.0))
    fwd_bytes = float(P) * (16 * d + 16 * d + 4 + 8 * d)    # v_raw read; v, rms, gate_pre, b written
    bwd_bytes = float(P) * (16 * d + 16 * d + 8 * d + 16 * d)   # v_raw, d_v_units, gate_pre and d_b read; d_v_raw written
    kernel_ms = fwd_ms + bwd_ms
    achieved = (fwd_bytes + bwd_bytes) / (kernel_ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": GATE_METRIC, "value": P / (kernel_ms * 1e-3), "unit": "slots/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": kernel_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 norm, bf16 products", "data": "synthetic",
        "config": {"workload": WORKLOADS[name], "l2": "the pass's tensors (300 MB) are larger than L2",
                   "forward_ms": fwd_ms, "backward_ms": bwd_ms, "step_ms": spread(each),
                   "torch_rmsnorm_linear_sigmoid_autocast_autograd_ms": spread(torch_each)},
        "gpu_launches": 3 * args.steps,
        "roofline": {"bound": "hbm", "kernel": "k_gate_fwd + k_gate_bwd", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": None, "peak_source": "measured" if peaks else "fallback",
                     "forward": {"achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9, "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak},
                     "backward": {"achieved": bwd_bytes / (bwd_ms * 1e-3) / 1e9, "frac": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / peak},
                     "how": "per slot 40 d + 4 bytes forward (v_raw read; v, rms, gate_pre, b written) and 56 d backward (v_raw, the unit pass's gradient, gate_pre, d_b read; d_v_raw written) / the calls' event time, mean of five profiled steps"},
        "cpu_baseline": cpu, "clocks": clocks_summary(clock_lines, 0)}))  # fmt: skip


MSG_METRIC = "replay messages slots/s (forward + backward)"


def run_messages(args, c: dict, name: str) -> None:
    """`--config messages`: `hsnw_messages_forward` + `hsnw_messages_backward` over the benchmark window's slots through
    the C ABI on buffers made once; a step = both. Beside it the CPU restatement on a sample of the positions, and the
    reference's lines in PyTorch on the same device."""
    import ctypes

    import torch

    from hsn_b200 import _lib
    from hsn_b200.kernels.messages import messages_backward, messages_forward
    from hsn_b200.window import launch_profile

    world, rank, local, dev = dist_setup()
    R, N, d, K, D = c["R"], c["N"], c["d"], c["K"], c["D"]
    gen = torch.Generator(device=dev).manual_seed(0)
    f = lambda *shape, scale=1.0: torch.randn(*shape, generator=gen, device=dev) * scale  # noqa: E731
    u, eps, h = f(R, d, scale=0.7), f(R, d, scale=0.4), f(R, N, d, scale=0.5)
    cells = torch.rand(R, N, generator=gen, device=dev).argsort(dim=1)[:, :K].contiguous()
    pad_src = torch.randint(0, N, (N, D), generator=gen, device=dev)
    edge_w = torch.softmax(f(N, D), dim=1)
    v_w, d_v_raw = f(d, d, scale=d**-0.5), f(R, K, 4 * d)
    lib = _lib.library()
    if not lib.hsnw_prepared(local):
        _lib.check(lib.hsnw_prepare(local))
    st = _lib.HsnwMessages(d=d, n_cells=N, degree=D, k=K, prod_bf16=1, reserved=0, v_w=v_w.data_ptr(), edge_w=edge_w.data_ptr(),
                           pad_src=pad_src.data_ptr())  # fmt: skip
    v_raw = torch.empty(R, K, 4 * d, device=dev)
    d_u, d_eps, d_ew, d_vw = torch.empty(R, d, device=dev), torch.empty(R, d, device=dev), torch.empty(N, D, device=dev), torch.empty(d, d, device=dev)
    need = int(lib.hsnw_messages_scratch_bytes(ctypes.byref(st), R))
    scratch = torch.empty(need, dtype=torch.uint8, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    def step(i):   # (the recorded state alone, 537 MB, is four times L2)
        _lib.check(lib.hsnw_messages_forward(ctypes.byref(st), u.data_ptr(), eps.data_ptr(), h.data_ptr(), cells.data_ptr(), R, v_raw.data_ptr(), stream))
        _lib.check(lib.hsnw_messages_backward(ctypes.byref(st), h.data_ptr(), cells.data_ptr(), d_v_raw.data_ptr(), R, d_u.data_ptr(), d_eps.data_ptr(),
                                              d_ew.data_ptr(), d_vw.data_ptr(), scratch.data_ptr(), need, stream))  # fmt: skip

    for i in range(max(3, args.warmup)):
        step(i)
    want = messages_forward(u, eps, h, cells, pad_src, edge_w, v_w)
    wantb = messages_backward(h, cells, pad_src, edge_w, v_w, d_v_raw)
    if not (torch.equal(v_raw, want) and all(torch.equal(a, w) for a, w in zip((d_u, d_eps, d_ew, d_vw), wantb, strict=True))):
        raise SystemExit("bench.py --config messages: the direct calls and the Python wrappers disagree")
    clock_lines: list = []
    stop = threading.Event()
    threading.Thread(target=sample_clocks, args=(stop, clock_lines), daemon=True).start()
    fwd_ms = bwd_ms = 0.0
    for i in range(5):
        with launch_profile() as prof:
            step(i)
        fwd_ms += prof.ms.get("msg_fwd", 0.0) / 5
        bwd_ms += prof.ms.get("msg_bwd", 0.0) / 5
    ms_total, each = timed_steps(step, args.steps, torch.cuda.synchronize)
    stop.set()
    lin = torch.nn.Linear(d, d, bias=False, device=dev)
    ew = edge_w.clone().requires_grad_(True)

    def torch_step(i):
        ur, er = u.clone().requires_grad_(True), eps.clone().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            index = pad_src[cells].reshape(R, K * D, 1).expand(R, K * D, d)
            sources = lin(h.gather(1, index)).reshape(R, K, D, d)
            m = (sources * ew.to(sources.dtype)[cells][..., None]).sum(dim=2)
        h_sel = h.gather(1, cells[..., None].expand(R, K, d))
        out = torch.cat([ur[:, None].expand(R, K, d), er[:, None].expand(R, K, d), h_sel, m.to(torch.float32)], dim=-1)
        out.backward(d_v_raw)
        lin.weight.grad = ew.grad = None

    for i in range(3):
        torch_step(i)
    torch_total, torch_each = timed_steps(torch_step, max(3, args.steps // 4), torch.cuda.synchronize)
    cpu = None
    if not args.no_cpu_baseline:
        from oracle import messages_oracle as MO

        n = 128
        hu, he, hh, hc, hs, hw, hv, hd = (t.cpu().numpy() for t in (u[:n], eps[:n], h[:n], cells[:n], pad_src, edge_w, v_w, d_v_raw[:n]))
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 10.0:
            MO.forward_messages(hu, he, hh, hc, hs, hw, hv, bf16=True)
            MO.backward_messages(hh, hc, hs, hw, hv, hd, bf16=True)
            reps += 1
        cpu = {"value": reps * n * K / (time.perf_counter() - t0), "unit": "slots/s", "cores": blas_threads(), "kind": "port",
               "sample": f"{reps} passes of forward + backward over {n} of the window's positions (numpy restatement, bf16 rounding emulated)"}
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = float(peaks.get("hbm_gbs", 6650.0))
    P = float(R) * K
    fwd_bytes = P * (4 * d * (D + 1) + 8 + 16 * d) + R * 8.0 * d     # D + 1 rows of the state and the cell index read, v_raw written; u, eps a row
    bwd_bytes = P * (4 * d * D + 8 + 16 * d) + R * 8.0 * d           # D rows of the state, the cell index, d_v_raw read; d_u, d_eps written
    kernel_ms = fwd_ms + bwd_ms
    achieved = (fwd_bytes + bwd_bytes) / (kernel_ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": MSG_METRIC, "value": P / (kernel_ms * 1e-3), "unit": "slots/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": kernel_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 products, f32 tensors", "data": "synthetic",
        "config": {"workload": WORKLOADS[name], "l2": "the recorded state (537 MB) is larger than L2",
                   "forward_ms": fwd_ms, "backward_ms": bwd_ms, "step_ms": spread(each),
                   "torch_gather_linear_sum_cat_autocast_autograd_ms": spread(torch_each)},
        "gpu_launches": 5 * args.steps,
        "roofline": {"bound": "hbm", "kernel": "k_msg_fwd + k_msg_bwd", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": None, "peak_source": "measured" if peaks else "fallback",
                     "forward": {"achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9, "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak},
                     "backward": {"achieved": bwd_bytes / (bwd_ms * 1e-3) / 1e9, "frac": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / peak},
                     "how": "per slot 4 d (D + 1) + 8 + 16 d bytes forward (the cell's and its D in-neighbours' rows of the state, the cell index; v_raw written) and 4 d D + 8 + 16 d backward (the in-neighbours' rows, the cell index, d_v_raw) / the calls' event time, mean of five profiled steps"},
        "cpu_baseline": cpu, "clocks": clocks_summary(clock_lines, 0)}))  # fmt: skip


def run_trainer_sharded(args, c: dict, name: str, world: int, rank: int, dev) -> None:
    """`--config adamw --gpus N`: the same parameter vector replicated on N ranks, a step = the gradient exchange
    and the AdamW step as ONE kernel per rank over peer memory (`ShardedAdamW`: reduce-scatter, step, all-gather),
    with the unfused sequence beside it (NCCL all-reduce of the flat gradients, then `hsn_tr_adamw` on every
    rank). Strong scaling: the vector does not grow with N."""
    import torch
    import torch.distributed as dist

    from hsn_b200.kernels import trainer
    from hsn_b200.parallel import ShardedAdamW

    total = c["tensors"] * c["elements"]
    hyper = dict(lr=2.5e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    opt = ShardedAdamW(total, **hyper)
    gen = torch.Generator(device=dev).manual_seed(rank)
    opt.params.copy_(torch.randn(opt.params.numel(), generator=torch.Generator(device=dev).manual_seed(0), device=dev) * 0.1)
    opt.grads.copy_(torch.randn(opt.grads.numel(), generator=gen, device=dev))

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        opt.step()
    ms_total, each = timed_steps(lambda i: opt.step(), args.steps, barrier)
    # the unfused sequence on plain buffers
    flat_g = opt.grads.clone()
    p, m, v = opt.params.clone(), torch.zeros_like(opt.params), torch.zeros_like(opt.params)
    count = [0]

    def unfused(i):
        count[0] += 1
        dist.all_reduce(flat_g)
        flat_g.mul_(1.0 / world)
        trainer.adamw([p], [flat_g], [m], [v], lr=2.5e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01, step=count[0])

    for i in range(3):
        unfused(i)
    other_total, _ = timed_steps(unfused, max(3, args.steps // 2), barrier)
    times = torch.tensor([ms_total, other_total], device=dev)
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    if rank == 0:
        step_ms, other_ms = float(times[0]) / args.steps, float(times[1]) / max(3, args.steps // 2)
        link = 2 * 4.0 * (world - 1) * opt.shard   # bytes that ARRIVE at a rank a step: what it reads from its peers and what they write into it (as many leave)
        print(json.dumps({
            "metric": "trainer AdamW elements/s", "value": total / (step_ms * 1e-3), "unit": "elements/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "step_ms": spread(each), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOADS[name] + f", replicated on {world} ranks: gradient exchange + step fused over peer memory",
                       "shard_elements": opt.shard, "unfused_nccl_allreduce_then_adamw_ms_per_step": other_ms},
            "gpu_launches": args.steps,
            "roofline": {"bound": "nvlink", "kernel": "k_exchange_adamw", "achieved": link / (step_ms * 1e-3) / 1e9, "peak": 770.0,
                         "unit": "GB/s", "frac": link / (step_ms * 1e-3) / 1e9 / 770.0, "traffic": None,
                         "how": "bytes arriving at a rank a step (its reads of the peers' gradients + the peers' writes of its parameters; as many leave) / the step's time, of the measured 770 GB/s a direction"}}))  # fmt: skip
    dist.destroy_process_group()


def _torch_adamw(torch, ps, gs, ms, vs, step, lr=2.5e-3, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.01) -> None:
    """The multi-tensor sequence `hsn_tr_adamw` replaces (reference python/hsn/train/lazy_adam.py:462-486)."""
    torch._foreach_mul_(ps, 1 - lr * wd)
    torch._foreach_lerp_(ms, gs, 1 - beta1)
    torch._foreach_mul_(vs, beta2)
    torch._foreach_addcmul_(vs, gs, gs, value=1 - beta2)
    den = torch._foreach_sqrt(vs)
    torch._foreach_div_(den, (1 - beta2**step) ** 0.5)
    torch._foreach_add_(den, eps)
    torch._foreach_addcdiv_(ps, ms, den, value=-(lr / (1 - beta1**step)))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2", choices=sorted(CONFIGS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--phases", action="store_true",
                    help="run the batch-synchronous phase kernels instead of the per-row cluster kernels")
    ap.add_argument("--positions", type=int, default=0,
                    help="shorten the window to this many positions (profiler captures only; not a benchmark number)")
    ap.add_argument("--rows", type=int, default=0, help="rows per GPU instead of the configuration's")
    args = ap.parse_args()
    c = dict(CONFIGS[args.config])
    if args.positions > 0:
        c["T"] = args.positions
    if c.get("decoder"):
        if args.steps == 100:
            args.steps = 20
        run_decoder(args, c, args.config)
    elif c.get("units") or c.get("scorer") or c.get("tail") or c.get("gate") or c.get("messages"):
        if args.steps == 100:
            args.steps = 20
        if args.impl == "reference":
            run_side_reference(args, c, args.config)
        elif c.get("units"):
            run_units(args, c, args.config)
        elif c.get("tail"):
            run_tail(args, c, args.config)
        elif c.get("gate"):
            run_gate(args, c, args.config)
        elif c.get("messages"):
            run_messages(args, c, args.config)
        else:
            run_scorer(args, c, args.config)
    elif c.get("trainer"):
        if args.steps == 100:
            args.steps = 20 if args.impl == "ours" else 5
        run_trainer(args, c, args.config)
    elif args.impl == "reference":
        if args.steps == 100:   # the default is sized for the GPU arm
            args.steps = 20
        run_reference(args, c, args.config)
    elif c.get("resident"):
        if args.steps == 100:
            args.steps = 10
        run_resident(args, c, args.config)
    else:
        if args.steps == 100 and c.get("windows", 1) > 1:
            args.steps = 10
        run_taped(args, c, args.config)


if __name__ == "__main__":
    main()
