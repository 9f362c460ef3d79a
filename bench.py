"""Benchmark of the HSN window path: window row-positions per second, forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c2|c3|c1]

A *step* is one TBPTT window for the rank's rows: the forward sweep (tape + record) and the
state-gradient reverse sweep with synthetic cotangents, on seeded synthetic inputs of the
benchmark configuration's shapes (uniform random bytes stand in for the reference's data set; the
window reads them as encoder outputs ``z``, context embeddings and scorer scalars). One JSON line
is printed by rank 0. ``--impl reference`` times the CPU restatement of the reference's window
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
    "c3": dict(B=64, T=512, N=512, d=64, K=8, H=512, M=8, D=4, S=9, p=1 / 1024, prod="bf16"),
    # the resident contract (no state tape; the state lives in HBM between calls): one GPU's share at 8 GPUs
    "c4": dict(B=32, T=1024, N=4096, d=128, K=16, H=1024, M=8, D=4, S=9, p=1 / 1024, prod="bf16", resident=True),
    "c5": dict(B=512, T=32, N=1024, d=64, K=8, H=512, M=8, D=4, S=9, p=1 / 4096, prod="bf16", resident=True,
               forward_only=True),
    # the same streams token by token: one hsnw_stream_step, then hsnw_stream_continue per position
    "c5s": dict(B=512, T=32, N=1024, d=64, K=8, H=512, M=8, D=4, S=9, p=1 / 4096, prod="bf16", resident=True,
                forward_only=True, stream=True),
}
WORKLOADS = {
    "c1": "tiny gradcheck-shape window B2 T8 N16 d32 K2 H32",
    "c2": "reference-shape window fwd+bwd: B32 T256 N256 d64 K8 H512 M8 D4, bf16 products, fp32 state, resets p=1/1024",
    "c3": "one window of the split-window chain: B64 T512 N512 d64 K8 H512, bf16 products",
    "c4": "scaled sparse routing, one GPU's 32 rows of B256: T1024 N4096 d128 K16 H1024, resident state, fwd+bwd",
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
NCU_TRAFFIC_PER_LAUNCH: dict[str, dict[str, float]] = {
    "c2": {"rows_fwd": 852.4e6, "rows_bwd": 293.3e6, "front": 2.798e6, "row": 1.375e6, "unit": 3.419e6, "update": 0.526e6, "mid": 2.254e6, "tail_head": 1.703e6},
}


def synthetic(c: dict, rank: int, rows: int):
    """Seeded inputs of the configuration's shapes; every row's data depends on its global row
    index only, so the result does not depend on the number of GPUs."""
    from hsn_b200.window import synthetic_weights

    W = synthetic_weights(np.random.default_rng(0), N=c["N"], d=c["d"], K=c["K"], H=c["H"], M=c["M"],
                          D=c["D"], S=c["S"], age_max=2**31 - 1)  # fmt: skip
    T, N, d, K, S = c["T"], c["N"], c["d"], c["K"], c["S"]
    parts = []
    for r in range(rows):
        rng = np.random.default_rng(1000 + rank * rows + r)
        tokens = rng.integers(0, 256, T)  # uniform bytes; the window sees them through z
        z = rng.standard_normal((T, d)).astype(np.float32) * 0.5 + (tokens[:, None] / 255.0 - 0.5).astype(np.float32)
        ctx = (rng.standard_normal((T, d)) * 0.02).astype(np.float32)
        scalars = rng.random((T, N, S)).astype(np.float32)
        reset = rng.random(T) < c["p"]
        reset[0] = True
        cot = [rng.standard_normal(s).astype(np.float32) * 0.1 for s in ((T, d), (T, d), (T, K, d))]
        parts.append((z, ctx, scalars, reset, *cot))
    stack = [np.stack([p[i] for p in parts]) for i in range(7)]
    return W, stack


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


def cpu_window(W, data, rows: int, positions: int):
    """The oracle's window forward + state-gradient backward on ``rows`` x ``positions`` of the
    workload; returns seconds."""
    from oracle import window_oracle as O

    W = O.WindowWeights(**vars(W))   # the same weights in the oracle's container
    z, ctx, scalars, reset, pre, post, sel = (a[:rows, :positions] for a in data)
    N, d = W.pad_src.shape[0], z.shape[-1]
    state = (np.zeros((rows, N, d), np.float32), np.zeros((rows, d), np.float32), np.zeros((rows, N), np.int64),
             np.zeros(rows, np.int64))  # fmt: skip
    t0 = time.perf_counter()
    tape = O.window_forward(W, z, ctx, scalars, reset, *state)
    valid = tape["sel_valid"]
    rec = {k: tape["rec_" + k] for k in ("y", "hidden", "gate_pre", "m", "rms")}
    O.state_gradient_backward(
        W, tape["rec_c"], tape["rec_b"], tape["rec_h_old"], np.where(valid, tape["sel_cell_idx"], 0),
        np.where(valid, tape["sel_unit_idx"], 0), valid, reset, N, pre, post, sel, rec,
    )  # fmt: skip
    return time.perf_counter() - t0


def cpu_baseline(c: dict, W, data, budget_s: float = 12.0) -> dict:
    rows = min(c["B"], data[0].shape[0])
    probe = min(2, c["T"])
    dt = cpu_window(W, data, rows, probe)
    positions = int(max(probe, min(c["T"], budget_s / max(dt / probe, 1e-6))))
    seconds = cpu_window(W, data, rows, positions)
    try:
        from threadpoolctl import threadpool_info

        threads = max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
    except Exception:
        threads = os.cpu_count() or 1
    return {
        "value": rows * positions / seconds,
        "unit": "row-positions/s",
        "cores": int(threads),
        "kind": "port",
        "sample": f"{rows} rows x {positions} positions of the workload, fp32, numpy oracle (BLAS threads = cores), {seconds:.1f} s",
    }


def run_reference(args, c: dict, name: str) -> None:
    """The CPU arm: the reference's window as restated in oracle/ (the reference is Python and is
    not present on the benchmark machine; the restatement is pinned to it by tests/golden)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    positions = min(c["T"], 4)
    if c.get("resident"):   # only the sampled positions are drawn: the full inputs are too large for the host
        c = dict(c, T=positions)
    W, data = synthetic(c, 0, min(c["B"], 8))
    rows = data[0].shape[0]
    for _ in range(args.warmup):
        cpu_window(W, data, rows, positions)
    times = [cpu_window(W, data, rows, positions) for _ in range(args.steps)]
    sec = float(np.mean(times))
    value = rows * positions / sec
    try:
        from threadpoolctl import threadpool_info

        threads = max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
    except Exception:
        threads = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": "window row-positions/s fwd+bwd", "value": value, "unit": "row-positions/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOADS[name], "sample": f"{rows} rows x {positions} positions per step"},
        "cpu_baseline": {"value": value, "unit": "row-positions/s", "cores": int(threads), "kind": "port",
                         "sample": f"{rows} rows x {positions} positions per step, numpy oracle"},
        "e2e": {"value": value, "unit": "row-positions/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }  # fmt: skip
    print(json.dumps(line), flush=True)


def run_resident(args, c: dict, name: str) -> None:
    """The configurations of the resident contract (one GPU): inputs drawn on the device from a
    seed (their host copies would not fit a pinned buffer), the state updated in place from call
    to call, CUDA events around ``steps`` calls. Not the headline line: no end-to-end leg."""
    import torch

    from hsn_b200.window import WindowModel, launch_profile, synthetic_weights, window_backward, window_forward

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the window path has no CPU fallback")
    dev = torch.device("cuda", 0)
    B, T, N, d, K, S = c["B"], c["T"], c["N"], c["d"], c["K"], c["S"]
    W = synthetic_weights(np.random.default_rng(0), N=N, d=d, K=K, H=c["H"], M=c["M"], D=c["D"], S=S,
                          age_max=2**31 - 1)  # fmt: skip
    model = WindowModel.from_weights(W, device=dev, prod=c["prod"], row_clusters=not args.phases)
    gen = torch.Generator(device=dev).manual_seed(1)
    z = torch.randn((B, T, d), device=dev, generator=gen) * 0.5
    ctx = torch.randn((B, T, model.dims["dc"]), device=dev, generator=gen) * 0.02
    scalars = torch.rand((B, T, N, S), device=dev, generator=gen)
    reset = torch.rand((B, T), device=dev, generator=gen) < c["p"]
    cots = [torch.randn(shape, device=dev, generator=gen) * 0.1 for shape in ((B, T, d), (B, T, d), (B, T, K, d))]
    state = (torch.zeros((B, N, d), device=dev), torch.zeros((B, d), device=dev),
             torch.zeros((B, N), dtype=torch.int64, device=dev), torch.zeros(B, dtype=torch.int64, device=dev))  # fmt: skip
    forward_only = bool(c.get("forward_only"))
    out: dict = {}
    bw_scratch = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    per_position = [tuple(a[:, t].contiguous() for a in (z, ctx, scalars, reset)) for t in range(T)] if c.get("stream") else []
    calls = [0]

    def step():
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
        window_backward(model, tape["rec_c"], tape["rec_b"], tape["rec_h_old"], tape["sel_cell_idx"],
                        tape["sel_unit_idx"], tape["sel_valid"], reset, cots[0], cots[1], cots[2], rec,
                        scratch=bw_scratch)  # fmt: skip

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    stop, lines = threading.Event(), []
    sampler = threading.Thread(target=sample_clocks, args=(stop, lines), daemon=True)
    sampler.start()
    time.sleep(0.3)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    stop.set()
    sampler.join(timeout=2)
    with launch_profile() as prof:
        step()
    torch.cuda.synchronize()
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    peaks = json.loads(peaks_file.read_text()) if peaks_file.exists() else {}
    peak = float(peaks.get("hbm_gbs", 6650.0))
    per = bytes_per_row_position(c)
    achieved = per * B * T / (ms * 1e-3) / 1e9
    total_ms = sum(prof.ms.values()) or 1.0
    kernels = {k: {"launches_per_step": n, "us_per_launch": round(1e3 * prof.ms[k] / n, 3),
                   "share": round(prof.ms[k] / total_ms, 4)} for k, n in prof.launches.items() if n}  # fmt: skip
    line = {
        "metric": "window row-positions/s " + ("fwd" if forward_only else "fwd+bwd"), "value": B * T / (ms * 1e-3),
        "unit": "row-positions/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 products, f32 state",
        "data": "synthetic (drawn on the device)",
        "config": {"workload": WORKLOADS[name], "rows_per_gpu": B, "positions": T,
                   "kernels": "batch-synchronous phases" if args.phases else "library's choice",
                   "l2": "state and inputs larger than L2"},
        "e2e": None, "gpu_launches": args.steps * sum(prof.launches.values()),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": "measured" if peaks else "fallback",
                     "bytes_per_row_position": per, "kernels": kernels},
        "clocks": clocks_summary(lines, 0),
    }  # fmt: skip
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2", choices=sorted(CONFIGS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--phases", action="store_true",
                    help="run the batch-synchronous phase kernels instead of the per-row cluster kernels")
    ap.add_argument("--positions", type=int, default=0,
                    help="shorten the window to this many positions (profiler captures only; not a benchmark number)")
    args = ap.parse_args()
    c = dict(CONFIGS[args.config])
    if args.positions > 0:
        c["T"] = args.positions
    if args.impl == "reference":
        run_reference(args, c, args.config)
        return
    if c.get("resident"):
        run_resident(args, c, args.config)
        return

    import torch
    import torch.distributed as dist

    from hsn_b200.window import WindowModel, launch_profile, window_backward, window_forward

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the window path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)
    B, T, N, d, K = c["B"], c["T"], c["N"], c["d"], c["K"]
    W, host = synthetic(c, rank, B)
    model = WindowModel.from_weights(W, device=dev, prod=c["prod"], row_clusters=not args.phases)
    pinned = [torch.from_numpy(a).pin_memory() for a in host]
    z, ctx, scalars, reset, pre, post, sel = (t.to(dev, non_blocking=True) for t in pinned)
    state = (torch.zeros((B, N, d), device=dev), torch.zeros((B, d), device=dev),
             torch.zeros((B, N), dtype=torch.int64, device=dev), torch.zeros(B, dtype=torch.int64, device=dev))  # fmt: skip
    n_params = sum(int(np.prod(getattr(W, k).shape)) for k in
                   "s_w1 s_b1 s_w2 s_b2 p_w1 p_b1 p_w2 p_b2 score_w score_b v_w wout_w gate_w gate_b norm_w cand_w w1 b1 w2 b2".split())  # fmt: skip
    grads = torch.zeros(n_params, device=dev)
    out: dict = {}
    bw_scratch = torch.empty(64 << 20, dtype=torch.uint8, device=dev)

    def step(zz, cc, ss, rr, cots):
        tape = window_forward(model, zz, cc, ss, rr, state, out=out)
        rec = {k: tape["rec_" + k] for k in ("y", "hidden", "gate_pre", "m", "rms")}
        dc, db, carry = window_backward(
            model, tape["rec_c"], tape["rec_b"], tape["rec_h_old"], tape["sel_cell_idx"], tape["sel_unit_idx"],
            tape["sel_valid"], rr, cots[0], cots[1], cots[2], rec, scratch=bw_scratch,
        )  # fmt: skip
        if world > 1:  # the training-gradient exchange after each window backward
            dist.all_reduce(grads)
        return tape, dc, db, carry

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step(z, ctx, scalars, reset, (pre, post, sel))
    barrier()
    stop, lines = threading.Event(), []
    sampler = threading.Thread(target=sample_clocks, args=(stop, lines), daemon=True)
    sampler.start()
    time.sleep(0.3)
    # device-resident steps
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step(z, ctx, scalars, reset, (pre, post, sel))
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    # end to end: host buffers in, results back to the host, every step
    host_out = {k: torch.empty(s, dtype=t).pin_memory() for k, (s, t) in
                {"dc": ((B, T, K, d), torch.float32), "db": ((B, T, K, d), torch.float32),
                 "h": ((B, N, d), torch.float32), "q": ((B, d), torch.float32)}.items()}  # fmt: skip
    # Two staging sets: step i + 1's inputs cross the bus on a copy stream while step i computes (what a
    # data loader does); every step's host-to-device copy and read-back is inside the timed region.
    staged = [[torch.empty_like(t, device=dev) for t in pinned] for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream(dev)
    landed = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def upload(i):
        buf = i & 1
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[buf])   # the step that last read this set is done with it
            for dst, src in zip(staged[buf], pinned):
                dst.copy_(src, non_blocking=True)
            landed[buf].record(copy_stream)

    readback = torch.cuda.Stream(device=dev)
    computed = torch.cuda.Event()

    def e2e_step(i):
        buf = i & 1
        upload(i + 1)
        main_stream.wait_event(landed[buf])
        st = staged[buf]
        tape, dc, db, _ = step(st[0], st[1], st[2], st[3], st[4:7])
        consumed[buf].record(main_stream)
        # the final state lives in the tape's static buffer, which the next step rewrites: read it back
        # in order; the gradients are this step's own tensors and cross the bus beside the next step
        host_out["h"].copy_(tape["h"], non_blocking=True)
        host_out["q"].copy_(tape["q"], non_blocking=True)
        computed.record(main_stream)
        with torch.cuda.stream(readback):
            readback.wait_event(computed)
            host_out["dc"].copy_(dc, non_blocking=True)
            host_out["db"].copy_(db, non_blocking=True)
        dc.record_stream(readback)
        db.record_stream(readback)

    for ev in consumed:
        ev.record(main_stream)
    upload(0)
    e2e_step(0)   # untimed: fills the pipeline
    barrier()
    e0.record()
    for i in range(1, args.steps + 1):
        e2e_step(i)
    main_stream.wait_stream(readback)   # the last step's read-back ends before the closing event
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1) / args.steps
    stop.set()
    sampler.join(timeout=2)
    # one more step, untimed, with an event before every launch: the per-kernel times and counts
    with launch_profile() as prof:
        step(z, ctx, scalars, reset, (pre, post, sel))
    barrier()
    times = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, ms_e2e = (float(x) for x in times.cpu())
    if rank == 0:
        peaks_file = ROOT / "MEASURED_PEAKS.json"
        peaks = json.loads(peaks_file.read_text()) if peaks_file.exists() else {}
        peak = float(peaks.get("hbm_gbs", 6650.0))
        row_pos = B * T
        per = bytes_per_row_position(c)
        achieved = per * row_pos / (ms * 1e-3) / 1e9
        # the step's kernels by measured time (the profiled step); the dominant one's roofline
        launches_per_step = sum(prof.launches.values())
        total_ms = sum(prof.ms.values()) or 1.0
        split = kernel_bytes_per_row_position(c)
        traffic = NCU_TRAFFIC_PER_LAUNCH.get(args.config, {}) if args.positions == 0 else {}
        kernels = {}
        for name, n in prof.launches.items():
            if n:
                us = 1e3 * prof.ms[name] / n
                alg = split.get(name, 0) * B
                kernels[name] = {"launches_per_step": n, "us_per_launch": round(us, 3),
                                 "share": round(prof.ms[name] / total_ms, 4), "algorithmic_bytes_per_launch": alg,
                                 "achieved_gbs": round(alg / (us * 1e-6) / 1e9, 3) if us > 0 else None,
                                 "traffic": traffic.get(name)}  # fmt: skip
        top = max(kernels, key=lambda k: kernels[k]["share"])
        roofline = {
            "bound": "hbm", "kernel": top, "achieved": kernels[top]["achieved_gbs"], "peak": peak, "unit": "GB/s",
            "frac": kernels[top]["achieved_gbs"] / peak, "traffic": kernels[top]["traffic"],
            "peak_source": "measured" if peaks else "fallback",
            "how": "algorithmic bytes of the kernel's launch / its mean event-to-event time in a profiled step",
            "step": {"achieved": achieved, "frac": achieved / peak, "bytes_per_row_position": per},
            "kernels": kernels,
        }  # fmt: skip
        h2d = sum(t.numel() * t.element_size() for t in pinned)
        d2h = sum(t.numel() * t.element_size() for t in host_out.values())
        line = {
            "metric": "window row-positions/s fwd+bwd", "value": world * row_pos / (ms * 1e-3),
            "unit": "row-positions/s", "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 products, f32 state" if c["prod"] == "bf16" else "f32", "data": "synthetic",
            "config": {"workload": WORKLOADS[args.config] + (f" [shortened to {T} positions]" if args.positions else ""),
                       "rows_per_gpu": B, "positions": T,
                       "kernels": "batch-synchronous phases" if args.phases else "per-row clusters",
                       "l2": "inputs larger than L2 (tape 0.5 GiB + scalars 75 MB per step)",
                       "allreduce_floats_per_step": n_params if world > 1 else 0},
            "e2e": {"value": world * row_pos / (ms_e2e * 1e-3), "unit": "row-positions/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "note": "the next step's inputs are uploaded on a copy stream while this step computes; the final state is read back on the compute stream, the gradients dc/db on a read-back stream beside the next step; every copy ends inside the timed region"},
            "gpu_launches": args.steps * launches_per_step,
            "roofline": roofline,
            "clocks": clocks_summary(lines, local),
        }  # fmt: skip
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(c, W, host)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
