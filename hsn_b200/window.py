"""The whole-window entry points on torch tensors: forward sweep, reverse sweep, streaming step.

Thin host code over the C ABI (``include/hsn_window_b200.h``): it validates tensors, allocates
outputs and scratch with torch's caching allocator, passes ``data_ptr()`` and the current stream,
and names the results as the reference does (the tape keys of
``python/hsn/train/compile.py:1196-1231``, the arguments of ``state_gradient_backward``,
``python/hsn/train/state_gradient.py:357-376``). No arithmetic happens here.
"""

from __future__ import annotations

import ctypes
import math
from collections.abc import Mapping
from dataclasses import dataclass
from typing import Any

import torch
from torch import Tensor

from . import _lib

__all__ = ["WindowModel", "WindowPrologue", "WindowDecoder", "window_forward", "window_backward", "window_prologue",
           "window_decode", "stream_step", "front_projection", "prepare"]  # fmt: skip

_WEIGHT_KEYS = (
    "s_w1 s_b1 s_w2 s_b2 p_w1 p_b1 p_w2 p_b2 score_w score_b v_w wout_w gate_w gate_b norm_w cand_w "
    "w1 b1 w2 b2 pad_src edge_w cost"
).split()
#: The weights a matrix product reads: rounded to bfloat16 once per window in the bf16 mode.
_PRODUCT_KEYS = (
    "s_w1 s_b1 s_w2 s_b2 p_w1 p_b1 p_w2 p_b2 score_w score_b v_w wout_w gate_w gate_b w1 b1 w2 b2"
).split()


def prepare(device: int | torch.device = 0) -> None:
    """Make the library ready on ``device`` (idempotent). Fails loudly without the library."""
    index = device.index or 0 if isinstance(device, torch.device) else int(device)
    _lib.check(_lib.library().hsnw_prepare(index))


def _stream(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _ptr(t: Tensor | None) -> ctypes.c_void_p | None:
    return None if t is None else ctypes.c_void_p(t.data_ptr())


@dataclass
class WindowModel:
    """A window's weights on the device in the kernels' layouts (``HsnwModel``).

    ``weights`` holds torch-layout tensors or arrays under the names of the reference's modules:
    ``s_*`` = ``shared`` and ``p_*`` = ``predictor`` (``fc1``/``fc2`` weight and bias,
    ``python/hsn/model/encoder.py``), ``score_w/score_b`` = the linear scorer
    (``python/hsn/model/router.py:319-321``), ``v_w``, ``wout_w``, ``gate_w/gate_b``, ``norm_w``,
    ``cand_w`` = the cell (``python/hsn/model/cell.py:192-212``), ``w1 b1 w2 b2`` = the unit bank,
    ``pad_src`` / ``edge_w`` = the padded cell graph with the window's edge weights, ``cost`` = the
    router's cost table. ``prod="bf16"`` rounds the products' weights to bfloat16 here, once, as
    the reference's sweep twin does per window (``python/hsn/train/compile.py:776-840``), and packs
    the unit bank as bf16 operand tiles for the tcgen05 kernels (``tensor_cores=False`` keeps the
    CUDA-core kernels with the same roundings: a cross-check for the tests).
    """

    struct: _lib.HsnwModel
    tensors: dict[str, Tensor]
    device: torch.device
    dims: dict[str, int]
    prod: str

    @staticmethod
    def build(
        weights: Mapping[str, Any],
        *,
        k: int,
        device: torch.device | str = "cuda",
        prod: str = "fp32",
        age_max: int = 64,
        probes: bool = True,
        lambda_cost: float = 0.0,
        cell_overhead: float = 0.0,
        shared_cost: float = 0.0,
        limit: float = 1.00001,
        norm_eps: float = 1e-6,
        cand_eps: float = 1e-6,
        tensor_cores: bool = True,
        row_clusters: bool = True,
    ) -> "WindowModel":
        if prod not in ("fp32", "bf16"):
            raise ValueError(f"prod must be 'fp32' or 'bf16', got {prod!r}")
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("the window kernels run on a CUDA device only (no CPU path)")
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        missing = [key for key in _WEIGHT_KEYS if key not in weights]
        if missing:
            raise KeyError(f"window weights missing: {missing}")
        w: dict[str, Tensor] = {}
        for key in _WEIGHT_KEYS:
            t = torch.as_tensor(weights[key]).detach()
            if key == "pad_src":
                w[key] = t.to(device=device, dtype=torch.int32).contiguous()
                continue
            t = t.to(device=device, dtype=torch.float32)
            if prod == "bf16" and key in _PRODUCT_KEYS:
                t = t.to(torch.bfloat16).to(torch.float32)
            w[key] = t.contiguous()
        M, in4, H = (int(n) for n in w["w1"].shape)
        d = in4 // 4
        N, D = (int(n) for n in w["pad_src"].shape)
        dc = int(w["s_w1"].shape[1]) - 2 * d
        S = int(w["score_w"].shape[1]) - 3 * d - 1
        if in4 != 4 * d or dc < 0 or S < 0 or tuple(w["w2"].shape) != (M, H, d):
            raise ValueError("window weights have inconsistent shapes")
        s_w1 = w["s_w1"]
        packed = {
            "s_w1zc_t": torch.cat([s_w1[:, :d], s_w1[:, 2 * d :]], dim=1).t().contiguous(),
            "f_w1q_t": torch.cat([s_w1[:, d : 2 * d].t(), w["p_w1"].t()], dim=1).contiguous(),
            "f_b1": torch.cat([w["s_b1"], w["p_b1"]]).contiguous(),
            "f_w2_t": torch.cat([w["s_w2"].t(), w["p_w2"].t()], dim=0).contiguous(),
            "f_b2": torch.cat([w["s_b2"], w["p_b2"]]).contiguous(),
            "score_w_t": w["score_w"].t().contiguous(),
            "score_b": w["score_b"],
            "v_t": w["v_w"].t().contiguous(),
            "wout_t": w["wout_w"].t().contiguous(),
            "gate_t": w["gate_w"].t().contiguous(),
            "gate_b": w["gate_b"],
            "norm_w": w["norm_w"],
            "cand_w": w["cand_w"],
            "w1": w["w1"],
            "b1": w["b1"],
            "w2": w["w2"],
            "b2": w["b2"],
            "pad_src": w["pad_src"],
            "edge_w": w["edge_w"],
            "cost": w["cost"],
        }
        if prod == "bf16" and tensor_cores:
            packed.update(_umma_images(w["w1"], w["w2"], packed["gate_t"]))
        if prod == "bf16" and row_clusters and H % 128 == 0 and d % 8 == 0:
            packed.update(_row_images(w["w1"], w["w2"], packed["f_w1q_t"], packed["f_w2_t"]))
        struct = _lib.HsnwModel()
        dims = dict(N=N, d=d, K=int(k), H=H, M=M, D=D, S=S, dc=dc)
        for name, value in dims.items():
            setattr(struct, name, value)
        struct.prod_bf16 = int(prod == "bf16")
        struct.phases_only = int(not row_clusters)
        struct.probes = int(bool(probes))
        struct.age_max = int(min(age_max, 2**31 - 1))
        struct.lambda_cost, struct.cell_overhead = float(lambda_cost), float(cell_overhead)
        struct.shared_cost, struct.limit = float(shared_cost), float(limit)
        struct.norm_eps, struct.cand_eps = float(norm_eps), float(cand_eps)
        for name in _lib.MODEL_POINTERS:
            if name in packed:
                setattr(struct, name, packed[name].data_ptr())
        prepare(device)
        return WindowModel(struct=struct, tensors=packed, device=device, dims=dims, prod=prod)

    @staticmethod
    def from_oracle_weights(W: Any, *, device: torch.device | str = "cuda", prod: str = "fp32",
                            tensor_cores: bool = True, row_clusters: bool = True) -> "WindowModel":
        """From an object with the weights as attributes and the router's scalars (the fixtures'
        ``WindowWeights``): a convenience of the tests and the benchmark."""
        weights = {key: getattr(W, key) for key in _WEIGHT_KEYS}
        return WindowModel.build(
            weights, k=W.k, device=device, prod=prod, age_max=W.age_max, probes=W.probes,
            lambda_cost=W.lambda_cost, cell_overhead=W.cell_overhead, shared_cost=W.shared_cost,
            limit=W.limit, norm_eps=W.norm_eps, cand_eps=W.cand_eps, tensor_cores=tensor_cores,
            row_clusters=row_clusters,
        )  # fmt: skip

    from_weights = from_oracle_weights

    @staticmethod
    def from_hsn(model: Any, *, prod: str = "fp32", probes: bool = True) -> "WindowModel":
        """From a reference ``HSN`` module (``python/hsn/model/hsn.py``), inside or outside its
        ``cell.window()``: reads the modules' parameters and the graph's padded edge weights."""
        cell, router, scorer = model.cell, model.router, model.scorer
        with cell.window():
            edge_w = cell.graph._padded_weights().detach().clone()
        weights = {
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
        device = next(model.parameters()).device
        return WindowModel.build(
            weights, k=int(model.cfg.k_select), device=device, prod=prod, age_max=int(router.age_max),
            probes=probes, lambda_cost=float(router.lambda_cost),
            cell_overhead=float(router.cell_overhead), shared_cost=float(router.shared_cost),
            limit=float(model.cfg.budget) * (1.0 + 1e-5), norm_eps=float(cell.norm.eps),
            cand_eps=float(cell.cand_norm.eps),
        )  # fmt: skip


def synthetic_weights(rng: Any, *, N: int, d: int, K: int, H: int, M: int, D: int, S: int = 9,
                      dc: int | None = None, std: float = 0.02, age_max: int = 1 << 30) -> Any:  # fmt: skip
    """Seeded N(0, ``std``) weights of the reference's shapes for a benchmark or a demonstration
    (biases zero, the gate's bias -3, gains one, a ring-like padded graph with softmax edge weights):
    an object with one numpy array per weight under the names :meth:`WindowModel.from_weights`
    reads (``nn.Linear`` layouts, ``[out, in]``) and the router's scalars. ``rng`` is a
    ``numpy.random.Generator``."""
    import types

    import numpy as np

    dc = d if dc is None else dc
    f32 = np.float32

    def w(*shape: int) -> Any:
        return (rng.standard_normal(shape) * std).astype(f32)

    src = np.stack([(np.arange(N) + 1 + e * 7) % N for e in range(D)], axis=1).astype(np.int64)
    logit = rng.standard_normal((N, D))
    edge = np.exp(logit) / np.exp(logit).sum(axis=1, keepdims=True)
    return types.SimpleNamespace(
        s_w1=w(H, 2 * d + dc), s_b1=np.zeros(H, f32), s_w2=w(d, H), s_b2=np.zeros(d, f32),
        p_w1=w(H, d), p_b1=np.zeros(H, f32), p_w2=w(d, H), p_b2=np.zeros(d, f32),
        score_w=w(M, 3 * d + 1 + S), score_b=np.zeros(M, f32),
        v_w=w(d, d), wout_w=w(d, d), gate_w=w(d, 4 * d), gate_b=np.full(d, -3.0, f32),
        norm_w=np.ones(4 * d, f32), cand_w=np.ones(d, f32),
        w1=w(M, 4 * d, H), b1=np.zeros((M, H), f32), w2=w(M, H, d), b2=np.zeros((M, d), f32),
        pad_src=src, edge_w=edge.astype(f32), cost=np.full(M, 1.0 / (8 * N), f32),
        age_max=age_max, lambda_cost=0.0, cell_overhead=0.0, shared_cost=0.0, limit=1.00001,
        norm_eps=1e-6, cand_eps=1e-6, k=K, probes=True,
    )  # fmt: skip


def _sw128(tile: Tensor) -> Tensor:
    """``[..., rows, 64]`` bf16 (one 128-byte row per row of a K-block of 64) in the tensor cores'
    128-byte swizzle: the 16-byte unit ``u`` of row ``r`` is stored at unit ``u ^ (r % 8)``."""
    *lead, rows, k = tile.shape
    assert k == 64
    units = tile.reshape(*lead, rows, 8, 8)
    r = torch.arange(rows, device=tile.device) % 8
    u = torch.arange(8, device=tile.device)
    src = (u[None, :] ^ r[:, None])  # the unit stored at position p of row r is unit p ^ (r % 8)
    idx = src.view(*([1] * len(lead)), rows, 8, 1).expand(*lead, rows, 8, 8)
    return torch.gather(units, -2, idx).reshape(*lead, rows, 64)


def _row_images(w1: Tensor, w2: Tensor, f_w1q_t: Tensor, f_w2_t: Tensor) -> dict[str, Tensor]:
    """bf16 images for the per-row cluster kernels (``hsn_b200/csrc/window_rows.cu``,
    ``window_rows_bwd.cu``) and per block of the cluster its 256 columns of the merged front first
    layer ``[d][256]`` followed by the same columns' rows of the second layer ``[256][d]``. Forward
    (``rows_bank``): per unit and block of 128 hidden columns three K-major tensor-core tiles, ``W1``'s
    rows of the inputs ``[0, 2d)``, of ``[2d, 4d)`` (each ``[128 columns][2d]``) and ``W2`` (``[d
    outputs][128 columns]``). Reverse (``rows_bank_bw``): per unit and block of 128 columns ``W2`` as
    ``[128 columns][d]`` then the state rows of ``W1`` as ``[2d][128 columns]``. ``d == 64``: 128-byte
    swizzled K-blocks of 64. Other ``d``: the unswizzled core-matrix layout ``[K/8][rows][8]`` of
    ``umma.cuh``."""
    M, in4, H = (int(n) for n in w1.shape)
    d = int(w2.shape[2])
    bf = torch.bfloat16
    C = H // 128
    if d == 64:
        # forward: per unit and block of 128 columns, W1 as four K-blocks [128 columns][64 inputs] (two pieces of
        # two), then W2 as two K-blocks [d outputs][64 columns]
        a = w1.reshape(M, in4 // 64, 64, C, 128).permute(0, 3, 1, 4, 2).to(bf)  # [M, C, K-block, column, input]
        a = _sw128(a).reshape(M, C, -1)
        b = w2.reshape(M, C, 2, 64, d).permute(0, 1, 2, 4, 3).to(bf)  # [M, C, K-block, output, column]
        b = _sw128(b).reshape(M, C, -1)
        # reverse: per unit and block of 128 columns, W2 as [128 columns][d outputs], then the state rows of W1 as
        # two K-blocks [2d state inputs][64 columns]
        ba = _sw128(w2.reshape(M, C, 128, d).to(bf)).reshape(M, C, -1)  # [M, C, column, output]
        bb = w1[:, 2 * d :, :].reshape(M, 2 * d, C, 2, 64).permute(0, 2, 3, 1, 4).to(bf)  # [M, C, K-block, state input, column]
        bb = _sw128(bb).reshape(M, C, -1)
    else:
        a = w1.reshape(M, in4 // 8, 8, C, 128).permute(0, 3, 1, 4, 2).to(bf).reshape(M, C, -1)  # [M,C,(4d/8)*128*8]
        b = w2.reshape(M, C, 16, 8, d).permute(0, 1, 2, 4, 3).to(bf).reshape(M, C, -1)  # [M,C,16*d*8]
        ba = w2.reshape(M, C, 128, d // 8, 8).permute(0, 1, 3, 2, 4).to(bf).reshape(M, C, -1)  # [M,C,(d/8)*128*8]
        bb = w1[:, 2 * d :, :].reshape(M, 2 * d, C, 16, 8).permute(0, 2, 3, 1, 4).to(bf).reshape(M, C, -1)  # [M,C,16*2d*8]
    bank = torch.cat([a, b], dim=2).contiguous()
    bank_bw = torch.cat([ba, bb], dim=2).contiguous()
    f1 = f_w1q_t.reshape(d, C, 256).permute(1, 0, 2).to(bf).reshape(C, -1)  # [C, d*256]
    f2 = f_w2_t.reshape(C, 256, d).to(bf).reshape(C, -1)  # [C, 256*d]
    front = torch.stack([f1, f2], dim=1).contiguous()  # [C, 2, 256 d]
    return {"rows_bank": bank, "rows_front": front, "rows_bank_bw": bank_bw}


def _umma_images(w1: Tensor, w2: Tensor, gate_t: Tensor) -> dict[str, Tensor]:
    """The unit bank as bf16 operand tiles for the tensor cores: 128-row tiles in the K-major
    core-matrix layout ``[K/8][128][8]`` of ``hsn_b200/csrc/umma.cuh``, zero padded."""
    M, in4, H = (int(n) for n in w1.shape)
    d = int(w2.shape[2])
    nB = (H + 127) // 128
    pad_h = nB * 128 - H
    bf = torch.bfloat16
    a1 = torch.nn.functional.pad(w1, (0, pad_h))  # [M, 4d, nB*128]
    a1 = a1.reshape(M, in4 // 8, 8, nB, 128).permute(0, 3, 1, 4, 2).to(bf).contiguous()
    g = torch.nn.functional.pad(gate_t, (0, 128 - d))  # [4d, 128]
    g = g.reshape(in4 // 8, 8, 128).permute(0, 2, 1).to(bf).contiguous()
    a2 = torch.nn.functional.pad(w2, (0, 128 - d, 0, pad_h))  # [M, nB*128, 128]
    a2 = a2.reshape(M, nB, 16, 8, 128).permute(0, 1, 2, 4, 3).to(bf).contiguous()
    out = {"umma_w1": a1, "umma_gate": g, "umma_w2": a2}
    if d % 16 == 0 and d <= 128:
        # the reverse sweep's transposed products
        nT = (2 * d + 127) // 128
        pad_i = nT * 128 - 2 * d
        b2 = torch.nn.functional.pad(w2, (0, 0, 0, pad_h))  # [M, nB*128, d]
        b2 = b2.reshape(M, nB, 128, d // 8, 8).permute(0, 1, 3, 2, 4).to(bf).contiguous()
        b1 = torch.nn.functional.pad(w1[:, 2 * d :, :], (0, pad_h, 0, pad_i))  # [M, nT*128, nB*128]
        b1 = b1.reshape(M, nT, 128, nB, 16, 8).permute(0, 3, 1, 4, 2, 5).to(bf).contiguous()
        bg = torch.nn.functional.pad(gate_t[2 * d :, :], (0, 0, 0, pad_i))  # [nT*128, d]
        bg = bg.reshape(nT, 128, d // 8, 8).permute(0, 2, 1, 3).to(bf).contiguous()
        out.update(umma_bw_w2=b2, umma_bw_w1=b1, umma_bw_gate=bg)
    return out


def _check(name: str, t: Tensor, shape: tuple[int, ...], dtype: torch.dtype, device: torch.device,
           in_place: bool = False) -> Tensor:  # fmt: skip
    """``t`` if it is what the kernels take. A read-only tensor that is not contiguous is copied; one the
    kernels update in place (``in_place``) must be contiguous already: a copy would take the update and
    leave the caller's tensor stale."""
    if t.device != device or t.dtype != dtype or tuple(t.shape) != shape:
        raise ValueError(
            f"{name} must be a {dtype} tensor of shape {shape} on {device}, got {t.dtype} "
            f"{tuple(t.shape)} on {t.device}"
        )
    if in_place and not t.is_contiguous():
        raise ValueError(f"{name} is updated in place and must be contiguous")
    return t.contiguous()


def window_forward(
    model: WindowModel,
    z: Tensor,
    ctx: Tensor,
    scalars: Tensor,
    reset: Tensor,
    state: tuple[Tensor, Tensor, Tensor, Tensor],
    *,
    record: bool = True,
    tape_state: bool = True,
    forced: tuple[Tensor, Tensor, Tensor] | None = None,
    want_logits: bool = False,
    want_us: bool = False,
    scratch: Tensor | None = None,
    out: dict[str, Tensor] | None = None,
    carried: bool = False,
    _entry: str = "hsnw_window_forward",
) -> dict[str, Tensor]:
    """The forward sweep of one window (``hsnw_window_forward``): the reference's tape
    (``python/hsn/train/compile.py:1196-1213``) for ``z [B,T,d]``, ``ctx [B,T,dc]``, ``scalars
    [B,T,N,S]`` (the prologue's, ``python/hsn/model/hsn.py:1741-1830``), ``reset [B,T]`` bool and
    the carried ``state = (h, q, age, pos)``, which is not modified with ``tape_state`` (the final
    state is returned under ``h q age pos``). ``record`` adds ``rec_*``: the per-slot values the
    state-gradient sweep reads. ``forced = (cells, units, valid)`` replays a recorded decision.
    ``tape_state=False`` keeps no state tape and updates ``state`` in place (large ``N``).
    ``want_us`` adds ``us [B,T,d]``, the shared path's output ``u_t`` (with ``qs`` the decoder's input,
    :func:`window_decode`). ``out`` reuses the buffers of an earlier call's result (static addresses).
    ``carried`` (with ``tape_state=False`` and the previous call's result as ``out``, same ``B`` and
    ``T``): the next chunk of positions on the same resident state, ``hsnw_stream_continue``; the
    cells' derived values are taken from the previous call's scratch instead of being recomputed
    from the whole state."""
    if carried:
        if tape_state or out is None or "_scratch" not in out:
            raise ValueError("a carried call continues a resident state: tape_state=False and out=the previous result")
        _entry = "hsnw_stream_continue"
    dm = model.dims
    dev = model.device
    B, T = int(reset.shape[0]), int(reset.shape[1])
    N, d, K, H, M, S, dc = dm["N"], dm["d"], dm["K"], dm["H"], dm["M"], dm["S"], dm["dc"]
    f32, i64 = torch.float32, torch.int64
    z = _check("z", z, (B, T, d), f32, dev)
    ctx = _check("ctx", ctx, (B, T, dc), f32, dev)
    scalars = _check("scalars", scalars, (B, T, N, S), f32, dev)
    reset_u8 = _check("reset", reset, (B, T), torch.bool, dev).view(torch.uint8)
    resident = not tape_state
    h0 = _check("state.h", state[0], (B, N, d), f32, dev, in_place=resident)
    q0 = _check("state.q", state[1], (B, d), f32, dev, in_place=resident)
    age0 = _check("state.age", state[2], (B, N), i64, dev, in_place=resident)
    pos = _check("state.pos", state[3], (B,), i64, dev, in_place=resident)
    if tape_state:
        pos = pos.clone()
    lib = _lib.library()
    o = out if out is not None else {}

    def buf(name: str, shape: tuple[int, ...], dtype: torch.dtype) -> Tensor:
        # a buffer of an earlier call is reused only if it is exactly what this call writes: the kernels
        # take sizes from the call, not from the buffer
        have = o.get(name)
        if have is not None and (tuple(have.shape) != shape or have.dtype != dtype or have.device != dev
                                 or not have.is_contiguous()):  # fmt: skip
            if carried:
                raise ValueError(
                    f"out[{name!r}] is {have.dtype} {tuple(have.shape)}; a carried call needs the previous "
                    f"call's buffers of the same B and T ({dtype} {shape})"
                )
            have = None
        if have is None:
            o[name] = have = torch.empty(shape, dtype=dtype, device=dev)
        return have

    io = _lib.HsnwForward()
    io.B, io.T, io.tape_state, io.forced = B, T, int(tape_state), int(forced is not None)
    io.z, io.ctx, io.scalars, io.reset = z.data_ptr(), ctx.data_ptr(), scalars.data_ptr(), reset_u8.data_ptr()
    io.h0, io.q0, io.age0, io.pos = h0.data_ptr(), q0.data_ptr(), age0.data_ptr(), pos.data_ptr()
    if tape_state:
        io.tape_h = buf("_tape_h", (B, T + 1, N, d), f32).data_ptr()
        io.tape_q = buf("_tape_q", (B, T + 1, d), f32).data_ptr()
        io.tape_age = buf("_tape_age", (B, T + 1, N), i64).data_ptr()
    cells = buf("sel_cell_idx", (B, T, K), i64)
    units = buf("sel_unit_idx", (B, T, K), i64)
    valid = buf("sel_valid", (B, T, K), torch.bool)
    if forced is not None:
        cells.copy_(_check("forced cells", forced[0], (B, T, K), i64, dev))
        units.copy_(_check("forced units", forced[1], (B, T, K), i64, dev))
        valid.copy_(_check("forced valid", forced[2], (B, T, K), torch.bool, dev))
    io.cells, io.units, io.valid = cells.data_ptr(), units.data_ptr(), valid.data_ptr()
    io.refreshed = buf("sel_refreshed", (B, T, K), torch.bool).data_ptr()
    io.theta = buf("tape_theta", (B, T), f32).data_ptr()
    io.h_sel = buf("tape_hsel", (B, T, K, d), f32).data_ptr()
    io.qs = buf("qs", (B, T, d), f32).data_ptr()
    if tape_state:
        io.h_max = buf("h_max", (B, T), f32).data_ptr()
    if record:
        for name in ("c", "b", "h_old", "y", "gate_pre", "m"):
            setattr(io, "rec_" + name, buf("rec_" + name, (B, T, K, d), f32).data_ptr())
        io.rec_rms = buf("rec_rms", (B, T, K), f32).data_ptr()
        # (bfloat16 with bf16 products: the values are bfloat16, and the reference's record holds them so)
        io.rec_hidden = buf("rec_hidden", (B, T, K, H), torch.bfloat16 if model.prod == "bf16" else f32).data_ptr()
    if want_logits:
        io.logits = buf("logits", (B, T, N, M), f32).data_ptr()
    if want_us:
        io.us = buf("us", (B, T, d), f32).data_ptr()
    need = int(lib.hsnw_forward_scratch_bytes(ctypes.byref(model.struct), B, T))
    if scratch is None:
        scratch = buf("_scratch", (need,), torch.uint8)
    if scratch.numel() < need or scratch.device != dev or scratch.dtype != torch.uint8 or not scratch.is_contiguous():
        raise ValueError(f"scratch must be a contiguous uint8 tensor of at least {need} bytes on {dev}")
    io.scratch, io.scratch_bytes = scratch.data_ptr(), scratch.numel()
    with torch.cuda.device(dev):
        _lib.check(getattr(lib, _entry)(ctypes.byref(model.struct), ctypes.byref(io), _stream(dev)))
    if tape_state:
        o["tape_h"], o["tape_q"], o["tape_age"] = o["_tape_h"][:, :T], o["_tape_q"][:, :T], o["_tape_age"][:, :T]
        o["h"], o["q"], o["age"] = o["_tape_h"][:, T], o["_tape_q"][:, T], o["_tape_age"][:, T]
        o["state_abs_max"] = o["h_max"].amax(dim=0)
    else:
        o["h"], o["q"], o["age"] = h0, q0, age0
    o["pos"] = pos
    o["status"] = scratch[:4].view(torch.int32)  # 0, or 1 when a bounded device-side wait ran out
    o["path"] = lib.hsnw_last_path().decode()  # "rows": the per-row cluster kernel ran; "phases": the batch-synchronous kernels
    if forced is None:
        o["refreshed"] = o["sel_refreshed"].float().sum(dim=2).mean(dim=0)
    o["explored"] = torch.zeros(T, dtype=f32, device=dev)
    return o


def stream_step(
    model: WindowModel,
    z_t: Tensor,
    ctx_t: Tensor,
    scalars_t: Tensor,
    reset_t: Tensor,
    state: tuple[Tensor, Tensor, Tensor, Tensor],
    *,
    out: dict[str, Tensor] | None = None,
    carried: bool = False,
    want_us: bool = False,
) -> dict[str, Tensor]:
    """One position on a resident state, updated in place (``hsnw_stream_step``): the serving
    step's state update (``python/hsn/train/compile.py:1913-2006``). ``z_t [B,d]``, ``ctx_t
    [B,dc]``, ``scalars_t [B,N,S]``, ``reset_t [B]`` bool. Returns the decision and the slots'
    states (``sel_*``, ``tape_hsel``, ``qs``) of the position; with ``want_us`` also ``us``, so that
    ``window_decode(decoder, step["qs"][:, 0], step["us"][:, 0])`` are the step's logits ``[B, V]``.

    ``carried`` (``hsnw_stream_continue``): ``out`` is the result of the previous step on this
    state (it holds the scratch with every cell's derived values), the weights are the same and
    the state was not touched in between; the step then skips the pass over the whole state that
    recomputes them."""
    if carried and (out is None or "_scratch" not in out):
        raise ValueError("a carried step needs the previous step's result as `out`")
    return window_forward(
        model, z_t[:, None], ctx_t[:, None], scalars_t[:, None], reset_t[:, None], state,
        record=False, tape_state=False, out=out, want_us=want_us,
        _entry="hsnw_stream_continue" if carried else "hsnw_stream_step",
    )  # fmt: skip


def window_backward(
    model: WindowModel,
    c: Tensor,
    b: Tensor,
    h_old: Tensor,
    cells: Tensor,
    units: Tensor | None,
    valid: Tensor,
    reset: Tensor,
    d_q_pre: Tensor | None,
    d_q_post: Tensor | None,
    d_h_sel: Tensor | None,
    record: Mapping[str, Tensor] | None,
    *,
    initial: tuple[Tensor, Tensor] | None = None,
    full_cut: bool = False,
    scratch: Tensor | None = None,
    info: dict[str, Any] | None = None,
) -> tuple[Tensor, Tensor, tuple[Tensor, Tensor]]:
    """The reverse sweep of one window (``hsnw_window_backward``): ``(dc, db, (A, R))``.

    The arguments are ``state_gradient_backward``'s (``python/hsn/train/state_gradient.py:357-376``;
    ``record`` holds ``y gate_pre m rms hidden``; ``hidden`` is bfloat16 with bf16 products, as the
    forward sweep records it, and a float32 one is converted), or with ``full_cut`` ``recurrence_backward``'s
    (``python/hsn/train/split.py:128-139``; ``units`` and ``record`` unused). ``initial`` is the
    cotangent of the state after the last position (the next window's returned ``(A, R)``); the
    returned ``(A, R)`` is the cotangent of the state this window started from. ``info``, a dict,
    receives ``status`` (an int32 tensor of one element on the device: 0, or 1 when a bounded
    device-side wait ran out and the results are not to be trusted) and ``path`` (``"rows"`` or
    ``"phases"``: the kernels that served the call)."""
    dm = model.dims
    dev = model.device
    B, T, K, d = (int(n) for n in c.shape)
    N, H = dm["N"], dm["H"]
    f32, i64 = torch.float32, torch.int64
    if K != dm["K"] or d != dm["d"]:
        raise ValueError(f"c must be [B, T, {dm['K']}, {dm['d']}], got {tuple(c.shape)}")
    io = _lib.HsnwBackward()
    io.B, io.T, io.full_cut = B, T, int(full_cut)
    keep: list[Tensor] = []

    def put(field: str, t: Tensor | None, shape: tuple[int, ...], dtype: torch.dtype) -> None:
        if t is None:
            return
        t = _check(field, t, shape, dtype, dev)
        keep.append(t)
        setattr(io, field, t.data_ptr())

    put("c", c, (B, T, K, d), f32)
    put("b", b, (B, T, K, d), f32)
    put("h_old", h_old, (B, T, K, d), f32)
    put("cells", cells, (B, T, K), i64)
    valid_u8 = _check("valid", valid, (B, T, K), torch.bool, dev).view(torch.uint8)
    reset_u8 = _check("reset", reset, (B, T), torch.bool, dev).view(torch.uint8)
    io.valid, io.reset = valid_u8.data_ptr(), reset_u8.data_ptr()
    put("d_q_pre", d_q_pre, (B, T, d), f32)
    put("d_q_post", d_q_post, (B, T, d), f32)
    put("d_h_sel", d_h_sel, (B, T, K, d), f32)
    if not full_cut:
        if record is None or units is None:
            raise ValueError("the state-gradient sweep needs units and the round's record")
        put("units", units, (B, T, K), i64)
        put("y", record["y"], (B, T, K, d), f32)
        put("gate_pre", record["gate_pre"], (B, T, K, d), f32)
        put("m", record["m"], (B, T, K, d), f32)
        put("rms", record["rms"], (B, T, K), f32)
        hidden_dtype = torch.bfloat16 if model.prod == "bf16" else f32
        hidden = record["hidden"]
        if hidden.dtype != hidden_dtype and hidden.dtype in (f32, torch.bfloat16):
            hidden = hidden.to(hidden_dtype)   # (exact for a record made with bf16 products)
        put("hidden", hidden, (B, T, K, H), hidden_dtype)
    dc = torch.empty((B, T, K, d), dtype=f32, device=dev)
    db = torch.empty((B, T, K, d), dtype=f32, device=dev)
    if initial is None:
        A = torch.zeros((B, N, d), dtype=f32, device=dev)
        R = torch.zeros((B, d), dtype=f32, device=dev)
    else:
        A = _check("initial A", initial[0], (B, N, d), f32, dev).clone()
        R = _check("initial R", initial[1], (B, d), f32, dev).clone()
    io.dc, io.db, io.A, io.R = dc.data_ptr(), db.data_ptr(), A.data_ptr(), R.data_ptr()
    lib = _lib.library()
    need = int(lib.hsnw_backward_scratch_bytes(ctypes.byref(model.struct), B, T))
    if scratch is None:
        scratch = torch.empty((max(need, 256),), dtype=torch.uint8, device=dev)
    if scratch.numel() < need or scratch.device != dev or scratch.dtype != torch.uint8 or not scratch.is_contiguous():
        raise ValueError(f"scratch must be a contiguous uint8 tensor of at least {need} bytes on {dev}")
    io.scratch, io.scratch_bytes = scratch.data_ptr(), scratch.numel()
    with torch.cuda.device(dev):
        _lib.check(lib.hsnw_window_backward(ctypes.byref(model.struct), ctypes.byref(io), _stream(dev)))
    if info is not None:
        info["status"] = scratch[:4].view(torch.int32)
        info["path"] = lib.hsnw_last_path().decode()
        info["_scratch"] = scratch
    return dc, db, (A, R)


_PROLOGUE_KEYS = ("byte_emb enc_w1 enc_b1 enc_w2 enc_b2 ctx_emb byte_codes cell_addresses ema_utility ema_selected").split()


@dataclass
class WindowPrologue:
    """The tables and numbers ``HSN._window_prologue`` reads (``python/hsn/model/hsn.py:1707-1860``), on
    the device: the byte embedding, the encoder ``E`` (``fc1``/``fc2`` in ``nn.Linear`` layout), the
    context embedding, the scorer's fixed byte codes and cell addresses (``model.key_address``), its two
    running averages, and ``budget``, ``round / r_max``, ``n_context``, ``unroll`` and the position
    rule (``python/hsn/model/router.py:727-765``)."""

    struct: _lib.HsnwPrologue
    tensors: dict[str, Tensor]
    device: torch.device

    @staticmethod
    def build(tables: Mapping[str, Any], *, device: torch.device | str = "cuda", prod: str = "fp32",
              budget_frac: float = 1.0, round_frac: float = 0.0, n_context: float = 16.0, unroll: float = 256.0,
              position: str = "document", bos: int = 1) -> "WindowPrologue":  # fmt: skip
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("the window kernels run on a CUDA device only (no CPU path)")
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        if position not in ("document", "clamp", "wrap") or prod not in ("fp32", "bf16"):
            raise ValueError("position must be document | clamp | wrap (model.scorer_position) and prod fp32 | bf16")
        t = {k: torch.as_tensor(tables[k]).detach().to(device=device, dtype=torch.float32).contiguous()
             for k in _PROLOGUE_KEYS if tables.get(k) is not None}  # fmt: skip
        for key in ("byte_emb", "enc_w1", "enc_b1", "enc_w2", "enc_b2", "ctx_emb", "ema_utility", "ema_selected"):
            if key not in t:
                raise KeyError(f"prologue tables missing: {key}")
        V, d = (int(n) for n in t["byte_emb"].shape)
        H = int(t["enc_w1"].shape[0])
        addressed = "byte_codes" in t and "cell_addresses" in t
        N = int(t["ema_utility"].shape[-1])
        if tuple(t["enc_w1"].shape) != (H, d) or tuple(t["enc_w2"].shape) != (d, H) or (addressed and tuple(t["cell_addresses"].shape) != (N, d)):
            raise ValueError("prologue tables have inconsistent shapes")
        st = _lib.HsnwPrologue()
        st.V, st.d, st.H, st.dc, st.N, st.S = V, d, H, int(t["ctx_emb"].shape[1]), N, 9 if addressed else 7
        st.prod_bf16 = int(prod == "bf16")
        st.position_mode = ("document", "clamp", "wrap").index(position)
        st.ema_per_row = int(t["ema_utility"].ndim == 2)
        st.bos = int(bos)
        st.budget_frac, st.round_frac, st.n_context, st.unroll = float(budget_frac), float(round_frac), float(n_context), float(unroll)
        for key, value in t.items():
            setattr(st, key, value.data_ptr())
        prepare(device)
        return WindowPrologue(struct=st, tensors=t, device=device)


def window_prologue(pro: WindowPrologue, tokens: Tensor, ctx_ids: Tensor, reset: Tensor, pos0: Tensor,
                    prev_tokens: Tensor | None = None, *, out: dict[str, Tensor] | None = None) -> dict[str, Tensor]:  # fmt: skip
    """``hsnw_window_prologue``: ``tokens``, ``ctx_ids`` ``[B, T]`` int64, ``reset [B, T]`` bool, ``pos0
    [B]`` int64 (the carried state's ``pos``) and optionally the byte before the window ``prev_tokens
    [B]`` to ``z [B,T,d]``, ``ctx [B,T,dc]``, ``scalars [B,T,N,S]`` and ``positions [B,T]``: the inputs
    of :func:`window_forward`. ``out`` reuses an earlier result's buffers."""
    dev = pro.device
    B, T = (int(n) for n in tokens.shape)
    i64, f32 = torch.int64, torch.float32
    st = pro.struct
    io = _lib.HsnwPrologue.from_buffer_copy(st)
    io.B, io.T = B, T
    tokens = _check("tokens", tokens, (B, T), i64, dev)
    ctx_ids = _check("ctx_ids", ctx_ids, (B, T), i64, dev)
    reset_u8 = _check("reset", reset, (B, T), torch.bool, dev).view(torch.uint8)
    pos0 = _check("pos0", pos0, (B,), i64, dev)
    if st.ema_per_row and int(pro.tensors["ema_utility"].shape[0]) != B:
        raise ValueError("the running averages are per row and do not have this window's rows")
    io.tokens, io.ctx_ids, io.reset, io.pos0 = tokens.data_ptr(), ctx_ids.data_ptr(), reset_u8.data_ptr(), pos0.data_ptr()
    if prev_tokens is not None:
        prev_tokens = _check("prev_tokens", prev_tokens, (B,), i64, dev)
        io.prev_tokens = prev_tokens.data_ptr()
    o = out if out is not None else {}

    def buf(name: str, shape: tuple[int, ...], dtype: torch.dtype) -> Tensor:
        have = o.get(name)
        if have is None or tuple(have.shape) != shape or have.dtype != dtype or have.device != dev:
            o[name] = have = torch.empty(shape, dtype=dtype, device=dev)
        return have

    io.z = buf("z", (B, T, st.d), f32).data_ptr()
    io.ctx = buf("ctx", (B, T, st.dc), f32).data_ptr()
    io.scalars = buf("scalars", (B, T, st.N, st.S), f32).data_ptr()
    io.positions = buf("positions", (B, T), i64).data_ptr()
    lib = _lib.library()
    need = int(lib.hsnw_prologue_scratch_bytes(ctypes.byref(io)))
    scratch = buf("_scratch", (need,), torch.uint8)
    io.scratch, io.scratch_bytes = scratch.data_ptr(), need
    with torch.cuda.device(dev):
        _lib.check(lib.hsnw_window_prologue(ctypes.byref(io), _stream(dev)))
    return o


def front_projection(model: WindowModel, z: Tensor, ctx: Tensor) -> Tensor:
    """The window-invariant half of the shared path's first layer for every position
    (``hsnw_front_projection``): ``[z; ctx] [R, d + dc] @ W + b -> [R, H]``, the part of
    ``shared.fc1`` (``python/hsn/model/encoder.py``) that does not read the carried summary. With
    bf16 products it runs as tcgen05 tensor-core tiles. ``window_forward`` calls it itself."""
    dm, dev = model.dims, model.device
    rows = int(z.shape[0])
    z = _check("z", z, (rows, dm["d"]), torch.float32, dev)
    ctx = _check("ctx", ctx, (rows, dm["dc"]), torch.float32, dev)
    out = torch.empty((rows, dm["H"]), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(
            _lib.library().hsnw_front_projection(
                ctypes.byref(model.struct), z.data_ptr(), ctx.data_ptr(), rows, out.data_ptr(), _stream(dev)
            )
        )
    return out


@dataclass
class WindowDecoder:
    """The decoder ``D`` (``python/hsn/model/encoder.py:175-182``: ``fc1 [H, 2d]``, ``fc2 [V, H]`` with biases, in
    ``nn.Linear`` layout) on the device; with ``prod="bf16"`` the weights are rounded to bfloat16 once here, as
    autocast rounds them at every use."""

    struct: _lib.HsnwDecoder
    tensors: dict[str, Tensor]
    device: torch.device

    @staticmethod
    def build(w1: Any, b1: Any, w2: Any, b2: Any, *, d_q: int, device: torch.device | str = "cuda",
              prod: str = "fp32") -> "WindowDecoder":  # fmt: skip
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("the window kernels run on a CUDA device only (no CPU path)")
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        if prod not in ("fp32", "bf16"):
            raise ValueError("prod must be fp32 | bf16")
        t = {k: torch.as_tensor(v).detach().to(device=device, dtype=torch.float32).contiguous()
             for k, v in (("w1", w1), ("b1", b1), ("w2", w2), ("b2", b2))}  # fmt: skip
        if prod == "bf16":
            t = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in t.items()}
        H, K = (int(n) for n in t["w1"].shape)
        V = int(t["w2"].shape[0])
        if tuple(t["w2"].shape) != (V, H) or tuple(t["b1"].shape) != (H,) or tuple(t["b2"].shape) != (V,) or not 0 < d_q <= K:
            raise ValueError("decoder weights have inconsistent shapes")
        st = _lib.HsnwDecoder()
        st.d_q, st.d_u, st.H, st.V, st.prod_bf16 = int(d_q), K - int(d_q), H, V, int(prod == "bf16")
        for key, value in t.items():
            setattr(st, key, value.data_ptr())
        prepare(device)
        return WindowDecoder(struct=st, tensors=t, device=device)


def window_decode(decoder: WindowDecoder, qs: Tensor, us: Tensor | None, *, out: dict[str, Tensor] | None = None) -> Tensor:
    """``hsnw_window_decode``: the logits ``D([q_t; u_t])`` for ``qs [..., d_q]`` and ``us [..., d_u]`` (the forward
    sweep's outputs of those names: ``window_forward(..., want_us=True)``), shape ``[..., V]``; the window's
    epilogue (``python/hsn/model/hsn.py:2004-2049``, ``:2374-2390``) without its diagnostics. ``out`` reuses an
    earlier call's buffers (``out["logits"]`` is the result)."""
    dev, st = decoder.device, decoder.struct
    lead = tuple(int(n) for n in qs.shape[:-1])
    rows = math.prod(lead)
    qs = _check("qs", qs, lead + (st.d_q,), torch.float32, dev)
    if st.d_u:
        if us is None:
            raise ValueError("this decoder reads [q; u]: us is missing")
        us = _check("us", us, lead + (st.d_u,), torch.float32, dev)
    o = out if out is not None else {}
    lib = _lib.library()
    need = int(lib.hsnw_decode_scratch_bytes(ctypes.byref(st), rows))

    def buf(name: str, shape: tuple[int, ...], dtype: torch.dtype) -> Tensor:
        have = o.get(name)
        if have is None or tuple(have.shape) != shape or have.dtype != dtype or have.device != dev:
            o[name] = have = torch.empty(shape, dtype=dtype, device=dev)
        return have

    logits = buf("logits", lead + (st.V,), torch.float32)
    scratch = buf("_decode_scratch", (need,), torch.uint8)
    with torch.cuda.device(dev):
        _lib.check(lib.hsnw_window_decode(ctypes.byref(st), qs.data_ptr(), us.data_ptr() if st.d_u else None, rows,
                                          logits.data_ptr(), scratch.data_ptr(), need, _stream(dev)))  # fmt: skip
    o["decode_status"] = scratch[:4].view(torch.int32)
    return logits


class launch_profile:
    """``with launch_profile() as prof: ...`` times every kernel launch of the window entry points
    made inside the block (``hsnw_profile_begin`` / ``hsnw_profile_end``): afterwards ``prof.ms``
    and ``prof.launches`` map a kernel kind ("rows_fwd", "rows_bwd", "pre", or the phases' "front",
    "row", "unit", "update", "head", "mid", "tail_head", "init") to its summed time in milliseconds and its launch count. For
    measurement runs: it adds an event per launch."""

    def __init__(self) -> None:
        self.ms: dict[str, float] = {}
        self.launches: dict[str, int] = {}

    def __enter__(self) -> "launch_profile":
        _lib.check(_lib.library().hsnw_profile_begin())
        return self

    def __exit__(self, *exc: object) -> None:
        lib = _lib.library()
        kinds = int(lib.hsnw_profile_kinds())
        ms = (ctypes.c_double * kinds)()
        count = (ctypes.c_int64 * kinds)()
        _lib.check(lib.hsnw_profile_end(ms, count, kinds))
        for k in range(kinds):
            name = lib.hsnw_profile_kind_name(k).decode()
            self.ms[name] = float(ms[k])
            self.launches[name] = int(count[k])
