"""The window kernels behind the reference's own Python interface.

Function names, argument order and meaning, return values and the "decline by returning
``None``" behaviour are those of the reference module ``python/hsn/kernels/window.py`` (cited per
function), and the torch custom ops keep its names and schemas (``hsn::window_select``,
``hsn::window_select_tape``, ``hsn::window_select_fold``, ``hsn::window_cell_update``,
``hsn::window_update_tape``, ``hsn::window_update_fold``), so ``hsn.train.compile`` and
``hsn.train.split`` can import this module in its place. Underneath, every call packs the
reference's launch descriptor and goes through the C ABI (``hsnw_launch``) to this library's own
sm_100a kernels. Import never initialises CUDA; :func:`prepare` readies a device. There is no
PyTorch fallback in here: a missing library raises.
"""

from __future__ import annotations

import ctypes
from typing import TYPE_CHECKING, Any, NamedTuple, cast

import torch
from torch import Tensor, nn

from .. import _lib

if TYPE_CHECKING:  # the reference's classes, duck-typed at run time
    PDGCell = Any
    CellGraphState = Any

_prepared: set[int] = set()


def available() -> bool:
    """Artifact presence only: never initialises CUDA or loads a library
    (reference ``window.py:56-62``)."""
    return _lib.available()


def prepare(device: int = 0) -> None:
    """Ready the kernels on ``device`` (idempotent; reference ``window.py:94-97``)."""
    _lib.check(_lib.library().hsnw_prepare(int(device)))
    _prepared.add(int(device))


def prepared(device: torch.device) -> bool:
    """Reference ``window.py:100-101``."""
    return device.type == "cuda" and (device.index or 0) in _prepared


def _launch(name: str, tensors: list[Tensor], ints: list[int], floats: list[float]) -> None:
    """Pack the descriptor as the reference's launcher does (``window_ext.cpp:75-103``: tensors'
    addresses in order, then ints, then floats) and launch ``name`` on the current stream with
    the launch shape the library asks for."""
    if not tensors or len(tensors) > _lib.HSN_WIN_POINTERS or len(ints) > _lib.HSN_WIN_INTS \
            or len(floats) > _lib.HSN_WIN_FLOATS:  # fmt: skip
        raise RuntimeError("HSN window kernels: launch descriptor overflow")
    device = tensors[0].device
    args = _lib.HsnWinArgs()
    for k, t in enumerate(tensors):
        if not t.is_cuda or t.device != device:
            raise RuntimeError(f"HSN window kernels: tensor {k} must be a CUDA tensor on one device")
        args.p[k] = t.data_ptr()
    for k, v in enumerate(ints):
        args.i[k] = int(v)
    for k, v in enumerate(floats):
        args.f[k] = float(v)
    lib = _lib.library()
    grid, block, shared = ctypes.c_int64(), ctypes.c_int(), ctypes.c_int()
    encoded = name.encode()
    with torch.cuda.device(device):
        _lib.check(lib.hsnw_launch_shape(encoded, ctypes.byref(args), ctypes.byref(grid), ctypes.byref(block), ctypes.byref(shared)))
        stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        _lib.check(lib.hsnw_launch(encoded, ctypes.byref(args), grid.value, block.value, shared.value, stream))


def _shape_error(name: str, ints: list[int]) -> str | None:
    args = _lib.HsnWinArgs()
    for k, v in enumerate(ints):
        args.i[k] = int(v)
    lib = _lib.library()
    grid, block, shared = ctypes.c_int64(), ctypes.c_int(), ctypes.c_int()
    code = lib.hsnw_launch_shape(name.encode(), ctypes.byref(args), ctypes.byref(grid), ctypes.byref(block), ctypes.byref(shared))
    return None if code == _lib.OK else lib.hsnw_last_error().decode()


# --------------------------------------------------------------------------------------------------
# The backward state recurrence (full cut)
# --------------------------------------------------------------------------------------------------


def recurrence_backward(
    c: Tensor,
    b: Tensor,
    h_old: Tensor,
    cells: Tensor,
    valid: Tensor,
    reset: Tensor,
    n_cells: int,
    d_q_pre: Tensor | None,
    d_q_post: Tensor | None,
    d_h_sel: Tensor | None,
    initial: tuple[Tensor, Tensor] | None = None,
) -> tuple[Tensor, Tensor] | None:
    """``hsn.train.split.recurrence_backward`` as one kernel launch, one block per row (reference
    ``window.py:108-153``), or ``None`` when the inputs are not fp32 tensors on a prepared CUDA
    device or the row's cotangents ``(N + 1) d`` floats do not fit a block's shared memory (227 KB
    here, 48 KB in the reference). ``initial`` (an addition): ``(A [B,N,d], R [B,d])``, the
    cotangent of the state after the window, replaced in place by that of the state before it."""
    if not prepared(c.device) or c.dtype != torch.float32 or cells.dtype != torch.int64:
        return None
    B, T, K, d = (int(n) for n in c.shape)
    N = int(n_cells)
    for cot in (d_q_pre, d_q_post, d_h_sel):
        if cot is not None and cot.dtype != torch.float32:
            return None
    ints = [B, T, K, d, N, d_q_pre is not None, d_q_post is not None, d_h_sel is not None, initial is not None]
    if _shape_error("hsn_win_recurrence", [int(v) for v in ints]) is not None:
        return None
    dc = torch.empty_like(c, memory_format=torch.contiguous_format)
    db = torch.empty_like(c, memory_format=torch.contiguous_format)
    absent = dc  # an unread placeholder address for the cotangents a window did not produce
    tensors = [
        c.contiguous(),
        b.contiguous(),
        h_old.contiguous(),
        cells.contiguous(),
        valid.contiguous(),
        reset.contiguous(),
        absent if d_q_pre is None else d_q_pre.contiguous(),
        absent if d_q_post is None else d_q_post.contiguous(),
        absent if d_h_sel is None else d_h_sel.contiguous(),
        dc,
        db,
    ]
    if initial is not None:
        A, R = initial
        if A.dtype != torch.float32 or not A.is_contiguous() or not R.is_contiguous() \
                or tuple(A.shape) != (B, N, d) or tuple(R.shape) != (B, d):  # fmt: skip
            raise ValueError("initial must be contiguous fp32 (A [B,N,d], R [B,d])")
        tensors += [A, R]
    _launch("hsn_win_recurrence", tensors, [int(v) for v in ints], [])
    return dc, db


def dense_recurrence_backward(
    c: Tensor,
    b: Tensor,
    h_old: Tensor,
    reset: Tensor,
    n_cells: int,
    d_q_pre: Tensor | None,
    d_q_post: Tensor | None,
) -> tuple[Tensor, Tensor] | None:
    """``hsn.train.split.dense_recurrence_backward`` as one launch (reference
    ``window.py:156-192``), or ``None`` for inputs it does not take."""
    if not prepared(c.device) or c.dtype != torch.float32:
        return None
    Bd, T, N, d = (int(n) for n in c.shape)
    if N != int(n_cells):
        return None
    for cot in (d_q_pre, d_q_post):
        if cot is not None and cot.dtype != torch.float32:
            return None
    ints = [Bd, T, N, d, int(d_q_pre is not None), int(d_q_post is not None)]
    if _shape_error("hsn_win_recurrence_dense", ints) is not None:
        return None
    dc = torch.empty_like(c, memory_format=torch.contiguous_format)
    db = torch.empty_like(c, memory_format=torch.contiguous_format)
    absent = dc
    tensors = [
        c.contiguous(),
        b.contiguous(),
        h_old.contiguous(),
        reset.contiguous(),
        absent if d_q_pre is None else d_q_pre.contiguous(),
        absent if d_q_post is None else d_q_post.contiguous(),
        dc,
        db,
    ]
    _launch("hsn_win_recurrence_dense", tensors, ints, [])
    return dc, db


# --------------------------------------------------------------------------------------------------
# The abandoned fused cell round of the reference (window.py:202-353, 1007-1051)
# --------------------------------------------------------------------------------------------------


def cell_round_error(cell: "PDGCell") -> str | None:
    """Why the fused cell round cannot run (reference ``window.py:202-230`` returns ``None`` when
    it can). Here it never can: the reference measured its five-kernel round slower than the
    products it replaced and no window runs it; the whole round lives in ``hsnw_window_forward``."""
    return "hsn_b200 does not ship the reference's abandoned five-kernel cell round; use window_forward"


def cell_round(*args: Any, **kwargs: Any) -> Any:
    raise RuntimeError(cell_round_error(None))


# --------------------------------------------------------------------------------------------------
# The router's hard decision
# --------------------------------------------------------------------------------------------------

_NAMESPACE = "hsn"
try:  # the reference module may already own the names in this process
    _taken = hasattr(torch.ops.hsn, "window_select")
except Exception:  # pragma: no cover
    _taken = False
if _taken:
    _NAMESPACE = "hsn_b200"


def _select_launch(
    logits: Tensor, age: Tensor, cost: Tensor, cells: Tensor, units: Tensor, valid: Tensor, theta: Tensor,
    refreshed: Tensor, ints: list[int], floats: list[float],
) -> None:  # fmt: skip
    _launch("hsn_win_select", [logits, age, cost, cells, units, valid, theta, refreshed], ints, floats)


@torch.library.custom_op(f"{_NAMESPACE}::window_select", mutates_args=(), device_types="cuda")
def select_op(
    logits: Tensor,
    age: Tensor,
    cost: Tensor,
    k: int,
    age_max: int,
    probes: bool,
    lambda_cost: float,
    cell_overhead: float,
    shared_cost: float,
    limit: float,
    reserved: int = 0,
    reserved_units: bool = False,
) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    """The hard decision of one position, forward only: ``(cells, units, valid, theta,
    refreshed)`` (reference ``window.py:356-393``). ``logits [B, N, M]`` fp32, ``age [B, N]`` int64
    and ``cost [M]`` fp32, contiguous on one prepared CUDA device."""
    B, N, M = (int(n) for n in logits.shape)
    device = logits.device
    cells = torch.empty((B, k), dtype=torch.int64, device=device)
    units = torch.empty((B, k), dtype=torch.int64, device=device)
    valid = torch.empty((B, k), dtype=torch.bool, device=device)
    theta = torch.empty((B,), dtype=torch.float32, device=device)
    refreshed = torch.empty((B, k), dtype=torch.bool, device=device)
    _select_launch(
        logits, age, cost, cells, units, valid, theta, refreshed,
        [B, N, M, k, age_max, int(probes), 0, 1, 1, 0, 0, reserved, int(reserved_units)],
        [lambda_cost, cell_overhead, shared_cost, limit],
    )  # fmt: skip
    return cells, units, valid, theta, refreshed


@select_op.register_fake
def _select_fake(
    logits: Tensor, age: Tensor, cost: Tensor, k: int, age_max: int, probes: bool, lambda_cost: float,
    cell_overhead: float, shared_cost: float, limit: float, reserved: int = 0, reserved_units: bool = False,
) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:  # fmt: skip
    B = logits.shape[0]
    return (
        logits.new_empty((B, k), dtype=torch.int64),
        logits.new_empty((B, k), dtype=torch.int64),
        logits.new_empty((B, k), dtype=torch.bool),
        logits.new_empty((B,), dtype=torch.float32),
        logits.new_empty((B, k), dtype=torch.bool),
    )


@torch.library.custom_op(
    f"{_NAMESPACE}::window_select_tape",
    mutates_args=("cells", "units", "valid", "theta", "refreshed"),
    device_types="cuda",
)
def select_tape_op(
    logits: Tensor,
    age: Tensor,
    cost: Tensor,
    cells: Tensor,
    units: Tensor,
    valid: Tensor,
    theta: Tensor,
    refreshed: Tensor,
    t: int,
    age_max: int,
    probes: bool,
    lambda_cost: float,
    cell_overhead: float,
    shared_cost: float,
    limit: float,
    reserved: int = 0,
    reserved_units: bool = False,
) -> None:
    """:func:`select_op` written into record ``t`` of a tape (reference ``window.py:421-461``): no
    other record is touched."""
    B, N, M = (int(n) for n in logits.shape)
    n, k = int(cells.shape[1]), int(cells.shape[2])
    _select_launch(
        logits, age, cost, cells, units, valid, theta, refreshed,
        [B, N, M, k, age_max, int(probes), t, n, int(age.shape[1]), 0, 0, reserved, int(reserved_units)],
        [lambda_cost, cell_overhead, shared_cost, limit],
    )  # fmt: skip


@select_tape_op.register_fake
def _select_tape_fake(
    logits: Tensor, age: Tensor, cost: Tensor, cells: Tensor, units: Tensor, valid: Tensor, theta: Tensor,
    refreshed: Tensor, t: int, age_max: int, probes: bool, lambda_cost: float, cell_overhead: float,
    shared_cost: float, limit: float, reserved: int = 0, reserved_units: bool = False,
) -> None:  # fmt: skip
    return None


@torch.library.custom_op(
    f"{_NAMESPACE}::window_select_fold",
    mutates_args=("cells", "units", "valid", "theta", "refreshed"),
    device_types="cuda",
)
def select_fold_op(
    scored: Tensor,
    age: Tensor,
    cost: Tensor,
    cells: Tensor,
    units: Tensor,
    valid: Tensor,
    theta: Tensor,
    refreshed: Tensor,
    t: int,
    n_units: int,
    age_max: int,
    probes: bool,
    lambda_cost: float,
    cell_overhead: float,
    shared_cost: float,
    limit: float,
    reserved: int = 0,
    reserved_units: bool = False,
) -> None:
    """:func:`select_tape_op` on the scorer's matrix product as it is (reference
    ``window.py:487-530``): ``scored [B * N, W]`` fp32 or bf16 holds the logits in its first
    ``n_units`` columns."""
    rows, width = int(scored.shape[0]), int(scored.shape[1])
    B = int(cells.shape[0])
    N = rows // B
    n, k = int(cells.shape[1]), int(cells.shape[2])
    half = scored.dtype == torch.bfloat16
    _select_launch(
        scored, age, cost, cells, units, valid, theta, refreshed,
        [B, N, n_units, k, age_max, int(probes), t, n, int(age.shape[1]), width, int(half), reserved,
         int(reserved_units)],
        [lambda_cost, cell_overhead, shared_cost, limit],
    )  # fmt: skip


@select_fold_op.register_fake
def _select_fold_fake(
    scored: Tensor, age: Tensor, cost: Tensor, cells: Tensor, units: Tensor, valid: Tensor, theta: Tensor,
    refreshed: Tensor, t: int, n_units: int, age_max: int, probes: bool, lambda_cost: float,
    cell_overhead: float, shared_cost: float, limit: float, reserved: int = 0, reserved_units: bool = False,
) -> None:  # fmt: skip
    return None


def select_unsupported(n_cells: int, k: int, n_units: int = 1) -> str | None:
    """Why :func:`select` cannot take a model of this shape (``None``: it can; reference
    ``window.py:557-565`` refuses more than 256 cells, this kernel takes any ``N`` whose scores
    fit a block's shared memory)."""
    if k > n_cells:
        return f"k_select={k} exceeds model.n_cells={n_cells}"
    return _shape_error("hsn_win_select", [1, n_cells, n_units, k])


def select(
    logits: Tensor,
    age: Tensor,
    cost_table: Tensor,
    *,
    k: int,
    age_max: int,
    probes: bool,
    lambda_cost: float,
    cell_overhead: float,
    shared_cost: float,
    limit: float,
    reserved: int = 0,
    reserved_units: bool = False,
) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    """``Router.select`` for the forward sweep (mode ``topk``, the hard decision, no exploration,
    the refresh probes when ``probes``) as one kernel (reference ``window.py:568-602``)."""
    decision: tuple[Tensor, Tensor, Tensor, Tensor, Tensor] = select_op(
        logits.to(torch.float32).contiguous(),
        age.contiguous(),
        cost_table.to(torch.float32).contiguous(),
        k, age_max, probes, lambda_cost, cell_overhead, shared_cost, limit, reserved, reserved_units,
    )  # fmt: skip
    return decision


def select_tape(
    logits: Tensor, tape_age: Tensor, cost_table: Tensor, cells: Tensor, units: Tensor, valid: Tensor,
    theta: Tensor, refreshed: Tensor, *, t: int, age_max: int, probes: bool, lambda_cost: float,
    cell_overhead: float, shared_cost: float, limit: float, reserved: int = 0, reserved_units: bool = False,
) -> None:  # fmt: skip
    """:func:`select` for position ``t`` of a block, written into record ``t`` of the block's
    decision tape (reference ``window.py:923-965``)."""
    select_tape_op(
        logits.to(torch.float32).contiguous(), tape_age, cost_table.to(torch.float32).contiguous(),
        cells, units, valid, theta, refreshed, t, age_max, probes, lambda_cost, cell_overhead,
        shared_cost, limit, reserved, reserved_units,
    )  # fmt: skip


def select_fold(
    scored: Tensor, tape_age: Tensor, cost_table: Tensor, cells: Tensor, units: Tensor, valid: Tensor,
    theta: Tensor, refreshed: Tensor, *, t: int, n_units: int, age_max: int, probes: bool,
    lambda_cost: float, cell_overhead: float, shared_cost: float, limit: float, reserved: int = 0,
    reserved_units: bool = False,
) -> None:  # fmt: skip
    """:func:`select_tape` from the scorer's matrix product ``scored [B * N, W]`` as it is
    (reference ``window.py:1054-1096``)."""
    select_fold_op(
        scored, tape_age, cost_table.to(torch.float32).contiguous(), cells, units, valid, theta,
        refreshed, t, n_units, age_max, probes, lambda_cost, cell_overhead, shared_cost, limit,
        reserved, reserved_units,
    )  # fmt: skip


# --------------------------------------------------------------------------------------------------
# The end of a position's round
# --------------------------------------------------------------------------------------------------


@torch.library.custom_op(f"{_NAMESPACE}::window_cell_update", mutates_args=(), device_types="cuda")
def cell_update_op(
    y: Tensor,
    gate: Tensor,
    h: Tensor,
    q: Tensor,
    age: Tensor,
    pos: Tensor,
    cells: Tensor,
    valid: Tensor,
    cand_w: Tensor,
    cand_norm: bool,
    cand_eps: float,
) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """The end of one position's round, forward only: ``(h, q, age, pos, h_sel, h_max)``
    (reference ``window.py:605-655``)."""
    B, N, d = (int(n) for n in h.shape)
    K = int(cells.shape[1])
    h_next = torch.empty_like(h)
    q_next = torch.empty_like(q)
    age_next = torch.empty_like(age)
    pos_next = torch.empty_like(pos)
    h_sel = h.new_empty((B, K, d))
    h_max = h.new_empty((B,))
    _launch(
        "hsn_win_cell_update",
        [y, gate, h, q, age, pos, cells, valid, cand_w, h_next, q_next, age_next, pos_next, h_sel, h_max],
        [B, N, d, K, int(cand_norm), 0, 1, 1, 0, 0, 1, 0],
        [cand_eps],
    )
    return h_next, q_next, age_next, pos_next, h_sel, h_max


@cell_update_op.register_fake
def _cell_update_fake(
    y: Tensor, gate: Tensor, h: Tensor, q: Tensor, age: Tensor, pos: Tensor, cells: Tensor, valid: Tensor,
    cand_w: Tensor, cand_norm: bool, cand_eps: float,
) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:  # fmt: skip
    return (
        torch.empty_like(h),
        torch.empty_like(q),
        torch.empty_like(age),
        torch.empty_like(pos),
        h.new_empty((*cells.shape, h.shape[2])),
        h.new_empty((h.shape[0],)),
    )


@torch.library.custom_op(
    f"{_NAMESPACE}::window_update_tape",
    mutates_args=("tape_h", "tape_q", "tape_age", "tape_hsel", "h_max", "qs"),
    device_types="cuda",
)
def update_tape_op(
    y: Tensor,
    gate: Tensor,
    tape_h: Tensor,
    tape_q: Tensor,
    tape_age: Tensor,
    cells: Tensor,
    valid: Tensor,
    cand_w: Tensor,
    reset: Tensor,
    tape_hsel: Tensor,
    h_max: Tensor,
    qs: Tensor,
    t: int,
    cand_norm: bool,
    cand_eps: float,
) -> None:
    """:func:`cell_update_op` on a tape: reads record ``t``, writes record ``t + 1`` with the
    next position's reset applied (reference ``window.py:682-741``)."""
    B, n_state, N, d = (int(n) for n in tape_h.shape)
    n, K = int(cells.shape[1]), int(cells.shape[2])
    _launch(
        "hsn_win_cell_update",
        [y, gate, tape_h, tape_q, tape_age, tape_age, cells, valid, cand_w, tape_h, tape_q, tape_age,
         tape_age, tape_hsel, h_max, reset, qs],
        [B, N, d, K, int(cand_norm), t, n_state, n, t + 1, int(t + 1 < n), 0, 1],
        [cand_eps],
    )  # fmt: skip


@update_tape_op.register_fake
def _update_tape_fake(
    y: Tensor, gate: Tensor, tape_h: Tensor, tape_q: Tensor, tape_age: Tensor, cells: Tensor, valid: Tensor,
    cand_w: Tensor, reset: Tensor, tape_hsel: Tensor, h_max: Tensor, qs: Tensor, t: int, cand_norm: bool,
    cand_eps: float,
) -> None:  # fmt: skip
    return None


@torch.library.custom_op(
    f"{_NAMESPACE}::window_update_fold",
    mutates_args=("tape_h", "tape_q", "tape_age", "tape_hsel", "h_max", "qs", "x"),
    device_types="cuda",
)
def update_fold_op(
    y: Tensor,
    gate: Tensor,
    tape_h: Tensor,
    tape_q: Tensor,
    tape_age: Tensor,
    cells: Tensor,
    valid: Tensor,
    cand_w: Tensor,
    reset: Tensor,
    tape_hsel: Tensor,
    h_max: Tensor,
    qs: Tensor,
    x: Tensor,
    z: Tensor,
    context: Tensor,
    t: int,
    cand_norm: bool,
    cand_eps: float,
    n_fast: int = 0,
) -> None:
    """:func:`update_tape_op` on the round's matrix products as they are, fp32 or bf16, ``gate`` a
    strided view, and the next position's input row ``[z; q; ctx (; f)]`` written into ``x``
    (reference ``window.py:765-853``)."""
    B, n_state, N, d = (int(n) for n in tape_h.shape)
    n, K = int(cells.shape[1]), int(cells.shape[2])
    d_z, d_c = int(z.shape[2]), int(context.shape[2])
    if tuple(x.shape) != (n, B, d_z + d + d_c + (d if n_fast else 0)):
        raise ValueError(f"x must be [n, B, d_z + d + d_c (+ d)], got {tuple(x.shape)}")
    if not 0 <= n_fast <= N:
        raise ValueError(f"n_fast must lie in [0, {N}], got {n_fast}")
    ints = [B, N, d, K, int(cand_norm), t, n_state, n, t + 1, int(t + 1 < n), 0, 1]
    ints += [
        int(y.dtype == torch.bfloat16),
        int(gate.dtype == torch.bfloat16),
        int(gate.stride(0)),
        1,
        int(x.dtype == torch.bfloat16),
        d_z,
        int(z.dtype == torch.bfloat16),
        d_c,
        int(context.dtype == torch.bfloat16),
        n_fast,
    ]
    _launch(
        "hsn_win_cell_update",
        [y, gate, tape_h, tape_q, tape_age, tape_age, cells, valid, cand_w, tape_h, tape_q, tape_age,
         tape_age, tape_hsel, h_max, reset, qs, x, z, context],
        ints,
        [cand_eps],
    )  # fmt: skip


@update_fold_op.register_fake
def _update_fold_fake(
    y: Tensor, gate: Tensor, tape_h: Tensor, tape_q: Tensor, tape_age: Tensor, cells: Tensor, valid: Tensor,
    cand_w: Tensor, reset: Tensor, tape_hsel: Tensor, h_max: Tensor, qs: Tensor, x: Tensor, z: Tensor,
    context: Tensor, t: int, cand_norm: bool, cand_eps: float, n_fast: int = 0,
) -> None:  # fmt: skip
    return None


def cell_update_unsupported(n_cells: int, d: int, k: int) -> str | None:
    """Why :func:`cell_update` cannot take a model of this shape (``None``: it can; reference
    ``window.py:881-887``)."""
    return _shape_error("hsn_win_cell_update", [1, n_cells, d, k])


def _cand(cell: "PDGCell") -> tuple[Tensor, bool, float]:
    cand_norm = cell.cand_norm_kind != "none"
    weight = cell.cand_norm.weight if cand_norm else cell.norm.weight
    eps = float(cast(nn.RMSNorm, cell.cand_norm).eps or 0.0) if cand_norm else 0.0
    return weight, cand_norm, eps


def cell_update(
    cell: "PDGCell", y: Tensor, gate: Tensor, state: "CellGraphState", cells: Tensor, valid: Tensor
) -> tuple["CellGraphState", Tensor, Tensor]:
    """The round of one position from its matrix products on: the candidate (its norm, ``tanh``),
    the gate's sigmoid, the gated update and the tick as one kernel (reference
    ``window.py:890-920``). Returns the state after the position (the same class as ``state``),
    the slots' cells after the update ``[B, K, d]`` and each row's ``max |h|`` ``[B]``."""
    weight, cand_norm, eps = _cand(cell)
    h, q, age, pos, h_sel, h_max = cell_update_op(
        y.contiguous(), gate.contiguous(), state.h.contiguous(), state.q.contiguous(),
        state.age.contiguous(), state.pos.contiguous(), cells.contiguous(), valid.contiguous(),
        weight, cand_norm, eps,
    )  # fmt: skip
    return type(state)._make(h=h, q=q, age=age, pos=pos), h_sel, h_max


def update_tape(
    cell: "PDGCell", y: Tensor, gate: Tensor, tape_h: Tensor, tape_q: Tensor, tape_age: Tensor,
    cells: Tensor, valid: Tensor, reset: Tensor, tape_hsel: Tensor, h_max: Tensor, qs: Tensor, *, t: int,
) -> None:  # fmt: skip
    """:func:`cell_update` for position ``t`` of a block on its tapes (reference
    ``window.py:968-1004``)."""
    weight, cand_norm, eps = _cand(cell)
    update_tape_op(
        y.contiguous(), gate.contiguous(), tape_h, tape_q, tape_age, cells, valid, weight, reset,
        tape_hsel, h_max, qs, t, cand_norm, eps,
    )  # fmt: skip


def update_fold(
    cell: "PDGCell", y: Tensor, gate: Tensor, tape_h: Tensor, tape_q: Tensor, tape_age: Tensor,
    cells: Tensor, valid: Tensor, reset: Tensor, tape_hsel: Tensor, h_max: Tensor, qs: Tensor, x: Tensor,
    z: Tensor, context: Tensor, *, t: int, n_fast: int = 0,
) -> None:  # fmt: skip
    """:func:`update_tape` from the round's matrix products as they are, with the next position's
    input of the first product written into ``x`` (reference ``window.py:1099-1143``)."""
    weight, cand_norm, eps = _cand(cell)
    update_fold_op(
        y, gate, tape_h, tape_q, tape_age, cells, valid, weight, reset, tape_hsel, h_max, qs, x, z,
        context, t, cand_norm, eps, n_fast,
    )  # fmt: skip


# --------------------------------------------------------------------------------------------------
# The reverse sweep's glue kernels (reference window.py:1147-1290)
# --------------------------------------------------------------------------------------------------

ACTIVATION_CODES: dict[str, int] = {"gelu": 0, "relu": 1, "silu": 2, "tanh": 3}
"""The activation's code in ``hsn_win_back_mid`` (reference ``python/hsn/train/state_sweep.py:67``)."""


class SweepShape(NamedTuple):
    """The sizes a reverse sweep is built for, in the reference's order
    (``python/hsn/train/state_sweep.py:70-86``): ``n_fast`` leading slots have a fixed unit and
    their own operands, ``n_read`` cells are read after every position, ``in_dim`` is the width the
    cell norm averages over, ``d_out`` the largest number of cells one cell is a message source of."""

    B: int
    T: int
    K: int
    N: int
    d: int
    H: int
    M: int
    n_fast: int
    n_read: int
    in_dim: int
    d_out: int


class SweepBuffers:
    """The static buffers of a reverse sweep under the reference's names, shapes and dtypes
    (``ReverseSweep.__init__``, ``state_sweep.py:143-198``): what :func:`back_head`,
    :func:`back_mid` and :func:`back_tail` read and write. The reference's own ``ReverseSweep``
    can be passed to those functions instead; this class exists for callers that hold no
    reference object. The two products between the kernels stay the caller's."""

    def __init__(self, shape: SweepShape, *, device: torch.device, product_dtype: torch.dtype = torch.float32,
                 activation: str = "gelu", cand_norm: bool = True, cand_eps: float = 1e-6,
                 cell_norm: bool = True) -> None:  # fmt: skip
        if product_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("the products' dtype is float32 or bfloat16")
        B, T, K, N, d, H, M, F, n_read, _, d_out = shape
        if not 0 <= F < K:
            raise ValueError(f"n_fast={F} must leave a routed slot of the {K} slots")
        self.shape, self.device = shape, device
        self.state_dtype, self.product_dtype = torch.float32, product_dtype
        self.activation, self.cand_norm, self.cand_eps, self.cell_norm = activation, cand_norm, float(cand_eps), cell_norm
        self.routed = K - F
        rows = B * self.routed

        def state(*size: int) -> Tensor:
            return torch.zeros(*size, dtype=torch.float32, device=device)

        def product(*size: int) -> Tensor:
            return torch.zeros(*size, dtype=product_dtype, device=device)

        def index(*size: int) -> Tensor:
            return torch.zeros(*size, dtype=torch.int64, device=device)

        self.A, self.R = state(B, N, d), state(B, d)
        self.c, self.b, self.h_old = state(B, T, K, d), state(B, T, K, d), state(B, T, K, d)
        self.y, self.gate_pre, self.mv = state(B, T, K, d), state(B, T, K, d), state(B, T, K, d)
        self.rms = state(B, T, K)
        self.hidden = product(B, T, K, H)
        self.cells, self.units = index(B, T, K), index(B, T, K)
        self.valid = torch.zeros(B, T, K, dtype=torch.bool, device=device)
        self.reset = torch.zeros(B, T, dtype=torch.bool, device=device)
        self.d_q_pre, self.d_q_post = state(B, T, d), state(B, T, d)
        self.d_h_sel = state(B, T, K, d)
        self.d_h_fast = state(B, T, max(n_read, 1), d)
        self.cand_gain, self.gate_bias, self.b1 = state(d), state(d), state(M, H)
        self.out_tgt = torch.full((N, d_out), -1, dtype=torch.int32, device=device)
        self.out_w = state(N, d_out)
        self.op1, self.op2 = product(rows, M * d), product(rows, M * H + d)
        self.op1_fast, self.op2_fast = product(max(F, 1), B, d), product(max(F, 1), B, H + d)
        self.act_r, self.dv_r = product(rows, H), product(rows, 2 * d)
        self.act_f, self.dv_f = product(max(F, 1), B, H), product(max(F, 1), B, 2 * d)
        self.sigma = state(B, K)
        self.dc, self.db = state(B, T, K, d), state(B, T, K, d)


def _half(t: Tensor) -> int:
    return int(t.dtype == torch.bfloat16)


def _back_head_ints(s: SweepShape, t: int, cand_norm: bool, half: int) -> list[int]:
    return [s.B, s.T, s.K, s.d, s.N, s.M, s.H, s.n_fast, t, s.n_read, int(cand_norm), half]


def back_unsupported(shape: SweepShape) -> str | None:
    """Why the reverse sweep's kernels cannot take this shape (``None``: they can; reference
    ``window.py:1166-1178``, whose limits of 32 slots and of the reference kernels' shared memory
    do not exist here: the only limit is the tail's ``2 K d + N`` words of shared memory)."""
    s = SweepShape(*shape)
    for name, ints in (
        ("hsn_win_back_head", _back_head_ints(s, 0, True, 0)),
        ("hsn_win_back_mid", [s.B, s.T, s.K, s.d, s.M, s.H, s.n_fast, 0, 0, 0, 0]),
        ("hsn_win_back_tail", [s.B, s.T, s.K, s.d, s.N, s.n_fast, 0, s.d_out, 1, s.in_dim, 0]),
    ):
        reason = _shape_error(name, ints)
        if reason is not None:
            return reason
    return None


def _position(s: SweepShape, t: int) -> None:
    if not 0 <= t < s.T:
        raise ValueError(f"position {t} is outside the window's {s.T}")


def back_head(sweep: Any, t: int) -> None:
    """The head of position ``t`` of a reverse sweep on its buffers (``hsn_win_back_head``;
    reference ``window.py:1185-1221``, contract ``ReverseSweep.head_reference``,
    ``state_sweep.py:441-477``): ``R += d_q_post``, the read cells' and the selected cells'
    cotangents into ``A``, ``dc``/``db`` of the position, the written cells' rows of ``A``
    replaced, the candidate norm's backward, and the first product's operand ``op1`` (block of the
    slot's unit, the block position ``t + 1`` used cleared), the gate columns of ``op2`` and
    ``sigma``."""
    s = SweepShape(*sweep.shape)
    _position(s, t)
    _launch(
        "hsn_win_back_head",
        [sweep.A, sweep.R, sweep.c, sweep.b, sweep.h_old, sweep.y, sweep.cells, sweep.units, sweep.valid,
         sweep.d_q_post, sweep.d_h_sel, sweep.d_h_fast, sweep.cand_gain, sweep.gate_pre, sweep.gate_bias,
         sweep.dc, sweep.db, sweep.op1, sweep.op1_fast, sweep.op2, sweep.op2_fast, sweep.sigma],
        _back_head_ints(s, t, bool(sweep.cand_norm), _half(sweep.op1)),
        [float(sweep.cand_eps)],
    )  # fmt: skip


def back_mid(sweep: Any, t: int) -> None:
    """The middle of position ``t`` (``hsn_win_back_mid``; reference ``window.py:1224-1250``,
    contract ``ReverseSweep.middle_reference``, ``state_sweep.py:487-495``): the first product's
    result ``act_r``/``act_f`` through the activation's derivative at ``hidden`` into the hidden
    blocks of ``op2``, and its part of ``sigma``."""
    s = SweepShape(*sweep.shape)
    _position(s, t)
    _launch(
        "hsn_win_back_mid",
        [sweep.act_r, sweep.act_f, sweep.hidden, sweep.units, sweep.valid, sweep.b1, sweep.op2,
         sweep.op2_fast, sweep.sigma],
        [s.B, s.T, s.K, s.d, s.M, s.H, s.n_fast, t, _half(sweep.act_r), _half(sweep.hidden),
         ACTIVATION_CODES[sweep.activation]],
        [],
    )  # fmt: skip


def back_tail(sweep: Any, t: int) -> None:
    """The tail of position ``t`` (``hsn_win_back_tail``; reference ``window.py:1253-1281``,
    contract ``ReverseSweep.tail_reference``, ``state_sweep.py:497-533`` without a row limit): the
    second product's result ``dv_r``/``dv_f`` through the cell norm, its state half added to the
    selected cells' rows of ``A``, its message half to every source of a selected cell along
    ``out_tgt``/``out_w``, ``R += d_q_pre``, and the reset."""
    s = SweepShape(*sweep.shape)
    _position(s, t)
    _launch(
        "hsn_win_back_tail",
        [sweep.A, sweep.R, sweep.dv_r, sweep.dv_f, sweep.sigma, sweep.rms, sweep.h_old, sweep.mv, sweep.cells,
         sweep.valid, sweep.out_tgt, sweep.out_w, sweep.d_q_pre, sweep.reset],
        [s.B, s.T, s.K, s.d, s.N, s.n_fast, t, s.d_out, int(bool(sweep.cell_norm)), s.in_dim,
         _half(sweep.dv_r)],
        [],
    )  # fmt: skip
