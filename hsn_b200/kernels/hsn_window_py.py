"""A stand-in for the reference's pybind launcher module ``hsn_window_py``
(``python/hsn/kernels/window_ext.cpp:216-222``): ``prepare``, ``launch``, ``launch_views``, ``loop`` and
``launch_table`` with the reference's signatures, forwarding to this library's C ABI.

The reference's own ``python/hsn/kernels/window.py`` can import this module in place of its compiled
extension (it looks the module up as ``hsn_window_py`` next to its fatbin): the kernels here keep the
reference's names and ``HsnWinArgs`` slot layouts. Two differences, both on purpose:

* the ``grid``, ``block`` and ``shared`` a caller passes are the reference kernels' launch shapes
  (``window.py:38-53``); these kernels use other block sizes and shared-memory layouts, so the shape
  is taken from ``hsnw_launch_shape`` for the sizes in the descriptor instead (``grid <= 0`` still
  launches nothing, ``window_ext.cpp:96``);
* ``launch_table`` (the trainer's multi-tensor kernels, ``window_ext.cpp:155-213``) ignores ``block``
  for the same reason: ``hsnw_launch_table`` sizes its own grid.
"""

from __future__ import annotations

import ctypes
from collections.abc import Sequence

import torch
from torch import Tensor

from .. import _lib

__all__ = ["prepare", "launch", "launch_views", "loop", "launch_table"]


def prepare(path: str, device: int) -> None:
    """``window_ext.cpp:41-56``: make ``device`` ready. ``path`` (the reference's fatbin) is not
    read: the kernels are linked into the library."""
    del path
    _lib.check(_lib.library().hsnw_prepare(int(device)))


def _pack(tensors: Sequence[Tensor], ints: Sequence[int], floats: Sequence[float], views: Sequence[int] = ()):
    """``window_ext.cpp:75-103``: the tensors' addresses in order, then the ints, then the floats; every
    tensor on one CUDA device and contiguous unless named in ``views``."""
    if not tensors or len(tensors) > _lib.HSN_WIN_POINTERS or len(ints) > _lib.HSN_WIN_INTS \
            or len(floats) > _lib.HSN_WIN_FLOATS:  # fmt: skip
        raise RuntimeError("HSN window kernels: launch descriptor overflow")
    device = tensors[0].device
    args = _lib.HsnWinArgs()
    for k, t in enumerate(tensors):
        if not t.is_cuda or t.device != device or not (k in views or t.is_contiguous()):
            raise RuntimeError(f"HSN window kernels: tensor {k} must be a contiguous CUDA tensor on one device")
        args.p[k] = t.data_ptr()
    for k, v in enumerate(ints):
        if not -(2**31) <= int(v) < 2**31:
            raise RuntimeError("HSN window kernels: int range")
        args.i[k] = int(v)
    for k, v in enumerate(floats):
        args.f[k] = float(v)
    return args, device


def _shape(name: bytes, args) -> tuple[int, int, int]:
    grid, block, shared = ctypes.c_int64(), ctypes.c_int(), ctypes.c_int()
    _lib.check(_lib.library().hsnw_launch_shape(name, ctypes.byref(args), ctypes.byref(grid), ctypes.byref(block),
                                                ctypes.byref(shared)))  # fmt: skip
    return grid.value, block.value, shared.value


def _check(code: int) -> None:
    try:
        _lib.check(code)
    except _lib.WindowKernelError as error:  # the reference raises RuntimeError (TORCH_CHECK)
        raise RuntimeError(str(error)) from error


def launch(name: str, grid: int, block: int, shared: int, tensors: Sequence[Tensor], ints: Sequence[int],
           floats: Sequence[float]) -> None:  # fmt: skip
    """``window_ext.cpp:105-115``: one launch of ``name`` on the tensors' device's current stream."""
    launch_views(name, grid, block, shared, tensors, (), ints, floats)


def launch_views(name: str, grid: int, block: int, shared: int, tensors: Sequence[Tensor], views: Sequence[int],
                 ints: Sequence[int], floats: Sequence[float]) -> None:  # fmt: skip
    """``window_ext.cpp:117-127``: :func:`launch` for a kernel that reads the tensors ``views`` as
    strided views (it gets the address of their first element; the caller passes the strides in
    ``ints``)."""
    del block, shared
    args, device = _pack(tensors, ints, floats, views)
    if grid <= 0:
        return
    encoded = name.encode()
    with torch.cuda.device(device):
        try:
            g, b, s = _shape(encoded, args)
        except _lib.WindowKernelError as error:
            raise RuntimeError(str(error)) from error
        stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        _check(_lib.library().hsnw_launch(encoded, ctypes.byref(args), g, b, s, stream))


def loop(names: Sequence[str], grids: Sequence[int], blocks: Sequence[int], shareds: Sequence[int],
         tensors: Sequence[Tensor], ints: Sequence[int], floats: Sequence[float], steps: int, slot: int) -> None:  # fmt: skip
    """``window_ext.cpp:129-153``: ``steps`` rounds of the kernels ``names`` in order; round ``t`` runs
    them with ``ints[slot] = t``."""
    if not (len(names) == len(grids) == len(blocks) == len(shareds)) or not 0 <= slot < min(_lib.HSN_WIN_INTS, len(ints)):
        raise RuntimeError("HSN window kernels: invalid loop descriptor")
    args, device = _pack(tensors, ints, floats)
    count = len(names)
    encoded = [n.encode() for n in names]
    with torch.cuda.device(device):
        try:
            shapes = [_shape(n, args) for n in encoded]
        except _lib.WindowKernelError as error:
            raise RuntimeError(str(error)) from error
        c_names = (ctypes.c_char_p * count)(*encoded)
        # a kernel the caller gives no blocks (grid <= 0) launches nothing, as in launch()
        c_grids = (ctypes.c_int64 * count)(*[s[0] if g > 0 else 0 for s, g in zip(shapes, grids)])
        c_blocks = (ctypes.c_int * count)(*[s[1] for s in shapes])
        c_shareds = (ctypes.c_int * count)(*[s[2] for s in shapes])
        stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        _check(_lib.library().hsnw_loop(c_names, count, c_grids, c_blocks, c_shareds, ctypes.byref(args), int(steps),
                                        int(slot), stream))  # fmt: skip


def launch_table(name: str, block: int, rows: Sequence[Sequence[Tensor]], elementwise: int, ints: Sequence[int],
                 floats: Sequence[float], doubles: Sequence[float], units: Sequence[Sequence[float]]) -> bool:  # fmt: skip
    """``window_ext.cpp:155-213``: launch the trainer kernel ``name`` over the tensors of ``rows`` (up to four
    operands per tensor, ``rows[r][j]`` the r-th operand of tensor ``j``; an empty row is one the kernel
    does not read). The first ``elementwise`` rows are fp32 tensors of row 0's element counts; the other
    rows only have to be on the device. ``False``, with nothing launched, when a tensor is not a contiguous
    tensor of the expected kind on row 0's CUDA device (the caller keeps its PyTorch path); an overflowing
    descriptor raises. More tensors than a descriptor holds go out in several launches; tensors without
    elements are skipped. ``ints`` fill ``i[1..]``."""
    if not rows or len(rows) > _lib.HSN_TR_ROWS or not rows[0] or len(ints) >= _lib.HSN_TR_INTS \
            or len(floats) > _lib.HSN_TR_FLOATS or len(doubles) > _lib.HSN_TR_DOUBLES or len(units) > _lib.HSN_TR_COEFS \
            or not 1 <= elementwise <= len(rows) or block <= 0:  # fmt: skip
        raise RuntimeError("HSN trainer kernels: launch descriptor overflow")
    first = rows[0]
    if not first[0].is_cuda:
        return False
    device = first[0].device
    for r, row in enumerate(rows):
        if row and len(row) != len(first):
            raise RuntimeError(f"HSN trainer kernels: row {r} must be empty or hold one tensor per tensor of row 0")
        for j, t in enumerate(row):
            if not t.is_cuda or t.device != device or not t.is_contiguous():
                return False
            if r < elementwise and (t.dtype != torch.float32 or t.numel() != first[j].numel()):
                return False
    args = _lib.HsnTrainArgs()
    for k, v in enumerate(ints):
        if not -(2**31) <= int(v) < 2**31:
            raise RuntimeError("HSN trainer kernels: int range")
        args.i[k + 1] = int(v)
    for k, v in enumerate(floats):
        args.f[k] = float(v)
    for k, v in enumerate(doubles):
        args.g[k] = float(v)
    for c, coefficients in enumerate(units):
        if len(coefficients) > _lib.HSN_TR_UNITS:
            raise RuntimeError("HSN trainer kernels: too many units")
        for m, v in enumerate(coefficients):
            args.u[c][m] = float(v)
    lib = _lib.library()
    with torch.cuda.device(device):
        stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        todo = [j for j in range(len(first)) if first[j].numel() > 0]
        for at in range(0, len(todo), _lib.HSN_TR_TENSORS):
            total = 0
            for count, j in enumerate(todo[at : at + _lib.HSN_TR_TENSORS]):
                for r, row in enumerate(rows):
                    args.p[r][count] = row[j].data_ptr() if row else None
                total += first[j].numel()
                args.end[count] = total
            args.i[0] = len(todo[at : at + _lib.HSN_TR_TENSORS])
            _lib.check(lib.hsnw_launch_table(name.encode(), ctypes.byref(args), stream))
    return True
