"""The carried window state off the device and back: versioned snapshots and the trainer's checkpoint
payload.

A streaming session or a training run carries ``(h [B,N,d], q [B,d], age [B,N] int64, pos [B] int64)``
between calls of :func:`hsn_b200.window.window_forward` / :func:`~hsn_b200.window.stream_step`. This
module is the hand-off of that state to storage, in the reference's own formats, so that a state written
here is restored by the reference (``hsn.chat``, the trainer's resume) and the other way round:

* :func:`snapshot` / :func:`restore` follow ``CellGraphState.snapshot`` / ``.restore``
  (reference ``python/hsn/model/state.py:363-430``): host copies of the four tensors bound to a
  :class:`StateMeta` under a blake2b-256 digest, and a restore that refuses, in this order, another tenant,
  another model version, another state-schema version, a digest that does not match, an expired snapshot
  — before any tensor reaches the device. The digest's byte layout is the reference's
  (``model/state.py:162-188``): the tag ``hsn.model.state/1``; per tensor the line
  ``\\n<name>:<torch dtype>:<d0>x<d1>..:<bytes>\\n`` and the raw little-endian bytes; then
  ``\\nmeta:<bytes>\\n`` and the meta as canonical JSON.
* :func:`pack_cell_state` / :func:`unpack_cell_state` follow ``train/checkpoint.py:260-292``: the plain
  mapping of the four host tensors a checkpoint stores as ``carried_state``.

On the device side a snapshot is four device-to-host copies on the current stream; a restore is four
host-to-device copies. After a restore the first streaming call must be :func:`~hsn_b200.window.stream_step`
without ``carried`` (the cells' derived values in the previous call's scratch belong to another state).
"""

from __future__ import annotations

import hmac
import json
import math
import time
from collections.abc import Mapping
from dataclasses import asdict, dataclass
from hashlib import blake2b
from typing import Any

import torch
from torch import Tensor

__all__ = [
    "FIELDS", "IntegrityError", "SchemaMismatch", "StateExpired", "StateMeta", "StateRestoreError", "StateSnapshot",
    "TenantMismatch", "VersionMismatch", "check_state", "pack_cell_state", "restore", "snapshot", "state_digest",
    "unpack_cell_state",
]  # fmt: skip

FIELDS = ("h", "q", "age", "pos")
_TAG = b"hsn.model.state/1"
_HEX = 64  # characters of a 32-byte digest


class StateRestoreError(Exception):
    """Every refusal of :func:`restore`."""


class VersionMismatch(StateRestoreError):
    """Written by another model version."""


class SchemaMismatch(StateRestoreError):
    """Written under another state-schema version."""


class TenantMismatch(StateRestoreError):
    """Belongs to another tenant."""


class IntegrityError(StateRestoreError):
    """The digest does not match the tensors and the meta."""


class StateExpired(StateRestoreError):
    """``expires_at`` of the snapshot's own meta has passed."""


def check_state(h: Tensor, q: Tensor, age: Tensor, pos: Tensor, where: str = "state") -> tuple[int, int, int]:
    """The layout every holder of a state must have (reference ``model/state.py:482-509``): ``h [B,N,d]``
    floating, ``q [B,d]`` of the same dtype, ``age [B,N]`` and ``pos [B]`` int64, all sizes >= 1, one device.
    Returns ``(B, N, d)``."""
    named = dict(zip(FIELDS, (h, q, age, pos), strict=True))
    for name, t in named.items():
        if not isinstance(t, Tensor):
            raise TypeError(f"{where}.{name} must be a torch.Tensor, got {type(t).__name__}")
    if h.dim() != 3 or min(h.shape) < 1:
        raise ValueError(f"{where}.h must have shape [B, N, d] with B, N, d >= 1, got {tuple(h.shape)}")
    if not h.is_floating_point():
        raise ValueError(f"{where}.h must be floating point, got {h.dtype}")
    B, N, d = (int(n) for n in h.shape)
    want = {"q": ((B, d), h.dtype), "age": ((B, N), torch.int64), "pos": ((B,), torch.int64)}
    for name, (shape, dtype) in want.items():
        t = named[name]
        if tuple(t.shape) != shape:
            raise ValueError(f"{where}.{name} must have shape {shape}, got {tuple(t.shape)}")
        if t.dtype != dtype:
            raise ValueError(f"{where}.{name} must have dtype {dtype}, got {t.dtype}")
    if len({str(t.device) for t in named.values()}) != 1:
        raise ValueError(f"{where} tensors must share one device")
    return B, N, d


@dataclass(frozen=True)
class StateMeta:
    """What a snapshot is bound to (reference ``model/state.py:97-130``): the model and state-schema
    versions that produced the state, its tenant, and the POSIX time after which it must not be restored
    (``None``: never expires)."""

    model_version: str
    state_schema_version: int
    tenant_id: str
    expires_at: float | None

    def __post_init__(self) -> None:
        for name in ("model_version", "tenant_id"):
            value = getattr(self, name)
            if not isinstance(value, str) or not value:
                raise ValueError(f"StateMeta.{name} must be a non-empty str, got {value!r}")
        schema = self.state_schema_version
        if isinstance(schema, bool) or not isinstance(schema, int) or schema < 1:
            raise ValueError(f"StateMeta.state_schema_version must be an int >= 1, got {schema!r}")
        if self.expires_at is not None:
            e = self.expires_at
            if isinstance(e, bool) or not isinstance(e, (int, float)) or not math.isfinite(e):
                raise ValueError(f"StateMeta.expires_at must be None or a finite POSIX time, got {e!r}")
            object.__setattr__(self, "expires_at", float(e))

    def to_bytes(self) -> bytes:
        """The hashed form: JSON with sorted keys and compact separators, UTF-8."""
        return json.dumps(asdict(self), sort_keys=True, separators=(",", ":")).encode("utf-8")


def state_digest(h: Tensor, q: Tensor, age: Tensor, pos: Tensor, meta: StateMeta) -> str:
    """blake2b-256 over the tag, each tensor's header line and raw bytes, and the meta (the module
    docstring gives the layout). A header names dtype and shape, so the same bytes under another dtype or
    shape do not verify."""
    hasher = blake2b(digest_size=_HEX // 2)
    hasher.update(_TAG)
    for name, t in zip(FIELDS, (h, q, age, pos), strict=True):
        flat = t.detach().to("cpu").contiguous().reshape(-1)
        shape = "x".join(str(int(n)) for n in t.shape)
        hasher.update(f"\n{name}:{t.dtype}:{shape}:{flat.numel() * flat.element_size()}\n".encode("ascii"))
        hasher.update(flat.view(torch.uint8).numpy())  # (a byte view: bfloat16 has no numpy dtype)
    blob = meta.to_bytes()
    hasher.update(f"\nmeta:{len(blob)}\n".encode("ascii"))
    hasher.update(blob)
    return hasher.hexdigest()


@dataclass(frozen=True, eq=False)
class StateSnapshot:
    """Host copies of the four tensors, their meta and the digest over both (reference
    ``model/state.py:133-160``). Made by :func:`snapshot`, loaded only through :func:`restore`."""

    h: Tensor
    q: Tensor
    age: Tensor
    pos: Tensor
    meta: StateMeta
    digest: str

    def __post_init__(self) -> None:
        if not isinstance(self.meta, StateMeta):
            raise TypeError(f"StateSnapshot.meta must be a StateMeta, got {type(self.meta).__name__}")
        if not isinstance(self.digest, str) or len(self.digest) != _HEX:
            raise ValueError(f"StateSnapshot.digest must be {_HEX} hex characters, got {self.digest!r}")
        try:
            bytes.fromhex(self.digest)
        except ValueError as exc:
            raise ValueError(f"StateSnapshot.digest is not hexadecimal: {self.digest!r}") from exc
        check_state(self.h, self.q, self.age, self.pos, "StateSnapshot")
        for name in FIELDS:
            t = getattr(self, name)
            if t.device.type != "cpu" or t.requires_grad:
                raise ValueError(f"StateSnapshot.{name} must be a CPU tensor without grad")


def _host_copy(t: Tensor) -> Tensor:
    return t.detach().contiguous().to(device="cpu", copy=True)


def snapshot(state: tuple[Tensor, Tensor, Tensor, Tensor], meta: StateMeta) -> StateSnapshot:
    """Host copies of ``state = (h, q, age, pos)`` bound to ``meta``. Always copies, so later in-place
    updates of the device state (the streaming calls) cannot alter the snapshot."""
    if not isinstance(meta, StateMeta):
        raise TypeError(f"snapshot needs a StateMeta, got {type(meta).__name__}")
    check_state(*state, where="snapshot")
    host = [_host_copy(t) for t in state]
    return StateSnapshot(*host, meta=meta, digest=state_digest(*host, meta))


def restore(snap: StateSnapshot, expected: StateMeta, device: torch.device | str) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """``(h, q, age, pos)`` of ``snap`` on ``device`` after verification against ``expected``: tenant,
    model version, schema version, then the digest, then the expiry of the snapshot's own (now verified)
    meta against ``time.time()``; ``expected.expires_at`` is the caller's own value and is not compared.
    Anything but a :class:`StateSnapshot` is refused: tensors are never loaded because their shapes fit."""
    if not isinstance(snap, StateSnapshot):
        raise TypeError(f"restore accepts a StateSnapshot, got {type(snap).__name__}")
    if not isinstance(expected, StateMeta):
        raise TypeError(f"restore needs the expected StateMeta, got {type(expected).__name__}")
    found = snap.meta
    if found.tenant_id != expected.tenant_id:
        raise TenantMismatch(f"snapshot belongs to tenant {found.tenant_id!r}, expected {expected.tenant_id!r}")
    if found.model_version != expected.model_version:
        raise VersionMismatch(f"snapshot of model version {found.model_version!r}, expected {expected.model_version!r}")
    if found.state_schema_version != expected.state_schema_version:
        raise SchemaMismatch(f"snapshot of state schema {found.state_schema_version}, expected {expected.state_schema_version}")
    actual = state_digest(snap.h, snap.q, snap.age, snap.pos, found)
    if not hmac.compare_digest(actual, snap.digest):
        raise IntegrityError(f"digest {snap.digest[:16]}... does not match the snapshot's tensors and meta ({actual[:16]}...)")
    if found.expires_at is not None and time.time() >= found.expires_at:
        raise StateExpired(f"snapshot expired at {found.expires_at:.3f}")
    dev = torch.device(device)
    return tuple(getattr(snap, name).to(device=dev, copy=True) for name in FIELDS)


def pack_cell_state(state: tuple[Tensor, Tensor, Tensor, Tensor]) -> dict[str, Tensor]:
    """The checkpoint's ``carried_state`` entry: detached contiguous host copies keyed ``h q age pos``."""
    check_state(*state, where="pack_cell_state")
    return {name: _host_copy(t) for name, t in zip(FIELDS, state, strict=True)}


def unpack_cell_state(payload: Mapping[str, Any], device: torch.device | str) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """What :func:`pack_cell_state` (or the reference's) wrote, on ``device``, with the layout checked again;
    exactly the four keys, tensors only."""
    if not isinstance(payload, Mapping):
        raise TypeError(f"carried cell state must be a mapping of tensors, got {type(payload).__name__}")
    missing = [n for n in FIELDS if n not in payload]
    unknown = sorted(n for n in payload if n not in FIELDS)
    if missing or unknown:
        raise ValueError(f"carried cell state must hold exactly {FIELDS}: missing {missing}, unknown {unknown}")
    for name in FIELDS:
        if not isinstance(payload[name], Tensor):
            raise TypeError(f"carried cell state {name!r} must be a tensor, got {type(payload[name]).__name__}")
    dev = torch.device(device)
    state = tuple(payload[name].to(device=dev) for name in FIELDS)
    check_state(*state, where="carried cell state")
    return state
