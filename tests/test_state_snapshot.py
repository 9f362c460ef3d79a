"""The carried state's snapshot and checkpoint formats (``hsn_b200/state.py``) against the reference's
own digests (``tests/golden/snapshot_*.npz``, written by ``CellGraphState.snapshot``) and its refusal
rules (reference ``tests/test_p1_3_state.py:169-278``)."""

from __future__ import annotations

import time
from dataclasses import replace

import numpy as np
import pytest
import torch

from conftest import load_golden
from hsn_b200 import state as S


def _case(name: str):
    z = load_golden(f"snapshot_{name}")
    bf = str(z["dtype"]) == "torch.bfloat16"
    as_t = (lambda a: torch.from_numpy(a.copy()).view(torch.bfloat16)) if bf else (lambda a: torch.from_numpy(a.copy()))
    tensors = (as_t(z["h"]), as_t(z["q"]), torch.from_numpy(z["age"].copy()), torch.from_numpy(z["pos"].copy()))
    expires = float(z["expires_at"])
    meta = S.StateMeta(str(z["model_version"]), int(z["state_schema_version"]), str(z["tenant_id"]),
                       None if np.isnan(expires) else expires)  # fmt: skip
    return tensors, meta, str(z["digest"]), str(z["meta_json"])


@pytest.mark.parametrize("name", ["f32", "bf16"])
def test_digest_and_meta_bytes_are_the_references(name: str) -> None:
    tensors, meta, digest, meta_json = _case(name)
    assert meta.to_bytes() == meta_json.encode("utf-8")
    assert S.state_digest(*tensors, meta) == digest
    snap = S.snapshot(tensors, meta)
    assert snap.digest == digest
    # a snapshot written by the reference (its tensors, meta and digest) restores here
    theirs = S.StateSnapshot(*tensors, meta=meta, digest=digest)
    back = S.restore(theirs, meta, "cpu")
    for got, want in zip(back, tensors):
        assert got.dtype == want.dtype and torch.equal(got, want)
    # the same bytes under another dtype or shape do not verify
    h = tensors[0]
    assert S.state_digest(h.reshape(h.shape[0], h.shape[2], h.shape[1]).contiguous(), *tensors[1:], meta) != digest


def test_snapshot_copies_and_restore_refuses_in_order() -> None:
    tensors, meta, _, _ = _case("f32")
    live = tuple(t.clone() for t in tensors)
    snap = S.snapshot(live, meta)
    live[0].add_(1.0)   # the live state moves on; the snapshot does not
    assert torch.equal(snap.h, tensors[0])
    assert S.snapshot(tensors, replace(meta, tenant_id="tenant-b")).digest != snap.digest
    assert S.snapshot(tensors, replace(meta, expires_at=time.time() + 60)).digest != snap.digest
    with pytest.raises(S.VersionMismatch):
        S.restore(snap, replace(meta, model_version="other"), "cpu")
    with pytest.raises(S.SchemaMismatch):
        S.restore(snap, replace(meta, state_schema_version=2), "cpu")
    with pytest.raises(S.TenantMismatch):   # the tenant is checked first
        S.restore(snap, replace(meta, tenant_id="tenant-b", model_version="other"), "cpu")
    for field, change in (("h", lambda t: t + 1e-3), ("age", lambda t: t + 1), ("pos", lambda t: t + 1)):
        with pytest.raises(S.IntegrityError):
            S.restore(replace(snap, **{field: change(getattr(snap, field))}), meta, "cpu")
    relabelled = replace(snap, meta=replace(meta, tenant_id="tenant-b"))   # a re-labelled snapshot keeps the old digest
    with pytest.raises(S.IntegrityError):
        S.restore(relabelled, replace(meta, tenant_id="tenant-b"), "cpu")
    flipped = ("0" if snap.digest[0] != "0" else "1") + snap.digest[1:]
    with pytest.raises(S.IntegrityError):
        S.restore(replace(snap, digest=flipped), meta, "cpu")
    # expiry is judged from the snapshot's own meta
    past = replace(meta, expires_at=time.time() - 1.0)
    with pytest.raises(S.StateExpired):
        S.restore(S.snapshot(tensors, past), past, "cpu")
    later = replace(meta, expires_at=time.time() + 3600.0)
    S.restore(S.snapshot(tensors, later), replace(later, expires_at=None), "cpu")
    S.restore(snap, past, "cpu")   # `snap` itself never expires
    with pytest.raises(TypeError):
        S.restore({"h": tensors[0]}, meta, "cpu")  # bare tensors are never loaded
    with pytest.raises(TypeError):
        S.snapshot(tensors, {"tenant_id": "tenant-a"})


def test_meta_and_layout_validation() -> None:
    with pytest.raises(ValueError):
        S.StateMeta("", 1, "t", None)
    with pytest.raises(ValueError):
        S.StateMeta("m", 0, "t", None)
    with pytest.raises(ValueError):
        S.StateMeta("m", True, "t", None)
    with pytest.raises(ValueError):
        S.StateMeta("m", 1, "t", float("inf"))
    assert S.StateMeta("m", 1, "t", 5).expires_at == 5.0
    h, q, age, pos = torch.zeros(2, 3, 4), torch.zeros(2, 4), torch.zeros(2, 3, dtype=torch.int64), torch.zeros(2, dtype=torch.int64)
    assert S.check_state(h, q, age, pos) == (2, 3, 4)
    for bad in ((h, q[:, :3], age, pos), (h, q.double(), age, pos), (h, q, age.int(), pos), (h, q, age, pos[:1]),
                (h.long(), q, age, pos), (h[0], q, age, pos)):  # fmt: skip
        with pytest.raises(ValueError):
            S.check_state(*bad)


def test_checkpoint_payload_round_trip() -> None:
    tensors, _, _, _ = _case("bf16")
    packed = S.pack_cell_state(tensors)
    assert tuple(packed) == S.FIELDS and all(t.device.type == "cpu" for t in packed.values())
    assert packed["h"].data_ptr() != tensors[0].data_ptr()
    back = S.unpack_cell_state(packed, "cpu")
    assert all(torch.equal(a, b) for a, b in zip(back, tensors))
    with pytest.raises(ValueError):
        S.unpack_cell_state({k: v for k, v in packed.items() if k != "pos"}, "cpu")
    with pytest.raises(ValueError):
        S.unpack_cell_state(dict(packed, extra=packed["h"]), "cpu")
    with pytest.raises(TypeError):
        S.unpack_cell_state(dict(packed, h=packed["h"].float().numpy()), "cpu")
    with pytest.raises(TypeError):
        S.unpack_cell_state([packed["h"]], "cpu")


@pytest.mark.gpu
def test_a_streaming_session_is_saved_and_resumed_bit_for_bit() -> None:
    """Stream four positions, snapshot the device state, stream four more; a second session restored from
    the snapshot (first call without the carried derived values) produces the same state and summaries."""
    from conftest import dev, synthetic_window
    from hsn_b200.window import WindowModel, window_forward

    rng = np.random.default_rng(4)
    B, T, N, d, K, H, M, D = 5, 8, 64, 32, 4, 128, 3, 2
    W, z, ctx, scalars, reset, state = synthetic_window(rng, B, T, N, d, K, H, M, D, 0.1)
    reset[:, 0] = False
    model = WindowModel.from_oracle_weights(W, device="cuda", prod="bf16")
    live = tuple(dev(s) for s in state)
    live[0].copy_(dev((rng.standard_normal(state[0].shape) * 0.3).astype(np.float32)))
    live[1].copy_(live[0].mean(dim=1))
    cut = lambda a, lo, hi: dev(np.ascontiguousarray(a[:, lo:hi]))  # noqa: E731
    first = window_forward(model, *(cut(a, 0, 4) for a in (z, ctx, scalars, reset)), live, record=False, tape_state=False)
    meta = S.StateMeta("hsn-b200-test", 1, "tenant-a", None)
    snap = S.snapshot(live, meta)
    second = window_forward(model, *(cut(a, 4, 8) for a in (z, ctx, scalars, reset)), live, record=False, tape_state=False,
                            out=first, carried=True)  # fmt: skip
    qs_live = second["qs"].clone()
    resumed = S.restore(snap, meta, "cuda")
    again = window_forward(model, *(cut(a, 4, 8) for a in (z, ctx, scalars, reset)), resumed, record=False, tape_state=False)
    assert torch.equal(again["qs"], qs_live)
    for a, b in zip(resumed, live):
        assert torch.equal(a, b)
    assert S.snapshot(resumed, meta).digest == S.snapshot(live, meta).digest != snap.digest
