"""ctypes binding of ``libhsn_window_b200.so`` (``include/hsn_window_b200.h``).

Import never initialises CUDA and never builds anything; :func:`library` loads the shared object
on first use and raises if it is missing: there is no CPU or PyTorch fallback on this path.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_void_p
from functools import lru_cache
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
LIBRARY = PACKAGE / "lib" / "libhsn_window_b200.so"

HSN_WIN_POINTERS, HSN_WIN_INTS, HSN_WIN_FLOATS = 48, 32, 8
OK, E_ARG, E_UNSUPPORTED, E_CUDA, E_NAME, E_STATE = 0, -1, -2, -3, -4, -5


class HsnWinArgs(Structure):
    """The launch descriptor of the kernels launched by name (544 bytes, the reference's)."""

    _fields_ = [
        ("p", c_void_p * HSN_WIN_POINTERS),
        ("i", c_int32 * HSN_WIN_INTS),
        ("f", c_float * HSN_WIN_FLOATS),
    ]


HSN_TR_ROWS, HSN_TR_TENSORS, HSN_TR_INTS, HSN_TR_FLOATS, HSN_TR_DOUBLES, HSN_TR_COEFS, HSN_TR_UNITS = 4, 40, 8, 8, 2, 6, 64


class HsnTrainArgs(Structure):
    """The launch descriptor of the trainer kernels (``include/hsn_trainer_b200.h``; 3760 bytes, the
    reference's ``kernels/include/hsn_trainer_launch.h``)."""

    _fields_ = [
        ("p", (c_void_p * HSN_TR_TENSORS) * HSN_TR_ROWS),
        ("end", c_int64 * HSN_TR_TENSORS),
        ("g", c_double * HSN_TR_DOUBLES),
        ("i", c_int32 * HSN_TR_INTS),
        ("f", c_float * HSN_TR_FLOATS),
        ("u", (c_float * HSN_TR_UNITS) * HSN_TR_COEFS),
    ]


class HsnwExchange(Structure):
    """``include/hsn_trainer_b200.h``: the fused gradient exchange and AdamW step of one rank."""

    _fields_ = [
        ("world", c_int32), ("rank", c_int32), ("average", c_int32), ("weight_decay_on", c_int32), ("shard", c_int64),
        ("grads", c_void_p * 8), ("params", c_void_p * 8), ("exp_avg", c_void_p), ("exp_avg_sq", c_void_p),
        ("f", c_float * HSN_TR_FLOATS),
    ]  # fmt: skip


MODEL_INTS = ("N", "d", "K", "H", "M", "D", "S", "dc", "prod_bf16", "probes", "age_max", "phases_only")
MODEL_FLOATS = ("lambda_cost", "cell_overhead", "shared_cost", "limit", "norm_eps", "cand_eps")
MODEL_POINTERS = (
    "s_w1zc_t", "f_w1q_t", "f_b1", "f_w2_t", "f_b2", "score_w_t", "score_b", "v_t", "wout_t", "gate_t",
    "gate_b", "norm_w", "cand_w", "w1", "b1", "w2", "b2", "pad_src", "edge_w", "cost",
    "umma_w1", "umma_gate", "umma_w2", "umma_bw_w2", "umma_bw_w1", "umma_bw_gate", "rows_bank", "rows_front", "rows_bank_bw",
)  # fmt: skip


class HsnwModel(Structure):
    _fields_ = (
        [(n, c_int32) for n in MODEL_INTS]
        + [(n, c_float) for n in MODEL_FLOATS]
        + [(n, c_void_p) for n in MODEL_POINTERS]
    )


FORWARD_POINTERS = (
    "z", "ctx", "scalars", "reset", "h0", "q0", "age0", "pos", "tape_h", "tape_q", "tape_age", "cells",
    "units", "valid", "refreshed", "theta", "h_sel", "qs", "h_max", "rec_c", "rec_b", "rec_h_old", "rec_y",
    "rec_gate_pre", "rec_m", "rec_rms", "rec_hidden", "logits", "us", "scratch",
)  # fmt: skip


class HsnwForward(Structure):
    _fields_ = (
        [(n, c_int32) for n in ("B", "T", "tape_state", "forced")]
        + [(n, c_void_p) for n in FORWARD_POINTERS]
        + [("scratch_bytes", c_int64)]
    )


BACKWARD_POINTERS = (
    "c", "b", "h_old", "y", "gate_pre", "m", "rms", "hidden", "cells", "units", "valid", "reset",
    "d_q_pre", "d_q_post", "d_h_sel", "dc", "db", "A", "R", "scratch",
)  # fmt: skip


class HsnwBackward(Structure):
    _fields_ = (
        [(n, c_int32) for n in ("B", "T", "full_cut", "pad_")]
        + [(n, c_void_p) for n in BACKWARD_POINTERS]
        + [("scratch_bytes", c_int64)]
    )


PROLOGUE_INTS = ("B", "T", "V", "d", "H", "dc", "N", "S", "prod_bf16", "position_mode", "ema_per_row", "bos")
PROLOGUE_FLOATS = ("budget_frac", "round_frac", "n_context", "unroll")
PROLOGUE_POINTERS = (
    "byte_emb", "enc_w1", "enc_b1", "enc_w2", "enc_b2", "ctx_emb", "byte_codes", "cell_addresses", "ema_utility",
    "ema_selected", "tokens", "ctx_ids", "reset", "pos0", "prev_tokens", "z", "ctx", "scalars", "positions", "scratch",
)  # fmt: skip


class HsnwDecoder(Structure):
    _fields_ = [(n, c_int32) for n in ("d_q", "d_u", "H", "V", "prod_bf16", "reserved")] + [
        (n, c_void_p) for n in ("w1", "b1", "w2", "b2")
    ]


class HsnwUnits(Structure):
    _fields_ = [(n, c_int32) for n in ("n_units", "d_in", "hidden", "d_out", "prod_bf16", "reserved")] + [
        (n, c_void_p) for n in ("w1", "b1", "w2", "b2")
    ]


class HsnwScorer(Structure):
    _fields_ = [(n, c_int32) for n in ("d", "n_cells", "n_units", "n_scalars", "prod_bf16")] + [("age_max", c_float)] + [
        (n, c_void_p) for n in ("weight", "bias")
    ]


class HsnwTail(Structure):
    _fields_ = [("d", c_int32), ("prod_bf16", c_int32), ("norm_eps", c_float), ("reserved", c_int32), ("w_out", c_void_p), ("norm_weight", c_void_p)]  # fmt: skip


class HsnwGate(Structure):
    _fields_ = [("d", c_int32), ("prod_bf16", c_int32), ("norm_eps", c_float), ("reserved", c_int32), ("norm_weight", c_void_p),
                ("gate_w", c_void_p), ("gate_b", c_void_p)]  # fmt: skip


class HsnwMessages(Structure):
    _fields_ = [(n, c_int32) for n in ("d", "n_cells", "degree", "k", "prod_bf16", "reserved")] + [(n, c_void_p) for n in ("v_w", "edge_w", "pad_src")]


class HsnwPrologue(Structure):
    _fields_ = (
        [(n, c_int32) for n in PROLOGUE_INTS]
        + [(n, c_float) for n in PROLOGUE_FLOATS]
        + [(n, c_void_p) for n in PROLOGUE_POINTERS]
        + [("scratch_bytes", c_int64)]
    )


#: Every symbol ``include/hsn_window_b200.h`` and ``include/hsn_trainer_b200.h`` declare: (restype, argtypes).
SYMBOLS: dict[str, tuple[object, list[object]]] = {
    "hsnw_version": (c_int, []),
    "hsnw_last_error": (c_char_p, []),
    "hsnw_last_path": (c_char_p, []),
    "hsnw_prepare": (c_int, [c_int]),
    "hsnw_prepared": (c_int, [c_int]),
    "hsnw_sm_count": (c_int, [c_int]),
    "hsnw_launch": (c_int, [c_char_p, POINTER(HsnWinArgs), c_int64, c_int, c_int, c_void_p]),
    "hsnw_loop": (
        c_int,
        [POINTER(c_char_p), c_int, POINTER(c_int64), POINTER(c_int), POINTER(c_int), POINTER(HsnWinArgs),
         c_int64, c_int, c_void_p],
    ),  # fmt: skip
    "hsnw_launch_shape": (
        c_int, [c_char_p, POINTER(HsnWinArgs), POINTER(c_int64), POINTER(c_int), POINTER(c_int)]
    ),
    "hsnw_forward_scratch_bytes": (c_int64, [POINTER(HsnwModel), c_int32, c_int32]),
    "hsnw_window_forward": (c_int, [POINTER(HsnwModel), POINTER(HsnwForward), c_void_p]),
    "hsnw_stream_step": (c_int, [POINTER(HsnwModel), POINTER(HsnwForward), c_void_p]),
    "hsnw_stream_continue": (c_int, [POINTER(HsnwModel), POINTER(HsnwForward), c_void_p]),
    "hsnw_backward_scratch_bytes": (c_int64, [POINTER(HsnwModel), c_int32, c_int32]),
    "hsnw_window_backward": (c_int, [POINTER(HsnwModel), POINTER(HsnwBackward), c_void_p]),
    "hsnw_static_scratch_bytes": (c_int64, []),
    "hsnw_window_backward_static": (c_int, [POINTER(HsnwModel), POINTER(HsnwBackward), c_void_p]),
    "hsnw_front_projection": (c_int, [POINTER(HsnwModel), c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "hsnw_selftest_wait_timeout": (c_int, [c_void_p, c_void_p]),
    "hsnw_prologue_scratch_bytes": (c_int64, [POINTER(HsnwPrologue)]),
    "hsnw_window_prologue": (c_int, [POINTER(HsnwPrologue), c_void_p]),
    "hsnw_decode_scratch_bytes": (c_int64, [POINTER(HsnwDecoder), c_int64]),
    "hsnw_window_decode": (c_int, [POINTER(HsnwDecoder), c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p]),
    "hsnw_scorer_scratch_bytes": (c_int64, [POINTER(HsnwScorer), c_int64, c_int]),
    "hsnw_scorer_logits": (c_int, [POINTER(HsnwScorer), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                   c_int64, c_void_p]),
    "hsnw_scorer_logits_backward": (c_int, [POINTER(HsnwScorer), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
                                            c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "hsnw_messages_scratch_bytes": (c_int64, [POINTER(HsnwMessages), c_int64]),
    "hsnw_messages_forward": (c_int, [POINTER(HsnwMessages), c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "hsnw_messages_backward": (c_int, [POINTER(HsnwMessages), c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_int64, c_void_p]),
    "hsnw_gate_scratch_bytes": (c_int64, [POINTER(HsnwGate), c_int64, c_int]),
    "hsnw_gate_forward": (c_int, [POINTER(HsnwGate), c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "hsnw_gate_backward": (c_int, [POINTER(HsnwGate), c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_int64, c_void_p]),
    "hsnw_tail_scratch_bytes": (c_int64, [POINTER(HsnwTail), c_int64]),
    "hsnw_tail_forward": (c_int, [POINTER(HsnwTail), c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "hsnw_tail_backward": (c_int, [POINTER(HsnwTail), c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_int64, c_void_p]),
    "hsnw_units_scratch_bytes": (c_int64, [POINTER(HsnwUnits), c_int64, c_int]),
    "hsnw_units_forward": (c_int, [POINTER(HsnwUnits), c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "hsnw_units_backward": (c_int, [POINTER(HsnwUnits), c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "hsnw_exchange_adamw": (c_int, [POINTER(HsnwExchange), c_void_p]),
    "hsnw_launch_table": (c_int, [c_char_p, POINTER(HsnTrainArgs), c_void_p]),
    "hsnw_profile_begin": (c_int, []),
    "hsnw_profile_kinds": (c_int, []),
    "hsnw_profile_kind_name": (c_char_p, [c_int]),
    "hsnw_profile_end": (c_int, [POINTER(c_double), POINTER(c_int64), c_int]),
}


class WindowKernelError(RuntimeError):
    """An entry point of the library returned an error code."""

    def __init__(self, code: int, message: str) -> None:
        super().__init__(f"hsn_window_b200: {message} (code {code})")
        self.code = code


def available() -> bool:
    """Artifact presence only: never initialises CUDA or loads the library."""
    return LIBRARY.is_file()


@lru_cache(maxsize=1)
def library() -> ctypes.CDLL:
    if not available():
        raise RuntimeError(
            f"{LIBRARY} is missing: build it with `python -m hsn_b200.build`. The window path has no "
            "CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(str(LIBRARY))
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def check(code: int) -> None:
    if code != OK:
        raise WindowKernelError(code, library().hsnw_last_error().decode())
