"""ctypes binding of the C-ABI library (include/foscar_b200.h).

The library is the product's only compute path. Loading fails loudly: there is no CPU or
PyTorch fallback for any operation.
"""
from __future__ import annotations

import ctypes as C
import os

from . import _build

ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_TOO_LARGE = -1, -2, -3
ERR_SCRATCH_TOO_SMALL = -4
STATIC_SCRATCH_BYTES = 8 << 20
STATUS_BITS = {0x1: "slot outside the cache", 0x2: "page id outside the pool",
               0x4: "output row outside the buffer", 0x8: "bad sequence length",
               0x10: "device wait timed out"}
WORK_WORDS = 8
STATUS_TIMEOUT = 0x10


def tile_tokens(bits: int, head_dim: int) -> int:
    """Tokens per sequence tile of the decode kernel's build for (bits, head_dim)."""
    n = load().fq_tile_tokens(bits, head_dim)
    if n < 0:
        check(n, "tile_tokens")
    return int(n)


def ctas_per_sm(bits: int, head_dim: int) -> int:
    """CTAs of the decode kernel's build for (bits, head_dim) that share an SM (1 or 2)."""
    n = load().fq_ctas_per_sm(bits, head_dim)
    if n < 0:
        check(n, "ctas_per_sm")
    return int(n)


def piece_overhead(bits: int, head_dim: int) -> int:
    """Fixed cost of a work piece in tile units, as the balanced planner counts it."""
    n = load().fq_piece_overhead(bits, head_dim)
    if n < 0:
        check(n, "piece_overhead")
    return int(n)


class Pools(C.Structure):
    _fields_ = [("bits", C.c_int32), ("head_dim", C.c_int32), ("num_kv_heads", C.c_int32),
                ("k_groups", C.c_int32), ("scale_bf16", C.c_int32), ("num_pages", C.c_int32),
                ("k_channel_group", C.c_int32), ("reserved", C.c_int32),
                ("k_codes", C.c_void_p), ("v_codes", C.c_void_p), ("scales", C.c_void_p),
                ("v_page_max", C.c_void_p), ("v_max_hist", C.c_void_p)]


class DecodeArgs(C.Structure):
    _fields_ = [("batch", C.c_int32), ("num_qo_heads", C.c_int32), ("out_dtype", C.c_int32),
                ("kv_splits", C.c_int32), ("max_splits", C.c_int32), ("num_work", C.c_int32),
                ("max_ctas", C.c_int32), ("flags", C.c_int32),
                ("sm_scale", C.c_float), ("o_scale", C.c_float),
                ("worklist", C.c_void_p), ("seq_lens", C.c_void_p), ("page_table", C.c_void_p),
                ("table_offsets", C.c_void_p), ("table_len", C.c_int64), ("q", C.c_void_p),
                ("q_descale", C.c_void_p), ("q_descale_stride_b", C.c_int64),
                ("q_descale_stride_h", C.c_int64), ("out", C.c_void_p), ("lse", C.c_void_p),
                ("o_partial", C.c_void_p), ("l_partial", C.c_void_p), ("m_partial", C.c_void_p),
                ("status", C.c_void_p), ("unit_counters", C.c_void_p),
                ("split_counts", C.c_void_p), ("wait_budget_cycles", C.c_int64),
                ("q_len", C.c_int32), ("reserved", C.c_int32)]


_P = C.c_void_p
_I32, _I64, _F32 = C.c_int32, C.c_int64, C.c_float
_PROTOTYPES = {
    "fq_version": (C.c_char_p, []),
    "fq_error_string": (C.c_char_p, [C.c_int]),
    "fq_append": (C.c_int, [C.POINTER(Pools), _P, _P, _I64, _I64, _P, _I32, _I32, _I32, _P, _P]),
    "fq_append_quantized": (C.c_int, [C.POINTER(Pools), _P, _P, _P, _P, _P, _P, _P, _I32, _P, _P]),
    "fq_append_page_groups": (C.c_int, [C.POINTER(Pools), _P, _P, _I64, _I64, _P, _P, _I32, _P,
                                        _P]),
    "fq_append_quantized_page_groups": (C.c_int, [C.POINTER(Pools), _P, _P, _P, _P, _P, _P, _P, _P,
                                                  _I32, _P, _P]),
    "fq_dequantize": (C.c_int, [C.POINTER(Pools), _P, _P, _I64, _I64, _I64, _P, _P, _I32, _P, _P,
                                _I32, _I32, _P, _P]),
    "fq_recount_vmax": (C.c_int, [C.POINTER(Pools), _P]),
    "fq_decode": (C.c_int, [C.POINTER(Pools), C.POINTER(DecodeArgs), _P]),
    "fq_decode_split_static": (C.c_int, [C.POINTER(Pools), C.POINTER(DecodeArgs), _P]),
    "fq_merge": (C.c_int, [_P, _P, _P, _P, _I32, _I32, _I32, _I32, _I32, _I32, _F32, _P, _I32,
                           _P, _P]),
    "fq_merge_states": (C.c_int, [_P, _P, _I32, _I32, _I32, _I32, _P, _I32, _P, _I64, _I64, _P]),
    "fq_exchange_bytes": (_I64, [_I32, _I32, _I32, _I32]),
    "fq_exchange_merge": (C.c_int, [_P, _I32, _I32, _P, _P, _I32, _I32, _I32, _I64, _P, _I32, _P,
                                    _I64, _P, _P]),
    "fq_plan_splits": (C.c_int, [_I32, _I32, _I32, _I32, _I32, _I32, _I32]),
    "fq_plan_worklist": (C.c_int, [_P, _I32, _I32, _I32, _I32, _I32, _P, _I32, _P, _I32, _I32]),
    "fq_workspace_bytes": (_I64, [_I32, _I32, _I32, _I32]),
    "fq_worklist_words": (_I64, [_I32, _I32, _I32, _I32]),
    "fq_worklist_attach_requests": (C.c_int, [_P, _I64, _P, _P, _I32]),
    "fq_umma_selftest": (C.c_int, [_I32, _P, _P, _P, _P, _P, _P, _P, _P]),
    "fq_ctas_per_sm": (C.c_int, [_I32, _I32]),
    "fq_tile_tokens": (C.c_int, [_I32, _I32]),
    "fq_piece_overhead": (C.c_int, [_I32, _I32]),
    "fq_wait_selftest": (C.c_int, [_I64, _P, _P, _P]),
}
EXPORTS = tuple(_PROTOTYPES)

_lib = None


def library_path() -> str:
    """The library to load: the in-tree build, or FOSCAR_B200_LIB (a diagnostic build)."""
    return os.environ.get("FOSCAR_B200_LIB") or _build.LIB_PATH


def load():
    """The loaded library. Raises RuntimeError when it is missing or lacks a symbol."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"the CUDA extension {path} is not built; run `python -m foscar_b200._build` "
            f"(needs nvcc). foscar_b200 has no CPU or PyTorch fallback")
    lib = C.CDLL(path)
    for name, (res, args) in _PROTOTYPES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            raise RuntimeError(f"{path} does not export {name}; rebuild it") from None
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(code: int, what: str) -> None:
    """Raise for a non-zero return code of a C-ABI call."""
    if code == 0:
        return
    text = load().fq_error_string(code).decode()
    if code == ERR_UNSUPPORTED:
        raise NotImplementedError(f"{what}: {text}")
    if code in (ERR_BAD_ARG, ERR_TOO_LARGE, ERR_SCRATCH_TOO_SMALL):
        raise ValueError(f"{what}: {text}")
    raise RuntimeError(f"{what}: CUDA error {code}: {text}")


def describe_status(word: int) -> str:
    return ", ".join(text for bit, text in STATUS_BITS.items() if word & bit) or "ok"
