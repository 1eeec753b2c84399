"""ctypes binding of libkvq.so (the C ABI declared in include/kvq.h).

The library is the only compute path of this package: if it cannot be loaded
the import of any kernel entry point raises; there is no CPU or torch fallback.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

KVQ_OK = 0
KVQ_EINVAL = -1
KVQ_EUNSUPPORTED = -2
KVQ_ECUDA = -3
KVQ_EWORKSPACE = -4
KVQ_ELIMIT = -5

FMT_FP16, FMT_INT8, FMT_INT4 = 0, 1, 2
SCALE_STATIC, SCALE_DYNAMIC_PCT, SCALE_ASYM_MINMAX = 0, 1, 2
F_ADAPTIVE, F_MIXED_RESCUE, F_RESCUE_THR, F_UNPACKED, F_ADAPT_SKIP_K, F_ADAPT_SKIP_V = 1, 2, 4, 8, 16, 32

_i64, _i32, _vp, _f32 = C.c_int64, C.c_int32, C.c_void_p, C.c_float


class KvqAppendSide(C.Structure):
    _fields_ = [
        ("src", _vp), ("src_stride_b", _i64), ("src_stride_h", _i64), ("src_stride_t", _i64),
        ("payload", _vp), ("pay_stride_b", _i64), ("pay_stride_h", _i64), ("pay_stride_s", _i64),
        ("scale", _vp), ("zp", _vp), ("scale_f32", _vp),
        ("sc_stride_b", _i64), ("sc_stride_h", _i64), ("sc_stride_s", _i64),
        ("side", _vp), ("side_stride_b", _i64), ("side_stride_h", _i64), ("side_stride_s", _i64),
        ("static_scale", _vp), ("static_scale_is_f32", _i32), ("rescue_threshold", _vp),
    ]


class KvqAppendArgs(C.Structure):
    _fields_ = [
        ("format", _i32), ("policy", _i32), ("flags", _i32),
        ("B", _i32), ("Hkv", _i32), ("T", _i32), ("D", _i32), ("group_size", _i32),
        ("adaptive_margin", _f32), ("quantile", _f32),
        ("n_out", _i32), ("outlier_idx", _vp),
        ("write_pos", _i64), ("write_pos_dev", _vp), ("max_slots", _i64),
        ("k", KvqAppendSide), ("v", KvqAppendSide),
        ("rope_cos", _vp), ("rope_sin", _vp), ("rope_stride_b", _i64), ("rope_stride_t", _i64),
        ("rotary_dim", _i32), ("Hq", _i32),
        ("q_src", _vp), ("q_stride_b", _i64), ("q_stride_h", _i64), ("q_stride_t", _i64),
        ("q_out", _vp), ("qo_stride_b", _i64), ("qo_stride_h", _i64), ("qo_stride_t", _i64),
    ]


class KvqCacheSide(C.Structure):
    _fields_ = [
        ("payload", _vp), ("pay_stride_b", _i64), ("pay_stride_h", _i64), ("pay_stride_s", _i64),
        ("scale", _vp), ("zp", _vp),
        ("sc_stride_b", _i64), ("sc_stride_h", _i64), ("sc_stride_s", _i64),
        ("side", _vp), ("side_stride_b", _i64), ("side_stride_h", _i64), ("side_stride_s", _i64),
    ]


class KvqAttnArgs(C.Structure):
    _fields_ = [
        ("format", _i32), ("B", _i32), ("Hq", _i32), ("Hkv", _i32), ("D", _i32),
        ("group_size", _i32), ("max_ctx", _i32),
        ("q", _vp), ("q_stride_b", _i64), ("q_stride_h", _i64),
        ("inv_tau", _vp), ("sm_scale", _f32),
        ("k", KvqCacheSide), ("v", KvqCacheSide),
        ("n_out", _i32), ("outlier_idx", _vp),
        ("context_lens", _vp),
        ("splits", _i32), ("stages", _i32), ("fast_dequant", _i32), ("tail_tokens", _i32),
        ("workspace", _vp), ("workspace_bytes", C.c_size_t),
        ("out", _vp), ("out_stride_b", _i64), ("out_stride_h", _i64),
        ("q_chan_scale", _vp), ("qcs_stride_b", _i64), ("qcs_stride_h", _i64),
        ("part_o", _vp), ("part_m", _vp), ("part_l", _vp),
        ("part_o_stride", _i64), ("part_ml_stride", _i64),
    ]


class KvqCombineArgs(C.Structure):
    _fields_ = [
        ("P", _i32), ("B", _i32), ("Hq", _i32), ("D", _i32),
        ("part_o", _vp), ("part_m", _vp), ("part_l", _vp),
        ("out", _vp), ("out_stride_b", _i64), ("out_stride_h", _i64),
        ("part_o_stride", _i64), ("part_ml_stride", _i64), ("part_o_stride_p", _i64), ("part_ml_stride_p", _i64),
    ]


class KvqDequantArgs(C.Structure):
    _fields_ = [
        ("format", _i32), ("B", _i32), ("Hkv", _i32), ("S", _i32), ("D", _i32), ("group_size", _i32),
        ("n_out", _i32), ("outlier_idx", _vp),
        ("k", KvqCacheSide), ("v", KvqCacheSide),
        ("k_out", _vp), ("v_out", _vp),
        ("out_stride_b", _i64), ("out_stride_h", _i64), ("out_stride_s", _i64),
    ]


class KvqAbsmaxArgs(C.Structure):
    _fields_ = [
        ("B", _i32), ("H", _i32), ("S", _i32), ("D", _i32), ("group_size", _i32),
        ("x", _vp), ("stride_b", _i64), ("stride_h", _i64), ("stride_s", _i64),
        ("out", _vp),
    ]


class KvqKiviArgs(C.Structure):
    _fields_ = [
        ("bits", _i32), ("B", _i32), ("H", _i32), ("T", _i32), ("D", _i32), ("init_k_params", _i32),
        ("k_src", _vp), ("v_src", _vp), ("src_stride_b", _i64), ("src_stride_h", _i64), ("src_stride_t", _i64),
        ("k_payload", _vp), ("v_payload", _vp), ("pay_stride_b", _i64), ("pay_stride_h", _i64), ("pay_stride_s", _i64),
        ("k_scale", _vp), ("k_zp", _vp), ("v_scale", _vp), ("v_zp", _vp), ("vs_stride_b", _i64), ("vs_stride_h", _i64),
        ("write_pos", _i64), ("write_pos_dev", _vp), ("max_slots", _i64),
        ("k_out", _vp), ("v_out", _vp), ("out_stride_b", _i64), ("out_stride_h", _i64), ("out_stride_s", _i64),
        ("v_scale_h", _vp), ("v_zp_h", _vp),
        ("k_lo", _vp), ("k_hi", _vp), ("v_lo", _vp), ("v_hi", _vp),
    ]


class KvqQuantileArgs(C.Structure):
    _fields_ = [
        ("sorted", _vp), ("rows", _i64), ("n", _i32), ("q_lo", _f32), ("q_hi", _f32), ("out_lo", _vp), ("out_hi", _vp),
    ]


MAX_PEERS = 16


class KvqExchangeArgs(C.Structure):
    _fields_ = [
        ("B", _i32), ("Hq", _i32), ("D", _i32), ("splits", _i32),
        ("workspace", _vp), ("workspace_bytes", C.c_size_t),
        ("rank", _i32), ("world", _i32),
        ("peer_base", C.POINTER(_vp)),
        ("slot", _i32), ("slots", _i32),
        ("epoch", _vp), ("wait_ns", C.c_uint64), ("status", _vp),
        ("out", _vp), ("out_stride_b", _i64), ("out_stride_h", _i64),
        ("tail_attn", C.POINTER(KvqAttnArgs)),
    ]


# every symbol include/kvq.h declares: (name, restype, argtypes)
EXPORTS = (
    ("kvq_quantize_append", C.c_int, (C.POINTER(KvqAppendArgs), _vp)),
    ("kvq_decode_attn", C.c_int, (C.POINTER(KvqAttnArgs), _vp)),
    ("kvq_decode_attn_static", C.c_int, (C.POINTER(KvqAttnArgs), _vp)),
    ("kvq_decode_workspace_bytes", C.c_size_t, (_i32, _i32, _i32, _i32)),
    ("kvq_decode_pick_splits", _i32, (C.POINTER(KvqAttnArgs),)),
    ("kvq_lse_combine", C.c_int, (C.POINTER(KvqCombineArgs), _vp)),
    ("kvq_exchange_bytes", C.c_size_t, (_i32, _i32, _i32, _i32, _i32)),
    ("kvq_combine_exchange", C.c_int, (C.POINTER(KvqExchangeArgs), _vp)),
    ("kvq_kivi_append", C.c_int, (C.POINTER(KvqKiviArgs), _vp)),
    ("kvq_sorted_quantile", C.c_int, (C.POINTER(KvqQuantileArgs), _vp)),
    ("kvq_kivi_dequantize", C.c_int, (C.POINTER(KvqKiviArgs), _vp)),
    ("kvq_group_absmax", C.c_int, (C.POINTER(KvqAbsmaxArgs), _vp)),
    ("kvq_dequantize", C.c_int, (C.POINTER(KvqDequantArgs), _vp)),
    ("kvq_debug_error_flag", C.c_int, (C.c_int,)),
    ("kvq_selftest_division", C.c_int, (C.c_int, C.c_uint32, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64))),
    ("kvq_decode_kernel_kind", C.c_int, (C.POINTER(KvqAttnArgs),)),
    ("kvq_strerror", C.c_char_p, (C.c_int,)),
    ("kvq_last_cuda_error", C.c_int, ()),
    ("kvq_abi_version", C.c_int, ()),
    ("kvq_struct_size", C.c_size_t, (C.c_int,)),
)

ABI_VERSION = 5
# ids of kvq_struct_size, in the order of include/kvq.h
STRUCTS = (KvqAppendSide, KvqAppendArgs, KvqCacheSide, KvqAttnArgs, KvqCombineArgs, KvqDequantArgs, KvqKiviArgs,
           KvqAbsmaxArgs, KvqExchangeArgs, KvqQuantileArgs)

_LIB = None


class KvqError(RuntimeError):
    """A libkvq entry point returned a non-zero status."""

    def __init__(self, fn: str, code: int, text: str):
        super().__init__(f"{fn} failed: {text} (code {code})")
        self.code = code


def lib_path() -> str:
    """The library this process loads: `KVQ_LIBRARY` (a variant built with `build.py --out`), else the in-tree build."""
    return os.environ.get("KVQ_LIBRARY") or _build.LIB_PATH


def load():
    """Load libkvq.so (once).  Raises if the library is missing: there is no fallback."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing. Build it with `python -m llm_kvcache_quantization_b200.build` "
            "(needs nvcc); this package has no CPU or pure-torch fallback.")
    lib = C.CDLL(path)
    for name, restype, argtypes in EXPORTS:
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = list(argtypes)
    if lib.kvq_abi_version() != ABI_VERSION:
        raise ImportError(f"{path} has ABI version {lib.kvq_abi_version()}, this package binds version {ABI_VERSION}: "
                          "rebuild it with `python -m llm_kvcache_quantization_b200.build --force`")
    for i, st in enumerate(STRUCTS):
        if lib.kvq_struct_size(i) != C.sizeof(st):
            raise ImportError(f"{path}: struct {st.__name__} is {lib.kvq_struct_size(i)} bytes in the library, "
                              f"{C.sizeof(st)} in the binding")
    _LIB = lib
    return lib


def check(fn: str, code: int) -> None:
    if code == KVQ_OK:
        return
    lib = load()
    text = lib.kvq_strerror(code).decode()
    if code == KVQ_ECUDA:
        text += f" [cudaError {lib.kvq_last_cuda_error()}]"
    raise KvqError(fn, code, text)
