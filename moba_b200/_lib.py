"""ctypes binding of libmoba_b200.so (the C ABI declared in include/moba_b200.h).

The library is built in-tree by ``python moba_b200/build.py``. There is no fallback: if the shared
library is missing, importing this module raises.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmoba_b200.so")

DTYPE_BF16, DTYPE_F16, DTYPE_F32 = 0, 1, 2
HEAD_DIM = 128
TILE = 128


class PlanInfo(ctypes.Structure):
    """Mirror of ``moba_plan_info``."""

    _fields_ = [
        ("batch", ctypes.c_int32),
        ("chunk_size", ctypes.c_int32),
        ("topk", ctypes.c_int32),
        ("kk", ctypes.c_int32),
        ("total_tokens", ctypes.c_int32),
        ("n_chunks", ctypes.c_int32),
        ("n_filtered", ctypes.c_int32),
        ("n_qtiles", ctypes.c_int32),
        ("max_cand", ctypes.c_int32),
        ("max_seq_chunks", ctypes.c_int32),
        ("rows_per_head", ctypes.c_int64),
        ("cand_per_head", ctypes.c_int64),
        ("max_work_tiles_per_head", ctypes.c_int64),
        ("off_chunk_start", ctypes.c_int32),
        ("off_chunk_seq_first", ctypes.c_int32),
        ("off_chunk_seq_last", ctypes.c_int32),
        ("off_qtile_chunk", ctypes.c_int32),
        ("off_qtile_start", ctypes.c_int32),
        ("off_qtile_cand_off", ctypes.c_int32),
        ("off_chunk_qtile_first", ctypes.c_int32),
        ("meta_ints", ctypes.c_int32),
    ]


class KvLayout(ctypes.Structure):
    """Mirror of ``moba_kv_layout``."""

    _fields_ = [
        ("kv_heads", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("stride_s", ctypes.c_int64),
        ("stride_h", ctypes.c_int64),
    ]


_P = ctypes.c_void_p
_I32 = ctypes.c_int32
_I64 = ctypes.c_int64
_F32 = ctypes.c_float
_INFO = ctypes.POINTER(PlanInfo)
_KV = ctypes.POINTER(KvLayout)      # None passes NULL: K / V laid out like q

# symbol -> (restype, argtypes); must list every function include/moba_b200.h declares
SIGNATURES = {
    "moba_version": (ctypes.c_int, []),
    "moba_last_error_string": (ctypes.c_char_p, []),
    "moba_plan_sizes": (ctypes.c_int, [_P, _I32, _I32, _I32, _INFO]),
    "moba_plan_fill": (ctypes.c_int, [_P, _I32, _I32, _I32, _INFO, _P]),
    "moba_pool_ws_floats": (_I64, [_INFO, _I32]),
    "moba_pool_keys": (ctypes.c_int, [_P, _I32, _I32, _I64, _I64, _INFO, _P, _P, _P, _I32, _P]),
    "moba_pool_keys_static_max_floats": (_I64, []),
    "moba_pool_keys_static": (ctypes.c_int, [_P, _I32, _I32, _I64, _I64, _INFO, _P, _P, _I32, _P]),
    "moba_gate_topk": (ctypes.c_int, [_P, _I32, _I32, _I64, _I64, _P, _I32, _INFO, _P, _P, _P, _P, _P, _I32, _P]),
    "moba_build_lists": (ctypes.c_int, [_I32, _INFO, _P, _P, _P, _P, _P, _P, _P, _P, _I32, _P]),
    "moba_tile_records": (ctypes.c_int, [_I32, _INFO, _P, _P, _P, _P, _I32, _P]),
    "moba_attn_fwd": (ctypes.c_int, [_P, _P, _P, _I32, _I32, _I64, _I64, _KV, _INFO, _P, _P, _P, _P, _P, _P, _P, _P,
                                     _P, _I32, _F32, _P, _I32, _P]),
    "moba_merge_fwd": (ctypes.c_int, [_P, _P, _I32, _I32, _INFO, _P, _P, _P, _I32, _P]),
    "moba_bwd_delta": (ctypes.c_int, [_P, _P, _I32, _I32, _I64, _P, _I32, _P]),
    "moba_gather_rows": (ctypes.c_int, [_P, _P, _P, _P, _I32, _I32, _I64, _I64, _INFO, _P, _P, _P, _P, _P, _P, _P, _P,
                                        _I32, _P]),
    "moba_attn_bwd_dkdv": (ctypes.c_int, [_P, _P, _P, _P, _I32, _I32, _I64, _I64, _KV, _INFO, _P, _P, _P, _P, _P, _P,
                                          _P, _P, _P, _P, _I32, _F32, _P, _I32, _P]),
    "moba_attn_bwd_dq": (ctypes.c_int, [_P, _P, _P, _P, _I32, _I32, _I64, _I64, _KV, _INFO, _P, _P, _P, _P, _P, _P, _P,
                                        _P, _P, _P, _P, _P, _P, _I32, _F32, _P, _I32, _P]),
    "moba_memcpy_2d": (ctypes.c_int, [_P, _I64, _P, _I64, _I64, _I64, _I32, _I32, _P]),
    "moba_merge_dq": (ctypes.c_int, [_P, _I32, _I32, _INFO, _P, _P, _P, _I32, _P]),
    "moba_decode_ws_floats": (_I64, [_I32, _I32, _I32, _I32, _I32]),
    "moba_decode_attn": (ctypes.c_int, [_P, _P, _P, _I32, _I32, _I32, _I32, _I32, _I32, _I64, _I64, _I64, _I64, _I64,
                                        ctypes.c_float, _P, _P, _P, _I32, _P]),
    "moba_check_status": (ctypes.c_int, [_P, _I32, _P]),
    "moba_selftest_umma": (ctypes.c_int, [_I32, _P, _P, _P, _I32, _P, _I32, _P]),
    "moba_selftest_umma_gather": (ctypes.c_int, [_I32, _P, _I32, _P, _P, _P, _I32, _P, _I32, _P]),
    "moba_selftest_umma_pair": (ctypes.c_int, [_P, _P, _P, _P, _P, _I32, _P, _I32, _P]),
    "moba_selftest_wait_timeout": (ctypes.c_int, [_I64, _I32, _P, _I32, _P]),
}


class MobaError(RuntimeError):
    """A non-zero return from the C ABI."""

    def __init__(self, fn, code, msg):
        super().__init__(f"{fn} failed with code {code}: {msg}")
        self.code = code


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python moba_b200/build.py` (needs nvcc). "
            "moba_b200 has no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(fn_name, code):
    if code != 0:
        raise MobaError(fn_name, code, lib.moba_last_error_string().decode("utf-8", "replace"))


def call(fn_name, *args):
    """Call a status-returning entry point and raise MobaError on a non-zero return."""
    check(fn_name, getattr(lib, fn_name)(*args))
