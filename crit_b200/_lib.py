"""ctypes binding of libcrit_b200.so (include/crit_b200.h).  There is no fallback: without the library every call
raises."""
import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p
from pathlib import Path

LIBRARY = Path(__file__).resolve().parent / "_native" / "libcrit_b200.so"
ABI_VERSION = 3

KIND_16BIT, KIND_FP8, KIND_FP8_ROW, KIND_INT8, KIND_FP8_PAGE = range(5)
DTYPE_BF16, DTYPE_FP16, DTYPE_FP32 = range(3)


class AppendParams(Structure):
    _fields_ = [("keys", c_void_p), ("values", c_void_p), ("slots", c_void_p), ("key_pages", c_void_p),
                ("value_pages", c_void_p), ("key_scales", c_void_p), ("value_scales", c_void_p), ("status", c_void_p),
                ("tokens", c_int64), ("slots_total", c_int64), ("key_stride_token", c_int64), ("key_stride_head", c_int64),
                ("value_stride_token", c_int64), ("value_stride_head", c_int64),
                ("kv_heads", c_int32), ("head_dim", c_int32), ("value_dim", c_int32), ("page", c_int32),
                ("kind", c_int32), ("in_dtype", c_int32), ("page_dtype", c_int32),
                ("key_multiplier", c_float), ("value_multiplier", c_float)]


class GatherParams(Structure):
    _fields_ = [("pages", c_void_p), ("scales", c_void_p), ("table", c_void_p), ("slots", c_void_p), ("out", c_void_p),
                ("status", c_void_p), ("count", c_int64), ("slots_total", c_int64), ("kv_heads", c_int32), ("dim", c_int32), ("page", c_int32),
                ("kind", c_int32), ("page_dtype", c_int32), ("out_dtype", c_int32), ("multiplier", c_float)]


class SlotsParams(Structure):
    _fields_ = [("tables", c_void_p), ("rows", c_void_p), ("positions", c_void_p), ("capacity", c_void_p),
                ("slots", c_void_p), ("n", c_int64), ("table_stride", c_int64),
                ("table_width", c_int32), ("page", c_int32), ("dump", c_int32)]


class MoveParams(Structure):
    _fields_ = [("store", c_void_p), ("source", c_void_p), ("target", c_void_p), ("lists", c_int64), ("width", c_int64),
                ("slots", c_int64), ("row_bytes", c_int64), ("layers", c_int32), ("status", c_void_p)]


class CompactParams(Structure):
    _fields_ = [("tables", c_void_p), ("rows", c_void_p), ("starts", c_void_p), ("counts", c_void_p), ("firsts", c_void_p),
                ("blocks", c_void_p), ("out_tables", c_void_p), ("out_counts", c_void_p), ("out_firsts", c_void_p),
                ("out", c_void_p), ("lse", c_void_p), ("n_rows", c_int64), ("table_stride", c_int64),
                ("out_stride_token", c_int64), ("out_stride_head", c_int64), ("table_width", c_int32), ("columns", c_int32),
                ("blocks_k", c_int32), ("block_size", c_int32), ("page", c_int32), ("dump", c_int32), ("q_heads", c_int32),
                ("value_dim", c_int32), ("out_dtype", c_int32)]


class AttendParams(Structure):
    _fields_ = [("q", c_void_p), ("out", c_void_p), ("lse", c_void_p), ("key_pages", c_void_p),
                ("value_pages", c_void_p), ("key_scales", c_void_p), ("value_scales", c_void_p),
                ("tables", c_void_p), ("rows", c_void_p), ("starts", c_void_p), ("counts", c_void_p),
                ("firsts", c_void_p), ("offsets", c_void_p), ("workspace", c_void_p), ("status", c_void_p),
                ("workspace_floats", c_int64), ("slots", c_int64), ("q_stride_token", c_int64), ("q_stride_head", c_int64),
                ("out_stride_token", c_int64), ("out_stride_head", c_int64), ("table_stride", c_int64),
                ("n_rows", c_int32), ("columns", c_int32), ("partial_rows", c_int32),
                ("q_heads", c_int32), ("kv_heads", c_int32), ("head_dim", c_int32), ("value_dim", c_int32),
                ("page", c_int32), ("kind", c_int32), ("page_dtype", c_int32), ("q_dtype", c_int32),
                ("chunk", c_int32), ("max_splits", c_int32), ("flags", c_int32),
                ("scale", c_float), ("key_multiplier", c_float), ("value_multiplier", c_float),
                ("parents", c_void_p), ("sinks", c_void_p), ("sliding", c_int32),
                ("blocks_k", c_int32), ("block_size", c_int32), ("blocks", c_void_p)]


class MergeShardsParams(Structure):
    _fields_ = [("outs", c_void_p), ("lses", c_void_p), ("out", c_void_p), ("lse", c_void_p), ("n", c_int64),
                ("parts", c_int32), ("dim", c_int32), ("in_dtype", c_int32), ("out_dtype", c_int32)]


class PrefillParams(Structure):
    _fields_ = [("q", c_void_p), ("out", c_void_p), ("lse", c_void_p), ("key_pages", c_void_p),
                ("value_pages", c_void_p), ("key_scales", c_void_p), ("value_scales", c_void_p),
                ("table", c_void_p), ("position_ptr", c_void_p), ("status", c_void_p), ("position", c_int64), ("slots", c_int64),
                ("q_stride_token", c_int64), ("q_stride_head", c_int64), ("out_stride_token", c_int64),
                ("out_stride_head", c_int64), ("tokens", c_int32), ("q_heads", c_int32), ("kv_heads", c_int32),
                ("head_dim", c_int32), ("value_dim", c_int32), ("page", c_int32), ("kind", c_int32),
                ("page_dtype", c_int32), ("q_dtype", c_int32), ("flags", c_int32),
                ("scale", c_float), ("key_multiplier", c_float), ("value_multiplier", c_float),
                ("starts", c_void_p), ("positions", c_void_p), ("sequences", c_int32), ("table_stride", c_int32)]


class ExchangeParams(Structure):
    _fields_ = [("mine", c_void_p), ("peers", c_void_p), ("step", c_void_p), ("gathered", c_void_p), ("status", c_void_p),
                ("floats", c_int64), ("wait_ns", c_int64), ("world", c_int32), ("rank", c_int32)]


STRUCTS = (AppendParams, GatherParams, SlotsParams, AttendParams, MergeShardsParams, PrefillParams, ExchangeParams, MoveParams,
           CompactParams)

# name -> (restype, argtypes): every symbol include/crit_b200.h declares
SYMBOLS = {
    "crit_b200_append": (c_int, [POINTER(AppendParams), c_void_p]),
    "crit_b200_gather": (c_int, [POINTER(GatherParams), c_void_p]),
    "crit_b200_slots": (c_int, [POINTER(SlotsParams), c_void_p]),
    "crit_b200_attend_plan": (c_int, [c_int32] * 8 + [POINTER(c_int32)]),
    "crit_b200_decode": (c_int, [POINTER(AttendParams), c_void_p]),
    "crit_b200_merge": (c_int, [POINTER(AttendParams), c_void_p]),
    "crit_b200_attend": (c_int, [POINTER(AttendParams), c_void_p]),
    "crit_b200_attend_static": (c_int, [POINTER(AttendParams), c_void_p]),
    "crit_b200_merge_shards": (c_int, [POINTER(MergeShardsParams), c_void_p]),
    "crit_b200_move_rows": (c_int, [POINTER(MoveParams), c_void_p]),
    "crit_b200_compact_blocks": (c_int, [POINTER(CompactParams), c_void_p]),
    "crit_b200_prefill": (c_int, [POINTER(PrefillParams), c_void_p]),
    "crit_b200_shard_push": (c_int, [POINTER(ExchangeParams), c_void_p]),
    "crit_b200_shard_wait": (c_int, [POINTER(ExchangeParams), c_void_p]),
    "crit_b200_merge_push": (c_int, [POINTER(AttendParams), POINTER(ExchangeParams), c_void_p]),
    "crit_b200_wait_merge": (c_int, [POINTER(ExchangeParams), POINTER(MergeShardsParams), c_void_p]),
    "crit_b200_exchange_merge": (c_int, [POINTER(AttendParams), POINTER(ExchangeParams), POINTER(MergeShardsParams), c_void_p]),
    "crit_b200_exchange_bytes": (c_int64, [c_int32, c_int64]),
    "crit_b200_pager_create": (c_void_p, [c_int32]),
    "crit_b200_pager_destroy": (None, [c_void_p]),
    "crit_b200_pager_take": (c_int32, [c_void_p]),
    "crit_b200_pager_drop": (c_int32, [c_void_p, c_int32]),
    "crit_b200_pager_share": (c_int32, [c_void_p, c_int32]),
    "crit_b200_pager_refs": (c_int32, [c_void_p, c_int32]),
    "crit_b200_pager_free": (c_int32, [c_void_p]),
    "crit_b200_pager_floor": (c_int32, [c_void_p]),
    "crit_b200_pager_shared": (c_int32, [c_void_p]),
    "crit_b200_pager_grow": (c_int64, [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int64]),
    "crit_b200_abi_version": (c_int, []),
    "crit_b200_params_size": (c_int, [c_int32]),
    "crit_b200_error": (c_char_p, [c_int32]),
    "crit_b200_device_sms": (c_int, []),
}

_lib = None


def load():
    """The library, loaded once; raises when it is not built or its ABI is not this binding's."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIBRARY.exists():
        raise RuntimeError(f"crit_b200's native library is not built ({LIBRARY}): run `python -m crit_b200.build` "
                           "(nvcc for sm_100a); there is no CPU or torch fallback")
    lib = ctypes.CDLL(str(LIBRARY))
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = restype, argtypes
    if lib.crit_b200_abi_version() != ABI_VERSION:
        raise RuntimeError(f"libcrit_b200.so speaks ABI {lib.crit_b200_abi_version()}, this binding {ABI_VERSION}: rebuild")
    for which, struct in enumerate(STRUCTS):
        if lib.crit_b200_params_size(which) != ctypes.sizeof(struct):
            raise RuntimeError(f"{struct.__name__} is {ctypes.sizeof(struct)} bytes here and "
                               f"{lib.crit_b200_params_size(which)} in libcrit_b200.so: rebuild")
    _lib = lib
    return lib


def check(code, what):
    """0 passes; a negative code is a ValueError (the parameters), a positive one a RuntimeError (CUDA)."""
    if code == 0:
        return
    text = load().crit_b200_error(code).decode()
    if code < 0:
        raise ValueError(f"{what}: {text}")
    raise RuntimeError(f"{what}: CUDA error {code}: {text}")
