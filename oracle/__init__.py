"""CPU oracle of the paged KV-cache hot path: numpy/ctypes front of oracle.c.  TEST INFRASTRUCTURE ONLY.

Nothing in crit_b200 imports this package; the tests, the smoke check and the bench's CPU-baseline leg do, as the
checker.  Every function names the reference code (crit 0.21.0, path:line inside the reference project) it restates.

Parity status: pinned against the reference's own torch path through the fixtures under tests/golden/ (made by
tests/golden/make_golden.py, which imports the reference) and against the reference's E4M3 known-answer file.  The
per-(page, kv head) FP8 rule (quantize_pages) has no reference implementation: parity unpinned for that rule alone.
"""
import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "_ref" / "liboracle.so"

KINDS = {"bf16": 0, "fp16": 0, "fp32": 0, "fp8": 1, "fp8:row": 2, "int8": 3, "fp8:page": 4}


def build(force=False):
    """Compile oracle.c with gcc into oracle/_ref/liboracle.so (the Makefile's recipe)."""
    if force or not LIB.exists() or LIB.stat().st_mtime < (HERE / "oracle.c").stat().st_mtime:
        env = dict(os.environ)
        env.pop("CC", None)
        subprocess.run(["make", "-C", str(HERE), "-B"], check=True, capture_output=True, env=env)
    return LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(LIB))
        _lib.crit_oracle_e4m3_encode.restype = ctypes.c_uint8
        _lib.crit_oracle_e4m3_encode.argtypes = [ctypes.c_float]
        _lib.crit_oracle_e4m3_decode.restype = ctypes.c_float
        _lib.crit_oracle_e4m3_decode.argtypes = [ctypes.c_uint8]
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


# -- E4M3 ---------------------------------------------------------------------------------------------------------------
def e4m3_encode(x):
    """FP32 array -> E4M3FN bytes (RNE, saturating at 448).  ref: kernels/core/python/crit_kcore/formats.py:61-79."""
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint8)
    lib().crit_oracle_e4m3_encode_n(_p(x), ctypes.c_int64(x.size), _p(out))
    return out


_DECODE = None


def e4m3_decode(codes):
    """E4M3FN bytes -> FP32 (exact).  ref: kernels/core/python/crit_kcore/formats.py:81-90."""
    global _DECODE
    if _DECODE is None:
        f = lib().crit_oracle_e4m3_decode
        _DECODE = np.array([f(b) for b in range(256)], np.float32)
    return _DECODE[np.asarray(codes, np.uint8)]


# -- quantise rules -----------------------------------------------------------------------------------------------------
def quantize_rows(x, kind, multiplier=1.0):
    """x [..., dim] -> (codes uint8 [..., dim], scales FP32 [...] or None) by the page kind's rule ("fp8", "fp8:row",
    "int8"; int8 codes are returned as their bytes).  ref: inference/attention-state/code/pages.py:442-445, :872-895."""
    x = _c(x, np.float32)
    k = KINDS[kind]
    rows, dim = int(np.prod(x.shape[:-1])), x.shape[-1]
    codes = np.empty(x.shape, np.uint8)
    scales = np.empty(x.shape[:-1], np.float32) if k in (2, 3) else None
    lib().crit_oracle_quantize_rows(_p(x), ctypes.c_int64(rows), ctypes.c_int64(dim), ctypes.c_int(k),
                                    ctypes.c_float(multiplier), _p(codes), _p(scales))
    return codes, scales


def quantize_pages(x, slots, page, codes, scales):
    """One write() of the per-(page, kv head) FP8 kind: x [tokens][heads][dim] into codes [slots][heads][dim] (uint8)
    and scales [pages][heads] in place (the rule is stated in oracle.c; no reference counterpart, parity unpinned)."""
    x = _c(x, np.float32)
    slots = _c(slots, np.int64)
    assert codes.dtype == np.uint8 and codes.flags.c_contiguous and scales.dtype == np.float32 and scales.flags.c_contiguous
    tokens, heads, dim = x.shape
    lib().crit_oracle_quantize_pages(_p(x), _p(slots), ctypes.c_int64(tokens), ctypes.c_int64(heads),
                                     ctypes.c_int64(dim), ctypes.c_int64(page), _p(codes), _p(scales))


def dequantize(codes, kind, scales=None, multiplier=1.0, page=None):
    """Stored pages [slots][heads][dim] -> FP32 values: code * scale (exact in FP32 for FP8 and INT8 codes).
    ref: pages.py:471-477 (gather), :485-491 (rows_at)."""
    k = KINDS[kind]
    if k == 0:
        return np.asarray(codes, np.float32)
    if k == 3:
        values = np.asarray(codes).view(np.int8).astype(np.float32)
    else:
        values = e4m3_decode(np.asarray(codes).view(np.uint8))
    if k == 1:
        return values * np.float32(multiplier)
    if k == 4:
        return values * np.repeat(np.asarray(scales, np.float32), page, axis=0)[..., None]
    return values * np.asarray(scales, np.float32)[..., None]


# -- slots --------------------------------------------------------------------------------------------------------------
def slots(table, positions, page):
    """table[p // page] * page + p % page.  ref: pages.py:721-722."""
    table, positions = _c(table, np.int32), _c(positions, np.int64)
    out = np.empty(positions.shape, np.int64)
    lib().crit_oracle_slots(_p(table), _p(positions), ctypes.c_int64(positions.size), ctypes.c_int64(page), _p(out))
    return out


def round_slots(tables, capacity, slot, positions, page, dump):
    """Captured-round slots, the dump page's first slot outside [0, capacity).  ref: pages.py:653-660."""
    tables, capacity = _c(tables, np.int32), _c(capacity, np.int64)
    slot, positions = _c(slot, np.int64), _c(positions, np.int64)
    out = np.empty(positions.shape, np.int64)
    lib().crit_oracle_round_slots(_p(tables), ctypes.c_int64(tables.shape[1]), _p(capacity), _p(slot), _p(positions),
                                  ctypes.c_int64(positions.size), ctypes.c_int64(page), ctypes.c_int64(dump), _p(out))
    return out


# -- attention ----------------------------------------------------------------------------------------------------------
def attend(q, k, v, tables, rows, starts, firsts, columns, page, scale=None, counts=None, lo=0, hi=None):
    """Window rows over dequantised pages: q [T][hq][d]; k [slots][hkv][d], v [slots][hkv][dv] FP32; the metadata as
    the product's attend() takes it.  -> (out [T][hq][dv] FP32, lse [T][hq] FP32); tokens no row names stay 0 / -inf.
    [lo, hi): only these positions (one KV-range shard's partial).
    ref: inference/attention-state/code/device_attention.py:1204-1288, :1301-1335."""
    q, k, v = _c(q, np.float32), _c(k, np.float32), _c(v, np.float32)
    tables = _c(tables, np.int32)
    if tables.ndim == 1:
        tables = tables[None]
    rows, starts = _c(rows, np.int32), _c(starts, np.int32)
    firsts = _c(firsts, np.int64)
    counts = _c(counts, np.int32) if counts is not None else None
    T, hq, d = q.shape
    hkv, dv = k.shape[-2], v.shape[-1]
    scale = float(scale if scale is not None else d ** -0.5)
    out = np.zeros((T, hq, dv), np.float32)
    lse = np.full((T, hq), -np.inf, np.float32)
    hi = (1 << 62) if hi is None else int(hi)
    i64 = ctypes.c_int64
    lib().crit_oracle_attend(_p(q), i64(hq), i64(d), _p(k), _p(v), i64(hkv), i64(dv), _p(tables),
                             i64(tables.shape[1]), _p(rows), _p(starts), _p(counts), _p(firsts), i64(rows.size),
                             i64(columns), i64(page), ctypes.c_float(scale), i64(int(lo)), i64(hi), _p(out), _p(lse))
    return out, lse


def attend_tree(q, k, v, tables, rows, starts, firsts, columns, page, parents, scale=None, counts=None, sinks=None,
                sliding=0, blocks=None, block_size=0):
    """attend() with the reference's other visibility rules.  parents [T] (or None: causal) is each token's parent column
    in its row, -1 for none: a column sees the context before its row's first position and, of the window, itself and its
    ancestors.  sliding > 0: a column sees only the `sliding` positions up to its own.  sinks [hq] (or None): a logit a
    query head that joins the softmax's maximum and sum (and the lse) without a value.  blocks [T][k] (or None): the KV
    blocks of block_size positions a token sees, -1 for none.
    ref: paged_kv_attention/_kernels.py:154-165, :325-333; device_attention.py:1301-1335."""
    q, k, v = _c(q, np.float32), _c(k, np.float32), _c(v, np.float32)
    tables = _c(tables, np.int32)
    if tables.ndim == 1:
        tables = tables[None]
    rows, starts = _c(rows, np.int32), _c(starts, np.int32)
    parents = _c(parents, np.int32) if parents is not None else None
    sinks = _c(sinks, np.float32) if sinks is not None else None
    blocks = _c(blocks, np.int32) if blocks is not None else None
    firsts = _c(firsts, np.int64)
    counts = _c(counts, np.int32) if counts is not None else None
    T, hq, d = q.shape
    hkv, dv = k.shape[-2], v.shape[-1]
    scale = float(scale if scale is not None else d ** -0.5)
    out = np.zeros((T, hq, dv), np.float32)
    lse = np.full((T, hq), -np.inf, np.float32)
    i64 = ctypes.c_int64
    lib().crit_oracle_attend_tree(_p(q), i64(hq), i64(d), _p(k), _p(v), i64(hkv), i64(dv), _p(tables),
                                  i64(tables.shape[1]), _p(rows), _p(starts), _p(counts), _p(firsts), _p(parents),
                                  _p(sinks), i64(int(sliding)), _p(blocks), i64(blocks.shape[1] if blocks is not None else 0),
                                  i64(int(block_size)), i64(rows.size), i64(columns), i64(page),
                                  ctypes.c_float(scale), _p(out), _p(lse))
    return out, lse


def merge(outs, lses):
    """outs [parts][...][dv], lses [parts][...] -> (out, lse).  ref: inference/partitioned-attention/plugin.py:52-64."""
    outs, lses = _c(outs, np.float32), _c(lses, np.float32)
    parts, dv = outs.shape[0], outs.shape[-1]
    n = int(np.prod(lses.shape[1:]))
    out, lse = np.empty(outs.shape[1:], np.float32), np.empty(lses.shape[1:], np.float32)
    lib().crit_oracle_merge(_p(outs), _p(lses), ctypes.c_int64(parts), ctypes.c_int64(n), ctypes.c_int64(dv),
                            _p(out), _p(lse))
    return out, lse


def fold(po, pm, pl):
    """Split states in split order -> (out [dv], lse).  ref: paged_kv_attention/_kernels.py:558-604 (_merge_kernel)."""
    po, pm, pl = _c(po, np.float32), _c(pm, np.float32), _c(pl, np.float32)
    out, lse = np.empty(po.shape[-1], np.float32), np.empty(1, np.float32)
    lib().crit_oracle_fold(_p(po), _p(pm), _p(pl), ctypes.c_int64(po.shape[0]), ctypes.c_int64(po.shape[-1]),
                           _p(out), _p(lse))
    return out, float(lse[0])
