"""crit_b200: the paged KV-cache hot path of crit, hand-written for B200 (sm_100a).

This module is the kernel-module boundary: the object crit's KVPool and DeviceAttention take as `kernels=`
(reference: kernels/techniques/attention/paged-kv-attention/torch-ext/paged_kv_attention/__init__.py, loaded by
crit_plugins.kernels.load_kernel("paged-kv-attention")).  It keeps that module's names, argument meanings and errors
for write / attend / prefill / partitions / piece_size / tile_for / workspace_floats / owner / release, and reaches
the CUDA kernels through the C ABI of include/crit_b200.h (ctypes, as the reference binds its own CUDA tile).  There
is no Triton, no torch fallback and no CPU path: without the native library, or on a tensor that is not on a CUDA
device, every entry point raises.

Page kinds: the reference's "bf16", "fp16", "fp8", "fp8:row", "int8", and "fp8:page": E4M3 codes with one FP32 scale
per (page, kv head), scales [pages][kv_heads] (scale = amax / 448 over the page's rows of that head).

A row's positions are read in contiguous splits of `chunk` positions (one per cache geometry, chunk_for()); the splits'
states are folded in split order.  This is the reference's "flash" split shape (contiguous splits, __init__.py:580-612)
rather than its interleaved pieces; attention outputs agree with the reference's within its own kernel-vs-torch
tolerance, integer and byte results (slots, codes, scales) bit for bit.
"""
import contextlib
import ctypes
import math
import threading

import torch

from . import _lib

__all__ = ["KINDS", "MAX_COLUMNS", "attend", "chunk_for", "gather", "merge_shards", "move_rows", "owner", "partitions", "parts_for",
           "engine_for", "piece_size", "plan", "prefill", "prefill_serves", "release", "slots_at", "states_for", "status", "tcgen05_serves",
           "tcgen05p_serves", "tile_for", "workspace_floats", "write"]

KINDS = {"bf16": 0, "fp16": 0, "fp8": 1, "fp8:row": 2, "int8": 3, "fp8:page": 4}
MAX_COLUMNS = 64            # columns of one row a launch reads
TILE = 16                   # positions a warp reads per step: chunks and pages are multiples of it
DEFAULT_CHUNK = 1024

_DTYPES = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_FP16, torch.float32: _lib.DTYPE_FP32}
_PAGE_DTYPES = {"bf16": _lib.DTYPE_BF16, "fp16": _lib.DTYPE_FP16}


def _check_kind(kind, key_scales):
    if kind not in KINDS:
        raise ValueError(f"page kinds are {', '.join(KINDS)}, not {kind!r}")
    if (KINDS[kind] >= 2) != (key_scales is not None):
        raise ValueError(f"{kind} pages {'take' if KINDS[kind] >= 2 else 'have no'} scales beside their codes")
    return KINDS[kind]


def _cuda(tensor, what):
    if not tensor.is_cuda:
        raise RuntimeError(f"crit_b200 runs on CUDA devices only: {what} is on {tensor.device} (there is no CPU path)")
    return tensor


def _ptr(tensor):
    return ctypes.c_void_p(tensor.data_ptr()) if tensor is not None else None


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _page_dtype(kind, pages):
    if KINDS[kind] != 0:
        return _lib.DTYPE_BF16
    if pages.dtype not in _DTYPES:
        raise ValueError(f"{kind} pages are 16-bit tensors, not {pages.dtype}")
    return _DTYPES[pages.dtype]


# -- workspaces -----------------------------------------------------------------------------------------------------------
# One per (device, owner): a launch writes its partials and the merge reads them back, so two engines of one process
# never share one (reference: paged_kv_attention/__init__.py:129-171).  A workspace a launch outgrew is kept: a CUDA
# graph captured over it replays into it.
_workspaces, _retired = {}, []
_owner = threading.local()


@contextlib.contextmanager
def owner(key):
    """Launches inside this block take a workspace of their own, apart from every other owner's."""
    before = getattr(_owner, "key", None)
    _owner.key = key
    try:
        yield
    finally:
        _owner.key = before


def release(key):
    """Drop an owner's workspaces (its captured graphs must be gone: they replay into them)."""
    for at in [at for at in _workspaces if at[1] == key]:
        del _workspaces[at]
    _retired[:] = [(k, found) for k, found in _retired if k != key]


def _workspace(device, floats, given):
    if given is not None:
        if given.dtype != torch.float32 or given.numel() < floats or not given.is_contiguous():
            raise ValueError(f"attend's workspace holds {given.numel()} floats; this launch needs {floats} "
                             "(workspace_floats)")
        return given
    at = (str(device), getattr(_owner, "key", None))
    found = _workspaces.get(at)
    if found is None or found.numel() < floats:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("crit_b200.attend: run a launch of this size once before capturing it (its partials' "
                               "workspace is allocated outside the capture)")
        if found is not None:
            _retired.append((at[1], found))
        found = _workspaces[at] = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device)
    return found


_status = {}


def _status_word(device):
    """One int32 a device: a kernel sets it (and never clears it) when one of its bounded waits gave up."""
    found = _status.get(str(device))
    if found is None:
        if torch.cuda.is_current_stream_capturing():
            return None
        found = _status[str(device)] = torch.zeros(1, dtype=torch.int32, device=device)
    return found


def status(device=None):
    """0, or what a kernel recorded on `device` since load, when one of its bounded waits ran out (the block concerned
    wrote nothing): 1 = a TMA copy of the m16n8k16 decode kernel; 0x110 / 0x120 / 0x140 = the producer / MMA / softmax
    warps of the tcgen05 prefill kernel (0x1ff: its shared memory was not 1 KB aligned); 0x410 / 0x420 / 0x440 = the
    producer / MMA / softmax warps of the tcgen05 decode kernel; 0x800 + rank = the peer exchange of the shards' partials
    waited in vain for another rank's message.  Reads the device word (one synchronisation)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    found = _status.get(str(device))
    return 0 if found is None else int(found.item())


# -- geometry rules -----------------------------------------------------------------------------------------------------
def chunk_for(head_dim, value_dim, heads, kv_heads, page, kind="bf16", engine=None, columns=1):
    """Positions per split of a launch over a cache of this geometry (a multiple of 16).  One per cache for the
    m16n8k16 kernel, never by the batch, so a column's bits are the same alone and in any window.  Launches of the
    tcgen05 kernel that gives a unit one kv head (engine "tcgen05", or attend's own choice for windows of several columns
    over E4M3 pages) use splits of 2,048: a unit's fold of its lane replicas is paid once per split."""
    if engine is None:
        engine = engine_for(kind, head_dim, value_dim, heads, kv_heads, columns)
    return 2 * DEFAULT_CHUNK if engine in ("tcgen05", "tcgen05t") else DEFAULT_CHUNK


def tcgen05_serves(kind, head_dim, value_dim, heads, kv_heads, columns, chunk, rows=1):
    """Whether the tcgen05 kernel takes a launch: E4M3 pages of 128-wide heads, at most 32 query rows a unit (columns
    x heads of a kv head's group), splits of whole 128-position tiles up to 2,048 positions, up to 256 window rows (the
    same test the library makes: decode.cu, tc_serves)."""
    return (str(kind).startswith("fp8") and head_dim == 128 and value_dim == 128 and columns * (heads // kv_heads) <= 32
            and chunk % 128 == 0 and chunk <= 2048 and rows <= 256)


def tcgen05p_serves(kind, head_dim, value_dim, heads, kv_heads, columns, chunk, rows=1):
    """Whether the tcgen05 kernel over whole page rows takes a launch: E4M3 pages of 128-wide heads, 8 kv heads, at most 8
    query rows a kv head (columns x heads of a group), splits of whole 16-position tiles up to 2,048 positions, up to 256
    window rows (the same test the library makes: decode.cu, ph_serves)."""
    return (str(kind).startswith("fp8") and head_dim == 128 and value_dim == 128 and kv_heads == 8 and
            columns * (heads // kv_heads) <= 8 and chunk % 16 == 0 and chunk <= 2048 and rows <= 256)


# Launches below this many positions (window rows x the positions their tables hold) stay on the m16n8k16 kernel: the
# whole-page-rows kernel deals whole splits to its blocks, and a small launch has too few to fill the device.
PAGE_ROWS_FROM = 1 << 16


def engine_for(kind, head_dim, value_dim, heads, kv_heads, columns, rows=1, positions=None, engine=None):
    """The kernel a launch runs on: `engine` when one is named, else attend's own choice: "tcgen05p" (whole page rows:
    every kv head of a position in one contiguous read) for E4M3 pages of 8 kv heads x 128 with at most 8 query rows a
    kv head, when the launch is large enough to fill the device that way; "tcgen05" for other windows of several
    columns over E4M3 pages of 128-wide heads; "mma.sync" (m16n8k16) for everything else.  Only the last gives a column
    the same bits alone and in any window or batch."""
    if engine is not None:
        return engine
    if tcgen05p_serves(kind, head_dim, value_dim, heads, kv_heads, columns, DEFAULT_CHUNK, rows) and \
            positions is not None and rows * positions >= PAGE_ROWS_FROM:
        return "tcgen05p"
    if columns > 1 and tcgen05_serves(kind, head_dim, value_dim, heads, kv_heads, columns, 2 * DEFAULT_CHUNK, rows):
        return "tcgen05"
    return "mma.sync"


def states_for(parts, engine):
    """Split states a partial row takes in the workspace for `parts` splits: the whole-page-rows kernel deals the
    launch's tiles out evenly, so a split may be shared by two blocks and has two states (its head and its tail)."""
    return 2 * parts if engine == "tcgen05p" else parts


def parts_for(positions, chunk):
    """Splits a partial row takes over page tables holding `positions` positions a row."""
    return max(1, -(-int(positions) // int(chunk)))


_plans = {}


def plan(heads, kv_heads, head_dim, value_dim, page, kind="bf16", columns=1, device=None):
    """What the library would launch for a cache of this geometry on `device`: a dict of chunk (positions per split),
    smem (bytes of shared memory a block takes), rows (query rows a block's tile holds), per_sm (blocks resident per
    SM) and sms.  Asked of the library once per geometry and device (crit_b200_attend_plan)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (str(device), heads, kv_heads, head_dim, value_dim, page, kind, columns)
    found = _plans.get(key)
    if found is None:
        out = (ctypes.c_int32 * 5)()
        dtype = _lib.DTYPE_FP16 if kind == "fp16" else _lib.DTYPE_BF16
        with torch.cuda.device(device):
            _lib.check(_lib.load().crit_b200_attend_plan(heads, kv_heads, head_dim, value_dim, page, KINDS[kind], dtype, columns, out),
                       "crit_b200.plan")
        found = _plans[key] = dict(chunk=out[0], smem=out[1], rows=out[2], per_sm=out[3], sms=out[4])
    return found


def partitions(device, kv_heads, kind, head_dim=None, value_dim=None):
    """The most splits a partial row takes in a launch whose caller sizes the workspace by a count per cache
    (reference: paged_kv_attention/__init__.py:260-273, a rule over the device's SMs, the kv heads and the code width).
    Here: enough splits for two waves of the device's resident blocks from ONE row (its splits x kv_heads blocks), as
    a power of two in 8..128.  attend(partitions=P) never makes more than P splits: it raises the chunk where a row's
    tables hold more than P * chunk positions."""
    head_dim = head_dim or 128
    value_dim = value_dim or head_dim
    found = plan(kv_heads, kv_heads, head_dim, value_dim, TILE, kind, 1, device)
    want = max(1, 2 * found["sms"] * max(found["per_sm"], 1) // max(kv_heads, 1))
    return min(128, max(8, 1 << (want.bit_length() - 1)))


def piece_size(head_dim, value_dim, kind="bf16", kv_heads=None):
    """Positions a warp reads per step (reference: __init__.py:276-286; here the tile is 16 for every geometry)."""
    return TILE


def tile_for(columns, group, capability, fused=False):
    """(rows, warps, stages) of a launch's query tile (reference: __init__.py:335-356): 8, 16 or 32 query rows (columns
    x the group's heads, in tiles of 8), four warps, each with its own ring of 3 or 4 stages (4 where a warp's
    iteration takes two 16-position tiles, which 8-bit pages of heads up to 128 wide do; the width is not an argument
    here, so the deeper ring is reported)."""
    rows = columns * group
    return (8 if rows <= 8 else (16 if rows <= 16 else 32)), 4, 4


def workspace_floats(tokens, heads, partitions, value_dim):
    """FP32 floats of the partials a launch needs for `tokens` partial rows (reference: __init__.py:359-362)."""
    return tokens * heads * partitions * (value_dim + 2)


# -- KV append ----------------------------------------------------------------------------------------------------------
def write(keys, values, slots, key_pages, value_pages, kind, key_scales=None, value_scales=None,
          multipliers=(1.0, 1.0)):
    """A step's keys [tokens][kv_heads][dim] and values [tokens][kv_heads][value_dim] (bf16, fp16 or fp32) into their
    slots ([tokens] int64; a slot below 0 is skipped) of one layer's pages (any view whose storage is
    [slots][kv_heads][dim]), encoded for the page kind, in one launch.  values and value_pages None: keys only; keys
    and key_pages None: values only, at the value multiplier.  "fp8:page" takes scales [pages][kv_heads] and the page
    size from the pages' shape ([pages][page][kv_heads][dim]).  Reference: paged_kv_attention/__init__.py:289-324."""
    if keys is None:
        if values is None:
            raise ValueError("write takes keys, values or both")
        return write(values, None, slots, value_pages, None, kind, value_scales, None,
                     multipliers=(multipliers[1], multipliers[1]))
    k_kind = _check_kind(kind, key_scales)
    _cuda(keys, "keys")
    T, hkv, d = keys.shape
    if T == 0:
        return
    if keys.dtype not in _DTYPES or (values is not None and values.dtype != keys.dtype):
        raise ValueError("keys and values are bf16, fp16 or fp32 tensors of one dtype")
    if keys.stride(-1) != 1:
        keys = keys.contiguous()
    if values is not None and values.stride(-1) != 1:
        values = values.contiguous()
    if slots.dtype != torch.int64 or not slots.is_contiguous() or slots.numel() != T:
        raise ValueError(f"slots are contiguous int64 [{T}]")
    if not key_pages.is_contiguous() or (value_pages is not None and not value_pages.is_contiguous()):
        raise ValueError("pages are contiguous [slots][kv_heads][dim] storage")
    page = 1
    if k_kind == 4:
        if key_pages.dim() != 4:
            raise ValueError("fp8:page pages are given as [pages][page][kv_heads][dim]")
        page = key_pages.shape[1]
    p = _lib.AppendParams()
    p.keys, p.values, p.slots = _ptr(keys), _ptr(values), _ptr(slots)
    p.key_pages, p.value_pages = _ptr(key_pages), _ptr(value_pages)
    p.key_scales, p.value_scales = _ptr(key_scales), _ptr(value_scales)
    p.tokens = T
    p.slots_total = key_pages.numel() // (hkv * d)
    p.status = _ptr(_status_word(keys.device))
    p.key_stride_token, p.key_stride_head = keys.stride(0), keys.stride(1)
    if values is not None:
        p.value_stride_token, p.value_stride_head = values.stride(0), values.stride(1)
    p.kv_heads, p.head_dim, p.page = hkv, d, page
    p.value_dim = values.shape[-1] if values is not None else d
    p.kind, p.in_dtype, p.page_dtype = k_kind, _DTYPES[keys.dtype], _page_dtype(kind, key_pages)
    p.key_multiplier, p.value_multiplier = float(multipliers[0]), float(multipliers[1])
    with torch.cuda.device(keys.device):
        _lib.check(_lib.load().crit_b200_append(ctypes.byref(p), _stream(keys.device)), "crit_b200.write")


# -- gather and slots ---------------------------------------------------------------------------------------------------
def gather(pages, kind, page, *, table=None, slots=None, count=None, scales=None, multiplier=1.0, dtype=torch.bfloat16):
    """Rows of one page tensor ([pages][page][kv_heads][dim] or [slots][kv_heads][dim]) dequantised to `dtype`: the
    first `count` positions of the page table `table` (int32), or the rows at `slots` (int64, any shape).
    -> [count][kv_heads][dim] (or slots' shape + [kv_heads][dim]).  Reference: pages.py:455-493."""
    _cuda(pages, "pages")
    k_kind = _check_kind(kind, scales)
    hkv, dim = pages.shape[-2], pages.shape[-1]
    shape = None
    if slots is not None:
        shape, slots = tuple(slots.shape), slots.reshape(-1).contiguous()
        count = slots.numel()
    elif table is None or count is None:
        raise ValueError("gather reads a page table's first `count` positions, or rows at `slots`")
    out = torch.empty((count, hkv, dim), dtype=dtype, device=pages.device)
    if count == 0:
        return out if shape is None else out.view(*shape, hkv, dim)
    p = _lib.GatherParams()
    p.pages, p.scales, p.out = _ptr(pages), _ptr(scales), _ptr(out)
    p.table = _ptr(table.contiguous()) if table is not None else None
    p.slots = _ptr(slots)
    if not pages.is_contiguous():
        raise ValueError("pages are contiguous [slots][kv_heads][dim] storage")
    p.slots_total = pages.numel() // (hkv * dim)
    p.status = _ptr(_status_word(pages.device))
    p.count, p.kv_heads, p.dim, p.page = count, hkv, dim, int(page)
    p.kind, p.page_dtype, p.out_dtype = k_kind, _page_dtype(kind, pages), _DTYPES[dtype]
    p.multiplier = float(multiplier)
    with torch.cuda.device(pages.device):
        _lib.check(_lib.load().crit_b200_gather(ctypes.byref(p), _stream(pages.device)), "crit_b200.gather")
    return out if shape is None else out.view(*shape, hkv, dim)


def slots_at(tables, rows, positions, page, dump, capacity=None, out=None):
    """Each position's slot through its table row, on the device: tables [S][width] int32, rows and positions int64 of
    one shape; with capacity [S] int64 a position outside [0, capacity[row]) gets the dump page's first slot.
    Reference: pages.py:653-660."""
    _cuda(tables, "tables")
    shape = tuple(positions.shape)
    rows, positions = rows.reshape(-1).contiguous(), positions.reshape(-1).contiguous()
    if rows.dtype != torch.int64 or positions.dtype != torch.int64 or tables.dtype != torch.int32:
        raise ValueError("tables are int32, rows and positions int64")
    out = torch.empty(positions.numel(), dtype=torch.int64, device=tables.device) if out is None else out
    p = _lib.SlotsParams()
    p.tables, p.rows, p.positions, p.capacity, p.slots = _ptr(tables), _ptr(rows), _ptr(positions), _ptr(capacity), _ptr(out)
    p.n, p.table_stride, p.table_width = positions.numel(), tables.stride(0), tables.shape[1]
    p.page, p.dump = int(page), int(dump)
    with torch.cuda.device(tables.device):
        _lib.check(_lib.load().crit_b200_slots(ctypes.byref(p), _stream(tables.device)), "crit_b200.slots_at")
    return out.view(shape)


def move_rows(store, source, target):
    """Rows of one store moved between slots, in place: store [layers][slots][...] (keys, values or their row scales),
    source / target [lists][width] int64 slots; for every list, in order j = 0 .. width - 1, the row at source[l][j] of
    every layer goes to target[l][j] (nothing where the two are equal).  A list's moves happen one after another; lists
    are independent.  What the pool's commit_round brings an accepted draft-tree path's KV together with
    (reference: inference/attention-state/code/pages.py:662-684)."""
    _cuda(store, "store")
    if not store.is_contiguous() or store.dim() < 2:
        raise ValueError("a store is contiguous [layers][slots][...]")
    if source.dtype != torch.int64 or target.dtype != torch.int64 or source.shape != target.shape or source.dim() != 2:
        raise ValueError("source and target are int64 [lists][width]")
    source, target = source.contiguous(), target.contiguous()
    layers, slots = store.shape[0], store.shape[1]
    row_bytes = store[0, 0].numel() * store.element_size()
    if row_bytes % 4:
        raise ValueError("a store's rows are a multiple of 4 bytes")
    p = _lib.MoveParams()
    p.store, p.source, p.target = _ptr(store), _ptr(source), _ptr(target)
    p.lists, p.width, p.slots, p.row_bytes, p.layers = source.shape[0], source.shape[1], slots, row_bytes, layers
    p.status = _ptr(_status_word(store.device))
    with torch.cuda.device(store.device):
        _lib.check(_lib.load().crit_b200_move_rows(ctypes.byref(p), _stream(store.device)), "crit_b200.move_rows")


def _listed_rows(tables, rows, starts, counts, firsts, blocks, block_size, page, columns, out, lse):
    """Block lists as page tables of their own (crit_b200_compact_blocks): (tables, rows, starts, firsts, counts) of
    one-column rows, a row a token, whose tables hold the pages of the token's listed blocks only; tokens that see
    nothing get zeros in out (and -inf in lse) here."""
    device = tables.device
    R = int(starts.shape[0])
    n, per = R * columns, block_size // page
    t2 = torch.empty(n, blocks.shape[1] * per, dtype=torch.int32, device=device)
    c2 = torch.empty(n, dtype=torch.int32, device=device)
    f2 = torch.empty(n, dtype=torch.int64, device=device)
    p = _lib.CompactParams()
    p.tables, p.rows, p.starts, p.counts, p.firsts, p.blocks = (_ptr(x) for x in (tables, rows, starts, counts, firsts, blocks))
    p.out_tables, p.out_counts, p.out_firsts, p.out, p.lse = _ptr(t2), _ptr(c2), _ptr(f2), _ptr(out), _ptr(lse)
    p.n_rows, p.table_stride, p.table_width = R, tables.stride(0), tables.shape[1]
    p.out_stride_token, p.out_stride_head = out.stride(0), out.stride(1)
    p.columns, p.blocks_k, p.block_size, p.page = columns, blocks.shape[1], block_size, page
    p.dump = 0              # (entries past a row's listed pages are never read: its last position ends before them)
    p.q_heads, p.value_dim, p.out_dtype = out.shape[1], out.shape[2], _DTYPES[out.dtype]
    with torch.cuda.device(device):
        _lib.check(_lib.load().crit_b200_compact_blocks(ctypes.byref(p), _stream(device)), "crit_b200.attend (block lists)")
    tokens = (starts[:, None] + torch.arange(columns, dtype=torch.int32, device=device)[None, :]).reshape(-1).contiguous()
    return t2, torch.arange(n, dtype=torch.int32, device=device), tokens, f2, c2


# -- decode and verify windows ------------------------------------------------------------------------------------------
def _refuse(**given):
    asked = [name for name, value in given.items()
             if value is not None and value is not False and not (isinstance(value, int) and value == 0)]
    if asked:
        raise NotImplementedError(f"crit_b200.attend does not serve {', '.join(asked)} yet: causal windows over the "
                                  "whole context only")


def attend(q, key_pages, value_pages, kind, tables, rows, starts, firsts, columns, page, *, counts=None,
           offsets=None, tokens=None, key_scales=None, value_scales=None, multipliers=(1.0, 1.0), scale=None,
           partitions=None, parents=None, blocks=None, block_size=None, out=None, lse=None, workspace=None, piece=None,
           fused=False, fresh=None, vsplit=None, tile=None, num_warps=None, num_stages=None, maxnreg=None,
           flash=False, chunk=None, ramp=None, sinks=None, sliding=0, derive=None, launch="both", staging=None,
           persistent=False, engine=None, shards=None, context=False):
    """Decode and verify windows over paged KV (reference: paged_kv_attention/__init__.py:396-445, same arguments).

    q [tokens][heads][dim] bf16 or fp16 (fp16 for "fp16" pages); key_pages / value_pages one layer's pages
    ([pages][page][kv_heads][dim]), key_scales / value_scales their scales; tables [S][width] int32; rows [R] int32 the
    table row of each batch row; starts [R] int32 its first token in q; firsts [R] int64 its column 0's position;
    counts [R] int32 its columns (None: `columns` each; more read as `columns`); columns the widest row (<= 64).
    offsets [R] int32 and tokens: each row's first partial row and the partial rows the launch takes.  Writes
    out [tokens][heads][value_dim] (q's dtype) at the rows' tokens and lse [tokens][heads] FP32 when given; returns out.
    chunk: positions per split (default chunk_for()); partitions: the most splits a partial row may take (the
    workspace's, see partitions()).  piece, fused, vsplit, tile, num_warps, num_stages, maxnreg, flash and ramp are
    accepted and change nothing (one launch shape per geometry).  parents [tokens]: each token's parent column in its
    row, -1 for none (a draft tree in topological order): a column then sees the context before its row's first position,
    itself and its ancestors.  sinks [heads] FP32: a logit a query head that joins the softmax's maximum and sum (and
    the lse) without a value; sliding: the positions a column sees up to its own, 0 for all (all three on the m16n8k16
    kernel).  blocks [tokens][k] int32 with block_size: the KV blocks (block_size positions each, -1 for none) a token
    sees.  Where block_size is a multiple of the page (and no tree, sink or sliding window is asked for) the launch
    reads the listed blocks only: every token becomes a one-column row over a page table of its blocks, built on the
    device, on whichever kernel serves it; otherwise the lists are a mask over the m16n8k16 kernel's tiles (every
    position is read).  context: every column of a row sees the positions before firsts[r] and none from there on (the
    part of a prompt chunk's attention that reads the pages when its own keys and values are read fresh; an extension
    of this module).  fresh (the reference's in-kernel fresh rows) and derive are not served: DeviceAttention reads a
    pool's fresh rows as context rows + a prefill over the fresh chunk + merge_shards.  launch: "both", or "decode" / "merge" alone (a measurement's).  staging: how pages reach shared memory:
    None (TMA tiled loads for 16-bit pages of 128- or 256-wide heads, cp.async otherwise: what measured faster), "tma"
    (TMA wherever the geometry allows it) or "cp.async" (never TMA); the same bits either way.  persistent: a fixed
    number of blocks walk a work list built on the device from the rows' lengths, instead of one block per (split, kv
    head, row) of a 3-D grid (the same bits; measured slower on the bench workloads, hence off).  engine: None (the
    library's choice), "mma.sync" (the m16n8k16 kernel) or "tcgen05" (E4M3 page bytes straight into tcgen05.mma: E4M3
    pages of 128-wide heads, columns x group heads <= 32, chunk a multiple of 128; refused elsewhere).
    shards: a crit_b200.dist.ShardMerge: these pages hold one KV range of a context sharded over the ranks; every
    split state stays in the workspace, the fold of this rank's splits is stored into every rank's exchange buffer and
    out / lse get the merge over all ranks (three launches: decode, fold + push, wait + merge)."""
    _refuse(fresh=fresh, derive=derive)
    if context and (parents is not None or blocks is not None or sinks is not None or sliding or shards is not None or
                    engine not in (None, "mma.sync")):
        raise NotImplementedError("context rows (every column sees the positions before its row's first only) are the "
                                  "m16n8k16 kernel's plain rows")
    k_kind = _check_kind(kind, key_scales)
    _cuda(q, "q")
    T, hq, d = q.shape
    hkv, dv = key_pages.shape[-2], value_pages.shape[-1]
    R = int(starts.shape[0])
    if hq % hkv or not 1 <= columns <= MAX_COLUMNS or R == 0:
        raise ValueError("query heads a multiple of the KV heads, 1..64 columns a row, one row or more")
    if q.stride(-1) != 1:
        raise ValueError("q's last dimension is contiguous")
    if q.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("q is bf16 or fp16")
    if (offsets is None) != (tokens is None):
        raise ValueError("offsets come with the partial rows they take (tokens)")
    if tables.dtype != torch.int32 or tables.stride(-1) != 1 or rows.dtype != torch.int32 or \
            starts.dtype != torch.int32 or firsts.dtype != torch.int64:
        raise ValueError("tables, rows and starts are int32, firsts int64")
    page = int(page)
    if page % TILE:
        raise ValueError(f"crit_b200 reads pages of a multiple of {TILE} positions, not {page}")
    if not key_pages.is_contiguous() or not value_pages.is_contiguous():
        raise ValueError("pages are contiguous [slots][kv_heads][dim] storage")
    device = q.device
    positions = tables.shape[1] * page
    if parents is not None:
        # a draft tree: parents [tokens] is each token's parent column in its row, -1 for none (topological order)
        if engine not in (None, "mma.sync"):
            raise NotImplementedError("draft trees (parents) are served by the m16n8k16 kernel: engine None or mma.sync")
        parents = parents.reshape(-1)
        if parents.dtype not in (torch.int32, torch.int64) or parents.numel() != T:
            raise ValueError("parents are int32 or int64, one per token of q")
        parents = _cuda(parents, "parents").to(torch.int32).contiguous()
        engine = "mma.sync"
    if blocks is not None:
        # block lists: blocks [tokens][k] KV block ids (-1 for none) of block_size positions: a token sees only those
        if blocks.dim() != 2 or blocks.shape[0] != T or not block_size or int(block_size) < 1:
            raise ValueError("blocks are [tokens][k] block ids, with the positions a block holds (block_size)")
        blocks = _cuda(blocks, "blocks").to(torch.int32).contiguous()
        if (int(block_size) % page == 0 and parents is None and sinks is None and not sliding and offsets is None and
                shards is None and launch == "both" and not torch.cuda.is_current_stream_capturing()):
            # the sparse reader: every token becomes a row of one column over a page table of its listed blocks only
            # (built on the device), so the launch reads those blocks and nothing else, on whichever kernel serves it
            out = torch.empty(T, hq, dv, dtype=q.dtype, device=q.device) if out is None else out
            listed = _listed_rows(tables, rows, starts, counts, firsts, blocks, int(block_size), page, int(columns), out, lse)
            return attend(q, key_pages, value_pages, kind, listed[0], listed[1], listed[2], listed[3], 1, page,
                          counts=listed[4], key_scales=key_scales, value_scales=value_scales, multipliers=multipliers,
                          scale=scale, partitions=partitions, out=out, lse=lse, workspace=workspace, chunk=chunk,
                          engine=engine)
        if engine not in (None, "mma.sync"):
            raise NotImplementedError("block lists of blocks that are no multiple of the page, or with a tree, sinks or a "
                                      "sliding window, are a mask of the m16n8k16 kernel: engine None or mma.sync")
        engine = "mma.sync"             # as a mask over the m16n8k16 kernel's tiles: every position is read
    sliding = int(sliding or 0)
    if sinks is not None or sliding:
        # a sink logit a query head (joins the softmax's maximum and sum, and the lse, in the fold of the splits), and a
        # window of the `sliding` positions up to a column's own: the m16n8k16 kernel's
        if engine not in (None, "mma.sync"):
            raise NotImplementedError("sinks and sliding windows are served by the m16n8k16 kernel: engine None or mma.sync")
        if shards is not None and sinks is not None:
            raise NotImplementedError("a sharded context's merge does not take sinks")
        if sliding < 0:
            raise ValueError("sliding is the number of positions a column sees, 0 for all")
        if sinks is not None:
            sinks = _cuda(sinks, "sinks").reshape(-1)
            if sinks.numel() != hq:
                raise ValueError(f"sinks are one logit a query head ({hq}), not {sinks.numel()}")
            sinks = sinks.float().contiguous()
        engine = "mma.sync"
    if context:
        engine = "mma.sync"
    chosen = engine is None
    if chosen and (shards is not None or persistent or staging is not None):
        engine = "mma.sync"               # what those arguments are about
    engine = engine_for(kind, d, dv, hq, hkv, int(columns), R, positions, engine)
    chunk = int(chunk or chunk_for(d, dv, hq, hkv, page, kind, engine, int(columns)))
    if partitions:
        chunk = max(chunk, -(-positions // int(partitions)))
    chunk = -(-chunk // TILE) * TILE
    if chosen and ((engine == "tcgen05p" and not tcgen05p_serves(kind, d, dv, hq, hkv, int(columns), chunk, R)) or
                   (engine == "tcgen05" and not tcgen05_serves(kind, d, dv, hq, hkv, int(columns), chunk, R))):
        engine = "mma.sync"               # the caller's chunk is not one the chosen kernel takes
    splits = states_for(parts_for(positions, chunk), engine)
    partial_rows = R * columns if offsets is None else int(tokens)
    out = torch.empty(T, hq, dv, dtype=q.dtype, device=device) if out is None else out
    if out.dtype != q.dtype or out.stride(-1) != 1:
        raise ValueError("out is in q's dtype, its last dimension contiguous")
    p = _lib.AttendParams()
    if splits > 1 or shards is not None or sinks is not None:
        floats = workspace_floats(partial_rows, hq, splits, dv)
        space = _workspace(device, floats, workspace)
        p.workspace, p.workspace_floats = _ptr(space), space.numel()
    p.q, p.out, p.lse = _ptr(q), _ptr(out), _ptr(lse)
    if lse is not None and (lse.dtype != torch.float32 or not lse.is_contiguous() or tuple(lse.shape) != (T, hq)):
        raise ValueError(f"lse is contiguous FP32 [{T}][{hq}]")
    p.key_pages, p.value_pages = _ptr(key_pages), _ptr(value_pages)
    p.key_scales, p.value_scales = _ptr(key_scales), _ptr(value_scales)
    p.tables, p.rows, p.starts, p.counts = _ptr(tables), _ptr(rows), _ptr(starts), _ptr(counts)
    p.firsts, p.offsets = _ptr(firsts), _ptr(offsets)
    p.q_stride_token, p.q_stride_head = q.stride(0), q.stride(1)
    p.out_stride_token, p.out_stride_head = out.stride(0), out.stride(1)
    p.table_stride = tables.stride(0)
    p.n_rows, p.columns, p.partial_rows = R, int(columns), partial_rows
    p.q_heads, p.kv_heads, p.head_dim, p.value_dim, p.page = hq, hkv, d, dv, page
    p.kind, p.page_dtype, p.q_dtype = k_kind, _page_dtype(kind, key_pages), _DTYPES[q.dtype]
    p.chunk, p.max_splits = chunk, splits
    p.slots = key_pages.numel() // (hkv * d)
    if staging not in (None, "tma", "cp.async"):
        raise ValueError("staging is None, tma or cp.async")
    p.flags = ({None: 0, "cp.async": 1, "tma": 2}[staging] | (4 if persistent else 0) |
               {"tcgen05": 8, "mma.sync": 16, "tcgen05t": 64, "tcgen05p": 128}[engine] | (32 if shards is not None else 0) | (256 if context else 0))
    p.status = _ptr(_status_word(device))
    p.scale = float(scale if scale is not None else d ** -0.5)
    p.key_multiplier, p.value_multiplier = float(multipliers[0]), float(multipliers[1])
    p.parents, p.sinks, p.sliding = _ptr(parents), _ptr(sinks), sliding
    if blocks is not None:
        p.blocks, p.blocks_k, p.block_size = _ptr(blocks), blocks.shape[1], int(block_size)
    lib = _lib.load()
    if shards is not None:
        if lse is None:
            raise ValueError("a sharded context's merge writes lse too: pass lse")
        with torch.cuda.device(device):
            if launch in ("both", "decode", "push"):
                _lib.check(lib.crit_b200_decode(ctypes.byref(p), _stream(device)), "crit_b200.attend")
            if launch in ("both", "merge"):
                shards.attend(p, out, lse)
            elif launch == "push":             # decode and fold + push, no wait: a measurement's
                shards.attend(p, out, lse, wait=False)
        return out
    call = {"both": lib.crit_b200_attend, "decode": lib.crit_b200_decode, "merge": lib.crit_b200_merge}[launch]
    with torch.cuda.device(device):
        _lib.check(call(ctypes.byref(p), _stream(device)), "crit_b200.attend")
    return out


def merge_shards(outs, lses, dtype=None):
    """Partials of the same queries over disjoint keys (outs [parts][tokens][heads][dim], lses [parts][tokens][heads]
    FP32, -inf for a part with no key) -> (out [tokens][heads][dim], lse): the parts weighted by exp(lse - max); a
    token no part saw gets zeros and -inf.  Reference: inference/partitioned-attention/plugin.py:52-64."""
    if not torch.is_tensor(outs):
        outs = torch.stack(list(outs))
    if not torch.is_tensor(lses):
        lses = torch.stack(list(lses))
    _cuda(outs, "outs")
    outs, lses = outs.contiguous(), lses.float().contiguous()
    if outs.dtype not in _DTYPES:
        outs = outs.float()
    parts, dim = outs.shape[0], outs.shape[-1]
    n = lses[0].numel()
    dtype = dtype or torch.float32
    out = torch.empty(outs.shape[1:], dtype=dtype, device=outs.device)
    lse = torch.empty(lses.shape[1:], dtype=torch.float32, device=outs.device)
    p = _lib.MergeShardsParams()
    p.outs, p.lses, p.out, p.lse = _ptr(outs), _ptr(lses), _ptr(out), _ptr(lse)
    p.n, p.parts, p.dim, p.in_dtype, p.out_dtype = n, parts, dim, _DTYPES[outs.dtype], _DTYPES[dtype]
    with torch.cuda.device(outs.device):
        _lib.check(_lib.load().crit_b200_merge_shards(ctypes.byref(p), _stream(outs.device)), "crit_b200.merge_shards")
    return out, lse


def prefill_serves(head_dim, value_dim, q_dtype, kind, page):
    """Whether prefill() reads a cache of this geometry (else prompt rows go through attend in pieces)."""
    widths = (64, 128, 256) if kind in ("bf16", "fp16") else (64, 128)        # 256-wide heads: 16-bit pages (m16n8k16 tiles)
    return head_dim == value_dim and head_dim in widths and page % TILE == 0 and kind in KINDS and \
        q_dtype in (torch.bfloat16, torch.float16)


# -- prompt chunks ------------------------------------------------------------------------------------------------------
def prefill(q, key_pages, value_pages, kind, table, position, page, *, key_scales=None, value_scales=None,
            multipliers=(1.0, 1.0), scale=None, out=None, lse=None, int8_qk=False, fresh=None, flash=False,
            sinks=None, sliding=0, splits=None, workspace=None, derive=None, engine=None, starts=None):
    """A prompt chunk of one sequence: q [T][heads][dim] at positions position.. (their keys and values written),
    table [pages] int32 (or int64) -> out [T][heads][dim] in q's dtype (and lse [T][heads] FP32 when given), causal.  position: an
    int, or a one-element int64 device tensor read on the device.  Several sequences' chunks in ONE launch: table
    [S][pages], position a list of S ints or an int64 device tensor [S], q the sequences' tokens one after another
    (equal counts, or `starts`: S + 1 ints, sequence s's tokens being rows starts[s]..starts[s+1]).  engine: None
    (tcgen05.mma tiles with TMEM accumulators for 16-bit pages of 128-wide heads, m16n8k16 tiles otherwise), "mma.sync"
    or "tcgen05" (refused where not served); "tcgen05:single" / "tcgen05:pair" also name the block shape (128 query rows
    two blocks an SM / 256 rows over one ring of key and value tiles, which "tcgen05" picks by the launch's size).
    Reference: paged_kv_attention/__init__.py:1245-1332."""
    _refuse(int8_qk=int8_qk, fresh=fresh, sinks=sinks, sliding=sliding, derive=derive)
    k_kind = _check_kind(kind, key_scales)
    _cuda(q, "q")
    T, hq, d = q.shape
    hkv = key_pages.shape[-2]
    if value_pages.shape[-1] != d:
        raise ValueError("prompt chunks read keys and values of one width")
    if not key_pages.is_contiguous() or not value_pages.is_contiguous():
        raise ValueError("pages are contiguous [slots][kv_heads][dim] storage")
    out = torch.empty_like(q) if out is None else out
    if table.dtype not in (torch.int32, torch.int64) or table.dim() not in (1, 2):
        raise ValueError("table is the sequence's page ids, int32 (read in place) or int64 (converted)")
    if table.dtype != torch.int32 or not table.is_contiguous():
        table = table.to(torch.int32).contiguous()       # (the reference's pool hands its tables over as int64 slices)
    if q.stride(-1) != 1 or out.stride(-1) != 1:
        raise ValueError("q and out have contiguous last dimensions")
    p = _lib.PrefillParams()
    if table.dim() == 2:             # several sequences, one launch
        S = table.shape[0]
        if not torch.is_tensor(position):
            if len(position) != S:
                raise ValueError("one position a sequence")
            position = torch.tensor([int(x) for x in position], dtype=torch.int64, device=q.device)
        if position.dtype != torch.int64 or position.numel() != S or not position.is_cuda or not position.is_contiguous():
            raise ValueError("the sequences' positions are an int64 tensor [S] on the device")
        if starts is None:
            if T % S:
                raise ValueError("sequences of unequal token counts give `starts`")
            most = T // S
        else:
            starts = [int(x) for x in starts]
            if len(starts) != S + 1 or starts[0] != 0 or starts[-1] != T or any(b < a for a, b in zip(starts, starts[1:])):
                raise ValueError("starts: S + 1 rising row numbers from 0 to the number of tokens")
            most = max(b - a for a, b in zip(starts, starts[1:]))
            starts = torch.tensor(starts, dtype=torch.int32, device=q.device)
            p.starts = _ptr(starts)
        p.positions, p.sequences, p.table_stride = _ptr(position), S, table.stride(0)
        T, position = most, 0
    elif starts is not None:
        raise ValueError("starts goes with a table of several sequences")
    if torch.is_tensor(position) and (position.dtype != torch.int64 or position.numel() != 1 or not position.is_cuda):
        raise ValueError("a position read on the device is a one-element int64 tensor there")
    p.q, p.out, p.lse = _ptr(q), _ptr(out), _ptr(lse)
    p.key_pages, p.value_pages = _ptr(key_pages), _ptr(value_pages)
    p.key_scales, p.value_scales = _ptr(key_scales), _ptr(value_scales)
    p.table = _ptr(table)
    if torch.is_tensor(position):
        p.position_ptr = _ptr(position)
    else:
        p.position = int(position)
    p.q_stride_token, p.q_stride_head = q.stride(0), q.stride(1)
    p.out_stride_token, p.out_stride_head = out.stride(0), out.stride(1)
    p.slots = key_pages.numel() // (hkv * d)
    p.flags = {None: 0, "mma.sync": 1, "tcgen05": 2, "tcgen05:single": 2 | 4, "tcgen05:pair": 2 | 8}[engine]
    p.status = _ptr(_status_word(q.device))
    p.tokens, p.q_heads, p.kv_heads, p.head_dim, p.value_dim, p.page = T, hq, hkv, d, d, int(page)
    p.kind, p.page_dtype, p.q_dtype = k_kind, _page_dtype(kind, key_pages), _DTYPES[q.dtype]
    p.scale = float(scale if scale is not None else d ** -0.5)
    p.key_multiplier, p.value_multiplier = float(multipliers[0]), float(multipliers[1])
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().crit_b200_prefill(ctypes.byref(p), _stream(q.device)), "crit_b200.prefill")
    return out
