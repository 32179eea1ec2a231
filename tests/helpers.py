"""Shared pieces of the GPU parity tests: one layer's pages over shuffled page tables, written through the product's
write(), and the same pages as the CPU oracle reads them."""
import math

import numpy as np
import torch

import crit_b200 as pk
import oracle

STORE = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp8": torch.float8_e4m3fn, "fp8:row": torch.float8_e4m3fn,
         "int8": torch.int8, "fp8:page": torch.float8_e4m3fn}


class Cache:
    """Pages of several sequences, each over shuffled pages (the last page index is left unused, as a dump page)."""

    def __init__(self, kind, hkv, d, dv, page, lengths, seed=0, multipliers=(0.02, 0.03), spare=1, outliers=False,
                 poison=False):
        """poison: every byte of the pages and scales is 0xFF (NaN codes, NaN scales) before the sequences are written,
        so whatever a kernel reads past a row's last position is a NaN."""
        self.dev = torch.device("cuda")
        g = torch.Generator().manual_seed(seed)
        self.kind, self.hkv, self.d, self.dv, self.page = kind, hkv, d, dv, page
        self.multipliers = multipliers if kind == "fp8" else (1.0, 1.0)
        width = max(math.ceil((n + spare) / page) for n in lengths)
        n_pages = width * len(lengths) + 3
        self.k = torch.zeros(n_pages, page, hkv, d, dtype=STORE[kind], device=self.dev)
        self.v = torch.zeros(n_pages, page, hkv, dv, dtype=STORE[kind], device=self.dev)
        self.ks = self.vs = None
        if kind in ("fp8:row", "int8"):
            self.ks = torch.zeros(n_pages, page, hkv, dtype=torch.float32, device=self.dev)
            self.vs = torch.zeros_like(self.ks)
        elif kind == "fp8:page":
            self.ks = torch.zeros(n_pages, hkv, dtype=torch.float32, device=self.dev)
            self.vs = torch.zeros_like(self.ks)
        if poison:
            for t in (self.k, self.v, self.ks, self.vs):
                if t is not None:
                    t.view(torch.uint8).fill_(0xFF)
        order = torch.randperm(n_pages - 1, generator=g)
        self.tables = order[:width * len(lengths)].view(len(lengths), width).to(torch.int32).to(self.dev)
        self.lengths = list(lengths)
        for s, n in enumerate(lengths):
            keys, values = torch.randn(n, hkv, d, generator=g), torch.randn(n, hkv, dv, generator=g)
            if outliers:
                keys = torch.where(torch.rand(keys.shape, generator=g) < 0.01, keys * 20, keys)
                values = torch.where(torch.rand(values.shape, generator=g) < 0.01, values * 20, values)
            self.write(s, 0, keys.to(self.dev).bfloat16(), values.to(self.dev).bfloat16())

    def slots(self, s, positions):
        positions = torch.as_tensor(positions, device=self.dev)
        return self.tables[s][positions // self.page].long() * self.page + positions % self.page

    def write(self, s, start, keys, values):
        slots = self.slots(s, torch.arange(start, start + keys.shape[0], device=self.dev))
        pk.write(keys, values, slots, self.k, self.v, self.kind, self.ks, self.vs, multipliers=self.multipliers)

    def stored(self):
        """The pages as FP32 values [slots][hkv][dim], as the oracle reads them."""
        found = []
        for pages, scales, mult in ((self.k, self.ks, self.multipliers[0]), (self.v, self.vs, self.multipliers[1])):
            dim = pages.shape[-1]
            if pk.KINDS[self.kind] == 0:
                found.append(pages.float().cpu().numpy().reshape(-1, self.hkv, dim))
                continue
            codes = pages.view(torch.uint8).cpu().numpy().reshape(-1, self.hkv, dim)
            sc = scales.cpu().numpy() if scales is not None else None
            if sc is not None and self.kind != "fp8:page":
                sc = sc.reshape(-1, self.hkv)
            found.append(oracle.dequantize(codes, self.kind, sc, mult, page=self.page))
        return found

    def attend(self, q, rows, starts, firsts, columns, counts=None, **kw):
        i32 = dict(dtype=torch.int32, device=self.dev)
        if counts is not None:
            counts = torch.tensor(counts, **i32)
        return pk.attend(q, self.k, self.v, self.kind, self.tables, torch.tensor(rows, **i32),
                         torch.tensor(starts, **i32), torch.tensor(firsts, dtype=torch.int64, device=self.dev), columns,
                         self.page, counts=counts, key_scales=self.ks, value_scales=self.vs,
                         multipliers=self.multipliers, **kw)

    def oracle(self, q, rows, starts, firsts, columns, counts=None, scale=None):
        k, v = self.stored()
        return oracle.attend(q.float().cpu().numpy(), k, v, self.tables.cpu().numpy(), rows, starts, firsts, columns,
                             self.page, scale=scale, counts=counts)


def queries(tokens, hq, d, seed, dtype=torch.bfloat16):
    return torch.randn(tokens, hq, d, generator=torch.Generator().manual_seed(seed)).to("cuda").to(dtype)


def assert_attention_close(out, lse, want, want_lse, rows_tokens, max_abs=2e-2, mean_abs=2e-3, lse_abs=2e-3, rel=0.0):
    """The north-star bound in bf16: max-abs 2e-2 and mean-abs 2e-3 against the oracle, over the tokens the rows name.
    rel: for inputs with outliers, whose outputs reach magnitudes where bf16's own spacing passes 2e-2 (0.125 at 16),
    each error is first divided by 1 + rel * |want| / max_abs, i.e. the bound becomes max_abs + rel * |want|."""
    got = out.float().cpu().numpy()[rows_tokens]
    want = want[rows_tokens]
    err = np.abs(got - want) / (1.0 + (rel / max_abs) * np.abs(want))
    assert np.isfinite(got).all()
    assert err.max() <= max_abs, f"max-abs {err.max():.4g}"
    assert err.mean() <= mean_abs, f"mean-abs {err.mean():.4g}"
    if lse is not None:
        gl, wl = lse.cpu().numpy()[rows_tokens], want_lse[rows_tokens]
        assert np.abs(gl - wl).max() <= lse_abs, f"lse {np.abs(gl - wl).max():.4g}"


def attend_params(cache, q, out, lse, rows, starts, firsts, columns, chunk, workspace=None, counts=None, flags=0,
                  partial_rows=None, offsets=None, status=None):
    """The parameter block of include/crit_b200.h for one launch over a Cache, filled as crit_b200.attend fills it: for
    tests that call the C ABI themselves.  Returns (params, the tensors the block points at: keep them alive)."""
    from crit_b200 import _lib
    dev = q.device
    i32 = dict(dtype=torch.int32, device=dev)
    held = dict(rows=torch.tensor(rows, **i32), starts=torch.tensor(starts, **i32),
                firsts=torch.tensor(firsts, dtype=torch.int64, device=dev))
    T, hq, d = q.shape
    positions = cache.tables.shape[1] * cache.page
    p = _lib.AttendParams()
    p.q, p.out = q.data_ptr(), out.data_ptr()
    p.lse = lse.data_ptr() if lse is not None else None
    p.key_pages, p.value_pages = cache.k.data_ptr(), cache.v.data_ptr()
    if cache.ks is not None:
        p.key_scales, p.value_scales = cache.ks.data_ptr(), cache.vs.data_ptr()
    p.tables, p.rows, p.starts, p.firsts = (cache.tables.data_ptr(), held["rows"].data_ptr(), held["starts"].data_ptr(),
                                            held["firsts"].data_ptr())
    if counts is not None:
        held["counts"] = torch.tensor(counts, **i32)
        p.counts = held["counts"].data_ptr()
    if offsets is not None:
        held["offsets"] = torch.tensor(offsets, **i32)
        p.offsets = held["offsets"].data_ptr()
    if status is not None:
        p.status = status.data_ptr()
    p.q_stride_token, p.q_stride_head = q.stride(0), q.stride(1)
    p.out_stride_token, p.out_stride_head = out.stride(0), out.stride(1)
    p.table_stride = cache.tables.stride(0)
    p.n_rows, p.columns = len(rows), columns
    p.partial_rows = len(rows) * columns if partial_rows is None else partial_rows
    p.q_heads, p.kv_heads, p.head_dim, p.value_dim, p.page = hq, cache.hkv, d, cache.dv, cache.page
    p.kind, p.page_dtype = pk.KINDS[cache.kind], _lib.DTYPE_FP16 if cache.kind == "fp16" else _lib.DTYPE_BF16
    p.q_dtype = _lib.DTYPE_FP16 if q.dtype == torch.float16 else _lib.DTYPE_BF16
    p.chunk, p.max_splits = chunk, -(-positions // chunk)
    p.slots = cache.k.numel() // (cache.hkv * d)
    p.flags = flags
    p.scale = d ** -0.5
    p.key_multiplier, p.value_multiplier = cache.multipliers
    if workspace is not None:
        p.workspace, p.workspace_floats = workspace.data_ptr(), workspace.numel()
    return p, held


class Guarded:
    """A CUDA buffer between two guard regions filled with 0xFF bytes: a kernel that writes outside what it was given
    leaves a mark that intact() finds."""

    def __init__(self, nbytes, guard=4096, fill=0):
        self.nbytes, self.guard = int(nbytes), guard
        padded = -(-self.nbytes // 256) * 256
        self.raw = torch.full((padded + 2 * guard,), 0xFF, dtype=torch.uint8, device="cuda")
        self.bytes = self.raw[guard:guard + self.nbytes]
        self.bytes.fill_(fill)

    def view(self, dtype, *shape):
        return self.bytes.view(dtype).view(*shape)

    def intact(self):
        front, back = self.raw[:self.guard], self.raw[self.guard + self.nbytes:]
        return bool((front == 0xFF).all()) and bool((back == 0xFF).all())


class EmulatedRanks:
    """The peer exchange of `world` ranks on ONE GPU: every rank's exchange buffer lives on this device and the ranks'
    launches run one after another on one stream (a push never waits, so this order cannot block; a wait runs after the
    pushes it needs).  What two or more GPUs do with peer stores, minus the wire."""

    def __init__(self, world, tokens, heads, dim, wait_ms=50):
        import ctypes
        from crit_b200 import _lib
        self.ctypes, self.lib, self._lib = ctypes, _lib.load(), _lib
        self.world, self.n, self.dim = world, tokens * heads, dim
        self.floats = self.n * (dim + 1) + 3
        size = self.lib.crit_b200_exchange_bytes(world, self.floats)
        dev = torch.device("cuda")
        self.buffers = [torch.zeros(size // 4, dtype=torch.float32, device=dev) for _ in range(world)]
        self.peers = torch.tensor([b.data_ptr() for b in self.buffers], dtype=torch.int64, device=dev)
        self.steps = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(world)]
        self.status = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(world)]
        self.params = []
        for r in range(world):
            x = _lib.ExchangeParams()
            x.peers, x.step, x.status = self.peers.data_ptr(), self.steps[r].data_ptr(), self.status[r].data_ptr()
            x.floats, x.wait_ns, x.world, x.rank = self.floats, int(wait_ms) * 1000000, world, r
            self.params.append(x)

    def _stream(self):
        return self.ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def push(self, rank, attend_params):
        """Rank `rank` folds the split states its decode launch left and stores the result into every rank's buffer."""
        code = self.lib.crit_b200_merge_push(self.ctypes.byref(attend_params), self.ctypes.byref(self.params[rank]), self._stream())
        assert code == 0, self.lib.crit_b200_error(code)

    def exchange_merge(self, rank, attend_params, out, lse):
        """Fold + push and wait + merge in one call (one launch where the step's blocks are all resident): only a world
        of one rank can run it on one GPU, since the wait needs every rank's push."""
        code = self.lib.crit_b200_exchange_merge(self.ctypes.byref(attend_params), self.ctypes.byref(self.params[rank]),
                                                 self.ctypes.byref(self._merge_params(out, lse)), self._stream())
        assert code == 0, self.lib.crit_b200_error(code)

    def _merge_params(self, out, lse):
        m = self._lib.MergeShardsParams()
        m.out, m.lse, m.n, m.parts, m.dim = out.data_ptr(), lse.data_ptr(), self.n, self.world, self.dim
        m.in_dtype = self._lib.DTYPE_FP32
        m.out_dtype = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[out.dtype]
        return m

    def wait_merge(self, rank, out, lse):
        m = self._lib.MergeShardsParams()
        m.out, m.lse, m.n, m.parts, m.dim = out.data_ptr(), lse.data_ptr(), self.n, self.world, self.dim
        m.in_dtype = self._lib.DTYPE_FP32
        m.out_dtype = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[out.dtype]
        code = self.lib.crit_b200_wait_merge(self.ctypes.byref(self.params[rank]), self.ctypes.byref(m), self._stream())
        assert code == 0, self.lib.crit_b200_error(code)
