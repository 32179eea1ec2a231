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

    def __init__(self, kind, hkv, d, dv, page, lengths, seed=0, multipliers=(0.02, 0.03), spare=1, outliers=False):
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
