"""Parity of the CUDA kernels, called through the C ABI, against the CPU oracle and the golden fixtures: appends and
slot maps bit for bit, attention within max-abs 2e-2 / mean-abs 2e-3 (bf16)."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pk():
    import crit_b200
    return crit_b200


def _dev():
    return torch.device("cuda")


# -- KV append ----------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["bf16", "fp16", "fp8", "fp8:row", "int8"])
@pytest.mark.parametrize("d,dv", [(128, 128), (64, 128), (256, 256)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_writes_encode_as_the_oracle_does_and_skip_negative_slots(pk, kind, d, dv, dtype):
    from helpers import STORE
    g = torch.Generator().manual_seed(1)
    keys, values = (torch.randn(40, 3, d, generator=g) * 3).to(dtype), torch.randn(40, 3, dv, generator=g).to(dtype)
    keys[5] = 0.0
    dev = _dev()
    k = torch.zeros(64, 3, d, dtype=STORE[kind], device=dev)
    v = torch.zeros(64, 3, dv, dtype=STORE[kind], device=dev)
    ks = vs = None
    if kind in ("fp8:row", "int8"):
        ks, vs = torch.zeros(64, 3, device=dev), torch.zeros(64, 3, device=dev)
    slots = torch.randperm(64, generator=g)[:40]
    slots[7] = -1
    mult = (0.05, 0.07)
    pk.write(keys.to(dev), values.to(dev), slots.to(dev), k, v, kind, ks, vs, multipliers=mult)
    keep = (slots >= 0).numpy()
    at = slots.numpy()[keep]
    for x, store, scales, m in ((keys, k, ks, mult[0]), (values, v, vs, mult[1])):
        x = x.float().numpy()[keep]
        if kind in ("bf16", "fp16"):
            want = torch.from_numpy(x).to(STORE[kind])
            assert torch.equal(store.cpu()[at], want)
        else:
            want, want_scale = oracle.quantize_rows(x, kind, m)
            assert np.array_equal(store.view(torch.uint8).cpu().numpy()[at], want)
            if want_scale is not None:
                assert np.array_equal(scales.cpu().numpy()[at].view(np.uint32), want_scale.view(np.uint32))
        untouched = np.ones(64, bool)
        untouched[at] = False
        assert not store.view(torch.uint8 if store.element_size() == 1 else torch.int16).cpu().numpy()[untouched].any()
    if kind == "fp8:row":
        assert ks.cpu()[slots[5]].tolist() == [float(np.float32(1e-30))] * 3


def test_writes_match_the_references_golden_codes(pk, golden):
    data = golden("quantize.npz")
    x = torch.from_numpy(data["x"]).cuda()
    n, h, d = x.shape
    slots = torch.arange(n, device="cuda")
    for kind, codes, scales in (("fp8:row", "fp8row_codes", "fp8row_scales"), ("int8", "int8_codes", "int8_scales"),
                                ("fp8", "static_codes", None)):
        store = torch.zeros(n, h, d, dtype=torch.uint8, device="cuda")
        sc = torch.zeros(n, h, device="cuda") if scales else None
        pages = store.view(torch.float8_e4m3fn) if kind != "int8" else store.view(torch.int8)
        m = float(data["static_multiplier"])
        pk.write(x, None, slots, pages, None, kind, sc, None, multipliers=(m, m))
        assert np.array_equal(store.cpu().numpy(), data[codes].view(np.uint8)), kind
        if scales:
            assert np.array_equal(sc.cpu().numpy().view(np.uint32), data[scales].view(np.uint32)), kind


def test_page_scaled_writes_follow_the_oracle_through_appends(pk):
    page, hkv, d = 16, 2, 128
    g = torch.Generator().manual_seed(4)
    n_pages = 6
    k = torch.zeros(n_pages, page, hkv, d, dtype=torch.float8_e4m3fn, device="cuda")
    v = torch.zeros_like(k)
    ks, vs = torch.zeros(n_pages, hkv, device="cuda"), torch.zeros(n_pages, hkv, device="cuda")
    ok, ov = np.zeros((n_pages * page, hkv, d), np.uint8), np.zeros((n_pages * page, hkv, d), np.uint8)
    oks, ovs = np.zeros((n_pages, hkv), np.float32), np.zeros((n_pages, hkv), np.float32)
    table = [4, 1, 3, 0]
    slot = lambda p: table[p // page] * page + p % page
    at = 0
    # a prompt of 37 tokens, then decode tokens of growing magnitude (the tail page's scale grows and re-encodes)
    for count, mag in ((37, 1.0), (1, 0.5), (1, 3.0), (3, 9.0), (1, 1.0), (8, 30.0), (1, 0.1)):
        keys = (torch.randn(count, hkv, d, generator=g) * mag).bfloat16()
        values = (torch.randn(count, hkv, d, generator=g) * mag).bfloat16()
        slots = torch.tensor([slot(p) for p in range(at, at + count)])
        pk.write(keys.cuda(), values.cuda(), slots.cuda(), k, v, "fp8:page", ks, vs)
        oracle.quantize_pages(keys.float().numpy(), slots.numpy(), page, ok, oks)
        oracle.quantize_pages(values.float().numpy(), slots.numpy(), page, ov, ovs)
        at += count
        assert np.array_equal(k.view(torch.uint8).cpu().numpy().reshape(-1, hkv, d), ok), (count, mag)
        assert np.array_equal(v.view(torch.uint8).cpu().numpy().reshape(-1, hkv, d), ov), (count, mag)
        assert np.array_equal(ks.cpu().numpy().view(np.uint32), oks.view(np.uint32))
        assert np.array_equal(vs.cpu().numpy().view(np.uint32), ovs.view(np.uint32))


# -- gather, slots --------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["bf16", "fp8", "fp8:row", "int8", "fp8:page"])
def test_gather_reads_pages_back_through_the_table(pk, kind):
    from helpers import Cache
    cache = Cache(kind, 2, 64, 64, 16, [70, 33])
    k, v = cache.stored()
    for s, n in enumerate(cache.lengths):
        at = cache.slots(s, torch.arange(n)).cpu().numpy()
        for pages, scales, want, mult in ((cache.k, cache.ks, k, cache.multipliers[0]),
                                          (cache.v, cache.vs, v, cache.multipliers[1])):
            got = pk.gather(pages, kind, 16, table=cache.tables[s], count=n, scales=scales, multiplier=mult,
                            dtype=torch.float32)
            assert np.array_equal(got.cpu().numpy(), want[at])
            rounded = pk.gather(pages, kind, 16, table=cache.tables[s], count=n, scales=scales, multiplier=mult)
            assert torch.equal(rounded.cpu(), torch.from_numpy(want[at]).bfloat16())
            picked = pk.gather(pages, kind, 16, slots=torch.from_numpy(at[::3].copy()).cuda().view(-1, 1), scales=scales,
                               multiplier=mult, dtype=torch.float32)
            assert np.array_equal(picked.cpu().numpy()[:, 0], want[at[::3]])


def test_round_slots_match_the_references(pk, golden):
    data = golden("round_slots.npz")
    got = pk.slots_at(torch.from_numpy(data["tables"]).cuda(), torch.from_numpy(data["slot"]).cuda(),
                      torch.from_numpy(data["positions"]).cuda(), int(data["page"]), int(data["dump"]),
                      capacity=torch.from_numpy(data["capacity"]).cuda())
    assert np.array_equal(got.cpu().numpy(), data["slots"])


# -- decode and verify windows --------------------------------------------------------------------------------------------
SHAPES = [(8, 2, 128, 128), (24, 4, 256, 256), (56, 8, 128, 128), (12, 2, 64, 64), (40, 8, 128, 128)]


@pytest.mark.parametrize("kind", ["bf16", "fp16", "fp8", "fp8:row", "int8", "fp8:page"])
@pytest.mark.parametrize("hq,hkv,d,dv", SHAPES)
@pytest.mark.parametrize("page", [16, 48])
def test_windows_match_the_oracle(pk, kind, hq, hkv, d, dv, page):
    from helpers import Cache, assert_attention_close, queries
    cache = Cache(kind, hkv, d, dv, page, [130, 64, 1, 517])
    cols = 5
    rows, starts, firsts, counts = [0, 1, 2, 3], [0, 5, 10, 15], [125, 59, 0, 400], [5, 5, 1, 3]
    q = queries(20, hq, d, 3, torch.float16 if kind == "fp16" else torch.bfloat16)
    lse = torch.full((20, hq), 7.0, device="cuda")
    out = cache.attend(q, rows, starts, firsts, cols, counts=counts, lse=lse, chunk=128)
    want, want_lse = cache.oracle(q, rows, starts, firsts, cols, counts=counts)
    tokens = [s + c for s, n in zip(starts, counts) for c in range(n)]
    assert_attention_close(out, lse, want, want_lse, tokens)


# The tcgen05 engine: E4M3 page bytes straight into the tensor cores; the queries and probabilities enter as two E4M3
# terms each (an error below 2^-8 of each value, like bf16's own rounding), so the same bounds hold.
TC_ENGINES = ["tcgen05", "tcgen05t"]       # the query rows on the MMA's rows (replicated), or on its columns (operands swapped)


@pytest.mark.parametrize("engine", TC_ENGINES)
@pytest.mark.parametrize("kind", ["fp8", "fp8:row", "fp8:page"])
@pytest.mark.parametrize("hq,hkv", [(8, 2), (56, 8), (40, 8), (4, 4), (16, 1)])
@pytest.mark.parametrize("page,chunk", [(16, 128), (48, 256), (16, 1024)])
def test_windows_on_tcgen05_tiles_match_the_oracle(pk, kind, hq, hkv, page, chunk, engine):
    from helpers import Cache, assert_attention_close, queries
    cache = Cache(kind, hkv, 128, 128, page, [130, 64, 1, 517, 1300])
    G = hq // hkv
    cols = max(1, min(5, 32 // G))
    firsts = [125, 59, 0, 400, 1290]
    counts = [min(cols, n) for n in [5, 5, 1, 3, 5]]
    rows, starts = [0, 1, 2, 3, 4], [0, 5, 10, 15, 20]
    q = queries(25, hq, 128, 3)
    lse = torch.full((25, hq), 7.0, device="cuda")
    out = cache.attend(q, rows, starts, firsts, cols, counts=counts, lse=lse, chunk=chunk, engine=engine)
    assert pk.status() == 0
    want, want_lse = cache.oracle(q, rows, starts, firsts, cols, counts=counts)
    tokens = [s + c for s, n in zip(starts, counts) for c in range(n)]
    assert_attention_close(out, lse, want, want_lse, tokens)


@pytest.mark.parametrize("engine", TC_ENGINES)
@pytest.mark.parametrize("kind", ["fp8:page", "fp8:row"])
def test_tcgen05_tiles_with_outliers_and_long_rows(pk, kind, engine):
    from helpers import Cache, assert_attention_close, queries
    cache = Cache(kind, 2, 128, 128, 16, [1000, 37, 16, 2049, 5000], outliers=True)
    q = queries(5, 16, 128, 9)      # bf16 queries split into two E4M3 terms exactly; fp16 ones keep 8 of their 11 bits
    rows, starts, firsts = [0, 1, 2, 3, 4], [0, 1, 2, 3, 4], [999, 36, 15, 2048, 4999]
    lse = torch.empty(5, 16, device="cuda")
    out = cache.attend(q, rows, starts, firsts, 1, lse=lse, chunk=1024, engine=engine)
    assert pk.status() == 0
    want, want_lse = cache.oracle(q, rows, starts, firsts, 1)
    assert_attention_close(out, lse, want, want_lse, [0, 1, 2, 3, 4], rel=2.0 ** -7)


@pytest.mark.parametrize("engine", TC_ENGINES)
def test_tcgen05_tiles_edge_cases(pk, engine):
    """The tcgen05 engine on the edges the m16n8k16 engine is held to: a NaN query stays in its own token, rows with no
    columns and counts past the columns, FP16 queries, packed partial rows, and a row alone against the row in a batch."""
    from helpers import Cache, assert_attention_close, queries
    cache = Cache("fp8:page", 2, 128, 128, 16, [200, 1300, 40], spare=8)
    q = queries(12, 8, 128, 2)
    rows, starts, firsts = [0, 1, 2], [0, 4, 8], [196, 1296, 36]
    clean = cache.attend(q, rows, starts, firsts, 4, engine=engine)
    q2 = q.clone()
    q2[5, 3, 7] = float("nan")
    got = cache.attend(q2, rows, starts, firsts, 4, engine=engine)
    assert torch.isnan(got[5, 3]).all()
    keep = torch.ones(12, 8, dtype=torch.bool)
    keep[5, 3] = False
    assert torch.equal(got.cpu()[keep], clean.cpu()[keep])
    # a row without columns writes nothing; a count past the columns reads as the columns
    marked = torch.full_like(clean, 7.0)
    some = cache.attend(q, rows, starts, firsts, 4, counts=[4, 0, 9], out=marked, engine=engine)
    assert torch.equal(some[0:4], clean[0:4]) and torch.equal(some[8:12], clean[8:12]) and bool((some[4:8] == 7.0).all())
    # FP16 queries keep 8 of their 11 significant bits in the split: inside the bounds
    qh = queries(12, 8, 128, 4, torch.float16)
    cache16 = Cache("fp8:row", 2, 128, 128, 16, [200, 1300, 40], spare=8)
    lse = torch.empty(12, 8, device="cuda")
    out = cache16.attend(qh, rows, starts, firsts, 4, lse=lse, engine=engine)
    want, want_lse = cache16.oracle(qh, rows, starts, firsts, 4)
    assert_attention_close(out, lse, want, want_lse, list(range(12)))
    # packed partial rows (offsets) fold to the same bits as padded ones
    offsets = torch.tensor([0, 2, 3], dtype=torch.int32, device="cuda")
    splits = pk.parts_for(cache.tables.shape[1] * 16, 256)
    space = torch.empty(pk.workspace_floats(7, 8, splits, 128), device="cuda")
    padded = cache.attend(q, rows, starts, firsts, 4, counts=[2, 1, 4], chunk=256, engine=engine)
    packed = cache.attend(q, rows, starts, firsts, 4, counts=[2, 1, 4], offsets=offsets, tokens=7, workspace=space, chunk=256,
                          engine=engine)
    for start, count in zip(starts, [2, 1, 4]):
        assert torch.equal(packed[start:start + count], padded[start:start + count])
    # a row alone and in a batch of the same columns: the same unit, the same bits
    alone = cache.attend(q[4:8], [1], [0], [1296], 4, engine=engine)
    assert torch.equal(alone, clean[4:8])
    assert pk.status() == 0


# The tcgen05 engine over whole page rows: a unit reads all 8 kv heads of its positions (one contiguous piece of HBM a
# tile), kv head h's query rows on TMEM lanes 16 h .. 16 h + 15.
@pytest.mark.parametrize("kind", ["fp8", "fp8:row", "fp8:page"])
@pytest.mark.parametrize("hq,cols", [(64, 1), (32, 2), (16, 4), (8, 5), (56, 1), (24, 2)])
@pytest.mark.parametrize("page,chunk", [(16, 16), (16, 128), (48, 256), (16, 1024), (64, 2048)])
def test_windows_on_whole_page_rows_match_the_oracle(pk, kind, hq, cols, page, chunk):
    from helpers import Cache, assert_attention_close, queries
    cache = Cache(kind, 8, 128, 128, page, [130, 64, 1, 517, 1300])
    firsts = [125, 59, 0, 400, 1290]
    counts = [min(cols, n) for n in [5, 5, 1, 3, 5]]
    rows, starts = [0, 1, 2, 3, 4], [0, 5, 10, 15, 20]
    q = queries(25, hq, 128, 3)
    lse = torch.full((25, hq), 7.0, device="cuda")
    out = cache.attend(q, rows, starts, firsts, cols, counts=counts, lse=lse, chunk=chunk, engine="tcgen05p")
    assert pk.status() == 0
    want, want_lse = cache.oracle(q, rows, starts, firsts, cols, counts=counts)
    tokens = [s + c for s, n in zip(starts, counts) for c in range(n)]
    assert_attention_close(out, lse, want, want_lse, tokens)


@pytest.mark.parametrize("kind", ["fp8:page", "fp8:row"])
def test_whole_page_rows_with_outliers_and_long_rows(pk, kind):
    from helpers import Cache, assert_attention_close, queries
    cache = Cache(kind, 8, 128, 128, 16, [1000, 37, 16, 2049, 5000], outliers=True)
    q = queries(5, 64, 128, 9)
    rows, starts, firsts = [0, 1, 2, 3, 4], [0, 1, 2, 3, 4], [999, 36, 15, 2048, 4999]
    lse = torch.empty(5, 64, device="cuda")
    out = cache.attend(q, rows, starts, firsts, 1, lse=lse, chunk=512, engine="tcgen05p")
    assert pk.status() == 0
    want, want_lse = cache.oracle(q, rows, starts, firsts, 1)
    assert_attention_close(out, lse, want, want_lse, [0, 1, 2, 3, 4], rel=2.0 ** -7)
    again = cache.attend(q, rows, starts, firsts, 1, chunk=512, engine="tcgen05p")
    assert torch.equal(out, again)                                       # the same launch twice: the same bits
    # a row alone is cut into other units than in a batch (the launch's tiles are dealt out evenly): other bits, the
    # same attention
    alone = cache.attend(q[3:4], [3], [0], [2048], 1, chunk=512, engine="tcgen05p")
    assert_attention_close(alone, None, want[3:4], None, [0], rel=2.0 ** -7)


def test_whole_page_rows_edge_cases(pk):
    """A NaN query stays in its own token, rows with no columns write nothing, FP16 queries, packed partial rows, and what
    the engine does not serve is refused."""
    from helpers import Cache, assert_attention_close, queries
    cache = Cache("fp8:page", 8, 128, 128, 16, [200, 1300, 40], spare=8)
    q = queries(12, 16, 128, 2)
    rows, starts, firsts = [0, 1, 2], [0, 4, 8], [196, 1296, 36]
    clean = cache.attend(q, rows, starts, firsts, 4, engine="tcgen05p", chunk=256)
    q2 = q.clone()
    q2[5, 3, 7] = float("nan")
    got = cache.attend(q2, rows, starts, firsts, 4, engine="tcgen05p", chunk=256)
    assert torch.isnan(got[5, 3]).all()
    keep = torch.ones(12, 16, dtype=torch.bool)
    keep[5, 3] = False
    assert torch.equal(got.cpu()[keep], clean.cpu()[keep])
    marked = torch.full_like(clean, 7.0)
    some = cache.attend(q, rows, starts, firsts, 4, counts=[4, 0, 9], out=marked, engine="tcgen05p", chunk=256)
    # (the launch's tiles are dealt out evenly, so other rows in the launch mean other units: the same attention, not the same bits)
    assert bool((some[4:8] == 7.0).all())
    assert float((some[0:4].float() - clean[0:4].float()).abs().max()) <= 1e-2
    assert float((some[8:12].float() - clean[8:12].float()).abs().max()) <= 1e-2
    qh = queries(12, 16, 128, 4, torch.float16)
    cache16 = Cache("fp8:row", 8, 128, 128, 16, [200, 1300, 40], spare=8)
    lse = torch.empty(12, 16, device="cuda")
    out = cache16.attend(qh, rows, starts, firsts, 4, lse=lse, engine="tcgen05p", chunk=256)
    want, want_lse = cache16.oracle(qh, rows, starts, firsts, 4)
    assert_attention_close(out, lse, want, want_lse, list(range(12)))
    offsets = torch.tensor([0, 2, 3], dtype=torch.int32, device="cuda")
    splits = pk.parts_for(cache.tables.shape[1] * 16, 256)
    space = torch.empty(pk.workspace_floats(7, 16, 2 * splits, 128), device="cuda")       # a split's head and tail
    padded = cache.attend(q, rows, starts, firsts, 4, counts=[2, 1, 4], chunk=256, engine="tcgen05p")
    packed = cache.attend(q, rows, starts, firsts, 4, counts=[2, 1, 4], offsets=offsets, tokens=7, workspace=space, chunk=256,
                          engine="tcgen05p")
    for start, count in zip(starts, [2, 1, 4]):
        assert torch.equal(packed[start:start + count], padded[start:start + count])
    assert pk.status() == 0
    with pytest.raises(Exception):        # 4 kv heads
        Cache("fp8:page", 4, 128, 128, 16, [100]).attend(queries(1, 8, 128, 1), [0], [0], [99], 1, engine="tcgen05p")
    with pytest.raises(Exception):        # 5 columns x 2 heads of a group: more than 8 query rows a kv head
        cache.attend(queries(5, 16, 128, 1), [0], [0], [95], 5, engine="tcgen05p")
    with pytest.raises(Exception):        # bf16 pages
        Cache("bf16", 8, 128, 128, 16, [100]).attend(queries(1, 8, 128, 1), [0], [0], [99], 1, engine="tcgen05p")


def test_tcgen05_tiles_refuse_launches_they_do_not_serve(pk):
    from helpers import Cache, queries
    cache = Cache("bf16", 2, 128, 128, 16, [100])
    with pytest.raises(Exception):
        cache.attend(queries(1, 8, 128, 1), [0], [0], [99], 1, engine="tcgen05")
    cache = Cache("fp8:page", 2, 128, 128, 16, [100])
    with pytest.raises(Exception):
        cache.attend(queries(1, 8, 128, 1), [0], [0], [99], 1, chunk=64, engine="tcgen05")
    with pytest.raises(Exception):        # 9 columns x 4 heads of a group: more than 32 query rows a unit
        cache.attend(queries(9, 8, 128, 1), [0], [0], [91], 9, engine="tcgen05")


@pytest.mark.parametrize("kind", ["bf16", "fp8:page"])
@pytest.mark.parametrize("chunk", [16, 64, 1024])
def test_splits_of_any_size_fold_to_the_same_attention(pk, kind, chunk):
    from helpers import Cache, assert_attention_close, queries
    cache = Cache(kind, 2, 128, 128, 16, [1000, 37, 16, 2049], outliers=True)
    q = queries(4, 16, 128, 9)
    rows, starts, firsts = [0, 1, 2, 3], [0, 1, 2, 3], [999, 36, 15, 2048]
    lse = torch.empty(4, 16, device="cuda")
    out = cache.attend(q, rows, starts, firsts, 1, lse=lse, chunk=chunk)
    want, want_lse = cache.oracle(q, rows, starts, firsts, 1)
    # outliers x20 in keys and values: outputs reach 30, where a bf16 output is 0.06 from its FP32 value and a bf16
    # probability 2^-9 of it: the bound is 2e-2 + 2^-7 |want|
    assert_attention_close(out, lse, want, want_lse, [0, 1, 2, 3], rel=2.0 ** -7)


@pytest.mark.parametrize("kind", ["bf16", "fp8:row"])
def test_a_column_decodes_the_same_alone_and_in_a_window(pk, kind):
    from helpers import Cache, queries
    cache = Cache(kind, 4, 128, 128, 16, [700, 300, 2100], spare=8)
    q = queries(24, 24, 128, 5)
    together = cache.attend(q, [0, 1, 2], [0, 8, 16], [690, 290, 2090], 8, chunk=256)
    for s, start, first in zip([0, 1, 2], [0, 8, 16], [690, 290, 2090]):
        alone = cache.attend(q[start:start + 8], [s], [0], [first], 8, chunk=256)
        assert torch.equal(alone, together[start:start + 8])
        for c in range(8):
            one = cache.attend(q[start + c:start + c + 1], [s], [0], [first + c], 1, chunk=256)
            assert torch.equal(one[0], together[start + c])
        wide = cache.attend(q[start:start + 8], [s], [0], [first], 16, counts=[8], chunk=256)
        assert torch.equal(wide, together[start:start + 8])


@pytest.mark.parametrize("kind", ["bf16", "fp16", "fp8", "fp8:row", "int8", "fp8:page"])
@pytest.mark.parametrize("hq,hkv,d", [(32, 4, 128), (24, 4, 256), (40, 8, 128)])
def test_tma_and_cp_async_staging_give_the_same_bits(pk, kind, hq, hkv, d):
    from helpers import Cache, assert_attention_close, queries
    cache = Cache(kind, hkv, d, d, 16, [130, 64, 1, 517, 1000], outliers=kind == "fp8:page")
    rows, starts, firsts, counts = [0, 1, 2, 3, 4], [0, 5, 10, 15, 20], [125, 59, 0, 400, 990], [5, 5, 1, 3, 6]
    q = queries(26, hq, d, 3, torch.float16 if kind == "fp16" else torch.bfloat16)
    lse_a, lse_b = torch.empty(26, hq, device="cuda"), torch.empty(26, hq, device="cuda")
    tma = cache.attend(q, rows, starts, firsts, 6, counts=counts, lse=lse_a, chunk=128, engine="mma.sync")
    plain = cache.attend(q, rows, starts, firsts, 6, counts=counts, lse=lse_b, chunk=128, staging="cp.async")
    tokens = [s + c for s, n in zip(starts, counts) for c in range(n)]
    assert torch.equal(tma[tokens], plain[tokens]) and torch.equal(lse_a[tokens], lse_b[tokens])
    # ... and persistent blocks over a device-built work list instead of one block per grid slot
    listed = cache.attend(q, rows, starts, firsts, 6, counts=counts, lse=lse_b, chunk=128, persistent=True)
    assert torch.equal(listed[tokens], plain[tokens]) and torch.equal(lse_a[tokens], lse_b[tokens])
    want, want_lse = cache.oracle(q, rows, starts, firsts, 6, counts=counts)
    assert_attention_close(tma, lse_a, want, want_lse, tokens, rel=2.0 ** -7 if kind == "fp8:page" else 0.0)
    assert pk.status() == 0


def test_a_count_past_the_columns_reads_as_the_columns(pk):
    from helpers import Cache, queries
    cache = Cache("bf16", 2, 128, 128, 16, [300, 300], spare=8)
    q = queries(8, 8, 128, 11)
    want = cache.attend(q, [0, 1], [0, 4], [290, 280], 4)
    got = cache.attend(q, [0, 1], [0, 4], [290, 280], 4, counts=[9, 4])
    assert torch.equal(got, want)


def test_packed_partial_rows_follow_the_offsets(pk):
    from helpers import Cache, queries
    cache = Cache("fp8:row", 4, 128, 128, 16, [700, 300, 2100], spare=8)
    q = queries(24, 24, 128, 5)
    together = cache.attend(q, [0, 1, 2], [0, 8, 16], [690, 290, 2090], 8, chunk=128)
    offsets = torch.tensor([0, 3, 4], dtype=torch.int32, device="cuda")
    splits = pk.parts_for(cache.tables.shape[1] * 16, 128)
    space = torch.empty(pk.workspace_floats(8, 24, splits, 128), device="cuda")
    packed = cache.attend(q, [0, 1, 2], [0, 8, 16], [690, 290, 2090], 8, counts=[3, 1, 4], offsets=offsets, tokens=8,
                          workspace=space, chunk=128)
    for start, count in zip([0, 8, 16], [3, 1, 4]):
        assert torch.equal(packed[start:start + count], together[start:start + count])
    with pytest.raises(ValueError, match="workspace"):
        cache.attend(q, [0, 1, 2], [0, 8, 16], [690, 290, 2090], 8, workspace=space[:100], chunk=128)


def test_a_nan_query_poisons_only_its_own_token(pk):
    from helpers import Cache, queries
    cache = Cache("bf16", 2, 128, 128, 16, [200], spare=8)
    q = queries(4, 8, 128, 2)
    clean = cache.attend(q, [0], [0], [196], 4)
    q2 = q.clone()
    q2[1, 3, 5] = float("nan")
    got = cache.attend(q2, [0], [0], [196], 4)
    assert torch.isnan(got[1, 3]).all()
    keep = torch.ones(4, 8, dtype=torch.bool)
    keep[1, 3] = False
    assert torch.equal(got.cpu()[keep], clean.cpu()[keep])


def test_config_1_matches_the_references_outputs(pk, golden):
    """BASELINE config 1 (the reference's CPU-runnable decode step) on bf16 pages, against the reference's own FP32
    outputs: slots bit for bit, attention within the north-star bound."""
    from test_oracle import _c1_inputs
    from helpers import assert_attention_close
    data = golden("c1_full.npz")
    hq, hkv, d, page, pool_pages, _ = (int(x) for x in data["geometry"])
    lens, keys, values, new_k, new_v, q = _c1_inputs(data)
    tables = torch.from_numpy(np.where(data["tables"] < 0, pool_pages, data["tables"]).astype(np.int32)).cuda()
    k = torch.zeros(pool_pages + 1, page, hkv, d, dtype=torch.bfloat16, device="cuda")
    v = torch.zeros_like(k)
    rows = torch.arange(len(lens), device="cuda")
    for s, n in enumerate(lens):
        at = pk.slots_at(tables, torch.full((n,), s, device="cuda"), torch.arange(n, device="cuda"), page, pool_pages)
        pk.write(torch.from_numpy(keys[s]).cuda(), torch.from_numpy(values[s]).cuda(), at, k, v, "bf16")
    slots = pk.slots_at(tables, rows, torch.tensor(lens, device="cuda"), page, pool_pages)
    assert slots.cpu().tolist() == data["slots"].tolist()
    pk.write(torch.from_numpy(new_k).cuda(), torch.from_numpy(new_v).cuda(), slots, k, v, "bf16")
    qd = torch.from_numpy(q).cuda().bfloat16()
    lse = torch.empty(len(lens), hq, device="cuda")
    i32 = dict(dtype=torch.int32, device="cuda")
    out = pk.attend(qd, k, v, "bf16", tables, torch.arange(len(lens), **i32), torch.arange(len(lens), **i32),
                    torch.tensor(lens, device="cuda"), 1, page, lse=lse)
    assert_attention_close(out, lse, data["out"], data["lse"], list(range(len(lens))), lse_abs=2e-2)


# -- prompt chunks ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["bf16", "fp16", "fp8", "fp8:row", "int8", "fp8:page"])
@pytest.mark.parametrize("hq,hkv,d", [(8, 2, 128), (12, 2, 64), (32, 8, 128)])
@pytest.mark.parametrize("position,tokens", [(0, 70), (333, 150), (1000, 1), (64, 64)])
def test_prompt_chunks_match_the_oracle(pk, kind, hq, hkv, d, position, tokens):
    from helpers import Cache, assert_attention_close, queries
    cache = Cache(kind, hkv, d, d, 16, [position + tokens, 40], spare=20)
    dtype = torch.float16 if kind == "fp16" else torch.bfloat16
    q = queries(tokens, hq, d, 13, dtype)
    lse = torch.empty(tokens, hq, device="cuda")
    out = pk.prefill(q, cache.k, cache.v, kind, cache.tables[0].contiguous(), position, 16, key_scales=cache.ks,
                     value_scales=cache.vs, multipliers=cache.multipliers, lse=lse)
    want, want_lse = cache.oracle(q, [0], [0], [position], tokens)
    assert_attention_close(out, lse, want, want_lse, list(range(tokens)))
    # the position read on the device, no log-sum-exps: the same bits
    again = pk.prefill(q, cache.k, cache.v, kind, cache.tables[0].contiguous(), torch.tensor([position], device="cuda"), 16,
                       key_scales=cache.ks, value_scales=cache.vs, multipliers=cache.multipliers)
    assert torch.equal(again, out)


@pytest.mark.parametrize("kind", ["bf16", "fp16"])
@pytest.mark.parametrize("position,tokens", [(0, 70), (333, 150), (1000, 1), (2000, 300)])
def test_prompt_chunks_of_256_wide_heads_match_the_oracle(pk, kind, position, tokens):
    """24q/4kv x 256 (the long-context model's geometry) over 16-bit pages: the m16n8k16 prefill kernel."""
    from helpers import Cache, assert_attention_close, queries
    cache = Cache(kind, 4, 256, 256, 64, [position + tokens, 40], spare=20)
    assert pk.prefill_serves(256, 256, torch.bfloat16, kind, 64) and not pk.prefill_serves(256, 256, torch.bfloat16, "fp8", 64)
    q = queries(tokens, 24, 256, 13, torch.float16 if kind == "fp16" else torch.bfloat16)
    lse = torch.empty(tokens, 24, device="cuda")
    out = pk.prefill(q, cache.k, cache.v, kind, cache.tables[0].contiguous(), position, 64, lse=lse)
    want, want_lse = cache.oracle(q, [0], [0], [position], tokens)
    assert_attention_close(out, lse, want, want_lse, list(range(tokens)))


@pytest.mark.parametrize("kind", ["bf16", "fp16"])
@pytest.mark.parametrize("hq,hkv", [(8, 2), (32, 8), (5, 1), (16, 16)])
@pytest.mark.parametrize("position,tokens", [(0, 70), (333, 150), (1000, 1), (64, 64), (0, 32), (4090, 300)])
def test_prompt_chunks_on_tcgen05_tiles_match_the_oracle(pk, kind, hq, hkv, position, tokens):
    """The tcgen05 / TMEM engine: 128-row blocks (partly filled last blocks and warps, one tile and many)."""
    from helpers import Cache, assert_attention_close, queries
    cache = Cache(kind, hkv, 128, 128, 16, [position + tokens, 40], spare=20)
    dtype = torch.float16 if kind == "fp16" else torch.bfloat16
    q = queries(tokens, hq, 128, 13, dtype)
    lse = torch.empty(tokens, hq, device="cuda")
    table = cache.tables[0].contiguous()
    out = pk.prefill(q, cache.k, cache.v, kind, table, position, 16, lse=lse, engine="tcgen05")
    assert pk.status() == 0
    want, want_lse = cache.oracle(q, [0], [0], [position], tokens)
    assert_attention_close(out, lse, want, want_lse, list(range(tokens)))
    again = pk.prefill(q, cache.k, cache.v, kind, table, torch.tensor([position], device="cuda"), 16, engine="tcgen05")
    assert torch.equal(again, out)
    # against the m16n8k16 engine: the same tiles of 64 positions and the same lazy maximum, so nearly the same bits
    other = pk.prefill(q, cache.k, cache.v, kind, table, position, 16, engine="mma.sync")
    torch.testing.assert_close(out.float(), other.float(), atol=1e-2, rtol=2e-2)


@pytest.mark.parametrize("kind,engine", [("bf16", "tcgen05:single"), ("bf16", "tcgen05:pair"), ("bf16", "mma.sync"),
                                         ("fp8:row", None), ("fp8:page", None)])
@pytest.mark.parametrize("counts", [[150, 150, 150], [150, 1, 300, 37], [150]])
def test_several_sequences_chunks_in_one_launch_give_each_sequences_own_launchs_bits(pk, kind, engine, counts):
    """One prefill launch over several sequences (a table a sequence, a position a sequence, equal counts or ragged
    ones through `starts`): every sequence's rows carry the bits of a launch of its own, and match the oracle."""
    from helpers import Cache, assert_attention_close, queries
    firsts = [333, 0, 1000, 64][:len(counts)]
    cache = Cache(kind, 2, 128, 128, 16, [a + n for a, n in zip(firsts, counts)], spare=20)
    T = sum(counts)
    q = queries(T, 8, 128, 21)
    scales = dict(key_scales=cache.ks, value_scales=cache.vs)
    lse = torch.full((T, 8), 7.0, device="cuda")
    starts = [0]
    for n in counts:
        starts.append(starts[-1] + n)
    ragged = len(set(counts)) > 1
    out = pk.prefill(q, cache.k, cache.v, kind, cache.tables.contiguous(), firsts, 16, lse=lse, engine=engine,
                     starts=starts if ragged else None, **scales)
    assert pk.status() == 0
    for s, n in enumerate(counts):
        span = slice(starts[s], starts[s + 1])
        own_lse = torch.empty(n, 8, device="cuda")
        own = pk.prefill(q[span], cache.k, cache.v, kind, cache.tables[s].contiguous(), firsts[s], 16, lse=own_lse,
                         engine=engine, **scales)
        assert torch.equal(out[span], own) and torch.equal(lse[span], own_lse), s
    want, want_lse = cache.oracle(q, list(range(len(counts))), starts[:-1], firsts, max(counts), counts=counts)
    assert_attention_close(out, lse, want, want_lse, list(range(T)))
    with pytest.raises(ValueError):
        pk.prefill(q, cache.k, cache.v, kind, cache.tables.contiguous(), firsts[:-1], 16, **scales)
    with pytest.raises(ValueError):
        pk.prefill(q, cache.k, cache.v, kind, cache.tables.contiguous(), firsts, 16, starts=[0] * len(counts) + [T + 1], **scales)


@pytest.mark.parametrize("kind", ["bf16", "fp16"])
@pytest.mark.parametrize("hq,hkv", [(8, 2), (32, 8), (5, 1), (16, 16)])
@pytest.mark.parametrize("position,tokens", [(0, 70), (333, 150), (1000, 1), (64, 64), (0, 32), (4090, 300), (100, 129)])
def test_prompt_chunks_on_paired_tcgen05_blocks_match_the_oracle(pk, kind, hq, hkv, position, tokens):
    """Blocks of 256 query rows (two halves over one ring of key and value tiles): half-filled blocks, a second half
    without rows, one tile and many, more tiles than the ring holds."""
    from helpers import Cache, assert_attention_close, queries
    cache = Cache(kind, hkv, 128, 128, 16, [position + tokens, 40], spare=20)
    dtype = torch.float16 if kind == "fp16" else torch.bfloat16
    q = queries(tokens, hq, 128, 13, dtype)
    lse = torch.empty(tokens, hq, device="cuda")
    table = cache.tables[0].contiguous()
    out = pk.prefill(q, cache.k, cache.v, kind, table, position, 16, lse=lse, engine="tcgen05:pair")
    assert pk.status() == 0
    want, want_lse = cache.oracle(q, [0], [0], [position], tokens)
    assert_attention_close(out, lse, want, want_lse, list(range(tokens)))
    # a row's arithmetic is that of the blocks of 128 rows: the same tiles, the same lazy maximum
    other_lse = torch.empty_like(lse)
    other = pk.prefill(q, cache.k, cache.v, kind, table, position, 16, lse=other_lse, engine="tcgen05:single")
    torch.testing.assert_close(out.float(), other.float(), atol=1e-2, rtol=2e-2)
    torch.testing.assert_close(lse, other_lse, atol=1e-4, rtol=0)


def test_tcgen05_tiles_refuse_what_they_do_not_serve(pk):
    from helpers import Cache, queries
    cache = Cache("fp8:row", 2, 128, 128, 16, [100], spare=4)
    q = queries(20, 8, 128, 1)
    with pytest.raises(Exception):
        pk.prefill(q, cache.k, cache.v, "fp8:row", cache.tables[0].contiguous(), 80, 16, key_scales=cache.ks,
                   value_scales=cache.vs, engine="tcgen05")
    cache = Cache("bf16", 2, 64, 64, 16, [100], spare=4)
    with pytest.raises(Exception):
        pk.prefill(queries(20, 8, 64, 1), cache.k, cache.v, "bf16", cache.tables[0].contiguous(), 80, 16, engine="tcgen05")


def test_a_prompt_token_reads_the_same_alone_and_in_its_chunk(pk):
    from helpers import Cache, queries
    cache = Cache("bf16", 2, 128, 128, 16, [700], spare=8)
    q = queries(200, 8, 128, 3)
    table = cache.tables[0].contiguous()
    whole = pk.prefill(q, cache.k, cache.v, "bf16", table, 500, 16)
    part = pk.prefill(q[64:130], cache.k, cache.v, "bf16", table, 564, 16)
    torch.testing.assert_close(part.float(), whole[64:130].float(), atol=2e-2, rtol=2e-2)


# -- merges ---------------------------------------------------------------------------------------------------------------
def test_merge_of_shards_matches_the_references(pk, golden):
    data = golden("merge.npz")
    out, lse = pk.merge_shards(torch.from_numpy(data["outs"]).cuda(), torch.from_numpy(data["lses"]).cuda())
    np.testing.assert_allclose(out.cpu().numpy(), data["out"], atol=1e-6, rtol=1e-5)
    got = lse.cpu().numpy()
    assert np.array_equal(np.isneginf(got), np.isneginf(data["lse"]))
    keep = ~np.isneginf(got)
    np.testing.assert_allclose(got[keep], data["lse"][keep], atol=1e-6, rtol=1e-6)
    assert not out[4, 1].any()


def test_merged_shards_equal_attention_over_the_whole_sequence(pk):
    """The reference's own device test (inference/partitioned-attention/tests/test_device.py:44-68): a sequence cut in
    two shards, each attended with its log-sum-exp, merged."""
    from helpers import Cache, queries
    g = torch.Generator().manual_seed(1)
    q = queries(1, 4, 64, 1)
    whole = Cache("bf16", 2, 64, 64, 16, [300], seed=3)
    k, v = whole.stored()
    at = whole.slots(0, torch.arange(300)).cpu().numpy()
    keys, values = torch.from_numpy(k[at]).cuda().bfloat16(), torch.from_numpy(v[at]).cuda().bfloat16()
    shards = Cache("bf16", 2, 64, 64, 16, [120, 180], seed=4)
    shards.write(0, 0, keys[:120], values[:120])
    shards.write(1, 0, keys[120:], values[120:])
    lse = torch.empty(1, 4, device="cuda")
    out = whole.attend(q, [0], [0], [299], 1, lse=lse)
    parts = []
    for s, n in ((0, 120), (1, 180)):
        part_lse = torch.empty(1, 4, device="cuda")
        parts.append((shards.attend(q, [s], [0], [n - 1], 1, lse=part_lse), part_lse))
    merged, merged_lse = pk.merge_shards([o for o, _ in parts], [x for _, x in parts])
    torch.testing.assert_close(merged, out.float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(merged_lse, lse, atol=2e-3, rtol=1e-4)


# -- the exchange of the shards' partials over peer memory ----------------------------------------------------------------
def test_the_peer_exchange_lands_every_ranks_message_and_a_missing_rank_runs_the_wait_out(pk):
    """Two ranks' exchange buffers on one GPU, the launches one after another on one stream: messages land in both
    buffers, the slots alternate from step to step, and a rank whose partner never pushes gets the status word after its
    bounded wait and no data (the way the path detects a lost rank without any GPU fault)."""
    from crit_b200.dist import PeerExchange
    dev, world, floats = torch.device("cuda"), 2, 1003
    size = PeerExchange.exchange_bytes(world, floats)
    buffers = [torch.zeros(size // 4, dtype=torch.float32, device=dev) for _ in range(world)]
    peers = torch.tensor([b.data_ptr() for b in buffers], dtype=torch.int64, device=dev)
    mine = [torch.zeros(floats, device=dev) for _ in range(world)]
    gathered = [torch.full((world, floats), -1.0, device=dev) for _ in range(world)]
    status = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(world)]
    ranks = [PeerExchange(peers, r, world, mine[r], gathered[r], wait_ms=30, status=status[r]) for r in range(world)]
    g = torch.Generator().manual_seed(3)
    # step 1: rank 1 never pushes; rank 0's wait runs out, says so and publishes nothing
    mine[0].copy_(torch.randn(floats, generator=g))
    ranks[0].push()
    ranks[0].wait()
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0x800 and bool((gathered[0] == -1.0).all())
    status[0].zero_()
    # ... then rank 1 joins the step: both ranks see both messages
    mine[1].copy_(torch.randn(floats, generator=g))
    ranks[1].push()
    for r in range(world):
        ranks[r].wait()
    torch.cuda.synchronize()
    for r in range(world):
        assert torch.equal(gathered[r][0], mine[0]) and torch.equal(gathered[r][1], mine[1]) and int(status[r].item()) == 0
    # steps 2 and 3: new messages through the other slot and back
    for _ in range(2):
        for r in range(world):
            mine[r].copy_(torch.randn(floats, generator=g))
            ranks[r].push()
        for r in range(world):
            ranks[r].wait()
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.equal(gathered[r][0], mine[0]) and torch.equal(gathered[r][1], mine[1]) and int(status[r].item()) == 0


# -- draft trees: a column sees the context, itself and its ancestors ----------------------------------------------------
def _random_tree(rng, count):
    """Parents of `count` columns in topological order: column 0 a root, every later column under an earlier one or a
    root of its own."""
    return [-1] + [int(rng.integers(-1, c)) for c in range(1, count)]


@pytest.mark.parametrize("kind", ["bf16", "fp8", "fp8:row", "int8", "fp8:page"])
@pytest.mark.parametrize("hq,hkv,d", [(8, 2, 128), (24, 4, 256), (64, 8, 128), (4, 4, 64)])
@pytest.mark.parametrize("page,chunk", [(16, 64), (48, 1024)])
def test_draft_tree_windows_match_the_oracle(pk, kind, hq, hkv, d, page, chunk):
    import oracle
    from helpers import Cache, assert_attention_close, queries
    cache = Cache(kind, hkv, d, d, page, [130, 64, 9, 517, 1300])
    cols = min(8, 64 // (hq // hkv))
    firsts = [130 - cols, 64 - 3, 0, 400, 1300 - cols]
    counts = [cols, 3, min(cols, 9), min(cols, 5), cols]
    rows, starts = [0, 1, 2, 3, 4], [0, 8, 16, 24, 32]
    rng = np.random.default_rng(11)
    parents = np.full(40, -1, np.int32)
    for s, n in zip(starts, counts):
        parents[s:s + n] = _random_tree(rng, n)
    q = queries(40, hq, d, 3)
    lse = torch.full((40, hq), 7.0, device="cuda")
    out = cache.attend(q, rows, starts, firsts, cols, counts=counts, lse=lse, chunk=chunk,
                       parents=torch.tensor(parents, device="cuda"))
    assert pk.status() == 0
    k, v = cache.stored()
    want, want_lse = oracle.attend_tree(q.float().cpu().numpy(), k, v, cache.tables.cpu().numpy(), rows, starts, firsts, cols,
                                        page, parents, counts=counts)
    tokens = [s + c for s, n in zip(starts, counts) for c in range(n)]
    assert_attention_close(out, lse, want, want_lse, tokens)
    # a chain is the plain causal window, bit for bit; int64 parents are taken too
    chain = np.full(40, -1, np.int64)
    for s, n in zip(starts, counts):
        chain[s:s + n] = np.arange(n) - 1
    a = cache.attend(q, rows, starts, firsts, cols, counts=counts, chunk=chunk, parents=torch.tensor(chain, device="cuda"))
    b = cache.attend(q, rows, starts, firsts, cols, counts=counts, chunk=chunk, engine="mma.sync")
    assert torch.equal(a[tokens], b[tokens])


def test_draft_trees_match_the_references_torch_path(pk, golden):
    """The reference's own torch windows over a draft tree (tests/golden/make_golden.py: tree_windows), bf16 pages."""
    from helpers import assert_attention_close
    f = golden("tree_bf16.npz")
    hq, hkv, d, page = (int(x) for x in f["geometry"])
    dev = "cuda"
    k = torch.tensor(f["k_pages"]).bfloat16().to(dev).reshape(-1, hkv, d)
    v = torch.tensor(f["v_pages"]).bfloat16().to(dev).reshape(-1, hkv, d)
    q = torch.tensor(f["q"]).bfloat16().to(dev)
    lse = torch.empty(12, hq, device=dev)
    out = pk.attend(q, k.view(-1, page, hkv, d), v.view(-1, page, hkv, d), "bf16", torch.tensor(f["tables"], device=dev),
                    torch.tensor([0, 1], dtype=torch.int32, device=dev), torch.tensor(f["starts"], dtype=torch.int32, device=dev),
                    torch.tensor(f["firsts"], dtype=torch.int64, device=dev), 7, page,
                    counts=torch.tensor(f["counts"], dtype=torch.int32, device=dev), lse=lse,
                    parents=torch.tensor(f["parents"], device=dev))
    assert_attention_close(out, lse, f["out"], f["lse"], list(range(12)))


def test_draft_trees_are_refused_by_the_tcgen05_kernels(pk):
    from helpers import Cache, queries
    cache = Cache("fp8:page", 8, 128, 128, 16, [100])
    parents = torch.tensor([-1, 0], dtype=torch.int32, device="cuda")
    for engine in ("tcgen05", "tcgen05p"):
        with pytest.raises(NotImplementedError):
            cache.attend(queries(2, 16, 128, 1), [0], [0], [98], 2, parents=parents, engine=engine)


# -- sliding windows and sinks --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["bf16", "fp8:row", "fp8:page"])
@pytest.mark.parametrize("hq,hkv,d", [(8, 2, 128), (24, 4, 256), (64, 8, 128)])
@pytest.mark.parametrize("sliding,with_sinks,tree", [(100, False, False), (0, True, False), (37, True, False), (300, True, True)])
@pytest.mark.parametrize("chunk", [64, 1024])
def test_sliding_windows_and_sinks_match_the_oracle(pk, kind, hq, hkv, d, sliding, with_sinks, tree, chunk):
    import oracle
    from helpers import Cache, assert_attention_close, queries
    cache = Cache(kind, hkv, d, d, 16, [130, 64, 9, 517, 1300])
    cols = 4
    firsts = [126, 61, 0, 400, 1296]
    counts = [4, 3, 4, 2, 4]
    rows, starts = [0, 1, 2, 3, 4], [0, 4, 8, 12, 16]
    rng = np.random.default_rng(5)
    parents = None
    if tree:
        parents = np.full(20, -1, np.int32)
        for s, n in zip(starts, counts):
            parents[s:s + n] = _random_tree(rng, n)
    sinks = (rng.standard_normal(hq) * 2).astype(np.float32) if with_sinks else None
    q = queries(20, hq, d, 3)
    lse = torch.full((20, hq), 7.0, device="cuda")
    out = cache.attend(q, rows, starts, firsts, cols, counts=counts, lse=lse, chunk=chunk, sliding=sliding,
                       sinks=torch.tensor(sinks, device="cuda") if with_sinks else None,
                       parents=torch.tensor(parents, device="cuda") if tree else None)
    assert pk.status() == 0
    k, v = cache.stored()
    want, want_lse = oracle.attend_tree(q.float().cpu().numpy(), k, v, cache.tables.cpu().numpy(), rows, starts, firsts, cols,
                                        16, parents, counts=counts, sinks=sinks, sliding=sliding)
    tokens = [s + c for s, n in zip(starts, counts) for c in range(n)]
    assert_attention_close(out, lse, want, want_lse, tokens)


@pytest.mark.parametrize("case", ["sliding", "sinks", "all"])
def test_sliding_windows_and_sinks_match_the_references_torch_path(pk, golden, case):
    from helpers import assert_attention_close
    f = golden("tree_bf16.npz")
    hq, hkv, d, page = (int(x) for x in f["geometry"])
    dev = "cuda"
    k = torch.tensor(f["k_pages"]).bfloat16().to(dev).reshape(-1, page, hkv, d)
    v = torch.tensor(f["v_pages"]).bfloat16().to(dev).reshape(-1, page, hkv, d)
    q = torch.tensor(f["q"]).bfloat16().to(dev)
    lse = torch.empty(12, hq, device=dev)
    out = pk.attend(q, k, v, "bf16", torch.tensor(f["tables"], device=dev), torch.tensor([0, 1], dtype=torch.int32, device=dev),
                    torch.tensor(f["starts"], dtype=torch.int32, device=dev), torch.tensor(f["firsts"], dtype=torch.int64, device=dev),
                    7, page, counts=torch.tensor(f["counts"], dtype=torch.int32, device=dev), lse=lse,
                    parents=torch.tensor(f["parents"], device=dev) if case == "all" else None,
                    sinks=torch.tensor(f["sinks"], device=dev) if case != "sliding" else None,
                    sliding=int(f["sliding"]) if case != "sinks" else 0)
    assert_attention_close(out, lse, f["out_" + case], f["lse_" + case], list(range(12)))


# -- block lists ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["bf16", "fp8:row", "fp8:page"])
@pytest.mark.parametrize("hq,hkv,d", [(8, 2, 128), (24, 4, 256), (64, 8, 128)])
@pytest.mark.parametrize("chunk", [64, 1024])
@pytest.mark.parametrize("block_size,engine", [(32, None), (24, None), (64, "tcgen05p"), (128, "tcgen05")])
def test_block_lists_match_the_oracle(pk, kind, hq, hkv, d, chunk, block_size, engine):
    """Blocks of a multiple of the page: the sparse reader (a page table of the listed blocks a token, on any kernel);
    blocks of 24 positions over pages of 16: the lists as a mask over the m16n8k16 kernel's tiles."""
    import oracle
    if engine == "tcgen05p" and not (hkv == 8 and kind != "bf16"):
        pytest.skip("the whole-page-rows kernel reads E4M3 pages of 8 kv heads")
    if engine == "tcgen05" and (kind == "bf16" or d != 128 or chunk % 128):
        pytest.skip("the tcgen05 kernel reads E4M3 pages of 128-wide heads in splits of whole 128-position tiles")
    from helpers import Cache, assert_attention_close, queries
    cache = Cache(kind, hkv, d, d, 16, [130, 64, 9, 517, 1300])
    cols, firsts, counts = 4, [126, 61, 0, 400, 1296], [4, 3, 4, 2, 4]
    rows, starts = [0, 1, 2, 3, 4], [0, 4, 8, 12, 16]
    rng = np.random.default_rng(8)
    blocks = np.full((20, 5), -1, np.int32)
    for s, n, first in zip(starts, counts, firsts):
        for c in range(n):
            own = (first + c) // block_size
            picks = rng.permutation(own + 1)[:rng.integers(1, 5)]
            blocks[s + c, :len(picks)] = picks
            blocks[s + c, 4] = own if (s + c) % 4 else -1           # most tokens see their own block; a few may see nothing
    q = queries(20, hq, d, 3)
    lse = torch.full((20, hq), 7.0, device="cuda")
    blocks[3, 1] = blocks[3, 0]                                      # an id listed twice counts once
    out = cache.attend(q, rows, starts, firsts, cols, counts=counts, lse=lse, chunk=chunk, blocks=torch.tensor(blocks, device="cuda"),
                       block_size=block_size, engine=engine)
    assert pk.status() == 0
    k, v = cache.stored()
    want, want_lse = oracle.attend_tree(q.float().cpu().numpy(), k, v, cache.tables.cpu().numpy(), rows, starts, firsts, cols,
                                        16, None, counts=counts, blocks=blocks, block_size=block_size)
    tokens = [s + c for s, n in zip(starts, counts) for c in range(n)]
    assert_attention_close(out, lse, want, want_lse, tokens)


def test_block_lists_match_the_references_torch_path(pk, golden):
    from helpers import assert_attention_close
    f = golden("tree_bf16.npz")
    hq, hkv, d, page = (int(x) for x in f["geometry"])
    dev = "cuda"
    k = torch.tensor(f["k_pages"]).bfloat16().to(dev).reshape(-1, page, hkv, d)
    v = torch.tensor(f["v_pages"]).bfloat16().to(dev).reshape(-1, page, hkv, d)
    q = torch.tensor(f["q"]).bfloat16().to(dev)
    lse = torch.empty(12, hq, device=dev)
    out = pk.attend(q, k, v, "bf16", torch.tensor(f["tables"], device=dev), torch.tensor([0, 1], dtype=torch.int32, device=dev),
                    torch.tensor(f["starts"], dtype=torch.int32, device=dev), torch.tensor(f["firsts"], dtype=torch.int64, device=dev),
                    7, page, counts=torch.tensor(f["counts"], dtype=torch.int32, device=dev), lse=lse,
                    blocks=torch.tensor(f["blocks"], device=dev), block_size=16)
    assert_attention_close(out, lse, f["out_blocks"], f["lse_blocks"], list(range(12)))
