"""What stands in for a memory checker on this path: every kernel family run over buffers that sit between guard
regions (0xFF bytes, verified afterwards), over pages whose unused rows are poisoned with NaN codes, and with plans,
slots and page ids that do not fit what the launch was given: the kernels skip the access, say so in the status word and
never write outside their buffers.  Also the fused peer exchange with the ranks emulated on one GPU: messages land, a
missing rank runs the bounded wait out, a message of another step is refused.
Reference surrogates: core/python/crit_plugins/memory.py:446-448 (POISON fill),
kernels/techniques/attention/paged-kv-attention/tests/test_cuda.py:177-200."""
import ctypes

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pk():
    import crit_b200
    return crit_b200


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _lib():
    from crit_b200 import _lib as binding
    return binding, binding.load()


# -- guard regions ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["bf16", "fp8", "fp8:row", "int8", "fp8:page"])
def test_appends_and_gathers_stay_inside_their_buffers(pk, kind):
    from helpers import Guarded, STORE
    hkv, d, page, pages, n = 3, 128, 16, 7, 53
    store = STORE[kind]
    size = torch.empty(0, dtype=store).element_size()
    k, v = Guarded(pages * page * hkv * d * size), Guarded(pages * page * hkv * d * size)
    shape = (pages, hkv) if kind == "fp8:page" else (pages, page, hkv)
    ks = vs = None
    held = [k, v]
    if kind in ("fp8:row", "int8", "fp8:page"):
        ks, vs = Guarded(int(np.prod(shape)) * 4), Guarded(int(np.prod(shape)) * 4)
        held += [ks, vs]
    g = torch.Generator().manual_seed(2)
    keys, values = torch.randn(n, hkv, d, generator=g).bfloat16().cuda(), torch.randn(n, hkv, d, generator=g).bfloat16().cuda()
    slots = torch.arange(n, device="cuda") + 2 * page
    kp, vp = k.view(store, pages, page, hkv, d), v.view(store, pages, page, hkv, d)
    ksc = ks.view(torch.float32, *shape) if ks else None
    vsc = vs.view(torch.float32, *shape) if vs else None
    pk.write(keys, values, slots, kp, vp, kind, ksc, vsc, multipliers=(0.05, 0.05))
    out = Guarded(n * hkv * d * 4)
    table = torch.arange(2, pages, dtype=torch.int32, device="cuda")
    got = pk.gather(kp, kind, page, table=table, count=n, scales=ksc, multiplier=0.05, dtype=torch.float32)
    torch.cuda.synchronize()
    assert all(b.intact() for b in held + [out]) and bool(torch.isfinite(got).all()) and pk.status() == 0
    if kind == "bf16":
        assert torch.equal(got, keys.float())


@pytest.mark.parametrize("kind,engine", [("bf16", None), ("fp8:page", "mma.sync"), ("fp8:page", "tcgen05"), ("fp8:row", "tcgen05")])
def test_attention_stays_inside_its_buffers_and_ignores_poison_past_the_rows(pk, kind, engine):
    """Outputs, log-sum-exps and the partials' workspace between guard regions; the pages' unused rows hold NaN codes
    and NaN scales.  The attention matches the oracle and no guard byte changes."""
    from helpers import Cache, Guarded, assert_attention_close, queries
    cache = Cache(kind, 2, 128, 128, 16, [700, 37, 1300, 1], spare=3, poison=True)
    cols, hq = 3, 8
    rows, starts, firsts, counts = [0, 1, 2, 3], [0, 3, 6, 9], [697, 34, 1297, 0], [3, 3, 3, 1]
    q = queries(12, hq, 128, 4)
    out, lse = Guarded(12 * hq * 128 * 2), Guarded(12 * hq * 4)
    chunk = 256
    splits = pk.parts_for(cache.tables.shape[1] * 16, chunk)
    space = Guarded(pk.workspace_floats(12, hq, splits, 128) * 4)
    got = cache.attend(q, rows, starts, firsts, cols, counts=counts, out=out.view(torch.bfloat16, 12, hq, 128),
                       lse=lse.view(torch.float32, 12, hq), workspace=space.view(torch.float32, -1), chunk=chunk, engine=engine)
    torch.cuda.synchronize()
    assert out.intact() and lse.intact() and space.intact() and pk.status() == 0
    # the oracle reads the rows' own positions only: the poison elsewhere must not reach the outputs
    k, v = cache.stored()
    k, v = np.nan_to_num(k, nan=0.0), np.nan_to_num(v, nan=0.0)
    want, want_lse = oracle.attend(q.float().cpu().numpy(), k, v, cache.tables.cpu().numpy(), rows, starts, firsts, cols, 16,
                                   counts=counts)
    tokens = [s + c for s, n in zip(starts, counts) for c in range(n)]
    assert_attention_close(got, lse.view(torch.float32, 12, hq), want, want_lse, tokens)


def test_prompt_chunks_and_the_merge_of_shards_stay_inside_their_buffers(pk):
    from helpers import Cache, Guarded, queries
    for engine in (None, "mma.sync"):
        cache = Cache("bf16", 2, 128, 128, 16, [300], spare=3, poison=True)
        q = queries(100, 8, 128, 4)
        out, lse = Guarded(100 * 8 * 128 * 2), Guarded(100 * 8 * 4)
        pk.prefill(q, cache.k, cache.v, "bf16", cache.tables[0], 200, 16, out=out.view(torch.bfloat16, 100, 8, 128),
                   lse=lse.view(torch.float32, 100, 8), engine=engine)
        torch.cuda.synchronize()
        assert out.intact() and lse.intact() and bool(torch.isfinite(out.view(torch.bfloat16, 100, 8, 128).float()).all())
    outs, lses = torch.randn(3, 5, 4, 64, device="cuda"), torch.randn(3, 5, 4, device="cuda")
    binding, lib = _lib()
    merged, merged_lse = Guarded(5 * 4 * 64 * 4), Guarded(5 * 4 * 4)
    m = binding.MergeShardsParams()
    m.outs, m.lses, m.out, m.lse = outs.data_ptr(), lses.data_ptr(), merged.bytes.data_ptr(), merged_lse.bytes.data_ptr()
    m.n, m.parts, m.dim, m.in_dtype, m.out_dtype = 20, 3, 64, binding.DTYPE_FP32, binding.DTYPE_FP32
    assert lib.crit_b200_merge_shards(ctypes.byref(m), _stream()) == 0
    torch.cuda.synchronize()
    assert merged.intact() and merged_lse.intact() and pk.status() == 0
    want, want_lse = oracle.merge(outs.cpu().numpy(), lses.cpu().numpy())
    assert np.abs(merged.view(torch.float32, 5, 4, 64).cpu().numpy() - want).max() < 1e-5


# -- plans, slots and page ids that do not fit --------------------------------------------------------------------------
@pytest.mark.parametrize("flags", [0, 4, 8])
def test_a_plan_too_small_for_a_row_is_reported_and_nothing_is_written_outside(pk, flags):
    """max_splits and partial_rows below what the rows need (a caller's mistake): the units that do not fit are dropped,
    the status word says 2, the workspace's guards hold.  On the 3-D grid, the persistent work list and the tcgen05
    kernel."""
    from helpers import Cache, Guarded, attend_params, queries
    binding, lib = _lib()
    cache = Cache("fp8:page", 2, 128, 128, 16, [2000, 900], spare=8)
    q = queries(2, 8, 128, 3)
    out, lse = torch.zeros(2, 8, 128, dtype=torch.bfloat16, device="cuda"), torch.zeros(2, 8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    chunk, splits_given = 256, 3                        # the rows take 8 and 4 splits
    space = Guarded(2 * 8 * splits_given * 130 * 4)
    p, held = attend_params(cache, q, out, lse, [0, 1], [0, 1], [1999, 899], 1, chunk, workspace=space.view(torch.float32, -1),
                            flags=flags, status=status)
    p.max_splits = splits_given
    assert lib.crit_b200_attend(ctypes.byref(p), _stream()) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 2 and space.intact()
    # partial rows: offsets that point past the rows the workspace holds
    status.zero_()
    space = Guarded(1 * 8 * 8 * 130 * 4)
    p, held = attend_params(cache, q, out, lse, [0, 1], [0, 1], [1999, 899], 1, chunk, workspace=space.view(torch.float32, -1),
                            flags=flags, status=status, offsets=[0, 1], partial_rows=1)
    assert lib.crit_b200_attend(ctypes.byref(p), _stream()) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 2 and space.intact()
    # without offsets the host refuses the same mistake before any launch
    p, held = attend_params(cache, q, out, lse, [0, 1], [0, 1], [1999, 899], 1, chunk, workspace=space.view(torch.float32, -1),
                            flags=flags, partial_rows=1)
    assert lib.crit_b200_attend(ctypes.byref(p), _stream()) == -1


def test_slots_and_page_ids_outside_the_pages_are_skipped_and_reported(pk):
    from helpers import Cache, Guarded, queries
    hkv, d, page, pages = 2, 128, 16, 4
    k, v = Guarded(pages * page * hkv * d * 2), Guarded(pages * page * hkv * d * 2)
    kp, vp = k.view(torch.bfloat16, pages, page, hkv, d), v.view(torch.bfloat16, pages, page, hkv, d)
    keys = torch.ones(3, hkv, d, dtype=torch.bfloat16, device="cuda")
    slots = torch.tensor([5, pages * page, pages * page + 1000], device="cuda")
    assert pk.status() == 0
    pk.write(keys, keys, slots, kp, vp, "bf16")
    torch.cuda.synchronize()
    assert k.intact() and v.intact() and pk.status() == 3
    assert float(kp.float().sum()) == hkv * d            # the one slot inside the pages was written
    pk._status_word(torch.device("cuda", torch.cuda.current_device())).zero_()
    got = pk.gather(kp, "bf16", page, slots=slots, dtype=torch.float32)
    assert pk.status() == 3 and float(got[1:].abs().sum()) == 0.0 and float(got[0].sum()) == hkv * d
    pk._status_word(torch.device("cuda", torch.cuda.current_device())).zero_()
    # a page id past the pages in a table: the launch reads a page inside the tensor instead and says so
    for kind, engine in (("bf16", None), ("fp8:page", "mma.sync"), ("fp8:page", "tcgen05")):
        cache = Cache(kind, 2, 128, 128, 16, [300], spare=3)
        cache.tables[0, 3] = cache.k.shape[0] + 50
        out = cache.attend(queries(1, 8, 128, 1), [0], [0], [299], 1, engine=engine, chunk=128)
        torch.cuda.synchronize()
        assert pk.status() == 3 and bool(torch.isfinite(out.float()).all()), (kind, engine)
        pk._status_word(torch.device("cuda", torch.cuda.current_device())).zero_()


# -- split states kept for the exchange -----------------------------------------------------------------------------------
@pytest.mark.parametrize("kind,engine", [("bf16", None), ("fp8:page", "mma.sync"), ("fp8:page", "tcgen05")])
def test_split_states_kept_in_the_workspace_fold_to_the_ordinary_bits(pk, kind, engine):
    """CRIT_B200_ATTEND_PARTIALS: rows of one split leave their state in the workspace too, and crit_b200_merge folds
    every row to the bits the ordinary launch pair writes."""
    from helpers import Cache, attend_params, queries
    binding, lib = _lib()
    cache = Cache(kind, 2, 128, 128, 16, [700, 37, 1300], spare=3)
    q = queries(6, 8, 128, 4)
    rows, starts, firsts = [0, 1, 2], [0, 2, 4], [698, 35, 1298]
    chunk = 256
    flags = {None: 0, "mma.sync": 16, "tcgen05": 8}[engine]
    splits = pk.parts_for(cache.tables.shape[1] * 16, chunk)
    space = torch.empty(pk.workspace_floats(6, 8, splits, 128), device="cuda")
    want, want_lse = torch.zeros(6, 8, 128, dtype=torch.bfloat16, device="cuda"), torch.zeros(6, 8, device="cuda")
    got, got_lse = torch.zeros_like(want), torch.zeros_like(want_lse)
    p, held = attend_params(cache, q, want, want_lse, rows, starts, firsts, 2, chunk, workspace=space, flags=flags)
    assert lib.crit_b200_attend(ctypes.byref(p), _stream()) == 0
    p, held2 = attend_params(cache, q, got, got_lse, rows, starts, firsts, 2, chunk, workspace=space, flags=flags | 32)
    assert lib.crit_b200_decode(ctypes.byref(p), _stream()) == 0
    torch.cuda.synchronize()
    assert float(got.float().abs().sum()) == 0.0         # the first launch wrote no output
    assert lib.crit_b200_merge(ctypes.byref(p), _stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, want) and torch.equal(got_lse, want_lse) and float(want.float().abs().sum()) > 0


# -- the fused exchange, ranks emulated on one GPU ------------------------------------------------------------------------
def test_the_fused_exchange_merges_two_ranks_and_refuses_missing_and_stale_messages(pk):
    """Two ranks on one GPU, each over its half of one context: fold + push (crit_b200_merge_push), wait + merge
    (crit_b200_wait_merge).  The merged attention equals the attention over the whole; a rank whose partner never pushed
    gets 0x800 after its bounded wait and its output untouched; so does a rank that finds a later step's floats where it
    waits for its own step's (every float carries its step)."""
    from helpers import Cache, EmulatedRanks, assert_attention_close, attend_params, queries
    binding, lib = _lib()
    whole = Cache("bf16", 2, 128, 128, 16, [1000], seed=7)
    k, v = whole.stored()
    at = whole.slots(0, torch.arange(1000)).cpu().numpy()
    keys, values = torch.from_numpy(k[at]).cuda().bfloat16(), torch.from_numpy(v[at]).cuda().bfloat16()
    halves = Cache("bf16", 2, 128, 128, 16, [480, 520], seed=8)
    halves.write(0, 0, keys[:480], values[:480])
    halves.write(1, 0, keys[480:], values[480:])
    q = queries(1, 8, 128, 5)
    lse = torch.empty(1, 8, device="cuda")
    want = whole.attend(q, [0], [0], [999], 1, lse=lse, chunk=128)
    ranks = EmulatedRanks(2, 1, 8, 128, wait_ms=30)
    chunk = 128
    splits = pk.parts_for(halves.tables.shape[1] * 16, chunk)
    spaces = [torch.empty(pk.workspace_floats(1, 8, splits, 128), device="cuda") for _ in range(2)]
    scratch = torch.zeros(1, 8, 128, dtype=torch.bfloat16, device="cuda")
    blocks = [attend_params(halves, q, scratch, None, [r], [0], [n - 1], 1, chunk, workspace=spaces[r], flags=32)
              for r, n in ((0, 480), (1, 520))]
    merged = [(torch.full((1, 8, 128), 7.0, dtype=torch.bfloat16, device="cuda"), torch.full((1, 8), 7.0, device="cuda"))
              for _ in range(2)]

    def decode_and_push(r):
        assert lib.crit_b200_decode(ctypes.byref(blocks[r][0]), _stream()) == 0
        ranks.push(r, blocks[r][0])
    # step 1: rank 1 stays away.  Rank 0's wait runs out: 0x800, its output untouched
    decode_and_push(0)
    ranks.wait_merge(0, *merged[0])
    torch.cuda.synchronize()
    assert int(ranks.status[0].item()) == 0x800 and bool((merged[0][0] == 7.0).all()) and bool((merged[0][1] == 7.0).all())
    ranks.status[0].zero_()
    # ... rank 1 joins the step: both ranks merge both partials to the attention over the whole context
    decode_and_push(1)
    for r in range(2):
        ranks.wait_merge(r, *merged[r])
    torch.cuda.synchronize()
    assert all(int(s.item()) == 0 for s in ranks.status)
    assert torch.equal(merged[0][0], merged[1][0]) and torch.equal(merged[0][1], merged[1][1])
    torch.testing.assert_close(merged[0][0].float(), want.float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(merged[0][1], lse, atol=2e-3, rtol=1e-4)
    # steps 2 and 3: the slots alternate
    for _ in range(2):
        for r in range(2):
            decode_and_push(r)
        for r in range(2):
            merged[r][0].fill_(7.0)
            ranks.wait_merge(r, *merged[r])
        torch.cuda.synchronize()
        assert all(int(s.item()) == 0 for s in ranks.status) and torch.equal(merged[0][0], merged[1][0])
        torch.testing.assert_close(merged[0][0].float(), want.float(), atol=2e-2, rtol=2e-2)
    # a message of another step: rank 1 pushes three times (its counter runs ahead and comes round to the same slot),
    # rank 0 once; in the slot of its own step rank 0 finds floats stamped step + 2: not its step's, so they never "arrive"
    for _ in range(3):
        decode_and_push(1)
    decode_and_push(0)
    merged[0][0].fill_(7.0)
    ranks.wait_merge(0, *merged[0])
    torch.cuda.synchronize()
    assert int(ranks.status[0].item()) == 0x800 and bool((merged[0][0] == 7.0).all())


@pytest.mark.parametrize("tokens,columns", [(1, 1), (3, 3), (40, 1)])
def test_the_one_launch_exchange_of_a_single_rank_equals_the_plain_attention(pk, tokens, columns):
    """crit_b200_exchange_merge with a world of one rank: the launch folds and stores into its own buffer, waits for its own
    flag (raised by its last block) and merges the one part: the output is the ordinary launch pair's within FP32 rounding.
    3 tokens x 8 heads run as one launch (24 blocks), 40 x 8 = 320 blocks pass the SM count and run as the two launches."""
    from helpers import Cache, EmulatedRanks, attend_params, queries
    binding, lib = _lib()
    rows_n = tokens // columns
    cache = Cache("bf16", 2, 128, 128, 16, [700 + 13 * r for r in range(rows_n)], spare=4, seed=3)
    q = queries(tokens, 8, 128, 2)
    rows, starts = list(range(rows_n)), [r * columns for r in range(rows_n)]
    firsts = [700 + 13 * r - columns for r in range(rows_n)]
    want_lse = torch.empty(tokens, 8, device="cuda")
    want = cache.attend(q, rows, starts, firsts, columns, lse=want_lse, chunk=128)
    ranks = EmulatedRanks(1, tokens, 8, 128, wait_ms=50)
    splits = pk.parts_for(cache.tables.shape[1] * 16, 128)
    space = torch.empty(pk.workspace_floats(tokens, 8, splits, 128), device="cuda")
    scratch = torch.zeros(tokens, 8, 128, dtype=torch.bfloat16, device="cuda")
    p, held = attend_params(cache, q, scratch, None, rows, starts, firsts, columns, 128, workspace=space, flags=32)
    for _ in range(3):                       # step after step: the slots alternate, the ticket comes back to zero
        got, got_lse = torch.full_like(want, 7.0), torch.full_like(want_lse, 7.0)
        assert lib.crit_b200_decode(ctypes.byref(p), _stream()) == 0
        ranks.exchange_merge(0, p, got, got_lse)
        torch.cuda.synchronize()
        assert int(ranks.status[0].item()) == 0
        torch.testing.assert_close(got.float(), want.float(), atol=1e-2, rtol=1e-2)
        torch.testing.assert_close(got_lse, want_lse, atol=1e-4, rtol=1e-5)
