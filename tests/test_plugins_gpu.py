"""The plugin boundary on the GPU: crit_b200's pool and attention driven as crit's model plugin drives the
reference's (reserve -> write -> forward -> keep), checked against the CPU oracle; the cases follow the reference's own
plugin tests (inference/attention-state/tests/test_pages.py, inference/partitioned-attention/tests/test_device.py)."""
import math

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def parts(page=16, window_engine="mma.sync", **kw):
    """The two plugin objects; window_engine "mma.sync" unless a test asks otherwise: the tests of row-exact bits hold
    that engine to them (the default, "auto", sends verify windows over E4M3 pages to the tcgen05 kernel)."""
    from crit_b200.attention import DeviceAttention, PartitionedAttention
    from crit_b200.kv_state import KVStateCache
    import crit_b200
    kv = KVStateCache(page=page, kernels=crit_b200, **kw)
    return kv, PartitionedAttention(kv, {"world": 2, "page_size": 256}, DeviceAttention(device="cuda", window_engine=window_engine))


def rows_of(n, hkv, d, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, hkv, d, generator=g).bfloat16().cuda()


def step(pool, rows, layer=0, seed=0):
    from crit_b200.batch import StepBatch
    batch = StepBatch.build(rows, "cuda")
    slots = pool.reserve(batch)
    keys = rows_of(batch.tokens, pool.kv_heads, pool.head_dim, seed)
    values = rows_of(batch.tokens, pool.kv_heads, pool.value_dim, seed + 1)
    pool.write(layer, slots, keys, values)
    return batch, keys, values


def stored(pool, layer=0):
    i = pool.layers[layer]
    found = []
    for pages, scales, mult in ((pool.k[i], pool.k_scales, pool.scale_values[i][0]),
                                (pool.v[i], pool.v_scales, pool.scale_values[i][1])):
        dim = pages.shape[-1]
        if pool.dtype in ("bf16", "fp16"):
            found.append(pages.float().cpu().numpy().reshape(-1, pool.kv_heads, dim))
            continue
        codes = pages.view(torch.uint8).cpu().numpy().reshape(-1, pool.kv_heads, dim)
        sc = scales[i].cpu().numpy() if scales is not None else None
        if sc is not None and pool.dtype != "fp8:page":
            sc = sc.reshape(-1, pool.kv_heads)
        found.append(oracle.dequantize(codes, pool.dtype, sc, mult, page=pool.page))
    return found


def oracle_rows(pool, batch, q, layer=0):
    k, v = stored(pool, layer)
    width = max(len(pool.table(s)) for s in batch.sequences)
    tables = np.full((batch.rows, width), pool.dump, np.int32)
    for r, s in enumerate(batch.sequences):
        tables[r, :len(pool.table(s))] = pool.table(s)
    counts = [batch.row(r)[2] for r in range(batch.rows)]
    return oracle.attend(q.float().cpu().numpy(), k, v, tables, list(range(batch.rows)), batch.starts[:-1],
                         [batch.row(r)[3] for r in range(batch.rows)], max(counts), pool.page, counts=counts)


@pytest.mark.parametrize("dtype", ["bf16", "fp8", "fp8:row", "int8", "fp8:page"])
def test_a_step_of_many_sequences_writes_each_where_it_reads_back(dtype):
    kv, _ = parts()
    pool = kv.pool([0, 3], 2, 64, 256, "cuda", dtype)
    if dtype == "fp8":
        pool.set_scales(3, 0.05, 0.07)
    for s in "abc":
        pool.open(s)
    batch, keys, values = step(pool, [("a", 0, 20), ("b", 0, 1), ("c", 0, 5)], layer=3)
    k, v = stored(pool, 3)
    for r in range(batch.rows):
        s, first, count, _ = batch.row(r)
        got_k, got_v = pool.gather(3, s, count)
        at = oracle.slots(np.array(pool.table(s), np.int32), np.arange(count), 16)
        assert torch.equal(got_k.cpu(), torch.from_numpy(k[at]).bfloat16())
        assert torch.equal(got_v.cpu(), torch.from_numpy(v[at]).bfloat16())
        if dtype == "bf16":
            assert torch.equal(got_k, keys[first:first + count])
    assert float(pool.gather(0, "a", 20)[0].float().abs().sum()) == 0.0      # another layer is apart
    assert pool.free_pages() == 16 - 2 - 1 - 1
    if dtype == "fp8:row":
        codes, scale = oracle.quantize_rows(keys.float().cpu().numpy(), "fp8:row")
        at = oracle.slots(np.array(pool.table("a"), np.int32), np.arange(20), 16)
        assert np.array_equal(pool.k[1].view(torch.uint8).cpu().numpy().reshape(-1, 2, 64)[at], codes[:20])
        assert np.array_equal(pool.k_scales[1].cpu().numpy().reshape(-1, 2)[at], scale[:20])


def test_keep_rolls_a_verify_window_back_and_a_fork_copies_on_write():
    kv, _ = parts()
    pool = kv.pool([0], 2, 64, 256, "cuda", "fp8:row")
    pool.open("a")
    _, keys, _ = step(pool, [("a", 0, 20)])
    pool.keep("a", 20)
    before = pool.gather(0, "a", 20)[0].clone()
    pool.fork("a", "b")
    assert pool.table("a") == pool.table("b")
    step(pool, [("b", 20, 3)], seed=9)           # into the page they share: b copies it first, scales too
    assert pool.table("a")[0] == pool.table("b")[0] and pool.table("a")[1] != pool.table("b")[1]
    assert torch.equal(pool.gather(0, "b", 20)[0], before) and torch.equal(pool.gather(0, "a", 20)[0], before)
    step(pool, [("a", 20, 4)], seed=5)           # a verify window of 4
    pool.keep("a", 21)
    assert (pool.length("a"), len(pool.table("a"))) == (21, 2)
    pool.keep("a", 16)
    assert len(pool.table("a")) == 1
    pool.close("a")
    pool.close("b")
    assert pool.free_pages() == 16


def test_the_device_block_table_follows_the_host_when_one_flush_holds_an_entry_twice():
    """An entry of the block table can be queued twice before one upload: a closed sequence's row taken by the next
    open(), a page rolled back by keep() and grown again, the shared and then the copied tail of a bound sequence's
    fork.  The device table must end with the last value of each (a scatter with one index twice has no order)."""
    kv, _ = parts(round_rows=4)
    pool = kv.pool([0], 2, 64, 16 * 32, "cuda", "bf16")

    def mirrors():
        pool._flush()
        torch.cuda.synchronize()
        for s, table in pool.tables.items():
            row = pool.block_tables[pool.row_of[s]].tolist()
            assert row[:len(table)] == table and set(row[len(table):]) <= {pool.dump}, s
    for turn in range(20):                      # many turns: a lost race shows up in some of them
        pool.open("a")
        step(pool, [("a", 0, 40)])
        pool.keep("a", 40)
        pool.close("a")
        pool.open("b")                          # takes a's row; its reserve flushes a's entries and its own together
        step(pool, [("b", 0, 20)])
        mirrors()
        pool.keep("b", 10)                      # page 1 back to the pool ...
        step(pool, [("b", 10, 10)])             # ... and grown again before any flush
        mirrors()
        pool.keep("b", 20)
        pool.bind(0, "b", 64)
        pool.fork("b", "c")                     # the tail page: shared, then copied, in one flush
        mirrors()
        assert pool.table("b")[1] != pool.table("c")[1]
        pool.unbind(0)
        pool.close("b")
        pool.close("c")
        assert pool.free_pages() == 32


@pytest.mark.parametrize("dtype", ["bf16", "fp8:page"])
def test_a_decode_step_and_a_verify_window_match_the_oracle(dtype):
    from crit_b200.batch import StepBatch
    from helpers import assert_attention_close
    kv, attention = parts()
    pool = kv.pool([0], 4, 128, 16 * 400, "cuda", dtype)
    lens = {"a": 700, "b": 64, "c": 1, "d": 2100}
    for s, n in lens.items():
        pool.open(s)
        step(pool, [(s, 0, n)], seed=len(s) + n)
        pool.keep(s, n)
    batch, _, _ = step(pool, [("a", 700, 1), ("b", 64, 6), ("c", 1, 1), ("d", 2100, 4)], seed=77)
    q = torch.randn(batch.tokens, 24, 128, generator=torch.Generator().manual_seed(5)).bfloat16().cuda()
    out, lse = attention.forward(0, q, pool, batch, lse=True)
    want, want_lse = oracle_rows(pool, batch, q)
    assert_attention_close(out, lse, want, want_lse, list(range(batch.tokens)))
    again = attention.forward(0, q, pool, batch)           # without lse: the same bits
    assert torch.equal(again, out)
    # every row alone decodes to the same bits as in the batch
    for r in range(batch.rows):
        s, first, count, position = batch.row(r)
        alone = StepBatch.build([(s, position, count)], "cuda")
        pool.reserve(alone)
        assert torch.equal(attention.forward(0, q[first:first + count], pool, alone), out[first:first + count])


def test_verify_windows_through_the_tcgen05_engine_match_the_oracle():
    """window_engine tcgen05: the verify windows it serves go through the tcgen05 kernel (within the bounds, not the
    same bits as the m16n8k16 kernel), the launches it does not serve fall back."""
    from crit_b200.attention import DeviceAttention, PartitionedAttention
    from helpers import assert_attention_close
    kv, plain = parts()
    fast = PartitionedAttention(kv, {"world": 2, "page_size": 256}, DeviceAttention(device="cuda", window_engine="tcgen05"))
    assert fast.exactness()["decode"] == "repeatable" and plain.exactness()["decode"] == "row-exact"
    assert DeviceAttention(device="cuda").exactness()["decode"] == "repeatable"        # the default, "auto"
    pool = kv.pool([0], 4, 128, 16 * 400, "cuda", "fp8:page")
    for s, n in {"a": 700, "b": 64, "d": 2100}.items():
        pool.open(s)
        step(pool, [(s, 0, n)], seed=len(s) + n)
        pool.keep(s, n)
    batch, _, _ = step(pool, [("a", 700, 5), ("b", 64, 2), ("d", 2100, 4)], seed=77)
    q = torch.randn(batch.tokens, 24, 128, generator=torch.Generator().manual_seed(5)).bfloat16().cuda()
    out, lse = fast.forward(0, q, pool, batch, lse=True)
    want, want_lse = oracle_rows(pool, batch, q)
    assert_attention_close(out, lse, want, want_lse, list(range(batch.tokens)))
    assert torch.equal(fast.forward(0, q, pool, batch), out)
    other = plain.forward(0, q, pool, batch)
    torch.testing.assert_close(out.float(), other.float(), atol=1e-2, rtol=2e-2)
    import crit_b200
    assert crit_b200.status() == 0


def test_a_prompt_row_past_the_window_is_causal_over_its_own_chunk():
    from helpers import assert_attention_close
    kv, attention = parts()
    pool = kv.pool([0], 2, 128, 16 * 64, "cuda", "bf16")
    pool.open("a")
    step(pool, [("a", 0, 150)], seed=1)
    pool.keep("a", 150)
    batch, _, _ = step(pool, [("a", 150, 100)], seed=2)     # 100 tokens > window 16: a prompt row
    q = torch.randn(100, 8, 128, generator=torch.Generator().manual_seed(6)).bfloat16().cuda()
    out, lse = attention.forward(0, q, pool, batch, lse=True)
    k, v = stored(pool)
    want, want_lse = oracle.attend(q.float().cpu().numpy(), k, v, np.array([pool.table("a")], np.int32), [0], [0],
                                   [150], 100, 16)
    assert_attention_close(out, lse, want, want_lse, list(range(100)))


@pytest.mark.parametrize("dtype", ["bf16", "fp8:row"])
def test_a_steps_prompt_rows_take_one_launch_and_match_the_oracle(dtype, monkeypatch):
    """Three sequences' chunks of different lengths (and a decode row between the steps): the prompt rows, which follow
    one another in q, go to the prefill kernel in ONE launch, and every row matches the oracle over its own sequence."""
    import crit_b200
    from helpers import assert_attention_close
    kv, attention = parts()
    pool = kv.pool([0], 2, 128, 16 * 96, "cuda", dtype)
    for name in "abc":
        pool.open(name)
    step(pool, [("a", 0, 150), ("b", 0, 40)], seed=1)
    pool.keep("a", 150), pool.keep("b", 40)
    batch, _, _ = step(pool, [("a", 150, 100), ("b", 40, 33), ("c", 0, 70)], seed=2)
    q = torch.randn(203, 8, 128, generator=torch.Generator().manual_seed(6)).bfloat16().cuda()
    calls = []
    real = crit_b200.prefill
    monkeypatch.setattr(crit_b200, "prefill", lambda *a, **k: (calls.append(a[4].dim()), real(*a, **k))[1])
    out, lse = attention.forward(0, q, pool, batch, lse=True)
    assert calls == [2]                                   # one launch, a table of three rows
    want, want_lse = oracle_rows(pool, batch, q)
    assert_attention_close(out, lse, want, want_lse, list(range(203)))


def test_merged_shards_equal_attention_over_the_whole_sequence():
    """inference/partitioned-attention/tests/test_device.py:44-68, on this pool and attention."""
    from crit_b200.batch import StepBatch
    kv, attention = parts()
    g = torch.Generator().manual_seed(1)
    keys, values = torch.randn(300, 2, 64, generator=g).bfloat16().cuda(), torch.randn(300, 2, 64, generator=g).bfloat16().cuda()
    q = torch.randn(1, 4, 64, generator=g).bfloat16().cuda()

    def pool_of(rows):
        pool = kv.pool([0], 2, 64, 2048, "cuda", "bf16")
        for s, (k, v) in rows.items():
            pool.open(s)
            batch = StepBatch.build([(s, 0, k.shape[0])], "cuda")
            pool.write(0, pool.reserve(batch), k, v)
            pool.keep(s, k.shape[0])
        return pool
    whole = pool_of({"s": (keys, values)})
    shards = pool_of({"a": (keys[:120], values[:120]), "b": (keys[120:], values[120:])})

    def attend(pool, s, position):
        batch = StepBatch.build([(s, position, 1)], "cuda")
        pool.reserve(batch)
        return attention.forward(0, q, pool, batch, lse=True)
    out, lse = attend(whole, "s", 299)
    found = [attend(shards, s, n - 1) for s, n in (("a", 120), ("b", 180))]
    merged, merged_lse = attention.merge([o for o, _ in found], [x for _, x in found])
    torch.testing.assert_close(merged.float(), out.float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(merged_lse, lse, atol=2e-3, rtol=1e-4)
    k = whole.gather(0, "s", 300)[0].double()
    for h in range(4):
        s = k[:, h // 2] @ q[0, h].double() / math.sqrt(64)
        assert abs(float(lse[0, h]) - float(torch.logsumexp(s, 0))) < 2e-3
    outs = [torch.ones(2, 1, 3).cuda(), torch.zeros(2, 1, 3).cuda()]
    lses = [torch.tensor([[0.5], [float("-inf")]]).cuda(), torch.full((2, 1), float("-inf")).cuda()]
    out, lse = attention.merge(outs, lses)
    assert out[0].tolist() == [[1.0, 1.0, 1.0]]
    assert (out[1].tolist(), lse[1].tolist()) == ([[0.0, 0.0, 0.0]], [float("-inf")])
    assert abs(float(lse[0, 0]) - 0.5) < 1e-6


def test_a_decode_step_replays_in_a_cuda_graph_over_the_step_buffers():
    """The pool's step buffers keep a step's slots and window rows at fixed addresses: a graph captured over one step
    replays after the next reserve() (other lengths, other rows) and gives that step's attention."""
    from crit_b200.batch import StepBatch
    from helpers import assert_attention_close
    kv, attention = parts(step_rows=4, step_tokens=512)
    pool = kv.pool([0], 2, 128, 16 * 64, "cuda", "bf16")
    lens = {"a": 40, "b": 300, "c": 5}
    for s, n in lens.items():
        pool.open(s)
        step(pool, [(s, 0, n)], seed=n)
        pool.keep(s, n)
    q = torch.zeros(3, 8, 128, dtype=torch.bfloat16, device="cuda")
    keys = torch.zeros(3, 2, 128, dtype=torch.bfloat16, device="cuda")
    values = torch.zeros_like(keys)
    g = torch.Generator().manual_seed(8)

    def fill():
        q.copy_(torch.randn(3, 8, 128, generator=g).bfloat16())
        keys.copy_(torch.randn(3, 2, 128, generator=g).bfloat16())
        values.copy_(torch.randn(3, 2, 128, generator=g).bfloat16())
    batch = StepBatch.build([(s, lens[s], 1) for s in "abc"], "cuda")
    slots = pool.reserve(batch)
    fill()
    pool.write(0, slots, keys, values)
    attention.forward(0, q, pool, batch, lse=True)              # warm: workspaces are made outside the capture
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            pool.write(0, slots, keys, values)
            out, lse = attention.forward(0, q, pool, batch, lse=True)
    for turn in range(3):
        for s in "abc":
            pool.keep(s, lens[s] + 1)
            lens[s] += 1
        batch = StepBatch.build([(s, lens[s], 1) for s in "abc"], "cuda")
        assert pool.reserve(batch).data_ptr() == slots.data_ptr()
        fill()
        graph.replay()
        torch.cuda.synchronize()
        want, want_lse = oracle_rows(pool, batch, q)
        assert_attention_close(out, lse, want, want_lse, [0, 1, 2])


def test_facts_count_the_bytes_a_token_takes():
    kv, attention = parts()
    kv.pool([0, 1], 8, 128, 1024, "cuda", "fp8:page")
    assert kv.facts()["kv_bytes_per_token"] == 2 * (8 * 128 * 2 + 8 * 2 * 4 / 16)
    assert attention.exactness()["decode"] == "row-exact"


# -- draft trees: the window reads a tree, the round's commit brings the accepted path together ----------------------------
def test_move_rows_moves_a_lists_rows_in_order():
    """crit_b200.move_rows against gather-then-scatter: a path whose targets are other moves' sources (node 2 -> 1, node
    3 -> 2), moves from a slot to itself, two stores of different row sizes."""
    import crit_b200 as pk
    g = torch.Generator().manual_seed(3)
    store = torch.randn(3, 40, 2, 64, generator=g).bfloat16().cuda()
    scales = torch.randn(3, 40, 2, generator=g).cuda()
    source = torch.tensor([[5, 7, 8, 9, 39], [20, 23, 22, 39, 39]], dtype=torch.int64, device="cuda")
    target = torch.tensor([[5, 6, 7, 8, 39], [20, 21, 22, 39, 39]], dtype=torch.int64, device="cuda")
    for s in (store, scales):
        want = s.clone()
        want.index_copy_(1, target.reshape(-1), s.index_select(1, source.reshape(-1)))
        pk.move_rows(s, source, target)
        assert torch.equal(s, want)
    assert pk.status() == 0


@pytest.mark.parametrize("dtype", ["bf16", "fp8:row", "fp8"])
def test_a_round_over_a_draft_tree_reads_ancestors_and_commits_the_accepted_path(dtype):
    """A bound sequence, a round whose window is a draft tree: every node's KV is written at position start + node, the
    attention sees a node's ancestors (parents), and commit_round(view.tree_path) moves the accepted nodes' KV to
    consecutive positions, once, in every layer, codes and scales alike."""
    import types
    from crit_b200.batch import StepBatch
    from helpers import assert_attention_close
    kv, attention = parts(round_rows=2)
    pool = kv.pool([0, 1], 2, 128, 16 * 40, "cuda", dtype)
    if dtype == "fp8":
        pool.set_scales(0, 0.05, 0.04), pool.set_scales(1, 0.03, 0.06)
    pool.open("a")
    first = pool.reserve(StepBatch.build([("a", 0, 45)], "cuda"))
    for layer in (0, 1):
        pool.write(layer, first, rows_of(45, 2, 128, 1 + layer), rows_of(45, 2, 128, 5 + layer))
    pool.keep("a", 45)
    pool.bind(0, "a", 45 + 16)
    # the tree: node 0 the pending token; 1 and 2 its children; 3 under 1; 4 under 3; 5 under 2
    parents = torch.tensor([-1, 0, 0, 1, 3, 2], dtype=torch.int32, device="cuda")
    view = types.SimpleNamespace(rows=1, n_emitted=torch.tensor([4], device="cuda"), frontier=torch.tensor([49], device="cuda"),
                                 tree_path=torch.tensor([[0, 1, 3, 4, -1, -1]], device="cuda"))
    pool.start_round(view)
    slots = pool.slots_at(torch.zeros(6, dtype=torch.int64, device="cuda"), 45 + torch.arange(6, device="cuda"))
    for layer in (0, 1):
        pool.write(layer, slots, rows_of(6, 2, 128, 20 + layer), rows_of(6, 2, 128, 30 + layer))
    # the attention over the tree, layer 0
    q = torch.randn(6, 8, 128, generator=torch.Generator().manual_seed(9)).bfloat16().cuda()
    rb = types.SimpleNamespace(round=True, prompt=False, rows=1, width=5, slots_t=torch.zeros(1, dtype=torch.int64, device="cuda"),
                               starts_t=torch.zeros(1, dtype=torch.int32, device="cuda"), frontier_t=torch.tensor([45], device="cuda"))
    out, lse = attention.forward(0, q, pool, rb, parents=parents, lse=True)
    k, v = stored(pool, 0)
    table = pool.round_tables[0].cpu().numpy()[None]
    want, want_lse = oracle.attend_tree(q.float().cpu().numpy(), k, v, table, [0], [0], [45], 6, pool.page, parents.cpu().numpy())
    assert_attention_close(out, lse, want, want_lse, list(range(6)))
    # the accepted path 0 -> 1 -> 3 -> 4 comes together at positions 45..48
    stores = [pool.k, pool.v] + ([pool.k_scales, pool.v_scales] if pool.k_scales is not None else [])
    snapshot = [t.clone() for t in stores]
    pool.commit_round(view)

    def flat(t):                # [layers][slots][...]
        return t.reshape(t.shape[0], t.shape[1] * t.shape[2], *t.shape[3:])
    s = slots.cpu().tolist()
    for was, now in zip(snapshot, stores):
        was, now = flat(was), flat(now)
        for j, node in enumerate([0, 1, 3, 4]):
            assert torch.equal(now[:, s[j]].contiguous().view(torch.uint8), was[:, s[node]].contiguous().view(torch.uint8))
    assert int(pool.round_lengths[0]) == 49
    # a second commit of the same round moves nothing more
    again = [t.clone() for t in stores]
    pool.commit_round(view)
    for was, now in zip(again, stores):
        assert torch.equal(was.view(torch.uint8), now.view(torch.uint8))
    pool.unbind(0)
    assert pool.length("a") == 49
    with pytest.raises(NotImplementedError):
        paged = kv.pool([0], 2, 128, 16 * 8, "cuda", "fp8:page", )
        paged._compact(1, view.n_emitted, view.tree_path)


# -- fresh rows: a prompt chunk over quantised pages is scored with the keys and values it was given ---------------------
@pytest.mark.parametrize("dtype", ["fp8:row", "fp8:page", "int8", "fp8"])
@pytest.mark.parametrize("position,count", [(0, 70), (333, 150), (1000, 40)])
def test_prompt_rows_read_their_own_chunk_fresh(dtype, position, count):
    """A pool of quantised pages with a fresh buffer: a prompt row attends its chunk's own positions from the 16-bit rows
    write() got and the earlier ones from the pages (reference: device_attention.py:1136-1145).  The oracle reads the
    stored (dequantised) pages with the chunk's slots replaced by the rows as given."""
    from crit_b200.attention import DeviceAttention, PartitionedAttention
    from crit_b200.batch import StepBatch
    from crit_b200.kv_state import KVStateCache
    from crit_b200.pool import FreshBuffer
    from helpers import assert_attention_close
    import crit_b200
    fresh = FreshBuffer(torch.empty(1 << 20, dtype=torch.uint8, device="cuda"))
    kv = KVStateCache(page=16, kernels=crit_b200, fresh=fresh)
    attention = PartitionedAttention(kv, {"world": 2, "page_size": 256}, DeviceAttention(device="cuda"))
    pool = kv.pool([0], 2, 128, 16 * 100, "cuda", dtype)
    if dtype == "fp8":
        pool.set_scales(0, 0.05, 0.04)
    assert pool.fresh_tokens == (1 << 20) // (2 * 256 * 2)
    pool.open("a")
    if position:
        step(pool, [("a", 0, position)], seed=1)
        pool.keep("a", position)
    batch, keys, values = step(pool, [("a", position, count)], seed=7)
    got = pool.fresh_rows(0, count)
    assert got is not None and torch.equal(got[0], keys) and torch.equal(got[1], values)
    q = torch.randn(count, 8, 128, generator=torch.Generator().manual_seed(3)).bfloat16().cuda()
    out, lse = attention.forward(0, q, pool, batch, lse=True)
    k, v = stored(pool, 0)
    slots = pool.reserve(batch).cpu().numpy()            # (the same slots again: the chunk's)
    k[slots], v[slots] = keys.float().cpu().numpy(), values.float().cpu().numpy()
    table = np.array(pool.table("a"), np.int32)[None]
    want, want_lse = oracle.attend(q.float().cpu().numpy(), k, v, table, [0], [0], [position], count, pool.page)
    assert_attention_close(out, lse, want, want_lse, list(range(count)))
    # without the buffer the chunk is read from the pages: the two differ by the pages' quantisation
    plain_kv = KVStateCache(page=16, kernels=crit_b200)
    assert plain_kv.pool([0], 2, 128, 16 * 8, "cuda", dtype).fresh_rows(0, count) is None
    # a decode step after it keeps nothing fresh (no prompt row in the step)
    pool.keep("a", position + count)
    step(pool, [("a", position + count, 1)], seed=9)
    assert pool.fresh_rows(0, 1) is None


def test_a_fresh_prompt_chunk_matches_the_references_torch_path(golden):
    """The reference pool's fresh chunk (tests/golden/make_golden.py: fresh_chunk): its stored codes and scales installed
    in a pool here, the chunk written again through write() with a fresh buffer, forward() against the reference's
    outputs."""
    from crit_b200.attention import DeviceAttention
    from crit_b200.batch import StepBatch
    from crit_b200.kv_state import KVStateCache
    from crit_b200.pool import FreshBuffer
    from helpers import assert_attention_close
    import crit_b200
    f = golden("fresh_fp8row.npz")
    hq, hkv, d, page, n, count = (int(x) for x in f["geometry"])
    kv = KVStateCache(page=page, kernels=crit_b200, fresh=FreshBuffer(torch.empty(1 << 18, dtype=torch.uint8, device="cuda")))
    pool = kv.pool([0], hkv, d, 24 * page, "cuda", "fp8:row")
    pool.open("a")
    pool.reserve(StepBatch.build([("a", 0, n)], "cuda"))
    pool.keep("a", n)
    assert pool.table("a") == f["table"].tolist()[:len(pool.table("a"))]          # the same page order as the reference's pool
    pool.k[0].view(torch.uint8).copy_(torch.tensor(f["k_codes"]).view(pool.k[0].shape).cuda())
    pool.v[0].view(torch.uint8).copy_(torch.tensor(f["v_codes"]).view(pool.v[0].shape).cuda())
    pool.k_scales[0].copy_(torch.tensor(f["k_scales"]).cuda()), pool.v_scales[0].copy_(torch.tensor(f["v_scales"]).cuda())
    batch = StepBatch.build([("a", n, count)], "cuda")
    slots = pool.reserve(batch)
    assert slots.cpu().tolist() == f["slots"].tolist()
    pool.write(0, slots, torch.tensor(f["k1"]).bfloat16().cuda(), torch.tensor(f["v1"]).bfloat16().cuda())
    q = torch.tensor(f["q"]).bfloat16().cuda()
    out, lse = DeviceAttention(device="cuda").forward(0, q, pool, batch, lse=True)
    assert_attention_close(out, lse, f["out"], f["lse"], list(range(count)))
