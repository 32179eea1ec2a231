"""Parity at the benchmark's own geometry: every workload bench.py times is built here exactly as bench.py builds it
(same generator, same pages, same step), one step is run, and a seeded sample of its output rows is held to the CPU
oracle within the north-star bounds (max-abs 2e-2, mean-abs 2e-3 in bf16; lse 2e-3).  So the numbers the bench reports
rest on outputs checked at size, not on small cases of the same templates.  The reference's own tests compare its
kernel with float64 over the stored values the same way (paged-kv-attention/tests/test_paged_kv_attention.py:132-152).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(name, engine=None, rank=0, world=1, **change):
    import bench
    w = dict(bench.WORKLOADS[name], **change)
    state = bench.build_state(w, torch.device("cuda"), rank, world)
    state["engine"], state["staging"] = engine, None
    bench.step(state)
    torch.cuda.synchronize()
    return bench, state


def _held(found):
    assert found["ok"], found
    assert found["max_abs"] <= 2e-2 and found["mean_abs"] <= 2e-3 and found["lse_abs"] <= 2e-3, found


@pytest.mark.parametrize("name", ["c2", "c2row"])
def test_fp8_decode_of_64_rows_of_4096_positions(name):
    """64 rows x 4,096 positions, 64q/8kv x 128, page 16, x20 outliers, a scale per (page, kv head) and per (slot, kv
    head): 16 sampled rows of the timed step against the oracle."""
    import crit_b200 as pk
    bench, state = _run(name)
    assert state["kv_bytes"] == 262144 * (2052 if name == "c2" else 2112)
    _held(bench.parity(state, rows=16))
    assert pk.status() == 0


def test_long_context_decode_of_200000_positions_over_pages_of_64():
    """One row of 200,000 positions, 24q/4kv x 256, page 64, bf16: every split of the launch and their fold."""
    import crit_b200 as pk
    bench, state = _run("c3")
    assert state["kv_bytes"] == 200000 * 4096
    splits = -(-200000 // state["chunk"])
    assert splits > 100 and state["chunk"] % 16 == 0
    _held(bench.parity(state))
    # the library's own chunk too (the bench picks one that fills the device in whole waves)
    state["chunk"] = None
    bench.step(state)
    _held(bench.parity(state))
    assert pk.status() == 0


@pytest.mark.parametrize("world", [2, 8])
def test_long_context_decode_sharded_by_kv_range(world):
    """The same context cut into `world` KV ranges at page boundaries: every range's split-K decode, its fold stored
    into every rank's exchange buffer and the merge of shards out of a rank's own buffer (the ranks emulated on one
    GPU), against the oracle over the whole context."""
    import crit_b200 as pk
    import oracle
    from crit_b200.dist import chunk_to_fill, kv_ranges
    from helpers import EmulatedRanks
    bench, state = _run("c3")
    w = state["w"]
    page, hq, d = w["page"], w["hq"], w["d"]
    ranges = kv_ranges(w["ctx"], world, partition=page)
    assert all(b > a for a, b in ranges) and ranges[-1][1] == w["ctx"]
    ranks = EmulatedRanks(world, 1, hq, d)
    q = state["sets"][0]["q"]
    dev = q.device
    i32 = dict(dtype=torch.int32, device=dev)
    found = pk.plan(hq, w["hkv"], d, d, page, "bf16", 1, dev)
    keep = []

    class Push:            # stands where a ShardMerge stands in attend(): this rank's fold + push only
        def __init__(self, rank):
            self.rank = rank

        def attend(self, params, out, lse):
            ranks.push(self.rank, params)
    for rank, (a, b) in enumerate(ranges):
        table = state["tables"][0][a // page:-(-b // page)].contiguous()[None]
        chunk = chunk_to_fill(b - a, w["hkv"], found["sms"] * max(found["per_sm"], 1))
        out, lse = torch.zeros(1, hq, d, dtype=torch.bfloat16, device=dev), torch.zeros(1, hq, device=dev)
        keep.append((table, out, lse))
        pk.attend(q, state["k"], state["v"], "bf16", table, torch.zeros(1, **i32), torch.zeros(1, **i32),
                  torch.tensor([b - a - 1], dtype=torch.int64, device=dev), 1, page, out=out, lse=lse, chunk=chunk,
                  shards=Push(rank))
    merged = [(torch.zeros(1, hq, d, dtype=torch.bfloat16, device=dev), torch.zeros(1, hq, device=dev)) for _ in range(world)]
    for rank in range(world):
        ranks.wait_merge(rank, *merged[rank])
    torch.cuda.synchronize()
    assert all(int(s.item()) == 0 for s in ranks.status)
    k, v = bench.stored_rows(state, 0)
    want, want_lse = oracle.attend(q.float().cpu().numpy(), k, v, np.arange(-(-w["ctx"] // page), dtype=np.int32), [0], [0],
                                   [w["ctx"] - 1], 1, page)
    for out, lse in merged:
        assert torch.equal(out, merged[0][0]) and torch.equal(lse, merged[0][1])       # every rank: the same bits
    err = np.abs(merged[0][0].float().cpu().numpy() - want)
    assert err.max() <= 2e-2 and err.mean() <= 2e-3, (err.max(), err.mean())
    assert np.abs(merged[0][1].cpu().numpy() - want_lse).max() <= 2e-3


@pytest.mark.parametrize("engine", [None, "mma.sync", "tcgen05"])
def test_speculative_verify_of_six_columns_over_lognormal_contexts(engine):
    """32 sequences x 6 draft tokens, 40q/8kv x 128 (30 query rows a kv head), contexts 512..65,536 with the longest
    row sampled, FP8 pages with a scale per (page, kv head): the library's choice of engine and each engine by name."""
    import crit_b200 as pk
    bench, state = _run("c5", engine=engine, rank=2, world=8)          # the third GPU's 32 sequences: one of 65,536 positions
    assert max(state["lens"]) == 65536 and len(state["lens"]) == 32
    _held(bench.parity(state, rows=6))
    assert pk.status() == 0


@pytest.mark.parametrize("engine", [None, "mma.sync"])
def test_chunked_prefill_of_2048_tokens_at_position_32768(engine):
    """4 sequences, a chunk of 2,048 tokens appended at position 32,768 and attended causally, 32q/8kv x 128, page 16,
    bf16: 16 sampled tokens of every sequence (the chunk's first and last among them)."""
    import crit_b200 as pk
    bench, state = _run("c4", engine=engine)
    found = bench.parity(state, tokens_per_row=16)
    assert found["tokens"] == 64
    _held(found)
    assert pk.status() == 0


def test_the_bench_refuses_outputs_outside_the_bounds():
    """The bench's own check is a check: a corrupted output row fails it."""
    bench, state = _run("c2", batch=4)
    assert bench.parity(state)["ok"]
    state["sets"][0]["out"][1] += 0.25
    assert not bench.parity(state)["ok"]
