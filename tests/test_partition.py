"""The attention slot's host form: every query's softmax taken shard by shard (interleaved ownership) and merged by
the shards' log-sum-exps equals the direct softmax, equals the reference's recorded partials
(tests/golden/merge_host.json, written by the reference's own host implementation), and refuses what the reference
refuses (the cases of its host tests, tests/test_reusable_techniques.py:106-193)."""
import math
import random

import numpy as np
import pytest

from crit_b200 import host_form as m


def _direct(query, keys, values, last, scale, chosen=None):
    seen = [(k, v) for p, (k, v) in enumerate(zip(keys, values)) if p <= last and (chosen is None or p in chosen)]
    weights = [math.exp(sum(a * b for a, b in zip(query, k)) * scale) for k, _ in seen]
    out = [sum(w * v[c] for w, (_, v) in zip(weights, seen)) / sum(weights) for c in range(len(values[0]))]
    return out, math.log(sum(weights))


def test_partials_match_the_references_recorded_ones(golden):
    host = golden("merge_host.json")
    assert [p for p, _, _ in host["rows"]] == list(range(len(host["rows"])))
    keys, values = [k for _, k, _ in host["rows"]], [v for _, _, v in host["rows"]]
    for world, found in host["worlds"].items():
        outs, lses = m.shard_partials(host["query"], keys, values, host["position"], int(world), host["scale"])
        for r, want in enumerate(found["partials"]):
            assert np.allclose(outs[r], want[0], rtol=0, atol=1e-13) and abs(lses[r] - want[1]) < 1e-13
        out, lse = m.merge_partials(outs, lses)
        assert np.allclose(out, found["merged"][0], rtol=0, atol=1e-13) and abs(lse - found["merged"][1]) < 1e-13


def test_shards_of_any_count_merge_to_the_direct_softmax():
    rng = random.Random(51)
    keys = [[rng.uniform(-2, 2) for _ in range(3)] for _ in range(19)]
    values = [[rng.uniform(-3, 3) for _ in range(2)] for _ in range(19)]
    for last in (0, 1, 6, 18):
        query = [rng.uniform(-1, 1) for _ in range(3)]
        want, want_lse = _direct(query, keys, values, last, 0.5)
        for world in (1, 2, 4, 23):
            outs, lses = m.shard_partials(query, keys, values, last, world, 0.5)
            owners_with_rows = {p % world for p in range(last + 1)}
            assert {r for r in range(world) if lses[r] > -math.inf} == owners_with_rows
            out, lse = m.merge_partials(outs, lses)
            assert np.allclose(out, want, rtol=0, atol=1e-13) and abs(lse - want_lse) < 1e-13
            assert np.allclose(m.attend(query, keys, values, last, world, 0.5), want, rtol=0, atol=1e-13)
    # explicit positions (a shard's own rows, in any order) give the same partials
    order = list(range(19))
    rng.shuffle(order)
    outs, lses = m.shard_partials(query, [keys[p] for p in order], [values[p] for p in order], 12, 4, 0.5, positions=order)
    again, again_lses = m.shard_partials(query, keys, values, 12, 4, 0.5)
    assert np.allclose(outs, again, rtol=0, atol=1e-13) and np.allclose(lses, again_lses, rtol=0, atol=1e-13)


def test_extreme_scores_empty_shards_and_nonfinite_inputs():
    out, lse = m.merge_partials([[2., 4.], [10., 20.], [0., 0.]], [10000., 9999., -math.inf])
    assert abs(out[0] - (2 + 10 / math.e) / (1 + 1 / math.e)) < 1e-12 and abs(lse - (10000 + math.log1p(1 / math.e))) < 1e-9
    with pytest.raises(ValueError, match="no visible keys"):
        m.merge_partials([[0., 0.], [0., 0.]], [-math.inf, -math.inf])
    for bad in (math.nan, math.inf):
        with pytest.raises(ValueError):
            m.merge_partials([[0.]], [bad])
    with pytest.raises(ValueError):
        m.merge_partials([[1., 2.], [1., 2.]], [0.])
    with pytest.raises(ValueError):
        m.shard_partials([1.], [[math.nan]], [[1.]], 0, 1)
    with pytest.raises(ValueError, match="overflow"):
        m.shard_partials([1e200], [[1e200]], [[1.]], 0, 1)
    for world in (0, True, 1.5):
        with pytest.raises(ValueError):
            m.shard_partials([1.], [[1.]], [[1.]], 0, world)
    # hierarchical merging equals merging at once
    outs, lses = [[float(r)] for r in range(4)], [float(r) for r in range(4)]
    left, right = m.merge_partials(outs[:2], lses[:2]), m.merge_partials(outs[2:], lses[2:])
    both, _ = m.merge_partials([left[0], right[0]], [left[1], right[1]])
    assert abs(both[0] - m.merge_partials(outs, lses)[0][0]) < 1e-12


def test_rows_are_transactional_and_grow():
    rows = m.Rows(2, 1, 40)
    rows.append([[1.0, 2.0], [3.0, 4.0]], [[5.0], [6.0]])
    assert len(rows.view()[0]) == 0 and len(rows.view(staged=True)[0]) == 2
    rows.settle(1)
    assert rows.view()[0].tolist() == [[1.0, 2.0]] and rows.view(staged=True)[1].tolist() == [[5.0]]
    rows.append([[0.0, 0.0]] * 30, [[1.0]] * 30)           # past the first allocation
    rows.drop()
    assert rows.view(staged=True)[0].tolist() == [[1.0, 2.0]]
    other = rows.fork()
    other.append([[7.0, 7.0]], [[7.0]])
    other.settle()
    assert len(other.view()[0]) == 2 and len(rows.view()[0]) == 1
    with pytest.raises(ValueError, match="capacity exhausted"):
        rows.append([[0.0, 0.0]] * 40, [[0.0]] * 40)
    with pytest.raises(ValueError, match="geometry differs"):
        rows.append([[0.0]], [[0.0]])
    with pytest.raises(ValueError, match="finite"):
        rows.append([[math.inf, 0.0]], [[0.0]])
    with pytest.raises(ValueError, match="commit exceeds"):
        rows.settle(3)
    for bad in ((0, 1, 1), (1, True, 1), (1, 1, -2)):
        with pytest.raises(ValueError):
            m.Rows(*bad)


def test_the_host_form_of_the_plugin_merges_interleaved_ranks():
    from crit_b200.attention import PartitionedAttention
    from crit_b200.kv_state import KVStateCache
    kv = KVStateCache()
    kv.open("s", 3, 2, 32)
    rng = random.Random(3)
    keys = [[rng.uniform(-1, 1) for _ in range(3)] for _ in range(9)]
    values = [[rng.uniform(-1, 1) for _ in range(2)] for _ in range(9)]
    kv.stage("s", keys, values)
    kv.commit("s")
    attention = PartitionedAttention(kv, {"world": 3, "page_size": 4}, device_form=None)
    query = [0.3, -0.2, 0.9]
    got = attention.attend("s", [query], [5])[0]
    want, _ = _direct(query, keys, values, 5, 1 / math.sqrt(3))
    assert all(abs(a - b) < 1e-12 for a, b in zip(got, want))
    kv.stage("s", [[0.5, 0.5, 0.5]], [[9.0, 9.0]])
    assert attention.attend("s", [query], [9])[0] == attention.attend("s", [query], [8])[0]     # staged rows: only when asked
    assert attention.attend("s", [query], [9], pending=True)[0] != got


def test_the_slot_cases_of_the_plugin_contract_run_on_the_host_forms():
    """The sequence of calls crit's own slot cases make (core/python/crit_plugins/slots.py:224-257), against the direct
    softmax."""
    from crit_b200.attention import PartitionedAttention
    from crit_b200.kv_state import KVStateCache
    kv = KVStateCache()
    attention = PartitionedAttention(kv, {"world": 2, "page_size": 256}, device_form=None)
    rng = random.Random(5)
    rows = lambda n, w: [[round(rng.uniform(-1, 1), 3) for _ in range(w)] for _ in range(n)]
    kv.open(11, 8, 5, 64)
    keys, values = rows(13, 8), rows(13, 5)
    kv.stage(11, keys, values)
    kv.commit(11)
    queries = rows(4, 8)
    for got, (query, last, scale) in zip(attention.attend(11, queries, [0, 5, 9, 12]),
                                         [(q, p, 8 ** -0.5) for q, p in zip(queries, [0, 5, 9, 12])]):
        assert np.allclose(got, _direct(query, keys, values, last, scale)[0], rtol=1e-7, atol=1e-9)
    got = attention.attend(11, queries[1:3], [7, 12], scale=0.5)
    assert np.allclose(got[0], _direct(queries[1], keys, values, 7, 0.5)[0], rtol=1e-7, atol=1e-9)
    more_k, more_v = rows(3, 8), rows(3, 5)
    kv.stage(11, more_k, more_v)
    got = attention.attend(11, queries[:3], [13, 14, 15], pending=True)
    assert np.allclose(got[2], _direct(queries[2], keys + more_k, values + more_v, 15, 8 ** -0.5)[0], rtol=1e-7, atol=1e-9)
    kv.rollback(11)
    assert len(kv.rows(11)) == 13
    kv.release(11)
    with pytest.raises(ValueError, match="is not open"):
        kv.rows(11)
