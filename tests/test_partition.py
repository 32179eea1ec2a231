"""The attention slot's host form: ownership is a bijection, partials of disjoint shards merge to the direct softmax
(the cases of the reference's own host tests, tests/test_reusable_techniques.py:106-193, and its recorded outputs)."""
import math
import random

import pytest

from crit_b200 import partition as m


def test_partition_is_bijective_balanced_and_respects_page_boundaries():
    for world in (1, 2, 3, 8):
        for count in (0, 1, 7, 16, 33, 257):
            shards = [m.SequencePartition(world, r, 4) for r in range(world)]
            restored = []
            for shard in shards:
                positions = [shard.global_position(i) for i in range(shard.length(count))]
                restored.extend(positions)
                for p in positions:
                    page, row = shard.address(p)
                    assert page * 4 + row == shard.local(p) and page < shard.pages(count)
            assert sorted(restored) == list(range(count))
            assert max(s.length(count) for s in shards) - min(s.length(count) for s in shards) <= 1
    with pytest.raises(ValueError):
        m.SequencePartition(2, 0).local(1)
    for args in ((0, 0), (2, 2), (True, 0)):
        with pytest.raises(ValueError):
            m.SequencePartition(*args)


def test_partials_match_the_references_recorded_ones(golden):
    host = golden("merge_host.json")
    rows = [(p, tuple(k), tuple(v)) for p, k, v in host["rows"]]
    for world, found in host["worlds"].items():
        world = int(world)
        partials = [m.attention_partial(tuple(host["query"]), [r for r in rows if r[0] % world == rank], value_width=2,
                                        query_position=host["position"], scale=host["scale"]) for rank in range(world)]
        for got, want in zip(partials, found["partials"]):
            assert list(got.output) == want[0] and got.log_normalizer == want[1]
        merged = m.merge_partials(partials)
        assert list(merged.output) == found["merged"][0] and merged.log_normalizer == found["merged"][1]


def test_dense_and_sparse_causal_partials_match_direct_softmax():
    rng = random.Random(51)
    rows = [(i, tuple(rng.uniform(-2, 2) for _ in range(3)), tuple(rng.uniform(-3, 3) for _ in range(2))) for i in range(19)]
    for query_position in (0, 1, 6, 18):
        for selected in (None, (0, 3, 7, 12, 18)):
            query = tuple(rng.uniform(-1, 1) for _ in range(3))
            visible = [(k, v) for p, k, v in rows if p <= query_position and (selected is None or p in selected)]
            weights = [math.exp(sum(q * x for q, x in zip(query, k)) * .5) for k, _ in visible]
            expected = [sum(w * v[c] for w, (_, v) in zip(weights, visible)) / sum(weights) for c in range(2)]
            for world in (1, 2, 4, 23):
                partials = [m.attention_partial(query, [row for row in rows if row[0] % world == rank], value_width=2,
                                                query_position=query_position, scale=.5, selected_positions=selected)
                            for rank in range(world)]
                merged = m.merge_partials(partials)
                for a, b in zip(expected, merged.output):
                    assert abs(a - b) < 1e-13
                assert abs(merged.log_normalizer - math.log(sum(weights))) < 1e-13


def test_extreme_scores_empty_shards_and_nonfinite_inputs():
    empty = m.AttentionPartial((0., 0.), -math.inf)
    a, b = m.AttentionPartial((2., 4.), 10000.), m.AttentionPartial((10., 20.), 9999.)
    merged = m.merge_partials((a, b, empty))
    assert abs(merged.output[0] - (2 + 10 / math.e) / (1 + 1 / math.e)) < 1e-12
    with pytest.raises(ValueError):
        m.merge_partials((empty, empty))
    for lse in (math.nan, math.inf, True):
        with pytest.raises(ValueError):
            m.AttentionPartial((0.,), lse)
    with pytest.raises(ValueError):
        m.AttentionPartial((1.,), -math.inf)
    with pytest.raises(ValueError):
        m.merge_partials((a, m.AttentionPartial((1.,), 0.)))
    with pytest.raises(ValueError):
        m.attention_partial((1.,), [(5, (math.nan,), (1.,))], value_width=1, query_position=0)


def test_head_major_scatter_and_hierarchical_normalizers():
    shards = tuple(tuple(tuple(m.AttentionPartial((10 * rank + head + q,), float(rank)) for head in range(4))
                         for q in range(3)) for rank in range(2))
    scattered = m.combine_and_scatter(shards)
    for rank in range(2):
        for local in range(2):
            for q in range(3):
                head = rank * 2 + local
                assert scattered[rank][local][q] == m.merge_partials((shards[0][q][head], shards[1][q][head]))
    parts = [m.AttentionPartial((float(r),), float(r)) for r in range(4)]
    hierarchical = m.merge_partials((m.merge_partials(parts[:2]), m.merge_partials(parts[2:])))
    assert abs(hierarchical.output[0] - m.merge_partials(parts).output[0]) < 1e-12
    with pytest.raises(ValueError):
        m.combine_and_scatter((shards[0], (shards[1][0][:3],)))


def test_duplicate_positions_masks_and_immutable_outputs():
    row = (0, (1.,), (2.,))
    for rows, selected in (((row, row), None), ((row,), (0, 0))):
        with pytest.raises(ValueError):
            m.attention_partial((1.,), rows, value_width=1, query_position=1, selected_positions=selected)
    p = m.attention_partial((1.,), (row,), value_width=1, query_position=0, selected_positions=())
    assert p == m.AttentionPartial((0.,), -math.inf)
    values = [2.]
    p = m.AttentionPartial(values, 0.)
    values[0] = 100.
    assert p.output == (2.,)


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
    scores = [sum(a * b for a, b in zip(query, k)) / math.sqrt(3) for k in keys[:6]]
    w = [math.exp(s - max(scores)) for s in scores]
    want = [sum(wi * v[c] for wi, v in zip(w, values)) / sum(w) for c in range(2)]
    assert all(abs(a - b) < 1e-12 for a, b in zip(got, want))
