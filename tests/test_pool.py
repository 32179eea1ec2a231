"""The pool's host logic (page tables, slot maps, copy on write, rollback) against the reference pool's own trace
(tests/golden/pool_script.json, recorded from the reference's KVPool on the CPU), bit for bit; no GPU needed."""
import numpy as np
import pytest
import torch

from crit_b200.batch import StepBatch
from crit_b200.pool import KVPool


def test_tables_slots_and_free_pages_follow_the_references_trace(golden):
    script = golden("pool_script.json")
    pool = KVPool([0], 2, 64, script["pages"] * script["page"], "cpu", "bf16", page=script["page"])
    for step in script["trace"]:
        op, slots = step["op"], None
        if op[0] == "open":
            pool.open(op[1])
        elif op[0] == "close":
            pool.close(op[1])
        elif op[0] == "fork":
            pool.fork(op[1], op[2])
        elif op[0] == "keep":
            pool.keep(op[1], op[2])
        else:
            slots = pool.reserve(StepBatch.build([tuple(r) for r in op[1]], "cpu")).tolist()
        assert slots == step["slots"], op
        assert {s: pool.table(s) for s in sorted(pool.tables)} == step["tables"], op
        assert {s: pool.lengths[s] for s in sorted(pool.tables)} == step["lengths"], op
        assert pool.free_pages() == step["free"] and pool.floor == step["floor"], op
        # the block table on the device mirrors the host lists, unused entries at the dump page
        pool._flush()
        for s, table in step["tables"].items():
            row = pool.block_tables[pool.row_of[s]].tolist()
            assert row[:len(table)] == table and set(row[len(table):]) <= {pool.dump}, (op, s)


def test_a_full_pool_is_refused_with_the_references_message(golden):
    pool = KVPool([0], 2, 64, 32, "cpu", page=16)
    pool.open("a")
    with pytest.raises(MemoryError) as refused:
        pool.reserve(StepBatch.build([("a", 0, 40)], "cpu"))
    assert str(refused.value) == golden("pool_script.json")["refused"]


def test_on_exhausted_is_asked_before_the_pool_refuses():
    pool = KVPool([0], 1, 64, 32, "cpu", page=16)
    pool.open("old")
    pool.reserve(StepBatch.build([("old", 0, 32)], "cpu"))
    pool.open("new")
    asked = []

    def room():
        asked.append(1)
        if "old" in pool.tables:
            pool.close("old")
            return True
        return False
    pool.on_exhausted(room)
    assert pool.reserve(StepBatch.build([("new", 0, 20)], "cpu")).tolist() == list(range(20))
    assert asked


def test_errors_name_the_sequence():
    pool = KVPool([0], 1, 64, 64, "cpu", page=16)
    pool.open("a")
    with pytest.raises(ValueError, match="is open already"):
        pool.open("a")
    with pytest.raises(ValueError, match="is not open"):
        pool.keep("b", 0)
    pool.reserve(StepBatch.build([("a", 0, 16)], "cpu"))
    with pytest.raises(ValueError, match="holds 16 reserved positions, not 20"):
        pool.keep("a", 20)
    with pytest.raises(ValueError, match="stores"):
        KVPool([0], 1, 64, 64, "cpu", "fp4")


def test_round_slots_on_a_cpu_pool_match_the_references(golden):
    data = golden("round_slots.npz")
    pool = KVPool([0], 2, 64, 32 * 8, "cpu", page=8, round_rows=4)
    for s, n in (("a", 13), ("b", 1), ("c", 30)):
        pool.open(s)
        pool.reserve(StepBatch.build([(s, 0, n)], "cpu"))
        pool.keep(s, n)
    pool.bind(0, "a", 40)
    pool.bind(2, "c", 64)
    pool.bind(1, "b", 9)
    assert np.array_equal(pool.round_tables.numpy(), data["tables"])
    assert np.array_equal(pool.round_capacity.numpy(), data["capacity"])
    got = pool.slots_at(torch.from_numpy(data["slot"]), torch.from_numpy(data["positions"]))
    assert np.array_equal(got.numpy(), data["slots"])
    pool.unbind(1)
    assert pool.length("b") == 1 and len(pool.table("b")) == 1
    with pytest.raises(ValueError, match="holds no sequence"):
        pool.unbind(1)


def test_the_block_table_grows_with_the_sequences():
    pool = KVPool([0], 1, 64, 16 * 40, "cpu", page=16, sequences=2)
    for s in range(5):
        pool.open(s)
        pool.reserve(StepBatch.build([(s, 0, 17)], "cpu"))
    pool._flush()
    assert pool.block_tables.shape[0] >= 5
    for s in range(5):
        assert pool.block_tables[pool.row_of[s], :2].tolist() == pool.table(s)


def test_kv_state_host_form_is_transactional():
    from crit_b200.kv_state import KVStateCache
    kv = KVStateCache()
    kv.open("a", 2, 1, 4)
    kv.stage("a", [[1.0, 2.0], [3.0, 4.0]], [[5.0], [6.0]])
    assert kv.rows("a") == [] and len(kv.rows("a", pending=True)) == 2
    kv.commit("a", 1)
    assert kv.rows("a") == [(0, [1.0, 2.0], [5.0])]
    kv.stage("a", [[0.0, 0.0]], [[1.0]])
    kv.rollback("a")
    kv.fork("a", "b")
    assert kv.rows("b") == kv.rows("a")
    kv.release("a")
    with pytest.raises(ValueError, match="is not open"):
        kv.rows("a")
    with pytest.raises(ValueError, match="KV capacity exhausted"):
        kv.stage("b", [[0.0, 0.0]] * 4, [[0.0]] * 4)


def test_the_native_page_allocator_takes_the_lowest_free_page():
    """crit_b200_pager_* (csrc/pager.cu): the lowest free page first, reference counts, the floor, a step's rows grown in one
    call in the order a row-by-row loop would take their pages, and what is left when the pool runs out."""
    from crit_b200.pool import Pager
    pager = Pager(8)
    assert [pager.take() for _ in range(3)] == [0, 1, 2] and (pager.free(), pager.floor(), pager.shared()) == (5, 3, 0)
    assert pager.share(1) == 2 and pager.shared() == 1 and pager.refs(1) == 2
    assert pager.drop(1) == 1 and pager.shared() == 0 and pager.free() == 5           # still held once
    assert pager.drop(1) == 0 and pager.free() == 6 and pager.floor() == 3
    assert pager.drop(2) == 0 and pager.floor() == 1                                  # the floor falls past both
    assert pager.drop(5) == -1 and pager.share(5) == -1 and pager.refs(99) == -1
    pages, short = pager.grow([1, 0, 2], [3, 1, 2])                                   # rows gain 2, 1 and 0 pages
    assert (pages, short) == ([1, 2, 3], False) and pager.floor() == 4
    pages, short = pager.grow([0, 0], [3, 3])                                         # 4 free, 6 wanted
    assert (pages, short) == ([4, 5, 6, 7], True) and pager.free() == 0 and pager.take() == -1
