"""The multi-GPU path's host logic on CPU ranks (gloo, world_size 2): KV-range ownership, the all-gather of
(out, lse) partials and their merge in rank order, and failure detection made on the host (a stale message, a rank
that leaves) — no GPU is involved or faulted."""
import datetime
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from crit_b200 import dist as shard


def test_sequences_are_balanced_by_length():
    lengths = [65536, 512, 9000, 8000, 700, 30000, 1200, 2500]
    found = shard.assign_sequences(lengths, 4)
    assert sorted(s for rows in found for s in rows) == list(range(8))
    loads = [sum(lengths[s] for s in rows) for rows in found]
    blocks = [sum(lengths[s] for s in rows) for rows in shard.assign_sequences(lengths, 4, balance=False)]
    assert max(loads) <= max(blocks) and max(loads) == 65536
    assert shard.assign_sequences([5, 5, 5], 2, balance=False) == [[0, 1], [2]]


def test_kv_ranges_are_contiguous_whole_partitions():
    for world in (1, 2, 4, 8):
        ranges = shard.kv_ranges(200000, world)
        assert ranges[0][0] == 0 and max(b for _, b in ranges) == 200000
        assert all(a % 4096 == 0 or a == 200000 for a, _ in ranges)
        covered = sum(b - a for a, b in ranges)
        assert covered == 200000
        for (a, b), (c, d) in zip(ranges, ranges[1:]):
            assert b == c or (c == d)
    assert shard.kv_ranges(5000, 4) == [(0, 4096), (4096, 5000), (5000, 5000), (5000, 5000)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _case(seed=3, n=300, hq=4, hkv=2, d=16, page=4):
    g = np.random.default_rng(seed)
    pages = -(-n // page)
    table = g.permutation(pages + 2)[:pages].astype(np.int32)
    k = g.normal(size=((pages + 2) * page, hkv, d)).astype(np.float32)
    v = g.normal(size=((pages + 2) * page, hkv, d)).astype(np.float32)
    q = g.normal(size=(2, hq, d)).astype(np.float32)
    return q, k, v, table, n, page


def _numpy_merge(outs, lses):
    out, lse = oracle.merge(outs.numpy(), lses.numpy())
    return torch.from_numpy(out), torch.from_numpy(lse)


def _rank(rank, world, port, mode, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        q, k, v, table, n, page = _case()
        ranges = shard.kv_ranges(n, world, partition=128)
        lo, hi = ranges[rank]
        # each rank's partial over its own KV range: two decode tokens at positions n - 2, n - 1 (a window of 2)
        out, lse = oracle.attend(q, k, v, table, [0], [0], [n - 2], 2, page, lo=lo, hi=hi)
        merger = shard.ShardMerge(2, q.shape[1], v.shape[-1], "cpu", merge=_numpy_merge)
        if mode == "ok":
            for step in range(2):       # the buffers are reused step after step
                merged, merged_lse = merger.merge(torch.from_numpy(out), torch.from_numpy(lse), check=True)
            want, want_lse = oracle.attend(q, k, v, table, [0], [0], [n - 2], 2, page)
            queue.put((rank, float(np.abs(merged.numpy() - want).max()), float(np.abs(merged_lse.numpy() - want_lse).max())))
        elif mode == "stale":
            try:
                merger.merge(torch.from_numpy(out), torch.from_numpy(lse), check=True, epoch=7 if rank == 0 else 6)
                queue.put((rank, "published"))
            except RuntimeError as error:
                queue.put((rank, "refused" if "missing or stale" in str(error) else str(error)))
        elif mode == "leaves":
            if rank == 1:
                queue.put((rank, "left"))      # leaves between steps, nothing of its own in flight
                return
            try:
                merger.merge(torch.from_numpy(out), torch.from_numpy(lse), check=True)
                queue.put((rank, "published"))
            except Exception as error:          # the collective ends with an error, not a hang
                queue.put((rank, "refused"))
    finally:
        if mode != "leaves":
            dist.destroy_process_group()


def _run(mode, world=2):
    ctx = mp.get_context("spawn")
    queue, port = ctx.Queue(), _free_port()
    procs = [ctx.Process(target=_rank, args=(r, world, port, mode, queue)) for r in range(world)]
    for p in procs:
        p.start()
    found = [queue.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(60)
        if p.is_alive():
            p.kill()
    return sorted(found)


def test_kv_range_shards_merge_to_the_whole_on_two_ranks():
    for rank, err, lse_err in _run("ok"):
        assert err < 2e-5 and lse_err < 2e-5, (rank, err, lse_err)


def test_four_ranks_with_an_empty_shard_merge_to_the_whole():
    found = _run("ok", world=4)          # 300 positions in partitions of 128: the fourth rank owns nothing
    assert len(found) == 4 and all(err < 2e-5 and lse_err < 2e-5 for _, err, lse_err in found)


def test_a_stale_partial_blocks_publication_on_every_rank():
    assert _run("stale") == [(0, "refused"), (1, "refused")]


def test_a_rank_that_leaves_ends_the_collective_with_an_error():
    assert _run("leaves") == [(0, "refused"), (1, "left")]
