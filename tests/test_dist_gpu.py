"""Two GPUs, one process each: a context sharded by KV range, each rank's split-K decode over its own pages, the
(out, lse) partials exchanged (NCCL all-gather; and the library's own exchange, the fold of a rank's splits stored
straight into every rank's memory and the merge of shards read out of a rank's own) and merged, against the CPU oracle
over the whole context; the fused exchange gives the same bits step after step and from a CUDA graph.
Skipped with fewer than two GPUs."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rank(rank, world, port, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    import crit_b200 as pk
    import oracle
    from crit_b200.dist import ShardMerge, kv_ranges
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        hq, hkv, d, page, n = 24, 4, 128, 16, 5000
        g = torch.Generator().manual_seed(11)
        keys = torch.randn(n, hkv, d, generator=g).bfloat16()
        values = torch.randn(n, hkv, d, generator=g).bfloat16()
        q = torch.randn(1, hq, d, generator=g).bfloat16()
        lo, hi = kv_ranges(n, world, partition=1024)[rank]
        mine = hi - lo
        pages = -(-max(mine, 1) // page) + 1
        table = torch.randperm(pages, generator=torch.Generator().manual_seed(rank))[:pages - 1].to(torch.int32).to(dev)[None]
        k = torch.zeros(pages, page, hkv, d, dtype=torch.bfloat16, device=dev)
        v = torch.zeros_like(k)
        out = torch.zeros(1, hq, d, dtype=torch.bfloat16, device=dev)
        lse = torch.full((1, hq), float("-inf"), device=dev)
        if mine:
            slots = pk.slots_at(table, torch.zeros(mine, dtype=torch.int64, device=dev), torch.arange(mine, device=dev), page, pages - 1)
            pk.write(keys[lo:hi].to(dev), values[lo:hi].to(dev), slots, k, v, "bf16")
            i32 = dict(dtype=torch.int32, device=dev)
            pk.attend(q.to(dev), k, v, "bf16", table, torch.zeros(1, **i32), torch.zeros(1, **i32),
                      torch.tensor([mine - 1], device=dev), 1, page, out=out, lse=lse, chunk=256)
        merger = ShardMerge(1, hq, d, dev, exchange="nccl")
        merged, merged_lse = merger.merge(out, lse, check=True)
        # the peer-memory exchange, fused with the fold and the merge (decode, fold + push, wait + merge of shards): within
        # the bounds of the NCCL road (FP32 partials cross the wire here, the output's dtype there), the same bits step
        # after step (the slots alternate) and replayed from a graph
        peer = ShardMerge(1, hq, d, dev, exchange="auto", wait_ms=500)
        same = peer.peer is not None
        if same:
            i32 = dict(dtype=torch.int32, device=dev)
            fused, fused_lse = torch.zeros_like(out), torch.zeros_like(lse)
            count, zero = torch.tensor([1 if mine else 0], **i32), torch.zeros(1, **i32)
            last, q_dev = torch.tensor([max(mine - 1, 0)], device=dev), q.to(dev)

            def fused_step():
                return pk.attend(q_dev, k, v, "bf16", table, zero, zero, last, 1, page, counts=count, out=fused,
                                 lse=fused_lse, chunk=256, shards=peer)
            fused_step()
            first, first_lse = fused.clone(), fused_lse.clone()
            same = same and bool((first.float() - merged.float()).abs().max() <= 2e-2)
            same = same and bool((first_lse - merged_lse).abs().max() <= 2e-3)
            for _ in range(3):
                fused.zero_()
                fused_step()
                same = same and torch.equal(fused, first) and torch.equal(fused_lse, first_lse)
            stream = torch.cuda.Stream(dev)
            with torch.cuda.stream(stream):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    fused_step()
                for _ in range(3):
                    fused.zero_()
                    graph.replay()
                stream.synchronize()
            peer.raise_on_status()
            same = same and torch.equal(fused, first) and torch.equal(fused_lse, first_lse) and pk.status(dev) == 0
            merged, merged_lse = fused, fused_lse
        whole_table = np.arange(-(-n // page), dtype=np.int32)
        kf = np.zeros((len(whole_table) * page, hkv, d), np.float32)
        vf = np.zeros_like(kf)
        kf[:n], vf[:n] = keys.float().numpy(), values.float().numpy()
        want, want_lse = oracle.attend(q.float().numpy(), kf, vf, whole_table, [0], [0], [n - 1], 1, page)
        err = np.abs(merged.float().cpu().numpy() - want)
        queue.put((rank, float(err.max()), float(err.mean()), float(np.abs(merged_lse.cpu().numpy() - want_lse).max()),
                   "peer exchange not set up" if peer.peer is None else bool(same)))
    finally:
        dist.destroy_process_group()


def test_kv_range_shards_over_two_gpus_merge_to_the_whole():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    found = [queue.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(60)
    for rank, max_abs, mean_abs, lse_abs, peer in found:
        assert max_abs <= 2e-2 and mean_abs <= 2e-3 and lse_abs <= 2e-3, (rank, max_abs, mean_abs, lse_abs)
        assert peer is True, (rank, peer)
