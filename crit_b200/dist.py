"""The hot path across the GPUs of one node: one process per GPU, torch.distributed (NCCL over NVLink) for the only
exchange the path has.

The reference has no distributed runtime; it states the technique on the host (interleaved ownership, partials merged
by their log-normalisers: inference/partitioned-attention/code/implementation.py:21-162, README "all-gather
normalizers, reduce-scatter weighted outputs") and tests it with two pools on one device
(inference/partitioned-attention/tests/test_device.py:44-68).  Here:

  - batches shard BY SEQUENCE (each rank owns whole sequences and their pages): no collective at all, outputs are
    disjoint rows.  assign_sequences() balances ranks by context length (longest first onto the lightest rank).
  - one long context shards BY KV RANGE: rank g owns a contiguous run of `partition`-position partitions, its pages are
    resident on its own GPU, every rank has the same queries.  Each rank runs the split-K decode over its own range
    and folds its splits locally into one (out, lse) per (token, head); ShardMerge exchanges those (tokens x heads x
    (dim + 1) floats a rank: 24.7 KB at 24 heads x 256) and folds them in rank order with the merge-of-shards kernel,
    identically on every rank.  A rank with no positions contributes zeros and -inf.  The exchange is the library's own
    by default, fused with the arithmetic either side of it: the launch that folds a rank's splits STORES each (token,
    head)'s result straight into every rank's buffer over NVLink peer memory (symmetric memory mapped once;
    crit_b200_merge_push), and the launch that waits for the ranks' flags (system-scope release / acquire, a bounded
    wait) merges the shards out of its own buffer (crit_b200_wait_merge): a decode step is decode, merge+push,
    wait+merge, three launches, because the payload is latency, not bandwidth.  NCCL's all-gather stays as the
    fallback (no symmetric memory) and as the baseline.

Failure detection without faulting a GPU: every rank's message carries (rank, epoch, rows) in its last three floats;
with check=True the gathered headers are read on the host and a stale, missing or foreign message raises before the
merged result is used (the reference's stated rule: a failed collective must block publication,
inference/partitioned-attention/README.md:100-102).  A rank that never joins ends the collective through the process
group's timeout.
"""
import math

HEADER = 3      # floats after a rank's payload: rank, epoch, rows


def assign_sequences(lengths, world, balance=True):
    """Sequence indices per rank.  balance: longest sequence first onto the rank with the least positions so far (LPT);
    else contiguous blocks of ceil(n / world)."""
    n = len(lengths)
    if not balance:
        per = -(-n // world)
        return [list(range(r * per, min(n, (r + 1) * per))) for r in range(world)]
    found, load = [[] for _ in range(world)], [0] * world
    for s in sorted(range(n), key=lambda i: (-lengths[i], i)):
        r = min(range(world), key=lambda i: (load[i], len(found[i]), i))
        found[r].append(s)
        load[r] += lengths[s]
    return [sorted(rows) for rows in found]


def kv_ranges(context, world, partition=4096):
    """[(first, end)] positions each rank owns of one context: contiguous runs of whole partitions, ceil(parts / world)
    a rank; ranks past the context get an empty range.  partition: the unit ownership is cut at.  A page (or a few) is
    the natural unit: every rank then gets work (49 partitions of 4,096 leave the eighth of 8 ranks with none, 3,125
    pages of 64 give each 388 to 391); the split-K partitions INSIDE a rank's range are the kernels' own matter."""
    parts = -(-context // partition)
    per = -(-parts // world)
    return [(min(min(r * per, parts) * partition, context), min(min((r + 1) * per, parts) * partition, context))
            for r in range(world)]


def chunk_to_fill(positions, kv_heads, blocks, chunk=1024, tile=16, waves=None):
    """Positions per split for ONE long row of `positions` so that its launch's blocks (splits x kv_heads) fill the
    device's `blocks` resident blocks in whole waves: as many waves as the default chunk comes nearest to (at least
    one), or `waves` when given (a shard of a context takes one: fewer splits to fold before its partial can leave).
    A row's own choice: it changes the split boundaries, so only a caller that always reads the row alone (one long
    context over a KV range) uses it."""
    positions, blocks = max(int(positions), 1), max(int(blocks), 1)
    units = -(-positions // chunk) * kv_heads
    waves = max(1, round(units / blocks)) if waves is None else max(1, int(waves))
    splits = max(1, waves * blocks // kv_heads)
    return max(tile, -(-(-(-positions // splits)) // tile) * tile)


class PeerExchange:
    """The two launches of the peer-memory exchange for one rank (crit_b200_shard_push / crit_b200_shard_wait): `peers`
    is an int64 device tensor of this GPU's addresses of every rank's exchange buffer (exchange_bytes() each, zeroed
    before the first step), `mine` this rank's FP32 message and `gathered` [world][floats] where the ranks' messages
    land.  status: an int32 device tensor the wait sets (0x800 + rank) when it ran out, or None."""

    def __init__(self, peers, rank, world, mine, gathered, wait_ms=2000, status=None):
        import ctypes
        import torch
        from . import _lib
        self._lib, self._ctypes, self._torch = _lib, ctypes, torch
        self.step = torch.zeros(1, dtype=torch.int32, device=mine.device)
        p = self.params = _lib.ExchangeParams()
        p.mine, p.peers, p.step, p.gathered = mine.data_ptr(), peers.data_ptr(), self.step.data_ptr(), gathered.data_ptr()
        p.status = status.data_ptr() if status is not None else None
        p.floats, p.wait_ns, p.world, p.rank = mine.numel(), int(wait_ms) * 1000000, world, rank
        self._keep = (peers, mine, gathered, status)

    @staticmethod
    def exchange_bytes(world, floats):
        from . import _lib
        return int(_lib.load().crit_b200_exchange_bytes(world, floats))

    def _launch(self, fn, what):
        stream = self._torch.cuda.current_stream().cuda_stream
        with self._torch.cuda.device(self._keep[1].device):
            self._lib.check(fn(self._ctypes.byref(self.params), stream), what)

    def push(self):
        self._launch(self._lib.load().crit_b200_shard_push, "crit_b200.dist.PeerExchange.push")

    def wait(self):
        self._launch(self._lib.load().crit_b200_shard_wait, "crit_b200.dist.PeerExchange.wait")


class ShardMerge:
    """Buffers (made once, so a captured step replays over them) and the exchange for rows of `tokens` x `heads`
    partials of width `dim`."""

    def __init__(self, tokens, heads, dim, device, group=None, merge=None, out_dtype=None, exchange="auto", wait_ms=2000):
        """exchange: "peer" (stores into the ranks' symmetric buffers; raises where symmetric memory cannot be set up),
        "nccl" (all_gather_into_tensor) or "auto" (peer where it can be set up, else nccl; the choice is agreed between
        the ranks).  wait_ms: the bound of the peer exchange's wait for the other ranks' messages."""
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.group = torch, dist, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.tokens, self.heads, self.dim = tokens, heads, dim
        self.rows = tokens * heads
        self.size = self.rows * (dim + 1) + HEADER
        self.mine = torch.zeros(self.size, dtype=torch.float32, device=device)
        self.all = torch.zeros(self.world, self.size, dtype=torch.float32, device=device)
        self.merge_fn, self.out_dtype = merge, out_dtype
        self.mine[-3], self.mine[-1] = float(self.rank), float(self.rows)
        self.peer, self.status = None, None
        if exchange not in ("auto", "peer", "nccl"):
            raise ValueError(f"exchange is auto, peer or nccl, not {exchange!r}")
        if self.world > 1 and exchange != "nccl" and torch.device(device).type == "cuda":
            self.peer = self._peer_setup(device, wait_ms, must=exchange == "peer")

    def _peer_setup(self, device, wait_ms, must):
        """Maps one exchange buffer per rank into every rank (a collective) and returns the launch parameters, or None
        when a rank could not (then every rank falls back together)."""
        torch, dist = self.torch, self.dist
        found, error = None, None
        try:
            import torch.distributed._symmetric_memory as symm
            import crit_b200
            words = PeerExchange.exchange_bytes(self.world, self.size) // 4
            group = self.group if self.group is not None else dist.group.WORLD
            buffer = symm.empty(words, dtype=torch.float32, device=device)
            buffer.zero_()
            handle = symm.rendezvous(buffer, group)
            peers = torch.tensor([int(a) for a in handle.buffer_ptrs], dtype=torch.int64, device=device)
            self.status = crit_b200._status_word(torch.device(device))
            found = PeerExchange(peers, self.rank, self.world, self.mine, self.all, wait_ms, self.status)
            found._symmetric = (buffer, handle)
        except Exception as problem:       # no symmetric memory here (driver, permissions, an older torch)
            error = problem
        # every rank takes the same road, and nobody pushes before every buffer is zeroed
        torch.cuda.synchronize()
        agreed = torch.tensor([1 if found is not None else 0], dtype=torch.int32, device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=self.group)
        if int(agreed.item()) == 0:
            if must:
                raise RuntimeError(f"the peer exchange could not be set up on every rank ({error})")
            return None
        return found

    def attend(self, params, out, lse, wait=True):
        """The fused step after a decode launch that left every split state in its workspace (crit_b200.attend with
        shards=self passes its parameter block here): fold + push, wait + merge of shards into out [tokens][heads][dim]
        and lse [tokens][heads].  Device work only, capturable.  wait=False: the fold + push alone (a measurement's).
        Without the peer exchange: the fold into out / lse and merge() over NCCL."""
        import ctypes
        torch = self.torch
        from . import _lib
        lib = _lib.load()
        stream = ctypes.c_void_p(torch.cuda.current_stream(out.device).cuda_stream)
        if self.peer is None:
            _lib.check(lib.crit_b200_merge(ctypes.byref(params), stream), "crit_b200.dist.ShardMerge.attend")
            merged, merged_lse = self.merge(out, lse)
            out.copy_(merged)
            lse.copy_(merged_lse)
            return out, lse
        if not out.is_contiguous() or not lse.is_contiguous() or out.numel() != self.rows * self.dim:
            raise ValueError(f"the merged output is contiguous [{self.tokens}][{self.heads}][{self.dim}]")
        m = _lib.MergeShardsParams()
        m.out, m.lse, m.n, m.parts, m.dim = out.data_ptr(), lse.data_ptr(), self.rows, self.world, self.dim
        m.in_dtype = _lib.DTYPE_FP32
        m.out_dtype = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_FP16, torch.float32: _lib.DTYPE_FP32}[out.dtype]
        x = self.peer.params
        with torch.cuda.device(out.device):
            if wait:
                _lib.check(lib.crit_b200_exchange_merge(ctypes.byref(params), ctypes.byref(x), ctypes.byref(m), stream),
                           "crit_b200.dist.ShardMerge.attend")
            else:
                _lib.check(lib.crit_b200_merge_push(ctypes.byref(params), ctypes.byref(x), stream), "crit_b200.dist.ShardMerge.attend (push)")
        return out, lse

    def raise_on_status(self):
        """Reads this device's status word (one wait) and raises when the exchange recorded a wait that ran out
        (0x800 + rank) or a message of another step or shape (0x900 + sender): the step's output is not published."""
        if self.status is None:
            return
        word = int(self.status.item())
        if word & 0xf00 in (0x800, 0x900):
            what = "waited in vain for the other ranks' partials" if word & 0xf00 == 0x800 else \
                f"got a partial of another step or shape from rank {word & 0xff}"
            raise RuntimeError(f"rank {self.rank}: the exchange {what} (status {word:#x}): the partial is missing or stale, "
                               "the merged attention is not published; zero the exchange buffers and synchronise the "
                               "ranks before the next step")

    def merge(self, out, lse, check=False, epoch=None):
        """This rank's (out [tokens][heads][dim], lse [tokens][heads]; lse -inf and out 0 where it saw no key) ->
        the merged (out, lse) over every rank, in rank order.  Device work only (it can be captured in a CUDA graph):
        the message's epoch is a counter kept on the device, one more every call.  epoch: set the counter instead (outside
        a capture); check: read the gathered headers on the host (one wait) and raise on a message that is missing,
        stale (another epoch than this rank's) or another shape's."""
        rows, dim = self.rows, self.dim
        self.mine[:rows * dim].copy_(out.reshape(-1))
        self.mine[rows * dim:rows * (dim + 1)].copy_(lse.reshape(-1))
        if epoch is None:
            self.mine[-2:-1].add_(1.0)
        else:
            self.mine[-2:-1].fill_(float(epoch))
        if self.peer is not None:
            self.peer.push()
            self.peer.wait()
        elif self.world > 1:
            self.dist.all_gather_into_tensor(self.all.view(-1), self.mine, group=self.group)
        else:
            self.all[0].copy_(self.mine)
        if check:
            self.verify()
        outs = self.all[:, :rows * dim].view(self.world, self.tokens, self.heads, dim)
        lses = self.all[:, rows * dim:rows * (dim + 1)].view(self.world, self.tokens, self.heads)
        if self.merge_fn is not None:
            return self.merge_fn(outs, lses)
        import crit_b200
        return crit_b200.merge_shards(outs, lses, dtype=self.out_dtype)

    def verify(self):
        """Raise unless every rank's message of this epoch and shape arrived (host read of world x 3 floats and of this
        rank's own message: the epoch every header must carry is the one this rank SENT, not the one it finds in the
        gathered copy, which a wait that ran out leaves at the step before)."""
        self.raise_on_status()
        headers = self.all[:, -HEADER:].cpu().tolist()
        want = float(self.mine[-2].item())
        for r, (rank, epoch, rows) in enumerate(headers):
            if rank != float(r) or epoch != want or rows != float(self.rows) or not all(map(math.isfinite, (rank, epoch, rows))):
                raise RuntimeError(f"rank {self.rank}: the partial of rank {r} is missing or stale (header rank {rank}, "
                                   f"epoch {epoch}, rows {rows}; expected rank {r}, epoch {want}, rows {self.rows}): "
                                   "the merged attention is not published")
