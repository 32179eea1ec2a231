"""The attention slot's device form over a paged KV pool, with the interface of crit's DeviceAttention and
PartitionedAttention (reference: inference/attention-state/code/device_attention.py:187-441, :659-716, :1082-1105;
inference/partitioned-attention/plugin.py:15-64).

forward() classifies a step's rows as the reference does (a row of up to pool.window tokens is a window row: decode
tokens, verify windows; a longer one a prompt row) and launches crit_b200's kernels: window rows through the split-K
decode/verify kernel and its merge, prompt rows through the prefill kernel where it serves the pool, else as pieces of
up to 64 columns through the decode kernel (the reference's prompt_reader "decode": one reduction for every row).
There is no torch fallback.

With crit_b200's own pool the rows' page tables are never rebuilt: the launch reads the pool's block table in place
and the step's metadata is one small upload of five numbers a row.  Any pool with the reference's attributes
(table(), layer_pages(), dump, page, window) is served too, through padded tables built per step as the reference
builds them.
"""
import math
from dataclasses import dataclass

from . import host_form

TABLE_WIDTH = 16      # a generic pool's per-step tables are this many pages wide or a multiple (reference :1079)
PIECE_COLUMNS = 64    # columns of a prompt row's piece when it is read by the decode kernel


@dataclass
class Windows:
    """The window rows of one launch, on the device.  Row r reads the page table tables[rows[r]]; its tokens are
    starts[r] .. starts[r] + counts[r] - 1 of the step's queries (counts None: `columns` each) and its column 0 sits at
    position firsts[r].  offsets[r] (optional) is its first partial row when the rows' partials are packed by their
    tokens; packed[r] is then the host's copy of its token count and total the tokens of all rows."""
    tables: object
    rows: object
    starts: object
    counts: object
    firsts: object
    columns: int
    offsets: object = None
    packed: object = None
    total: object = None

    def __len__(self):
        return int(self.starts.shape[0])


class DeviceAttention:
    def __init__(self, kernels=None, mode="auto", int8_qk=False, decode="split", partitions=0, piece=0, device=None,
                 kernels_mib=128, flashinfer="off", flashinfer_mib=128, prompt_reader="prefill", reader="split",
                 latent=None, scratch=None, chunk=0, window_engine="auto"):
        """kernels: the crit_b200 module (default).  partitions: the most splits of a partial row (0: what the tables
        need); chunk: positions per split (0: the kernels' rule).  kernels_mib: the most partials a launch takes from
        `scratch` (the engine's Scratch, crit_plugins.memory) when one is given.  prompt_reader: "prefill" or "decode".
        window_engine: "auto" (the kernels' choice, crit_b200.engine_for: E4M3 pages through tcgen05.mma where a kernel for
        it serves the step, m16n8k16 tiles otherwise; a column's bits then depend on the window and the step it is read
        in: exactness "repeatable"), "mma.sync" (the m16n8k16 kernel always: a column's bits are the same alone and in
        any window or batch, "row-exact"), "tcgen05" (one kv head a unit, wherever that kernel serves a launch) or
        "tcgen05p" (whole page rows a unit, where that kernel serves the step).
        mode "torch", decode "flashinfer", flashinfer "auto", int8_qk and latent are the reference's other readers: not
        served here."""
        if mode == "torch" or decode != "split" or flashinfer != "off" or int8_qk or latent is not None:
            raise ValueError("crit_b200 serves its own CUDA kernels only (mode auto, decode split, flashinfer off)")
        if window_engine not in ("auto", "mma.sync", "tcgen05", "tcgen05p"):
            raise ValueError(f"window_engine is auto, mma.sync, tcgen05 or tcgen05p, not {window_engine!r}")
        self.window_engine = window_engine
        if prompt_reader not in ("prefill", "decode"):
            raise ValueError(f"prompt_reader is prefill or decode, not {prompt_reader!r}")
        if kernels is None:
            import crit_b200 as kernels
        self.kernels = kernels
        self.mode, self.prompt_reader, self.reader = mode, prompt_reader, reader
        self.partitions, self.chunk, self.device = int(partitions), int(chunk), device
        self.partial_bytes = (int(kernels_mib) << 20) if scratch is not None else 0
        self.scratch = scratch
        self._steps = {}
        self._prompt_rows = {}

    # -- facts -----------------------------------------------------------------------------------------------------------
    def facts(self):
        return {"reader": "crit_b200: a row's positions in contiguous splits of one chunk per pool, folded in split order; " +
                          ("a column's bits are the same alone and in any window" if self.window_engine == "mma.sync" else
                           "E4M3 pages through tcgen05.mma where served: a column's bits depend on its window and its step"),
                "prompt_reads": "through the prefill kernel" if self.prompt_reader == "prefill" else
                                "in the decode's reduction (pieces of up to 64 columns)",
                "split_kv_wide_windows": "16- or 32-row tiles; wider windows read their pages once per tile"}

    def exactness(self):
        return {"decode": "row-exact" if self.window_engine == "mma.sync" else "repeatable",
                "prompt": "exact" if self.prompt_reader == "decode" else "repeatable"}

    def close(self):
        self._steps.clear()
        self._prompt_rows.clear()

    # -- the device form -------------------------------------------------------------------------------------------------
    def forward(self, layer, queries, pool, batch, scale=None, blocks=None, block_size=None, parents=None, lse=False,
                sinks=None, sliding=0, latent=0):
        """queries [tokens][heads][dim] of a StepBatch, RoundBatch or PromptBatch over the pool's KV (written for this
        step already); each token sees its sequence's positions up to its own.  lse: also return each token's
        log-sum-exp ([tokens][heads] FP32).  Returns out [tokens][heads][value dim] in the queries' dtype (and lse)."""
        import torch
        if latent:
            raise NotImplementedError("crit_b200's attention does not serve latent attention yet")
        if blocks is not None and (not block_size or blocks.dim() != 2 or blocks.shape[0] != queries.shape[0]):
            raise ValueError("blocks are [tokens][k] KV block ids with block_size positions each")
        if sinks is not None:
            sinks = sinks.reshape(-1).float().contiguous()
            if sinks.numel() != queries.shape[1] or not sinks.is_cuda:
                raise ValueError("sinks are one logit a query head, on the queries' device")
        # (the call's sinks and sliding window, for the launches below: reference device_attention.py:188-189, :382-386)
        self._sinks, self._sliding = sinks, int(sliding or 0)
        self._blocks = (blocks, int(block_size)) if blocks is not None else None
        if parents is not None and getattr(batch, "prompt", False):
            raise NotImplementedError("draft trees (parents) are read in window rows, not in a staged prompt chunk")
        if not queries.is_cuda:
            raise RuntimeError("crit_b200's attention runs on CUDA devices only (there is no CPU path)")
        scale = scale if scale is not None else queries.shape[-1] ** -0.5
        q = queries if queries.dtype == pool.compute and queries.stride(-1) == 1 else queries.to(pool.compute).contiguous()
        tokens, heads = q.shape[0], q.shape[1]
        out = q.new_empty(tokens, heads, pool.value_dim)
        found = q.new_empty(tokens, heads, dtype=torch.float32) if lse else None
        if getattr(batch, "prompt", False):
            self._prompt(layer, q, pool, batch, scale, out, found)
        elif getattr(batch, "round", False):
            rows, cols = batch.rows, batch.width + 1
            meta = Windows(pool.round_tables, batch.slots_t[:rows].to(torch.int32), batch.starts_t[:rows], None,
                           batch.frontier_t, cols)
            self._windows(layer, q, pool, meta, scale, out, found, parents)
        elif getattr(pool, "step_rows", 0):
            n = len(pool.windows)
            if n:
                bounds = [batch.row(r)[2] for r in pool.windows]
                meta = Windows(pool.d_tables, pool.d_rows[:n], pool.d_starts[:n], pool.d_counts[:n], pool.d_firsts[:n],
                               pool.window, offsets=pool.d_offsets[:n], packed=bounds, total=q.shape[0])
                self._windows(layer, q, pool, meta, scale, out, found, parents)
            chosen = set(pool.windows)
            self._prompts(layer, q, pool, batch, [r for r in range(batch.rows) if r not in chosen], scale, out, found, parents)
        else:
            short = [r for r in range(batch.rows) if batch.row(r)[2] <= pool.window]
            if short:
                self._windows(layer, q, pool, self._step_windows(pool, batch, short, q.device), scale, out, found, parents)
            self._prompts(layer, q, pool, batch, [r for r in range(batch.rows) if batch.row(r)[2] > pool.window],
                          scale, out, found, parents)
        self._sinks, self._sliding, self._blocks = None, 0, None
        out = out if out.dtype == queries.dtype else out.to(queries.dtype)
        return (out, found) if lse else out

    def merge(self, outs, lses):
        """Partials of the same queries over disjoint keys -> (out, lse), the parts weighted by exp(lse - max) in part
        order; a token no part saw gets zeros and -inf.  Reference: partitioned-attention/plugin.py:52-64."""
        return self.kernels.merge_shards(outs, lses)

    # -- window rows -----------------------------------------------------------------------------------------------------
    def _step_windows(self, pool, batch, chosen, device):
        key = (id(pool), pool.steps, tuple(chosen))
        cached = self._steps.get("windows")
        if cached is not None and cached[0] == key:
            return cached[1]
        found = windows_of(pool, [batch.row(r) for r in chosen], device)
        self._steps["windows"] = (key, found)
        return found

    def _windows(self, layer, q, pool, meta, scale, out, found, parents=None):
        pages = pool.layer_pages(layer)
        scaled = len(pages) == 4
        multipliers = pool.scale_values[pool.layers[layer]] if pool.dtype == "fp8" else (1.0, 1.0)
        kernels = self.kernels
        positions = meta.tables.shape[1] * pool.page
        geometry = (pool.dtype, pool.head_dim, pool.value_dim, q.shape[1], pool.kv_heads, meta.columns)
        # the kernel the step's windows run on: the kernels' choice for the whole step, or the one the option names
        named = kernels.engine_for(*geometry, len(meta), positions, None if self.window_engine == "auto" else self.window_engine)
        sinks, sliding = getattr(self, "_sinks", None), getattr(self, "_sliding", 0)
        listed = getattr(self, "_blocks", None)
        sparse = listed is not None and listed[1] % pool.page == 0           # the lists as page tables of their own: any kernel
        if parents is not None or sinks is not None or sliding or (listed is not None and not sparse):
            named = "mma.sync"             # draft trees, sinks, sliding windows and lists as masks are the m16n8k16 kernel's
        chunk = self.chunk or kernels.chunk_for(pool.head_dim, pool.value_dim, q.shape[1], pool.kv_heads, pool.page, pool.dtype,
                                                named, meta.columns)
        if self.partitions:
            chunk = max(chunk, -(-positions // self.partitions))
        chunk = -(-chunk // 16) * 16
        if named == "tcgen05p" and not kernels.tcgen05p_serves(*geometry, chunk, len(meta)):
            named = "mma.sync"
        parts = kernels.states_for(kernels.parts_for(positions, chunk), named)
        launches, workspace = [(slice(0, len(meta)), meta.total)], None
        if self.partial_bytes and (parts > 1 or sinks is not None):
            # the partials come from the engine's scratch: as many rows a launch as its share of the scratch holds
            per = kernels.workspace_floats(1, q.shape[1], parts, pool.value_dim)
            launches = launch_cuts(meta, self.partial_bytes // 4 // per)
            most = max((cut.stop - cut.start) * meta.columns if tokens is None else tokens for cut, tokens in launches)
            import torch
            workspace = self.scratch.take(min(self.partial_bytes, 4 * per * most)).view(torch.float32)

        def engine(rows):
            if named == "tcgen05":
                return "tcgen05" if kernels.tcgen05_serves(*geometry, chunk, rows) else "mma.sync"
            return named

        for cut, tokens in launches:
            part = (lambda t: t[cut]) if not cut.start else (lambda t: t[cut].clone())
            offsets = part(meta.offsets) if meta.offsets is not None and tokens is not None else None
            kernels.attend(q, pages[0], pages[1], pool.dtype, meta.tables, part(meta.rows), part(meta.starts),
                           part(meta.firsts), meta.columns, pool.page,
                           counts=part(meta.counts) if meta.counts is not None else None, offsets=offsets,
                           tokens=tokens if offsets is not None else None,
                           key_scales=pages[2] if scaled else None, value_scales=pages[3] if scaled else None,
                           multipliers=multipliers, scale=scale, chunk=chunk, out=out, lse=found, workspace=workspace,
                           engine=engine(cut.stop - cut.start), parents=parents, sinks=sinks, sliding=sliding,
                           blocks=listed[0] if listed else None, block_size=listed[1] if listed else None)

    # -- prompt rows -----------------------------------------------------------------------------------------------------
    def _prompts(self, layer, q, pool, batch, rows, scale, out, found, parents=None):
        if not rows:
            return
        if parents is not None:
            raise NotImplementedError("draft trees (parents) are read in window rows: a row of more than the pool's "
                                      f"window of {pool.window} columns is a prompt row")
        special = (getattr(self, "_sinks", None) is not None or getattr(self, "_sliding", 0) or
                   getattr(self, "_blocks", None) is not None)                                  # the decode kernel's rules
        fresh = None
        if not special and callable(getattr(pool, "fresh_rows", None)):
            fresh = pool.fresh_rows(layer, q.shape[0])
        if fresh is not None and self._fresh_serves(pool, q):
            return self._fresh_prompts(layer, q, pool, batch, rows, scale, out, found, fresh)
        if self.prompt_reader == "prefill" and self._prefill_serves(pool, q) and not special:
            pages = pool.layer_pages(layer)
            scaled = len(pages) == 4
            multipliers = pool.scale_values[pool.layers[layer]] if pool.dtype == "fp8" else (1.0, 1.0)
            spans = [batch.row(r) for r in rows]
            joined = all(a[1] + a[2] == b[1] for a, b in zip(spans, spans[1:]))
            if len(spans) > 1 and joined and hasattr(pool, "block_tables") and hasattr(pool, "row_of") and \
                    hasattr(self.kernels, "engine_for"):          # (crit_b200's own kernels and pool)
                # the rows' chunks follow one another in q: one launch over all of them, a table row and a position each
                import torch
                pool._flush()
                ids = torch.tensor([pool.row_of[sequence] for sequence, _, _, _ in spans], device=q.device)
                span = slice(spans[0][1], spans[-1][1] + spans[-1][2])
                starts = [first - spans[0][1] for _, first, _, _ in spans] + [span.stop - span.start]
                self.kernels.prefill(q[span], pages[0], pages[1], pool.dtype, pool.block_tables[ids],
                                     [position for _, _, _, position in spans], pool.page,
                                     key_scales=pages[2] if scaled else None, value_scales=pages[3] if scaled else None,
                                     multipliers=multipliers, scale=scale, out=out[span],
                                     lse=found[span] if found is not None else None, starts=starts)
                return
            for r in rows:
                sequence, first, count, position = batch.row(r)
                span = slice(first, first + count)
                self.kernels.prefill(q[span], pages[0], pages[1], pool.dtype, pool.device_tables.get(sequence), position,
                                     pool.page, key_scales=pages[2] if scaled else None,
                                     value_scales=pages[3] if scaled else None, multipliers=multipliers, scale=scale,
                                     out=out[span], lse=found[span] if found is not None else None)
            return
        pieces = []
        for r in rows:
            sequence, first, count, position = batch.row(r)
            for at in range(0, count, PIECE_COLUMNS):
                pieces.append((sequence, first + at, min(PIECE_COLUMNS, count - at), position + at))
        self._windows(layer, q, pool, windows_of(pool, pieces, q.device), scale, out, found)

    def _fresh_serves(self, pool, q):
        serves = getattr(self.kernels, "prefill_serves", None)
        kind = "fp16" if q.dtype == getattr(__import__("torch"), "float16") else "bf16"
        return bool(serves and serves(pool.head_dim, pool.value_dim, q.dtype, kind, 16))

    def _fresh_prompts(self, layer, q, pool, batch, rows, scale, out, found, fresh):
        """Prompt rows of a pool that kept the step's keys and values as it got them (quantised pages, a fresh buffer): a
        token attends its own chunk from those and the earlier positions from the pages, so it is scored with what it
        was given (reference: device_attention.py:1136-1145, pages.py:300-308).  Three launches a row: the pages'
        part as context rows (pieces of up to 64 columns that all see the positions before the chunk), the chunk's
        part as a causal prefill over 16-bit pages made of the fresh rows, and the merge of the two by their lse."""
        import torch
        kernels = self.kernels
        kind = "fp16" if q.dtype == torch.float16 else "bf16"
        pages_ = pool.layer_pages(layer)
        scaled = len(pages_) == 4
        multipliers = pool.scale_values[pool.layers[layer]] if pool.dtype == "fp8" else (1.0, 1.0)
        hkv, d, dv = pool.kv_heads, pool.head_dim, pool.value_dim
        for r in rows:
            sequence, first, count, position = batch.row(r)
            span = slice(first, first + count)
            heads = q.shape[1]
            parts_o = q.new_zeros(2, count, heads, dv, dtype=torch.float32)
            parts_l = q.new_full((2, count, heads), float("-inf"), dtype=torch.float32)
            # the chunk's own part: the fresh rows as 16-bit pages of 16 positions, read causally from position 0
            n_pages = -(-count // 16)
            tk = q.new_zeros(n_pages * 16, hkv, d)
            tv = q.new_zeros(n_pages * 16, hkv, dv)
            tk[:count].copy_(fresh[0][span])
            tv[:count].copy_(fresh[1][span])
            own = q.new_empty(count, heads, dv)
            kernels.prefill(q[span], tk.view(n_pages, 16, hkv, d), tv.view(n_pages, 16, hkv, dv), kind,
                            torch.arange(n_pages, dtype=torch.int32, device=q.device), 0, 16, scale=scale, out=own,
                            lse=parts_l[1])
            parts_o[1].copy_(own)
            # the pages' part: every column of a piece sees the positions before the chunk
            if position > 0:
                pieces = [(sequence, at, min(PIECE_COLUMNS, count - at), position) for at in range(0, count, PIECE_COLUMNS)]
                meta = windows_of(pool, pieces, q.device)
                before = q.new_empty(count, heads, dv)
                kernels.attend(q[span], pages_[0], pages_[1], pool.dtype, meta.tables, meta.rows, meta.starts, meta.firsts,
                               meta.columns, pool.page, counts=meta.counts, key_scales=pages_[2] if scaled else None,
                               value_scales=pages_[3] if scaled else None, multipliers=multipliers, scale=scale,
                               out=before, lse=parts_l[0], context=True)
                parts_o[0].copy_(before)
            merged, lse = kernels.merge_shards(parts_o, parts_l, dtype=q.dtype)
            out[span].copy_(merged)
            if found is not None:
                found[span].copy_(lse)

    def _prefill_serves(self, pool, q):
        serves = getattr(self.kernels, "prefill_serves", None)
        return bool(serves and serves(pool.head_dim, pool.value_dim, q.dtype, pool.dtype, pool.page))

    def _prompt(self, layer, q, pool, batch, scale, out, found):
        """A PromptBatch: the bucket's tokens over the pool's prompt table, causal from batch.frontier_t, read on the
        device: window rows of up to 64 columns (reference: device_attention.py:577-641)."""
        import torch
        key = (batch.bucket, str(q.device))
        made = self._prompt_rows.get(key)
        if made is None:
            columns = min(PIECE_COLUMNS, batch.bucket)
            count = -(-batch.bucket // columns)
            starts = torch.arange(count, dtype=torch.int32, device=q.device) * columns
            counts = torch.tensor([min(columns, batch.bucket - r * columns) for r in range(count)], dtype=torch.int32,
                                  device=q.device)
            made = self._prompt_rows[key] = (torch.zeros(count, dtype=torch.int32, device=q.device), starts, counts,
                                             starts.long(), columns)
        rows, starts, counts, offsets, columns = made
        meta = Windows(pool.prompt_table, rows, starts, counts, batch.frontier_t + offsets, columns)
        self._windows(layer, q, pool, meta, scale, out, found)


def launch_cuts(meta, capacity):
    """Consecutive runs of window rows whose partial rows fit a workspace of `capacity` partial rows:
    [(slice of rows, partial rows of the run or None)].  Rows without packed partials take `columns` partial rows each
    (None: the launch counts them itself); packed rows take their own token counts, found by one cumulative sum and a
    search per run.  A row that alone passes the capacity is refused."""
    import numpy as np
    n = len(meta)
    if meta.offsets is None or meta.packed is None:
        step = capacity // meta.columns
        if step < 1:
            raise _too_small(meta.columns)
        return [(slice(a, min(n, a + step)), None) for a in range(0, n, step)]
    upto = np.cumsum(np.asarray(meta.packed, dtype=np.int64))
    cuts, first, before = [], 0, 0
    while first < n:
        end = int(np.searchsorted(upto, before + capacity, side="right"))
        if end <= first:
            raise _too_small(int(meta.packed[first]))
        cuts.append((slice(first, end), int(upto[end - 1] - before)))
        first, before = end, int(upto[end - 1])
    return cuts


def _too_small(tokens):
    return ValueError(f"a row of {tokens} tokens needs more partials than the split-KV reader's workspace holds: raise "
                      "the attention plugin's workspace_mib")


def windows_of(pool, rows, device):
    """Windows of host rows (sequence, first token, count, first position): their metadata in one copy to the device,
    their partials packed by their tokens.  crit_b200's pool: the launch reads its block table in place; another pool:
    padded tables built from pool.table() as the reference builds them (device_attention.py:1082-1105)."""
    import torch
    counts = [count for _, _, count, _ in rows]
    offsets = [sum(counts[:i]) for i in range(len(rows))]
    own = hasattr(pool, "block_tables")
    if own:
        pool._flush()
        tables, ids = pool.block_tables, [pool.row_of[sequence] for sequence, _, _, _ in rows]
    else:
        lists = [pool.table(sequence)[:math.ceil((position + count) / pool.page)] for sequence, _, count, position in rows]
        width = -(-max(len(t) for t in lists) // TABLE_WIDTH) * TABLE_WIDTH
        grid = torch.full((len(rows), width), pool.dump, dtype=torch.int32)
        for i, t in enumerate(lists):
            grid[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
        tables, ids = grid.to(device), list(range(len(rows)))
    meta = torch.tensor([[first, count, position, offset, row] for (_, first, count, position), offset, row
                         in zip(rows, offsets, ids)], dtype=torch.int64)
    meta = (meta.pin_memory() if torch.device(device).type == "cuda" else meta).to(device, non_blocking=True)
    return Windows(tables, meta[:, 4].to(torch.int32), meta[:, 0].to(torch.int32), meta[:, 1].to(torch.int32),
                   meta[:, 2].contiguous(), max(counts), offsets=meta[:, 3].to(torch.int32), packed=counts,
                   total=sum(counts))


class PartitionedAttention:
    """The attention slot's plugin object: the host form (every query's softmax taken shard by shard over interleaved
    ownership and merged by the shards' log-sum-exps: host_form) and the device form above.  The plugin it stands in
    for: inference/partitioned-attention/plugin.py:15-64."""

    def __init__(self, kv, options, device_form):
        self.kv, self.device_form, self.world = kv, device_form, int(options["world"])

    def attend(self, sequence, queries, positions, scale=None, pending=False):
        """Each query over the sequence's rows at positions up to its own -> [output row] (lists of floats)."""
        keys, values = self.kv.arrays(sequence, pending) if hasattr(self.kv, "arrays") else _matrices(self.kv.rows(sequence, pending))
        if not len(keys):
            raise ValueError("no rows to attend")
        if len(queries) != len(positions):
            raise ValueError("one position per query")
        return [host_form.attend(query, keys, values, position, self.world, scale).tolist()
                for query, position in zip(queries, positions)]

    def forward(self, layer, queries, pool, batch, scale=None, blocks=None, block_size=None, parents=None, lse=False):
        return self.device_form.forward(layer, queries, pool, batch, scale, blocks, block_size, parents, lse)

    def merge(self, outs, lses):
        return self.device_form.merge(outs, lses)

    def facts(self):
        return self.device_form.facts()

    def exactness(self):
        return self.device_form.exactness()

    def close(self):
        self.device_form.close()


def _matrices(rows):
    """[(position, key, value)] in position order -> (keys, values) matrices (another plugin's kv_cache host form)."""
    import numpy as np
    if not rows:
        return np.empty((0, 0)), np.empty((0, 0))
    return np.array([key for _, key, _ in rows], dtype=np.float64), np.array([value for _, _, value in rows], dtype=np.float64)
