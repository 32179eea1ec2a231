"""Paged KV of many sequences on a B200: the kv_cache slot's device form, with the interface of crit's KVPool
(reference: inference/attention-state/code/pages.py:74-869; the KV_POOL contract of
core/python/crit_plugins/device.py:207-220).

What stays as in the reference, because callers and tests observe it: one uint8 allocation holding every layer's keys
and values as [layers][pages + 1][page][kv_heads][dim] (the dump page last), pages taken lowest-free-first, forks
sharing pages until one writes (copy on write), keep() rolling a sequence back and freeing its pages, the error
messages, and slot = table[p // page] * page + p % page.

What is built for the GPU instead of translated:
  - every open sequence owns one row of ONE device-resident block table ([sequences][table_pages] int32, unused
    entries at the dump page).  reserve() uploads only the entries that changed (a grown or copied page) and computes
    the step's slots with a kernel from that table; the attention reads the same table rows in place, so no step
    rebuilds or re-uploads padded page tables, and host work is O(rows + new pages), not O(tokens).
  - writes, gathers and row reads go through the CUDA kernels of crit_b200 (there is no torch fallback: a pool on the
    CPU keeps page tables and slot maps only, for host-side tests).
  - "fp8:page": E4M3 pages with one FP32 scale per (page, kv head), scales [layers][pages + 1][kv_heads].

Not served (the reference's other pool features): sliding rings, lending and elastic backing.
"""
import ctypes
import heapq
import math

DTYPES = ("bf16", "fp16", "fp8", "fp8:row", "int8", "fp8:page")
ROW_SCALED = ("fp8:row", "int8")
SCALED = ROW_SCALED + ("fp8:page",)
KERNEL_KINDS = DTYPES
QUANTIZED = ("fp8", "fp8:row", "int8", "fp8:page")


class _Tables:
    """pool.device_tables: sequence -> its page ids on the device (a view of its block-table row)."""

    def __init__(self, pool):
        self.pool = pool

    def get(self, sequence, default=None):
        pool = self.pool
        if sequence not in pool.tables:
            return default
        return pool.block_tables[pool.row_of[sequence], :max(len(pool.tables[sequence]), 1)]

    def __getitem__(self, sequence):
        found = self.get(sequence)
        if found is None:
            raise KeyError(sequence)
        return found

    def pop(self, sequence, default=None):
        return default


class Pager:
    """The pool's page allocator, native (csrc/pager.cu behind the C ABI's crit_b200_pager_*): a min-heap of the free
    page ids (the lowest free page is the next one taken), a reference count per page, the floor (one past the highest
    page in use).  Host code: it needs the library, not a GPU."""

    def __init__(self, pages):
        from . import _lib
        self._lib = _lib.load()
        self._handle = ctypes.c_void_p(self._lib.crit_b200_pager_create(int(pages)))
        if not self._handle:
            raise MemoryError(f"no page allocator for {pages} pages")

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            self._lib.crit_b200_pager_destroy(handle)

    def take(self):
        return self._lib.crit_b200_pager_take(self._handle)

    def drop(self, page):
        return self._lib.crit_b200_pager_drop(self._handle, int(page))

    def share(self, page):
        return self._lib.crit_b200_pager_share(self._handle, int(page))

    def refs(self, page):
        return self._lib.crit_b200_pager_refs(self._handle, int(page))

    def free(self):
        return self._lib.crit_b200_pager_free(self._handle)

    def floor(self):
        return self._lib.crit_b200_pager_floor(self._handle)

    def shared(self):
        return self._lib.crit_b200_pager_shared(self._handle)

    def grow(self, have, need):
        """Pages for a step's rows at once (row i from have[i] to need[i] pages, in row order, lowest free page first):
        (the pages, whether the pool ran out before the last one)."""
        rows = len(have)
        most = sum(max(0, n - h) for h, n in zip(have, need))
        out = (ctypes.c_int32 * max(most, 1))()
        a, b = (ctypes.c_int32 * max(rows, 1))(*have), (ctypes.c_int32 * max(rows, 1))(*need)
        taken = self._lib.crit_b200_pager_grow(self._handle, rows, a, b, out, most)
        if taken < 0:
            return list(out[:-taken - 1]), True
        return list(out[:taken]), False


class FreshBuffer:
    """A prompt chunk's keys and values as the projections gave them, one buffer for a plugin's pools: `data` the uint8
    device buffer, `tag` (pool, layer, tokens, reserve) of the write that holds it now, so a pool reads it only while
    its own write of that layer and step is the last one.  Reference: pages.py:65-71."""

    def __init__(self, data):
        self.data, self.tag = data, None


class KVPool:
    """window: the most tokens of a row read as a window row; a longer row is a prompt row.  step_rows > 0 keeps a
    step's slots and window-row metadata at fixed device addresses (a model captures its decode step in a CUDA graph
    over them).  round_rows: the round slots bind() may use.  sequences: block-table rows made at first (it grows)."""

    def __init__(self, layers, kv_heads, head_dim, tokens, device, dtype="bf16", *, page=16, value_dim=None,
                 step_rows=0, step_tokens=0, window=16, round_rows=8, kernels=None, sequences=64, positions=None,
                 spare=0, fresh=None, sliding=0, span=None, elastic=False, host_bytes=0):
        import torch
        if dtype not in DTYPES:
            raise ValueError(f"a KV pool stores {', '.join(DTYPES)}, not {dtype!r}")
        if kv_heads < 1 or head_dim < 1 or tokens < 1 or page < 1 or window < 1:
            raise ValueError("a KV pool has heads, a head dimension, tokens, a page size and a window of a token or more")
        if spare or sliding or elastic or host_bytes:
            raise ValueError("crit_b200's KV pool does not serve spare bytes, sliding rings or elastic pages")
        self.torch = torch
        self.layers = {layer: i for i, layer in enumerate(layers)}
        self.kv_heads, self.head_dim = kv_heads, head_dim
        self.value_dim = head_dim if value_dim is None else int(value_dim)
        self.page, self.device, self.dtype = page, torch.device(device), dtype
        self.storage = {"bf16": torch.bfloat16, "fp16": torch.float16, "int8": torch.int8}.get(dtype, torch.float8_e4m3fn)
        self.compute = torch.float16 if dtype == "fp16" else torch.bfloat16
        self.pages = math.ceil(tokens / page)
        self.sliding, self.ring = 0, 0
        self.table_pages = max(math.ceil(int(positions) / page) if positions else self.pages, self.pages)
        n, stored = len(self.layers), self.pages + 1
        self.dump, self.stored_slots = self.pages, stored * page
        shapes = [((n, stored, page, kv_heads, head_dim), self.storage),
                  ((n, stored, page, kv_heads, self.value_dim), self.storage)]
        if dtype in ROW_SCALED:
            shapes += [((n, stored, page, kv_heads), torch.float32)] * 2
        elif dtype == "fp8:page":
            shapes += [((n, stored, kv_heads), torch.float32)] * 2
        offsets, sizes, end = [], [], 0
        for shape, kind in shapes:
            offsets.append(end)
            sizes.append(math.prod(shape) * torch.empty(0, dtype=kind).element_size())
            end = -(-(end + sizes[-1]) // 256) * 256
        self.memory = torch.zeros(end, dtype=torch.uint8, device=self.device)
        tensors = [self.memory[first:first + size].view(kind).view(shape)
                   for first, size, (shape, kind) in zip(offsets, sizes, shapes)]
        self.k, self.v = tensors[0], tensors[1]
        self.k_scales, self.v_scales = (tensors[2], tensors[3]) if dtype in SCALED else (None, None)
        self.scales = torch.ones(n, 2, dtype=torch.float32, device=self.device)
        self.scale_values = [(1.0, 1.0)] * n
        self.steps = 0
        # A prompt chunk's keys and values as write() got them (pools of quantised pages given a fresh buffer: an object
        # with .data, a uint8 tensor on the pool's device, and .tag): the attention reads the chunk's own positions from
        # them and the earlier ones from the pages, so what a prompt token is scored with is what it was given.
        # Reference: pages.py:180-196.
        self.fresh_k = self.fresh_v = None
        self.fresh_tokens, self._staging, self._reserves, self._fresh_buffer = 0, False, 0, None
        if fresh is not None and dtype in QUANTIZED and self.value_dim and fresh.data.device.type == self.device.type:
            size = torch.empty(0, dtype=self.compute).element_size()
            self.fresh_tokens = fresh.data.numel() // (kv_heads * (head_dim + self.value_dim) * size)
        if self.fresh_tokens:
            cap = self.fresh_tokens
            keys = cap * kv_heads * head_dim * size
            self._fresh_buffer = fresh
            self.fresh_k = fresh.data[:keys].view(self.compute).view(cap, kv_heads, head_dim)
            self.fresh_v = fresh.data[keys:keys + cap * kv_heads * self.value_dim * size].view(self.compute).view(
                cap, kv_heads, self.value_dim)
        # pages: a heap of the free ones (lowest first), a reference count each, and the floor (one past the highest
        # page in use)
        self.pager = Pager(self.pages)
        self._room = None
        self.tables, self.lengths = {}, {}
        self.kernels = kernels
        if self.device.type == "cuda" and kernels is None:
            import crit_b200
            self.kernels = crit_b200
        # the block table: a row per open sequence
        self.row_of, self._free_rows = {}, list(range(int(sequences)))
        self.block_tables = torch.full((int(sequences), self.table_pages), self.dump, dtype=torch.int32,
                                       device=self.device)
        self._updates = {}          # flat index -> page id: block-table entries not yet on the device (the last write of
                                    # an entry wins: a scatter with one index twice has no defined order on the device)
        self.device_tables = _Tables(self)
        self.window, self.step_rows, self.step_tokens = int(window), int(step_rows), int(step_tokens)
        self.windows, self.window_tokens = [], 0
        if self.step_rows:
            if self.device.type != "cuda" or self.step_tokens < self.step_rows:
                raise ValueError("step buffers are a CUDA pool's, for at least one token per row")
            long, int32 = dict(dtype=torch.int64, device=self.device), dict(dtype=torch.int32, device=self.device)
            self.d_slots = torch.zeros(self.step_tokens, **long)
            self.d_starts, self.d_counts = torch.zeros(self.step_rows, **int32), torch.zeros(self.step_rows, **int32)
            self.d_firsts, self.d_offsets = torch.zeros(self.step_rows, **long), torch.zeros(self.step_rows, **int32)
            self.d_rows = torch.arange(self.step_rows, **int32)
            self.d_tables = torch.full((self.step_rows, self.table_pages), self.dump, **int32)
            self._d_token_rows, self._d_positions = torch.zeros(self.step_tokens, **long), torch.zeros(self.step_tokens, **long)
        self.round_rows = int(round_rows)
        self.bound, self.slot_of = {}, {}
        slots = max(1, self.round_rows)
        self.round_tables = torch.full((slots, self.table_pages), self.dump, dtype=torch.int32, device=self.device)
        self.round_capacity = torch.zeros(slots, dtype=torch.int64, device=self.device)
        self.round_lengths = torch.zeros(slots, dtype=torch.int64, device=self.device)
        self._start = torch.zeros(slots, dtype=torch.int64, device=self.device)
        self._moved = torch.zeros(slots, dtype=torch.int64, device=self.device)     # a round's tree paths moved already
        self.prompt_slots = None
        self.prompt_table = torch.full((1, self.table_pages), self.dump, dtype=torch.int32, device=self.device)

    # -- sequences -------------------------------------------------------------------------------------------------------
    def open(self, sequence):
        if sequence in self.tables:
            raise ValueError(f"sequence {sequence!r} is open already")
        if not self._free_rows:
            self._more_rows()
        self.tables[sequence], self.lengths[sequence] = [], 0
        self.row_of[sequence] = heapq.heappop(self._free_rows)

    def close(self, sequence):
        if sequence in self.slot_of:
            self._release(self.slot_of[sequence])
        table = self.tables.pop(sequence, None)
        if table is None:
            return
        for page in table:
            self._drop(page)
        self.lengths.pop(sequence, None)
        row = self.row_of.pop(sequence)
        self._updates.update((row * self.table_pages + p, self.dump) for p in range(len(table)))
        heapq.heappush(self._free_rows, row)

    def fork(self, sequence, new):
        """A new sequence sharing `sequence`'s pages up to its valid length (a page is copied when either writes it)."""
        if new in self.tables:
            raise ValueError(f"sequence {new!r} is open already")
        length = self.length(sequence)
        shared = self._table(sequence)[:math.ceil(length / self.page)]
        self.open(new)
        for page in shared:
            self.pager.share(page)
        self.tables[new], self.lengths[new] = list(shared), length
        self._note(new, range(len(shared)))
        if sequence in self.slot_of and length % self.page:     # a bound sequence writes its tail without the host
            tail = (length - 1) // self.page
            self.tables[new][tail] = self._copy(shared[tail])
            self._note(new, [tail])

    def length(self, sequence):
        self._table(sequence)
        if sequence in self.slot_of:
            self.lengths[sequence] = int(self.round_lengths[self.slot_of[sequence]])
        return self.lengths[sequence]

    def keep(self, sequence, length):
        """The sequence's valid KV is its first `length` positions; pages past them are freed."""
        table = self._table(sequence)
        if not 0 <= length <= len(table) * self.page:
            raise ValueError(f"sequence {sequence!r} holds {len(table) * self.page} reserved positions, not {length}")
        self.lengths[sequence] = length
        if sequence in self.slot_of:
            self.round_lengths[self.slot_of[sequence]] = length
            return
        needed = math.ceil(length / self.page)
        row = self.row_of[sequence]
        for p in range(needed, len(table)):
            self._drop(table[p])
            self._updates[row * self.table_pages + p] = self.dump
        del table[needed:]

    def set_scales(self, layer, key_scale, value_scale):
        """An fp8 pool's multipliers for a layer (stored = value / multiplier)."""
        self.scales[self.layers[layer]] = self.torch.tensor([key_scale, value_scale], dtype=self.torch.float32)
        self.scale_values[self.layers[layer]] = (float(key_scale), float(value_scale))

    def fresh_rows(self, layer, tokens):
        """The keys and values the last write() of `layer` stored for this step's `tokens` tokens, as it got them
        ([tokens][kv_heads][dim] each, the compute dtype), where the pool keeps them (quantised pages, a fresh buffer, a
        step with prompt rows), else None.  Reference: pages.py:300-308."""
        if self.fresh_k is None or self._fresh_buffer.tag != (id(self), layer, tokens, self._reserves):
            return None
        return self.fresh_k[:tokens], self.fresh_v[:tokens]

    def layer_pages(self, layer):
        """A layer's pages as stored: (keys [pages][page][kv_heads][head_dim], values); scaled kinds add their scales."""
        i = self.layers[layer]
        if self.dtype in SCALED:
            return self.k[i], self.v[i], self.k_scales[i], self.v_scales[i]
        return self.k[i], self.v[i]

    def table(self, sequence):
        return list(self._table(sequence))

    def held(self, sequence):
        return len(self._table(sequence))

    def free_pages(self):
        return self.pager.free()

    @property
    def floor(self):
        """One past the highest page in use."""
        return self.pager.floor()

    # -- a step ----------------------------------------------------------------------------------------------------------
    def reserve(self, batch):
        """Each token's slot at its position ([tokens] int64 on the pool's device), pages taken as the sequences grow
        and a page a fork still shares copied before it is written.  Reference: pages.py:320-357."""
        self._reserves += 1
        # prompt tokens' keys and values are kept fresh for the step's attention: a PromptBatch's, a StepBatch's with a
        # row past the window (a prompt row); never a round's (reference: pages.py:325-329)
        self._staging = bool(getattr(batch, "prompt", False)) or (
            not getattr(batch, "round", False) and any(batch.row(r)[2] > self.window for r in range(batch.rows)))
        if getattr(batch, "prompt", False):
            if self.prompt_slots is None:
                raise ValueError("a prompt batch reads the slots stage_prompt(batch) staged: stage it first")
            return self.prompt_slots[:batch.bucket]
        if getattr(batch, "round", False):
            return self._reserve_round(batch)
        self.steps += 1
        rows = []
        if self.pager.shared() == 0 and self._room is None:
            # no page is shared (nothing to copy before a write) and nobody to ask for room: the step's rows grow in one
            # call of the allocator, the pages in the order a row-by-row loop would take them
            found = [batch.row(r) for r in range(batch.rows)]
            tables = [self._table(sequence) for sequence, _, _, _ in found]
            have = [len(table) for table in tables]
            need = [max(len(table), (position + count - 1) // self.page + 1) for table, (_, _, count, position) in zip(tables, found)]
            pages, short = self.pager.grow(have, need)
            at = 0
            for table, (sequence, _, _, _), h, n in zip(tables, found, have, need):
                got = pages[at:at + n - h]
                at += len(got)
                table.extend(got)
                self._note(sequence, range(h, len(table)))
                rows.append(self.row_of[sequence])
            if short:
                raise MemoryError(f"the KV pool's {self.pages} pages of {self.page} tokens are all in use")
        else:
            for r in range(batch.rows):
                sequence, _, count, position = batch.row(r)
                table = self._table(sequence)
                last = position + count - 1
                grown = len(table)
                while len(table) < last // self.page + 1:
                    table.append(self._take())
                changed = list(range(grown, len(table)))
                for p in range(position // self.page, last // self.page + 1):
                    if self.pager.refs(table[p]) > 1:
                        table[p] = self._copy(table[p])
                        changed.append(p)
                self._note(sequence, changed)
                rows.append(self.row_of[sequence])
        if self.step_rows:
            return self._step_buffers(batch, rows)
        if self.device.type != "cuda":
            # a pool without a GPU keeps page tables and slot maps (host-side logic and tests): slots from the host lists
            self._flush()
            slots = [self._slot(self.tables[batch.row(r)[0]], q) for r in range(batch.rows)
                     for q in range(batch.row(r)[3], batch.row(r)[3] + batch.row(r)[2])]
            return self.torch.tensor(slots, dtype=self.torch.int64)
        self._flush()
        torch = self.torch
        ids = self._upload(rows, torch.int64)
        token_rows = ids.index_select(0, batch.rows_t)
        return self.kernels.slots_at(self.block_tables, token_rows, batch.positions_t, self.page, self.dump)

    def _step_buffers(self, batch, rows):
        """The step's slots and its window rows' metadata into the step buffers (fixed addresses): one small upload of
        per-row numbers, everything per token computed on the device."""
        torch = self.torch
        windows = [r for r in range(batch.rows) if batch.row(r)[2] <= self.window]
        if batch.tokens > self.step_tokens or len(windows) > self.step_rows:
            raise ValueError(f"a step of {batch.tokens} tokens and {len(windows)} rows of up to {self.window} tokens is "
                             f"larger than the pool's step buffers ({self.step_tokens} tokens, {self.step_rows} rows)")
        self._flush()
        k, n = batch.tokens, len(windows)
        ids = self._upload(rows, torch.int64)
        self._d_token_rows[:k].copy_(ids.index_select(0, batch.rows_t))
        self._d_positions[:k].copy_(batch.positions_t)
        self.kernels.slots_at(self.block_tables, self._d_token_rows[:k], self._d_positions[:k], self.page, self.dump,
                              out=self.d_slots[:k])
        if n:
            offset, meta = 0, []
            for r in windows:
                _, first, count, position = batch.row(r)
                meta.append((first, count, position, offset, rows[r]))
                offset += count
            found = self._upload([x for row in meta for x in row], torch.int64).view(n, 5)
            self.d_starts[:n].copy_(found[:, 0])
            self.d_counts[:n].copy_(found[:, 1])
            self.d_firsts[:n].copy_(found[:, 2])
            self.d_offsets[:n].copy_(found[:, 3])
            self.d_tables[:n].copy_(self.block_tables.index_select(0, found[:, 4]))
        self.windows, self.window_tokens = windows, sum(batch.row(r)[2] for r in windows)
        return self.d_slots[:k]

    def write(self, layer, slots, keys, values):
        """Store a layer's keys [tokens][kv_heads][head_dim] and values at their slots; a slot below 0 is skipped."""
        self._on_gpu("write")
        i = self.layers[layer]
        if self.fresh_k is not None and self._staging and keys.shape[0] <= self.fresh_tokens:
            tokens = keys.shape[0]
            self.fresh_k[:tokens].copy_(keys)
            self.fresh_v[:tokens].copy_(values)
            self._fresh_buffer.tag = (id(self), layer, tokens, self._reserves)
        scaled = self.dtype in SCALED
        self.kernels.write(keys, values if self.value_dim else None, slots, self.k[i],
                           self.v[i] if self.value_dim else None, self.dtype, self.k_scales[i] if scaled else None,
                           self.v_scales[i] if scaled and self.value_dim else None, multipliers=self.scale_values[i])

    def gather(self, layer, sequence, count):
        """The sequence's first `count` positions of a layer: keys [count][kv_heads][head_dim] and values, in the
        compute dtype (dequantised).  Reference: pages.py:455-477."""
        self._on_gpu("gather")
        table = self._table(sequence)
        if count > len(table) * self.page:
            raise ValueError(f"sequence {sequence!r} holds {len(table) * self.page} positions, not {count}")
        self._flush()
        i = self.layers[layer]
        row = self.block_tables[self.row_of[sequence]]
        scaled = self.dtype in SCALED
        mult = self.scale_values[i]
        found = []
        for pages, scales, m in ((self.k[i], self.k_scales[i] if scaled else None, mult[0]),
                                 (self.v[i], self.v_scales[i] if scaled else None, mult[1])):
            found.append(self.kernels.gather(pages, self.dtype, self.page, table=row, count=count, scales=scales,
                                             multiplier=m, dtype=self.compute))
        return tuple(found)

    def rows_at(self, layer, slots):
        """The keys and values at `slots` (any shape of int64 slots) of a layer, dequantised to FP32."""
        self._on_gpu("rows_at")
        i = self.layers[layer]
        scaled = self.dtype in SCALED
        mult = self.scale_values[i]
        torch = self.torch
        return tuple(self.kernels.gather(pages, self.dtype, self.page, slots=slots, scales=scales, multiplier=m,
                                         dtype=torch.float32)
                     for pages, scales, m in ((self.k[i], self.k_scales[i] if scaled else None, mult[0]),
                                              (self.v[i], self.v_scales[i] if scaled else None, mult[1])))

    def slots_at(self, round_slots, positions):
        """The KV slots of `positions` of the sequences bound to `round_slots` (int64 tensors of one shape); a position
        outside its slot's capacity gets the dump page's first slot.  Device work only.  Reference: pages.py:495-501."""
        torch = self.torch
        if self.device.type != "cuda":
            slot, pos = round_slots.reshape(-1).long(), positions.reshape(-1).long()
            page = self.round_tables[slot, (pos // self.page).clamp(0, self.table_pages - 1)]
            inside = (pos >= 0) & (pos < self.round_capacity.index_select(0, slot))
            return torch.where(inside, page.long() * self.page + pos % self.page, self.dump * self.page).view(positions.shape)
        return self.kernels.slots_at(self.round_tables, round_slots.long(), positions.long(), self.page, self.dump,
                                     capacity=self.round_capacity)

    # -- captured prompt chunks ------------------------------------------------------------------------------------------
    def stage_prompt(self, batch):
        """A captured prompt chunk's sequence in the prompt buffers, outside the graph: pages taken up to
        frontier + count, its tokens' slots in prompt_slots (the padding's at the dump page), its page table in
        prompt_table.  Reference: pages.py:516-554."""
        torch = self.torch
        if self.prompt_slots is None or self.prompt_slots.numel() < batch.tokens_max:
            self.prompt_slots = torch.full((batch.tokens_max,), self.dump * self.page, dtype=torch.int64, device=self.device)
        frontier, count = batch.frontier, batch.count
        slots, table = [], []
        if batch.sequence is not None:
            sequence = batch.sequence
            if sequence in self.slot_of:
                raise ValueError(f"sequence {sequence!r} decodes in round slot {self.slot_of[sequence]}: its prompt "
                                 "chunks run before it is bound")
            table = self._table(sequence)
            if count:
                last = frontier + count - 1
                grown = len(table)
                while len(table) < last // self.page + 1:
                    table.append(self._take())
                changed = list(range(grown, len(table)))
                for p in range(frontier // self.page, last // self.page + 1):
                    if self.pager.refs(table[p]) > 1:
                        table[p] = self._copy(table[p])
                        changed.append(p)
                self._note(sequence, changed)
            slots = [self._slot(table, q) for q in range(frontier, frontier + count)]
        self._flush()
        host = torch.full((batch.bucket,), self.dump * self.page, dtype=torch.int64)
        if slots:
            host[:len(slots)] = torch.tensor(slots, dtype=torch.int64)
        self.prompt_slots[:batch.bucket].copy_(host)
        row = torch.full((self.table_pages,), self.dump, dtype=torch.int32)
        if table:
            row[:len(table)] = torch.tensor(table, dtype=torch.int32)
        self.prompt_table[0].copy_(row)

    def commit_prompt(self, batch):
        if batch.sequence is not None:
            self.lengths[batch.sequence] = batch.frontier + batch.count

    # -- captured rounds -------------------------------------------------------------------------------------------------
    def bind(self, slot, sequence, capacity):
        """Round slot `slot` holds `sequence`, whose pages are taken now up to `capacity` positions, so a captured
        round reserves and writes without the host.  Reference: pages.py:562-601."""
        torch = self.torch
        if not 0 <= slot < self.round_rows:
            raise ValueError(f"round slot {slot} is outside the pool's {self.round_rows} round slots")
        if slot in self.bound:
            raise ValueError(f"round slot {slot} holds {self.bound[slot]!r} already")
        if sequence in self.slot_of:
            raise ValueError(f"sequence {sequence!r} is in round slot {self.slot_of[sequence]} already")
        table, length = self._table(sequence), self.lengths[sequence]
        capacity = int(capacity)
        if capacity < max(length, 1):
            raise ValueError(f"sequence {sequence!r} holds {length} positions: a capacity of {capacity} is too small")
        if capacity > self.table_pages * self.page:
            raise ValueError(f"a capacity of {capacity} positions is past the pool's page tables "
                             f"({self.table_pages * self.page} positions: KVPool positions)")
        logical = math.ceil(capacity / self.page)
        wanted = max(0, logical - len(table))
        if wanted > self.pager.free():
            raise MemoryError(f"binding {sequence!r} up to {capacity} positions takes {wanted} pages; "
                              f"{self.pager.free()} of the KV pool's {self.pages} are free")
        grown = len(table)
        while len(table) < logical:
            table.append(self._take())
        changed = list(range(grown, len(table)))
        for p in range(length // self.page, max(logical, len(table))):
            if self.pager.refs(table[p]) > 1:
                table[p] = self._copy(table[p])
                changed.append(p)
        self._note(sequence, changed)
        row = torch.full((self.table_pages,), self.dump, dtype=torch.int32)
        row[:len(table)] = torch.tensor(table, dtype=torch.int32)
        self.round_tables[slot].copy_(row)
        self.round_capacity[slot] = capacity
        self.round_lengths[slot] = length
        self._start[slot] = length
        self.bound[slot], self.slot_of[sequence] = sequence, slot

    def unbind(self, slot):
        """Round slot `slot` holds no sequence; its length is read back (one wait) and the pages past it are freed."""
        if slot not in self.bound:
            raise ValueError(f"round slot {slot} holds no sequence")
        sequence = self.bound[slot]
        length = int(self.round_lengths[slot])
        self._release(slot)
        self.keep(sequence, length)

    def start_round(self, view):
        """A round begins: each row's valid length as the round finds it, and no row's draft-tree path moved yet.
        Reference: pages.py:624-629."""
        rows = view.rows
        self._start[:rows].copy_(self.round_lengths[:rows])
        self._moved[:rows].zero_()

    def commit_round(self, view):
        """Each row's valid length becomes its frontier where it emitted, and stays where it emitted nothing; on the
        device.  With a draft tree (view.tree_path [rows][width + 1]: node 0, then the accepted nodes in order, -1 past
        them) the accepted nodes' keys and values first move from their nodes' positions to consecutive ones, once a
        round (a second commit of the same round finds the path moved).  Device work only.
        Reference: pages.py:631-644, :662-684."""
        rows = view.rows
        emitted = view.n_emitted[:rows]
        path = getattr(view, "tree_path", None)
        if path is not None:
            self._compact(rows, emitted, path[:rows])
        self.round_lengths[:rows].copy_(self.torch.where(emitted > 0, view.frontier[:rows], self._start[:rows]))

    def _compact(self, rows, emitted, path):
        """The accepted path's KV (node path[j], stored at position start + path[j]) to positions start + j, j < the row's
        emitted count.  The slots come from the round tables on the device; the rows are moved by the kernels' move_rows,
        a row's moves in order of j (path[j] >= j: no move reads what an earlier one of its row wrote over)."""
        torch = self.torch
        if self.dtype == "fp8:page":
            raise NotImplementedError("a draft tree's accepted path is not compacted over fp8:page pages: a moved row "
                                      "would change pages, and with them its scale")
        width = path.shape[1]
        columns = torch.arange(width, device=self.device)
        start = self._start[:rows]
        keep = (columns[None, :] < emitted[:, None]) & (columns[None, :] > 0) & (path >= 0) & (self._moved[:rows, None] == 0)
        slot = torch.arange(rows, device=self.device)[:, None].expand(rows, width)
        # columns not kept go from the dump page to itself (position -1 lies outside every slot's capacity): no move
        source = self.slots_at(slot, torch.where(keep, start[:, None] + path.long(), -1))
        target = self.slots_at(slot, torch.where(keep, start[:, None] + columns[None, :], -1))
        n, held = len(self.layers), self.stored_slots
        stores = [self.k.view(n, held, self.kv_heads, self.head_dim)]
        if self.value_dim:
            stores.append(self.v.view(n, held, self.kv_heads, self.value_dim))
        if self.k_scales is not None:
            stores += [scales.view(n, held, self.kv_heads) for scales in (self.k_scales, self.v_scales)]
        if self.device.type != "cuda":
            raise RuntimeError("a draft tree's accepted path is moved by the CUDA kernels: this pool is on the CPU "
                               "(page tables and slot maps only)")
        for store in stores:
            self.kernels.move_rows(store, source, target)
        self._moved[:rows] = 1

    def _reserve_round(self, batch):
        if batch.rows > self.round_rows:
            raise ValueError(f"a round of {batch.rows} rows reads round slots 0 .. {batch.rows - 1}; this KV pool has "
                             f"{self.round_rows} (attention-state's round_rows)")
        slot = batch.slots_t.index_select(0, batch.rows_t)
        return self.slots_at(slot, batch.positions_t)

    def _release(self, slot):
        sequence = self.bound.pop(slot)
        del self.slot_of[sequence]
        self.round_capacity[slot] = 0
        self.round_tables[slot].fill_(self.dump)

    # -- pages -----------------------------------------------------------------------------------------------------------
    def on_exhausted(self, callback):
        """callback() -> whether it freed anything: asked while a page is needed and none is free."""
        self._room = callback

    def _table(self, sequence):
        try:
            return self.tables[sequence]
        except KeyError:
            raise ValueError(f"sequence {sequence!r} is not open") from None

    def _slot(self, table, q):
        return table[q // self.page] * self.page + q % self.page

    def _take(self):
        page = self.pager.take()
        while page < 0 and self._room is not None and self._room():
            page = self.pager.take()
        if page < 0:
            raise MemoryError(f"the KV pool's {self.pages} pages of {self.page} tokens are all in use")
        return page

    def _drop(self, page):
        self.pager.drop(page)

    def _copy(self, page):
        """A page of its own for a writer: every layer's rows (and scales) of `page` copied to a new page."""
        new = self._take()
        self.k[:, new].copy_(self.k[:, page])
        self.v[:, new].copy_(self.v[:, page])
        if self.k_scales is not None:
            self.k_scales[:, new].copy_(self.k_scales[:, page])
            self.v_scales[:, new].copy_(self.v_scales[:, page])
        self._drop(page)
        return new

    # -- the block table on the device -----------------------------------------------------------------------------------
    def _note(self, sequence, indices):
        row, table = self.row_of[sequence], self.tables[sequence]
        self._updates.update((row * self.table_pages + p, table[p]) for p in indices)

    def _upload(self, values, dtype):
        torch = self.torch
        host = torch.tensor(values, dtype=dtype)
        if self.device.type != "cuda":
            return host
        return host.pin_memory().to(self.device, non_blocking=True)

    def _flush(self):
        """The block table's changed entries to the device: one small copy and one scatter, however many there are."""
        if not self._updates:
            return
        torch = self.torch
        packed = self._upload([x for pair in self._updates.items() for x in pair], torch.int64).view(-1, 2)
        self.block_tables.view(-1).index_copy_(0, packed[:, 0], packed[:, 1].to(torch.int32))
        self._updates = {}

    def _more_rows(self):
        torch = self.torch
        if self.device.type == "cuda" and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the block table grows outside a capture: make the pool with more `sequences`")
        have = self.block_tables.shape[0]
        grown = torch.full((have * 2, self.table_pages), self.dump, dtype=torch.int32, device=self.device)
        grown[:have].copy_(self.block_tables)
        self.block_tables = grown
        self._free_rows += list(range(have, have * 2))
        heapq.heapify(self._free_rows)

    def _on_gpu(self, what):
        if self.device.type != "cuda" or self.kernels is None:
            raise RuntimeError(f"KVPool.{what} runs crit_b200's CUDA kernels: a pool on {self.device} keeps page tables "
                               "and slot maps only (there is no CPU or torch path)")
