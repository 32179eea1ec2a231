"""The kv_cache slot's plugin object: the host form (rows staged after the committed ones stay pending until a commit
keeps the accepted prefix) and the device form pool().  Reference: inference/attention-state/plugin.py:14-117 and
code/implementation.py:5-50 (KVState)."""
import math

from . import pool as pages


class HostState:
    """One sequence's rows on the host: committed, and pending until commit(count) keeps a prefix of them."""

    def __init__(self, capacity, key_width, value_width):
        for x in (capacity, key_width, value_width):
            if type(x) is not int or x <= 0:
                raise ValueError("positive integer state geometry required")
        self.capacity, self.key_width, self.value_width = capacity, key_width, value_width
        self.committed, self.pending = [], []

    def stage(self, key, value):
        key, value = tuple(key), tuple(value)
        if len(key) != self.key_width or len(value) != self.value_width:
            raise ValueError("KV geometry differs")
        if not all(math.isfinite(x) for x in key + value):
            raise ValueError("finite KV values required")
        if len(self.committed) + len(self.pending) >= self.capacity:
            raise ValueError("KV capacity exhausted")
        self.pending.append((key, value))

    def commit(self, count=None):
        count = len(self.pending) if count is None else count
        if type(count) is not int or not 0 <= count <= len(self.pending):
            raise ValueError("commit exceeds staged state")
        self.committed += self.pending[:count]
        self.pending.clear()

    def rollback(self):
        self.pending.clear()


class KVStateCache:
    def __init__(self, page=16, step_rows=0, step_tokens=0, window=16, round_rows=8, kernels=None, sequences=64):
        self.states, self.page = {}, page
        self.step_rows, self.step_tokens, self.window = step_rows, step_tokens, window
        self.round_rows, self.kernels, self.sequences = round_rows, kernels, sequences
        self.pools = []

    def _state(self, sequence):
        try:
            return self.states[sequence]
        except KeyError:
            raise ValueError(f"sequence {sequence!r} is not open") from None

    # -- the host form ---------------------------------------------------------------------------------------------------
    def open(self, sequence, key_width, value_width, capacity):
        if sequence in self.states:
            raise ValueError(f"sequence {sequence!r} is open already")
        self.states[sequence] = HostState(capacity, key_width, value_width)

    def stage(self, sequence, keys, values):
        if len(keys) != len(values):
            raise ValueError("one value row per key row")
        state = self._state(sequence)
        for key, value in zip(keys, values):
            state.stage(key, value)

    def commit(self, sequence, count=None):
        self._state(sequence).commit(count)

    def rollback(self, sequence):
        self._state(sequence).rollback()

    def rows(self, sequence, pending=False):
        state = self._state(sequence)
        held = state.committed + (state.pending if pending else [])
        return [(position, list(key), list(value)) for position, (key, value) in enumerate(held)]

    def fork(self, sequence, new):
        state = self._state(sequence)
        self.open(new, state.key_width, state.value_width, state.capacity)
        self.states[new].committed = list(state.committed)

    def release(self, sequence):
        self.states.pop(sequence, None)

    # -- the device form -------------------------------------------------------------------------------------------------
    def pool(self, layers, kv_heads, head_dim, tokens, device, dtype="bf16", *, page=None, value_dim=None, spare=0,
             sliding=0, span=None, positions=None):
        """A paged KV pool of every sequence (pool.KVPool), `page` tokens a page (the plugin's option unless given)."""
        rows = self.step_rows if str(device).startswith("cuda") else 0
        made = pages.KVPool(layers, kv_heads, head_dim, tokens, device, dtype, page=page or self.page,
                            value_dim=value_dim, step_rows=rows, step_tokens=self.step_tokens if rows else 0,
                            window=self.window, round_rows=self.round_rows, kernels=self.kernels, spare=spare,
                            sliding=sliding, span=span, positions=positions, sequences=self.sequences)
        self.pools.append(made)
        return made

    def facts(self):
        """kv_bytes_per_token: the device bytes one more token of context takes across the pools made so far."""
        if not self.pools:
            return {}
        def per_token(pool):
            total = 0
            for tensor in (pool.k, pool.v, pool.k_scales, pool.v_scales):
                if tensor is None:
                    continue
                if tensor.dim() == 3:       # a scale per (page, kv head): its share of a token
                    total += tensor[:, 0].numel() * tensor.element_size() / pool.page
                else:
                    total += tensor[:, 0, 0].numel() * tensor.element_size()
            return total
        return {"kv_bytes_per_token": sum(per_token(pool) for pool in self.pools)}

    def exactness(self):
        return {}
