"""The kv_cache slot's plugin object: the host form (rows staged after the committed ones stay pending until a commit
keeps the accepted prefix; host_form.Rows) and the device form pool().  The slot's interface:
core/python/crit_plugins/slots.py:62-70; the plugin it stands in for: inference/attention-state/plugin.py."""
from . import host_form
from . import pool as pages


class KVStateCache:
    def __init__(self, page=16, step_rows=0, step_tokens=0, window=16, round_rows=8, kernels=None, sequences=64, fresh=None):
        """fresh: a fresh buffer (pool.FreshBuffer) the plugin's pools of quantised pages keep a prompt chunk's keys and
        values in as they got them (reference: inference/attention-state/plugin.py:15-19, :145-151)."""
        self.page, self.kernels, self.sequences, self.fresh = page, kernels, sequences, fresh
        self.step_rows, self.step_tokens, self.window, self.round_rows = step_rows, step_tokens, window, round_rows
        self.held = {}              # sequence -> host_form.Rows
        self.pools = []

    # -- the host form ---------------------------------------------------------------------------------------------------
    def _rows(self, sequence):
        found = self.held.get(sequence)
        if found is None:
            raise ValueError(f"sequence {sequence!r} is not open")
        return found

    def open(self, sequence, key_width, value_width, capacity):
        if sequence in self.held:
            raise ValueError(f"sequence {sequence!r} is open already")
        self.held[sequence] = host_form.Rows(key_width, value_width, capacity)

    def stage(self, sequence, keys, values):
        self._rows(sequence).append(keys, values)

    def commit(self, sequence, count=None):
        self._rows(sequence).settle(count)

    def rollback(self, sequence):
        self._rows(sequence).drop()

    def rows(self, sequence, pending=False):
        keys, values = self._rows(sequence).view(staged=pending)
        return [(position, key, value) for position, (key, value) in enumerate(zip(keys.tolist(), values.tolist()))]

    def arrays(self, sequence, pending=False):
        """The same rows as two float64 matrices (keys [n][key width], values [n][value width]): what the attention
        slot's host form reads."""
        return self._rows(sequence).view(staged=pending)

    def fork(self, sequence, new):
        if new in self.held:
            raise ValueError(f"sequence {new!r} is open already")
        self.held[new] = self._rows(sequence).fork()

    def release(self, sequence):
        self.held.pop(sequence, None)

    # -- the device form -------------------------------------------------------------------------------------------------
    def pool(self, layers, kv_heads, head_dim, tokens, device, dtype="bf16", *, page=None, value_dim=None, spare=0,
             sliding=0, span=None, positions=None):
        """A paged KV pool of every sequence (pool.KVPool), `page` tokens a page (the plugin's option unless given)."""
        rows = self.step_rows if str(device).startswith("cuda") else 0
        made = pages.KVPool(layers, kv_heads, head_dim, tokens, device, dtype, page=page or self.page,
                            value_dim=value_dim, step_rows=rows, step_tokens=self.step_tokens if rows else 0,
                            window=self.window, round_rows=self.round_rows, kernels=self.kernels, spare=spare,
                            sliding=sliding, span=span, positions=positions, sequences=self.sequences, fresh=self.fresh)
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
