"""The host forms of the kv_cache and attention slots, on numpy arrays.

crit's plugin contract gives every slot a host form beside its device form: small, exact, list-in list-out, used by
the engine's self-checks and by the cases crit compares a plugin with its reference on
(core/python/crit_plugins/slots.py:62-74: open / stage / commit / rollback / rows / fork / release, and
attend(sequence, queries, positions, scale=None, pending=False)).  Here a sequence's rows are two float64 matrices
that grow by doubling, and the attention of a query is computed the way the device computes it across GPUs: the rows are
dealt to `world` shards (position p to shard p mod world: the interleaved ownership of
inference/partitioned-attention/README.md), every shard's softmax partial is taken in one vectorised pass, and the
partials are merged by their log-sum-exps (the formula of inference/partitioned-attention/plugin.py:52-64).
"""
import numpy as np


class Rows:
    """One sequence's key and value rows: rows [0, kept) are committed, rows [kept, held) staged."""

    def __init__(self, key_width, value_width, capacity):
        for name, x in (("key width", key_width), ("value width", value_width), ("capacity", capacity)):
            if isinstance(x, bool) or not isinstance(x, int) or x < 1:
                raise ValueError(f"a sequence's {name} is a positive integer, not {x!r}")
        self.key_width, self.value_width, self.capacity = key_width, value_width, capacity
        self.keys = np.empty((8, key_width))
        self.values = np.empty((8, value_width))
        self.kept = self.held = 0

    def _room(self, more):
        need = self.held + more
        if need > self.capacity:
            raise ValueError(f"KV capacity exhausted: {self.held} rows held, {more} more asked, capacity {self.capacity}")
        if need > len(self.keys):
            size = max(need, 2 * len(self.keys))
            for name in ("keys", "values"):
                old = getattr(self, name)
                grown = np.empty((size, old.shape[1]))
                grown[:self.held] = old[:self.held]
                setattr(self, name, grown)

    def append(self, keys, values):
        """Stage rows after the last one held."""
        keys, values = np.asarray(keys, dtype=np.float64), np.asarray(values, dtype=np.float64)
        if keys.ndim != 2 or values.ndim != 2 or len(keys) != len(values):
            raise ValueError("one value row per key row")
        if keys.shape[1] != self.key_width or values.shape[1] != self.value_width:
            raise ValueError(f"KV geometry differs: rows of {keys.shape[1]} and {values.shape[1]} numbers, the sequence "
                             f"holds {self.key_width} and {self.value_width}")
        if not (np.isfinite(keys).all() and np.isfinite(values).all()):
            raise ValueError("finite KV values required")
        self._room(len(keys))
        self.keys[self.held:self.held + len(keys)] = keys
        self.values[self.held:self.held + len(keys)] = values
        self.held += len(keys)

    def settle(self, count=None):
        """Commit the first `count` staged rows (all by default) and drop the rest."""
        staged = self.held - self.kept
        count = staged if count is None else count
        if isinstance(count, bool) or not isinstance(count, int) or not 0 <= count <= staged:
            raise ValueError(f"commit exceeds staged state: {count!r} of {staged} staged rows")
        self.kept += count
        self.held = self.kept

    def drop(self):
        self.held = self.kept

    def view(self, staged=False):
        """(keys, values) of the committed rows, the staged ones too when asked; row i is position i."""
        n = self.held if staged else self.kept
        return self.keys[:n], self.values[:n]

    def fork(self):
        """A new sequence's rows: a copy of the committed ones."""
        new = Rows(self.key_width, self.value_width, self.capacity)
        new._room(self.kept)
        new.keys[:self.kept], new.values[:self.kept] = self.keys[:self.kept], self.values[:self.kept]
        new.kept = new.held = self.kept
        return new


def shard_partials(query, keys, values, last, world, scale=None, positions=None):
    """The softmax partial of every shard for one query: rows at positions <= last are seen, position p belongs to shard
    p mod world.  -> (outs [world][value width], lses [world]); a shard that sees nothing has zeros and -inf.
    One pass over the rows for all shards (segment maxima and sums by np.maximum.at / np.add.at)."""
    query = np.asarray(query, dtype=np.float64)
    keys, values = np.asarray(keys, dtype=np.float64), np.asarray(values, dtype=np.float64)
    if query.ndim != 1 or keys.ndim != 2 or keys.shape[1] != len(query) or len(values) != len(keys):
        raise ValueError("a query of the keys' width, one value row per key row")
    if isinstance(world, bool) or not isinstance(world, int) or world < 1:
        raise ValueError("one shard or more")
    if not np.isfinite(query).all():
        raise ValueError("finite queries required")
    scale = len(query) ** -0.5 if scale is None else float(scale)
    if not np.isfinite(scale) or scale <= 0:
        raise ValueError("a positive finite scale")
    positions = np.arange(len(keys)) if positions is None else np.asarray(positions)
    seen = positions <= last
    owner = (positions % world)[seen]
    with np.errstate(over="ignore", invalid="ignore"):
        scores = (keys[seen] @ query) * scale
    if not np.isfinite(scores).all():
        raise ValueError("attention score overflow")
    top = np.full(world, -np.inf)
    np.maximum.at(top, owner, scores)
    weights = np.exp(scores - top[owner])
    total = np.zeros(world)
    np.add.at(total, owner, weights)
    outs = np.zeros((world, values.shape[1]))
    np.add.at(outs, owner, weights[:, None] * values[seen])
    some = total > 0
    outs[some] /= total[some, None]
    lses = np.where(some, top + np.log(np.where(some, total, 1.0)), -np.inf)
    return outs, lses


def merge_partials(outs, lses):
    """Partials of one query over disjoint rows -> (out [value width], lse): weights exp(lse - max lse), a shard at -inf
    weighs nothing.  Refused when no shard saw a row."""
    outs, lses = np.asarray(outs, dtype=np.float64), np.asarray(lses, dtype=np.float64)
    if outs.ndim != 2 or lses.shape != (len(outs),) or not len(outs):
        raise ValueError("outs [shards][width] and lses [shards]")
    if np.isnan(lses).any() or (lses == np.inf).any() or not np.isfinite(outs).all():
        raise ValueError("a partial's log-sum-exp is finite or -inf, its output finite")
    top = lses.max()
    if top == -np.inf:
        raise ValueError("attention has no visible keys")
    weights = np.where(lses == -np.inf, 0.0, np.exp(lses - top))
    total = weights.sum()
    return (weights[:, None] * outs).sum(0) / total, float(top + np.log(total))


def attend(query, keys, values, last, world, scale=None):
    """One query over the rows at positions <= last, computed shard by shard and merged -> [value width] floats."""
    out, _ = merge_partials(*shard_partials(query, keys, values, last, world, scale))
    return out
