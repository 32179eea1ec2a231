"""Sequence ownership across ranks and the merge of attention partials by their log-normalisers, on the host in Python
floats: the attention slot's host form and the formula every device merge here follows.
Reference: inference/partitioned-attention/code/implementation.py:21-162."""
import math
from dataclasses import dataclass


def _whole(value, least=0):
    if type(value) is not int or value < least:
        raise ValueError(f"integer >= {least} required")
    return value


def _numbers(values, width=None):
    values = tuple(values)
    if not values or (width is not None and len(values) != width):
        raise ValueError("nonempty consistent vector geometry required")
    for x in values:
        if isinstance(x, bool) or not isinstance(x, (int, float)) or not math.isfinite(x):
            raise ValueError("finite numeric vector required")
    return values


@dataclass(frozen=True)
class SequencePartition:
    """Interleaved ownership: position p belongs to rank p % world, where it is local position p // world."""
    world: int
    rank: int
    page_size: int = 256

    def __post_init__(self):
        _whole(self.world, 1)
        _whole(self.rank)
        _whole(self.page_size, 1)
        if self.rank >= self.world:
            raise ValueError("rank outside partition group")

    def owner(self, position):
        return _whole(position) % self.world

    def local(self, position):
        if self.owner(position) != self.rank:
            raise ValueError("position belongs to another rank")
        return position // self.world

    def global_position(self, local):
        return _whole(local) * self.world + self.rank

    def length(self, total):
        total = _whole(total)
        return total // self.world + (1 if self.rank < total % self.world else 0)

    def pages(self, capacity):
        return -(-self.length(capacity) // self.page_size)

    def address(self, position):
        """(local page, row in it) of a position this rank owns."""
        return divmod(self.local(position), self.page_size)


@dataclass(frozen=True)
class AttentionPartial:
    """One shard's normalised output and the log of its softmax sum (-inf, with a zero output: a shard without keys)."""
    output: tuple
    log_normalizer: float

    def __post_init__(self):
        object.__setattr__(self, "output", _numbers(self.output))
        lse = self.log_normalizer
        if isinstance(lse, bool) or not isinstance(lse, (int, float)) or math.isnan(lse) or lse == math.inf:
            raise ValueError("finite log normalizer or explicit empty -inf required")
        if lse == -math.inf and any(x != 0 for x in self.output):
            raise ValueError("empty shard must supply a zero output")


def attention_partial(query, rows, *, value_width, query_position, scale=None, selected_positions=None):
    """A shard's partial for one query: rows of (global position, key, value); positions past query_position, and
    outside selected_positions when given, are not seen."""
    query = _numbers(query)
    _whole(value_width, 1)
    _whole(query_position)
    scale = 1 / math.sqrt(len(query)) if scale is None else scale
    if isinstance(scale, bool) or not isinstance(scale, (int, float)) or not math.isfinite(scale) or scale <= 0:
        raise ValueError("positive finite scale required")
    chosen = None
    if selected_positions is not None:
        listed = tuple(selected_positions)
        for p in listed:
            _whole(p)
        chosen = set(listed)
        if len(chosen) != len(listed):
            raise ValueError("duplicate selected position")
    met, scores, seen_values = set(), [], []
    for position, key, value in rows:
        _whole(position)
        if position in met:
            raise ValueError("duplicate shard position")
        met.add(position)
        key, value = _numbers(key, len(query)), _numbers(value, value_width)
        if position > query_position or (chosen is not None and position not in chosen):
            continue
        score = math.fsum(a * b for a, b in zip(query, key)) * scale
        if not math.isfinite(score):
            raise ValueError("attention score overflow")
        scores.append(score)
        seen_values.append(value)
    if not scores:
        return AttentionPartial((0.0,) * value_width, -math.inf)
    top = max(scores)
    weights = [math.exp(s - top) for s in scores]
    total = math.fsum(weights)
    output = tuple(math.fsum((w / total) * v[c] for w, v in zip(weights, seen_values)) for c in range(value_width))
    return AttentionPartial(output, top + math.log(total))


def merge_partials(partials):
    """Disjoint shards of one query -> the whole: weights exp(lse - max), out = sum w o / sum w, lse = max + log sum w.
    All-empty input is refused; a shard is never dropped silently."""
    partials = tuple(partials)
    if not partials or any(not isinstance(p, AttentionPartial) for p in partials):
        raise ValueError("attention partials required")
    width = len(partials[0].output)
    if any(len(p.output) != width for p in partials):
        raise ValueError("partial output geometry differs")
    top = max(p.log_normalizer for p in partials)
    if top == -math.inf:
        raise ValueError("attention has no visible keys")
    weights = [math.exp(p.log_normalizer - top) for p in partials]
    total = math.fsum(weights)
    output = tuple(math.fsum((w / total) * p.output[c] for w, p in zip(weights, partials)) for c in range(width))
    return AttentionPartial(output, top + math.log(total))


def combine_and_scatter(shards):
    """[rank][query][head] partials -> [rank][local head][query] merged partials: what an all-gather of normalisers and
    a weighted reduce-scatter over heads computes."""
    shards = tuple(tuple(tuple(row) for row in shard) for shard in shards)
    if not shards or not shards[0] or not shards[0][0]:
        raise ValueError("nonempty rank/query/head geometry required")
    world, queries, heads = len(shards), len(shards[0]), len(shards[0][0])
    if heads % world or any(len(s) != queries or any(len(r) != heads for r in s) for s in shards):
        raise ValueError("matching query/head geometry and divisible head count required")
    flat = [p for shard in shards for row in shard for p in row]
    if any(not isinstance(p, AttentionPartial) for p in flat) or any(len(p.output) != len(flat[0].output) for p in flat):
        raise ValueError("matching partial value width required")
    merged = tuple(tuple(merge_partials(shards[r][q][h] for r in range(world)) for q in range(queries))
                   for h in range(heads))
    per_rank = heads // world
    return tuple(merged[r * per_rank:(r + 1) * per_rank] for r in range(world))
