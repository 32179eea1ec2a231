"""Generates the golden fixtures of tests/golden/ by running the REFERENCE's own torch path (crit 0.21.0).

Run where a checkout of the reference is present:  python tests/golden/make_golden.py /path/to/reference
(or with CRIT_REFERENCE set to that path).  It imports, unmodified, the reference's
  inference/attention-state/code/pages.py            (KVPool, fp8_rows, int8_rows)
  inference/attention-state/code/device_attention.py (DeviceAttention: _gathered SDPA, windows_dense, windows_torch)
  inference/partitioned-attention/plugin.py          (PartitionedAttention.merge)
  inference/partitioned-attention/code/implementation.py (attention_partial, merge_partials)
  tests/inference/e4m3_scale_vectors.txt             (E4M3 known answers)
and writes small .npz / .json files next to this script.  The fixtures travel with the repository; the reference
does not, so no test reads the reference at run time.
"""
import importlib
import json
import math
import sys
import types
from pathlib import Path

import numpy as np
import torch

import os  # noqa: E402

if len(sys.argv) < 2 and "CRIT_REFERENCE" not in os.environ:
    raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["CRIT_REFERENCE"])
OUT = Path(__file__).resolve().parent
sys.path.insert(0, str(REF / "core" / "python"))
from crit_plugins import StepBatch  # noqa: E402

pkg = types.ModuleType("refstate")
pkg.__path__ = [str(REF / "inference" / "attention-state" / "code")]
sys.modules["refstate"] = pkg
pages = importlib.import_module("refstate.pages")
device_attention = importlib.import_module("refstate.device_attention")
ppkg = types.ModuleType("refpart")
ppkg.__path__ = [str(REF / "inference" / "partitioned-attention" / "code")]
sys.modules["refpart"] = ppkg
partitioned = importlib.import_module("refpart.implementation")


def merge_reference(outs, lses):
    """The reference's PartitionedAttention.merge, called unbound on the plugin module's class."""
    root = types.ModuleType("refplugin")
    root.__path__ = [str(REF / "inference" / "partitioned-attention")]
    sys.modules["refplugin"] = root
    sys.modules["refplugin.partitioned"] = ppkg
    sys.modules["refplugin.partitioned.implementation"] = partitioned
    sys.modules["refplugin.state"] = pkg
    sys.modules["refplugin.state.device_attention"] = device_attention
    plugin = importlib.import_module("refplugin.plugin")
    return plugin.PartitionedAttention.merge(None, outs, lses)


def u8(t):
    return t.view(torch.uint8).numpy()


# -- 1. E4M3 known answers ---------------------------------------------------------------------------------------------
def e4m3_vectors():
    bits, codes = [], []
    for line in (REF / "tests" / "inference" / "e4m3_scale_vectors.txt").read_text().splitlines():
        fields = line.split("#", 1)[0].split()
        if fields:
            bits.append(int(fields[0], 16))
            codes.append(int(fields[1], 16))
    np.savez(OUT / "e4m3_vectors.npz", bits=np.array(bits, np.uint32), codes=np.array(codes, np.uint8))


# -- 2. quantise rules -------------------------------------------------------------------------------------------------
def quantize():
    g = torch.Generator().manual_seed(11)
    x = torch.randn(48, 3, 64, generator=g) * 3
    x[5] = 0.0                                  # an all-zero row: scale 1e-30, codes 0
    x[6, 0, 3] = 1e-38                          # a denormal-scale row
    x[6, 0, :3] = 0.0
    x[7] *= 1e4                                 # large magnitudes
    x[8] = torch.where(torch.rand(3, 64, generator=g) < 0.05, x[8] * 20, x[8])   # outliers
    x[9] = x[9].bfloat16().float()              # bf16-representable inputs
    fp8_codes, fp8_scales = pages.fp8_rows(x)
    int8_codes, int8_scales = pages.int8_rows(x)
    mult = 0.05
    static = (x.float() / torch.full((), mult)).clamp(-448, 448).to(torch.float8_e4m3fn)
    # every finite E4M3 magnitude's neighbourhood: midpoints (ties) and their neighbours
    table = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float()
    finite = table[torch.isfinite(table)].unique()
    mids = (finite[:-1] + finite[1:]) / 2
    probes = torch.cat([finite, mids, torch.nextafter(mids, torch.tensor(1e9)), torch.nextafter(mids, torch.tensor(-1e9)),
                        torch.tensor([449.0, 464.0, 1e30, float("inf"), -float("inf"), 2.0 ** -10, 2.0 ** -11])])
    probe_codes = probes.clamp(-448, 448).to(torch.float8_e4m3fn)
    np.savez(OUT / "quantize.npz", x=x.numpy(), fp8row_codes=u8(fp8_codes), fp8row_scales=fp8_scales.numpy(),
             int8_codes=int8_codes.numpy(), int8_scales=int8_scales.numpy(), static_codes=u8(static),
             static_multiplier=np.float32(mult), probes=probes.numpy(), probe_codes=u8(probe_codes))


# -- 3. the pool's page tables and slot maps ---------------------------------------------------------------------------
def pool_script():
    """A script of pool operations; after each, the reference pool's tables, lengths, free pages and returned slots."""
    script = [
        ("open", "a"), ("open", "b"), ("open", "c"),
        ("reserve", [("a", 0, 20), ("b", 0, 1), ("c", 0, 5)]),
        ("keep", "a", 20), ("keep", "b", 1), ("keep", "c", 5),
        ("reserve", [("a", 20, 4), ("b", 1, 1)]),      # a verify window and a decode token
        ("keep", "a", 21), ("keep", "b", 2),
        ("fork", "a", "d"),
        ("reserve", [("d", 21, 3)]),                   # into the shared tail page: copy on write
        ("keep", "d", 24),
        ("reserve", [("a", 21, 30)]),                  # grows over two more pages
        ("keep", "a", 33),                             # roll back: a page is freed
        ("close", "b"),
        ("open", "e"),
        ("reserve", [("e", 0, 40), ("c", 5, 1)]),      # lowest free pages first (b's page reused)
        ("keep", "e", 40), ("keep", "c", 6),
        ("fork", "e", "f"),
        ("reserve", [("f", 40, 1), ("e", 40, 1)]),
        ("keep", "f", 41), ("keep", "e", 41),
        ("close", "a"), ("close", "d"),
        ("open", "g"),
        ("reserve", [("g", 0, 70)]),
        ("keep", "g", 64),
        ("keep", "g", 0),
        ("reserve", [("g", 0, 3)]),
    ]
    pool = pages.KVPool([0], 2, 4, 16 * 16, "cpu", "fp32", page=16)
    trace = []
    for op in script:
        slots = None
        if op[0] == "open":
            pool.open(op[1])
        elif op[0] == "close":
            pool.close(op[1])
        elif op[0] == "fork":
            pool.fork(op[1], op[2])
        elif op[0] == "keep":
            pool.keep(op[1], op[2])
        elif op[0] == "reserve":
            slots = pool.reserve(StepBatch.build(op[1], "cpu")).tolist()
        trace.append({"op": list(op), "slots": slots,
                      "tables": {s: pool.table(s) for s in sorted(pool.tables)},
                      "lengths": {s: pool.lengths[s] for s in sorted(pool.tables)},
                      "free": pool.free_pages(), "floor": pool.floor})
    # a full pool refuses
    small = pages.KVPool([0], 2, 4, 32, "cpu", "fp32", page=16)
    small.open("a")
    try:
        small.reserve(StepBatch.build([("a", 0, 40)], "cpu"))
        refused = None
    except MemoryError as error:
        refused = str(error)
    (OUT / "pool_script.json").write_text(json.dumps({"pages": 16, "page": 16, "trace": trace, "refused": refused},
                                                     indent=1))


# -- 4. captured-round slots -------------------------------------------------------------------------------------------
def round_slots():
    pool = pages.KVPool([0], 2, 4, 32 * 8, "cpu", "fp32", page=8, round_rows=4)
    for s, n in (("a", 13), ("b", 1), ("c", 30)):
        pool.open(s)
        pool.reserve(StepBatch.build([(s, 0, n)], "cpu"))
        pool.keep(s, n)
    pool.bind(0, "a", 40)
    pool.bind(2, "c", 64)
    pool.bind(1, "b", 9)
    slot = torch.tensor([0, 0, 0, 1, 1, 2, 2, 2, 3, 0, 2], dtype=torch.int64)
    positions = torch.tensor([0, 13, 39, 1, 9, 30, 63, 64, 5, -1, 200], dtype=torch.int64)
    found = pool.slots_at(slot, positions)
    np.savez(OUT / "round_slots.npz", tables=pool.round_tables.numpy(), capacity=pool.round_capacity.numpy(),
             slot=slot.numpy(), positions=positions.numpy(), slots=found.numpy(), page=8, dump=pool.dump)


# -- 5. attention ------------------------------------------------------------------------------------------------------
def install_tables(pool, tables, lengths):
    """Give a fresh reference pool these page tables (reserve alone always takes the lowest free page)."""
    used = set()
    for s, (table, n) in enumerate(zip(tables, lengths)):
        pool.tables[s], pool.lengths[s] = list(table), n
        pool.reached[s] = 0
        for p in table:
            pool.refs[p] = 1
            used.add(p)
    pool.free = sorted(set(range(pool.pages)) - used)
    pool.floor = max(used) + 1


def c1_step(hq, hkv, d, page, pool_pages, lens, seed, store_inputs):
    """BASELINE config 1's step on the reference's CPU pool: random disjoint permuted block tables, one appended
    token per sequence through reserve()'s slot mapping, decode attention over the full context."""
    g = torch.Generator().manual_seed(seed)
    if lens is None:
        lens = torch.randint(64, 1025, (4,), generator=g).tolist()
    perm = torch.randperm(pool_pages, generator=g).tolist()
    tables, at = [], 0
    for n in lens:
        need = math.ceil((n + 1) / page)
        tables.append(perm[at:at + need])
        at += need
    pool = pages.KVPool([0], hkv, d, pool_pages * page, "cpu", "fp32", page=page)
    install_tables(pool, tables, lens)
    keys = [torch.randn(n, hkv, d, generator=g) for n in lens]
    values = [torch.randn(n, hkv, d, generator=g) for n in lens]
    for s, n in enumerate(lens):
        slots = torch.tensor([tables[s][p // page] * page + p % page for p in range(n)])
        pool.write(0, slots, keys[s], values[s])
    batch = StepBatch.build([(s, lens[s], 1) for s in range(len(lens))], "cpu")
    slots = pool.reserve(batch)
    new_k = torch.randn(len(lens), hkv, d, generator=g)
    new_v = torch.randn(len(lens), hkv, d, generator=g)
    pool.write(0, slots, new_k, new_v)
    q = torch.randn(len(lens), hq, d, generator=g)
    form = device_attention.DeviceAttention(None, "torch", device="cpu")
    out_sdpa = form.forward(0, q, pool, batch)                       # _gathered: gather + SDPA
    out, lse = form.forward(0, q, pool, batch, lse=True)             # windows_dense
    decode = device_attention.DeviceAttention(None, "torch", device="cpu", prompt_reader="decode")
    out_w, lse_w = decode.forward(0, q, pool, batch, lse=True)       # windows_torch over the page tables
    found = dict(lens=np.array(lens), slots=slots.numpy(), out=out.numpy(), lse=lse.numpy(),
                 out_sdpa=out_sdpa.numpy(), out_windows=out_w.numpy(), lse_windows=lse_w.numpy(),
                 tables=np.array([t + [-1] * (max(map(len, tables)) - len(t)) for t in tables], np.int32),
                 geometry=np.array([hq, hkv, d, page, pool_pages, seed]),
                 checksum=np.array([float(q.double().sum()), float(sum(k.double().sum() for k in keys)),
                                    float(sum(v.double().sum() for v in values))]))
    if store_inputs:
        found.update(q=q.numpy(), new_k=new_k.numpy(), new_v=new_v.numpy(),
                     **{f"k{s}": k.numpy() for s, k in enumerate(keys)},
                     **{f"v{s}": v.numpy() for s, v in enumerate(values)})
    return found


def verify_window():
    """A 6-token verify window (causal inside the draft) over fp8:row pages, and a prompt chunk past the window, on
    the reference's three torch paths."""
    hq, hkv, d, page, n = 10, 2, 32, 16, 150
    g = torch.Generator().manual_seed(21)
    pool = pages.KVPool([0], hkv, d, 64 * page, "cpu", "fp8:row", page=page)
    pool.open("a")
    k0, v0 = torch.randn(n, hkv, d, generator=g).bfloat16(), torch.randn(n, hkv, d, generator=g).bfloat16()
    pool.write(0, pool.reserve(StepBatch.build([("a", 0, n)], "cpu")), k0, v0)
    pool.keep("a", n)
    found = {}
    for name, count in (("verify", 6), ("chunk", 40)):
        batch = StepBatch.build([("a", n, count)], "cpu")
        k1, v1 = torch.randn(count, hkv, d, generator=g).bfloat16(), torch.randn(count, hkv, d, generator=g).bfloat16()
        pool.write(0, pool.reserve(batch), k1, v1)
        q = torch.randn(count, hq, d, generator=g).bfloat16()
        eager = device_attention.DeviceAttention(None, "torch", device="cpu")
        out_sdpa = eager.forward(0, q, pool, batch)
        out, lse = eager.forward(0, q, pool, batch, lse=True)
        decode = device_attention.DeviceAttention(None, "torch", device="cpu", prompt_reader="decode")
        out_w, lse_w = decode.forward(0, q, pool, batch, lse=True)
        found.update({f"{name}_table": np.array(pool.table("a"), np.int32), f"{name}_q": q.float().numpy(), f"{name}_k": k1.float().numpy(), f"{name}_v": v1.float().numpy(),
                      f"{name}_out": out.float().numpy(), f"{name}_lse": lse.numpy(),
                      f"{name}_out_sdpa": out_sdpa.float().numpy(), f"{name}_out_windows": out_w.float().numpy(),
                      f"{name}_lse_windows": lse_w.numpy()})
        pool.keep("a", n)      # roll the window back before the next case
    table = pool.table("a")
    found.update(k0=k0.float().numpy(), v0=v0.float().numpy(), table=np.array(table, np.int32),
                 k_codes=u8(pool.k[0]), v_codes=u8(pool.v[0]), k_scales=pool.k_scales[0].numpy(),
                 v_scales=pool.v_scales[0].numpy(), geometry=np.array([hq, hkv, d, page, n]))
    np.savez_compressed(OUT / "verify_fp8row.npz", **found)


def tree_windows():
    """Two rows of draft trees (parents per token, -1 for none, topological order) over bf16 pages, on the reference's
    torch path: a column sees the context before its row's first position, itself and its ancestors."""
    hq, hkv, d, page = 8, 2, 64, 16
    g = torch.Generator().manual_seed(33)
    pool = pages.KVPool([0], hkv, d, 24 * page, "cpu", "bf16", page=page)
    lens = {"a": 150, "b": 37}
    stored = {}
    for s, n in lens.items():
        pool.open(s)
        k0, v0 = torch.randn(n, hkv, d, generator=g).bfloat16(), torch.randn(n, hkv, d, generator=g).bfloat16()
        pool.write(0, pool.reserve(StepBatch.build([(s, 0, n)], "cpu")), k0, v0)
        pool.keep(s, n)
        stored[s] = (k0, v0)
    batch = StepBatch.build([("a", 150, 7), ("b", 37, 5)], "cpu")
    parents = torch.tensor([-1, 0, 0, 1, 1, 2, 5, -1, 0, 1, 0, 3], dtype=torch.int32)
    k1, v1 = torch.randn(12, hkv, d, generator=g).bfloat16(), torch.randn(12, hkv, d, generator=g).bfloat16()
    pool.write(0, pool.reserve(batch), k1, v1)
    q = torch.randn(12, hq, d, generator=g).bfloat16()
    eager = device_attention.DeviceAttention(None, "torch", device="cpu")
    out, lse = eager.forward(0, q, pool, batch, parents=parents, lse=True)
    # ... and the other visibility rules: a sliding window of 24 positions, a sink logit a head, and all three together
    sinks = torch.randn(hq, generator=g) * 2.0
    out_w, lse_w = eager.forward(0, q, pool, batch, lse=True, sliding=24)
    out_s, lse_s = eager.forward(0, q, pool, batch, lse=True, sinks=sinks)
    out_a, lse_a = eager.forward(0, q, pool, batch, parents=parents, lse=True, sinks=sinks, sliding=24)
    # ... and block lists: each token sees 3 KV blocks of 16 positions (-1: none), its own position's block among them
    blocks = torch.full((12, 3), -1, dtype=torch.int32)
    positions = [150 + c for c in range(7)] + [37 + c for c in range(5)]
    for t, pos in enumerate(positions):
        own = pos // 16
        picks = torch.randperm(own + 1, generator=g)[:2].tolist()
        blocks[t, 0] = own
        blocks[t, 1] = picks[0]
        if t % 3:
            blocks[t, 2] = picks[-1]
    out_b, lse_b = eager.forward(0, q, pool, batch, blocks=blocks, block_size=16, lse=True)
    width = max(len(pool.table(s)) for s in lens)
    tables = np.zeros((2, width), np.int32)
    for i, s in enumerate(lens):
        tables[i, :len(pool.table(s))] = pool.table(s)
    np.savez_compressed(OUT / "tree_bf16.npz", q=q.float().numpy(), parents=parents.numpy(), tables=tables,
                        k_pages=pool.k[0].float().numpy(), v_pages=pool.v[0].float().numpy(), out=out.float().numpy(),
                        lse=lse.numpy(), geometry=np.array([hq, hkv, d, page]), firsts=np.array([150, 37]),
                        counts=np.array([7, 5]), starts=np.array([0, 7]), sinks=sinks.numpy(), sliding=np.array(24),
                        out_sliding=out_w.float().numpy(), lse_sliding=lse_w.numpy(), out_sinks=out_s.float().numpy(),
                        lse_sinks=lse_s.numpy(), out_all=out_a.float().numpy(), lse_all=lse_a.numpy(), blocks=blocks.numpy(),
                        out_blocks=out_b.float().numpy(), lse_blocks=lse_b.numpy())


def fresh_chunk():
    """A prompt chunk over fp8:row pages with a fresh buffer: the chunk's own positions are read from the 16-bit rows
    write() got, the earlier ones from the pages (the reference's torch path, device_attention.py:1136-1145)."""
    hq, hkv, d, page, n, count = 8, 2, 64, 16, 150, 40
    g = torch.Generator().manual_seed(44)
    fresh = pages.FreshBuffer(torch.empty(1 << 18, dtype=torch.uint8))
    pool = pages.KVPool([0], hkv, d, 24 * page, "cpu", "fp8:row", page=page, fresh=fresh)
    pool.open("a")
    k0, v0 = torch.randn(n, hkv, d, generator=g).bfloat16(), torch.randn(n, hkv, d, generator=g).bfloat16()
    pool.write(0, pool.reserve(StepBatch.build([("a", 0, n)], "cpu")), k0, v0)
    pool.keep("a", n)
    batch = StepBatch.build([("a", n, count)], "cpu")
    k1, v1 = torch.randn(count, hkv, d, generator=g).bfloat16(), torch.randn(count, hkv, d, generator=g).bfloat16()
    slots = pool.reserve(batch)
    pool.write(0, slots, k1, v1)
    assert pool.fresh_rows(0, count) is not None
    q = torch.randn(count, hq, d, generator=g).bfloat16()
    eager = device_attention.DeviceAttention(None, "torch", device="cpu")
    out, lse = eager.forward(0, q, pool, batch, lse=True)
    np.savez_compressed(OUT / "fresh_fp8row.npz", q=q.float().numpy(), k1=k1.float().numpy(), v1=v1.float().numpy(),
                        slots=slots.numpy(), table=np.array(pool.table("a"), np.int32), k_codes=u8(pool.k[0]),
                        v_codes=u8(pool.v[0]), k_scales=pool.k_scales[0].numpy(), v_scales=pool.v_scales[0].numpy(),
                        out=out.float().numpy(), lse=lse.numpy(), geometry=np.array([hq, hkv, d, page, n, count]))


# -- 6. merges ---------------------------------------------------------------------------------------------------------
def merges():
    g = torch.Generator().manual_seed(31)
    outs = torch.randn(5, 7, 3, 8, generator=g)
    lses = torch.randn(5, 7, 3, generator=g) * 4
    lses[1, 2] = float("-inf")
    lses[:, 4, 1] = float("-inf")          # a token no part saw
    lses[0, 0, 0], lses[1, 0, 0] = 10000.0, 9999.0
    outs = torch.where(lses[..., None] == float("-inf"), 0.0, outs)
    out, lse = merge_reference(list(outs), list(lses))
    # the host form on a small case: attention_partial over interleaved ownership, merged
    import random
    rng = random.Random(51)
    rows = [(i, tuple(rng.uniform(-2, 2) for _ in range(3)), tuple(rng.uniform(-3, 3) for _ in range(2)))
            for i in range(19)]
    query = tuple(rng.uniform(-1, 1) for _ in range(3))
    host = {}
    for world in (1, 2, 4):
        partials = [partitioned.attention_partial(query, [r for r in rows if r[0] % world == rank], value_width=2,
                                                  query_position=12, scale=0.5) for rank in range(world)]
        merged = partitioned.merge_partials(partials)
        host[str(world)] = {"partials": [[list(p.output), p.log_normalizer] for p in partials],
                            "merged": [list(merged.output), merged.log_normalizer]}
    np.savez(OUT / "merge.npz", outs=outs.numpy(), lses=lses.numpy(), out=out.numpy(), lse=lse.numpy())
    (OUT / "merge_host.json").write_text(json.dumps({"rows": rows, "query": query, "position": 12, "scale": 0.5,
                                                     "worlds": host}, indent=1))


if __name__ == "__main__":
    torch.set_num_threads(8)
    if sys.argv[2:] == ["tree"]:           # those fixtures alone: make_golden.py /path/to/reference tree
        tree_windows()
        fresh_chunk()
        raise SystemExit(0)
    e4m3_vectors()
    quantize()
    pool_script()
    round_slots()
    np.savez_compressed(OUT / "c1_small.npz", **c1_step(8, 2, 16, 4, 64, [9, 33, 1, 20], 7, True))
    np.savez_compressed(OUT / "c1_full.npz", **c1_step(32, 8, 128, 16, 512, None, 1, False))
    verify_window()
    tree_windows()
    fresh_chunk()
    merges()
    print("fixtures written to", OUT)
