"""Throughput of the paged KV-cache hot path on B200: KV GB/s of decode attention (and tokens/s), one JSON line.

python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2|c2row|c3|c4|c5] [--only]
N > 1 is launched by torch.distributed.run, one rank per GPU.

A step is one pass of the hot path over one batch: the step's tokens get their KV slots through the block tables,
their keys and values are appended into the pages, and decode attention reads every sequence's whole context (split-K
partials folded by their log-sum-exps).  `value` times steps whose inputs are already in HBM (CUDA-graph replays, the
median of 25 timed batches of K steps); `e2e` times the same step fed from pinned host buffers with the outputs read
back every step (two steps in flight: a step's copies run under its neighbour's kernels).  The roofline object is about
the dominant kernel (the split-K decode launch), timed alone with CUDA events in the same run.  After the timing, a
seeded sample of the step's output rows is compared with the CPU oracle (`parity`); the run fails beyond the bounds.
The line's own numbers are the --workload's (default: FP8 decode, batch 64 x 4,096); `workloads` carries the same
measurements for the other configurations (one long context over a KV range, chunked prefill, speculative verify, and
the FP8 decode on the reference's own per-row scales), each on a shorter run.
`--impl reference` times the reference's CPU path (gather + dequantise + torch SDPA, oracle/torch_path.py) on the host
cores instead: no CUDA and nothing of crit_b200 is loaded there.
"""
import argparse
import json
import math
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

WORKLOADS = {
    # FP8 e4m3 KV decode, batch 64, ctx 4096, 64q/8kv x 128, page 16, pool of 20,000 pages, a scale per (page, kv head)
    "c2": dict(batch=64, ctx=4096, hq=64, hkv=8, d=128, page=16, pool=20000, kind="fp8:page", columns=1, seed=2,
               name="FP8 e4m3 paged decode, batch 64 x ctx 4096, 64q/8kv x 128, page 16, scale per (page, kv head)"),
    # the same on the reference's own FP8 layout: a scale per (slot, kv head)
    "c2row": dict(batch=64, ctx=4096, hq=64, hkv=8, d=128, page=16, pool=20000, kind="fp8:row", columns=1, seed=2,
                  name="FP8 e4m3 paged decode, batch 64 x ctx 4096, 64q/8kv x 128, page 16, scale per (slot, kv head)"),
    # one long context, bf16, 24q/4kv x 256, page 64; the KV range is sharded over the ranks
    "c3": dict(batch=1, ctx=200000, hq=24, hkv=4, d=256, page=64, pool=3126, kind="bf16", columns=1, seed=3,
               name="bf16 long-context decode, batch 1 x ctx 200,000, 24q/4kv x 256, page 64, KV range over the GPUs"),
    # chunked prefill, 4 sequences, 32,768 positions in the pages + a chunk of 2,048, bf16 (tensor-bound)
    "c4": dict(batch=4, ctx=32768 + 2048, hq=32, hkv=8, d=128, page=16, pool=None, kind="bf16", columns=2048, seed=4,
               name="bf16 chunked prefill, 4 sequences x (32,768 prefix + 2,048 chunk), 32q/8kv x 128, page 16"),
    # speculative verify, 32 sequences per GPU, 6 draft tokens, lognormal contexts, FP8
    "c5": dict(batch=32, ctx=None, hq=40, hkv=8, d=128, page=16, pool=None, kind="fp8:page", columns=6, seed=5,
               name="FP8 speculative verify, 32 sequences per GPU x 6 draft tokens, lognormal contexts "
                    "(median 8192, 512..65536), 40q/8kv x 128, page 16"),
}
SAMPLES = 25            # timed batches of --steps steps; the median is reported
MAX_ABS, MEAN_ABS, LSE_ABS = 2e-2, 2e-3, 2e-3


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        found = json.loads(path.read_text())
        return float(found["hbm_gbs"]), float(found["bf16_tflops_sustained"]), "measured on this GPU pool (copy bandwidth / sustained bf16 GEMM)"
    return 6650.0, 1400.0, "fallback (6.65 TB/s, 1.4 PFLOP/s sustained)"


class Clocks:
    """Samples the SM clock and the throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz, self._stop = [], set(), None, threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nvml = None

    def _run(self):
        n = self.nvml
        names = {"hw_slowdown": getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                try:
                    mask = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.reasons |= {name for name, bit in names.items() if mask & bit}
            except Exception:
                pass
            self._stop.wait(0.005)

    def __enter__(self):
        if self.nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unsampled"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def lognormal_lengths(n, seed, median=8192, sigma=1.0, lo=512, hi=65536):
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(n, generator=g, dtype=torch.float64)
    return torch.round(torch.exp(math.log(median) + sigma * z)).clamp(lo, hi).long().tolist()


def kv_bytes_per_token(w):
    code = 1 if w["kind"].startswith("fp8") else 2
    scales = {"fp8:page": w["hkv"] * 2 * 4 / w["page"], "fp8:row": w["hkv"] * 2 * 4}.get(w["kind"], 0)
    return w["hkv"] * 2 * w["d"] * code + scales


def lengths_of(w, rank, world):
    """The context lengths this rank holds (its own tokens of the step included) and, for one context over a KV range,
    the range's first position."""
    if w["ctx"] is None:
        everyone = lognormal_lengths(w["batch"] * max(world, 8), w["seed"])
        return everyone[rank * w["batch"]:(rank + 1) * w["batch"]], 0
    if w["batch"] == 1 and world > 1:
        from crit_b200.dist import kv_ranges
        a, b = kv_ranges(w["ctx"], world, partition=w["page"])[rank]
        return [b - a], a
    return [w["ctx"]] * w["batch"], 0


BLOCK = 4096            # positions a generator seeds: a sequence's rows are made block by block, several at a time


def block_rows(w, rank, s, block):
    """Positions block * 4096 .. of sequence s of rank `rank`: (keys, values) [4096][hkv][d] bf16 on the CPU, from a
    generator seeded by (workload, rank, sequence, block), so the GPU arm and the CPU arm read the same numbers whatever
    part of a sequence they build.  FP8 workloads get about 1% of the entries x20."""
    hkv, d = w["hkv"], w["d"]
    g = torch.Generator().manual_seed(((w["seed"] * 1009 + rank) * 100003 + s) * 1021 + block)
    found = []
    for _ in range(2):
        x = torch.randn(BLOCK, hkv, d, generator=g)
        if w["kind"] != "bf16":
            at = torch.randint(0, x.numel(), (x.numel() // 100,), generator=g)
            x.view(-1)[at] *= 20.0
        found.append(x.bfloat16())
    return found


def sequence_blocks(w, rank, s, first, count, workers=8):
    """Yields (position, keys, values) pieces covering positions first .. first + count of a sequence, in order; the
    blocks are generated on a few threads ahead of the consumer."""
    from concurrent.futures import ThreadPoolExecutor
    blocks = list(range(first // BLOCK, -(-(first + count) // BLOCK)))
    with ThreadPoolExecutor(workers) as pool:
        for block, (k, v) in zip(blocks, pool.map(lambda b: block_rows(w, rank, s, b), blocks)):
            a, b = max(first, block * BLOCK), min(first + count, (block + 1) * BLOCK)
            yield a, k[a - block * BLOCK:b - block * BLOCK], v[a - block * BLOCK:b - block * BLOCK]


def sequence_rows(w, rank, s, first, count):
    """(keys, values) [count][hkv][d] bf16 on the CPU: positions first .. first + count of a sequence."""
    pieces = list(sequence_blocks(w, rank, s, first, count))
    return torch.cat([k for _, k, _ in pieces]), torch.cat([v for _, _, v in pieces])


def step_inputs(w, rank, tokens, shared_queries):
    """The step's queries, keys and values (CPU bf16): the queries of a context sharded by KV range are every rank's."""
    g = torch.Generator().manual_seed(w["seed"] * 7919 + 17 + (0 if shared_queries else rank))
    n = max(tokens, 1)
    q = torch.randn(n, w["hq"], w["d"], generator=g).bfloat16()
    g = torch.Generator().manual_seed(w["seed"] * 7919 + 31 + rank)
    return q, torch.randn(n, w["hkv"], w["d"], generator=g).bfloat16(), torch.randn(n, w["hkv"], w["d"], generator=g).bfloat16()


def packed(parts, pin, where):
    """One buffer holding every tensor of `parts` ([(shape, dtype)]) at 256-byte aligned offsets: (raw bytes, views)."""
    def nbytes(shape, dtype):
        return math.prod(shape) * torch.empty(0, dtype=dtype).element_size()
    sizes = [-(-nbytes(shape, dtype) // 256) * 256 for shape, dtype in parts]
    raw = torch.empty(sum(sizes), dtype=torch.uint8, device=where)
    raw = raw.pin_memory() if pin else raw
    views, at = [], 0
    for (shape, dtype), size in zip(parts, sizes):
        views.append(raw[at:at + nbytes(shape, dtype)].view(dtype).view(*shape))
        at += size
    return raw, views


def build_state(w, device, rank, world):
    """The workload's pages, tables and step inputs on `device` (synthetic, seeded).  Lengths count the step's own
    tokens: a sequence of context n has n - columns positions in the pages and gets `columns` more in the step.  Of one
    context over a KV range only the rank that owns its end appends; the others' ranges are whole already."""
    import crit_b200 as pk
    cpu = torch.Generator().manual_seed(w["seed"] * 1000 + rank)
    cols, page, hkv, d, hq = w["columns"], w["page"], w["hkv"], w["d"], w["hq"]
    lens, range_first = lengths_of(w, rank, world)
    sharded = w["batch"] == 1 and world > 1
    appends = (not sharded) or rank == world - 1
    need = [-(-n // page) for n in lens]
    pool = max(w["pool"] or sum(need) + 64, sum(need))
    order = torch.randperm(pool, generator=cpu)
    width = max(max(need), 1)
    tables = torch.full((len(lens), width), pool, dtype=torch.int32)
    at = 0
    for s, n in enumerate(need):
        tables[s, :n] = order[at:at + n].to(torch.int32)
        at += n
    tables = tables.to(device)
    store = torch.bfloat16 if w["kind"] == "bf16" else torch.float8_e4m3fn
    k = torch.zeros(pool + 1, page, hkv, d, dtype=store, device=device)
    v = torch.zeros_like(k)
    ks = vs = None
    if w["kind"] == "fp8:page":
        ks, vs = torch.zeros(pool + 1, hkv, device=device), torch.zeros(pool + 1, hkv, device=device)
    elif w["kind"] == "fp8:row":
        ks, vs = torch.zeros(pool + 1, page, hkv, device=device), torch.zeros(pool + 1, page, hkv, device=device)
    # fill the contexts (without the step's own tokens), a sequence at a time
    for s, n in enumerate(lens):
        have = max(n - cols, 0) if appends else n
        # whole pages at a time, so that a page's scale is its rows' amax / 448 however the fill is cut
        for a, keys, values in sequence_blocks(w, rank, s, 0, have):
            rows = torch.full((keys.shape[0],), s, dtype=torch.int64, device=device)
            slots = pk.slots_at(tables, rows, torch.arange(a, a + keys.shape[0], device=device), page, pool)
            pk.write(keys.to(device), values.to(device), slots, k, v, w["kind"], ks, vs)
    live = [s for s, n in enumerate(lens) if n > 0]
    tokens = len(live) * cols
    firsts = torch.tensor([lens[s] - cols for s in live], dtype=torch.int64)
    state = dict(w=w, lens=lens, live=live, tables=tables, k=k, v=v, ks=ks, vs=vs, pool=pool, tokens=tokens, rank=rank,
                 world=world, range_first=range_first, appends=appends and tokens > 0, sharded=sharded,
                 rows=torch.tensor(live, dtype=torch.int32, device=device),
                 starts=(torch.arange(len(live), dtype=torch.int32) * cols).to(device),
                 firsts=firsts.to(device),
                 token_rows=torch.tensor(live, dtype=torch.int64).repeat_interleave(cols).to(device),
                 positions=(firsts[:, None] + torch.arange(cols)[None, :]).reshape(-1).to(device))
    # The step's inputs (q, k, v) sit in ONE pinned host buffer and one device buffer, its results (out, lse) in another
    # pair, so the end-to-end step is one copy in and one copy out; two sets of device buffers, so that two steps can be
    # in flight (a step's copies under its neighbour's kernels).
    n = max(tokens, 1)
    ins = [((n, hq, d), torch.bfloat16), ((n, hkv, d), torch.bfloat16), ((n, hkv, d), torch.bfloat16)]
    outs = [((n, hq, d), torch.bfloat16), ((n, hq), torch.float32)]
    state["h_in"], host_in = packed(ins, True, "cpu")
    for h, x in zip(host_in, step_inputs(w, rank, tokens, sharded)):
        h.copy_(x)
    state["h_q"] = host_in[0]
    state["sets"] = []
    for _ in range(2):
        d_in, (dq, dk, dv) = packed(ins, False, device)
        d_in.copy_(state["h_in"])
        d_res, (out, lse) = packed(outs, False, device)
        h_res, (h_out, h_lse) = packed(outs, True, "cpu")
        state["sets"].append(dict(d_in=d_in, q=dq, k=dk, v=dv, d_res=d_res, out=out, lse=lse, h_res=h_res, h_out=h_out,
                                  h_lse=h_lse))
    state["slots"] = torch.empty(n, dtype=torch.int64, device=device)
    state["kv_bytes"] = sum(lens) * kv_bytes_per_token(w)
    state["merger"] = None
    state["chunk"] = None
    if sharded:
        from crit_b200.dist import ShardMerge, chunk_to_fill
        state["merger"] = ShardMerge(cols, hq, d, device, out_dtype=torch.bfloat16, exchange=w.get("exchange", "auto"))
    if w["batch"] == 1 and cols == 1 and lens[0] > 0:
        # one long row read alone: the split size that fills the device's resident blocks in whole waves
        from crit_b200.dist import chunk_to_fill
        found = pk.plan(hq, hkv, d, d, page, w["kind"], 1, device)
        state["chunk"] = chunk_to_fill(lens[0], hkv, found["sms"] * max(found["per_sm"], 1), waves=1 if sharded else None)
    return state


def step(state, launch="both", append=True, buffers=0):
    """One pass of the hot path: slot mapping, append, split-K decode attention + merge (or, for a context over a KV
    range, fold + push and wait + merge of shards)."""
    import crit_b200 as pk
    w, b = state["w"], state["sets"][buffers]
    if not state["live"]:
        return
    if append and state["appends"]:
        pk.slots_at(state["tables"], state["token_rows"], state["positions"], w["page"], state["pool"], out=state["slots"])
        pk.write(b["k"], b["v"], state["slots"], state["k"], state["v"], w["kind"], state["ks"], state["vs"])
    if w["columns"] > 64:        # a prompt chunk per sequence: one prefill launch over all the sequences' chunks
        if "prompt_tables" not in state:
            state["prompt_tables"] = state["tables"][state["rows"].long()].to(torch.int32).contiguous()
        pk.prefill(b["q"], state["k"], state["v"], w["kind"], state["prompt_tables"], state["firsts"], w["page"],
                   key_scales=state["ks"], value_scales=state["vs"], out=b["out"], lse=b["lse"],
                   engine=state.get("engine"))
        return
    pk.attend(b["q"], state["k"], state["v"], w["kind"], state["tables"], state["rows"], state["starts"],
              state["firsts"], w["columns"], w["page"], key_scales=state["ks"], value_scales=state["vs"],
              out=b["out"], lse=b["lse"], launch=launch, staging=state.get("staging"),
              engine=state.get("engine"), chunk=state.get("chunk"), shards=state["merger"])


def launches_per_step(state):
    if not state["live"]:
        return 0
    n = 2 if state["appends"] else 0
    if state["w"]["columns"] > 64:
        return n + 1
    return n + (3 if state["merger"] is not None and state["merger"].peer is not None else 2)


# dram__bytes_read.sum + dram__bytes_write.sum of the decode launch, from one ncu capture per workload (profiles/): the
# captured launch's traffic over its algorithmic bytes.  Traffic grows in proportion to the KV bytes (every byte is read
# once; the writes are the partial states, a fixed number per split), so a launch's traffic is its algorithmic bytes
# times the ratio.  None where no capture was made.
TRAFFIC_RATIO = {("c2", "mma.sync"): (540.9e6 + 9.7e6) / 537.9e6,      # decode_kernel, FP8 decode at full size
                 ("c2", "tcgen05p"): (270.6e6 + 4.3e6) / 269.0e6,      # decode_ph_kernel, FP8 decode at 32 sequences
                 ("c3", "mma.sync"): (819.4e6 + 7.6e6) / 819.2e6,      # decode_kernel (TMA), the long context at full size
                 ("c5", "tcgen05"): (167.9e6 + 4.7e6) / 167.0e6}       # decode_tc_kernel<4>, verify at 8 sequences


# -- parity: a seeded sample of the step's rows against the CPU oracle ------------------------------------------------------
def stored_rows(state, s):
    """Sequence s's pages as the oracle reads them: FP32 keys and values [positions][hkv][d] (dequantised exactly)."""
    import oracle
    w = state["w"]
    n = state["lens"][s]
    index = state["tables"][s][:-(-n // w["page"])].long()
    found = []
    for pages, scales in ((state["k"], state["ks"]), (state["v"], state["vs"])):
        rows = pages.index_select(0, index)
        if w["kind"] == "bf16":
            found.append(rows.float().cpu().numpy().reshape(-1, w["hkv"], w["d"]))
            continue
        codes = rows.view(torch.uint8).cpu().numpy().reshape(-1, w["hkv"], w["d"])
        sc = scales.index_select(0, index).cpu().numpy()
        if w["kind"] == "fp8:row":
            sc = sc.reshape(-1, w["hkv"])
        found.append(oracle.dequantize(codes, w["kind"], sc, page=w["page"]))
    return found


def parity(state, buffers=0, rows=None, tokens_per_row=None, seed=0):
    """The step's outputs of a seeded sample of rows against oracle.attend over the pages as they are stored.  rows: how
    many sequences (all when None); tokens_per_row: of a prompt chunk, how many of its tokens.  A context over a KV range:
    every rank's oracle partial over its own range is gathered and merged by the oracle's own merge, and compared with the
    merged output.  -> {"max_abs", "mean_abs", "lse_abs", "rows", "tokens", "ok"}."""
    import numpy as np
    import oracle
    w, b = state["w"], state["sets"][buffers]
    cols = w["columns"]
    torch.cuda.synchronize()
    out, lse = b["out"].float().cpu().numpy(), b["lse"].cpu().numpy()
    q = b["q"].float().cpu().numpy()
    g = torch.Generator().manual_seed(1234 + seed)
    live = state["live"]
    pick = list(range(len(live)))
    if rows is not None and rows < len(live):
        longest = max(pick, key=lambda i: state["lens"][live[i]])
        pick = sorted(set(torch.randperm(len(live), generator=g)[:rows - 1].tolist()) | {longest})
    errs, lse_errs, n_tokens = [], [], 0
    rel = 0.0 if w["kind"] == "bf16" else 2.0 ** -7

    def compare(got, want):
        # FP8 workloads carry x20 outliers: outputs reach magnitudes where bf16's own spacing passes 2e-2 (0.125 at 16),
        # so there the bound is 2e-2 + 2^-7 |want| (each error divided by 1 + |want| / 2.56), the GPU tests' rule
        return (np.abs(got - want) / (1.0 + (rel / MAX_ABS) * np.abs(want))).reshape(-1)
    if state["sharded"]:
        import torch.distributed as dist
        hq, d = w["hq"], w["d"]
        part = np.zeros((cols, hq, d), np.float32), np.full((cols, hq), -np.inf, np.float32)
        if live:
            k, v = stored_rows(state, 0)
            n = state["lens"][0]
            part = oracle.attend(q, k, v, np.arange(-(-n // w["page"]), dtype=np.int32), [0], [0], [n - cols], cols, w["page"])
        mine = torch.from_numpy(np.concatenate([part[0].reshape(-1), part[1].reshape(-1)])).to(b["out"].device)
        every = [torch.empty_like(mine) for _ in range(state["world"])]
        dist.all_gather(every, mine)
        every = torch.stack(every).cpu().numpy()
        want, want_lse = oracle.merge(every[:, :cols * hq * d].reshape(-1, cols, hq, d), every[:, cols * hq * d:].reshape(-1, cols, hq))
        errs.append(compare(out[:cols], want))
        lse_errs.append(np.abs(lse[:cols] - want_lse).reshape(-1))
        n_tokens = cols
    else:
        for i in pick:
            s = live[i]
            n = state["lens"][s]
            k, v = stored_rows(state, s)
            table = np.arange(-(-n // w["page"]), dtype=np.int32)
            span = list(range(cols))
            if tokens_per_row is not None and tokens_per_row < cols:
                span = sorted(set(torch.randperm(cols, generator=g)[:tokens_per_row - 2].tolist()) | {0, cols - 1})
            # each sampled token as a row of one column at its own position
            want, want_lse = oracle.attend(q[i * cols:(i + 1) * cols], k, v, table, [0] * len(span), span,
                                           [n - cols + c for c in span], 1, w["page"])
            errs.append(compare(out[i * cols:(i + 1) * cols][span], want[span]))
            lse_errs.append(np.abs(lse[i * cols:(i + 1) * cols][span] - want_lse[span]).reshape(-1))
            n_tokens += len(span)
    errs, lse_errs = np.concatenate(errs), np.concatenate(lse_errs)
    found = {"max_abs": float(errs.max()), "mean_abs": float(errs.mean()), "lse_abs": float(lse_errs.max()),
             "rows": len(pick) if not state["sharded"] else 1, "tokens": n_tokens, "against": "oracle.attend (CPU, double "
             "accumulation) over the pages as stored", "bounds": {"max_abs": MAX_ABS, "mean_abs": MEAN_ABS, "lse_abs": LSE_ABS,
                                                                  "relative_term": rel}}
    found["ok"] = bool(np.isfinite(errs).all() and found["max_abs"] <= MAX_ABS and found["mean_abs"] <= MEAN_ABS
                       and found["lse_abs"] <= LSE_ABS)
    return found


def leave():
    """The ranks leave together with nothing in flight; a communicator that will not close within 20 s (one whose
    all-gather sits in a captured graph has done that) does not keep the launcher waiting."""
    import torch.distributed as dist
    sys.stdout.flush()
    watchdog = threading.Timer(20.0, lambda: os._exit(0))
    watchdog.daemon = True
    watchdog.start()
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    watchdog.cancel()


def timed(fn, steps, warmup, stream, samples=1):
    """Seconds per step: `samples` timed batches of `steps` calls after `warmup` calls (CUDA events on `stream`); returns
    (median, min, max) over the batches."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    found = []
    for _ in range(samples):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(steps):
            fn()
        b.record(stream)
        b.synchronize()
        found.append(a.elapsed_time(b) / 1e3 / steps)
    return statistics.median(found), min(found), max(found)


def measure(name, w, args, device, rank, world, local, primary):
    """Everything the line says about one workload: the step from HBM, the decode launch alone, the append, the step end
    to end, and parity."""
    import torch.distributed as dist
    state = build_state(w, device, rank, world)
    state["staging"], state["engine"] = args.staging, args.engine
    if args.chunk:
        state["chunk"] = args.chunk
    torch.cuda.synchronize()
    steps = args.steps if primary else max(5, args.steps // 2)
    samples = SAMPLES if primary else 9
    prompt = w["columns"] > 64
    stream = torch.cuda.Stream(device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        for _ in range(2):
            for which in (0, 1):
                step(state, buffers=which)
        stream.synchronize()
        graphs = [None, None]
        if not args.no_graph:
            try:
                for which in (0, 1):
                    graphs[which] = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graphs[which], stream=stream):
                        step(state, buffers=which)
            except Exception as error:          # a collective that does not capture: time eager steps instead
                print(f"[bench] step not captured ({type(error).__name__}: {error}); timing eager steps", file=sys.stderr)
                graphs = [None, None]
                torch.cuda.synchronize()
        runs = [(lambda which=which: step(state, buffers=which)) if graphs[which] is None else graphs[which].replay
                for which in (0, 1)]
        barrier()
        with Clocks(local) as clocks:
            seconds, fastest, slowest = timed(runs[0], steps, args.warmup, stream, samples)
            # the dominant kernel alone (same stream, CUDA events): five launches back to back from a graph, so that the
            # launches' host cost is not what is timed
            decode_fn, reps = (lambda: step(state, launch="decode", append=False)), 1
            if not args.no_graph and state["live"]:
                try:
                    decode_graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(decode_graph, stream=stream):
                        for _ in range(5):
                            step(state, launch="decode", append=False)
                    decode_fn, reps = decode_graph.replay, 5
                except Exception:
                    torch.cuda.synchronize()
            decode_s = timed(decode_fn, max(4, steps // 2), 3, stream, 7)[0] / reps
        barrier()
        # the fold of the splits (a few microseconds): ten launches back to back from a graph, so that the launches' host
        # cost is not what is timed
        merge_s = None
        if not prompt and state["merger"] is None and state["live"]:
            merge_fn, reps = (lambda: step(state, launch="merge", append=False)), 1
            if not args.no_graph:
                try:
                    merge_graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(merge_graph, stream=stream):
                        for _ in range(10):
                            step(state, launch="merge", append=False)
                    merge_fn, reps = merge_graph.replay, 10
                except Exception:
                    torch.cuda.synchronize()
            merge_s = timed(merge_fn, 20, 3, stream)[0] / reps
        append = append_times(state, stream) if primary or prompt else None
        barrier()
        e2e_s = e2e_time(state, runs, stream, max(20, steps), device)
        barrier()
    checked = None
    if not args.no_check:
        runs[0]()
        torch.cuda.synchronize()
        checked = parity(state, 0, rows={"c2": 12, "c2row": 12, "c5": 5}.get(name), tokens_per_row=16 if prompt else None)
    kv, tokens = float(state["kv_bytes"]), float(state["tokens"]) if (not state["sharded"] or rank == 0) else 0.0
    if world > 1:
        t = torch.tensor([seconds, fastest, slowest, e2e_s, decode_s], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        seconds, fastest, slowest, e2e_s, decode_max = (float(x) for x in t)
        total = torch.tensor([kv, tokens, 0.0 if checked is None or checked["ok"] else 1.0], device=device, dtype=torch.float64)
        dist.all_reduce(total)
        kv_total, tokens_total, bad = (float(x) for x in total)
        if checked is not None:
            checked["ok"] = bad == 0.0
    else:
        kv_total, tokens_total, decode_max = kv, tokens, decode_s
    hbm_peak, tensor_peak, peak_source = peaks()
    engine = args.engine or ("library default: " + engine_of(args, state))
    found = {"workload": w["name"], "value": kv_total / seconds / 1e9, "unit": "GB/s", "ms_per_step": seconds * 1e3,
             "ms_per_step_min": fastest * 1e3, "ms_per_step_max": slowest * 1e3, "timed_batches": samples, "steps_per_batch": steps,
             "tokens_per_s": tokens_total / seconds, "hbm_frac_of_8TBps": kv_total / world / seconds / 8e12,
             "scaling": "strong" if w["batch"] == 1 else "weak",
             "sharding": "KV range per GPU (fold + peer stores, wait + merge of shards)" if state["sharded"] else "sequences per GPU, no collective",
             "kv": w["kind"], "engine": engine, "graph_replay": graphs[0] is not None,
             "steps_are": ("slot map + KV append + one prefill launch over the sequences' chunks" if prompt else
                           "slot map + KV append + split-K decode + " +
                           ("fold of the splits" if state["merger"] is None else
                            ("fold + push to every rank, wait + merge of shards" if state["merger"].peer is not None
                             else "fold, NCCL all-gather, merge of shards"))),
             "l2": ("inputs larger than L2: every step reads the whole KV context "
                    if state["kv_bytes"] > 2 * 126e6 else
                    "this rank's KV is under twice the L2's 126 MB: reads may hit L2, the figure is not an HBM figure ") +
                   f"({state['kv_bytes'] / 1e6:.1f} MB per GPU)",
             "gpu_launches_per_step": launches_per_step(state), "clocks": clocks.summary(),
             "e2e": {"value": kv_total / e2e_s / 1e9, "unit": "GB/s", "tokens_per_s": tokens_total / e2e_s,
                     "ms_per_step": e2e_s * 1e3, "h2d_bytes_per_step": state["h_in"].numel(),
                     "d2h_bytes_per_step": state["sets"][0]["h_res"].numel(),
                     "pipeline": "two steps in flight: every step's inputs are copied from pinned host memory and its "
                                 "outputs copied back and waited for on the host; the copies of a step run under the "
                                 "kernels of its neighbour"},
             "parity": checked}
    achieved = state["kv_bytes"] / decode_s / 1e9 if decode_s > 0 else 0.0
    found["roofline"] = {"bound": "hbm", "kernel": "split-K decode launch over paged KV (" + {"mma.sync": "decode_kernel: m16n8k16", "tcgen05": "decode_tc_kernel: tcgen05, one kv head a unit", "tcgen05t": "decode_sw_kernel: tcgen05, operands swapped", "tcgen05p": "decode_ph_kernel: tcgen05, whole page rows"}.get(engine_of(args, state), "decode_kernel") + ")",
                         "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                         "frac_of_8TBps": achieved / 8000.0, "peak_source": peak_source, "us_per_launch": decode_s * 1e6,
                         "us_per_launch_max_over_ranks": decode_max * 1e6,
                         "merge_us_per_launch": merge_s * 1e6 if merge_s is not None else None,
                         "algorithmic_bytes_per_launch": state["kv_bytes"],
                         "traffic": traffic(name, args, state)}
    if prompt:                   # a dense contraction: the roofline is the tensor cores'
        cols, hq, d = w["columns"], w["hq"], w["d"]
        pairs = sum(cols * (n - cols) + cols * (cols + 1) // 2 for n in state["lens"])
        flops = pairs * 4 * d * hq
        tf = flops / decode_s / 1e12
        found["tflops"] = flops / seconds / 1e12
        # the library's own choice between its two tcgen05 block shapes: 256-row blocks from one a multiprocessor on
        pairs = -(-cols * (hq // w["hkv"]) // 256) * w["hkv"] * len(state["live"])
        paired = args.engine == "tcgen05:pair" or (args.engine in (None, "tcgen05") and
                                                  pairs >= torch.cuda.get_device_properties(device).multi_processor_count)
        found["roofline"] = {"bound": "tensor", "kernel": "chunked prefill over paged KV (prefill_kernel: m16n8k16)"
                             if args.engine == "mma.sync" else "chunked prefill over paged KV (%s: tcgen05 / TMEM)"
                             % ("prefill_pair_kernel" if paired else "prefill_tc_kernel"),
                             "achieved": tf, "peak": tensor_peak, "unit": "TFLOP/s", "frac": tf / tensor_peak,
                             "peak_source": peak_source, "us_per_launch": decode_s * 1e6,
                             "algorithmic_flops_per_step": flops, "traffic": None}
    if append is not None:
        found["append"] = append
    return found, state


def engine_of(args, state):
    """The decode kernel the step's launch runs on: the one asked for, or crit_b200's own choice for the launch."""
    import crit_b200 as pk
    w = state["w"]
    if args.engine or state.get("merger") is not None or args.staging:
        return args.engine or "mma.sync"
    rows = int(state["rows"].shape[0]) if hasattr(state.get("rows"), "shape") else len(state["live"])
    return pk.engine_for(w["kind"], w["d"], w["d"], w["hq"], w["hkv"], min(w["columns"], 64), rows,
                         int(state["tables"].shape[1]) * w["page"])


def traffic(name, args, state):
    if args.staging or args.chunk:
        return None
    engine = engine_of(args, state)
    ratio = TRAFFIC_RATIO.get((name, engine))
    return None if ratio is None else ratio * state["kv_bytes"]


def append_times(state, stream):
    """The KV append alone: the step's own tokens (slot map + append: two launches) and a bulk fill of 4,096 tokens of one
    sequence; microseconds and GB/s of bytes read (bf16 inputs) plus bytes written (codes and scales)."""
    import crit_b200 as pk
    w, b = state["w"], state["sets"][0]
    if not state["live"] or not state["appends"]:
        return None
    per_token = w["hkv"] * 2 * w["d"] * 2 + kv_bytes_per_token(w)

    def own():
        pk.slots_at(state["tables"], state["token_rows"], state["positions"], w["page"], state["pool"], out=state["slots"])
        pk.write(b["k"], b["v"], state["slots"], state["k"], state["v"], w["kind"], state["ks"], state["vs"])
    found = {}
    seconds = timed(own, 20, 3, stream, 3)[0]
    found["step_tokens"] = {"tokens": state["tokens"], "us": seconds * 1e6, "gb_per_s": state["tokens"] * per_token / seconds / 1e9}
    s = max(state["live"], key=lambda x: state["lens"][x])
    n = min(4096, (state["lens"][s] - w["columns"]) // w["page"] * w["page"])
    if n >= w["page"]:
        keys, values = (x.to(state["k"].device) for x in sequence_rows(w, state["rank"], s, 0, n))
        slots = pk.slots_at(state["tables"], torch.full((n,), s, dtype=torch.int64, device=keys.device),
                            torch.arange(n, device=keys.device), w["page"], state["pool"])
        seconds = timed(lambda: pk.write(keys, values, slots, state["k"], state["v"], w["kind"], state["ks"], state["vs"]),
                        20, 3, stream, 3)[0]
        found["bulk_fill"] = {"tokens": n, "us": seconds * 1e6, "gb_per_s": n * per_token / seconds / 1e9}
    return found


def e2e_time(state, runs, stream, steps, device):
    """Seconds per step with every step's inputs copied from pinned host memory and its outputs copied back and waited for
    on the host, two steps in flight: three streams (copies in, kernels, copies out) and two sets of device buffers."""
    sets = state["sets"]
    h2d, d2h = torch.cuda.Stream(device), torch.cuda.Stream(device)
    ready = [torch.cuda.Event() for _ in (0, 1)]
    done = [torch.cuda.Event() for _ in (0, 1)]
    back = [torch.cuda.Event() for _ in (0, 1)]

    def loop(n):
        for i in range(n):
            b = i & 1
            with torch.cuda.stream(h2d):
                if i >= 2:
                    h2d.wait_event(done[b])                 # the kernels that read this set's inputs two steps ago
                sets[b]["d_in"].copy_(state["h_in"], non_blocking=True)
                ready[b].record(h2d)
            with torch.cuda.stream(stream):
                stream.wait_event(ready[b])
                if i >= 2:
                    stream.wait_event(back[b])              # this set's results of two steps ago have left
                runs[b]()
                done[b].record(stream)
            with torch.cuda.stream(d2h):
                d2h.wait_event(done[b])
                sets[b]["h_res"].copy_(sets[b]["d_res"], non_blocking=True)
                back[b].record(d2h)
            if i >= 1:
                back[1 - b].synchronize()                   # the host has the step before's results
        back[(n - 1) & 1].synchronize()
    loop(4)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    loop(steps)
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) / steps


# -- the reference arm: the reference's CPU path, no CUDA, nothing of the product ---------------------------------------------
def cpu_pages(w, rank, s, n):
    """Sequence s as the reference's CPU pool would hold it: (key codes [pages][page][hkv][d], value codes, key scales,
    value scales, table) quantised by the oracle's rules from the workload's seeded rows."""
    import numpy as np
    import oracle
    page, hkv, d = w["page"], w["hkv"], w["d"]
    pages = -(-n // page)
    keys, values = sequence_rows(w, rank, s, 0, n)
    table = torch.arange(pages, dtype=torch.int32)[None]
    if w["kind"] == "bf16":
        pad = pages * page - n
        grow = (lambda x: torch.cat([x, x.new_zeros(pad, hkv, d)]).view(pages, page, hkv, d))
        return grow(keys), grow(values), None, None, table
    found = []
    for x in (keys, values):
        x = x.float().numpy()
        if w["kind"] == "fp8:row":
            codes, scales = oracle.quantize_rows(x, "fp8:row")
            full = np.zeros((pages * page, hkv, d), np.uint8)
            full[:n] = codes
            sc = np.ones((pages * page, hkv), np.float32)
            sc[:n] = scales
            found += [torch.from_numpy(full).view(pages, page, hkv, d), torch.from_numpy(sc).view(pages, page, hkv)]
        else:
            codes, scales = np.zeros((pages * page, hkv, d), np.uint8), np.zeros((pages, hkv), np.float32)
            oracle.quantize_pages(x, np.arange(n, dtype=np.int64), page, codes, scales)
            found += [torch.from_numpy(codes).view(pages, page, hkv, d), torch.from_numpy(scales)]
    return found[0], found[2], found[1], found[3], table


def reference_arm(name, w, gpus, steps, warmup):
    """--impl reference: W + K passes of the reference's CPU path over a bounded sample of the workload's sequences."""
    from oracle import torch_path
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    lens, _ = lengths_of(w, 0, 1)
    cols = w["columns"]
    q, _, _ = step_inputs(w, 0, len(lens) * cols, False)
    order = sorted(range(len(lens)), key=lambda s: lens[s])
    per_token = kv_bytes_per_token(w)
    # grow the sample until one pass takes about a third of a second (or the workload is whole)
    sample, spent = [], 0.0
    for s in order:
        n = lens[s]
        built = cpu_pages(w, 0, s, n)
        sample.append((s, n, built))
        t0 = time.perf_counter()
        torch_path.decode_step(q[s * cols:(s + 1) * cols], built[0], built[1], built[2], built[3], built[4], [n - cols], [cols],
                               w["page"], w["kind"])
        spent += time.perf_counter() - t0
        if spent > 0.3:
            break

    def one_pass():
        for s, n, built in sample:
            torch_path.decode_step(q[s * cols:(s + 1) * cols], built[0], built[1], built[2], built[3], built[4], [n - cols],
                                   [cols], w["page"], w["kind"])
    for _ in range(warmup):
        one_pass()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_pass()
    seconds = (time.perf_counter() - t0) / steps
    positions = sum(n for _, n, _ in sample)
    gbs = positions * per_token / seconds / 1e9
    text = (f"{len(sample)} of {len(lens)} sequences ({positions} of {sum(lens)} context positions) a step, gather + "
            f"dequantise + torch SDPA on the host, {threads} threads")
    return {"impl": "reference", "metric": "decode_attention_kv_gbps", "value": gbs, "unit": "GB/s", "n_gpus": gpus,
            "steps": steps, "warmup": warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["name"], "kv": w["kind"], "sample_per_step": text,
                       "ms_per_whole_step": sum(lens) * per_token / gbs / 1e6},
            "tokens_per_s": len(sample) * cols / seconds,
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": text},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def cpu_baseline(name, w, seconds_budget):
    """The CPU leg beside the GPU line: the same path on the host cores for about `seconds_budget` seconds."""
    probe = reference_arm(name, w, 1, 1, 0)
    steps = max(1, min(40, int(seconds_budget / max(probe["ms_per_step"] / 1e3, 1e-3))))
    return reference_arm(name, w, 1, steps, 1)["cpu_baseline"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="crit_b200")
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--only", action="store_true", help="the --workload alone: no `workloads` object for the others")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison with the CPU oracle after the timing")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--staging", default=None, choices=["tma", "cp.async"])
    ap.add_argument("--engine", default=None, choices=["mma.sync", "tcgen05", "tcgen05t", "tcgen05p", "tcgen05:single", "tcgen05:pair"], help="the attention kernel instead of the library's choice")
    ap.add_argument("--exchange", default="auto", choices=["auto", "peer", "nccl"],
                    help="how the KV-range shards' partials cross the GPUs (c3 on N > 1): stores into peer memory or NCCL's all-gather")
    ap.add_argument("--chunk", type=int, default=None, help="positions per split instead of the library's choice")
    ap.add_argument("--batch", type=int, default=None,
                    help="sequences per GPU instead of the workload's own (a small case for a profiler capture)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))

    def workload(name):
        w = dict(WORKLOADS[name])
        if args.batch:
            w["batch"], w["name"] = args.batch, w["name"] + f" [--batch {args.batch}: a reduced case]"
        w["exchange"] = args.exchange
        return w

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(reference_arm(args.workload, workload(args.workload), args.gpus, args.steps, args.warmup)), flush=True)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product has no CPU path)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    found, state = measure(args.workload, workload(args.workload), args, device, rank, world, local, True)
    line = {"metric": "decode_attention_kv_gbps", "value": found["value"], "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": found["ms_per_step"], "higher_is_better": True,
            "scaling": found["scaling"], "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": found["workload"], "kv": found["kv"], "engine": found["engine"],
                       "steps_are": found["steps_are"], "l2": found["l2"], "sharding": found["sharding"],
                       "timing": f"median of {found['timed_batches']} timed batches of {found['steps_per_batch']} graph replays"},
            "ms_per_step_min": found["ms_per_step_min"], "ms_per_step_max": found["ms_per_step_max"],
            "tokens_per_s": found["tokens_per_s"], "hbm_frac_of_8TBps": found["hbm_frac_of_8TBps"],
            "clocks": found["clocks"], "e2e": found["e2e"],
            "gpu_launches": found["gpu_launches_per_step"] * args.steps, "roofline": found["roofline"],
            "parity": found["parity"], "graph_replay": found["graph_replay"]}
    for key in ("append", "tflops"):
        if key in found:
            line[key] = found[key]
    del state
    torch.cuda.empty_cache()
    failed = found["parity"] is not None and not found["parity"]["ok"]
    if not args.only and not args.batch:
        line["workloads"] = {}
        others = [n for n in ("c3", "c5", "c4", "c2row") if n != args.workload and not (n == "c4" and world > 1)]
        for name in others:
            more, state = measure(name, workload(name), args, device, rank, world, local, False)
            del state
            torch.cuda.empty_cache()
            line["workloads"][name] = more
            failed = failed or (more["parity"] is not None and not more["parity"]["ok"])
    if rank == 0 and world == 1:
        line["cpu_baseline"] = cpu_baseline(args.workload, workload(args.workload), args.cpu_seconds)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        leave()
    if failed:
        raise SystemExit("bench.py: the step's outputs are outside the parity bounds against the CPU oracle (see `parity`)")


if __name__ == "__main__":
    main()
