"""Throughput of the paged KV-cache hot path on B200: KV GB/s of decode attention (and tokens/s), one JSON line.

python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2|c3|c5]
N > 1 is launched by torch.distributed.run, one rank per GPU.

A step is one pass of the hot path over one batch: the step's tokens get their KV slots through the block tables,
their keys and values are appended into the pages, and decode attention reads every sequence's whole context (split-K
partials folded by their log-sum-exps).  `value` times steps whose inputs are already in HBM (a CUDA-graph replay per
step); `e2e` times the same step fed from pinned host buffers with the outputs read back every step.  The roofline
object is about the dominant kernel (the split-K decode launch), timed alone with CUDA events in the same run.
`--impl reference` times the reference's CPU path (gather + dequantise + torch SDPA, oracle/torch_path.py) on the
host cores instead.
"""
import argparse
import json
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
    # BASELINE.json configs[1]: FP8 e4m3 KV decode, batch 64, ctx 4096, 64q/8kv x 128, page 16, pool of 20,000 pages
    "c2": dict(batch=64, ctx=4096, hq=64, hkv=8, d=128, page=16, pool=20000, kind="fp8:page", columns=1, seed=2,
               name="configs[1]: FP8 e4m3 paged decode, batch 64 x ctx 4096, 64q/8kv x 128, page 16, "
                    "scale per (page, kv head)"),
    # configs[2]: one long context, bf16, 24q/4kv x 256, page 64; the KV range is sharded over the ranks
    "c3": dict(batch=1, ctx=200000, hq=24, hkv=4, d=256, page=64, pool=3126, kind="bf16", columns=1, seed=3,
               name="configs[2]: bf16 long-context decode, batch 1 x ctx 200,000, 24q/4kv x 256, page 64"),
    # configs[4]: speculative verify, 32 sequences per GPU, 6 draft tokens, lognormal contexts, FP8
    "c5": dict(batch=32, ctx=None, hq=40, hkv=8, d=128, page=16, pool=None, kind="fp8:page", columns=6, seed=5,
               name="configs[4]: FP8 speculative verify, 32 sequences per GPU x 6 draft tokens, lognormal contexts "
                    "(median 8192, 512..65536), 40q/8kv x 128, page 16"),
    # configs[3]: chunked prefill, 4 sequences, 32,768 positions in the pages + a chunk of 2,048, bf16 (tensor-bound)
    "c4": dict(batch=4, ctx=32768 + 2048, hq=32, hkv=8, d=128, page=16, pool=None, kind="bf16", columns=2048, seed=4,
               name="configs[3]: bf16 chunked prefill, 4 sequences x (32,768 prefix + 2,048 chunk), 32q/8kv x 128, page 16"),
}


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        found = json.loads(path.read_text())
        return float(found["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, an earlier measurement on this pool)"


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
    import math
    return torch.round(torch.exp(math.log(median) + sigma * z)).clamp(lo, hi).long().tolist()


def kv_bytes_per_token(w):
    code = 1 if w["kind"].startswith("fp8") else 2
    scales = w["hkv"] * 2 * 4 / w["page"] if w["kind"] == "fp8:page" else 0
    return w["hkv"] * 2 * w["d"] * code + scales


def build_state(w, device, rank, world):
    """The workload's pages, tables and step inputs on `device` (synthetic, seeded).  Lengths count the step's own
    tokens: a sequence of context n has n - columns positions in the pages and gets `columns` more in the step."""
    import crit_b200 as pk
    g = torch.Generator(device=device).manual_seed(w["seed"] * 1000 + rank)
    cpu = torch.Generator().manual_seed(w["seed"] * 1000 + rank)
    same = torch.Generator().manual_seed(w["seed"] * 1000)       # the queries of a KV-range-sharded context: one set
    cols, page, hkv, d, hq = w["columns"], w["page"], w["hkv"], w["d"], w["hq"]
    if w["ctx"] is None:
        everyone = lognormal_lengths(w["batch"] * max(world, 8), w["seed"])
        lens = everyone[rank * w["batch"]:(rank + 1) * w["batch"]]
    elif w["batch"] == 1 and world > 1:       # one long context: contiguous 4096-position partitions over the ranks
        parts = -(-w["ctx"] // 4096)
        per = -(-parts // world)
        a, b = min(rank * per, parts) * 4096, min(min((rank + 1) * per, parts) * 4096, w["ctx"])
        lens = [max(b - a, 0)]
    else:
        lens = [w["ctx"]] * w["batch"]
    need = [-(-n // page) for n in lens]
    pool = w["pool"] or sum(need) + 64
    pool = max(pool, sum(need))
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
    # fill the contexts (without the step's own tokens), a sequence at a time
    for s, n in enumerate(lens):
        have = max(n - cols, 0)
        for a in range(0, have, 32768):
            b = min(have, a + 32768)
            keys = torch.randn(b - a, hkv, d, generator=g, device=device)
            values = torch.randn(b - a, hkv, d, generator=g, device=device)
            if w["kind"] != "bf16":      # ~1% outliers x20, as BASELINE's FP8 configs ask
                keys = torch.where(torch.rand(keys.shape, generator=g, device=device) < 0.01, keys * 20, keys)
                values = torch.where(torch.rand(values.shape, generator=g, device=device) < 0.01, values * 20, values)
            rows = torch.full((b - a,), s, dtype=torch.int64, device=device)
            slots = pk.slots_at(tables, rows, torch.arange(a, b, device=device), page, pool)
            pk.write(keys.bfloat16(), values.bfloat16(), slots, k, v, w["kind"], ks, vs)
    live = [s for s, n in enumerate(lens) if n > 0]
    tokens = len(live) * cols
    firsts = torch.tensor([lens[s] - cols for s in live], dtype=torch.int64)
    state = dict(w=w, lens=lens, live=live, tables=tables, k=k, v=v, ks=ks, vs=vs, pool=pool, tokens=tokens,
                 rows=torch.tensor(live, dtype=torch.int32, device=device),
                 starts=(torch.arange(len(live), dtype=torch.int32) * cols).to(device),
                 firsts=firsts.to(device),
                 token_rows=torch.tensor(live, dtype=torch.int64).repeat_interleave(cols).to(device),
                 positions=(firsts[:, None] + torch.arange(cols)[None, :]).reshape(-1).to(device),
                 h_q=torch.randn(max(tokens, 1), hq, d, generator=same if w["batch"] == 1 else cpu).bfloat16().pin_memory(),
                 h_k=torch.randn(max(tokens, 1), hkv, d, generator=cpu).bfloat16().pin_memory(),
                 h_v=torch.randn(max(tokens, 1), hkv, d, generator=cpu).bfloat16().pin_memory())
    # The step's inputs (q, k, v) sit in ONE pinned host buffer and one device buffer, its results (out, lse) in another
    # pair, so the end-to-end step is one copy in and one copy out (256-byte aligned parts).
    def packed(parts, pin, where):
        sizes = [(-(-(int(torch.tensor(shape).prod()) * torch.empty(0, dtype=dtype).element_size()) // 256) * 256) for shape, dtype in parts]
        raw = torch.empty(sum(sizes), dtype=torch.uint8, device=where)
        raw = raw.pin_memory() if pin else raw
        views, at = [], 0
        for (shape, dtype), size in zip(parts, sizes):
            n = int(torch.tensor(shape).prod()) * torch.empty(0, dtype=dtype).element_size()
            views.append(raw[at:at + n].view(dtype).view(*shape))
            at += size
        return raw, views
    n = max(tokens, 1)
    ins = [((n, hq, d), torch.bfloat16), ((n, hkv, d), torch.bfloat16), ((n, hkv, d), torch.bfloat16)]
    outs = [((n, hq, d), torch.bfloat16), ((n, hq), torch.float32)]
    state["h_in"], host_in = packed(ins, True, "cpu")
    state["d_in"], dev_in = packed(ins, False, device)
    for name, h, dv in zip(("q", "k", "v"), host_in, dev_in):
        h.copy_(state["h_" + name])
        state["h_" + name], state["d_" + name] = h, dv
    state["d_in"].copy_(state["h_in"])
    state["slots"] = torch.empty(n, dtype=torch.int64, device=device)
    state["d_res"], (state["out"], state["lse"]) = packed(outs, False, device)
    state["h_res"], (state["h_out"], state["h_lse"]) = packed(outs, True, "cpu")
    state["kv_bytes"] = sum(lens) * kv_bytes_per_token(w)
    state["merger"] = None
    if w["batch"] == 1 and world > 1:
        # one context over the ranks by KV range: every rank keeps the step's token rows, an empty rank sends -inf
        from crit_b200.dist import ShardMerge
        state["merger"] = ShardMerge(cols, hq, d, device, out_dtype=torch.bfloat16, exchange=w.get("exchange", "auto"))
        state["out"].zero_()
        state["lse"].fill_(float("-inf"))
    return state


def step(state, launch="both", append=True):
    """One pass of the hot path: slot mapping, append, split-K decode attention + merge.  Four kernels."""
    import crit_b200 as pk
    w = state["w"]
    if not state["live"]:
        if state["merger"] is not None and launch == "both":
            state["merged"] = state["merger"].merge(state["out"], state["lse"])
        return
    if w["columns"] > 64:        # a prompt chunk per sequence: append, then one prefill launch a sequence
        cols = w["columns"]
        if append:
            pk.slots_at(state["tables"], state["token_rows"], state["positions"], w["page"], state["pool"], out=state["slots"])
            pk.write(state["d_k"], state["d_v"], state["slots"], state["k"], state["v"], w["kind"], state["ks"], state["vs"])
        for i, s in enumerate(state["live"]):
            span = slice(i * cols, (i + 1) * cols)
            pk.prefill(state["d_q"][span], state["k"], state["v"], w["kind"], state["tables"][s], state["lens"][s] - cols,
                       w["page"], key_scales=state["ks"], value_scales=state["vs"], out=state["out"][span],
                       lse=state["lse"][span], engine=state.get("engine"))
        return
    if append:
        pk.slots_at(state["tables"], state["token_rows"], state["positions"], w["page"], state["pool"], out=state["slots"])
        pk.write(state["d_k"], state["d_v"], state["slots"], state["k"], state["v"], w["kind"], state["ks"], state["vs"])
    pk.attend(state["d_q"], state["k"], state["v"], w["kind"], state["tables"], state["rows"], state["starts"],
              state["firsts"], w["columns"], w["page"], key_scales=state["ks"], value_scales=state["vs"],
              out=state["out"], lse=state["lse"], launch=launch, staging=state.get("staging"),
              engine=state.get("engine"), chunk=state.get("chunk"))
    if state["merger"] is not None and launch == "both":
        state["merged"] = state["merger"].merge(state["out"], state["lse"])


# dram__bytes_read.sum + dram__bytes_write.sum of the decode launch, from one ncu capture per workload (profiles/): the
# captured launch's traffic over its algorithmic bytes.  Traffic grows in proportion to the KV bytes (every byte is read
# once; the writes are the partial states, a fixed number per 1,024 positions), so a launch's traffic is its algorithmic
# bytes times the ratio.  None where no capture was made.
TRAFFIC_RATIO = {("c2", None): (540.9e6 + 9.7e6) / 537.9e6,            # decode_kernel, configs[1] at full size
                 ("c3", None): (819.4e6 + 7.6e6) / 819.2e6,            # decode_kernel (TMA), configs[2] at full size
                 ("c5", "tcgen05"): (167.9e6 + 4.7e6) / 167.0e6}       # decode_tc_kernel<4>, configs[4] at 8 sequences


def traffic(args, w, state):
    ratio = TRAFFIC_RATIO.get((args.workload, state.get("engine")))
    return None if ratio is None or args.staging else ratio * state["kv_bytes"]


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


def timed(fn, steps, warmup, stream):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(steps):
        fn()
    b.record(stream)
    torch.cuda.synchronize()
    return a.elapsed_time(b) / 1e3


def cpu_reference(w, state, budget_s=20.0, threads=None):
    """The reference's CPU path on a bounded sample of the workload's sequences; returns (GB/s of KV, sample text,
    seconds, threads)."""
    from oracle import torch_path
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    cols = w["columns"]
    order = sorted(state["live"], key=lambda s: state["lens"][s])
    k, v = state["k"], state["v"]
    done_bytes, spent, used = 0, 0.0, []
    q = state["h_q"]
    for i, s in enumerate(order):
        n = state["lens"][s]
        table = state["tables"][s].cpu()
        index = table[:-(-n // w["page"])].long()
        # the sequence's pages alone, renumbered, so the host copy stays small
        kc = k.view(torch.uint8 if k.element_size() == 1 else k.dtype).index_select(0, index.to(k.device)).cpu()
        vc = v.view(torch.uint8 if v.element_size() == 1 else v.dtype).index_select(0, index.to(v.device)).cpu()
        sk = state["ks"].index_select(0, index.to(k.device)).cpu() if state["ks"] is not None else None
        sv = state["vs"].index_select(0, index.to(k.device)).cpu() if state["vs"] is not None else None
        local = torch.arange(index.numel(), dtype=torch.int32)[None]
        t0 = time.perf_counter()
        torch_path.decode_step(q[i * cols:(i + 1) * cols], kc, vc, sk, sv, local, [n - cols], [cols], w["page"], w["kind"])
        spent += time.perf_counter() - t0
        done_bytes += n * kv_bytes_per_token(w)
        used.append(s)
        if spent > budget_s:
            break
    sample = (f"{len(used)} of {len(order)} sequences ({sum(state['lens'][s] for s in used)} of "
              f"{sum(state['lens'])} context positions), gather + dequantise + torch SDPA, {threads} threads")
    return done_bytes / spent / 1e9, sample, spent, threads


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="crit_b200")
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--staging", default=None, choices=["tma", "cp.async"])
    ap.add_argument("--engine", default=None, choices=["mma.sync", "tcgen05"], help="the attention kernel instead of the library's choice")
    ap.add_argument("--exchange", default="auto", choices=["auto", "peer", "nccl"],
                    help="how the KV-range shards' partials cross the GPUs (c3 on N > 1): stores into peer memory or NCCL's all-gather")
    ap.add_argument("--chunk", type=int, default=None, help="positions per split instead of the library's choice")
    ap.add_argument("--batch", type=int, default=None,
                    help="sequences per GPU instead of the workload's own (a small case for a profiler capture)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    w = dict(WORKLOADS[args.workload])
    if args.batch:
        w["batch"], w["name"] = args.batch, w["name"] + f" [--batch {args.batch}: a reduced case]"
    w["exchange"] = args.exchange
    reference = args.impl == "reference"
    if reference and rank != 0:
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product has no CPU path)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1 and not reference:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    state = build_state(w, device, rank, world)
    # the verify workload runs on the tcgen05 engine (the library's default keeps a column's bits independent of its
    # window, which costs 1.8-2x there); --engine mma.sync measures the default
    engine = args.engine or ("tcgen05" if args.workload == "c5" else None)
    state["staging"], state["engine"], state["chunk"] = args.staging, engine, args.chunk
    torch.cuda.synchronize()
    tokens_step = state["tokens"]
    steps_are = ("slot map + KV append + one prefill launch per sequence" if w["columns"] > 64
                 else "slot map + KV append + split-K decode + merge")
    if state["merger"] is not None:
        steps_are += (" + exchange of the shards' partials (" + ("stores into peer memory" if state["merger"].peer is not None
                                                                  else "NCCL all-gather") + ") + merge of shards")
    config = {"workload": w["name"], "kv": w["kind"], "engine": engine or "library default", "steps_are": steps_are,
              "l2": "inputs larger than L2: every step reads the whole KV context "
                    f"({state['kv_bytes'] / 1e6:.1f} MB per GPU, L2 is 126 MB)",
              "sharding": "sequences per GPU, no collective" if w["batch"] > 1 else "KV range per GPU"}
    unit = "GB/s"

    if reference:
        gbs, sample, spent, threads = cpu_reference(w, state, budget_s=max(5.0, args.cpu_seconds))
        line = {"impl": "reference", "metric": "decode_attention_kv_gbps", "value": gbs, "unit": unit, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": state["kv_bytes"] / gbs / 1e6,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": config, "tokens_per_s": tokens_step / (state["kv_bytes"] / gbs / 1e9),
                "cpu_baseline": {"value": gbs, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
                "e2e": {"value": gbs, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        for _ in range(2):
            step(state)
        stream.synchronize()
        graph = None
        if not args.no_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    step(state)
            except Exception as error:          # a collective that does not capture: time eager steps instead
                print(f"[bench] step not captured ({type(error).__name__}: {error}); timing eager steps", file=sys.stderr)
                graph = None
                torch.cuda.synchronize()
        run = (lambda: step(state)) if graph is None else graph.replay

        def barrier():
            if world > 1:
                import torch.distributed as dist
                dist.barrier()
            torch.cuda.synchronize()

        barrier()
        with Clocks(local) as clocks:
            seconds = timed(run, args.steps, args.warmup, stream)
            # the dominant kernel alone (same stream, CUDA events): the split-K decode launch
            decode_s = timed(lambda: step(state, launch="decode", append=False), max(20, args.steps // 4), 3, stream)
            # the fold of the splits is a few microseconds: launched back to back from a graph, so that the launches' host
            # cost is not what is timed
            merge_fn, merge_reps = (lambda: step(state, launch="merge", append=False)), 1
            if not args.no_graph and w["columns"] <= 64:
                try:
                    merge_graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(merge_graph, stream=stream):
                        for _ in range(10):
                            step(state, launch="merge", append=False)
                    merge_fn, merge_reps = merge_graph.replay, 10
                except Exception:
                    torch.cuda.synchronize()
            merge_s = timed(merge_fn, max(20, args.steps // 4), 3, stream) / merge_reps
        barrier()

        # end to end: the step's inputs from pinned host memory, the outputs read back, every step
        def e2e_step():
            state["d_in"].copy_(state["h_in"], non_blocking=True)          # q, k, v of the step: one copy
            run()
            state["h_res"].copy_(state["d_res"], non_blocking=True)        # out and lse: one copy
            stream.synchronize()
        e2e_steps = max(20, args.steps // 2)
        e2e_s = timed(e2e_step, e2e_steps, 3, stream)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([seconds, e2e_s / e2e_steps, decode_s], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total = torch.tensor([state["kv_bytes"], tokens_step], device=device, dtype=torch.float64)
        dist.all_reduce(total)
        seconds, e2e_step_s = float(t[0]), float(t[1])
        kv_total, tokens_total = float(total[0]), float(total[1])
    else:
        e2e_step_s, kv_total, tokens_total = e2e_s / e2e_steps, float(state["kv_bytes"]), float(tokens_step)
    if rank != 0:
        graph = None
        leave()
        return
    per_step = seconds / args.steps
    peak, peak_source = peaks()
    decode_step_s = decode_s / max(20, args.steps // 4)
    achieved = state["kv_bytes"] / decode_step_s / 1e9
    line = {"metric": "decode_attention_kv_gbps", "value": kv_total / per_step / 1e9, "unit": unit, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
            "scaling": "weak" if w["batch"] > 1 else "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config, "tokens_per_s": tokens_total / per_step,
            "hbm_frac_of_8TBps": kv_total / world / per_step / 8e12,
            "clocks": clocks.summary(),
            "e2e": {"value": kv_total / e2e_step_s / 1e9, "unit": unit, "tokens_per_s": tokens_total / e2e_step_s,
                    "ms_per_step": e2e_step_s * 1e3,
                    "h2d_bytes_per_step": state["h_in"].numel(), "d2h_bytes_per_step": state["h_res"].numel()},
            "gpu_launches": (4 + (0 if state["merger"] is None else (3 if state["merger"].peer is not None else 1))) * args.steps,
            "roofline": {"bound": "hbm", "kernel": ("decode_tc_kernel (tcgen05 split-K decode over paged E4M3 KV)" if state.get("engine") == "tcgen05"
                                                   else "decode_kernel (split-K decode over paged KV)"),
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_source, "us_per_launch": decode_step_s * 1e6,
                         "merge_us_per_launch": merge_s / max(20, args.steps // 4) * 1e6,
                         "algorithmic_bytes_per_launch": state["kv_bytes"], "traffic": traffic(args, w, state)},
            "graph_replay": graph is not None}
    if w["columns"] > 64:        # a dense contraction: the roofline is the tensor cores'
        cols, hq, d = w["columns"], w["hq"], w["d"]
        pairs = sum(cols * (n - cols) + cols * (cols + 1) // 2 for n in state["lens"])
        flops = pairs * 4 * d * hq
        tensor_peak = 1414.1
        path = ROOT / "MEASURED_PEAKS.json"
        if path.exists():
            tensor_peak = float(json.loads(path.read_text())["bf16_tflops_sustained"])
        tf = flops / decode_step_s / 1e12
        line["tflops"] = flops / per_step / 1e12
        line["gpu_launches"] = (2 + len(state["live"])) * args.steps
        line["roofline"] = {"bound": "tensor", "kernel": ("prefill_kernel (m16n8k16 chunked prefill over paged KV)" if args.engine == "mma.sync"
                                       else "prefill_tc_kernel (tcgen05 chunked prefill over paged KV)"), "achieved": tf,
                            "peak": tensor_peak, "unit": "TFLOP/s", "frac": tf / tensor_peak,
                            "peak_source": "measured (MEASURED_PEAKS.json bf16_tflops_sustained)" if path.exists() else "fallback",
                            "us_per_launch": decode_step_s * 1e6 / len(state["live"]), "algorithmic_flops_per_step": flops,
                            "traffic": None}
    if world == 1:
        gbs, sample, spent, threads = cpu_reference(w, state, budget_s=args.cpu_seconds)
        line["cpu_baseline"] = {"value": gbs, "unit": unit, "cores": threads, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)
    if world > 1:
        graph = None
        leave()


if __name__ == "__main__":
    main()
