"""The drop-in shown with the reference's own code: crit's plugin library loads crit_b200's two plugin folders and
finds every interface method, fact extension and pool attribute it asks of a plugin in those slots; the host forms give
the values the reference's plugins give on crit's own slot cases; and (GPU) the reference's KVPool and DeviceAttention,
unmodified, run a decode step, a verify window and a prompt row with crit_b200 passed as their `kernels=`.

The reference's Python is read from baseline/_ref/ (a git-ignored copy made by tests/reference_copy.py); the tests are
skipped where it is absent."""
import importlib
import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"

needs_reference = pytest.mark.skipif(not (REF / "core" / "python" / "crit_plugins").is_dir(),
                                     reason="no copy of the reference under baseline/_ref (tests/reference_copy.py makes it)")


def _crit_plugins():
    path = str(REF / "core" / "python")
    if path not in sys.path:
        sys.path.insert(0, path)
    import crit_plugins
    return crit_plugins


def _reference_state():
    """The reference's attention-state code as a package (its modules import each other relatively)."""
    _crit_plugins()
    if "refstate" not in sys.modules:
        pkg = types.ModuleType("refstate")
        pkg.__path__ = [str(REF / "inference" / "attention-state" / "code")]
        sys.modules["refstate"] = pkg
    return importlib.import_module("refstate.pages"), importlib.import_module("refstate.device_attention")


def _assembled(registry_root, use, options=None):
    plugins = _crit_plugins()
    registry = plugins.Registry.discover(Path(registry_root))
    return registry, plugins.assemble({"use": use, "options": options or {}}, registry, None, ())


@needs_reference
def test_crits_plugin_library_loads_the_plugin_folders_and_finds_every_interface():
    _crit_plugins()
    from crit_plugins.device import DEVICE_EXTENSIONS, POOL_EXTENSIONS, device_missing, extension_missing, pool_missing
    from crit_plugins.slots import missing
    registry, made = _assembled(ROOT / "crit_b200" / "plugins", {"kv_cache": "attention-state", "attention": "partitioned-attention"})
    try:
        assert sorted(registry.manifests) == ["attention-state", "partitioned-attention"]
        pool = made["kv_cache"].pool([0], 2, 8, 64, "cpu")
        assert pool_missing(pool) == []
        for plugin_id, slot in (("attention-state", "kv_cache"), ("partitioned-attention", "attention")):
            assert missing(slot, made[slot]) == [] and device_missing(slot, made[slot]) == []
            for fact in registry[plugin_id]["provides"]:
                if fact in DEVICE_EXTENSIONS:
                    objects = (pool,) if POOL_EXTENSIONS.get(fact) == slot else ()
                    assert extension_missing(fact, made[slot], objects) == [], fact
        assert set(made["attention"].exactness()) == {"decode", "prompt"} and isinstance(made["attention"].facts(), dict)
    finally:
        made.close()
    for folder in ("attention-state", "partitioned-attention"):
        spec = importlib.util.spec_from_file_location(f"dropin_{folder.replace('-', '_')}", ROOT / "crit_b200" / "plugins" / folder / "plugin.py")
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        assert module.memory(None, {}) == {"device": 0, "host": 0}


@needs_reference
def test_the_host_forms_give_the_references_values_on_crits_slot_cases():
    _crit_plugins()
    from crit_plugins.slots import CASES, compare
    _, ours = _assembled(ROOT / "crit_b200" / "plugins", {"kv_cache": "attention-state", "attention": "partitioned-attention"})
    torch_only = {"attention-state": {"kernels": "torch"}, "partitioned-attention": {"kernels": "torch"}}
    _, theirs = _assembled(REF / "inference", {"kv_cache": "attention-state", "attention": "partitioned-attention"}, torch_only)
    _, base = _assembled(REF / "inference", {"kv_cache": "attention-state", "attention": "softmax-attention"},
                         {"attention-state": {"kernels": "torch"}})
    try:
        for slot in ("kv_cache", "attention"):
            got = CASES[slot]({"kv_cache": ours["kv_cache"], "attention": ours["attention"]})
            for other in (theirs, base):
                want = CASES[slot]({"kv_cache": other["kv_cache"], "attention": other["attention"]})
                assert compare(got, want) is None, (slot, compare(got, want))
    finally:
        for made in (ours, theirs, base):
            made.close()


def _stored(pool, layer, oracle, torch):
    """A reference pool's pages of one layer as the oracle reads them (FP32 values [slots][hkv][dim])."""
    i = pool.layers[layer]
    found = []
    for pages, scales, mult in ((pool.k[i], pool.k_scales, pool.scale_values[i][0]), (pool.v[i], pool.v_scales, pool.scale_values[i][1])):
        dim = pages.shape[-1]
        if pool.dtype in ("bf16", "fp16"):
            found.append(pages.float().cpu().numpy().reshape(-1, pool.kv_heads, dim))
            continue
        codes = pages.view(torch.uint8).cpu().numpy().reshape(-1, pool.kv_heads, dim)
        sc = scales[i].cpu().numpy().reshape(-1, pool.kv_heads) if scales is not None else None
        found.append(oracle.dequantize(codes, pool.dtype, sc, mult, page=pool.page))
    return found


@needs_reference
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["bf16", "fp8:row", "fp8"])
@pytest.mark.parametrize("prompt_reader", ["prefill", "decode"])
def test_the_references_pool_and_attention_run_on_crit_b200_as_their_kernels(dtype, prompt_reader):
    """reserve -> write -> forward, as the model plugin drives them, on the reference's own KVPool and DeviceAttention with
    kernels=crit_b200: decode rows, a verify window of 5 and a prompt row of 100 tokens against the oracle over what the
    pool stored; the pool's codes and scales against the oracle's quantiser bit for bit."""
    import torch
    import crit_b200
    import oracle
    from helpers import assert_attention_close
    pages, device_attention = _reference_state()
    from crit_plugins import StepBatch
    pool = pages.KVPool([0, 1], 4, 128, 16 * 400, "cuda", dtype, page=16, kernels=crit_b200)
    attention = device_attention.DeviceAttention(crit_b200, "auto", device="cuda", reader="split", prompt_reader=prompt_reader)
    if dtype == "fp8":
        pool.set_scales(1, 0.05, 0.07)
    g = torch.Generator().manual_seed(3)

    def step(rows):
        batch = StepBatch.build(rows, "cuda")
        slots = pool.reserve(batch)
        keys = torch.randn(batch.tokens, 4, 128, generator=g).bfloat16().cuda()
        values = torch.randn(batch.tokens, 4, 128, generator=g).bfloat16().cuda()
        pool.write(1, slots, keys, values)
        return batch, keys
    lens = {"a": 700, "b": 64, "c": 1, "d": 2100}
    for s, n in lens.items():
        pool.open(s)
        step([(s, 0, n)])
        pool.keep(s, n)
    batch, keys = step([("a", 700, 1), ("b", 64, 5), ("c", 1, 1), ("d", 2100, 100)])
    if dtype == "fp8:row":
        want_codes, want_scales = oracle.quantize_rows(keys.float().cpu().numpy(), "fp8:row")
        at = oracle.slots(np.array(pool.table("a"), np.int32), np.array([700]), 16)
        assert np.array_equal(pool.k[1].view(torch.uint8).cpu().numpy().reshape(-1, 4, 128)[at], want_codes[:1])
        assert np.array_equal(pool.k_scales[1].cpu().numpy().reshape(-1, 4)[at], want_scales[:1])
    q = torch.randn(batch.tokens, 24, 128, generator=g).bfloat16().cuda()
    out, lse = attention.forward(1, q, pool, batch, lse=True)
    torch.cuda.synchronize()
    k, v = _stored(pool, 1, oracle, torch)
    width = max(len(pool.table(s)) for s in batch.sequences)
    tables = np.full((batch.rows, width), pool.dump, np.int32)
    for r, s in enumerate(batch.sequences):
        tables[r, :len(pool.table(s))] = pool.table(s)
    counts = [batch.row(r)[2] for r in range(batch.rows)]
    want, want_lse = oracle.attend(q.float().cpu().numpy(), k, v, tables, list(range(batch.rows)), batch.starts[:-1],
                                   [batch.row(r)[3] for r in range(batch.rows)], max(counts), 16, counts=counts)
    assert_attention_close(out, lse, want, want_lse, list(range(batch.tokens)))
    assert crit_b200.status() == 0
    attention.close()


def _own_parts(**kw):
    import crit_b200
    from crit_b200.attention import DeviceAttention, PartitionedAttention
    from crit_b200.kv_state import KVStateCache
    kv = KVStateCache(page=16, kernels=crit_b200, **kw)
    return kv, PartitionedAttention(kv, {"world": 2, "page_size": 256}, DeviceAttention(device="cuda", window_engine="mma.sync"))


def _filled(pool, lens, seed=0):
    """Sequences opened and filled to their lengths through reserve -> write -> keep, crit's StepBatch driving."""
    import torch
    from crit_plugins import StepBatch
    g = torch.Generator().manual_seed(seed)
    for s, n in lens.items():
        pool.open(s)
        batch = StepBatch.build([(s, 0, n)], "cuda")
        keys = torch.randn(n, pool.kv_heads, pool.head_dim, generator=g).bfloat16().cuda()
        values = torch.randn(n, pool.kv_heads, pool.value_dim, generator=g).bfloat16().cuda()
        pool.write(0, pool.reserve(batch), keys, values)
        pool.keep(s, n)
    return g


def _oracle_rows(pool, sequences, firsts, counts, q, oracle, torch):
    k, v = _stored(pool, 0, oracle, torch)
    width = max(len(pool.table(s)) for s in sequences)
    tables = np.full((len(sequences), width), pool.dump, np.int32)
    for r, s in enumerate(sequences):
        tables[r, :len(pool.table(s))] = pool.table(s)
    starts = np.concatenate([[0], np.cumsum(counts)])[:-1]
    return oracle.attend(q.float().cpu().numpy(), k, v, tables, list(range(len(sequences))), starts, firsts, max(counts), pool.page,
                         counts=counts)


@needs_reference
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["bf16", "fp8:page"])
def test_a_round_of_crits_round_driver_runs_on_the_pool_and_the_attention(dtype):
    """bind -> start_round -> reserve(RoundBatch) -> write -> forward -> commit_round -> unbind, with crit's own RoundBatch
    (core/python/crit_plugins/device.py:636-693) at fixed device addresses: the round's slots come from the round tables on
    the device, the attention reads the bound sequences through their round slots, and a row that emitted nothing keeps
    its length."""
    import types
    import torch
    import oracle
    from helpers import assert_attention_close
    _crit_plugins()
    from crit_plugins.device import RoundBatch
    kv, attention = _own_parts(round_rows=4)
    pool = kv.pool([0], 2, 128, 16 * 64, "cuda", dtype)
    g = _filled(pool, {"a": 40, "b": 300})
    pool.bind(0, "a", 40 + 32)
    pool.bind(1, "b", 300 + 32)
    batch = RoundBatch(4, 3, "cuda")
    frontier = torch.tensor([40, 300], device="cuda")
    batch.fill(2, 3, frontier, torch.zeros(2, 4, dtype=torch.int64, device="cuda"))
    view = types.SimpleNamespace(rows=2, n_emitted=torch.tensor([2, 0], device="cuda"), frontier=torch.tensor([42, 300], device="cuda"))
    pool.start_round(view)
    slots = pool.reserve(batch)
    assert slots.shape == (8,)
    keys = torch.randn(8, 2, 128, generator=g).bfloat16().cuda()
    values = torch.randn(8, 2, 128, generator=g).bfloat16().cuda()
    pool.write(0, slots, keys, values)
    q = torch.randn(8, 8, 128, generator=g).bfloat16().cuda()
    out, lse = attention.forward(0, q, pool, batch, lse=True)
    want, want_lse = _oracle_rows(pool, ["a", "b"], [40, 300], [4, 4], q, oracle, torch)
    assert_attention_close(out, lse, want, want_lse, list(range(8)))
    pool.commit_round(view)
    assert pool.length("a") == 42 and pool.length("b") == 300
    pool.unbind(0)
    pool.unbind(1)
    assert (pool.length("a"), len(pool.table("a"))) == (42, 3) and (pool.length("b"), len(pool.table("b"))) == (300, 19)
    with pytest.raises(ValueError, match="holds no sequence"):
        pool.unbind(0)


@needs_reference
@pytest.mark.gpu
def test_a_staged_prompt_chunk_of_crits_prompt_driver_runs_on_the_pool_and_the_attention():
    """stage_prompt -> reserve(PromptBatch) -> write -> forward -> commit_prompt with crit's own PromptBatch
    (core/python/crit_plugins/device.py:696-800): a bucket of 32 tokens, 20 of them real, after 50 positions; the padding's
    slots are the dump page's and change nothing."""
    import torch
    import oracle
    from helpers import assert_attention_close
    _crit_plugins()
    from crit_plugins.device import PromptBatch
    kv, attention = _own_parts()
    pool = kv.pool([0], 2, 128, 16 * 64, "cuda", "bf16")
    g = _filled(pool, {"p": 50})
    before = pool.gather(0, "p", 50)[0].clone()
    batch = PromptBatch(64, "cuda")
    batch.fill(32, "p", 50, list(range(20)))
    pool.stage_prompt(batch)
    slots = pool.reserve(batch)
    assert slots.shape == (32,) and bool((slots[20:] == pool.dump * pool.page).all())
    keys = torch.randn(32, 2, 128, generator=g).bfloat16().cuda()
    values = torch.randn(32, 2, 128, generator=g).bfloat16().cuda()
    pool.write(0, slots, keys, values)
    q = torch.randn(32, 8, 128, generator=g).bfloat16().cuda()
    out, lse = attention.forward(0, q, pool, batch, lse=True)
    pool.commit_prompt(batch)
    assert pool.length("p") == 70 and torch.equal(pool.gather(0, "p", 50)[0], before)
    want, want_lse = _oracle_rows(pool, ["p"], [50], [20], q[:20], oracle, torch)
    assert_attention_close(out[:20], lse[:20], want, want_lse, list(range(20)))


@pytest.mark.gpu
def test_window_rows_cut_into_launches_by_the_scratch_give_the_same_bits():
    """The engine's scratch holds the partials: with one that fits a few partial rows, a step's window rows run as several
    launches (attention.launch_cuts) and give the bits of one launch."""
    import torch
    from crit_b200.attention import DeviceAttention
    from crit_b200.batch import StepBatch
    from crit_b200.kv_state import KVStateCache
    import crit_b200

    class Scratch:
        def __init__(self):
            self.taken = []

        def take(self, nbytes):
            self.taken.append(int(nbytes))
            return torch.empty(int(nbytes), dtype=torch.uint8, device="cuda")
    kv = KVStateCache(page=16, kernels=crit_b200)
    pool = kv.pool([0], 4, 128, 16 * 400, "cuda", "bf16")
    g = torch.Generator().manual_seed(5)
    lens = {"a": 700, "b": 64, "c": 1300, "d": 2100}
    rows = []
    for s, n in lens.items():
        pool.open(s)
        batch = StepBatch.build([(s, 0, n)], "cuda")
        pool.write(0, pool.reserve(batch), torch.randn(n, 4, 128, generator=g).bfloat16().cuda(), torch.randn(n, 4, 128, generator=g).bfloat16().cuda())
        pool.keep(s, n)
        rows.append((s, n, 5))
    batch = StepBatch.build(rows, "cuda")
    slots = pool.reserve(batch)
    pool.write(0, slots, torch.randn(20, 4, 128, generator=g).bfloat16().cuda(), torch.randn(20, 4, 128, generator=g).bfloat16().cuda())
    q = torch.randn(20, 24, 128, generator=g).bfloat16().cuda()
    whole = DeviceAttention(device="cuda", window_engine="mma.sync", chunk=256).forward(0, q, pool, batch)
    scratch = Scratch()
    cut = DeviceAttention(device="cuda", window_engine="mma.sync", chunk=256, scratch=scratch, kernels_mib=3)
    # 3 MiB of partials: 24 heads x 25 splits x 130 floats a partial row -> a launch holds two of the four rows' partials
    got = cut.forward(0, q, pool, batch)
    assert torch.equal(got, whole) and len(scratch.taken) == 1
    per = crit_b200.workspace_floats(1, 24, crit_b200.parts_for(pool.block_tables.shape[1] * 16, 256), 128)
    assert 5 <= (3 << 20) // 4 // per < 20
