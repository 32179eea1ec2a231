"""The CPU oracle (oracle/) against the reference's own outputs: the golden fixtures tests/golden/make_golden.py
wrote by running the reference's torch path, and the reference's E4M3 known-answer vectors."""
import numpy as np
import pytest
import torch

import oracle


def test_e4m3_encoder_matches_the_references_known_answers(golden):
    vectors = golden("e4m3_vectors.npz")
    values = vectors["bits"].view(np.float32)
    assert np.array_equal(oracle.e4m3_encode(values), vectors["codes"])


def test_e4m3_encoder_equals_torchs_on_every_boundary(golden):
    data = golden("quantize.npz")
    probes = data["probes"]
    assert np.array_equal(oracle.e4m3_encode(np.clip(probes, -448, 448)), data["probe_codes"])
    # the encoder saturates by itself too
    assert np.array_equal(oracle.e4m3_encode(probes), data["probe_codes"])
    # and a dense sweep against torch's conversion in this process
    g = torch.Generator().manual_seed(3)
    x = torch.cat([torch.randn(200000, generator=g) * s for s in (1e-3, 0.05, 1.0, 30.0, 300.0)])
    want = x.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(oracle.e4m3_encode(x.numpy()), want)


def test_e4m3_decode_round_trips_every_code():
    codes = np.arange(256, dtype=np.uint8)
    values = oracle.e4m3_decode(codes)
    want = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.isnan(values), np.isnan(want))
    keep = ~np.isnan(want)
    assert np.array_equal(values[keep], want[keep])
    assert np.array_equal(oracle.e4m3_encode(values[keep]), codes[keep] & np.where(values[keep] == 0, 0x80 | 0, 0xFF))


@pytest.mark.parametrize("kind,codes,scales", [("fp8:row", "fp8row_codes", "fp8row_scales"),
                                               ("int8", "int8_codes", "int8_scales")])
def test_row_scaled_rules_are_bit_exact(golden, kind, codes, scales):
    data = golden("quantize.npz")
    got_codes, got_scales = oracle.quantize_rows(data["x"], kind)
    assert np.array_equal(got_codes, data[codes].view(np.uint8))
    assert np.array_equal(got_scales.view(np.uint32), data[scales].view(np.uint32))
    assert got_scales[5].tolist() == [np.float32(1e-30)] * 3 and not got_codes[5].any()


def test_static_fp8_rule_is_bit_exact(golden):
    data = golden("quantize.npz")
    got, _ = oracle.quantize_rows(data["x"], "fp8", float(data["static_multiplier"]))
    assert np.array_equal(got, data["static_codes"])


def test_page_rule_on_whole_pages_is_the_row_rule_widened():
    g = torch.Generator().manual_seed(5)
    page, heads, dim, pages = 16, 2, 32, 4
    x = torch.randn(page * 3, heads, dim, generator=g).numpy()
    codes = np.zeros(((pages + 1) * page, heads, dim), np.uint8)
    scales = np.zeros((pages + 1, heads), np.float32)
    order = [2, 0, 3]
    slots = np.concatenate([np.arange(p * page, (p + 1) * page) for p in order])
    oracle.quantize_pages(x, slots, page, codes, scales)
    for i, p in enumerate(order):
        block = torch.from_numpy(x[i * page:(i + 1) * page])
        amax = block.abs().amax(dim=(0, 2))
        want_scale = (amax / torch.full_like(amax, 448.0)).clamp(min=1e-30)
        want = (block / want_scale[None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        assert np.array_equal(scales[p], want_scale.numpy())
        assert np.array_equal(codes[p * page:(p + 1) * page], want)
    assert not codes[page:2 * page].any() and not scales[1].any()


def test_page_rule_appends_grow_the_scale_and_reencode_earlier_rows():
    page, heads, dim = 8, 1, 16
    codes = np.zeros((2 * page, heads, dim), np.uint8)
    scales = np.zeros((2, heads), np.float32)
    x0 = np.full((3, heads, dim), 1.0, np.float32)
    oracle.quantize_pages(x0, np.array([8, 9, 10]), page, codes, scales)
    assert scales[1, 0] == np.float32(1.0) / np.float32(448.0)
    small = np.full((1, heads, dim), 0.5, np.float32)
    before = codes.copy()
    oracle.quantize_pages(small, np.array([11]), page, codes, scales)       # below the page's amax: nothing re-encoded
    assert scales[1, 0] == np.float32(1.0) / np.float32(448.0) and np.array_equal(before[8:11], codes[8:11])
    big = np.full((1, heads, dim), 4.0, np.float32)
    oracle.quantize_pages(big, np.array([12]), page, codes, scales)
    assert scales[1, 0] == np.float32(4.0) / np.float32(448.0)
    values = oracle.dequantize(codes, "fp8:page", scales, page=page)
    assert np.allclose(values[8:11], 1.0) and np.allclose(values[11], 0.5) and np.allclose(values[12], 4.0)
    # a negative slot ends a run and is skipped
    oracle.quantize_pages(np.ones((2, heads, dim), np.float32), np.array([-1, 0]), page, codes, scales)
    assert scales[0, 0] == np.float32(1.0) / np.float32(448.0)


def test_slots_follow_the_page_table(golden):
    data = golden("c1_full.npz")
    lens, tables = data["lens"], data["tables"]
    page = int(data["geometry"][3])
    got = [int(oracle.slots(tables[s], np.array([lens[s]]), page)[0]) for s in range(len(lens))]
    assert got == data["slots"].tolist()


def test_round_slots_match_the_references(golden):
    data = golden("round_slots.npz")
    got = oracle.round_slots(data["tables"], data["capacity"], data["slot"], data["positions"], int(data["page"]),
                             int(data["dump"]))
    assert np.array_equal(got, data["slots"])


def _c1_inputs(data):
    """Config 1's tensors: stored in the small fixture, regenerated from the seed (and checked) for the full one."""
    import math
    hq, hkv, d, page, pool_pages, seed = (int(x) for x in data["geometry"])
    lens = data["lens"].tolist()
    if "q" in data:
        keys = [data[f"k{s}"] for s in range(len(lens))]
        values = [data[f"v{s}"] for s in range(len(lens))]
        return lens, keys, values, data["new_k"], data["new_v"], data["q"]
    g = torch.Generator().manual_seed(seed)
    assert torch.randint(64, 1025, (4,), generator=g).tolist() == lens
    torch.randperm(pool_pages, generator=g)
    keys = [torch.randn(n, hkv, d, generator=g) for n in lens]
    values = [torch.randn(n, hkv, d, generator=g) for n in lens]
    new_k = torch.randn(len(lens), hkv, d, generator=g)
    new_v = torch.randn(len(lens), hkv, d, generator=g)
    q = torch.randn(len(lens), hq, d, generator=g)
    checksum = [float(q.double().sum()), float(sum(k.double().sum() for k in keys)),
                float(sum(v.double().sum() for v in values))]
    assert np.allclose(checksum, data["checksum"], rtol=0, atol=1e-9), "torch's generator drifted from the fixture's"
    return lens, [k.numpy() for k in keys], [v.numpy() for v in values], new_k.numpy(), new_v.numpy(), q.numpy()


@pytest.mark.parametrize("name", ["c1_small.npz", "c1_full.npz"])
def test_decode_step_matches_the_references_torch_paths(golden, name):
    data = golden(name)
    hq, hkv, d, page, pool_pages, _ = (int(x) for x in data["geometry"])
    lens, keys, values, new_k, new_v, q = _c1_inputs(data)
    tables = data["tables"]
    k = np.zeros(((pool_pages + 1) * page, hkv, d), np.float32)
    v = np.zeros_like(k)
    for s, n in enumerate(lens):
        at = oracle.slots(tables[s], np.arange(n), page)
        k[at], v[at] = keys[s], values[s]
    k[data["slots"]], v[data["slots"]] = new_k, new_v
    width = tables.shape[1]
    padded = np.where(tables < 0, pool_pages, tables)
    out, lse = oracle.attend(q, k, v, padded, np.arange(len(lens)), np.arange(len(lens)), np.array(lens), 1, page)
    assert width * page >= max(lens) + 1
    np.testing.assert_allclose(out, data["out"], atol=2e-5, rtol=1e-5)
    np.testing.assert_allclose(lse, data["lse"], atol=2e-5, rtol=1e-5)
    np.testing.assert_allclose(out, data["out_sdpa"], atol=2e-5, rtol=1e-5)
    np.testing.assert_allclose(out, data["out_windows"], atol=2e-5, rtol=1e-5)
    np.testing.assert_allclose(lse, data["lse_windows"], atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("name,count", [("verify", 6), ("chunk", 40)])
def test_verify_window_and_prompt_chunk_over_fp8_rows(golden, name, count):
    data = golden("verify_fp8row.npz")
    hq, hkv, d, page, n = (int(x) for x in data["geometry"])
    table = data[f"{name}_table"]
    k_codes = data["k_codes"].reshape(-1, hkv, d).copy()
    v_codes = data["v_codes"].reshape(-1, hkv, d).copy()
    k_scales = data["k_scales"].reshape(-1, hkv).copy()
    v_scales = data["v_scales"].reshape(-1, hkv).copy()
    # the stored context equals the oracle's own encoding of what was written
    at = oracle.slots(table, np.arange(n), page)
    codes, scales = oracle.quantize_rows(data["k0"], "fp8:row")
    assert np.array_equal(k_codes[at], codes) and np.array_equal(k_scales[at], scales)
    # write the window's rows as the reference did, then attend
    new = oracle.slots(table, np.arange(n, n + count), page)
    for store, scale_store, rows in ((k_codes, k_scales, data[f"{name}_k"]), (v_codes, v_scales, data[f"{name}_v"])):
        store[new], scale_store[new] = oracle.quantize_rows(rows, "fp8:row")
    k = oracle.dequantize(k_codes, "fp8:row", k_scales)
    v = oracle.dequantize(v_codes, "fp8:row", v_scales)
    # the reference's torch paths round the dequantised rows to bf16 (its compute dtype) before multiplying
    k16 = torch.from_numpy(k).bfloat16().float().numpy()
    v16 = torch.from_numpy(v).bfloat16().float().numpy()
    out, lse = oracle.attend(data[f"{name}_q"], k16, v16, table, [0], [0], [n], count, page)
    np.testing.assert_allclose(out, data[f"{name}_out"], atol=1e-2, rtol=1e-2)      # the reference's output is bf16
    np.testing.assert_allclose(lse, data[f"{name}_lse"], atol=2e-5, rtol=1e-5)
    np.testing.assert_allclose(out, data[f"{name}_out_sdpa"], atol=2e-2, rtol=2e-2)
    # windows_torch reads rows_at (FP32 dequantised, no bf16 rounding)
    out32, lse32 = oracle.attend(data[f"{name}_q"], k, v, table, [0], [0], [n], count, page)
    np.testing.assert_allclose(lse32, data[f"{name}_lse_windows"], atol=2e-5, rtol=1e-5)
    np.testing.assert_allclose(out32, data[f"{name}_out_windows"], atol=1e-2, rtol=1e-2)


def test_shard_partials_merge_to_the_whole(golden):
    data = golden("c1_small.npz")
    hq, hkv, d, page, pool_pages, _ = (int(x) for x in data["geometry"])
    lens, keys, values, new_k, new_v, q = _c1_inputs(data)
    tables = np.where(data["tables"] < 0, pool_pages, data["tables"])
    k = np.zeros(((pool_pages + 1) * page, hkv, d), np.float32)
    v = np.zeros_like(k)
    for s, n in enumerate(lens):
        at = oracle.slots(tables[s], np.arange(n), page)
        k[at], v[at] = keys[s], values[s]
    k[data["slots"]], v[data["slots"]] = new_k, new_v
    meta = (np.arange(len(lens)), np.arange(len(lens)), np.array(lens), 1, page)
    bounds = [0, 8, 8, 20, 1 << 40]           # an empty shard among them
    parts = [oracle.attend(q, k, v, tables, *meta, lo=a, hi=b) for a, b in zip(bounds[:-1], bounds[1:])]
    out, lse = oracle.merge([p[0] for p in parts], [p[1] for p in parts])
    np.testing.assert_allclose(out, data["out"], atol=2e-5, rtol=1e-5)
    np.testing.assert_allclose(lse, data["lse"], atol=2e-5, rtol=1e-5)


def test_merge_matches_the_references(golden):
    data = golden("merge.npz")
    out, lse = oracle.merge(data["outs"], data["lses"])
    np.testing.assert_allclose(out, data["out"], atol=1e-6, rtol=1e-5)
    assert np.array_equal(np.isneginf(lse), np.isneginf(data["lse"]))
    keep = ~np.isneginf(lse)
    np.testing.assert_allclose(lse[keep], data["lse"][keep], atol=1e-6, rtol=1e-6)
    assert not out[4, 1].any() and np.isneginf(lse[4, 1])


def test_merge_matches_the_host_forms_partials(golden):
    host = golden("merge_host.json")
    for world, found in host["worlds"].items():
        outs = np.array([p[0] for p in found["partials"]], np.float32)
        lses = np.array([p[1] if p[1] is not None else -np.inf for p in found["partials"]], np.float32)
        out, lse = oracle.merge(outs[:, None, :], lses[:, None])
        np.testing.assert_allclose(out[0], found["merged"][0], atol=1e-5)
        assert abs(float(lse[0]) - found["merged"][1]) < 1e-5


def test_fold_in_split_order_equals_the_merge():
    g = np.random.default_rng(0)
    parts, dv = 6, 8
    m = g.normal(size=parts).astype(np.float32) * 3
    l = g.uniform(0.5, 4, size=parts).astype(np.float32)
    o = g.normal(size=(parts, dv)).astype(np.float32)
    m[2] = -np.inf
    l[2] = 0
    o[2] = 0
    out, lse = oracle.fold(o * l[:, None], m, l)             # po is unnormalised: o * l
    lses = np.where(l > 0, m + np.log(np.maximum(l, 1e-30)), -np.inf).astype(np.float32)
    want, want_lse = oracle.merge(o[:, None, :], lses[:, None])
    np.testing.assert_allclose(out, want[0], atol=1e-5)
    assert abs(lse - float(want_lse[0])) < 1e-5


def test_tree_windows_match_the_references_torch_path(golden):
    """Draft trees (parents per token): the oracle against the reference's own torch windows on bf16 pages
    (tests/golden/make_golden.py: tree_windows)."""
    import oracle
    f = golden("tree_bf16.npz")
    hq, hkv, d, page = (int(x) for x in f["geometry"])
    k = f["k_pages"].reshape(-1, hkv, d)
    v = f["v_pages"].reshape(-1, hkv, d)
    out, lse = oracle.attend_tree(f["q"], k, v, f["tables"], [0, 1], f["starts"], f["firsts"], 7, page, f["parents"],
                                  counts=f["counts"])
    assert np.abs(out - f["out"]).max() <= 8e-3          # the reference's outputs are bf16
    assert np.abs(lse - f["lse"]).max() <= 2e-5
    # a chain (parent = the column before) is the plain causal window
    chain = np.array([-1, 0, 1, 2, 3, 4, 5, -1, 0, 1, 2, 3], np.int32)
    a, la = oracle.attend_tree(f["q"], k, v, f["tables"], [0, 1], f["starts"], f["firsts"], 7, page, chain, counts=f["counts"])
    b, lb = oracle.attend(f["q"], k, v, f["tables"], [0, 1], f["starts"], f["firsts"], 7, page, counts=f["counts"])
    assert np.array_equal(a, b) and np.array_equal(la, lb)


@pytest.mark.parametrize("case", ["sliding", "sinks", "all"])
def test_sliding_windows_and_sinks_match_the_references_torch_path(golden, case):
    """A sliding window of 24 positions, a sink logit a head, and both over a draft tree: the oracle against the
    reference's own torch windows (tests/golden/make_golden.py: tree_windows)."""
    import oracle
    f = golden("tree_bf16.npz")
    hq, hkv, d, page = (int(x) for x in f["geometry"])
    k, v = f["k_pages"].reshape(-1, hkv, d), f["v_pages"].reshape(-1, hkv, d)
    out, lse = oracle.attend_tree(f["q"], k, v, f["tables"], [0, 1], f["starts"], f["firsts"], 7, page,
                                  f["parents"] if case == "all" else None, counts=f["counts"],
                                  sinks=f["sinks"] if case != "sliding" else None,
                                  sliding=int(f["sliding"]) if case != "sinks" else 0)
    assert np.abs(out - f["out_" + case]).max() <= 8e-3          # the reference's outputs are bf16
    assert np.abs(lse - f["lse_" + case]).max() <= 2e-5


def test_block_lists_match_the_references_torch_path(golden):
    """Each token sees only its listed KV blocks of 16 positions (tests/golden/make_golden.py: tree_windows)."""
    import oracle
    f = golden("tree_bf16.npz")
    hq, hkv, d, page = (int(x) for x in f["geometry"])
    k, v = f["k_pages"].reshape(-1, hkv, d), f["v_pages"].reshape(-1, hkv, d)
    out, lse = oracle.attend_tree(f["q"], k, v, f["tables"], [0, 1], f["starts"], f["firsts"], 7, page, None,
                                  counts=f["counts"], blocks=f["blocks"], block_size=16)
    assert np.abs(out - f["out_blocks"]).max() <= 8e-3
    assert np.abs(lse - f["lse_blocks"]).max() <= 2e-5


def test_a_fresh_prompt_chunk_matches_the_references_torch_path(golden):
    """A prompt chunk over fp8:row pages whose own positions are read from the 16-bit rows as given (the reference pool's
    fresh buffer): the oracle over the stored pages with the chunk's slots replaced by those rows."""
    import oracle
    f = golden("fresh_fp8row.npz")
    hq, hkv, d, page, n, count = (int(x) for x in f["geometry"])
    k = oracle.dequantize(f["k_codes"].reshape(-1, hkv, d), "fp8:row", f["k_scales"].reshape(-1, hkv), page=page)
    v = oracle.dequantize(f["v_codes"].reshape(-1, hkv, d), "fp8:row", f["v_scales"].reshape(-1, hkv), page=page)
    plain, _ = oracle.attend(f["q"], k, v, f["table"], [0], [0], [n], count, page)
    k[f["slots"]], v[f["slots"]] = f["k1"], f["v1"]
    out, lse = oracle.attend(f["q"], k, v, f["table"], [0], [0], [n], count, page)
    # (the reference's prompt rows gather their keys into bf16 before the SDPA: its lse carries that rounding)
    assert np.abs(out - f["out"]).max() <= 8e-3 and np.abs(lse - f["lse"]).max() <= 2e-3
    assert np.abs(plain - f["out"]).max() > np.abs(out - f["out"]).max()         # the pages alone are further away
