"""crit_b200_attend_static, the attend entry point for hosts that may not allocate device memory (an engine that plans
every device byte at load, a sandboxed plugin handed buffers but no allocator, a request path that cannot take the
device-wide synchronisation of a cudaMalloc): its split-K partials live in an array inside the library instead of a
caller's workspace.  Called through the C ABI, twice in a row over the same shared scratch, it must give the bits the
ordinary entry point gives with a caller-owned workspace; a launch that needs more partials than the array holds is
refused with its own error and launches nothing.  Collected last, so a failure here stops no other test."""
import ctypes
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu


def _params(pk, cache, q, out, lse, rows, starts, firsts, columns, chunk, workspace=None, **more):
    from helpers import attend_params
    return attend_params(cache, q, out, lse, rows, starts, firsts, columns, chunk, workspace=workspace, **more)


@pytest.mark.parametrize("kind", ["bf16", "fp8:page"])
def test_the_static_scratch_entry_point_gives_the_ordinary_ones_bits_twice_in_a_row(kind):
    import crit_b200 as pk
    from crit_b200 import _lib
    from helpers import Cache, queries
    lib = _lib.load()
    cache = Cache(kind, 4, 128, 128, 16, [700, 300, 2100, 40], spare=8)
    rows, starts, columns = [0, 1, 2, 3], [0, 4, 8, 12], 4
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for turn, chunk in enumerate((128, 256)):              # the second call finds the first call's partials in the array
        firsts = [690 - turn, 290, 2090 - 7 * turn, 30]
        q = queries(16, 24, 128, 5 + turn)
        want, want_lse = torch.zeros(16, 24, 128, dtype=torch.bfloat16, device="cuda"), torch.zeros(16, 24, device="cuda")
        got, got_lse = torch.zeros_like(want), torch.zeros_like(want_lse)
        splits = -(-cache.tables.shape[1] * 16 // chunk)
        space = torch.empty(pk.workspace_floats(16, 24, splits, 128), device="cuda")
        p, held = _params(pk, cache, q, want, want_lse, rows, starts, firsts, columns, chunk, workspace=space)
        assert lib.crit_b200_attend(ctypes.byref(p), stream) == 0
        p, held2 = _params(pk, cache, q, got, got_lse, rows, starts, firsts, columns, chunk)     # no workspace at all
        gc.collect()            # (tensors other tests left behind go now, not during the call)
        before = torch.cuda.memory_allocated()
        assert lib.crit_b200_attend_static(ctypes.byref(p), stream) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() <= before          # torch's allocator gave the call nothing
        torch.testing.assert_close(got.float(), want.float(), atol=0, rtol=0)
        torch.testing.assert_close(got_lse, want_lse, atol=0, rtol=0)
        assert want.float().abs().sum() > 0
    # more partials than the array holds: refused by name, nothing launched
    p, held = _params(pk, cache, q, got, got_lse, rows, starts, firsts, columns, 16)
    p.partial_rows = 1 << 20
    code = lib.crit_b200_attend_static(ctypes.byref(p), stream)
    assert code == -5 and b"16 MiB" in lib.crit_b200_error(code)
    # sizes whose product passes 64 bits are refused too, not wrapped under the limit
    p.partial_rows, p.max_splits = (1 << 31) - 1, (1 << 31) - 1
    assert lib.crit_b200_attend_static(ctypes.byref(p), stream) == -5


def test_the_static_scratch_holds_exactly_its_stated_floats():
    """The last launch that fits (its partials packed by offsets, so the count of partial rows is the caller's to
    state) passes with the ordinary entry point's bits; one partial row more is refused."""
    import crit_b200 as pk
    from crit_b200 import _lib
    from helpers import Cache, queries
    lib = _lib.load()
    cache = Cache("bf16", 4, 128, 128, 16, [700, 300, 2100, 40], spare=8)
    rows, starts, columns, chunk = [0, 1, 2, 3], [0, 4, 8, 12], 4, 256
    firsts = [690, 290, 2090, 30]
    splits = -(-cache.tables.shape[1] * 16 // chunk)
    per_row = 24 * splits * 130
    most = (4 * 1024 * 1024) // per_row                  # partial rows the array holds at this geometry
    assert most >= 16
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    q = queries(16, 24, 128, 8)
    want, want_lse = torch.zeros(16, 24, 128, dtype=torch.bfloat16, device="cuda"), torch.zeros(16, 24, device="cuda")
    got, got_lse = torch.zeros_like(want), torch.zeros_like(want_lse)
    space = torch.empty(most * per_row, device="cuda")
    p, held = _params(pk, cache, q, want, want_lse, rows, starts, firsts, columns, chunk, workspace=space,
                      offsets=[0, 4, 8, 12], partial_rows=most)
    assert lib.crit_b200_attend(ctypes.byref(p), stream) == 0
    p, held2 = _params(pk, cache, q, got, got_lse, rows, starts, firsts, columns, chunk, offsets=[0, 4, 8, 12], partial_rows=most)
    assert lib.crit_b200_attend_static(ctypes.byref(p), stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, want) and torch.equal(got_lse, want_lse) and want.float().abs().sum() > 0
    p.partial_rows = most + 1
    assert lib.crit_b200_attend_static(ctypes.byref(p), stream) == -5


def test_the_static_scratch_entry_point_on_one_split_and_on_tcgen05_tiles():
    """Rows of one split never touch the scratch; with CRIT_B200_ATTEND_TCGEN05 the tcgen05 kernel's partials go
    through it: both give the ordinary entry point's bits."""
    import crit_b200 as pk
    from crit_b200 import _lib
    from helpers import Cache, queries
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    cache = Cache("fp8:page", 4, 128, 128, 16, [700, 300, 2100, 40], spare=8)
    rows, starts, columns, firsts = [0, 1, 2, 3], [0, 4, 8, 12], 4, [690, 290, 2090, 30]
    q = queries(16, 24, 128, 6)
    for chunk, flags in ((cache.tables.shape[1] * 16, 0), (256, 8)):       # one split a row; the tcgen05 kernel's flag
        want, want_lse = torch.zeros(16, 24, 128, dtype=torch.bfloat16, device="cuda"), torch.zeros(16, 24, device="cuda")
        got, got_lse = torch.zeros_like(want), torch.zeros_like(want_lse)
        splits = -(-cache.tables.shape[1] * 16 // chunk)
        space = torch.empty(max(pk.workspace_floats(16, 24, splits, 128), 4), device="cuda")
        p, held = _params(pk, cache, q, want, want_lse, rows, starts, firsts, columns, chunk, workspace=space, flags=flags)
        assert lib.crit_b200_attend(ctypes.byref(p), stream) == 0
        p, held2 = _params(pk, cache, q, got, got_lse, rows, starts, firsts, columns, chunk, flags=flags)
        assert lib.crit_b200_attend_static(ctypes.byref(p), stream) == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want) and torch.equal(got_lse, want_lse) and want.float().abs().sum() > 0, (chunk, flags)
    assert pk.status() == 0
