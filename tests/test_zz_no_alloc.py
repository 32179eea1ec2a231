"""crit_b200_attend_static, the attend entry point for hosts that may not allocate device memory (an engine that plans
every device byte at load, a sandboxed plugin handed buffers but no allocator, a request path that cannot take the
device-wide synchronisation of a cudaMalloc): its split-K partials live in an array inside the library instead of a
caller's workspace.  Called through the C ABI, twice in a row over the same shared scratch, it must give the bits the
ordinary entry point gives with a caller-owned workspace; a launch that needs more partials than the array holds is
refused with its own error and launches nothing.  Collected last, so a failure here stops no other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _params(pk, cache, q, out, lse, rows, starts, firsts, columns, chunk, workspace=None):
    """The parameter block of include/crit_b200.h for one launch, filled as crit_b200.attend fills it."""
    from crit_b200 import _lib
    dev = q.device
    i32 = dict(dtype=torch.int32, device=dev)
    held = dict(rows=torch.tensor(rows, **i32), starts=torch.tensor(starts, **i32),
                firsts=torch.tensor(firsts, dtype=torch.int64, device=dev))
    T, hq, d = q.shape
    positions = cache.tables.shape[1] * cache.page
    p = _lib.AttendParams()
    p.q, p.out, p.lse = q.data_ptr(), out.data_ptr(), lse.data_ptr()
    p.key_pages, p.value_pages = cache.k.data_ptr(), cache.v.data_ptr()
    if cache.ks is not None:
        p.key_scales, p.value_scales = cache.ks.data_ptr(), cache.vs.data_ptr()
    p.tables, p.rows, p.starts, p.firsts = (cache.tables.data_ptr(), held["rows"].data_ptr(), held["starts"].data_ptr(),
                                            held["firsts"].data_ptr())
    p.q_stride_token, p.q_stride_head = q.stride(0), q.stride(1)
    p.out_stride_token, p.out_stride_head = out.stride(0), out.stride(1)
    p.table_stride = cache.tables.stride(0)
    p.n_rows, p.columns, p.partial_rows = len(rows), columns, len(rows) * columns
    p.q_heads, p.kv_heads, p.head_dim, p.value_dim, p.page = hq, cache.hkv, d, cache.dv, cache.page
    p.kind, p.page_dtype, p.q_dtype = pk.KINDS[cache.kind], _lib.DTYPE_BF16, _lib.DTYPE_BF16
    p.chunk, p.max_splits = chunk, -(-positions // chunk)
    p.slots = cache.k.numel() // (cache.hkv * d)
    p.scale = d ** -0.5
    p.key_multiplier, p.value_multiplier = cache.multipliers
    if workspace is not None:
        p.workspace, p.workspace_floats = workspace.data_ptr(), workspace.numel()
    return p, held


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
        before = torch.cuda.memory_allocated()
        assert lib.crit_b200_attend_static(ctypes.byref(p), stream) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        torch.testing.assert_close(got.float(), want.float(), atol=0, rtol=0)
        torch.testing.assert_close(got_lse, want_lse, atol=0, rtol=0)
        assert want.float().abs().sum() > 0
    # more partials than the array holds: refused by name, nothing launched
    p, held = _params(pk, cache, q, got, got_lse, rows, starts, firsts, columns, 16)
    p.partial_rows = 1 << 20
    code = lib.crit_b200_attend_static(ctypes.byref(p), stream)
    assert code == -5 and b"16 MiB" in lib.crit_b200_error(code)
