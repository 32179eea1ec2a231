"""The C-ABI library loads without a GPU and exports every symbol include/crit_b200.h declares, with parameter blocks
of the sizes the Python binding expects (no compute call is made here)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from crit_b200 import _lib, build
    build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported(lib):
    from crit_b200 import _lib
    header = (ROOT / "include" / "crit_b200.h").read_text()
    declared = set(re.findall(r"^(?:int|int32_t|int64_t|const char\*|void\*|void)\s+(crit_b200_\w+)\s*\(", header, flags=re.M))
    assert len(declared) >= 13
    assert declared == set(_lib.SYMBOLS), declared ^ set(_lib.SYMBOLS)
    raw = ctypes.CDLL(str(_lib.LIBRARY))
    for name in declared:
        assert getattr(raw, name) is not None


def test_parameter_blocks_have_the_headers_sizes(lib):
    from crit_b200 import _lib
    assert lib.crit_b200_abi_version() == _lib.ABI_VERSION
    for which, struct in enumerate(_lib.STRUCTS):
        assert lib.crit_b200_params_size(which) == ctypes.sizeof(struct), struct.__name__
    assert lib.crit_b200_params_size(99) < 0


def test_errors_have_names(lib):
    for code in (0, -1, -2, -3, -4):
        assert lib.crit_b200_error(code)
    assert b"no kernel" in lib.crit_b200_error(-2)


def test_bad_parameters_are_refused_before_any_launch(lib):
    from crit_b200 import _lib
    p = _lib.AttendParams()
    assert lib.crit_b200_attend(ctypes.byref(p), None) == -1
    assert lib.crit_b200_attend(None, None) == -1
    a = _lib.AppendParams()
    a.tokens = 3
    assert lib.crit_b200_append(ctypes.byref(a), None) == -1
    a.tokens = 0
    assert lib.crit_b200_append(ctypes.byref(a), None) == 0


def test_the_product_has_no_cpu_path():
    import torch
    import crit_b200 as pk
    q = torch.zeros(1, 2, 64, dtype=torch.bfloat16)
    pages = torch.zeros(2, 16, 1, 64, dtype=torch.bfloat16)
    i32 = torch.zeros(1, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA devices only"):
        pk.attend(q, pages, pages, "bf16", torch.zeros(1, 2, dtype=torch.int32), i32, i32, torch.zeros(1, dtype=torch.int64), 1, 16)
    with pytest.raises(RuntimeError, match="CUDA devices only"):
        pk.write(torch.zeros(1, 1, 64), torch.zeros(1, 1, 64), torch.zeros(1, dtype=torch.int64), pages, pages, "bf16")
    from crit_b200.pool import KVPool
    pool = KVPool([0], 1, 64, 64, "cpu")
    with pytest.raises(RuntimeError, match="no CPU or torch path"):
        pool.write(0, torch.zeros(1, dtype=torch.int64), torch.zeros(1, 1, 64), torch.zeros(1, 1, 64))


def test_nothing_in_the_package_imports_the_oracle():
    for path in (ROOT / "crit_b200").rglob("*.py"):
        text = path.read_text()
        assert "import oracle" not in text and "from oracle" not in text, path
    for path in (ROOT / "crit_b200" / "csrc").glob("*"):
        assert "oracle" not in path.read_text(), path
