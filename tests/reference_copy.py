"""Copies the parts of a checkout of the reference (crit 0.21.0) that the drop-in tests import to baseline/_ref/, which
is git-ignored: the reference's sources never enter this repository's history, but the copy travels with the working
tree to a machine that has no checkout of the reference.

    python tests/reference_copy.py /path/to/reference      (or CRIT_REFERENCE=/path/to/reference)

What is copied: the two plugins this library stands in for (inference/attention-state, inference/partitioned-attention),
the base attention plugin they are compared with (inference/base/softmax-attention), crit's plugin library
(core/python/crit_plugins) and the kernel package the reference loads on a GPU (kernels/techniques/attention/
paged-kv-attention with kernels/crit_kernels and kernels/core), unmodified.
"""
import os
import shutil
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
TARGET = ROOT / "baseline" / "_ref"
PARTS = ["inference/attention-state", "inference/partitioned-attention", "inference/base/softmax-attention",
         "core/python/crit_plugins", "kernels/techniques/attention/paged-kv-attention", "kernels/crit_kernels", "kernels/core",
         "pyproject.toml"]


def copy(reference, target=TARGET):
    reference = Path(reference)
    if not (reference / "core" / "python" / "crit_plugins").is_dir():
        raise SystemExit(f"{reference} is not a checkout of the reference (no core/python/crit_plugins)")
    if target.exists():
        shutil.rmtree(target)
    skip = shutil.ignore_patterns("__pycache__", "*.pyc", "*.so", "build", ".git")
    for part in PARTS:
        src, dst = reference / part, target / part
        dst.parent.mkdir(parents=True, exist_ok=True)
        if src.is_dir():
            shutil.copytree(src, dst, ignore=skip)
        elif src.exists():
            shutil.copy2(src, dst)
    return target


def find():
    """A checkout of the reference: CRIT_REFERENCE, or a folder named `reference` beside this repository."""
    given = os.environ.get("CRIT_REFERENCE")
    for candidate in ([Path(given)] if given else []) + [ROOT.parent / "reference"]:
        if (candidate / "core" / "python" / "crit_plugins").is_dir():
            return candidate
    return None


if __name__ == "__main__":
    where = sys.argv[1] if len(sys.argv) > 1 else find()
    if where is None:
        raise SystemExit("usage: python tests/reference_copy.py /path/to/reference")
    print(copy(where))
