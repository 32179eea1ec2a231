"""Builds the package's one native library, crit_b200/_native/libcrit_b200.so, for sm_100a with nvcc.

python -m crit_b200.build [--force] [--verbose].  nvcc cross-compiles without a GPU; the library links cudart
statically and nothing else, so it loads on a machine without a driver (its calls then fail with a CUDA error)."""
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCES = ["abi.cu", "append.cu", "gather.cu", "decode.cu", "prefill.cu", "exchange.cu", "pager.cu"]
LIBRARY = HERE / "_native" / "libcrit_b200.so"
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
         "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


def nvcc():
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("crit_b200 needs nvcc (CUDA 12.8 or later, for sm_100a) to build its kernels")
    return found


def stale():
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    deps = list((HERE / "csrc").glob("*.cu*")) + [HERE.parent / "include" / "crit_b200.h"]
    return any(d.stat().st_mtime > built for d in deps)


def build(force=False, verbose=False):
    """Compile every source of csrc/ and link the shared library; returns its path."""
    if not force and not stale():
        return LIBRARY
    LIBRARY.parent.mkdir(exist_ok=True)
    objects = []
    procs = []
    for name in SOURCES:
        obj = LIBRARY.parent / (name + ".o")
        cmd = [nvcc(), *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", str(HERE / "csrc" / name), "-o", str(obj)]
        procs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(str(obj))
    for name, proc in procs:
        out, _ = proc.communicate()
        if verbose and out:
            print(out)
        if proc.returncode:
            raise RuntimeError(f"nvcc failed on {name}:\n{out}")
    link = [nvcc(), "-shared", "-o", str(LIBRARY), *objects, "-cudart", "static"]
    done = subprocess.run(link, capture_output=True, text=True)
    if done.returncode:
        raise RuntimeError(f"linking libcrit_b200.so failed:\n{done.stdout}{done.stderr}")
    for obj in objects:
        os.unlink(obj)
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
