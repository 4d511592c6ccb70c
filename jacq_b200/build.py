"""Build libjacq_kivi_b200.so in-tree with nvcc for sm_100a.

``python -m jacq_b200.build`` (or ``build()``) compiles every ``csrc/*.cu`` into
``jacq_b200/_lib/libjacq_kivi_b200.so``. nvcc cross-compiles without a GPU. No fast-math: the
cache writer's scale and code arithmetic must stay IEEE to be bit-exact with the reference.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "_lib"
LIB = LIB_DIR / "libjacq_kivi_b200.so"

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default", "--expt-relaxed-constexpr",
]


# compile-time tunables that may be overridden from the environment when experimenting
TUNABLES = ("KIVI_DECODE_WARPS", "KIVI_DECODE_CTAS", "KIVI_SUB", "KIVI_QK_SPLIT", "KIVI_DECODE_TRACE")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "jacq_kivi_b200.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    LIB_DIR.mkdir(exist_ok=True)
    objs = []
    procs = []
    extra = [f"-D{name}={os.environ[name]}" for name in TUNABLES if name in os.environ]
    for src in sources():
        obj = LIB_DIR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src.name}\n{out}\n")
        failed |= proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see output above")
    subprocess.run([nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"],
                   check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
