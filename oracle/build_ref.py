"""Compile the reference's own CUDA for the KIVI path into ``oracle/_ref/libjacq_ref.so``.

TEST INFRASTRUCTURE ONLY. The reference sources are compiled from where they lie in the reference
checkout; nothing of them is copied into this repository. Outputs (a generated ``.cu`` dumped from
the reference's Python string, text-substituted TP=2 clones made exactly as the reference's own
``dsl_decode._materialize_tp2_local_variant`` makes them, and the shared library, which also holds
the generated-runtime templates ``kernels.cu`` / ``runtime.cu`` behind ``ref_runtime_shim.cu``) go to
``oracle/_ref/`` only, which is git-ignored.

Usage: ``python oracle/build_ref.py [--reference /path/to/jacq]``; without a reference checkout it
does nothing and reports so (a prebuilt ``oracle/_ref/libjacq_ref.so`` keeps working).
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
SNAP = "crates/jac-codegen-cuda/tests/snapshots/kernels"
TEMPLATES = "crates/jac-codegen-cuda/src/templates"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _load_source_patch(reference: Path):
    sys.path.insert(0, str(reference))
    try:
        spec = importlib.util.spec_from_file_location(
            "ref_source_patch", reference / "integrations/vllm_kivi/source_patch.py")
        mod = importlib.util.module_from_spec(spec)
        sys.modules["ref_source_patch"] = mod
        spec.loader.exec_module(mod)
        return mod
    finally:
        sys.path.pop(0)


def _tp2_clone(text: str, kind: str) -> str:
    """NH/NKV 40/8 -> 20/4 and a distinct symbol, as integrations/vllm_kivi/dsl_decode.py:267-319."""
    text = text.replace("static constexpr int NH = 40;", "static constexpr int NH = 20;")
    text = text.replace("static constexpr int NKV = 8;", "static constexpr int NKV = 4;")
    pairs = {
        "single": ('extern "C" void jac_launch(', "decode_attention_kivi_paged_kivi_flash_paged_decode"),
        "batched": ('extern "C" void jac_launch_batched(',
                    "decode_attention_kivi_paged_batched_kivi_flash_paged_decode_batched"),
        "sparse": ('extern "C" void jac_launch_sparse_retained(',
                   "decode_attention_kivi_sparse_retained_kivi_flash_sparse_retained_decode"),
    }
    sym, kern = pairs[kind]
    text = text.replace(sym, sym[:-1] + "_tp2_local(")
    text = text.replace(kern, kern + "_tp2_local")
    return text


def build(reference: Path) -> Path | None:
    if not (reference / SNAP).is_dir():
        print(f"reference checkout not found at {reference}; nothing built")
        return None
    OUT.mkdir(exist_ok=True)
    sp = _load_source_patch(reference)
    (OUT / "kivi_cache_write_hand.cu").write_text(sp.KIVI_CACHE_WRITE_SOURCE)
    snaps = {
        "single": reference / SNAP / "decode_attention_kivi_paged_library_flash.cu",
        "batched": reference / SNAP / "decode_attention_kivi_paged_batched_library_flash.cu",
        "sparse": reference / SNAP / "decode_attention_kivi_sparse_retained_library_flash.cu",
    }
    sources = [str(p) for p in snaps.values()]
    for kind, path in snaps.items():
        clone = OUT / f"{path.stem}_tp2_local.cu"
        clone.write_text(_tp2_clone(path.read_text(), kind))
        sources.append(str(clone))
    sources.append(str(HERE / "ref_writer_shim.cu"))
    sources.append(str(HERE / "ref_runtime_shim.cu"))   # includes the runtime templates from the checkout
    lib = OUT / "libjacq_ref.so"
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-O3", *ARCH, "-shared", "-Xcompiler", "-fPIC", "-I", str(OUT), "-I", str(HERE),
           "-I", str(reference / TEMPLATES), "-o", str(lib), *sources,
           "-lcublas"]
    subprocess.run(cmd, check=True)
    return lib


def find_reference() -> Path | None:
    """The reference checkout: $JACQ_REFERENCE, else a directory named `reference` beside this repository."""
    for cand in (os.environ.get("JACQ_REFERENCE"), HERE.parent.parent / "reference"):
        if cand and (Path(cand) / SNAP).is_dir():
            return Path(cand)
    return None


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None, help="reference checkout (default: $JACQ_REFERENCE or ../reference)")
    chosen = ap.parse_args().reference
    ref = Path(chosen) if chosen else find_reference()
    out = build(ref) if ref else None
    print(out if out else "skipped: no reference checkout found")
