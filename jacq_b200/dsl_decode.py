"""Kernel artefact wiring for the vLLM source lane, B200 library form.

The reference's ``integrations/vllm_kivi/dsl_decode.py`` has one artefact class per generated
kernel (``DslDecodeKernelArtifact`` :27, ``...Batched...`` :150, ``...SparseRetained...`` :323,
``DslCacheWriteKernelArtifact`` :440, ``...WriteBatched...`` :568): each runs the jacq CLI
(``--emit-cuda --kernel-library --kivi-flash``), checks that the emitted CUDA is a library
translation unit defining its ``jac_launch*`` symbol, and copies it to a fixed path under the vLLM
tree's ``csrc/kivi/``, where the patched CMake lists it.

Here the kernels are prebuilt in ``libjacq_kivi_b200.so``, so the artefact that lands at each of
those paths is a thin translation unit that only includes the library's header (it defines
nothing: the ``jac_launch*`` symbols the torch-op binding declares resolve against the shared
library), plus one CMake fragment that links the library into ``_C``. The file names, the
``serving_env`` keys and the report layout are the reference's, so its flow keeps working with
``source_label`` telling the two kinds of artefact apart.
"""
from __future__ import annotations

import argparse
import json
import shutil
import sys
from dataclasses import asdict, dataclass
from pathlib import Path

from jacq_b200 import abi

B200_SOURCE = "b200-kivi-library"
HEADER_NAME = "jacq_kivi_b200.h"
CMAKE_FRAGMENT_REL = Path("csrc/kivi/jacq_kivi_b200.cmake")

# destination under the vLLM tree -> (symbols the reference's generated file would define there, env key)
KERNEL_FILES: dict[str, tuple[tuple[str, ...], str]] = {
    "csrc/kivi/decode_attention_kivi_dsl.cu": (("jac_launch",), "JAC_VLLM_KIVI_DECODE_KERNEL_CU"),
    "csrc/kivi/decode_attention_kivi_tp2_local_dsl.cu": (("jac_launch_tp2_local",), "JAC_VLLM_KIVI_DECODE_TP2_KERNEL_CU"),
    "csrc/kivi/decode_attention_kivi_batched_dsl.cu": (("jac_launch_batched",), "JAC_VLLM_KIVI_DECODE_BATCHED_KERNEL_CU"),
    "csrc/kivi/decode_attention_kivi_batched_tp2_local_dsl.cu": (("jac_launch_batched_tp2_local",),
                                                                 "JAC_VLLM_KIVI_DECODE_BATCHED_TP2_KERNEL_CU"),
    "csrc/kivi/decode_attention_kivi_sparse_retained_dsl.cu": (("jac_launch_sparse_retained",),
                                                               "JAC_VLLM_KIVI_DECODE_SPARSE_KERNEL_CU"),
    "csrc/kivi/decode_attention_kivi_sparse_retained_tp2_local_dsl.cu": (("jac_launch_sparse_retained_tp2_local",),
                                                                         "JAC_VLLM_KIVI_DECODE_SPARSE_TP2_KERNEL_CU"),
    "csrc/kivi/kivi_cache_write_dsl.cu": (("jac_launch_cache_write",), "JAC_VLLM_KIVI_CACHE_WRITE_KERNEL_CU"),
    "csrc/kivi/kivi_cache_write_batched_dsl.cu": (("jac_launch_cache_write_batched",),
                                                  "JAC_VLLM_KIVI_CACHE_WRITE_BATCHED_KERNEL_CU"),
    "csrc/kivi/kivi_cache_write.cu": (("kivi_cache_write_launch", "kivi_cache_write_batched_launch"),
                                      "JAC_VLLM_KIVI_CACHE_WRITE_HAND_KERNEL_CU"),
}


def forwarding_tu(symbols: tuple[str, ...]) -> str:
    """Text of the translation unit that stands where a generated kernel file would."""
    names = ", ".join(symbols)
    return (
        "// Library artifact for embedding in a runtime extension (B200 form).\n"
        f"// {names}: defined in libjacq_kivi_b200.so, declared in {HEADER_NAME}; this translation unit\n"
        "// defines nothing and exists so that the source list of the extension stays as it is.\n"
        f"#include \"{HEADER_NAME}\"\n"
        f"static_assert(JACQ_KIVI_B200_ABI_VERSION == {abi.JACQ_KIVI_ABI_VERSION}, \"header and integration disagree on the ABI\");\n"
    )


def cmake_fragment(library: Path) -> str:
    return (
        "# Links the prebuilt B200 KIVI kernels into the extension (include from the patched CMakeLists).\n"
        "add_library(jacq_kivi_b200 SHARED IMPORTED)\n"
        f"set_target_properties(jacq_kivi_b200 PROPERTIES IMPORTED_LOCATION \"{library}\")\n"
        "target_include_directories(_C PRIVATE ${CMAKE_CURRENT_LIST_DIR})\n"
        "target_link_libraries(_C PRIVATE jacq_kivi_b200)\n"
    )


@dataclass(frozen=True)
class B200KernelLibraryArtifact:
    """All kernel files of the vLLM lane at once (the library holds every kernel)."""
    repo_root: str
    vllm_root: str
    source_label: str = B200_SOURCE

    @property
    def repo_path(self) -> Path:
        return Path(self.repo_root)

    @property
    def vllm_path(self) -> Path:
        return Path(self.vllm_root)

    @property
    def library_path(self) -> Path:
        return self.repo_path / "jacq_b200" / "_lib" / "libjacq_kivi_b200.so"

    @property
    def header_path(self) -> Path:
        return self.repo_path / "include" / HEADER_NAME

    def report(self) -> dict[str, object]:
        env = {"JAC_VLLM_KIVI_DECODE_KERNEL_SOURCE": self.source_label,
               "JAC_VLLM_KIVI_B200_LIBRARY": str(self.library_path)}
        env.update({key: str(self.vllm_path / rel) for rel, (_, key) in KERNEL_FILES.items()})
        return {
            **asdict(self),
            "library_exists": self.library_path.exists(),
            "header_exists": self.header_path.exists(),
            "abi_version": abi.JACQ_KIVI_ABI_VERSION,
            "symbols": sorted(s for syms, _ in KERNEL_FILES.values() for s in syms),
            "kernel_files": {rel: (self.vllm_path / rel).exists() for rel in KERNEL_FILES},
            "serving_env": env,
            "integrity_boundary": (
                "This only places forwarding translation units and a link fragment in the vLLM fork. "
                "It is not a CUDA bitcheck and not a served result; parity of the library is established by its own tests."
            ),
        }

    def emit(self) -> list[Path]:
        """Write the forwarding units, the header and the CMake fragment into the vLLM tree."""
        if not self.library_path.exists():
            raise FileNotFoundError(f"{self.library_path} is missing: build it with `python -m jacq_b200.build`")
        if not self.header_path.exists():
            raise FileNotFoundError(f"missing header: {self.header_path}")
        written = []
        for rel, (symbols, _) in KERNEL_FILES.items():
            dst = self.vllm_path / rel
            dst.parent.mkdir(parents=True, exist_ok=True)
            text = forwarding_tu(symbols)
            forbidden = ("int main(", "__global__", "extern \"C\" void jac_launch")
            if any(needle in text for needle in forbidden):
                raise RuntimeError("forwarding unit would define kernel symbols")
            dst.write_text(text)
            written.append(dst)
        header_dst = self.vllm_path / "csrc" / "kivi" / HEADER_NAME
        shutil.copy2(self.header_path, header_dst)
        fragment = self.vllm_path / CMAKE_FRAGMENT_REL
        fragment.write_text(cmake_fragment(self.library_path))
        return written + [header_dst, fragment]


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--repo-root", default=str(Path(__file__).resolve().parents[1]))
    ap.add_argument("--vllm-root", required=True)
    ap.add_argument("--emit", action="store_true", help="write the forwarding units into the vLLM source tree")
    args = ap.parse_args()
    artifact = B200KernelLibraryArtifact(args.repo_root, args.vllm_root)
    if args.emit:
        for path in artifact.emit():
            print(path, file=sys.stderr)
    print(json.dumps(artifact.report(), indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
