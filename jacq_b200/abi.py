"""Versioned description of the callable kernel surface, fail-closed.

Mirror of the reference's ``integrations/vllm_kivi/abi.py`` (constants :35-61, ``kernel_interface``
:88-122, checks :136-201). Version 1 is the reference lane (fixed geometry, 4096-token cap, the
``jac_launch*`` symbols); version 2 adds the runtime-geometry multi-sequence calls of
``include/jacq_kivi_b200.h`` and admits sm_100. The v1 constants and their checks are kept so a
caller written against the reference module behaves the same here.
"""
from __future__ import annotations

from dataclasses import dataclass

from jacq_b200.bindings import KiviDecodeBindingAbi, default_qwen32b_binding_abi
from jacq_b200.layout import KiviModelGeometry, KiviPageLayout


class UnsupportedAbiError(Exception):
    """A request or environment violates a hard ABI boundary."""


JACQ_KIVI_ABI_VERSION = 2          # 1 = the reference; 2 = + runtime-geometry v2 calls
V1_COMPATIBLE = True               # every v1 symbol keeps its order, shapes and constants

SUPPORTED_VLLM_VERSION = "0.8.5"
SUPPORTED_VLLM_SOURCE_HEAD = "3015d5634e74d59704e2b39bab0dbe2e6f86a38a"
SUPPORTED_CUDA_ARCHES = ("sm_100",)   # this library ships sm_100a code only

OLD_BLOCKS_CAP = 124
BLOCK_SIZE = 32
RESIDUAL_TOKENS = 128
MAX_SEQ_LEN = OLD_BLOCKS_CAP * BLOCK_SIZE + RESIDUAL_TOKENS  # 4096, the v1 cap

REQUIRED_TORCH_OPS = ("kivi_cache_write_dsl", "kivi_cache_write_jac_dsl", "kivi_decode_dsl")
CACHE_WRITE_KERNELS = ("hand_cuda", "jac_dsl")

V1_SYMBOLS = (
    "jac_launch", "jac_launch_tp2_local", "jac_launch_batched", "jac_launch_batched_tp2_local",
    "jac_launch_sparse_retained", "jac_launch_sparse_retained_tp2_local", "jac_launch_cache_write",
    "jac_launch_cache_write_batched", "kivi_b200_cache_write_launch", "kivi_b200_cache_write_batched_launch",
)
V2_SYMBOLS = (
    "kivi_b200_abi_version", "kivi_b200_status_string", "kivi_b200_validate_geometry", "kivi_b200_cache_write",
    "kivi_b200_decode_workspace_bytes", "kivi_b200_decode_workspace_init", "kivi_b200_decode", "kivi_b200_decode_f16", "kivi_b200_decode_noalloc", "kivi_b200_decode_sparse", "kivi_b200_gemv_f16", "kivi_b200_gemm_wait_failures", "kivi_b200_decode_wait_failures", "kivi_b200_writer_rejected_indices", "kivi_b200_decode_rejected_indices", "kivi_b200_decode_plan", "kivi_b200_decode_part_items",
    "kivi_b200_decode_step_workspace_bytes", "kivi_b200_decode_step", "kivi_b200_residual_rmsnorm",
    "kivi_b200_bias_rope", "kivi_b200_silu_mul", "kivi_b200_argmax",
    "kivi_b200_p2p_region_bytes", "kivi_b200_p2p_region_create", "kivi_b200_p2p_region_open",
    "kivi_b200_p2p_region_close", "kivi_b200_p2p_region_destroy", "kivi_b200_p2p_status",
)


def supported_geometry() -> KiviModelGeometry:
    """The one geometry the v1 symbols are compiled for."""
    return KiviModelGeometry.qwen25_coder_32b()


@dataclass(frozen=True)
class KernelCall:
    torch_op: str
    spec: str
    launch_order: tuple[str, ...] = ()

    def describe(self) -> dict[str, object]:
        return {"torch_op": self.torch_op, "spec": self.spec, "launch_order": list(self.launch_order)}


def _checked_binding(seq_len: int) -> KiviDecodeBindingAbi:
    if seq_len > MAX_SEQ_LEN:
        raise UnsupportedAbiError(
            f"seq_len {seq_len} exceeds the v1 KIVI ABI cap of {MAX_SEQ_LEN} ({OLD_BLOCKS_CAP} old pages x "
            f"{BLOCK_SIZE} tokens + {RESIDUAL_TOKENS}-token residual); use the v2 calls for longer contexts")
    return default_qwen32b_binding_abi(seq_len=seq_len)


def kernel_interface(seq_len: int = MAX_SEQ_LEN) -> dict[str, object]:
    """JSON-serialisable description of the v1 surface for one decode step."""
    abi = _checked_binding(seq_len)
    return {
        "abi_version": JACQ_KIVI_ABI_VERSION,
        "supported_vllm_version": SUPPORTED_VLLM_VERSION,
        "supported_cuda_arches": list(SUPPORTED_CUDA_ARCHES),
        "required_torch_ops": list(REQUIRED_TORCH_OPS),
        "cache_write_kernels": list(CACHE_WRITE_KERNELS),
        "seq_len": abi.seq_len,
        "old_pages": abi.old_pages,
        "kernels": [
            KernelCall("kivi_decode_dsl", "specs/kernels/decode_attention_kivi_paged.jac",
                       tuple(abi.jac_launch_order())).describe(),
            KernelCall("kivi_cache_write_jac_dsl", "specs/kernels/cache_write_kivi_paged.jac").describe(),
        ],
        "v1_symbols": list(V1_SYMBOLS),
        "v2_symbols": list(V2_SYMBOLS),
        "integrity_boundary": (
            "A description of the callable surface and nothing more: building it allocates no tensor and "
            "launches no kernel (CUDA is NOT RUN by this call). Parity and throughput of the library are "
            "established by its own GPU tests and benchmark, not by this report."
        ),
    }


def kernel_interface_v2(layout: KiviPageLayout, max_seq_len: int) -> dict[str, object]:
    """Description of the v2 surface for a runtime geometry."""
    try:
        layout.validate_for_b200_lane()
    except ValueError as exc:
        raise UnsupportedAbiError(str(exc)) from exc
    binding = KiviDecodeBindingAbi(layout, seq_len=max_seq_len)
    return {
        "abi_version": JACQ_KIVI_ABI_VERSION,
        "symbols": list(V2_SYMBOLS),
        "layout": layout.to_abi_dict(max_seq_len),
        "tensor_bindings": [b.to_dict() for b in binding.tensor_bindings()],
        "max_old_pages": binding.old_pages,
    }


def check_vllm_version(version: str, source_head: str | None = None) -> None:
    """Accept the pinned 0.8.5 release line only: `0.8.5`, `0.8.5.postN`, `.devN`, any `+local` tag; refuse
    look-alikes such as 0.8.50 or 0.8.5.1. With `source_head`, also require the pinned commit."""
    release = version.partition("+")[0].split(".")
    suffixes_ok = all(not part[:1].isdigit() for part in release[3:])
    if release[:3] != ["0", "8", "5"] or not suffixes_ok:
        raise UnsupportedAbiError(f"vLLM {version} is not the supported {SUPPORTED_VLLM_VERSION} line")
    if source_head not in (None, SUPPORTED_VLLM_SOURCE_HEAD):
        raise UnsupportedAbiError(
            f"vLLM source head {source_head[:12]}... is not the pinned {SUPPORTED_VLLM_SOURCE_HEAD[:12]}...")


def check_cuda_arch(arch: str) -> None:
    if arch not in SUPPORTED_CUDA_ARCHES:
        raise UnsupportedAbiError(f"CUDA arch {arch} is outside the built set {SUPPORTED_CUDA_ARCHES}")


def check_geometry(geometry: KiviModelGeometry) -> None:
    """v1 symbols only: the geometry they were compiled for."""
    lane = supported_geometry()
    wrong = [(a, getattr(geometry, a), getattr(lane, a)) for a in ("num_attention_heads", "num_kv_heads", "head_dim")
             if getattr(geometry, a) != getattr(lane, a)]
    if wrong:
        attr, got, want = wrong[0]
        raise UnsupportedAbiError(f"model geometry {attr}={got} does not match the v1 lane ({lane.name}: {attr}={want}); "
                                  "use the v2 calls")
