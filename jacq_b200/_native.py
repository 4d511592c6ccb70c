"""ctypes binding of ``libjacq_kivi_b200.so`` (declarations: ``include/jacq_kivi_b200.h``).

The library is the product; there is no Python or CPU fallback. Loading fails loudly when the
shared object has not been built (``python -m jacq_b200.build``).
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int32, c_size_t, c_uint32, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libjacq_kivi_b200.so"


class NativeLibraryMissing(RuntimeError):
    pass


class KiviGeometry(ctypes.Structure):
    """``kivi_geometry`` of the header."""

    _fields_ = [(n, c_int32) for n in
                ("num_q_heads", "num_kv_heads", "head_dim", "block_size", "group_size", "residual")]


class KiviCacheStruct(ctypes.Structure):
    """``kivi_cache`` of the header."""

    _fields_ = [(n, c_void_p) for n in
                ("k_code_pages", "k_scale_pages", "k_zero_pages", "v_code_pages", "v_scale_pages",
                 "v_zero_pages", "k_residual_scratch", "v_residual_scratch")] + \
               [("num_blocks", c_int32), ("num_slots", c_int32)]


class KiviStepConfig(ctypes.Structure):
    """``kivi_step_config`` of the header (head, FFN and vocabulary counts are per rank)."""

    _fields_ = [(n, c_int32) for n in ("layers", "hidden", "num_q_heads", "num_kv_heads", "head_dim", "ffn", "vocab",
                                        "vocab_offset", "attn_bias")] + \
               [("rope_base", c_float), ("norm_eps", c_float)] + \
               [(n, c_int32) for n in ("block_size", "group_size", "residual", "tp_size", "tp_rank")]


class KiviLayerWeights(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in ("attn_norm", "qkv", "qkv_bias", "o", "ffn_norm", "gate_up", "down")]


class KiviStepWeights(ctypes.Structure):
    _fields_ = [("embed", c_void_p), ("final_norm", c_void_p), ("lm_head", c_void_p),
                ("layers", ctypes.POINTER(KiviLayerWeights))]


class KiviStepState(ctypes.Structure):
    _fields_ = [("caches", ctypes.POINTER(KiviCacheStruct)), ("block_tables", c_void_p),
                ("max_blocks_per_seq", c_int32), ("seq_lens", c_void_p), ("slot_ids", c_void_p),
                ("workspace", c_void_p), ("workspace_bytes", c_size_t)]


ALLREDUCE_F16_FN = ctypes.CFUNCTYPE(c_int, c_void_p, c_void_p, c_size_t, c_void_p)
ALLGATHER_FN = ctypes.CFUNCTYPE(c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p)


class KiviStepComm(ctypes.Structure):
    _fields_ = [("allreduce_f16", ALLREDUCE_F16_FN), ("allgather", ALLGATHER_FN), ("user", c_void_p),
                ("peer_regions", ctypes.POINTER(c_void_p)), ("region_bytes", c_size_t), ("spin_limit", c_uint32)]


P2P_HANDLE_BYTES = 64


STATUS_NAMES = {
    0: "KIVI_OK", 1: "KIVI_ERR_NULL_POINTER", 2: "KIVI_ERR_GEOMETRY", 3: "KIVI_ERR_RANGE",
    4: "KIVI_ERR_ALIGNMENT", 5: "KIVI_ERR_WORKSPACE", 6: "KIVI_ERR_CUDA", 7: "KIVI_ERR_BLOCK_TABLE",
}

_P = c_void_p
_V1_CACHE = [_P] * 8

# name -> (restype, argtypes); every symbol include/jacq_kivi_b200.h declares.
SIGNATURES: dict[str, tuple[object, list[object]]] = {
    "kivi_b200_abi_version": (c_int, []),
    "kivi_b200_status_string": (ctypes.c_char_p, [c_int]),
    "kivi_b200_validate_geometry": (c_int, [ctypes.POINTER(KiviGeometry), ctypes.POINTER(c_int)]),
    "kivi_b200_cache_write": (c_int, [ctypes.POINTER(KiviGeometry), ctypes.POINTER(KiviCacheStruct), _P, _P, _P, c_int,
                                      _P, _P, _P, c_int, c_int, c_int, _P]),
    "kivi_b200_decode_workspace_bytes": (c_size_t, [ctypes.POINTER(KiviGeometry), c_int, c_int]),
    "kivi_b200_decode_workspace_init": (c_int, [_P, c_size_t, _P]),
    "kivi_b200_decode": (c_int, [ctypes.POINTER(KiviGeometry), ctypes.POINTER(KiviCacheStruct), _P, _P, c_int, _P, _P,
                                 c_int, c_int, _P, _P, c_size_t, _P]),
    "kivi_b200_decode_f16": (c_int, [ctypes.POINTER(KiviGeometry), ctypes.POINTER(KiviCacheStruct), _P, _P, c_int, _P, _P,
                                     c_int, c_int, _P, _P, c_size_t, _P]),
    "kivi_b200_decode_sparse": (c_int, [ctypes.POINTER(KiviGeometry), ctypes.POINTER(KiviCacheStruct), _P, _P, c_int, _P, _P,
                                        _P, c_int, c_int, _P, _P, c_size_t, _P]),
    "kivi_b200_decode_noalloc": (c_int, [ctypes.POINTER(KiviGeometry), ctypes.POINTER(KiviCacheStruct), _P, _P, c_int, _P,
                                         _P, c_int, c_int, _P, _P]),
    "kivi_b200_gemv_f16": (c_int, [_P, _P, _P, _P, c_int, c_int, c_int, _P]),
    "kivi_b200_gemm_wait_failures": (c_int, [ctypes.POINTER(c_uint32)]),
    "kivi_b200_decode_wait_failures": (c_int, [ctypes.POINTER(c_uint32)]),
    "kivi_b200_writer_rejected_indices": (c_int, [ctypes.POINTER(c_uint32)]),
    "kivi_b200_decode_rejected_indices": (c_int, [ctypes.POINTER(c_uint32)]),
    "kivi_b200_decode_part_items": (c_int, [ctypes.POINTER(KiviGeometry), c_int, c_int, c_int, ctypes.POINTER(c_int32)]),
    "kivi_b200_decode_plan": (c_int, [ctypes.POINTER(KiviGeometry), c_int, c_int, ctypes.POINTER(c_int32)]),
    "kivi_b200_decode_step_workspace_bytes": (c_size_t, [ctypes.POINTER(KiviStepConfig), c_int, c_int]),
    "kivi_b200_decode_step": (c_int, [ctypes.POINTER(KiviStepConfig), ctypes.POINTER(KiviStepWeights),
                                      ctypes.POINTER(KiviStepState), _P, c_int, c_int, _P, _P,
                                      ctypes.POINTER(KiviStepComm), _P]),
    "kivi_b200_p2p_region_bytes": (c_size_t, [ctypes.POINTER(KiviStepConfig), c_int]),
    "kivi_b200_p2p_region_create": (c_int, [c_size_t, ctypes.POINTER(c_void_p), _P]),
    "kivi_b200_p2p_region_open": (c_int, [_P, ctypes.POINTER(c_void_p)]),
    "kivi_b200_p2p_region_close": (c_int, [_P]),
    "kivi_b200_p2p_region_destroy": (c_int, [_P]),
    "kivi_b200_p2p_status": (c_int, [_P, ctypes.POINTER(c_uint32), _P]),
    "kivi_b200_residual_rmsnorm": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_float, _P]),
    "kivi_b200_bias_rope": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_float, _P]),
    "kivi_b200_silu_mul": (c_int, [_P, _P, c_int, c_int, _P]),
    "kivi_b200_argmax": (c_int, [_P, _P, c_int, c_int, _P, c_size_t, _P]),
    "jac_launch": (None, [_P, _P] + _V1_CACHE + [c_int, _P, _P]),
    "jac_launch_tp2_local": (None, [_P, _P] + _V1_CACHE + [c_int, _P, _P]),
    "jac_launch_batched": (None, [_P, _P, _P] + _V1_CACHE + [c_int, _P, _P]),
    "jac_launch_batched_tp2_local": (None, [_P, _P, _P] + _V1_CACHE + [c_int, _P, _P]),
    "jac_launch_sparse_retained": (None, [_P, _P] + _V1_CACHE + [c_int, c_int, _P, _P]),
    "jac_launch_sparse_retained_tp2_local": (None, [_P, _P] + _V1_CACHE + [c_int, c_int, _P, _P]),
    "jac_launch_cache_write": (None, _V1_CACHE + [_P, _P, _P, c_int, _P]),
    "jac_launch_cache_write_batched": (None, _V1_CACHE + [_P, _P, _P, c_int, c_int, _P]),
    "kivi_b200_cache_write_launch": (None, _V1_CACHE + [_P, _P, _P, _P, c_int, c_int, _P]),
    "kivi_b200_cache_write_batched_launch": (None, _V1_CACHE + [_P, _P, _P, _P, c_int, c_int, c_int, _P]),
}

_lib: ctypes.CDLL | None = None


def lib() -> ctypes.CDLL:
    """Load the shared library once and attach the prototypes."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise NativeLibraryMissing(
                f"{LIB_PATH} is missing: build it with `python -m jacq_b200.build`; "
                "there is no fallback path for the KIVI kernels")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


class KiviStatusError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        text = lib().kivi_b200_status_string(status).decode()
        super().__init__(f"{where}: {STATUS_NAMES.get(status, status)} ({text})")


def check(status: int, where: str) -> None:
    if status != 0:
        raise KiviStatusError(status, where)
