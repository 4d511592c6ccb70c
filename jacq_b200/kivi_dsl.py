"""ABI v1 host layer: the reference's ``kivi_dsl.py`` adapter, bound to libjacq_kivi_b200.so.

Mirror of the backend stub the reference materialises into vLLM
(``integrations/vllm_kivi/source_patch.py:28-554``): same function names, argument meaning,
validation order and exception types. Where the reference calls ``torch.ops._C.kivi_*`` (C++ torch
ops that forward to ``jac_launch*`` / ``kivi_cache_write*_launch``), this module calls those C
symbols of the B200 library directly through ctypes on the current CUDA stream. One sequence per
call, reference lane geometry only (NH/NKV 40/8 or 20/4, head_dim 128, block = group = 32,
residual 128, seq_len <= 4096); the many-sequence calls are in ``jacq_b200.cache``.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Any, Mapping

import torch

from jacq_b200 import _native
from jacq_b200.bindings import CACHE_TENSORS, JAC_LAUNCH_ORDER

KIVI_CACHE_KIND = "int4_kivi_dsl_paged"
_CACHE_TENSORS = CACHE_TENSORS
OLD_BLOCKS = 124
BLOCK_SIZE = 32
RESIDUAL = 128
MAX_SEQ_LEN = OLD_BLOCKS * BLOCK_SIZE + RESIDUAL
MAX_QUERIES = 160
HD = 128
CACHE_WRITE_KERNEL_ENV = "JAC_KIVI_CACHE_WRITE_KERNEL"
_GEOMETRIES = {(40, 8): "", (20, 4): "_tp2_local"}


_WRITER_ALIASES = {"hand_cuda": ("hand_cuda", "hand", "cuda", "legacy"), "jac_dsl": ("jac_dsl", "jac", "dsl")}
_CODE_TENSORS = ("K_CODE_PAGES", "V_CODE_PAGES")


def cache_write_kernel_source() -> str:
    """Which single-token writer entry point serves: ``hand_cuda`` (default) or ``jac_dsl``.

    The environment variable, its accepted spellings and the fail-closed error are the reference's
    (source_patch.py:67-85). Both names resolve to the same B200 kernels here; the selector picks the
    C symbol (``kivi_b200_cache_write_launch`` vs ``jac_launch_cache_write``)."""
    raw = os.environ.get(CACHE_WRITE_KERNEL_ENV, "hand_cuda")
    key = raw.strip().lower().replace("-", "_")
    for canonical, spellings in _WRITER_ALIASES.items():
        if key in spellings:
            return canonical
    raise ValueError(f"{CACHE_WRITE_KERNEL_ENV} must be hand_cuda or jac_dsl, got {raw!r}")


def validate_kivi_cache_bundle(cache: Mapping[str, Any]) -> None:
    """Kind tag, presence and dtype of the eight cache tensors (the checks of source_patch.py:210-226, in
    the same order, with the same exception types and messages)."""
    if cache.get("kind") != KIVI_CACHE_KIND:
        raise TypeError("expected GPUModelRunner int4_kivi_dsl_paged cache bundle")
    absent = [name for name in _CACHE_TENSORS if name not in cache]
    if absent:
        raise KeyError(f"KIVI cache bundle missing tensors: {absent}")
    for wanted, names, suffix in ((torch.uint8, _CODE_TENSORS, "torch.uint8 packed int4"),
                                  (torch.float16, tuple(n for n in _CACHE_TENSORS if n not in _CODE_TENSORS), "torch.float16")):
        for name in names:
            if cache[name].dtype != wanted:
                raise TypeError(f"{name} must be {suffix}")


def _require_dtype(tensor: torch.Tensor, dtype: torch.dtype, message: str) -> None:
    if tensor.dtype != dtype:
        raise TypeError(message)


def _check_decode_io(q: torch.Tensor, table: torch.Tensor, out: torch.Tensor, table_name: str) -> None:
    _require_dtype(table, torch.int32, f"{table_name} must be torch.int32")
    _require_dtype(q, torch.float16, "Q must be torch.float16")
    _require_dtype(out, torch.float32, "O must be torch.float32")


def _check_write_io(key: torch.Tensor, value: torch.Tensor, slot_mapping: torch.Tensor, block_table: torch.Tensor) -> None:
    if not (key.dtype == value.dtype == torch.float16):
        raise TypeError("KIVI cache write expects fp16 key/value tensors")
    _require_dtype(slot_mapping, torch.int64, "KIVI cache write expects int64 slot_mapping")
    _require_dtype(block_table, torch.int32, "KIVI cache write expects int32 block_table")


def _check_launch_order(cache: Mapping[str, Any]) -> None:
    if tuple(cache.get("jac_launch_order", ())) != JAC_LAUNCH_ORDER:
        raise RuntimeError("int4_kivi cache bundle has stale jac_launch_order")


def _check_seq_len(seq_len: int) -> None:
    if not 1 <= seq_len <= MAX_SEQ_LEN:
        raise ValueError("SEQ_LEN must be in [1, 4096] for the first KIVI DSL lane")


def make_cache_bundle(num_blocks: int, *, num_kv_heads: int = 8, device: torch.device | str = "cuda",
                      fill: int | None = None) -> dict[str, Any]:
    """Allocate a reference-lane cache bundle (the dict shape vLLM's model runner builds,
    source_patch.py:2260-2279) for one sequence."""
    def alloc(shape, dtype):
        if fill is None:
            return torch.zeros(shape, dtype=dtype, device=device)
        t = torch.empty(shape, dtype=dtype, device=device)
        t.view(torch.uint8).fill_(fill)
        return t

    nkv = num_kv_heads
    return {
        "kind": KIVI_CACHE_KIND,
        "jac_launch_order": JAC_LAUNCH_ORDER,
        "K_CODE_PAGES": alloc((num_blocks, nkv, BLOCK_SIZE, HD // 2), torch.uint8),
        "K_SCALE_PAGES": alloc((num_blocks, nkv, HD), torch.float16),
        "K_ZERO_PAGES": alloc((num_blocks, nkv, HD), torch.float16),
        "V_CODE_PAGES": alloc((num_blocks, nkv, BLOCK_SIZE, HD // 2), torch.uint8),
        "V_SCALE_PAGES": alloc((num_blocks, nkv, BLOCK_SIZE, HD // BLOCK_SIZE), torch.float16),
        "V_ZERO_PAGES": alloc((num_blocks, nkv, BLOCK_SIZE, HD // BLOCK_SIZE), torch.float16),
        "K_RESIDUAL_SCRATCH": alloc((nkv, RESIDUAL + BLOCK_SIZE, HD), torch.float16),
        "V_RESIDUAL_SCRATCH": alloc((nkv, RESIDUAL + BLOCK_SIZE, HD), torch.float16),
    }


def _check_block_table_width(block_table: torch.Tensor, seq_len: int, name: str = "BLOCK_TABLE") -> None:
    """check_block_table_width of the reference binding (source_patch.py:693-708)."""
    if block_table.dim() != 1:
        raise RuntimeError(f"{name} rank mismatch for the KIVI v1 ABI")
    if seq_len < 1 or seq_len > MAX_SEQ_LEN:
        raise ValueError("SEQ_LEN must be in [1, 4096] for KIVI BLOCK_TABLE validation")
    required = (seq_len - RESIDUAL) // BLOCK_SIZE if seq_len > RESIDUAL else 0
    if block_table.shape[0] < required:
        raise RuntimeError(f"{name} dim 0 must be at least {required} for the KIVI v1 ABI, got {block_table.shape[0]}")


def _check_cache_shapes(cache: Mapping[str, Any]) -> tuple[int, str]:
    """Shape checks of the reference binding (check_shape, source_patch.py:678-691) and the
    NH/NKV geometry selection (:743-760). Returns (NKV, symbol suffix)."""
    kc = cache["K_CODE_PAGES"]
    if kc.dim() != 4:
        raise RuntimeError("K_CODE_PAGES must be [num_blocks, NKV, 32, 64]")
    nb, nkv = int(kc.shape[0]), int(kc.shape[1])
    if (nkv * 5, nkv) not in _GEOMETRIES:
        raise RuntimeError(f"KIVI v1 ABI supports NH/NKV 40/8 or TP=2 local 20/4; got NKV={nkv}")
    hg = HD // BLOCK_SIZE
    want = {
        "K_CODE_PAGES": (nb, nkv, BLOCK_SIZE, HD // 2), "V_CODE_PAGES": (nb, nkv, BLOCK_SIZE, HD // 2),
        "K_SCALE_PAGES": (nb, nkv, HD), "K_ZERO_PAGES": (nb, nkv, HD),
        "V_SCALE_PAGES": (nb, nkv, BLOCK_SIZE, hg), "V_ZERO_PAGES": (nb, nkv, BLOCK_SIZE, hg),
        "K_RESIDUAL_SCRATCH": (nkv, RESIDUAL + BLOCK_SIZE, HD), "V_RESIDUAL_SCRATCH": (nkv, RESIDUAL + BLOCK_SIZE, HD),
    }
    for name, shape in want.items():
        t = cache[name]
        if tuple(t.shape) != shape:
            raise RuntimeError(f"{name} must have shape {shape} for the KIVI v1 ABI, got {tuple(t.shape)}")
        if not t.is_cuda or not t.is_contiguous():
            raise RuntimeError(f"{name} must be a contiguous CUDA tensor")
    return nkv, _GEOMETRIES[(nkv * 5, nkv)]


def _one_device(tensors, what: str, require_cuda: bool = True) -> torch.device:
    devices = {t.device for t in tensors}
    if len(devices) != 1:
        raise RuntimeError(f"{what} tensors span devices: {devices}")
    dev = next(iter(devices))
    if require_cuda and dev.type != "cuda":
        raise RuntimeError(f"{what} tensors must be CUDA tensors, got {dev}")
    return dev


def _p(t: torch.Tensor):
    return ctypes.c_void_p(t.data_ptr())


def _stream(device: torch.device, stream: Any = None):
    s = torch.cuda.current_stream(device) if stream is None else stream
    return ctypes.c_void_p(s.cuda_stream)


def _cache_ptrs(cache: Mapping[str, Any]):
    return [_p(cache[name]) for name in _CACHE_TENSORS]


@dataclass(frozen=True)
class KiviDslLaunchBinding:
    """Validated argument bundle for ``jac_launch`` (source_patch.py:179-211 of the reference)."""

    q: torch.Tensor
    block_table: torch.Tensor
    cache: Mapping[str, Any]
    seq_len: int
    out: torch.Tensor

    def jac_launch_args(self) -> tuple[Any, ...]:
        """The arguments in launch order, after the bundle, dtype, length and one-device checks."""
        validate_kivi_cache_bundle(self.cache)
        _check_launch_order(self.cache)
        _check_decode_io(self.q, self.block_table, self.out, "BLOCK_TABLE")
        _check_seq_len(self.seq_len)
        pools = tuple(self.cache[name] for name in _CACHE_TENSORS)
        _one_device((self.q, self.block_table, self.out) + pools, "KIVI jac_launch", require_cuda=False)
        return (self.q, self.block_table) + pools + (self.seq_len, self.out)


def launch_kivi_dsl_decode(q: torch.Tensor, block_table: torch.Tensor, cache: Mapping[str, Any], out: torch.Tensor,
                           *, seq_len: int, stream: Any = None) -> None:
    """Decode one query token of one sequence (reference: source_patch.py:294-315 -> C++
    ``kivi_decode_dsl`` :768-869 -> ``jac_launch``)."""
    args = KiviDslLaunchBinding(q, block_table, cache, seq_len, out).jac_launch_args()
    _one_device([a for a in args if isinstance(a, torch.Tensor)], "KIVI jac_launch")
    nkv, suffix = _check_cache_shapes(cache)
    if tuple(q.shape) != (nkv * 5, HD) or tuple(out.shape) != (nkv * 5, HD):
        raise RuntimeError(f"Q and O must be [{nkv * 5}, {HD}] for the KIVI v1 ABI")
    if not q.is_contiguous() or not out.is_contiguous() or not block_table.is_contiguous():
        raise RuntimeError("Q, O and BLOCK_TABLE must be contiguous for jac_launch")
    _check_block_table_width(block_table, seq_len)
    fn = getattr(_native.lib(), "jac_launch" + suffix)
    fn(_p(q), _p(block_table), *_cache_ptrs(cache), int(seq_len), _p(out), _stream(q.device, stream))


def launch_kivi_dsl_decode_batched(q: torch.Tensor, seq_lens: torch.Tensor, block_table: torch.Tensor,
                                   cache: Mapping[str, Any], out: torch.Tensor, *, num_queries: int,
                                   stream: Any = None) -> None:
    """``num_queries`` queries of one sequence, each with its own length
    (reference: source_patch.py:412-485 -> ``jac_launch_batched``). Like the reference this reads
    SEQ_LENS back to the host to bound the values before launching."""
    validate_kivi_cache_bundle(cache)
    _check_launch_order(cache)
    _check_decode_io(q, block_table, out, "BLOCK_TABLE")
    _require_dtype(seq_lens, torch.int32, "SEQ_LENS must be torch.int32")
    if num_queries < 1 or num_queries > MAX_QUERIES:
        raise ValueError(f"NUM_QUERIES must be in [1, {MAX_QUERIES}]")
    lens = [int(v) for v in seq_lens.detach().cpu().tolist()]
    for i, value in enumerate(lens):
        if value < 1 or value > MAX_SEQ_LEN:
            raise ValueError(f"SEQ_LENS[{i}] must be in [1, 4096] for the batched KIVI decode ABI, got {value}")
    q = q.contiguous()
    nkv, suffix = _check_cache_shapes(cache)
    if tuple(q.shape) != (num_queries, nkv * 5, HD) or tuple(out.shape) != (num_queries, nkv * 5, HD):
        raise RuntimeError(f"Q and O must be [{num_queries}, {nkv * 5}, {HD}]")
    if seq_lens.numel() != num_queries or not out.is_contiguous():
        raise RuntimeError("SEQ_LENS must hold one entry per query and O must be contiguous")
    _one_device((q, seq_lens, block_table, out) + tuple(cache[n] for n in _CACHE_TENSORS), "KIVI batched jac_launch")
    _check_block_table_width(block_table, max(lens))
    fn = getattr(_native.lib(), "jac_launch_batched" + suffix)
    fn(_p(q), _p(seq_lens), _p(block_table), *_cache_ptrs(cache), int(num_queries), _p(out), _stream(q.device, stream))


def launch_kivi_dsl_decode_sparse_retained(q: torch.Tensor, retained_block_table: torch.Tensor,
                                           cache: Mapping[str, Any], out: torch.Tensor, *, seq_len: int,
                                           num_retained_pages: int, stream: Any = None) -> None:
    """Sparse-retained decode over a compact page table (reference: source_patch.py:318-372 ->
    ``jac_launch_sparse_retained``); the serving telemetry the reference writes around the call is
    not part of the kernel path and is left to the caller."""
    validate_kivi_cache_bundle(cache)
    _check_decode_io(q, retained_block_table, out, "RETAINED_BLOCK_TABLE")
    if retained_block_table.numel() != OLD_BLOCKS:
        raise ValueError(f"RETAINED_BLOCK_TABLE must have {OLD_BLOCKS} entries")
    if num_retained_pages < 0 or num_retained_pages > OLD_BLOCKS:
        raise ValueError("NUM_RETAINED_PAGES must be in [0, OLD_BLOCKS]")
    _check_seq_len(seq_len)
    nkv, suffix = _check_cache_shapes(cache)
    _one_device((q, retained_block_table, out) + tuple(cache[n] for n in _CACHE_TENSORS), "KIVI sparse jac_launch")
    fn = getattr(_native.lib(), "jac_launch_sparse_retained" + suffix)
    fn(_p(q), _p(retained_block_table), *_cache_ptrs(cache), int(seq_len), int(num_retained_pages), _p(out),
       _stream(q.device, stream))


def require_kivi_cache_write(key: torch.Tensor, value: torch.Tensor, slot_mapping: torch.Tensor,
                             block_table: torch.Tensor, cache: Mapping[str, Any], seq_len: int) -> None:
    """Write one token's K/V; ``seq_len`` is the length after it (reference:
    source_patch.py:228-291 -> ``kivi_cache_write_dsl`` / ``kivi_cache_write_jac_dsl``)."""
    validate_kivi_cache_bundle(cache)
    _check_write_io(key, value, slot_mapping, block_table)
    heads, _, head_size = cache["K_RESIDUAL_SCRATCH"].shape
    new_k = key.reshape(-1, head_size).contiguous()
    new_v = value.reshape(-1, head_size).contiguous()
    for label, rows in (("key", new_k), ("value", new_v)):
        if tuple(rows.shape) != (heads, head_size):
            raise RuntimeError(f"KIVI {label} tensor does not match residual [num_kv_heads, head_size]")
    tensors = tuple(cache[name] for name in _CACHE_TENSORS) + (new_k, new_v, slot_mapping, block_table)
    dev = _one_device(tensors, "KIVI cache-write")
    nkv, _ = _check_cache_shapes(cache)
    _check_block_table_width(block_table, seq_len)
    if cache_write_kernel_source() == "jac_dsl":
        if nkv != 8:
            raise RuntimeError("jac_launch_cache_write is compiled for NKV=8; use hand_cuda for the TP=2 local lane")
        _native.lib().jac_launch_cache_write(*_cache_ptrs(cache), _p(new_k), _p(new_v), _p(block_table), int(seq_len),
                                             _stream(dev))
    else:
        _native.lib().kivi_b200_cache_write_launch(*_cache_ptrs(cache), _p(new_k), _p(new_v), _p(slot_mapping),
                                                   _p(block_table), int(seq_len), nkv, _stream(dev))


def require_kivi_cache_write_batched(key: torch.Tensor, value: torch.Tensor, slot_mapping: torch.Tensor,
                                     block_table: torch.Tensor, cache: Mapping[str, Any], start_seq_len: int,
                                     num_new: int) -> None:
    """Write ``num_new`` tokens ``[num_new, NKV, D]`` of one sequence (reference:
    source_patch.py:375-409 -> ``kivi_cache_write_batched_dsl``). The reference needs the chunk
    pre-split with ``plan_batched_write``; this writer also takes a chunk that crosses several
    age-out boundaries, as long as it fits the call's bound of 160 rows."""
    validate_kivi_cache_bundle(cache)
    _check_write_io(key, value, slot_mapping, block_table)
    if num_new < 1 or num_new > RESIDUAL + BLOCK_SIZE:
        raise ValueError(f"NUM_NEW must be in [1, {RESIDUAL + BLOCK_SIZE}]")
    if start_seq_len < 0 or start_seq_len + num_new > MAX_SEQ_LEN:
        raise ValueError("START_SEQ_LEN + NUM_NEW must stay within [1, 4096]")
    residual = cache["K_RESIDUAL_SCRATCH"]
    new_k = key.reshape(num_new, -1, residual.shape[-1]).contiguous()
    new_v = value.reshape(num_new, -1, residual.shape[-1]).contiguous()
    tensors = tuple(cache[name] for name in _CACHE_TENSORS) + (new_k, new_v, slot_mapping, block_table)
    dev = _one_device(tensors, "KIVI batched cache-write")
    nkv, _ = _check_cache_shapes(cache)
    if new_k.shape[1] != nkv or new_v.shape != new_k.shape:
        raise RuntimeError("KIVI batched key/value tensors do not match [num_new, num_kv_heads, head_size]")
    _check_block_table_width(block_table, start_seq_len + num_new)
    _native.lib().kivi_b200_cache_write_batched_launch(*_cache_ptrs(cache), _p(new_k), _p(new_v), _p(slot_mapping),
                                                       _p(block_table), int(start_seq_len), int(num_new), nkv,
                                                       _stream(dev))


def _split_old_tokens_batched(seq_len: int, residual: int, block_size: int) -> int:
    return max(0, seq_len - residual) // block_size * block_size


@dataclass(frozen=True)
class KiviWriteSubChunk:
    """One piece of a planned chunk (field names are the reference's, source_patch.py:488-501): the piece appends
    ``num_new`` rows at scratch row ``scratch_start``; when it fills the scratch, ``age_out_page`` is the logical
    page (key group) that is quantised and ``post_shift_residual_len`` the rows left afterwards."""
    start_seq_len: int
    num_new: int
    scratch_start: int
    age_out_page: int | None
    post_shift_residual_len: int | None

    @property
    def crosses_boundary(self) -> bool:
        return self.age_out_page is not None

    @property
    def end_seq_len(self) -> int:
        return self.start_seq_len + self.num_new


def plan_batched_write(start_seq_len: int, num_new_tokens: int, residual: int = 128,
                       block_size: int = 32) -> list[KiviWriteSubChunk]:
    """Cut a chunk into pieces that each cross at most one age-out boundary (reference:
    source_patch.py:504-553). Kept for callers of the v1 writer; ``block_size`` is the age-out
    unit (the key group)."""
    if start_seq_len < 0:
        raise ValueError(f"start_seq_len must be >= 0, got {start_seq_len}")
    if num_new_tokens < 1:
        raise ValueError(f"num_new_tokens must be >= 1, got {num_new_tokens}")
    if residual <= 0 or block_size <= 0:
        raise ValueError("residual and block_size must be positive")
    capacity = residual + block_size
    pieces: list[KiviWriteSubChunk] = []
    seq_len, remaining = start_seq_len, num_new_tokens
    while remaining > 0:
        old_before = _split_old_tokens_batched(seq_len, residual, block_size)
        filled = seq_len - old_before
        take = min(remaining, capacity - filled)
        if take <= 0:
            raise ValueError(f"planning invariant violated: scratch full at {filled} of {capacity} rows")
        old_after = _split_old_tokens_batched(seq_len + take, residual, block_size)
        crossed = old_after > old_before
        pieces.append(KiviWriteSubChunk(seq_len, take, filled, old_before // block_size if crossed else None,
                                        seq_len + take - old_after if crossed else None))
        seq_len += take
        remaining -= take
    return pieces
