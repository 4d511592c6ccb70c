"""ctypes front-end of the CPU oracle (``kivi_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the test suite, by the smoke check and by the benchmark's
CPU-baseline leg as the checker / the timed baseline. The product package never imports it.

All arrays are numpy: fp16 tensors travel as ``uint16`` bit patterns (``.view(np.uint16)``), codes
as ``uint8``, tables as ``int32``.
"""
from __future__ import annotations

import ctypes
import subprocess
from dataclasses import dataclass
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libkivi_oracle.so"


class _Geom(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("nh", "nkv", "d", "b", "g", "r")]


class _Pages(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("k_code", "k_scale", "k_zero", "v_code", "v_scale", "v_zero")]


def build(force: bool = False) -> Path:
    """Compile the oracle with the committed Makefile if the library is missing or stale."""
    src = _HERE / "kivi_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "all"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
        _lib.kivi_oracle_h2f.restype = ctypes.c_float
        _lib.kivi_oracle_h2f.argtypes = [ctypes.c_uint16]
        _lib.kivi_oracle_f2h.restype = ctypes.c_uint16
        _lib.kivi_oracle_f2h.argtypes = [ctypes.c_float]
    return _lib


@dataclass(frozen=True)
class Geometry:
    nh: int
    nkv: int
    d: int
    b: int
    g: int
    r: int

    @property
    def hd_groups(self) -> int:
        return -(-self.d // self.g)

    @property
    def scratch_rows(self) -> int:
        return self.r + self.g

    def c(self) -> _Geom:
        return _Geom(self.nh, self.nkv, self.d, self.b, self.g, self.r)

    def split_old(self, seq_len: int) -> int:
        return max(0, seq_len - self.r) // self.g * self.g


REF_LANE = Geometry(nh=40, nkv=8, d=128, b=32, g=32, r=128)


def _p(a: np.ndarray | None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(ctypes.c_void_p)


class OracleCache:
    """Host copy of one layer's page pool and scratch slots, in the reference tensor layout
    (integrations/vllm_kivi/bindings.py:105-118) with a leading slot dimension on the scratch."""

    def __init__(self, geom: Geometry, num_blocks: int, num_slots: int = 1, fill: int = 0):
        g = geom
        self.geom = g
        self.num_blocks = num_blocks
        self.num_slots = num_slots
        self.k_code = np.full((num_blocks, g.nkv, g.b, g.d // 2), fill, np.uint8)
        self.v_code = np.full((num_blocks, g.nkv, g.b, g.d // 2), fill, np.uint8)
        f16fill = fill | (fill << 8)
        self.k_scale = np.full((num_blocks, g.nkv, g.d), f16fill, np.uint16)
        self.k_zero = np.full((num_blocks, g.nkv, g.d), f16fill, np.uint16)
        self.v_scale = np.full((num_blocks, g.nkv, g.b, g.hd_groups), f16fill, np.uint16)
        self.v_zero = np.full((num_blocks, g.nkv, g.b, g.hd_groups), f16fill, np.uint16)
        self.k_scratch = np.full((num_slots, g.nkv, g.scratch_rows, g.d), f16fill, np.uint16)
        self.v_scratch = np.full((num_slots, g.nkv, g.scratch_rows, g.d), f16fill, np.uint16)

    PAGE_FIELDS = ("k_code", "k_scale", "k_zero", "v_code", "v_scale", "v_zero")
    ALL_FIELDS = PAGE_FIELDS + ("k_scratch", "v_scratch")

    def pages(self) -> _Pages:
        return _Pages(*[_p(getattr(self, n)) for n in self.PAGE_FIELDS])

    def copy(self) -> "OracleCache":
        out = OracleCache.__new__(OracleCache)
        out.geom, out.num_blocks, out.num_slots = self.geom, self.num_blocks, self.num_slots
        for n in self.ALL_FIELDS:
            setattr(out, n, getattr(self, n).copy())
        return out


def _u16(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view(np.uint16) if a.dtype == np.float16 else a


def write_tokens(cache: OracleCache, new_k, new_v, block_table, start_seq_len: int, slot: int = 0) -> None:
    """Append ``new_k/new_v [n, NKV, D]`` token by token (the reference single-token writer)."""
    g = cache.geom
    new_k, new_v = _u16(new_k), _u16(new_v)
    bt = np.ascontiguousarray(block_table, np.int32)
    pg = cache.pages()
    gm = g.c()
    rc = lib().kivi_oracle_write_tokens(
        ctypes.byref(gm), ctypes.byref(pg), _p(cache.k_scratch[slot]), _p(cache.v_scratch[slot]),
        _p(new_k), _p(new_v), _p(bt), ctypes.c_int(start_seq_len), ctypes.c_int(new_k.shape[0]))
    if rc:
        raise RuntimeError(f"oracle writer failed rc={rc}")


def write_batched(cache: OracleCache, new_k, new_v, block_table, start_seq_len: int, slot: int = 0) -> None:
    """The reference's batched writer: append all rows, then at most one age-out."""
    new_k, new_v = _u16(new_k), _u16(new_v)
    bt = np.ascontiguousarray(block_table, np.int32)
    pg = cache.pages()
    gm = cache.geom.c()
    rc = lib().kivi_oracle_write_batched(
        ctypes.byref(gm), ctypes.byref(pg), _p(cache.k_scratch[slot]), _p(cache.v_scratch[slot]),
        _p(new_k), _p(new_v), _p(bt), ctypes.c_int(start_seq_len), ctypes.c_int(new_k.shape[0]))
    if rc:
        raise ValueError("chunk overflows the scratch or crosses more than one age-out boundary")


def write_batch(cache: OracleCache, new_k, new_v, block_tables, start_seq_lens, offsets, slot_ids=None,
                nthreads: int = 1) -> None:
    """Multi-sequence writer: sequence i appends rows ``offsets[i]:offsets[i+1]``."""
    new_k, new_v = _u16(new_k), _u16(new_v)
    bts = np.ascontiguousarray(block_tables, np.int32)
    starts = np.ascontiguousarray(start_seq_lens, np.int32)
    offs = np.ascontiguousarray(offsets, np.int32)
    slots = None if slot_ids is None else np.ascontiguousarray(slot_ids, np.int32)
    pg = cache.pages()
    gm = cache.geom.c()
    rc = lib().kivi_oracle_write_batch(
        ctypes.byref(gm), ctypes.byref(pg), _p(cache.k_scratch), _p(cache.v_scratch), _p(new_k), _p(new_v),
        _p(bts), ctypes.c_int(bts.shape[1]), _p(starts), _p(offs), _p(slots), ctypes.c_int(len(starts)),
        ctypes.c_int(nthreads))
    if rc:
        raise RuntimeError("oracle multi-sequence writer failed")


def plan_batched_write(geom: Geometry, start_seq_len: int, num_new: int) -> list[tuple[int, int]]:
    cap = 4 + num_new // max(1, geom.g) + 2
    starts = np.zeros(cap, np.int32)
    nums = np.zeros(cap, np.int32)
    gm = geom.c()
    n = lib().kivi_oracle_plan_batched_write(ctypes.byref(gm), ctypes.c_int(start_seq_len), ctypes.c_int(num_new),
                                             _p(starts), _p(nums), ctypes.c_int(cap))
    if n < 0:
        raise ValueError("bad plan arguments")
    return [(int(starts[i]), int(nums[i])) for i in range(n)]


def decode(cache: OracleCache, q, block_table, seq_len: int, slot: int = 0, *, mode: int = 0,
           max_old_tokens: int = -1, num_retained_pages: int = -1) -> np.ndarray:
    """One sequence, all heads. ``mode`` 0 = reference-order online softmax, 1 = two-pass."""
    g = cache.geom
    q = _u16(q)
    bt = np.ascontiguousarray(block_table, np.int32)
    out = np.zeros((g.nh, g.d), np.float32)
    pg = cache.pages()
    gm = g.c()
    lib().kivi_oracle_decode(
        ctypes.byref(gm), ctypes.byref(pg), _p(q), _p(bt), _p(cache.k_scratch[slot]), _p(cache.v_scratch[slot]),
        ctypes.c_int(seq_len), ctypes.c_int(max_old_tokens), ctypes.c_int(num_retained_pages), ctypes.c_int(mode),
        _p(out))
    return out


def decode_batch(cache: OracleCache, q, block_tables, seq_lens, slot_ids=None, *, mode: int = 0,
                 max_old_tokens: int = -1, nthreads: int = 1) -> np.ndarray:
    g = cache.geom
    q = _u16(q)
    bts = np.ascontiguousarray(block_tables, np.int32)
    sl = np.ascontiguousarray(seq_lens, np.int32)
    slots = None if slot_ids is None else np.ascontiguousarray(slot_ids, np.int32)
    out = np.zeros((len(sl), g.nh, g.d), np.float32)
    pg = cache.pages()
    gm = g.c()
    lib().kivi_oracle_decode_batch(
        ctypes.byref(gm), ctypes.byref(pg), _p(q), _p(bts), ctypes.c_int(bts.shape[1]), _p(sl), _p(slots),
        _p(cache.k_scratch), _p(cache.v_scratch), ctypes.c_int(len(sl)), ctypes.c_int(max_old_tokens),
        ctypes.c_int(mode), ctypes.c_int(nthreads), _p(out))
    return out


def gemv(w, x, nthreads: int = 1) -> tuple[np.ndarray, np.ndarray]:
    """``y = W x`` for ``W [out, in]`` and ``x [in]`` or ``[batch, in]``; returns (fp16, fp32)."""
    w, x = _u16(w), _u16(x)
    x2 = x.reshape(-1, x.shape[-1])
    out_dim, in_dim = w.shape
    y16 = np.zeros((x2.shape[0], out_dim), np.uint16)
    y32 = np.zeros((x2.shape[0], out_dim), np.float32)
    lib().kivi_oracle_gemv(_p(w), _p(x2), _p(y16), _p(y32), ctypes.c_int(out_dim), ctypes.c_int(in_dim),
                           ctypes.c_int(x2.shape[0]), ctypes.c_int(nthreads))
    shape = x.shape[:-1] + (out_dim,)
    return y16.view(np.float16).reshape(shape), y32.reshape(shape)


def residual_rmsnorm(x, delta, weight, eps: float) -> tuple[np.ndarray, np.ndarray]:
    """``x_out = x + delta`` (``delta`` may be None), ``normed = RMSNorm(x_out) * weight``; rows [batch, hidden]."""
    x = _u16(x)
    batch, hidden = x.shape
    d = None if delta is None else _u16(delta)
    x_out = np.zeros_like(x)
    normed = np.zeros_like(x)
    lib().kivi_oracle_residual_rmsnorm(_p(x), _p(d), _p(_u16(weight)), _p(x_out), _p(normed), ctypes.c_int(batch),
                                       ctypes.c_int(hidden), ctypes.c_float(eps))
    return x_out.view(np.float16), normed.view(np.float16)


def bias_rope(qkv, bias, positions, nh: int, nkv: int, hd: int, rope_base: float):
    """Bias add, RoPE on q and k at ``positions``; returns q [batch, nh*hd], k, v [batch, nkv*hd]."""
    qkv = _u16(qkv)
    batch = qkv.shape[0]
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    b = None if bias is None else _u16(bias)
    q = np.zeros((batch, nh * hd), np.uint16)
    k = np.zeros((batch, nkv * hd), np.uint16)
    v = np.zeros((batch, nkv * hd), np.uint16)
    lib().kivi_oracle_bias_rope(_p(qkv), _p(b), _p(pos), _p(q), _p(k), _p(v), ctypes.c_int(batch), ctypes.c_int(nh),
                                ctypes.c_int(nkv), ctypes.c_int(hd), ctypes.c_float(rope_base))
    return q.view(np.float16), k.view(np.float16), v.view(np.float16)


def silu_mul(gate_up) -> np.ndarray:
    gate_up = _u16(gate_up)
    batch, two_ffn = gate_up.shape
    out = np.zeros((batch, two_ffn // 2), np.uint16)
    lib().kivi_oracle_silu_mul(_p(gate_up), _p(out), ctypes.c_int(batch), ctypes.c_int(two_ffn // 2))
    return out.view(np.float16)


def argmax(logits) -> np.ndarray:
    logits = _u16(logits)
    batch, n = logits.shape
    out = np.zeros(batch, np.int32)
    lib().kivi_oracle_argmax(_p(logits), _p(out), ctypes.c_int(batch), ctypes.c_int(n))
    return out


def h2f(bits: int) -> float:
    return float(lib().kivi_oracle_h2f(ctypes.c_uint16(bits)))


def f2h(value: float) -> int:
    return int(lib().kivi_oracle_f2h(ctypes.c_float(value)))
