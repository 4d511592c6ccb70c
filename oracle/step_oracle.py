"""CPU restatement of one decode step of the generated runtime around the KIVI cache.

TEST INFRASTRUCTURE ONLY (imported by tests, the smoke check and the benchmark's CPU legs).

The step follows ``forward()`` of the reference (crates/jac-codegen-cuda/src/templates/runtime.cu:125-187)
kernel by kernel, with every intermediate stored as fp16 like the reference's buffers, for a batch
of sequences and with the fp16 KV store and the three attention kernels (runtime.cu:160-164)
replaced by the int4-KIVI writer and paged decode of this oracle. Tensor parallelism over KV
heads is emulated rank by rank: the two partial projections per layer are summed in fp32 in rank
order and rounded to fp16 once.
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass, field

import numpy as np

from oracle import kivi_oracle as ko


@dataclass
class StepShape:
    layers: int
    hidden: int
    nh: int
    nkv: int
    hd: int
    ffn: int
    vocab: int
    rope_base: float = 10000.0
    norm_eps: float = 1e-5
    attn_bias: bool = False
    block: int = 16
    group: int = 32
    residual: int = 32

    @property
    def q_dim(self) -> int:
        return self.nh * self.hd

    @property
    def kv_dim(self) -> int:
        return self.nkv * self.hd


@dataclass
class StepWeights:
    """Weights in the reference's file layout (templates/export.py:69-92): row-major [out, in]."""
    embed: np.ndarray
    final_norm: np.ndarray
    lm_head: np.ndarray
    layers: list[dict[str, np.ndarray]] = field(default_factory=list)


def random_weights(shape: StepShape, seed: int, std: float = 0.02) -> StepWeights:
    """Random-init fp16 weights N(0, std); norm weights around 1."""
    rng = np.random.default_rng(seed)
    s = shape

    def mat(rows, cols):
        return (rng.standard_normal((rows, cols), dtype=np.float32) * std).astype(np.float16)

    def norm():
        return (1.0 + 0.1 * rng.standard_normal(s.hidden, dtype=np.float32)).astype(np.float16)

    w = StepWeights(mat(s.vocab, s.hidden), norm(), mat(s.vocab, s.hidden))
    for _ in range(s.layers):
        w.layers.append({
            "attn_norm": norm(),
            "qkv": mat(s.q_dim + 2 * s.kv_dim, s.hidden),
            "qkv_bias": (rng.standard_normal(s.q_dim + 2 * s.kv_dim, dtype=np.float32) * 0.1).astype(np.float16)
            if s.attn_bias else None,
            "o": mat(s.hidden, s.q_dim),
            "ffn_norm": norm(),
            "gate_up": mat(2 * s.ffn, s.hidden),
            "down": mat(s.hidden, s.ffn),
        })
    return w


def weights_checksum(w: StepWeights) -> int:
    """CRC-32 over every weight tensor, to tell whether a seed still reproduces stored golden runs."""
    crc = 0
    for a in (w.embed, w.final_norm, w.lm_head):
        crc = zlib.crc32(np.ascontiguousarray(a).view(np.uint8), crc)
    for lw in w.layers:
        for k in ("attn_norm", "qkv", "qkv_bias", "o", "ffn_norm", "gate_up", "down"):
            if lw[k] is not None:
                crc = zlib.crc32(np.ascontiguousarray(lw[k]).view(np.uint8), crc)
    return crc


def shard_layer(shape: StepShape, lw: dict[str, np.ndarray], rank: int, world: int) -> dict[str, np.ndarray]:
    """KV-head tensor-parallel shard of one layer: rows of q/k/v and gate/up, columns of o/down."""
    s = shape
    nh_l, nkv_l, ffn_l = s.nh // world, s.nkv // world, s.ffn // world
    q_rows = slice(rank * nh_l * s.hd, (rank + 1) * nh_l * s.hd)
    k_rows = slice(s.q_dim + rank * nkv_l * s.hd, s.q_dim + (rank + 1) * nkv_l * s.hd)
    v_rows = slice(s.q_dim + s.kv_dim + rank * nkv_l * s.hd, s.q_dim + s.kv_dim + (rank + 1) * nkv_l * s.hd)
    g_rows = slice(rank * ffn_l, (rank + 1) * ffn_l)
    u_rows = slice(s.ffn + rank * ffn_l, s.ffn + (rank + 1) * ffn_l)

    def rows(m, *slices):
        return None if m is None else np.ascontiguousarray(np.concatenate([m[sl] for sl in slices], axis=0))

    return {
        "attn_norm": lw["attn_norm"], "ffn_norm": lw["ffn_norm"],
        "qkv": rows(lw["qkv"], q_rows, k_rows, v_rows),
        "qkv_bias": rows(lw["qkv_bias"], q_rows, k_rows, v_rows),
        "o": np.ascontiguousarray(lw["o"][:, q_rows]),
        "gate_up": rows(lw["gate_up"], g_rows, u_rows),
        "down": np.ascontiguousarray(lw["down"][:, g_rows]),
    }


def _sum_partials(parts: list[np.ndarray]) -> np.ndarray:
    acc = np.zeros(parts[0].shape, np.float32)
    for p in parts:
        acc = acc + p.astype(np.float32)
    return acc.astype(np.float16)


class StepOracle:
    """State of ``batch`` sequences over ``world`` emulated ranks."""

    def __init__(self, shape: StepShape, weights: StepWeights, block_tables: np.ndarray, num_blocks: int,
                 world: int = 1, gemv_threads: int = 1):
        s = shape
        assert s.nkv % world == 0 and s.nh % world == 0 and s.ffn % world == 0 and s.vocab % world == 0
        self.shape, self.weights, self.world = s, weights, world
        self.block_tables = np.ascontiguousarray(block_tables, np.int32)
        self.batch = self.block_tables.shape[0]
        self.seq_lens = np.zeros(self.batch, np.int32)
        self.gemv_threads = gemv_threads
        self.geom = ko.Geometry(nh=s.nh // world, nkv=s.nkv // world, d=s.hd, b=s.block, g=s.group, r=s.residual)
        self.caches = [[ko.OracleCache(self.geom, num_blocks, self.batch) for _ in range(s.layers)]
                       for _ in range(world)]
        self.shards = [[shard_layer(s, lw, r, world) for lw in weights.layers] for r in range(world)]

    def _gemv(self, w, x):
        return ko.gemv(w, x, self.gemv_threads)[0]

    def step(self, tokens: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
        """Feed one token per sequence; returns (arg-max token ids, logits [batch, vocab] fp16)."""
        s, n, world = self.shape, self.batch, self.world
        tokens = np.asarray(tokens, np.int64)
        x = self.weights.embed[tokens].copy()
        delta = None
        offsets = np.arange(n + 1, dtype=np.int32)
        for l in range(s.layers):
            x, normed = ko.residual_rmsnorm(x, delta, self.weights.layers[l]["attn_norm"], s.norm_eps)
            parts = []
            for r in range(world):
                lw = self.shards[r][l]
                g = self.geom
                qkv = self._gemv(lw["qkv"], normed)
                q, k, v = ko.bias_rope(qkv, lw["qkv_bias"], self.seq_lens, g.nh, g.nkv, g.d, s.rope_base)
                cache = self.caches[r][l]
                ko.write_batch(cache, k.reshape(n, g.nkv, g.d), v.reshape(n, g.nkv, g.d), self.block_tables,
                               self.seq_lens, offsets)
                attn = ko.decode_batch(cache, q.reshape(n, g.nh, g.d), self.block_tables, self.seq_lens + 1)
                attn16 = attn.astype(np.float16).reshape(n, g.nh * g.d)
                parts.append(self._gemv(lw["o"], attn16))
            proj = parts[0] if world == 1 else _sum_partials(parts)
            x, normed = ko.residual_rmsnorm(x, proj, self.weights.layers[l]["ffn_norm"], s.norm_eps)
            parts = []
            for r in range(world):
                lw = self.shards[r][l]
                mid = ko.silu_mul(self._gemv(lw["gate_up"], normed))
                parts.append(self._gemv(lw["down"], mid))
            delta = parts[0] if world == 1 else _sum_partials(parts)
        x, normed = ko.residual_rmsnorm(x, delta, self.weights.final_norm, s.norm_eps)
        logits = self._gemv(self.weights.lm_head, normed)
        self.seq_lens = self.seq_lens + 1
        return ko.argmax(logits), logits
