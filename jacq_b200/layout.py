"""Byte accounting of the int4-KIVI page layout, for any (block, group, residual) geometry.

Mirror of the reference's ``integrations/vllm_kivi/layout.py`` (``KiviModelGeometry`` :22-40,
``KiviPageLayout`` :43-154): same class and attribute names, same numbers on the reference lane
(40,960 B quantised vs 131,072 B fp16 per layer-page; ``tests/test_layout_and_scaffold.py:162-174``
of the reference). What is new is ``validate_for_b200_lane``: a key group may span several pages
(``group_size % block_size == 0``); the reference's ``validate_for_vllm_lane`` keeps its rules.
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass


@dataclass(frozen=True)
class KiviModelGeometry:
    name: str
    num_layers: int
    num_attention_heads: int
    num_kv_heads: int
    head_dim: int
    dtype_bytes: int = 2

    @classmethod
    def qwen25_coder_32b(cls) -> "KiviModelGeometry":
        return cls("Qwen2.5-Coder-32B-Instruct", 64, 40, 8, 128)

    @classmethod
    def tinyllama_1b(cls) -> "KiviModelGeometry":
        return cls("TinyLlama-1.1B", 22, 32, 4, 64)

    @classmethod
    def qwen25_05b(cls) -> "KiviModelGeometry":
        return cls("Qwen2.5-0.5B", 24, 14, 2, 64)

    @classmethod
    def mistral_7b(cls) -> "KiviModelGeometry":
        return cls("Mistral-7B", 32, 32, 8, 128)

    @classmethod
    def qwen25_14b(cls) -> "KiviModelGeometry":
        return cls("Qwen2.5-14B", 48, 40, 8, 128)


@dataclass(frozen=True)
class KiviPageLayout:
    geometry: KiviModelGeometry
    block_size: int = 32
    group_size: int = 32
    nbits: int = 4
    residual_tokens: int = 128
    scale_zero_bytes: int = 4  # fp16 scale + fp16 zero

    # ---- validation -------------------------------------------------------------------------
    def validate_for_vllm_lane(self) -> None:
        """The reference lane's rules (layout.py:51-69 of the reference), with its messages."""
        d = self.geometry.head_dim
        rules = (
            (self.nbits == 4, f"first KIVI lane is int4 only, got nbits={self.nbits}"),
            (self.block_size == self.group_size,
             "KIVI key grouping must not straddle vLLM pages in the first serving lane; "
             f"require block_size==group_size, got {self.block_size}!={self.group_size}"),
            (self.block_size == 32, f"first vLLM KIVI lane requires block_size=32, got {self.block_size}"),
            (d % self.group_size == 0, f"head_dim={d} must be divisible by group_size={self.group_size}"),
            (self.residual_tokens % self.block_size == 0,
             f"residual_tokens={self.residual_tokens} must be page-aligned for the first lane"),
        )
        for holds, message in rules:
            if not holds:
                raise ValueError(message)

    def validate_for_b200_lane(self) -> None:
        """Rules of the generalised layout the B200 library implements (ABI v2)."""
        g = self.geometry
        if self.nbits != 4:
            raise ValueError(f"int4 only, got nbits={self.nbits}")
        if self.block_size <= 0 or self.group_size <= 0 or self.residual_tokens < 0:
            raise ValueError("block_size and group_size must be positive, residual_tokens >= 0")
        if self.group_size % self.block_size:
            raise ValueError(
                f"a key group must cover whole pages: group_size={self.group_size} "
                f"is not a multiple of block_size={self.block_size}")
        if g.num_attention_heads % g.num_kv_heads:
            raise ValueError("num_attention_heads must be a multiple of num_kv_heads")
        if g.head_dim % 8 or g.head_dim > 256:
            raise ValueError(f"head_dim={g.head_dim} must be a multiple of 8, at most 256")
        if g.head_dim % self.value_group_width or self.value_group_width % 8:
            raise ValueError(
                f"head_dim={g.head_dim} must split into value groups of width {self.value_group_width}")

    # ---- derived sizes ----------------------------------------------------------------------
    @property
    def value_group_width(self) -> int:
        return min(self.group_size, self.geometry.head_dim)

    @property
    def hd_groups(self) -> int:
        return math.ceil(self.geometry.head_dim / self.group_size)

    @property
    def scratch_rows(self) -> int:
        return self.residual_tokens + self.group_size

    @property
    def pages_per_group(self) -> int:
        return self.group_size // self.block_size

    def split_old_tokens(self, seq_len: int) -> int:
        """Tokens held as int4 pages at this length (whole key groups past the residual)."""
        return max(0, seq_len - self.residual_tokens) // self.group_size * self.group_size

    def old_pages(self, seq_len: int) -> int:
        return self.split_old_tokens(seq_len) // self.block_size

    @property
    def elems_per_token(self) -> int:
        return self.geometry.num_kv_heads * self.geometry.head_dim

    @property
    def fp16_page_bytes_per_layer(self) -> int:
        return 2 * self.block_size * self.elems_per_token * self.geometry.dtype_bytes

    @property
    def code_page_bytes_per_component(self) -> int:
        return self.block_size * self.elems_per_token * self.nbits // 8

    @property
    def key_param_page_bytes(self) -> int:
        # one scale/zero pair per channel per page; a group spanning several pages repeats it
        return math.ceil(self.block_size / self.group_size) * self.elems_per_token * self.scale_zero_bytes

    @property
    def value_param_page_bytes(self) -> int:
        return self.block_size * self.geometry.num_kv_heads * self.hd_groups * self.scale_zero_bytes

    @property
    def quantized_page_bytes_per_layer(self) -> int:
        return 2 * self.code_page_bytes_per_component + self.key_param_page_bytes + self.value_param_page_bytes

    @property
    def residual_pages(self) -> int:
        return self.residual_tokens // self.block_size

    def effective_bytes_per_layer(self, seq_len: int) -> int:
        pages = math.ceil(seq_len / self.block_size)
        residual_pages = min(self.residual_pages, pages)
        return (max(0, pages - residual_pages) * self.quantized_page_bytes_per_layer
                + residual_pages * self.fp16_page_bytes_per_layer)

    def effective_bytes_per_token_all_layers(self, seq_len: int) -> float:
        return self.effective_bytes_per_layer(seq_len) * self.geometry.num_layers / seq_len

    def fp16_bytes_per_token_all_layers(self) -> int:
        return 2 * self.elems_per_token * self.geometry.dtype_bytes * self.geometry.num_layers

    def capacity_ratio_vs_fp16(self, seq_len: int) -> float:
        return self.fp16_bytes_per_token_all_layers() / self.effective_bytes_per_token_all_layers(seq_len)

    def decode_algorithmic_bytes(self, seq_len: int) -> int:
        """Bytes one decode step of ONE sequence must move for one layer: int4 codes and value
        params once per kv head, key params once per group, the fp16 residual rows, q, the fp32
        output and the block-table entries."""
        g = self.geometry
        t_old = self.split_old_tokens(seq_len)
        t_res = seq_len - t_old
        qpk = g.num_attention_heads // g.num_kv_heads
        per_head = (2 * t_old * g.head_dim // 2
                    + (t_old // self.group_size) * g.head_dim * 4
                    + t_old * self.hd_groups * 4
                    + 2 * t_res * g.head_dim * 2
                    + qpk * g.head_dim * 2 + qpk * g.head_dim * 4)
        return g.num_kv_heads * per_head + math.ceil(t_old / self.block_size) * 4

    def to_abi_dict(self, seq_len: int = 4096) -> dict[str, object]:
        """The layout as the ABI report carries it (keys of the reference's report, layout.py:134-154, plus the
        decode bytes)."""
        self.validate_for_b200_lane()
        out: dict[str, object] = {"geometry": asdict(self.geometry)}
        for name in ("block_size", "group_size", "nbits", "residual_tokens", "fp16_page_bytes_per_layer",
                     "quantized_page_bytes_per_layer"):
            out[name] = getattr(self, name)
        out["key_code_bytes"] = out["value_code_bytes"] = self.code_page_bytes_per_component
        out["key_scale_zero_bytes"] = self.key_param_page_bytes
        out["value_scale_zero_bytes"] = self.value_param_page_bytes
        out["residual_pages"] = self.residual_pages
        out["effective_bytes_per_token_all_layers_at_seq_len"] = self.effective_bytes_per_token_all_layers(seq_len)
        out["capacity_ratio_vs_fp16_at_seq_len"] = self.capacity_ratio_vs_fp16(seq_len)
        out["decode_algorithmic_bytes_at_seq_len"] = self.decode_algorithmic_bytes(seq_len)
        return out
