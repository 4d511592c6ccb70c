"""Tensor names, dtypes, shapes and launch order of the KIVI entry points.

Mirror of the reference's ``integrations/vllm_kivi/bindings.py`` (``TensorBinding`` :16-44,
``KiviDecodeBindingAbi`` :47-143): the v1 launch order is identical (it is pinned in the tests
against the C header, as the reference pins it against its emitted CUDA,
``tests/test_launch_signature.py:37-57``); shapes follow the generalised layout, so a key group may
cover several pages and the scratch holds ``residual + group`` rows.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

from jacq_b200.layout import KiviModelGeometry, KiviPageLayout

JAC_LAUNCH_ORDER = (
    "Q", "BLOCK_TABLE", "K_CODE_PAGES", "K_SCALE_PAGES", "K_ZERO_PAGES", "V_CODE_PAGES", "V_SCALE_PAGES",
    "V_ZERO_PAGES", "K_RESIDUAL_SCRATCH", "V_RESIDUAL_SCRATCH", "SEQ_LEN", "O", "cudaStream_t stream",
)
CACHE_TENSORS = JAC_LAUNCH_ORDER[2:10]


@dataclass(frozen=True)
class TensorBinding:
    """One argument of the launch: name, dtype, shape (an entry may be a symbol instead of a number), element size
    and what it holds. The per-layer counts are "dynamic" as soon as one dimension is symbolic."""
    name: str
    dtype: str
    shape: tuple[int | str, ...]
    bytes_per_element: int
    role: str

    def _static_numel(self) -> int | None:
        if any(isinstance(dim, str) for dim in self.shape):
            return None
        return math.prod(self.shape)

    @property
    def numel_per_layer(self) -> int | str:
        n = self._static_numel()
        return "dynamic" if n is None else n

    @property
    def bytes_per_layer(self) -> int | str:
        n = self._static_numel()
        return "dynamic" if n is None else n * self.bytes_per_element

    def to_dict(self) -> dict[str, object]:
        out: dict[str, object] = {"name": self.name, "dtype": self.dtype, "shape": list(self.shape),
                                  "bytes_per_element": self.bytes_per_element, "role": self.role}
        out["numel_per_layer"] = self.numel_per_layer
        out["bytes_per_layer"] = self.bytes_per_layer
        return out


@dataclass(frozen=True)
class KiviDecodeBindingAbi:
    """Tensors one decode launch binds for ONE sequence of ``seq_len`` tokens."""

    layout: KiviPageLayout
    seq_len: int = 4096
    num_blocks: int | None = None
    max_blocks_per_seq: int | None = None

    def __post_init__(self) -> None:
        self.layout.validate_for_b200_lane()
        if self.seq_len < 0:
            raise ValueError("seq_len must be non-negative")
        if self.num_blocks is not None and self.num_blocks <= 0:
            raise ValueError("num_blocks must be positive")
        if self.max_blocks_per_seq is not None and self.max_blocks_per_seq <= 0:
            raise ValueError("max_blocks_per_seq must be positive")

    @property
    def old_tokens(self) -> int:
        return self.layout.split_old_tokens(self.seq_len)

    @property
    def old_pages(self) -> int:
        return self.old_tokens // self.layout.block_size

    @property
    def physical_blocks(self) -> int:
        return self.num_blocks if self.num_blocks is not None else max(1, self.old_pages)

    @property
    def block_table_len(self) -> int:
        return self.max_blocks_per_seq if self.max_blocks_per_seq is not None else max(1, self.old_pages)

    @property
    def geometry(self) -> KiviModelGeometry:
        return self.layout.geometry

    @property
    def hd_packed(self) -> int:
        return self.geometry.head_dim * self.layout.nbits // 8

    @property
    def hd_groups(self) -> int:
        return self.layout.hd_groups

    def tensor_bindings(self) -> list[TensorBinding]:
        g, lay, b = self.geometry, self.layout, self.physical_blocks
        nh, nkv, d, bs = g.num_attention_heads, g.num_kv_heads, g.head_dim, lay.block_size
        rows = lay.scratch_rows
        return [
            TensorBinding("Q", "torch.float16", (nh, d), 2, "one decode query per attention head"),
            TensorBinding("BLOCK_TABLE", "torch.int32", (self.block_table_len,), 4, "logical old page -> physical page"),
            TensorBinding("K_CODE_PAGES", "torch.uint8", (b, nkv, bs, self.hd_packed), 1, "packed int4 key codes"),
            TensorBinding("K_SCALE_PAGES", "torch.float16", (b, nkv, d), 2, "key scales, per channel over the token group"),
            TensorBinding("K_ZERO_PAGES", "torch.float16", (b, nkv, d), 2, "key zeros, per channel over the token group"),
            TensorBinding("V_CODE_PAGES", "torch.uint8", (b, nkv, bs, self.hd_packed), 1, "packed int4 value codes"),
            TensorBinding("V_SCALE_PAGES", "torch.float16", (b, nkv, bs, self.hd_groups), 2, "value scales, per token per channel group"),
            TensorBinding("V_ZERO_PAGES", "torch.float16", (b, nkv, bs, self.hd_groups), 2, "value zeros, per token per channel group"),
            TensorBinding("K_RESIDUAL_SCRATCH", "torch.float16", (nkv, rows, d), 2, "fp16 key tail, residual + one group"),
            TensorBinding("V_RESIDUAL_SCRATCH", "torch.float16", (nkv, rows, d), 2, "fp16 value tail, residual + one group"),
            TensorBinding("SEQ_LEN", "int", (), 8, "valid sequence length"),
            TensorBinding("O", "torch.float32", (nh, d), 4, "decode output per attention head"),
        ]

    def jac_launch_order(self) -> list[str]:
        return list(JAC_LAUNCH_ORDER)

    def old_page_bytes_per_layer(self) -> int:
        return self.layout.quantized_page_bytes_per_layer * self.physical_blocks

    def residual_bytes_per_sequence_layer(self) -> int:
        g = self.geometry
        return 2 * g.num_kv_heads * self.layout.residual_tokens * g.head_dim * g.dtype_bytes

    def to_report(self) -> dict[str, object]:
        """JSON-serialisable summary (keys as in the reference's report, bindings.py:131-143)."""
        report: dict[str, object] = {name: getattr(self, name) for name in ("seq_len", "old_tokens", "old_pages", "block_table_len")}
        report["physical_blocks_reported"] = self.physical_blocks
        report["jac_launch_order"] = self.jac_launch_order()
        report["tensor_bindings"] = [binding.to_dict() for binding in self.tensor_bindings()]
        for name in ("old_page_bytes_per_layer", "residual_bytes_per_sequence_layer"):
            report[name] = getattr(self, name)()
        return report


def default_qwen32b_binding_abi(seq_len: int = 4096) -> KiviDecodeBindingAbi:
    return KiviDecodeBindingAbi(KiviPageLayout(KiviModelGeometry.qwen25_coder_32b()), seq_len=seq_len)
