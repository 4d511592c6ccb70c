"""ABI v2 host layer: a paged int4-KIVI cache for many sequences and the two calls that act on it.

``KiviCache`` owns one layer's page pool and residual scratch slots as torch tensors in the
reference tensor layout (``integrations/vllm_kivi/bindings.py:105-118`` of the reference, with the
leading slot dimension vLLM adds to the scratch, ``source_patch.py:2260-2279``), hands out pages
like a block manager would, and keeps block tables and sequence lengths on the device.
``write`` and ``decode`` are one library call each for the whole batch; the reference instead
loops over requests and tokens in Python with two torch-op calls per token per layer
(``source_patch.py:3105-3288``).

torch is plumbing here (device memory, streams); all arithmetic is in libjacq_kivi_b200.so.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from jacq_b200 import _native
from jacq_b200.layout import KiviModelGeometry, KiviPageLayout


def _ptr(t: torch.Tensor | None):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream_ptr(device: torch.device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def geometry_struct(layout: KiviPageLayout) -> _native.KiviGeometry:
    g = layout.geometry
    return _native.KiviGeometry(g.num_attention_heads, g.num_kv_heads, g.head_dim, layout.block_size,
                                layout.group_size, layout.residual_tokens)


@dataclass
class KiviCacheTensors:
    K_CODE_PAGES: torch.Tensor
    K_SCALE_PAGES: torch.Tensor
    K_ZERO_PAGES: torch.Tensor
    V_CODE_PAGES: torch.Tensor
    V_SCALE_PAGES: torch.Tensor
    V_ZERO_PAGES: torch.Tensor
    K_RESIDUAL_SCRATCH: torch.Tensor
    V_RESIDUAL_SCRATCH: torch.Tensor

    def names(self):
        return tuple(self.__dataclass_fields__)


class KiviCache:
    """One layer's KIVI cache for up to ``num_slots`` live sequences."""

    def __init__(self, layout: KiviPageLayout, num_blocks: int, num_slots: int, max_blocks_per_seq: int,
                 device: torch.device | str = "cuda", fill: int | None = None):
        layout.validate_for_b200_lane()
        self.layout = layout
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("KiviCache needs a CUDA device; the KIVI kernels have no CPU path")
        g = layout.geometry
        nkv, d, b = g.num_kv_heads, g.head_dim, layout.block_size

        def alloc(shape, dtype):
            if fill is None:
                return torch.zeros(shape, dtype=dtype, device=self.device)
            t = torch.empty(shape, dtype=dtype, device=self.device)
            t.view(torch.uint8).fill_(fill)
            return t

        self.tensors = KiviCacheTensors(
            alloc((num_blocks, nkv, b, d // 2), torch.uint8),
            alloc((num_blocks, nkv, d), torch.float16),
            alloc((num_blocks, nkv, d), torch.float16),
            alloc((num_blocks, nkv, b, d // 2), torch.uint8),
            alloc((num_blocks, nkv, b, layout.hd_groups), torch.float16),
            alloc((num_blocks, nkv, b, layout.hd_groups), torch.float16),
            alloc((num_slots, nkv, layout.scratch_rows, d), torch.float16),
            alloc((num_slots, nkv, layout.scratch_rows, d), torch.float16),
        )
        self.num_blocks = num_blocks
        self.num_slots = num_slots
        self.max_blocks_per_seq = max_blocks_per_seq
        self.block_tables = torch.zeros((num_slots, max_blocks_per_seq), dtype=torch.int32, device=self.device)
        self.seq_lens = torch.zeros((num_slots,), dtype=torch.int32, device=self.device)
        self._geom = geometry_struct(layout)
        t = self.tensors
        self._struct = _native.KiviCacheStruct(
            t.K_CODE_PAGES.data_ptr(), t.K_SCALE_PAGES.data_ptr(), t.K_ZERO_PAGES.data_ptr(),
            t.V_CODE_PAGES.data_ptr(), t.V_SCALE_PAGES.data_ptr(), t.V_ZERO_PAGES.data_ptr(),
            t.K_RESIDUAL_SCRATCH.data_ptr(), t.V_RESIDUAL_SCRATCH.data_ptr(), num_blocks, num_slots)
        self._workspace: torch.Tensor | None = None
        self._workspace_key: tuple[int, int] | None = None
        # sparse-retained state: keep_mask[slot, logical page] is False for old pages that were dropped
        self.keep_mask = torch.ones((num_slots, max_blocks_per_seq), dtype=torch.bool, device=self.device)
        self._sparse = False

    # ---- page bookkeeping (host) ---------------------------------------------------------------
    def set_block_tables(self, tables: torch.Tensor) -> None:
        """Install block tables ``[num_slots, <= max_blocks_per_seq]`` (int32; host or device)."""
        tables = tables.to(device=self.device, dtype=torch.int32)
        self.block_tables.zero_()
        self.block_tables[: tables.shape[0], : tables.shape[1]] = tables

    def drop_pages(self, slot: int, logical_pages) -> list[int]:
        """Evict whole old pages of one sequence (the page-aware allocator's move,
        ``integrations/vllm_kivi/source_patch.py:1839-1900`` of the reference): later decodes skip them
        through a compact table; the writer keeps its dense table, whose entries for dropped pages are
        never read again. Returns the physical page ids that are now free for other sequences."""
        pages = torch.as_tensor(sorted({int(p) for p in logical_pages}), dtype=torch.long, device=self.device)
        if pages.numel() == 0:
            return []
        if int(pages.min()) < 0 or int(pages.max()) >= self.max_blocks_per_seq:
            raise ValueError("logical page outside the block table")
        self.keep_mask[slot, pages] = False
        self._sparse = True
        return [int(p) for p in self.block_tables[slot, pages].tolist()]

    def retained_tables(self, lens: torch.Tensor, tables: torch.Tensor, mask: torch.Tensor):
        """Compact tables and retained-page counts for the current lengths, built on the device:
        kept pages first (stable order), count = kept pages among each sequence's dense old pages."""
        lay = self.layout
        old = torch.clamp(lens.to(torch.int64) - lay.residual_tokens, min=0) // lay.group_size * lay.group_size
        dense_pages = (old // lay.block_size).to(torch.int64)
        idx = torch.arange(tables.shape[1], device=self.device)
        live = mask & (idx[None, :] < dense_pages[:, None])
        order = torch.argsort((~live).to(torch.int8), dim=1, stable=True)
        compact = torch.gather(tables, 1, order).contiguous()
        return compact, live.sum(dim=1).to(torch.int32).contiguous()

    def bytes_allocated(self) -> int:
        return sum(getattr(self.tensors, n).numel() * getattr(self.tensors, n).element_size()
                   for n in self.tensors.names())

    # ---- the two calls -------------------------------------------------------------------------
    def write(self, new_k: torch.Tensor, new_v: torch.Tensor, new_offsets: torch.Tensor, *, max_new_per_seq: int,
              max_start_seq_len: int, slot_ids: torch.Tensor | None = None, batch: int | None = None,
              start_seq_lens: torch.Tensor | None = None, advance: bool = True) -> None:
        """Append ``new_k/new_v [total_new, NKV, D]`` (fp16): sequence i takes rows
        ``new_offsets[i]:new_offsets[i+1]``. Sequence lengths are read from (and, with ``advance``,
        updated in) ``self.seq_lens`` on the device; nothing synchronises with the host."""
        if new_k.dtype != torch.float16 or new_v.dtype != torch.float16:
            raise TypeError("KIVI cache write expects fp16 key/value tensors")
        if new_offsets.dtype != torch.int32:
            raise TypeError("new_offsets must be torch.int32")
        if new_k.shape != new_v.shape or not new_k.is_contiguous() or not new_v.is_contiguous():
            raise RuntimeError("new_k/new_v must be contiguous tensors of equal shape [total_new, NKV, D]")
        n = int(new_offsets.numel() - 1) if batch is None else batch
        starts = self.seq_lens if start_seq_lens is None else start_seq_lens
        tables = self.block_tables
        if slot_ids is not None:
            if slot_ids.dtype != torch.int32:
                raise TypeError("slot_ids must be torch.int32")
            # tables and lengths are stored per slot; the library indexes them per batch row
            tables = self.block_tables.index_select(0, slot_ids.long())
            if start_seq_lens is None:
                starts = self.seq_lens.index_select(0, slot_ids.long())
        devices = {t.device for t in (new_k, new_v, new_offsets, starts, tables)}
        if devices != {self.device}:
            raise RuntimeError(f"KIVI cache-write tensors span devices: {devices}")
        rc = _native.lib().kivi_b200_cache_write(
            ctypes.byref(self._geom), ctypes.byref(self._struct), _ptr(new_k), _ptr(new_v), _ptr(tables),
            self.max_blocks_per_seq, _ptr(starts), _ptr(new_offsets), _ptr(slot_ids), n, max_new_per_seq,
            max_start_seq_len, _stream_ptr(self.device))
        _native.check(rc, "kivi_b200_cache_write")
        if advance and start_seq_lens is None:
            counts = new_offsets[1: n + 1] - new_offsets[:n]
            if slot_ids is None:
                self.seq_lens[:n] += counts
            else:
                self.seq_lens.index_add_(0, slot_ids.long(), counts)

    def workspace(self, batch: int, max_seq_len: int) -> tuple[torch.Tensor | None, int]:
        need = int(_native.lib().kivi_b200_decode_workspace_bytes(ctypes.byref(self._geom), batch, max_seq_len))
        if self._workspace is None or self._workspace.numel() < need:
            self._workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=self.device)
            rc = _native.lib().kivi_b200_decode_workspace_init(
                _ptr(self._workspace), self._workspace.numel(), _stream_ptr(self.device))
            _native.check(rc, "kivi_b200_decode_workspace_init")
        return self._workspace, self._workspace.numel()

    def decode(self, q: torch.Tensor, out: torch.Tensor | None = None, *, max_seq_len: int,
               slot_ids: torch.Tensor | None = None, seq_lens: torch.Tensor | None = None) -> torch.Tensor:
        """Decode attention for ``q [batch, NH, D]`` (fp16) -> ``out [batch, NH, D]``: fp32 as in the reference's
        launch contract, or fp16 when an fp16 ``out`` is passed (the form the O projection consumes)."""
        g = self.layout.geometry
        if q.dtype != torch.float16:
            raise TypeError("Q must be torch.float16")
        if q.dim() != 3 or q.shape[1] != g.num_attention_heads or q.shape[2] != g.head_dim or not q.is_contiguous():
            raise RuntimeError("Q must be a contiguous [batch, num_heads, head_dim] tensor")
        batch = q.shape[0]
        if out is None:
            out = torch.empty(q.shape, dtype=torch.float32, device=self.device)
        if out.dtype not in (torch.float32, torch.float16) or out.shape != q.shape or not out.is_contiguous():
            raise TypeError("O must be a contiguous torch.float32 (or float16) tensor shaped like Q")
        lens = self.seq_lens if seq_lens is None else seq_lens
        tables = self.block_tables
        if slot_ids is not None:
            tables = self.block_tables.index_select(0, slot_ids.long())
            if seq_lens is None:
                lens = self.seq_lens.index_select(0, slot_ids.long())
        if lens.dtype != torch.int32:
            raise TypeError("SEQ_LENS must be torch.int32")
        ws, ws_bytes = self.workspace(batch, max_seq_len)
        if self._sparse:
            if out.dtype != torch.float32:
                raise TypeError("the sparse-retained decode writes fp32 output only")
            mask = self.keep_mask if slot_ids is None else self.keep_mask.index_select(0, slot_ids.long())
            compact, counts = self.retained_tables(lens[:batch], tables[:batch], mask[:batch])
            rc = _native.lib().kivi_b200_decode_sparse(
                ctypes.byref(self._geom), ctypes.byref(self._struct), _ptr(q), _ptr(compact), self.max_blocks_per_seq,
                _ptr(lens), _ptr(counts), _ptr(slot_ids), batch, max_seq_len, _ptr(out), _ptr(ws), ws_bytes,
                _stream_ptr(self.device))
            _native.check(rc, "kivi_b200_decode_sparse")
            return out
        call = _native.lib().kivi_b200_decode if out.dtype == torch.float32 else _native.lib().kivi_b200_decode_f16
        rc = call(ctypes.byref(self._geom), ctypes.byref(self._struct), _ptr(q), _ptr(tables), self.max_blocks_per_seq,
                  _ptr(lens), _ptr(slot_ids), batch, max_seq_len, _ptr(out), _ptr(ws), ws_bytes, _stream_ptr(self.device))
        _native.check(rc, "kivi_b200_decode")
        return out


def gemv(w: torch.Tensor, x: torch.Tensor, *, out_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """``y = W x`` for fp16 ``W [out, in]`` and ``x [in]`` or ``[batch, in]`` (the generated
    runtime's ``gemv()``, ``crates/jac-codegen-cuda/src/templates/runtime.cu:15-26`` of the
    reference). ``out_dtype`` float16 is the runtime form, float32 the kernel-DSL form."""
    if w.dtype != torch.float16 or x.dtype != torch.float16:
        raise TypeError("gemv expects fp16 W and x")
    if not w.is_contiguous() or not x.is_contiguous():
        raise RuntimeError("gemv expects contiguous tensors")
    x2 = x.reshape(-1, x.shape[-1])
    out_dim, in_dim = w.shape
    if x2.shape[1] != in_dim:
        raise RuntimeError("x does not match W's inner dimension")
    y = torch.empty((x2.shape[0], out_dim), dtype=out_dtype, device=w.device)
    y16 = _ptr(y) if out_dtype == torch.float16 else None
    y32 = _ptr(y) if out_dtype == torch.float32 else None
    if y16 is None and y32 is None:
        raise TypeError("out_dtype must be float16 or float32")
    rc = _native.lib().kivi_b200_gemv_f16(_ptr(w), _ptr(x2), y16, y32, out_dim, in_dim, x2.shape[0],
                                          _stream_ptr(w.device))
    _native.check(rc, "kivi_b200_gemv_f16")
    return y.reshape(x.shape[:-1] + (out_dim,))


def model_layout(name: str) -> KiviPageLayout:
    """Layouts of the benchmark configurations."""
    table = {
        "tinyllama": KiviPageLayout(KiviModelGeometry.tinyllama_1b(), 16, 32, 4, 32),
        "qwen2.5-0.5b": KiviPageLayout(KiviModelGeometry.qwen25_05b(), 16, 32, 4, 32),
        "mistral-7b": KiviPageLayout(KiviModelGeometry.mistral_7b(), 16, 128, 4, 128),
        "qwen2.5-14b": KiviPageLayout(KiviModelGeometry.qwen25_14b(), 16, 128, 4, 128),
        "reference-lane": KiviPageLayout(KiviModelGeometry.qwen25_coder_32b(), 32, 32, 4, 128),
    }
    return table[name]
