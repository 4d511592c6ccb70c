"""Decode runtime around the KIVI cache: the host side of ``kivi_b200_decode_step``.

The reference's generated runtime (crates/jac-codegen-cuda/src/templates/runtime.cu) is a C++
``main()`` that loads ``layerNN_*.bin`` files, allocates its buffers and calls ``forward()`` once
per token. ``DecodeRuntime`` is the same thing for a batch of sequences on one GPU (or one rank of
a KV-head tensor-parallel group): it keeps the weights in the reference's file layout, one
``KiviCache`` page pool per layer, the block tables and sequence lengths on the device, and runs a
whole step with one library call, optionally replayed from a CUDA graph. With ``world > 1`` the
two all-reduces per layer and the arg-max gather go either through ``torch.distributed`` (NCCL) on
the step's stream, called back from the library (``comm="nccl"``), or through the library's own
peer-memory exchange over NVLink (``comm="p2p"``: plain peer stores, flags, the sum fused into the
consuming kernel).

torch is plumbing here (device memory, streams, process group); all arithmetic is in
libjacq_kivi_b200.so.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from pathlib import Path

import torch

from jacq_b200 import _native
from jacq_b200.cache import KiviCache, _ptr, _stream_ptr
from jacq_b200.layout import KiviModelGeometry, KiviPageLayout


@dataclass(frozen=True)
class DecodeModelConfig:
    """``Config`` of the generated runtime (crates/jac-codegen-cuda/src/lib.rs:114-136) plus the KIVI page geometry."""
    name: str
    layers: int
    hidden: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    rope_base: float = 10000.0
    norm_eps: float = 1e-5
    attn_bias: bool = False
    block_size: int = 16
    group_size: int = 128
    residual: int = 128

    @property
    def q_dim(self) -> int:
        return self.num_q_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def qkv_out(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    @classmethod
    def qwen25_14b(cls) -> "DecodeModelConfig":
        return cls("Qwen2.5-14B", 48, 5120, 40, 8, 128, 13824, 152064, rope_base=1000000.0, norm_eps=1e-6,
                   attn_bias=True)

    def weight_bytes(self, world: int = 1) -> int:
        """fp16 bytes one rank streams per step (layer matrices sharded, lm_head sharded by rows)."""
        per_layer = (self.qkv_out + self.q_dim + 3 * self.ffn) * self.hidden
        return 2 * (self.layers * per_layer + self.vocab * self.hidden) // world

    def layer_files(self, layer: int) -> dict[str, tuple[str, tuple[int, ...]]]:
        """File names and shapes of one layer in the reference's weight directory
        (templates/export.py:69-92; loader runtime.cu:59-97)."""
        p = f"layer{layer:02d}_"
        files = {
            "attn_norm": (p + "attn_norm.bin", (self.hidden,)),
            "qkv": (p + "qkv.bin", (self.qkv_out, self.hidden)),
            "o": (p + "o.bin", (self.hidden, self.q_dim)),
            "ffn_norm": (p + "ffn_norm.bin", (self.hidden,)),
            "gate_up": (p + "gate_up.bin", (2 * self.ffn, self.hidden)),
            "down": (p + "down.bin", (self.hidden, self.ffn)),
        }
        if self.attn_bias:
            files["qkv_bias"] = (p + "qkv_bias.bin", (self.qkv_out,))
        return files


def load_weight_dir(cfg: DecodeModelConfig, directory: str | Path) -> dict[str, object]:
    """Read a weight directory written by the reference exporter (raw little-endian fp16 ``.bin`` files)."""
    import numpy as np

    d = Path(directory)

    def read(name: str, shape: tuple[int, ...]) -> torch.Tensor:
        a = np.fromfile(d / name, dtype=np.float16)
        want = 1
        for s in shape:
            want *= s
        if a.size != want:
            raise RuntimeError(f"short read {d / name}: {a.size}/{want}")
        return torch.from_numpy(a.reshape(shape))

    out: dict[str, object] = {
        "embed": read("embed.bin", (cfg.vocab, cfg.hidden)),
        "final_norm": read("final_norm.bin", (cfg.hidden,)),
        "lm_head": read("lm_head.bin", (cfg.vocab, cfg.hidden)),
        "layers": [],
    }
    for l in range(cfg.layers):
        out["layers"].append({k: read(n, s) for k, (n, s) in cfg.layer_files(l).items()})
    return out


def save_weight_dir(cfg: DecodeModelConfig, weights: dict[str, object], directory: str | Path) -> None:
    """Write weights in the reference's directory layout."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    for name in ("embed", "final_norm", "lm_head"):
        weights[name].cpu().numpy().tofile(d / f"{name}.bin")
    for l, lw in enumerate(weights["layers"]):
        for k, (n, _) in cfg.layer_files(l).items():
            lw[k].cpu().numpy().tofile(d / n)


def shard_rows(cfg: DecodeModelConfig, rank: int, world: int) -> dict[str, list[slice]]:
    """Row (q|k|v, gate|up) and column (o, down) slices of rank ``rank`` under KV-head tensor parallelism."""
    if cfg.num_kv_heads % world or cfg.ffn % world or cfg.vocab % world:
        raise ValueError(f"{cfg.name}: {world} ranks do not divide kv heads / ffn / vocab")
    hd = cfg.head_dim
    nh_l, nkv_l, ffn_l = cfg.num_q_heads // world, cfg.num_kv_heads // world, cfg.ffn // world
    q = slice(rank * nh_l * hd, (rank + 1) * nh_l * hd)
    k = slice(cfg.q_dim + rank * nkv_l * hd, cfg.q_dim + (rank + 1) * nkv_l * hd)
    v = slice(cfg.q_dim + cfg.kv_dim + rank * nkv_l * hd, cfg.q_dim + cfg.kv_dim + (rank + 1) * nkv_l * hd)
    gate = slice(rank * ffn_l, (rank + 1) * ffn_l)
    up = slice(cfg.ffn + rank * ffn_l, cfg.ffn + (rank + 1) * ffn_l)
    vocab_l = cfg.vocab // world
    return {"qkv": [q, k, v], "o_cols": [q], "gate_up": [gate, up], "down_cols": [gate],
            "lm_head": [slice(rank * vocab_l, (rank + 1) * vocab_l)]}


def shard_layer(cfg: DecodeModelConfig, lw: dict[str, torch.Tensor], rank: int, world: int) -> dict[str, torch.Tensor]:
    if world == 1:
        return dict(lw)
    s = shard_rows(cfg, rank, world)
    out = {
        "attn_norm": lw["attn_norm"], "ffn_norm": lw["ffn_norm"],
        "qkv": torch.cat([lw["qkv"][r] for r in s["qkv"]], 0).contiguous(),
        "o": lw["o"][:, s["o_cols"][0]].contiguous(),
        "gate_up": torch.cat([lw["gate_up"][r] for r in s["gate_up"]], 0).contiguous(),
        "down": lw["down"][:, s["down_cols"][0]].contiguous(),
    }
    if lw.get("qkv_bias") is not None:
        out["qkv_bias"] = torch.cat([lw["qkv_bias"][r] for r in s["qkv"]], 0).contiguous()
    return out


def random_layer(cfg: DecodeModelConfig, generator: torch.Generator, device, std: float = 0.02,
                 rank: int = 0, world: int = 1) -> dict[str, torch.Tensor]:
    """Random-init N(0, std) fp16 weights of one layer, already in the shard shapes of ``rank``."""
    nh_l, nkv_l, ffn_l = cfg.num_q_heads // world, cfg.num_kv_heads // world, cfg.ffn // world
    qkv_l = (nh_l + 2 * nkv_l) * cfg.head_dim

    def mat(rows, cols):
        return (torch.randn((rows, cols), generator=generator, device=device, dtype=torch.float32) * std).half()

    def norm():
        return (1.0 + 0.1 * torch.randn((cfg.hidden,), generator=generator, device=device)).half()

    lw = {"attn_norm": norm(), "qkv": mat(qkv_l, cfg.hidden), "o": mat(cfg.hidden, nh_l * cfg.head_dim),
          "ffn_norm": norm(), "gate_up": mat(2 * ffn_l, cfg.hidden), "down": mat(cfg.hidden, ffn_l)}
    if cfg.attn_bias:
        lw["qkv_bias"] = (torch.randn((qkv_l,), generator=generator, device=device) * 0.1).half()
    return lw


class DecodeRuntime:
    """One rank's weights, caches and step state for ``batch`` sequences.

    ``weights`` holds this rank's shard (``shard_layer`` / ``random_layer``): ``embed`` (full table),
    ``final_norm``, ``lm_head`` (this rank's rows) and ``layers`` (list of dicts). ``group`` is the
    ``torch.distributed`` process group of the tensor-parallel ranks (None for one GPU)."""

    def __init__(self, cfg: DecodeModelConfig, weights: dict[str, object], *, batch: int, max_seq_len: int,
                 device: torch.device | str = "cuda", rank: int = 0, world: int = 1, group=None,
                 block_tables: torch.Tensor | None = None, comm: str = "nccl"):
        self.cfg, self.batch, self.max_seq_len = cfg, batch, max_seq_len
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("DecodeRuntime needs a CUDA device; the kernels have no CPU path")
        if cfg.num_kv_heads % world or cfg.ffn % world or cfg.vocab % world:
            raise ValueError(f"{world} ranks do not divide kv heads / ffn / vocab of {cfg.name}")
        if world > 1 and group is None:
            raise ValueError("tensor parallelism needs a torch.distributed process group")
        self.rank, self.world, self.group = rank, world, group
        nh_l, nkv_l = cfg.num_q_heads // world, cfg.num_kv_heads // world
        geometry = KiviModelGeometry(cfg.name, cfg.layers, nh_l, nkv_l, cfg.head_dim)
        self.layout = KiviPageLayout(geometry, cfg.block_size, cfg.group_size, 4, cfg.residual)
        self.layout.validate_for_b200_lane()
        self.max_blocks_per_seq = max(1, -(-self.layout.split_old_tokens(max_seq_len) // cfg.block_size))
        num_blocks = batch * self.max_blocks_per_seq
        self.caches = [KiviCache(self.layout, num_blocks, batch, self.max_blocks_per_seq, self.device)
                       for _ in range(cfg.layers)]
        if block_tables is None:
            block_tables = torch.arange(num_blocks, dtype=torch.int32).reshape(batch, self.max_blocks_per_seq)
        self.block_tables = block_tables.to(device=self.device, dtype=torch.int32).contiguous()
        if self.block_tables.shape != (batch, self.max_blocks_per_seq):
            raise ValueError(f"block_tables must be [{batch}, {self.max_blocks_per_seq}]")
        self.seq_lens = torch.zeros((batch,), dtype=torch.int32, device=self.device)
        self.weights = self._to_device(weights)

        self._cfg_struct = _native.KiviStepConfig(
            cfg.layers, cfg.hidden, nh_l, nkv_l, cfg.head_dim, cfg.ffn // world, cfg.vocab // world,
            rank * (cfg.vocab // world), int(cfg.attn_bias), cfg.rope_base, cfg.norm_eps, cfg.block_size,
            cfg.group_size, cfg.residual, world, rank)
        self._layer_structs = (_native.KiviLayerWeights * cfg.layers)()
        for l, lw in enumerate(self.weights["layers"]):
            self._layer_structs[l] = _native.KiviLayerWeights(
                lw["attn_norm"].data_ptr(), lw["qkv"].data_ptr(),
                lw["qkv_bias"].data_ptr() if cfg.attn_bias else None, lw["o"].data_ptr(),
                lw["ffn_norm"].data_ptr(), lw["gate_up"].data_ptr(), lw["down"].data_ptr())
        self._weights_struct = _native.KiviStepWeights(
            self.weights["embed"].data_ptr(), self.weights["final_norm"].data_ptr(),
            self.weights["lm_head"].data_ptr(), self._layer_structs)
        self._cache_structs = (_native.KiviCacheStruct * cfg.layers)(*[c._struct for c in self.caches])
        need = int(_native.lib().kivi_b200_decode_step_workspace_bytes(ctypes.byref(self._cfg_struct), batch,
                                                                       max_seq_len))
        if need == 0:
            raise RuntimeError("kivi_b200_decode_step_workspace_bytes rejected the configuration")
        self.workspace = torch.zeros((need,), dtype=torch.uint8, device=self.device)
        self._state = _native.KiviStepState(
            self._cache_structs, self.block_tables.data_ptr(), self.max_blocks_per_seq, self.seq_lens.data_ptr(),
            None, self.workspace.data_ptr(), need)
        self.tokens = torch.zeros((batch,), dtype=torch.int32, device=self.device)
        self.logits = torch.empty((batch, cfg.vocab // world), dtype=torch.float16, device=self.device)
        if comm not in ("nccl", "p2p"):
            raise ValueError("comm must be 'nccl' (torch.distributed hooks) or 'p2p' (the library's peer-memory exchange)")
        self.comm_kind = comm
        self._region = None
        self._peer_regions: list[int] = []
        if world > 1:
            self._comm = self._make_p2p_comm() if comm == "p2p" else self._make_comm()
        else:
            self._comm = None
        self._graph: torch.cuda.CUDAGraph | None = None

    def _to_device(self, weights: dict[str, object]) -> dict[str, object]:
        def dev(t: torch.Tensor) -> torch.Tensor:
            if t.dtype != torch.float16:
                raise TypeError("weights must be fp16")
            return t.to(self.device).contiguous()

        out = {k: dev(weights[k]) for k in ("embed", "final_norm", "lm_head")}
        out["layers"] = [{k: dev(v) for k, v in lw.items() if v is not None} for lw in weights["layers"]]
        if len(out["layers"]) != self.cfg.layers:
            raise ValueError("weights['layers'] does not match the layer count")
        return out

    # ---- collectives (tensor parallelism) ---------------------------------------------------
    def _view(self, ptr: int, nbytes: int) -> torch.Tensor:
        """The slice of the workspace (or the logits) a library-side pointer refers to."""
        base = self.workspace.data_ptr()
        if not (base <= ptr and ptr + nbytes <= base + self.workspace.numel()):
            raise RuntimeError("collective buffer outside the step workspace")
        return self.workspace[ptr - base: ptr - base + nbytes]

    def _make_comm(self) -> _native.KiviStepComm:
        import torch.distributed as dist

        def allreduce(_user, buf, count, _stream):
            try:
                dist.all_reduce(self._view(buf, count * 2).view(torch.float16), group=self.group)
                return 0
            except Exception:   # the library turns a non-zero return into KIVI_ERR_CUDA
                return 1

        def allgather(_user, send, recv, nbytes, _stream):
            try:
                dist.all_gather_into_tensor(self._view(recv, nbytes * self.world), self._view(send, nbytes),
                                            group=self.group)
                return 0
            except Exception:
                return 1

        self._callbacks = (_native.ALLREDUCE_F16_FN(allreduce), _native.ALLGATHER_FN(allgather))  # keep alive
        return _native.KiviStepComm(self._callbacks[0], self._callbacks[1], None)

    def _make_p2p_comm(self) -> _native.KiviStepComm:
        """Create this rank's exchange region, swap IPC handles over the process group (host side,
        once) and map every peer's region. No collective library is involved in a step afterwards."""
        import torch.distributed as dist

        lib = _native.lib()
        nbytes = int(lib.kivi_b200_p2p_region_bytes(ctypes.byref(self._cfg_struct), self.batch))
        if nbytes == 0:
            raise RuntimeError("kivi_b200_p2p_region_bytes rejected the configuration")
        region = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * _native.P2P_HANDLE_BYTES)()
        _native.check(lib.kivi_b200_p2p_region_create(nbytes, ctypes.byref(region), handle), "kivi_b200_p2p_region_create")
        self._region = region.value
        handles: list[bytes | None] = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=self.group)
        ptrs = (ctypes.c_void_p * self.world)()
        for r, h in enumerate(handles):
            if r == self.rank:
                ptrs[r] = self._region
                continue
            peer = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * _native.P2P_HANDLE_BYTES).from_buffer_copy(h)
            _native.check(lib.kivi_b200_p2p_region_open(buf, ctypes.byref(peer)), "kivi_b200_p2p_region_open")
            ptrs[r] = peer.value
            self._peer_regions.append(peer.value)
        self._peer_array = ptrs   # keep alive
        dist.barrier(group=self.group)   # every region is mapped everywhere before anybody pushes
        null_ar = ctypes.cast(None, _native.ALLREDUCE_F16_FN)
        null_ag = ctypes.cast(None, _native.ALLGATHER_FN)
        return _native.KiviStepComm(null_ar, null_ag, None, ptrs, nbytes, 0)

    def exchange_status(self) -> int:
        """0 when every wait of the peer-memory exchange was served; bit r set when a wait for
        rank r ran out of polls (the step's result is then undefined)."""
        if self._region is None:
            return 0
        out = ctypes.c_uint32(0)
        _native.check(_native.lib().kivi_b200_p2p_status(self._region, ctypes.byref(out), _stream_ptr(self.device)),
                      "kivi_b200_p2p_status")
        return int(out.value)

    def close(self) -> None:
        """Unmap the peers' regions and free this rank's (call on every rank, after the last step)."""
        lib = _native.lib()
        torch.cuda.synchronize(self.device)
        for p in self._peer_regions:
            lib.kivi_b200_p2p_region_close(p)
        self._peer_regions = []
        if self._region is not None:
            if self.group is not None:
                import torch.distributed as dist
                dist.barrier(group=self.group)   # nobody frees while a peer still has the mapping open
            lib.kivi_b200_p2p_region_destroy(self._region)
            self._region = None

    # ---- stepping -----------------------------------------------------------------------------
    def set_seq_lens(self, lens) -> None:
        self.seq_lens.copy_(torch.as_tensor(lens, dtype=torch.int32))

    def _launch(self) -> None:
        rc = _native.lib().kivi_b200_decode_step(
            ctypes.byref(self._cfg_struct), ctypes.byref(self._weights_struct), ctypes.byref(self._state),
            _ptr(self.tokens), self.batch, self.max_seq_len, _ptr(self.tokens), _ptr(self.logits),
            ctypes.byref(self._comm) if self._comm is not None else None, _stream_ptr(self.device))
        _native.check(rc, "kivi_b200_decode_step")

    def capture(self) -> None:
        """Record the step into a CUDA graph; later ``step`` calls replay it. Nothing runs during the
        capture, so the caches and lengths are untouched; the graph stays valid while every sequence
        is shorter than ``max_seq_len``. With tensor parallelism the process group must have
        communicated once before (NCCL sets itself up on first use, which cannot be captured)."""
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize(self.device)
        with torch.cuda.graph(graph):
            self._launch()
        self._graph = graph

    def step(self, tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Feed one token per sequence (default: the previous step's arg-max) and return the
        device tensor of next-token ids; ``self.logits`` holds this rank's logit rows."""
        if tokens is not None:
            self.tokens.copy_(tokens.to(dtype=torch.int32))
        if self._graph is not None:
            self._graph.replay()
        else:
            self._launch()
        return self.tokens

    def kv_bytes_per_step(self, seq_len: int) -> int:
        """Algorithmic KV-cache bytes the attention of one step reads on this rank (all layers, all sequences)."""
        return self.cfg.layers * self.batch * self.layout.decode_algorithmic_bytes(seq_len)
