"""Device-side helpers of the GPU tests (imported only when a CUDA device is present)."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from jacq_b200.cache import KiviCache
from tests import helpers
from oracle import kivi_oracle as ko

DEV = torch.device("cuda:0")


def f16_tensor(a: np.ndarray) -> torch.Tensor:
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.float16).to(DEV)
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def upload(oc: ko.OracleCache, case: helpers.Case, max_blocks_per_seq: int) -> KiviCache:
    """A device KiviCache holding exactly the oracle cache's bytes."""
    cache = KiviCache(helpers.layout_of(case), oc.num_blocks, oc.num_slots, max_blocks_per_seq, DEV)
    for name in cache.tensors.names():
        src = getattr(oc, helpers.ORACLE_FIELD[name])
        dst = getattr(cache.tensors, name)
        dst.copy_(f16_tensor(src).reshape(dst.shape) if src.dtype == np.uint16 else torch.from_numpy(src).to(DEV))
    return cache


def bundle_from_oracle(oc: ko.OracleCache) -> dict:
    """Reference-lane cache bundle (one sequence) with the oracle cache's bytes."""
    from jacq_b200 import kivi_dsl
    b = kivi_dsl.make_cache_bundle(oc.num_blocks, num_kv_heads=oc.geom.nkv, device=DEV)
    for name in kivi_dsl.CACHE_TENSORS:
        src = getattr(oc, helpers.ORACLE_FIELD[name])
        if name.endswith("SCRATCH"):
            src = src[0]
        b[name].copy_(f16_tensor(src) if src.dtype == np.uint16 else torch.from_numpy(src).to(DEV))
    return b


def oracle_copy(cache: KiviCache, case: helpers.Case, seqs):
    """Host copy (OracleCache) of the chosen sequences of a device cache, their pages renumbered densely;
    returns the copy and the matching block tables. Lets the CPU oracle decode what the library's writer built
    on the device without re-quantising the whole context on the host."""
    geom = helpers.oracle_geometry(case)
    pages = cache.max_blocks_per_seq
    seqs = list(seqs)
    idx = cache.block_tables[seqs].reshape(-1).long()
    oc = ko.OracleCache(geom, len(seqs) * pages, len(seqs))
    t = cache.tensors
    for name in helpers.PAGE_FIELDS:
        src = getattr(t, name).index_select(0, idx)
        getattr(oc, helpers.ORACLE_FIELD[name])[...] = helpers.to_bits(src)
    sel = torch.tensor(seqs, device=cache.device)
    oc.k_scratch[...] = helpers.to_bits(t.K_RESIDUAL_SCRATCH.index_select(0, sel))
    oc.v_scratch[...] = helpers.to_bits(t.V_RESIDUAL_SCRATCH.index_select(0, sel))
    tables = np.arange(len(seqs) * pages, dtype=np.int32).reshape(len(seqs), pages)
    return oc, tables


def ptr(t: torch.Tensor):
    return ctypes.c_void_p(t.data_ptr())


def stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream(DEV).cuda_stream)


def cache_ptrs(bundle: dict):
    from jacq_b200 import kivi_dsl
    return [ptr(bundle[n]) for n in kivi_dsl.CACHE_TENSORS]
