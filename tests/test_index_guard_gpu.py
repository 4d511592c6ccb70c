"""Page and slot ids that the kernels read from device memory are held against the pool sizes the caller
stated (kivi_cache.num_blocks / num_slots) before they become addresses. The pools in this test are allocated
LARGER than they are declared, so an id "outside the pool" still points into memory the test owns: a guard
that failed would show up as a modified page, never as a fault."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import kivi_oracle as ko
from tests import helpers

pytestmark = pytest.mark.gpu


def _counter(native_lib, fn):
    out = ctypes.c_uint32(0)
    assert fn(ctypes.byref(out)) == 0
    return int(out.value)


def test_writer_and_decode_refuse_ids_outside_the_declared_pools(native_lib):
    from jacq_b200.cache import KiviCache
    from tests.gpu_utils import DEV, f16_tensor
    case = helpers.CONFIGS["tinyllama"]
    geom = helpers.oracle_geometry(case)
    allocated, declared, slots_allocated, slots_declared = 64, 32, 4, 2
    pages, tokens = 4, case.r + case.g + 7            # one key group ages out on the way
    cache = KiviCache(helpers.layout_of(case), allocated, slots_allocated, pages, DEV, fill=0x5C)
    cache._struct.num_blocks, cache._struct.num_slots = declared, slots_declared
    tables = np.array([[3, 9, 17, 30], [5, 40, 6, 7]], np.int32)      # sequence 1 names page 40: outside the declared pool
    cache.set_block_tables(torch.from_numpy(tables))
    k0, v0 = helpers.make_kv(case, tokens, stream=0)
    k1, v1 = helpers.make_kv(case, tokens, stream=1)
    k, v = np.concatenate([k0, k1]), np.concatenate([v0, v1])
    offs = torch.tensor([0, tokens, 2 * tokens], dtype=torch.int32, device=DEV)
    before_w = _counter(native_lib, native_lib.kivi_b200_writer_rejected_indices)
    cache.write(f16_tensor(k), f16_tensor(v), offs, max_new_per_seq=tokens, max_start_seq_len=0)
    torch.cuda.synchronize()
    assert _counter(native_lib, native_lib.kivi_b200_writer_rejected_indices) > before_w
    # sequence 0 was written as the oracle writes it; nothing of sequence 1 landed anywhere
    oc = ko.OracleCache(geom, allocated, slots_allocated, fill=0x5C)
    ko.write_tokens(oc, k0, v0, tables[0], 0, slot=0)
    t = cache.tensors
    for name in helpers.PAGE_FIELDS:
        got, want = helpers.to_bits(getattr(t, name)), getattr(oc, helpers.ORACLE_FIELD[name])
        assert np.array_equal(got, want.reshape(got.shape)), name
    live = tokens - geom.split_old(tokens)
    assert np.array_equal(helpers.to_bits(t.K_RESIDUAL_SCRATCH)[0][:, :live], oc.k_scratch[0][:, :live])
    assert (helpers.to_bits(t.K_RESIDUAL_SCRATCH)[1] == 0x5C5C).all(), "the refused sequence's scratch slot was touched"

    # a slot id outside the declared slots: the second sequence is refused again, the first is appended to
    cache.seq_lens.copy_(torch.tensor([tokens, 0, 0, 0], dtype=torch.int32))
    one_k, one_v = helpers.make_kv(case, 2, stream=5)
    slot_ids = torch.tensor([0, 3], dtype=torch.int32, device=DEV)
    cache.block_tables[3].copy_(torch.tensor([5, 6, 7, 8], dtype=torch.int32))
    before_w = _counter(native_lib, native_lib.kivi_b200_writer_rejected_indices)
    cache.write(f16_tensor(one_k), f16_tensor(one_v), torch.tensor([0, 1, 2], dtype=torch.int32, device=DEV),
                max_new_per_seq=1, max_start_seq_len=tokens, slot_ids=slot_ids, advance=False)
    torch.cuda.synchronize()
    assert _counter(native_lib, native_lib.kivi_b200_writer_rejected_indices) > before_w
    assert (helpers.to_bits(t.K_RESIDUAL_SCRATCH)[3] == 0x5C5C).all()
    ko.write_tokens(oc, one_k[:1], one_v[:1], tables[0], tokens, slot=0)
    assert np.array_equal(helpers.to_bits(t.K_RESIDUAL_SCRATCH)[0][:, :live + 1], oc.k_scratch[0][:, :live + 1])

    # decode: the sequence with the bad page id reads page 0 instead and is counted; the good one is exact
    cache.seq_lens.copy_(torch.tensor([tokens + 1, tokens, 0, 0], dtype=torch.int32))
    q = helpers.make_q(case, 2)
    before_d = _counter(native_lib, native_lib.kivi_b200_decode_rejected_indices)
    out = cache.decode(f16_tensor(q), max_seq_len=tokens + 1)
    torch.cuda.synchronize()
    assert _counter(native_lib, native_lib.kivi_b200_decode_rejected_indices) > before_d
    want = ko.decode(oc, q[0], tables[0], tokens + 1, slot=0, mode=1)
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    assert (np.abs(got[0] - want) <= 1e-2 + 1e-2 * np.abs(want)).all()


def test_index_predicate_on_the_host():
    """The predicate is one unsigned compare: negative ids and ids at or past the pool size fail."""
    def in_pool(i, n):
        return (i & 0xFFFFFFFF) < (n & 0xFFFFFFFF)
    assert in_pool(0, 1) and in_pool(31, 32)
    assert not in_pool(32, 32) and not in_pool(-1, 32) and not in_pool(0, 0) and not in_pool(2**31 - 1, 64)
