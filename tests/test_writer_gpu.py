"""GPU parity of the cache writer: packed codes, block layout, fp16 scales/zeros and the live
scratch rows are compared BIT-EXACTLY with the CPU oracle (and, on the reference lane, with the
reference's own hand-CUDA writer compiled from its sources)."""
import ctypes

import numpy as np
import pytest
import torch

from tests import helpers
from oracle import kivi_oracle as ko

pytestmark = pytest.mark.gpu


def _run_v2_schedule(case, chunks_per_step, num_seqs, poison=0xAA):
    from jacq_b200.cache import KiviCache
    from tests.gpu_utils import DEV, f16_tensor
    geom = helpers.oracle_geometry(case)
    total = [sum(step[i] for step in chunks_per_step) for i in range(num_seqs)]
    pages_per_seq = (max(total) + max(max(st) for st in chunks_per_step)) // case.b + 1
    num_blocks = num_seqs * pages_per_seq + 3
    tables = helpers.shuffled_block_tables(num_seqs, pages_per_seq, num_blocks)
    slot_ids = np.random.default_rng(5).permutation(num_seqs + 2)[:num_seqs].astype(np.int32)
    oc = ko.OracleCache(geom, num_blocks, num_seqs + 2, fill=poison)
    cache = KiviCache(helpers.layout_of(case), num_blocks, num_seqs + 2, pages_per_seq, DEV, fill=poison)
    full_tables = np.zeros((num_seqs + 2, pages_per_seq), np.int32)
    full_tables[slot_ids] = tables
    cache.set_block_tables(torch.from_numpy(full_tables))
    k_all, v_all = zip(*[helpers.make_kv(case, total[i], stream=i) for i in range(num_seqs)])
    lens = np.zeros(num_seqs, np.int32)
    slots_t = torch.from_numpy(slot_ids).to(DEV)
    for step, counts in enumerate(chunks_per_step):
        counts = np.asarray(counts, np.int32)
        offs = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        nk = np.concatenate([k_all[i][lens[i]:lens[i] + counts[i]] for i in range(num_seqs)])
        nv = np.concatenate([v_all[i][lens[i]:lens[i] + counts[i]] for i in range(num_seqs)])
        if len(nk) == 0:
            continue
        ko.write_batch(oc, nk, nv, tables, lens, offs, slot_ids)
        cache.write(f16_tensor(nk), f16_tensor(nv), torch.from_numpy(offs).to(DEV),
                    max_new_per_seq=int(counts.max()), max_start_seq_len=int(lens.max()), slot_ids=slots_t)
        lens = lens + counts
        torch.cuda.synchronize()
        live = [0] * (num_seqs + 2)
        for i in range(num_seqs):
            live[slot_ids[i]] = int(lens[i] - geom.split_old(int(lens[i])))
        helpers.assert_cache_equal(cache.tensors, oc, live_rows=live, what=f"step {step}: ")
        got_lens = cache.seq_lens.cpu().numpy()
        assert np.array_equal(got_lens[slot_ids], lens)
    return cache, oc


@pytest.mark.parametrize("name", ["tinyllama", "qwen05b", "mistral7b", "reflane"])
def test_v2_writer_ragged_chunks_bit_exact(native_lib, name):
    """Every sequence gets a different chunk size each step: single tokens, chunks that end on,
    just before and just after a group boundary, and chunks that cross several boundaries."""
    case = helpers.CONFIGS[name]
    g, r = case.g, case.r
    steps = [
        [1, 2, g - 1, g],
        [r - 1, r, r + 1, 1],
        [g, g + 1, 1, r + g],
        [1, 1, 1, 1],
        [3 * g + 5, 2, g - 1, 0],
        [1, 512, 7, g],
        [g - 6, 1, 2 * g, 1],
    ]
    _run_v2_schedule(case, steps, 4)


def test_v2_writer_single_token_steps_cross_every_boundary(native_lib):
    """Token-by-token decode writes from empty through three age-outs (config 1 geometry)."""
    case = helpers.CONFIGS["tinyllama"]
    n = case.r + 3 * case.g + 2
    _run_v2_schedule(case, [[1, 1]] * n, 2)


def _ref_lane_inputs(tokens, nkv=8):
    case = helpers.CONFIGS["reflane"]
    case = helpers.Case(case.name, nkv * 5, nkv, case.d, case.b, case.g, case.r, 1, tokens, 3)
    k, v = helpers.make_kv(case, tokens)
    geom = helpers.oracle_geometry(case)
    pages = geom.split_old(tokens) // case.b
    table = helpers.shuffled_block_tables(1, 124, 130)[0]
    return case, geom, k, v, pages, table


@pytest.mark.parametrize("nkv", [8, 4])
def test_v1_writers_match_oracle_and_reference_cuda(native_lib, ref_lib, nkv):
    """jac_launch_cache_write / kivi_b200_cache_write_launch, token by token over 5 age-outs,
    against the oracle and against the reference's hand-CUDA writer on the same GPU."""
    from jacq_b200 import kivi_dsl
    from tests.gpu_utils import DEV, f16_tensor, ptr, stream_ptr, cache_ptrs
    tokens = 128 + 32 * 5 + 9
    case, geom, k, v, pages, table = _ref_lane_inputs(tokens, nkv)
    oc = ko.OracleCache(geom, 130, 1, fill=0x5A)
    mine = kivi_dsl.make_cache_bundle(130, num_kv_heads=nkv, device=DEV, fill=0x5A)
    theirs = kivi_dsl.make_cache_bundle(130, num_kv_heads=nkv, device=DEV, fill=0x5A)
    bt = torch.from_numpy(table).to(DEV)
    slot_mapping = torch.zeros(1, dtype=torch.int64, device=DEV)
    kd, vd = f16_tensor(k), f16_tensor(v)
    for t in range(tokens):
        ko.write_tokens(oc, k[t:t + 1], v[t:t + 1], table, t)
        kivi_dsl.require_kivi_cache_write(kd[t], vd[t], slot_mapping, bt, mine, t + 1)
        ref_lib.ref_kivi_cache_write_launch(*cache_ptrs(theirs), ptr(kd[t]), ptr(vd[t]), ptr(slot_mapping), ptr(bt),
                                            ctypes.c_int(t + 1), ctypes.c_int(nkv), stream_ptr())
        if t % 37 == 0 or t == tokens - 1 or (t + 1 - 128) % 32 == 0:
            torch.cuda.synchronize()
            live = [t + 1 - geom.split_old(t + 1)]
            helpers.assert_cache_equal(theirs, oc, live_rows=live, what=f"reference vs oracle, token {t}: ")
            helpers.assert_cache_equal(mine, oc, live_rows=live, what=f"b200 vs oracle, token {t}: ")


def test_v1_jac_dsl_selector_and_batched_writer(native_lib, ref_lib, monkeypatch):
    """The jac_dsl selector (jac_launch_cache_write) and the batched writers, with chunks planned
    by plan_batched_write, equal the token-by-token oracle; the reference's batched writer agrees."""
    from jacq_b200 import kivi_dsl
    from tests.gpu_utils import DEV, f16_tensor, ptr, stream_ptr, cache_ptrs
    tokens = 128 + 32 * 4 + 17
    case, geom, k, v, pages, table = _ref_lane_inputs(tokens)
    oc = ko.OracleCache(geom, 130, 1, fill=0x11)
    ko.write_tokens(oc, k, v, table, 0)
    bt = torch.from_numpy(table).to(DEV)
    slot_mapping = torch.zeros(1, dtype=torch.int64, device=DEV)
    kd, vd = f16_tensor(k), f16_tensor(v)
    live = [tokens - geom.split_old(tokens)]

    monkeypatch.setenv(kivi_dsl.CACHE_WRITE_KERNEL_ENV, "jac_dsl")
    a = kivi_dsl.make_cache_bundle(130, device=DEV, fill=0x11)
    for t in range(tokens):
        kivi_dsl.require_kivi_cache_write(kd[t], vd[t], slot_mapping, bt, a, t + 1)
    torch.cuda.synchronize()
    helpers.assert_cache_equal(a, oc, live_rows=live, what="jac_dsl single: ")

    b = kivi_dsl.make_cache_bundle(130, device=DEV, fill=0x11)
    c = kivi_dsl.make_cache_bundle(130, device=DEV, fill=0x11)
    for piece in kivi_dsl.plan_batched_write(0, tokens):
        s, n = piece.start_seq_len, piece.num_new
        kivi_dsl.require_kivi_cache_write_batched(kd[s:s + n], vd[s:s + n], slot_mapping, bt, b, s, n)
        ref_lib.ref_kivi_cache_write_batched_launch(*cache_ptrs(c), ptr(kd[s:s + n]), ptr(vd[s:s + n]),
                                                    ptr(slot_mapping), ptr(bt), ctypes.c_int(s), ctypes.c_int(n),
                                                    ctypes.c_int(8), stream_ptr())
    torch.cuda.synchronize()
    helpers.assert_cache_equal(b, oc, live_rows=live, what="b200 batched (planned): ")
    helpers.assert_cache_equal(c, oc, live_rows=live, what="reference batched (planned): ")

    # unplanned chunks of up to 160 rows may cross several boundaries in one call
    d = kivi_dsl.make_cache_bundle(130, device=DEV, fill=0x11)
    s = 0
    for n in [100, 160, 1, 12]:
        kivi_dsl.require_kivi_cache_write_batched(kd[s:s + n], vd[s:s + n], slot_mapping, bt, d, s, n)
        s += n
    assert s == tokens
    torch.cuda.synchronize()
    helpers.assert_cache_equal(d, oc, live_rows=live, what="b200 batched (unplanned): ")


def test_writer_edge_values_bit_exact(native_lib, ref_lib):
    """Constant groups (scale -> 1), all-zero groups with mixed signs, NaN and Inf lanes, the
    fp16 extremes: the three writers agree bit for bit."""
    from jacq_b200 import kivi_dsl
    from tests.gpu_utils import DEV, f16_tensor, ptr, stream_ptr, cache_ptrs
    tokens = 128 + 32 * 2
    case, geom, k, v, pages, table = _ref_lane_inputs(tokens)
    k = k.copy(); v = v.copy()
    k[:, 0, 0] = np.float16(1.5)                       # constant channel
    k[:, 0, 1] = np.float16(0.0); k[::2, 0, 1] = np.float16(-0.0)   # zeros of mixed sign
    k[:, 0, 2] = np.float16(np.nan)                    # all NaN
    k[5, 0, 3] = np.float16(np.nan)                    # one NaN
    k[7, 0, 4] = np.float16(np.inf); k[9, 0, 5] = np.float16(-np.inf)
    k[:, 0, 6] = np.float16(65504.0); k[::3, 0, 6] = np.float16(-65504.0)
    k[:, 0, 7] = np.float16(6e-8)                      # subnormal
    v[3, 1, :32] = np.float16(2.0)                     # constant value group
    v[4, 1, :32] = np.float16(0.0); v[4, 1, 1:32:2] = np.float16(-0.0)
    v[5, 1, 32:64] = np.float16(np.nan)
    v[6, 1, 64] = np.float16(np.nan)
    v[8, 1, 96] = np.float16(np.inf)
    v[10, 2, 0] = np.float16(65504.0); v[10, 2, 1] = np.float16(-65504.0)
    oc = ko.OracleCache(geom, 130, 1, fill=0)
    ko.write_tokens(oc, k, v, table, 0)
    bt = torch.from_numpy(table).to(DEV)
    slot_mapping = torch.zeros(1, dtype=torch.int64, device=DEV)
    kd, vd = f16_tensor(k), f16_tensor(v)
    mine = kivi_dsl.make_cache_bundle(130, device=DEV)
    theirs = kivi_dsl.make_cache_bundle(130, device=DEV)
    for t in range(tokens):
        kivi_dsl.require_kivi_cache_write(kd[t], vd[t], slot_mapping, bt, mine, t + 1)
        ref_lib.ref_kivi_cache_write_launch(*cache_ptrs(theirs), ptr(kd[t]), ptr(vd[t]), ptr(slot_mapping), ptr(bt),
                                            ctypes.c_int(t + 1), ctypes.c_int(8), stream_ptr())
    torch.cuda.synchronize()
    live = [tokens - geom.split_old(tokens)]
    helpers.assert_cache_equal(theirs, oc, live_rows=live, what="reference vs oracle (edge values): ")
    helpers.assert_cache_equal(mine, oc, live_rows=live, what="b200 vs oracle (edge values): ")


def test_v2_writer_rejects_bad_arguments_on_the_host(native_lib):
    """Bad shapes / ranges come back as status codes before any launch."""
    from jacq_b200 import _native
    from jacq_b200.cache import KiviCache
    from tests.gpu_utils import DEV
    case = helpers.CONFIGS["tinyllama"]
    cache = KiviCache(helpers.layout_of(case), 8, 2, 2, DEV)
    nk = torch.zeros((4, case.nkv, case.d), dtype=torch.float16, device=DEV)
    offs = torch.tensor([0, 2, 4], dtype=torch.int32, device=DEV)
    with pytest.raises(_native.KiviStatusError) as e:   # table of 2 pages cannot hold 500 tokens
        cache.write(nk, nk, offs, max_new_per_seq=2, max_start_seq_len=500)
    assert e.value.status == 7
    with pytest.raises(TypeError):
        cache.write(nk.float(), nk, offs, max_new_per_seq=2, max_start_seq_len=0)
    three = torch.tensor([0, 1, 2, 4], dtype=torch.int32, device=DEV)
    with pytest.raises(_native.KiviStatusError) as e:   # 3 sequences, 2 slots
        cache.write(nk, nk, three, max_new_per_seq=2, max_start_seq_len=0)
    assert e.value.status == 3
