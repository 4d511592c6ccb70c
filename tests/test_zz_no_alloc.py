"""The decode entry point for hosts that cannot allocate device memory.

Some programs that call this library own no CUDA allocator they may use at decode time: a serving
runtime that carved up all of HBM at start-up, a plugin invoked inside another framework's step, a
sandboxed C host. For them kivi_b200_decode_noalloc takes the split-context scratch from a fixed
array inside the library. This test drives it through the C ABI on a launch that really uses the
scratch (one long sequence, split over many CTAs) and checks, on two calls in a row, that it gives
what kivi_b200_decode gives with a caller-owned workspace (tolerance of the decode tests:
rtol = atol = 1e-2), and that a request beyond the fixed array is refused before anything launches.

Collected last on purpose: a run that stops at the first failure has by then run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import kivi_oracle as ko
from tests import helpers

pytestmark = pytest.mark.gpu

RTOL = ATOL = 1e-2
SCRATCH_BYTES = 1 << 20   # KIVI_B200_NOALLOC_SCRATCH_BYTES of include/jacq_kivi_b200.h


def _setup(case, seq_lens):
    from tests.gpu_utils import DEV, f16_tensor, upload
    geom = helpers.oracle_geometry(case)
    n = len(seq_lens)
    pages = max(1, max(geom.split_old(int(t)) for t in seq_lens) // case.b)
    tables = helpers.shuffled_block_tables(n, pages, n * pages + 3)
    oc = ko.OracleCache(geom, n * pages + 3, n)
    for i, t in enumerate(seq_lens):
        k, v = helpers.make_kv(case, int(t), stream=i)
        ko.write_tokens(oc, k, v, tables[i], 0, slot=i)
    cache = upload(oc, case, pages)
    cache.set_block_tables(torch.from_numpy(tables))
    cache.seq_lens.copy_(torch.from_numpy(np.asarray(seq_lens, np.int32)))
    q = f16_tensor(helpers.make_q(case, n))
    return oc, tables, cache, q


def _decode_noalloc(native_lib, cache, q, max_seq_len):
    from tests.gpu_utils import DEV, ptr, stream_ptr
    out = torch.full(q.shape, float("nan"), dtype=torch.float32, device=DEV)
    rc = native_lib.kivi_b200_decode_noalloc(
        ctypes.byref(cache._geom), ctypes.byref(cache._struct), ptr(q), ptr(cache.block_tables),
        cache.max_blocks_per_seq, ptr(cache.seq_lens), None, q.shape[0], max_seq_len, ptr(out), stream_ptr())
    return rc, out


def test_noalloc_decode_equals_workspace_decode_twice(native_lib):
    case = helpers.CONFIGS["mistral7b"]
    seq_lens = [case.r + 24 * case.g + 9, case.r + 3 * case.g]
    oc, tables, cache, q = _setup(case, seq_lens)
    max_len = max(seq_lens)
    need = native_lib.kivi_b200_decode_workspace_bytes(ctypes.byref(cache._geom), len(seq_lens), max_len)
    assert 4096 < need <= SCRATCH_BYTES, "the case must split the context and fit the fixed array"
    want = cache.decode(q, max_seq_len=max_len)
    torch.cuda.synchronize()
    oracle = ko.decode_batch(oc, helpers.to_bits(q), tables, np.asarray(seq_lens, np.int32), mode=1, nthreads=8)
    for call in range(2):
        rc, got = _decode_noalloc(native_lib, cache, q, max_len)
        torch.cuda.synchronize()
        assert rc == 0, f"call {call}: status {rc}"
        g, w = got.cpu().numpy(), want.cpu().numpy()
        assert np.isfinite(g).all(), f"call {call}: non-finite output"
        assert (np.abs(g - w) <= ATOL + RTOL * np.abs(w)).all(), f"call {call}: differs from kivi_b200_decode"
        assert (np.abs(g - oracle) <= ATOL + RTOL * np.abs(oracle)).all(), f"call {call}: differs from the oracle"
    # a different shape right after, sharing the same array, then the first one again
    case2 = helpers.CONFIGS["tinyllama"]
    lens2 = [case2.context] * 3
    oc2, tables2, cache2, q2 = _setup(case2, lens2)
    rc, got2 = _decode_noalloc(native_lib, cache2, q2, case2.context)
    torch.cuda.synchronize()
    assert rc == 0
    want2 = ko.decode_batch(oc2, helpers.to_bits(q2), tables2, np.asarray(lens2, np.int32), mode=1, nthreads=8)
    assert (np.abs(got2.cpu().numpy() - want2) <= ATOL + RTOL * np.abs(want2)).all()
    rc, again = _decode_noalloc(native_lib, cache, q, max_len)
    torch.cuda.synchronize()
    assert rc == 0
    w = want.cpu().numpy()
    assert (np.abs(again.cpu().numpy() - w) <= ATOL + RTOL * np.abs(w)).all()


def test_noalloc_decode_refuses_what_the_fixed_array_cannot_hold(native_lib):
    """The size check is pure host arithmetic on the launch plan: no launch, clear status."""
    from jacq_b200 import _native
    from tests.gpu_utils import DEV
    case = helpers.CONFIGS["mistral7b"]
    oc, tables, cache, q = _setup(case, [case.r + 2 * case.g])
    batch, max_len = 27, 1 << 20   # 216 (sequence, kv head) units: the plan splits the context in two
    geom = cache._geom
    need = native_lib.kivi_b200_decode_workspace_bytes(ctypes.byref(geom), batch, max_len)
    assert need > SCRATCH_BYTES
    # block tables wide enough for the stated bound, so the only thing wrong is the scratch size
    width = (max_len // case.b) + 1
    bts = torch.zeros((batch, width), dtype=torch.int32, device=DEV)
    lens = torch.zeros(batch, dtype=torch.int32, device=DEV)
    qq = torch.zeros((batch, case.nh, case.d), dtype=torch.float16, device=DEV)
    out = torch.zeros((batch, case.nh, case.d), dtype=torch.float32, device=DEV)
    slots = torch.zeros(batch, dtype=torch.int32, device=DEV)
    rc = native_lib.kivi_b200_decode_noalloc(
        ctypes.byref(geom), ctypes.byref(cache._struct), ctypes.c_void_p(qq.data_ptr()),
        ctypes.c_void_p(bts.data_ptr()), width, ctypes.c_void_p(lens.data_ptr()), ctypes.c_void_p(slots.data_ptr()),
        batch, max_len, ctypes.c_void_p(out.data_ptr()), None)
    assert rc == 5 and _native.STATUS_NAMES[rc] == "KIVI_ERR_WORKSPACE"
    assert b"workspace" in native_lib.kivi_b200_status_string(rc)


def test_zz_no_bounded_wait_gave_up_in_this_process(native_lib):
    """Every wait inside the kernels is bounded and counts itself when it gives up. After everything this
    process ran (the whole suite when it is run in one go) both counters must read zero."""
    for fn in (native_lib.kivi_b200_decode_wait_failures, native_lib.kivi_b200_gemm_wait_failures):
        out = ctypes.c_uint32(123)
        assert fn(ctypes.byref(out)) == 0
        assert out.value == 0, fn.__name__
