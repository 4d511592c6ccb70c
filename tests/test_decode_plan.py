"""Launch plan of the tensor-core decode kernel, checked on the host: how a launch's (sequence, kv head)
units are cut into jobs, and how the parts of a cut unit share its key groups and residual tiles. The same
functions run inside the kernel (csrc/decode_merge.cuh); the reference has no counterpart (one warp per query
head walks the whole context, crates/jac-codegen-cuda/src/variants.rs:2463-2502)."""
import ctypes

import numpy as np
import pytest

from jacq_b200 import _native

SMS = 148   # multiprocessors the plan assumes when no device is present


def _geom(nh, nkv, d, b, g, r):
    return _native.KiviGeometry(nh, nkv, d, b, g, r)


def _plan(native_lib, geom, batch, max_len):
    out = (ctypes.c_int32 * 4)()
    assert native_lib.kivi_b200_decode_plan(ctypes.byref(geom), batch, max_len, out) == 0
    return tuple(out)


@pytest.mark.parametrize("shape", [(32, 8, 128, 16, 128, 128), (40, 8, 128, 16, 128, 128), (14, 2, 64, 16, 32, 32),
                                   (32, 4, 64, 16, 32, 32), (40, 8, 128, 32, 32, 128), (5, 1, 128, 16, 128, 128)])
def test_plan_covers_every_unit_and_the_workspace_holds_its_partials(native_lib, shape):
    geom = _geom(*shape)
    nh, nkv, d = shape[:3]
    rng = np.random.default_rng(1)
    cases = [(1, 32768), (8, 32768), (128, 8192), (64, 4096), (4, 512), (1, 1), (3, 0), (256, 32768)]
    cases += [(int(rng.integers(1, 300)), int(rng.integers(0, 40000))) for _ in range(60)]
    for batch, max_len in cases:
        units1, k1, units2, k2 = _plan(native_lib, geom, batch, max_len)
        assert units1 + units2 == batch * nkv and units1 >= 0 and units2 >= 0
        assert 1 <= k1 <= k2
        assert units1 % (3 * SMS) == 0 and (units1 == 0 or k1 == 1)   # whole units come in full rounds of three per multiprocessor
        slots = (units1 * k1 if k1 > 1 else 0) + (units2 * k2 if k2 > 1 else 0)
        need = native_lib.kivi_b200_decode_workspace_bytes(ctypes.byref(geom), batch, max_len)
        assert need >= slots * (nh // nkv) * (d + 2) * 4


def test_known_plans_on_148_multiprocessors(native_lib):
    mistral = _geom(32, 8, 128, 16, 128, 128)
    # 1024 units are 6.9 per multiprocessor: the queues are even enough, nothing is cut
    assert _plan(native_lib, mistral, 128, 8192) == (0, 1, 1024, 1)
    assert _plan(native_lib, mistral, 111, 8192) == (0, 1, 888, 1)
    # 512 units: three whole units per multiprocessor, the other 68 cut so that they spread over more of them
    u1, k1, u2, k2 = _plan(native_lib, mistral, 64, 8192)
    assert (u1, k1, u2) == (444, 1, 68) and k2 >= 2
    # a lone long sequence: every multiprocessor gets a couple of parts
    u1, k1, u2, k2 = _plan(native_lib, _geom(40, 8, 128, 16, 128, 128), 1, 32768)
    assert (u1, k1, u2) == (0, 1, 8) and 18 <= k2 <= 56


def test_short_groups_and_narrow_heads_are_cut_too(native_lib):
    """Head 64 / group 32 (the two small configurations): a weight unit takes longer there and a lone CTA gets less
    of its multiprocessor, so launches that leave multiprocessors idle or with one CTA are cut; full ones are not."""
    qwen = _geom(14, 2, 64, 16, 32, 32)
    assert _plan(native_lib, qwen, 64, 4096) == (0, 1, 128, 3)      # 128 units -> 384 jobs: one round of three everywhere
    assert _plan(native_lib, qwen, 128, 4096) == (0, 1, 256, 1)     # two per multiprocessor already
    u1, k1, u2, k2 = _plan(native_lib, qwen, 16, 4096)
    assert (u1, k1, u2) == (0, 1, 32) and 4 <= k2 <= 13             # 32 units: at least a job per multiprocessor
    tiny = _geom(32, 4, 64, 16, 32, 32)
    assert _plan(native_lib, tiny, 4, 512) == (0, 1, 16, 1)         # 512 tokens: nothing to gain from a merge launch
    assert _plan(native_lib, tiny, 32, 2048) == (0, 1, 128, 1)


@pytest.mark.parametrize("g,r", [(128, 128), (32, 32), (64, 128), (32, 128)])
def test_parts_tile_the_groups_and_residual_tiles_exactly_once(native_lib, g, r):
    geom = _geom(8, 2, 128, 16, g, r)
    items = (ctypes.c_int32 * 4)()
    rng = np.random.default_rng(g + r)
    lens = [0, 1, r - 1, r, r + 1, r + g - 1, r + g, r + g + 1, r + 7 * g + 5, 32768]
    lens += [int(x) for x in rng.integers(0, 20000, 40)]
    for seq_len in lens:
        old = max(0, seq_len - r) // g * g
        ngroups, ntiles = old // g, -(-(seq_len - old) // 16)
        for parts in (1, 2, 3, 5, 8, 13, 34, 64):
            next_g = next_t = 0
            for part in range(parts):
                assert native_lib.kivi_b200_decode_part_items(ctypes.byref(geom), seq_len, part, parts, items) == 0
                g0, g1, t0, t1 = items
                assert g0 == next_g and g1 >= g0 and t0 == next_t and t1 >= t0, (seq_len, parts, part, tuple(items))
                next_g, next_t = g1, t1
                if t1 > t0:
                    assert g1 == ngroups          # tiles only after the last group
            assert (next_g, next_t) == (ngroups, ntiles), (seq_len, parts)
            # parts of equal weight: no part holds more than its share plus one item
            if parts > 1 and ngroups + ntiles > 0:
                wg, wt = g // 16, 4
                total = ngroups * wg + ntiles * wt
                for part in range(parts):
                    native_lib.kivi_b200_decode_part_items(ctypes.byref(geom), seq_len, part, parts, items)
                    weight = (items[1] - items[0]) * wg + (items[3] - items[2]) * wt
                    assert weight <= -(-total // parts) + max(wg, wt)
