"""Properties of the CPU oracle that need no reference: conversion helpers against numpy, the
writer against an independent numpy restatement, chunking invariance, the boundary table of the
reference's guard tests (tests/test_runtime_guards.py:163-165 of the reference)."""
import numpy as np
import pytest

from oracle import kivi_oracle as ko
from tests import helpers


def test_half_conversions_match_numpy_exhaustively():
    allh = np.arange(65536, dtype=np.uint16)
    want = allh.view(np.float16).astype(np.float32)
    got = np.array([ko.h2f(int(h)) for h in allh], np.float32)
    assert ((got == want) | (np.isnan(got) & np.isnan(want))).all()
    rng = np.random.default_rng(0)
    xs = (rng.standard_normal(20000) * rng.choice([1e-8, 1e-5, 1e-3, 1, 100, 65000], 20000)).astype(np.float32)
    xs = np.concatenate([xs, np.array([0, -0.0, 65504, 65519.9, 65520, 1e9, 2 ** -24, 2 ** -25, np.inf, -np.inf],
                                      np.float32)])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    got = np.array([ko.f2h(float(x)) for x in xs], np.uint16)
    assert np.array_equal(got, want)
    assert ko.f2h(float("nan")) == 0x7FFF


@pytest.mark.parametrize("seq_len,pages", [(128, 0), (129, 0), (159, 0), (160, 1), (191, 1), (192, 2), (4096, 124)])
def test_old_page_boundaries_of_the_reference_lane(seq_len, pages):
    assert ko.REF_LANE.split_old(seq_len) // ko.REF_LANE.b == pages
    gm = ko.REF_LANE.c()
    import ctypes
    assert ko.lib().kivi_oracle_split_old(ctypes.byref(gm), seq_len) // 32 == pages


def _numpy_group_quant(x):
    """x [n, m] fp32 -> (scale, zero, codes) over axis 0, the KIVI asymmetric int4 rule."""
    mn, mx = x.min(0), x.max(0)
    scale = ((mx - mn) / np.float32(15.0)).astype(np.float32)
    scale = np.where(scale > 0, scale, np.float32(1.0)).astype(np.float32)
    codes = np.clip(np.rint((x - mn) / scale), 0, 15).astype(np.uint8)
    return scale, mn, codes


@pytest.mark.parametrize("name", ["tinyllama", "mistral7b", "reflane"])
def test_writer_matches_independent_numpy_restatement(name):
    case = helpers.CONFIGS[name]
    geom = helpers.oracle_geometry(case)
    tokens = case.r + 2 * case.g + 3
    k, v = helpers.make_kv(case, tokens)
    pages = geom.split_old(tokens) // case.b
    table = helpers.shuffled_block_tables(1, pages, pages + 2)[0]
    oc = ko.OracleCache(geom, pages + 2, 1, fill=0xEE)
    ko.write_tokens(oc, k, v, table, 0)
    kf, vf = k.astype(np.float32), v.astype(np.float32)
    vg = min(case.g, case.d)
    for grp in range(2):
        rows = slice(grp * case.g, (grp + 1) * case.g)
        for h in range(case.nkv):
            ks, kz, kc = _numpy_group_quant(kf[rows, h, :])
            for t in range(case.g):
                page = table[(grp * case.g + t) // case.b]
                off = (grp * case.g + t) % case.b
                packed = (kc[t, 0::2] | (kc[t, 1::2] << 4)).astype(np.uint8)
                assert np.array_equal(oc.k_code[page, h, off], packed)
                assert np.array_equal(oc.k_scale[page, h], ks.astype(np.float16).view(np.uint16))
                assert np.array_equal(oc.k_zero[page, h], kz.astype(np.float16).view(np.uint16))
                for cg in range(case.d // vg):
                    seg = vf[grp * case.g + t, h, cg * vg:(cg + 1) * vg]
                    vs, vz, vc = _numpy_group_quant(seg[:, None])
                    assert oc.v_scale[page, h, off, cg] == vs.astype(np.float16).view(np.uint16)[0]
                    assert oc.v_zero[page, h, off, cg] == vz.astype(np.float16).view(np.uint16)[0]
                    packed = (vc[0::2, 0] | (vc[1::2, 0] << 4)).astype(np.uint8)
                    assert np.array_equal(oc.v_code[page, h, off, cg * vg // 2:(cg + 1) * vg // 2], packed)
    # the unquantised tail sits at the front of the scratch, oldest first; unused pages keep the poison
    live = tokens - geom.split_old(tokens)
    assert np.array_equal(oc.k_scratch[0][:, :live], np.swapaxes(k[tokens - live:], 0, 1).view(np.uint16))
    unused = [b for b in range(pages + 2) if b not in set(table.tolist())]
    assert (oc.k_code[unused] == 0xEE).all() and (oc.v_scale[unused] == 0xEEEE).all()


@pytest.mark.parametrize("name", ["tinyllama", "reflane"])
@pytest.mark.parametrize("chunk", [1, 2, 31, 32, 33, 160, 512])
def test_planned_batched_writes_equal_token_by_token(name, chunk):
    """The reference's batched writer fed by its planner == its single-token writer."""
    case = helpers.CONFIGS[name]
    geom = helpers.oracle_geometry(case)
    tokens = case.r + 4 * case.g + 7
    k, v = helpers.make_kv(case, tokens)
    pages = geom.split_old(tokens) // case.b
    table = helpers.shuffled_block_tables(1, pages, pages + 1)[0]
    a = ko.OracleCache(geom, pages + 1, 1)
    b = ko.OracleCache(geom, pages + 1, 1)
    ko.write_tokens(a, k, v, table, 0)
    s = 0
    while s < tokens:
        n = min(chunk, tokens - s)
        for ps, pn in ko.plan_batched_write(geom, s, n):
            ko.write_batched(b, k[ps:ps + pn], v[ps:ps + pn], table, ps)
        s += n
    live = tokens - geom.split_old(tokens)
    for f in ko.OracleCache.PAGE_FIELDS:
        assert np.array_equal(getattr(a, f), getattr(b, f)), f
    assert np.array_equal(a.k_scratch[0][:, :live], b.k_scratch[0][:, :live])
    with pytest.raises(ValueError):
        ko.write_batched(b, k[:case.r + 2 * case.g], v[:case.r + 2 * case.g], table, 0)   # crosses two boundaries


def test_planner_matches_the_python_mirror():
    from jacq_b200 import kivi_dsl
    for start, n in [(0, 1), (0, 512), (100, 60), (127, 1), (159, 1), (159, 2), (160, 160), (3000, 333)]:
        want = [(p.start_seq_len, p.num_new) for p in kivi_dsl.plan_batched_write(start, n)]
        assert ko.plan_batched_write(ko.REF_LANE, start, n) == want
        assert sum(c for _, c in want) == n


def test_decode_two_pass_agrees_with_online_and_is_a_convex_combination():
    case = helpers.CONFIGS["tinyllama"]
    geom = helpers.oracle_geometry(case)
    k, v = helpers.make_kv(case, 300)
    table = helpers.shuffled_block_tables(1, 16, 18)[0]
    oc = ko.OracleCache(geom, 18, 1)
    ko.write_tokens(oc, k, v, table, 0)
    q = helpers.make_q(case, 1)[0]
    a = ko.decode(oc, q, table, 300, mode=0)
    b = ko.decode(oc, q, table, 300, mode=1)
    assert np.abs(a - b).max() < 1e-4
    assert np.array_equal(ko.decode(oc, q, table, 0), np.zeros_like(a))
    # a constant V gives that constant back (softmax weights sum to 1), exactly representable in int4
    v2 = np.full_like(v, np.float16(0.75))
    oc2 = ko.OracleCache(geom, 18, 1)
    ko.write_tokens(oc2, k, v2, table, 0)
    np.testing.assert_allclose(ko.decode(oc2, q, table, 300, mode=1), 0.75, rtol=0, atol=1e-6)


def test_gemv_matches_numpy():
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((64, 256)) * 0.02).astype(np.float16)
    x = rng.standard_normal((3, 256)).astype(np.float16)
    y16, y32 = ko.gemv(w, x)
    np.testing.assert_allclose(y32, x.astype(np.float32) @ w.astype(np.float32).T, rtol=1e-5, atol=1e-6)
    assert np.array_equal(y16, y32.astype(np.float16))
