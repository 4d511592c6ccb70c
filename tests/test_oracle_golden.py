"""Pins the CPU oracle to the reference: the golden vectors under tests/golden/ are outputs of the
reference's own CUDA (hand-CUDA writer and emitted decode kernels, compiled unmodified and run on a
B200 by tests/golden/make_golden.py). Writer results must match bit for bit; decode within the
path's stated tolerance (rtol = atol = 1e-2; observed agreement is ~1e-6)."""
from pathlib import Path

import numpy as np
import pytest

from oracle import kivi_oracle as ko

GOLDEN = Path(__file__).resolve().parent / "golden"
GEOM = ko.Geometry(nh=20, nkv=4, d=128, b=32, g=32, r=128)   # the reference's TP=2 local-rank lane


def _load(name):
    path = GOLDEN / name
    if not path.exists():
        pytest.fail(f"golden fixture {name} is missing")
    return np.load(path)


def _written(z, num_blocks):
    oc = ko.OracleCache(GEOM, num_blocks, 1)
    tokens = int(z["tokens"])
    k = z["k"].reshape(tokens, GEOM.nkv, GEOM.d)
    v = z["v"].reshape(tokens, GEOM.nkv, GEOM.d)
    ko.write_tokens(oc, k, v, z["block_table"], 0)
    return oc, tokens


def _assert_cache_matches(oc, z, tokens):
    for name in ko.OracleCache.PAGE_FIELDS:
        got, want = getattr(oc, name), z[name]
        assert np.array_equal(got, want.reshape(got.shape)), f"{name} differs from the reference's output"
    live = tokens - GEOM.split_old(tokens)
    for name in ("k_scratch", "v_scratch"):
        assert np.array_equal(getattr(oc, name)[0][:, :live], z[name][:, :live]), name


def test_oracle_writer_equals_reference_cuda_bit_for_bit():
    z = _load("reflane_tp2_writer_decode.npz")
    oc, tokens = _written(z, 6)
    _assert_cache_matches(oc, z, tokens)
    assert GEOM.split_old(tokens) // GEOM.b == 3


def test_oracle_writer_edge_values_equal_reference_cuda():
    """NaN / Inf lanes, constant groups, mixed-sign zeros, fp16 extremes and subnormals."""
    z = _load("reflane_tp2_edge_values.npz")
    oc, tokens = _written(z, 2)
    _assert_cache_matches(oc, z, tokens)


def test_oracle_decode_matches_reference_cuda():
    z = _load("reflane_tp2_writer_decode.npz")
    oc, tokens = _written(z, 6)
    q = z["q"].reshape(4, GEOM.nh, GEOM.d)
    for seq_len in (100, 160, tokens):
        want = z[f"decode_{seq_len}"]
        for mode in (0, 1):
            got = ko.decode(oc, q[0], z["block_table"], seq_len, mode=mode, max_old_tokens=3968)
            np.testing.assert_allclose(got, want, rtol=1e-2, atol=1e-2)
            assert np.abs(got - want).max() < 1e-4
    lens = z["batched_lens"]
    for j, n in enumerate(lens):
        got = ko.decode(oc, q[j], z["block_table"], int(n), mode=0, max_old_tokens=3968)
        np.testing.assert_allclose(got, z["decode_batched"][j], rtol=1e-2, atol=1e-2)
        assert np.abs(got - z["decode_batched"][j]).max() < 1e-4
    got = ko.decode(oc, q[1], z["retained_table"], tokens, mode=0, max_old_tokens=3968, num_retained_pages=2)
    np.testing.assert_allclose(got, z["decode_sparse"], rtol=1e-2, atol=1e-2)
    assert np.abs(got - z["decode_sparse"]).max() < 1e-4
