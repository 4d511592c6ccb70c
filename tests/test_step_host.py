"""CPU checks of the decode step: the oracle's element-wise kernels against independent float64
formulas and against golden outputs of the reference's own kernels, the oracle step against the
reference's forward() (golden logits), tensor-parallel sharding, the weight directory layout and the
argument validation of the C entry points (no GPU call is made)."""
import ctypes
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import kivi_oracle as ko
from oracle import step_oracle as so

GOLDEN = Path(__file__).resolve().parent / "golden" / "runtime_kernels.npz"
TINY = so.StepShape(layers=2, hidden=256, nh=4, nkv=2, hd=64, ffn=512, vocab=1024, rope_base=10000.0,
                    norm_eps=1e-5, attn_bias=True, block=16, group=32, residual=32)


@pytest.fixture(scope="module")
def golden():
    if not GOLDEN.exists():
        pytest.skip("tests/golden/runtime_kernels.npz not generated yet")
    return np.load(GOLDEN)


def _ulp(a, b):
    return np.abs(a.view(np.uint16).astype(np.int32) - b.view(np.uint16).astype(np.int32))


# ---- oracle kernels vs float64 formulas ---------------------------------------------------------

def test_oracle_rmsnorm_formula():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 1000), dtype=np.float32).astype(np.float16)
    d = rng.standard_normal((3, 1000), dtype=np.float32).astype(np.float16)
    w = (1 + 0.1 * rng.standard_normal(1000, dtype=np.float32)).astype(np.float16)
    x_out, normed = ko.residual_rmsnorm(x, d, w, 1e-5)
    s = (x.astype(np.float64) + d.astype(np.float64)).astype(np.float16)
    assert np.array_equal(x_out.view(np.uint16), s.view(np.uint16))
    s64 = s.astype(np.float64)
    want = s64 / np.sqrt((s64 ** 2).mean(axis=1, keepdims=True) + 1e-5) * w.astype(np.float64)
    np.testing.assert_allclose(normed.astype(np.float64), want, rtol=2e-3, atol=1e-4)
    same_x, _ = ko.residual_rmsnorm(x, None, w, 1e-5)
    assert np.array_equal(same_x.view(np.uint16), x.view(np.uint16))


def test_oracle_rope_formula_and_norm_preservation():
    rng = np.random.default_rng(1)
    nh, nkv, hd = 4, 2, 64
    pos = np.array([0, 7, 513], np.int32)
    qkv = rng.standard_normal((3, (nh + 2 * nkv) * hd), dtype=np.float32).astype(np.float16)
    q, k, v = ko.bias_rope(qkv, None, pos, nh, nkv, hd, 10000.0)
    assert np.array_equal(v.view(np.uint16), qkv[:, (nh + nkv) * hd:].view(np.uint16))
    assert np.array_equal(q[0].view(np.uint16), qkv[0, : nh * hd].view(np.uint16))   # position 0 rotates by nothing
    i = np.arange(hd // 2)
    ang = pos[:, None].astype(np.float64) / 10000.0 ** (2.0 * i / hd)
    x = qkv[:, : nh * hd].astype(np.float64).reshape(3, nh, hd)
    x0, x1 = x[..., : hd // 2], x[..., hd // 2:]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    want = np.concatenate([x0 * c - x1 * s, x1 * c + x0 * s], axis=-1).reshape(3, nh * hd)
    np.testing.assert_allclose(q.astype(np.float64), want, rtol=2e-3, atol=2e-3)
    bias = (rng.standard_normal((nh + 2 * nkv) * hd, dtype=np.float32) * 0.1).astype(np.float16)
    _, _, vb = ko.bias_rope(qkv, bias, pos, nh, nkv, hd, 10000.0)
    want_v = (qkv[:, (nh + nkv) * hd:].astype(np.float64) + bias[(nh + nkv) * hd:].astype(np.float64)).astype(np.float16)
    assert np.array_equal(vb.view(np.uint16), want_v.view(np.uint16))


def test_oracle_silu_and_argmax():
    rng = np.random.default_rng(2)
    gu = (rng.standard_normal((2, 64), dtype=np.float32) * 3).astype(np.float16)
    g, u = gu[:, :32].astype(np.float64), gu[:, 32:].astype(np.float64)
    np.testing.assert_allclose(ko.silu_mul(gu).astype(np.float64), g / (1 + np.exp(-g)) * u, rtol=2e-3, atol=1e-4)
    logits = rng.standard_normal((4, 300), dtype=np.float32).astype(np.float16)
    logits[1, [10, 200]] = np.float16(20.0)
    logits[2, :] = np.float16(-np.inf)
    logits[3, :] = np.float16("nan")
    out = ko.argmax(logits)
    assert out[0] == int(np.argmax(logits[0].astype(np.float32))) and out[1] == 10 and out[2] == 0 and out[3] == 0


# ---- oracle vs the reference's own kernels (golden) -----------------------------------------------

def test_oracle_kernels_match_reference_golden(golden):
    g = golden
    for tag in ("h256", "h5120"):
        x_out, normed = ko.residual_rmsnorm(g[f"norm_{tag}_x"], g[f"norm_{tag}_delta"], g[f"norm_{tag}_w"],
                                            float(g[f"norm_{tag}_eps"]))
        assert np.array_equal(x_out.view(np.uint16), g[f"norm_{tag}_sum"].view(np.uint16))
        d = _ulp(normed, g[f"norm_{tag}_out"])
        assert d.max() <= 1 and (d == 0).mean() > 0.98      # device rsqrtf vs 1/sqrtf
    for tag in ("tiny", "q14b"):
        nh, nkv, hd = (int(v) for v in g[f"rope_{tag}_shape"])
        q, k, v = ko.bias_rope(g[f"rope_{tag}_qkv"], g[f"rope_{tag}_bias"], g[f"rope_{tag}_pos"], nh, nkv, hd,
                               float(g[f"rope_{tag}_base"]))
        want = g[f"rope_{tag}_out"]
        assert np.array_equal(v.view(np.uint16), want[:, (nh + nkv) * hd:].view(np.uint16))
        got = np.concatenate([q, k], axis=1).astype(np.float32)
        np.testing.assert_allclose(got, want[:, : (nh + nkv) * hd].astype(np.float32), rtol=2e-3, atol=4e-3)
    d = _ulp(ko.silu_mul(g["silu_gate_up"]), g["silu_out"])
    assert d.max() <= 1 and (d == 0).mean() > 0.98
    got = ko.argmax(g["argmax_logits"])
    assert got[0] == g["argmax_out"][0] and got[2] == g["argmax_out"][2] == 0
    assert g["argmax_logits"][1, got[1]] == g["argmax_logits"][1, g["argmax_out"][1]]


def test_oracle_step_matches_reference_forward(golden):
    """The reference's forward() keeps an fp16 dense cache; with R = G = 32 the KIVI cache holds every
    token in fp16 until token 64, so for 60 tokens both must agree to the contract's tolerance."""
    w = so.random_weights(TINY, int(golden["tiny_seed"]))
    if so.weights_checksum(w) != int(golden["tiny_weights_crc32"]):
        pytest.skip("numpy's generator no longer reproduces the weights the golden run used")
    oracle = so.StepOracle(TINY, w, np.arange(8, dtype=np.int32).reshape(1, 8), 8)
    tokens, want = golden["tiny_tokens"], golden["tiny_logits"].astype(np.float32)
    agree = 0
    for i in range(want.shape[0]):
        nxt, logits = oracle.step(np.array([tokens[i]]))
        np.testing.assert_allclose(logits[0].astype(np.float32), want[i], rtol=1e-2, atol=1e-2, err_msg=f"step {i}")
        agree += int(nxt[0] == tokens[i + 1])
    assert agree >= want.shape[0] - 2


# ---- tensor-parallel sharding -----------------------------------------------------------------------

def _torch_layer(lw):
    return {k: (None if v is None else torch.from_numpy(v)) for k, v in lw.items()}


def _config(shape):
    from jacq_b200.runtime import DecodeModelConfig
    return DecodeModelConfig("test", shape.layers, shape.hidden, shape.nh, shape.nkv, shape.hd, shape.ffn, shape.vocab,
                             rope_base=shape.rope_base, norm_eps=shape.norm_eps, attn_bias=shape.attn_bias,
                             block_size=shape.block, group_size=shape.group, residual=shape.residual)


@pytest.mark.parametrize("world", [1, 2])
def test_shard_layer_matches_oracle_and_reassembles(world):
    from jacq_b200.runtime import shard_layer
    w = so.random_weights(TINY, 5)
    cfg = _config(TINY)
    lw = w.layers[0]
    rng = np.random.default_rng(0)
    x = rng.standard_normal(TINY.hidden).astype(np.float64)
    full_qkv = lw["qkv"].astype(np.float64) @ x
    attn = rng.standard_normal(TINY.q_dim).astype(np.float64)
    full_o = lw["o"].astype(np.float64) @ attn
    o_sum = np.zeros(TINY.hidden)
    for r in range(world):
        mine = shard_layer(cfg, _torch_layer(lw), r, world)
        theirs = so.shard_layer(TINY, lw, r, world)
        for k, v in theirs.items():
            assert np.array_equal(mine[k].numpy().view(np.uint16), v.view(np.uint16)), k
        nh_l, nkv_l = TINY.nh // world, TINY.nkv // world
        got = mine["qkv"].numpy().astype(np.float64) @ x
        want = np.concatenate([
            full_qkv[r * nh_l * TINY.hd: (r + 1) * nh_l * TINY.hd],
            full_qkv[TINY.q_dim + r * nkv_l * TINY.hd: TINY.q_dim + (r + 1) * nkv_l * TINY.hd],
            full_qkv[TINY.q_dim + TINY.kv_dim + r * nkv_l * TINY.hd: TINY.q_dim + TINY.kv_dim + (r + 1) * nkv_l * TINY.hd]])
        np.testing.assert_allclose(got, want, rtol=1e-12)
        o_sum += mine["o"].numpy().astype(np.float64) @ attn[r * nh_l * TINY.hd: (r + 1) * nh_l * TINY.hd]
    np.testing.assert_allclose(o_sum, full_o, rtol=1e-9, atol=1e-12)


def test_shard_rejects_uneven_split():
    from jacq_b200.runtime import shard_rows
    with pytest.raises(ValueError):
        shard_rows(_config(TINY), 0, 3)


def test_two_rank_oracle_agrees_with_one_rank():
    w = so.random_weights(TINY, 9)
    bt = np.arange(16, dtype=np.int32).reshape(2, 8)
    one, two = so.StepOracle(TINY, w, bt, 16), so.StepOracle(TINY, w, bt, 16, world=2)
    tok = np.array([3, 700])
    for _ in range(70):   # crosses the first quantisation boundary at token 64
        t1, l1 = one.step(tok)
        _, l2 = two.step(tok)
        np.testing.assert_allclose(l1.astype(np.float32), l2.astype(np.float32), rtol=1e-2, atol=1e-2)
        tok = t1


# ---- weight directory, configuration, validation ------------------------------------------------------

def test_weight_dir_uses_the_reference_file_layout(tmp_path):
    from jacq_b200.runtime import load_weight_dir, save_weight_dir
    cfg = _config(TINY)
    w = so.random_weights(TINY, 4)
    tw = {"embed": torch.from_numpy(w.embed), "final_norm": torch.from_numpy(w.final_norm),
          "lm_head": torch.from_numpy(w.lm_head), "layers": [_torch_layer(lw) for lw in w.layers]}
    save_weight_dir(cfg, tw, tmp_path)
    names = sorted(p.name for p in tmp_path.iterdir())
    # names of crates/jac-codegen-cuda/src/templates/runtime.cu:61-96
    assert "embed.bin" in names and "final_norm.bin" in names and "lm_head.bin" in names
    for stem in ("attn_norm", "qkv", "qkv_bias", "o", "ffn_norm", "gate_up", "down"):
        assert f"layer00_{stem}.bin" in names and f"layer01_{stem}.bin" in names
    assert (tmp_path / "layer01_gate_up.bin").stat().st_size == 2 * TINY.ffn * TINY.hidden * 2
    back = load_weight_dir(cfg, tmp_path)
    assert torch.equal(back["layers"][1]["qkv"], tw["layers"][1]["qkv"])
    (tmp_path / "layer00_o.bin").write_bytes(b"\0" * 10)
    with pytest.raises(RuntimeError, match="short read"):
        load_weight_dir(cfg, tmp_path)


def test_qwen25_14b_config_bytes():
    from jacq_b200.runtime import DecodeModelConfig
    c = DecodeModelConfig.qwen25_14b()
    assert (c.qkv_out, c.q_dim, c.kv_dim) == (7168, 5120, 1024)
    per_layer = (7168 * 5120 + 5120 * 5120 + 27648 * 5120 + 5120 * 13824) * 2
    assert per_layer == 550_502_400                      # 550.5 MB of fp16 weights per layer
    assert c.weight_bytes() == 48 * per_layer + 152064 * 5120 * 2
    assert c.weight_bytes(8) * 8 == c.weight_bytes()


def test_runtime_needs_cuda():
    from jacq_b200.runtime import DecodeRuntime
    with pytest.raises(RuntimeError, match="CUDA"):
        DecodeRuntime(_config(TINY), {}, batch=1, max_seq_len=64, device="cpu")


def test_step_entry_points_validate_before_launching(native_lib):
    from jacq_b200 import _native
    lib = native_lib
    good = _native.KiviStepConfig(2, 256, 4, 2, 64, 512, 1024, 0, 1, 10000.0, 1e-5, 16, 32, 32, 1, 0)
    assert lib.kivi_b200_decode_step_workspace_bytes(ctypes.byref(good), 3, 160) > 0
    assert lib.kivi_b200_decode_step_workspace_bytes(ctypes.byref(good), 0, 160) == 0
    assert lib.kivi_b200_decode_step_workspace_bytes(ctypes.byref(good), 65, 160) == 0
    bad_heads = _native.KiviStepConfig(2, 256, 5, 2, 64, 512, 1024, 0, 1, 10000.0, 1e-5, 16, 32, 32, 1, 0)
    assert lib.kivi_b200_decode_step_workspace_bytes(ctypes.byref(bad_heads), 1, 160) == 0
    bad_group = _native.KiviStepConfig(2, 256, 4, 2, 64, 512, 1024, 0, 1, 10000.0, 1e-5, 16, 24, 32, 1, 0)
    assert lib.kivi_b200_decode_step_workspace_bytes(ctypes.byref(bad_group), 1, 160) == 0
    null = None
    rc = lib.kivi_b200_decode_step(ctypes.byref(good), null, null, null, 1, 10, null, null, null, null)
    assert rc == 1     # KIVI_ERR_NULL_POINTER
    rc = lib.kivi_b200_decode_step(ctypes.byref(bad_heads), null, null, null, 1, 10, null, null, null, null)
    assert rc == 2     # KIVI_ERR_GEOMETRY
    assert lib.kivi_b200_residual_rmsnorm(null, null, null, null, null, 1, 256, ctypes.c_float(1e-5), null) == 1
    assert lib.kivi_b200_silu_mul(null, null, 1, 512, null) == 1
    assert lib.kivi_b200_argmax(null, null, 1, 10, null, 0, null) == 1
    assert lib.kivi_b200_bias_rope(null, null, null, null, null, null, 1, 4, 2, 64, ctypes.c_float(1e4), null) == 1
