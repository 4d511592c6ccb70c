"""Seeded inputs and host<->device plumbing shared by the tests, the smoke check and bench.py.

Synthetic data stands in for real model activations: q, K, V ~ N(0,1) in fp16, a few key channels
per kv head scaled x10 (the per-channel outliers KIVI's per-channel key quantisation exists for),
block tables a Fisher-Yates permutation of the physical pages.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

BASE_SEED = 20261125


def reference_root():
    """The reference checkout, when one is at hand: $JACQ_REFERENCE, else a directory named `reference`
    beside this repository. None where neither exists (the GPU box), and the tests that read it skip."""
    import os
    from pathlib import Path
    cands = [os.environ.get("JACQ_REFERENCE"), Path(__file__).resolve().parent.parent.parent / "reference"]
    for c in cands:
        if c and (Path(c) / "integrations" / "vllm_kivi" / "source_patch.py").is_file():
            return Path(c)
    return None


@dataclass(frozen=True)
class Case:
    name: str
    nh: int
    nkv: int
    d: int
    b: int
    g: int
    r: int
    batch: int
    context: int
    outliers_per_head: int


CONFIGS = {
    "tinyllama": Case("tinyllama", 32, 4, 64, 16, 32, 32, 4, 512, 4),
    "qwen05b": Case("qwen05b", 14, 2, 64, 16, 32, 32, 64, 4096, 4),
    "mistral7b": Case("mistral7b", 32, 8, 128, 16, 128, 128, 128, 8192, 3),
    "reflane": Case("reflane", 40, 8, 128, 32, 32, 128, 1, 4096, 3),
}


def outlier_channels(case: Case, seed: int = BASE_SEED) -> np.ndarray:
    """[NKV, outliers_per_head] channel indices, fixed across tokens."""
    rng = np.random.default_rng(seed + 7)
    return np.stack([rng.choice(case.d, case.outliers_per_head, replace=False) for _ in range(case.nkv)])


def make_kv(case: Case, tokens: int, seed: int = BASE_SEED, stream: int = 0):
    """fp16 K, V of shape [tokens, NKV, D] with the key-channel outliers applied."""
    rng = np.random.default_rng([seed, 1, stream])
    k = rng.standard_normal((tokens, case.nkv, case.d), dtype=np.float32)
    v = rng.standard_normal((tokens, case.nkv, case.d), dtype=np.float32)
    ch = outlier_channels(case, seed)
    for h in range(case.nkv):
        k[:, h, ch[h]] *= 10.0
    return k.astype(np.float16), v.astype(np.float16)


def make_q(case: Case, batch: int, seed: int = BASE_SEED) -> np.ndarray:
    rng = np.random.default_rng([seed, 2])
    return rng.standard_normal((batch, case.nh, case.d), dtype=np.float32).astype(np.float16)


def shuffled_block_tables(num_seqs: int, pages_per_seq: int, num_blocks: int, seed: int = BASE_SEED) -> np.ndarray:
    """[num_seqs, pages_per_seq] distinct physical pages drawn from a permutation of the pool."""
    assert num_seqs * pages_per_seq <= num_blocks
    rng = np.random.default_rng([seed, 3])
    perm = rng.permutation(num_blocks).astype(np.int32)
    return perm[: num_seqs * pages_per_seq].reshape(num_seqs, pages_per_seq).copy()


def oracle_geometry(case: Case):
    from oracle import kivi_oracle as ko
    return ko.Geometry(case.nh, case.nkv, case.d, case.b, case.g, case.r)


def layout_of(case: Case):
    from jacq_b200.layout import KiviModelGeometry, KiviPageLayout
    return KiviPageLayout(KiviModelGeometry(case.name, 1, case.nh, case.nkv, case.d), case.b, case.g, 4, case.r)


PAGE_FIELDS = ("K_CODE_PAGES", "K_SCALE_PAGES", "K_ZERO_PAGES", "V_CODE_PAGES", "V_SCALE_PAGES", "V_ZERO_PAGES")
ORACLE_FIELD = {"K_CODE_PAGES": "k_code", "K_SCALE_PAGES": "k_scale", "K_ZERO_PAGES": "k_zero",
                "V_CODE_PAGES": "v_code", "V_SCALE_PAGES": "v_scale", "V_ZERO_PAGES": "v_zero",
                "K_RESIDUAL_SCRATCH": "k_scratch", "V_RESIDUAL_SCRATCH": "v_scratch"}


def to_bits(t) -> np.ndarray:
    """torch tensor -> numpy bit patterns (fp16 as uint16)."""
    import torch
    a = t.detach().cpu()
    if a.dtype == torch.float16:
        return a.view(torch.int16).numpy().view(np.uint16)
    return a.numpy()


def assert_cache_equal(device_tensors, oracle_cache, live_rows=None, what=""):
    """Bit-exact comparison of a device cache (object with the 8 tensor attributes, or a dict) with
    an OracleCache. live_rows[slot] limits the scratch comparison to the rows that hold tokens."""
    get = (lambda n: device_tensors[n]) if isinstance(device_tensors, dict) else (lambda n: getattr(device_tensors, n))
    for name in PAGE_FIELDS:
        got = to_bits(get(name))
        want = getattr(oracle_cache, ORACLE_FIELD[name])
        bad = np.argwhere(got != want.reshape(got.shape))
        assert bad.size == 0, f"{what}{name}: {len(bad)} mismatching elements, first at {bad[0].tolist()}"
    for name in ("K_RESIDUAL_SCRATCH", "V_RESIDUAL_SCRATCH"):
        got = to_bits(get(name))
        want = getattr(oracle_cache, ORACLE_FIELD[name]).reshape(got.shape) if got.ndim == 4 else \
            getattr(oracle_cache, ORACLE_FIELD[name])[0]
        if live_rows is None:
            assert np.array_equal(got, want), f"{what}{name} differs"
        else:
            for slot, rows in enumerate(live_rows):
                g_, w_ = (got[slot], want[slot]) if got.ndim == 4 else (got, want)
                assert np.array_equal(g_[:, :rows], w_[:, :rows]), f"{what}{name} slot {slot} rows<{rows} differ"
