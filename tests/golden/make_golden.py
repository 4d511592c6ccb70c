"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own CUDA.

Run on a machine with a B200 after `python oracle/build_ref.py` has compiled the reference sources
into oracle/_ref/libjacq_ref.so (the library travels to the GPU box; the reference checkout does
not). Inputs are seeded; outputs are what the reference's hand-CUDA writer
(integrations/vllm_kivi/source_patch.py:1500-1776) and its emitted decode kernels
(crates/jac-codegen-cuda/tests/snapshots/kernels/decode_attention_kivi_*_library_flash.cu,
TP=2 local-rank clones: NH/NKV 20/4) produce for them.

    python tests/golden/make_golden.py --out golden_out

Writes reflane_tp2_writer_decode.npz and reflane_tp2_edge_values.npz.
"""
from __future__ import annotations

import argparse
import ctypes
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from tests import helpers  # noqa: E402

NKV, NH, D, B, R = 4, 20, 128, 32, 128
DEV = torch.device("cuda:0")


def _bundle(num_blocks):
    z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=DEV)
    return [z((num_blocks, NKV, B, D // 2), torch.uint8), z((num_blocks, NKV, D), torch.float16),
            z((num_blocks, NKV, D), torch.float16), z((num_blocks, NKV, B, D // 2), torch.uint8),
            z((num_blocks, NKV, B, D // B), torch.float16), z((num_blocks, NKV, B, D // B), torch.float16),
            z((NKV, R + B, D), torch.float16), z((NKV, R + B, D), torch.float16)]


NAMES = ("k_code", "k_scale", "k_zero", "v_code", "v_scale", "v_zero", "k_scratch", "v_scratch")


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _f16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.float16).to(DEV)


def _write_all(ref, bundle, k, v, table):
    kd, vd = _f16(k.view(np.uint16)), _f16(v.view(np.uint16))
    bt = torch.from_numpy(table).to(DEV)
    sm = torch.zeros(1, dtype=torch.int64, device=DEV)
    for t in range(k.shape[0]):
        ref.ref_kivi_cache_write_launch(*[_p(x) for x in bundle], _p(kd[t]), _p(vd[t]), _p(sm), _p(bt),
                                        ctypes.c_int(t + 1), ctypes.c_int(NKV), None)
    torch.cuda.synchronize()
    return bt


def _dump(bundle):
    return {n: helpers.to_bits(t) for n, t in zip(NAMES, bundle)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(ROOT / "tests" / "golden"))
    out = Path(ap.parse_args().out)
    out.mkdir(parents=True, exist_ok=True)
    ref = ctypes.CDLL(str(ROOT / "oracle" / "_ref" / "libjacq_ref.so"))
    case = helpers.Case("reflane_tp2", NH, NKV, D, B, B, R, 1, 0, 3)

    # ---- writer + decode ------------------------------------------------------------------
    tokens, num_blocks = R + B * 3 + 5, 6
    k, v = helpers.make_kv(case, tokens)
    table = np.zeros(124, np.int32)
    table[:4] = [4, 1, 5, 2]
    bundle = _bundle(num_blocks)
    bt = _write_all(ref, bundle, k, v, table)
    q = helpers.make_q(case, 4)
    qd = _f16(q.view(np.uint16))
    res = {"k": k.view(np.uint16), "v": v.view(np.uint16), "q": q.view(np.uint16), "block_table": table,
           "tokens": np.int32(tokens), **_dump(bundle)}
    for seq_len in (100, 160, tokens):
        o = torch.zeros((NH, D), dtype=torch.float32, device=DEV)
        ref.jac_launch_tp2_local(_p(qd[0]), _p(bt), *[_p(x) for x in bundle], ctypes.c_int(seq_len), _p(o), None)
        torch.cuda.synchronize()
        res[f"decode_{seq_len}"] = o.cpu().numpy()
    lens = np.array([tokens, tokens - 1, 130, 7], np.int32)
    ob = torch.zeros((4, NH, D), dtype=torch.float32, device=DEV)
    ref.jac_launch_batched_tp2_local(_p(qd), _p(torch.from_numpy(lens).to(DEV)), _p(bt), *[_p(x) for x in bundle],
                                     ctypes.c_int(4), _p(ob), None)
    compact = np.zeros(124, np.int32)
    compact[:2] = [table[0], table[2]]
    osr = torch.zeros((NH, D), dtype=torch.float32, device=DEV)
    ref.jac_launch_sparse_retained_tp2_local(_p(qd[1]), _p(torch.from_numpy(compact).to(DEV)),
                                             *[_p(x) for x in bundle], ctypes.c_int(tokens), ctypes.c_int(2), _p(osr),
                                             None)
    torch.cuda.synchronize()
    res.update(batched_lens=lens, decode_batched=ob.cpu().numpy(), retained_table=compact,
               decode_sparse=osr.cpu().numpy())
    np.savez_compressed(out / "reflane_tp2_writer_decode.npz", **res)

    # ---- edge values through the writer ---------------------------------------------------
    tokens = R + B
    k, v = helpers.make_kv(case, tokens, stream=9)
    k, v = k.copy(), v.copy()
    f = np.float16
    k[:, 0, 0] = f(1.5)
    k[:, 0, 1] = f(0.0); k[::2, 0, 1] = f(-0.0)
    k[:, 0, 2] = f(np.nan)
    k[5, 0, 3] = f(np.nan)
    k[7, 0, 4] = f(np.inf); k[9, 0, 5] = f(-np.inf)
    k[:, 0, 6] = f(65504.0); k[::3, 0, 6] = f(-65504.0)
    k[:, 0, 7] = f(6e-8)
    v[3, 1, :32] = f(2.0)
    v[4, 1, :32] = f(0.0); v[4, 1, 1:32:2] = f(-0.0)
    v[5, 1, 32:64] = f(np.nan)
    v[6, 1, 64] = f(np.nan)
    v[8, 1, 96] = f(np.inf)
    v[10, 2, 0] = f(65504.0); v[10, 2, 1] = f(-65504.0)
    table = np.zeros(124, np.int32)
    table[0] = 1
    bundle = _bundle(2)
    _write_all(ref, bundle, k, v, table)
    np.savez_compressed(out / "reflane_tp2_edge_values.npz", k=k.view(np.uint16), v=v.view(np.uint16),
                        block_table=table, tokens=np.int32(tokens), **_dump(bundle))
    print("golden vectors written to", out)


if __name__ == "__main__":
    main()
