"""Generate tests/golden/runtime_kernels.npz by running the REFERENCE's generated-runtime CUDA.

Run on a machine with a B200 after `python oracle/build_ref.py` has compiled the reference's
templates (crates/jac-codegen-cuda/src/templates/kernels.cu and runtime.cu, behind
oracle/ref_runtime_shim.cu) into oracle/_ref/libjacq_ref.so. Inputs are seeded and stored with the
outputs, except the weights of the tiny model, which tests rebuild from the seed (a checksum is
stored).

    python tests/golden/make_runtime_golden.py --out golden_out

Cases: rmsnorm_kernel after vadd_kernel, bias_add_kernel + rope_qk_kernel (tiny and Qwen2.5-14B
head shapes, positions up to 32767), silu_mul_kernel, argmax_kernel, and 60 greedy tokens of the
reference's forward() on the tiny model (2 layers, hidden 256, 4 q / 2 kv heads, head_dim 64,
FFN 512, vocab 1024, qkv bias) with the logits of every step.
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
from oracle import step_oracle as so  # noqa: E402

DEV = torch.device("cuda:0")
TINY = so.StepShape(layers=2, hidden=256, nh=4, nkv=2, hd=64, ffn=512, vocab=1024, rope_base=10000.0,
                    norm_eps=1e-5, attn_bias=True, block=16, group=32, residual=32)
TINY_SEED = 7
TINY_STEPS = 60
TINY_FIRST_TOKEN = 5


def _dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16).copy()).view(torch.float16).to(DEV)


def _host(t: torch.Tensor) -> np.ndarray:
    return t.cpu().view(torch.int16).numpy().view(np.float16)


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="golden_out")
    args = ap.parse_args()
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    ref = ctypes.CDLL(str(ROOT / "oracle" / "_ref" / "libjacq_ref.so"))
    ref.ref_tiny_step.restype = ctypes.c_int
    ref.ref_tiny_set_weights.restype = ctypes.c_int
    rng = np.random.default_rng(2024)
    g: dict[str, np.ndarray] = {}

    # vadd + rmsnorm, one row per launch as forward() does
    for tag, hidden, rows, eps in (("h256", 256, 4, 1e-5), ("h5120", 5120, 2, 1e-6)):
        x = rng.standard_normal((rows, hidden), dtype=np.float32).astype(np.float16)
        d = (rng.standard_normal((rows, hidden), dtype=np.float32) * 0.5).astype(np.float16)
        w = (1.0 + 0.1 * rng.standard_normal(hidden, dtype=np.float32)).astype(np.float16)
        xd, dd, wd = _dev(x), _dev(d), _dev(w)
        summed, normed = torch.empty_like(xd), torch.empty_like(xd)
        for r in range(rows):
            ref.ref_vadd(_p(summed[r]), _p(xd[r]), _p(dd[r]), ctypes.c_int(hidden))
            ref.ref_rmsnorm(_p(normed[r]), _p(summed[r]), _p(wd), ctypes.c_int(hidden), ctypes.c_float(eps))
        torch.cuda.synchronize()
        g.update({f"norm_{tag}_x": x, f"norm_{tag}_delta": d, f"norm_{tag}_w": w, f"norm_{tag}_eps": np.float32(eps),
                  f"norm_{tag}_sum": _host(summed), f"norm_{tag}_out": _host(normed)})

    # bias_add + rope at several positions
    for tag, fn, nh, nkv, hd, base, positions in (
            ("tiny", ref.ref_tiny_rope, 4, 2, 64, 10000.0, [0, 1, 37, 511]),
            ("q14b", ref.ref_q14b_rope, 40, 8, 128, 1000000.0, [0, 5, 4097, 32767])):
        qkv_out = (nh + 2 * nkv) * hd
        qkv = rng.standard_normal((len(positions), qkv_out), dtype=np.float32).astype(np.float16)
        bias = (rng.standard_normal(qkv_out, dtype=np.float32) * 0.1).astype(np.float16)
        work = _dev(qkv)
        bd = _dev(bias)
        for r, pos in enumerate(positions):
            ref.ref_bias_add(_p(work[r]), _p(bd), ctypes.c_int(qkv_out))
            fn(_p(work[r]), _p(work[r][nh * hd:]), ctypes.c_int(pos))
        torch.cuda.synchronize()
        g.update({f"rope_{tag}_qkv": qkv, f"rope_{tag}_bias": bias, f"rope_{tag}_pos": np.array(positions, np.int32),
                  f"rope_{tag}_out": _host(work), f"rope_{tag}_base": np.float32(base),
                  f"rope_{tag}_shape": np.array([nh, nkv, hd], np.int32)})

    # silu * up
    gate_up = (rng.standard_normal((3, 2 * 512), dtype=np.float32) * 2.0).astype(np.float16)
    gud = _dev(gate_up)
    mid = torch.empty((3, 512), dtype=torch.float16, device=DEV)
    for r in range(3):
        ref.ref_silu_mul(_p(mid[r]), _p(gud[r]), _p(gud[r][512:]), ctypes.c_int(512))
    torch.cuda.synchronize()
    g.update({"silu_gate_up": gate_up, "silu_out": _host(mid)})

    # argmax: a plain row, a row of ties at the maximum, a row of -inf
    logits = rng.standard_normal((3, 1024), dtype=np.float32).astype(np.float16)
    logits[1, [100, 613, 900]] = np.float16(9.0)
    logits[2, :] = np.float16(-np.inf)
    ld = _dev(logits)
    idx = torch.zeros(3, dtype=torch.int32, device=DEV)
    for r in range(3):
        ref.ref_argmax(_p(idx[r:]), _p(ld[r]), ctypes.c_int(1024))
    torch.cuda.synchronize()
    g.update({"argmax_logits": logits, "argmax_out": idx.cpu().numpy()})

    # the reference's forward() on the tiny model
    w = so.random_weights(TINY, TINY_SEED)
    keep = [_dev(w.embed), _dev(w.final_norm), _dev(w.lm_head)]
    ptrs = (ctypes.c_void_p * (7 * TINY.layers))()
    for l, lw in enumerate(w.layers):
        for j, k in enumerate(("attn_norm", "qkv", "qkv_bias", "o", "ffn_norm", "gate_up", "down")):
            t = _dev(lw[k])
            keep.append(t)
            ptrs[7 * l + j] = t.data_ptr()
    rc = ref.ref_tiny_set_weights(_p(keep[0]), _p(keep[1]), _p(keep[2]), ptrs)
    assert rc == 0
    tokens = np.zeros(TINY_STEPS + 1, np.int32)
    tokens[0] = TINY_FIRST_TOKEN
    all_logits = np.zeros((TINY_STEPS, TINY.vocab), np.float16)
    for i in range(TINY_STEPS):
        nxt = ref.ref_tiny_step(ctypes.c_int(int(tokens[i])), ctypes.c_int(i),
                                all_logits[i].ctypes.data_as(ctypes.c_void_p))
        assert nxt >= 0
        tokens[i + 1] = nxt
    g.update({"tiny_tokens": tokens, "tiny_logits": all_logits, "tiny_seed": np.int32(TINY_SEED),
              "tiny_weights_crc32": np.uint32(so.weights_checksum(w))})

    np.savez_compressed(out_dir / "runtime_kernels.npz", **g)
    print("wrote", out_dir / "runtime_kernels.npz", {k: v.shape for k, v in g.items() if hasattr(v, "shape")})


if __name__ == "__main__":
    main()
