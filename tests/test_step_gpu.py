"""Decode step around the KIVI cache: element-wise kernels and the whole step.

Checked three ways: (1) bit-exactly against golden outputs of the reference's own kernels
(templates/kernels.cu, generated on a B200 by tests/golden/make_runtime_golden.py); (2) against the
reference's own forward() on the tiny model while every token is still in the fp16 residual window
(where KIVI attention is plain fp16 attention), logits within rtol = atol = 1e-2; (3) against the
CPU step oracle across the quantisation boundary and for several batch sizes.
"""
import ctypes
import threading
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import kivi_oracle as ko
from oracle import step_oracle as so

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).resolve().parent / "golden" / "runtime_kernels.npz"
TINY = so.StepShape(layers=2, hidden=256, nh=4, nkv=2, hd=64, ffn=512, vocab=1024, rope_base=10000.0,
                    norm_eps=1e-5, attn_bias=True, block=16, group=32, residual=32)


@pytest.fixture(scope="module")
def golden():
    if not GOLDEN.exists():
        pytest.skip("tests/golden/runtime_kernels.npz not generated yet")
    return np.load(GOLDEN)


def _dev(a):
    from tests.gpu_utils import DEV
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16:
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.float16).to(DEV)
    return torch.from_numpy(a).to(DEV)


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def _call(fn, *args):
    from jacq_b200 import _native
    _native.check(fn(*args), fn.__name__)


def _rmsnorm(native_lib, x, delta, w, eps):
    from tests.gpu_utils import ptr, stream_ptr
    xd, wd = _dev(x), _dev(w)
    dd = None if delta is None else _dev(delta)
    x_out, normed = torch.empty_like(xd), torch.empty_like(xd)
    _call(native_lib.kivi_b200_residual_rmsnorm, ptr(xd), ptr(dd) if dd is not None else None, ptr(wd), ptr(x_out),
          ptr(normed), x.shape[0], x.shape[1], ctypes.c_float(eps), stream_ptr())
    torch.cuda.synchronize()
    return x_out, normed


def _rope(native_lib, qkv, bias, pos, nh, nkv, hd, base):
    from tests.gpu_utils import DEV, ptr, stream_ptr
    n = qkv.shape[0]
    q = torch.empty((n, nh * hd), dtype=torch.float16, device=DEV)
    k = torch.empty((n, nkv * hd), dtype=torch.float16, device=DEV)
    v = torch.empty((n, nkv * hd), dtype=torch.float16, device=DEV)
    qd, pd = _dev(qkv), _dev(np.asarray(pos, np.int32))
    bd = None if bias is None else _dev(bias)
    _call(native_lib.kivi_b200_bias_rope, ptr(qd), ptr(bd) if bd is not None else None, ptr(pd), ptr(q), ptr(k), ptr(v),
          n, nh, nkv, hd, ctypes.c_float(base), stream_ptr())
    torch.cuda.synchronize()
    return q, k, v


def _silu(native_lib, gate_up):
    from tests.gpu_utils import DEV, ptr, stream_ptr
    n, two = gate_up.shape
    out = torch.empty((n, two // 2), dtype=torch.float16, device=DEV)
    gd = _dev(gate_up)
    _call(native_lib.kivi_b200_silu_mul, ptr(gd), ptr(out), n, two // 2, stream_ptr())
    torch.cuda.synchronize()
    return out


def _argmax(native_lib, logits):
    from tests.gpu_utils import DEV, ptr, stream_ptr
    n, vocab = logits.shape
    out = torch.zeros(n, dtype=torch.int32, device=DEV)
    ws = torch.zeros(n * (vocab // 8192 + 1) * 8, dtype=torch.uint8, device=DEV)
    ld = _dev(logits)
    _call(native_lib.kivi_b200_argmax, ptr(ld), ptr(out), n, vocab, ptr(ws), ws.numel(), stream_ptr())
    torch.cuda.synchronize()
    return out.cpu().numpy()


# ---- (1) the reference's kernels, bit for bit ------------------------------------------------

@pytest.mark.parametrize("tag", ["h256", "h5120"])
def test_residual_rmsnorm_bit_exact_vs_reference_kernels(native_lib, golden, tag):
    g = golden
    x_out, normed = _rmsnorm(native_lib, g[f"norm_{tag}_x"], g[f"norm_{tag}_delta"], g[f"norm_{tag}_w"],
                             float(g[f"norm_{tag}_eps"]))
    assert np.array_equal(_bits(x_out), g[f"norm_{tag}_sum"].view(np.uint16))
    assert np.array_equal(_bits(normed), g[f"norm_{tag}_out"].view(np.uint16))


@pytest.mark.parametrize("tag", ["tiny", "q14b"])
def test_bias_rope_bit_exact_vs_reference_kernels(native_lib, golden, tag):
    g = golden
    nh, nkv, hd = (int(v) for v in g[f"rope_{tag}_shape"])
    q, k, v = _rope(native_lib, g[f"rope_{tag}_qkv"], g[f"rope_{tag}_bias"], g[f"rope_{tag}_pos"], nh, nkv, hd,
                    float(g[f"rope_{tag}_base"]))
    want = g[f"rope_{tag}_out"].view(np.uint16)
    got = np.concatenate([_bits(q), _bits(k), _bits(v)], axis=1)
    assert np.array_equal(got[:, (nh + nkv) * hd:], want[:, (nh + nkv) * hd:])       # v: bias add only
    small = g[f"rope_{tag}_pos"] < 4096
    assert np.array_equal(got[small], want[small])
    # at positions in the thousands a few elements per ten thousand land one fp16 ulp away: the reference's
    # ROPE_BASE is a compile-time constant, which lets its compiler fold part of powf()
    dist = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert dist.max() <= 1 and (dist != 0).mean() < 1e-3, (int(dist.max()), float((dist != 0).mean()))


def test_silu_mul_bit_exact_vs_reference_kernel(native_lib, golden):
    out = _silu(native_lib, golden["silu_gate_up"])
    assert np.array_equal(_bits(out), golden["silu_out"].view(np.uint16))


def test_argmax_vs_reference_kernel(native_lib, golden):
    logits = golden["argmax_logits"]
    got = _argmax(native_lib, logits)
    want = golden["argmax_out"]
    assert got[0] == want[0]
    # equal maxima: the reference's pick depends on its thread layout, this library takes the lowest index
    assert logits[1, want[1]] == logits[1, got[1]] and got[1] == 100
    assert got[2] == want[2] == 0   # nothing beats the -1e30 floor: index 0


# ---- the same kernels against the CPU oracle on other shapes ----------------------------------

def _ulp_close(got_bits: np.ndarray, want_bits: np.ndarray, max_ulp=1, min_exact=0.98):
    diff = np.abs(got_bits.astype(np.int32) - want_bits.astype(np.int32))
    assert diff.max() <= max_ulp, f"max fp16 ulp distance {diff.max()}"
    assert (diff == 0).mean() >= min_exact


@pytest.mark.parametrize("batch,hidden", [(1, 8), (3, 1000), (64, 5120), (2, 16384)])
def test_residual_rmsnorm_vs_oracle(native_lib, batch, hidden):
    rng = np.random.default_rng(hidden + batch)
    x = rng.standard_normal((batch, hidden), dtype=np.float32).astype(np.float16)
    d = rng.standard_normal((batch, hidden), dtype=np.float32).astype(np.float16)
    w = (1 + 0.1 * rng.standard_normal(hidden, dtype=np.float32)).astype(np.float16)
    for delta in (d, None):
        x_out, normed = _rmsnorm(native_lib, x, delta, w, 1e-6)
        want_x, want_n = ko.residual_rmsnorm(x, delta, w, 1e-6)
        assert np.array_equal(_bits(x_out), want_x.view(np.uint16))   # fp16 add is exact arithmetic + one rounding
        _ulp_close(_bits(normed), want_n.view(np.uint16))             # rsqrtf differs from 1/sqrtf in the last place


@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 64), (32, 8, 128), (14, 2, 64), (5, 1, 128)])
@pytest.mark.parametrize("with_bias", [True, False])
def test_bias_rope_vs_oracle(native_lib, nh, nkv, hd, with_bias):
    rng = np.random.default_rng(nh * hd)
    pos = np.array([0, 3, 1000, 32767, 131071], np.int32)
    qkv = rng.standard_normal((len(pos), (nh + 2 * nkv) * hd), dtype=np.float32).astype(np.float16)
    bias = (rng.standard_normal((nh + 2 * nkv) * hd, dtype=np.float32) * 0.1).astype(np.float16) if with_bias else None
    q, k, v = _rope(native_lib, qkv, bias, pos, nh, nkv, hd, 1000000.0)
    wq, wk, wv = ko.bias_rope(qkv, bias, pos, nh, nkv, hd, 1000000.0)
    assert np.array_equal(_bits(v), wv.view(np.uint16))
    # powf / sinf / cosf of the device library are within a few fp32 ulp of libm: at most the last fp16 place,
    # except at large angles where an fp32 ulp of the angle is already visible
    for got, want in ((q, wq), (k, wk)):
        np.testing.assert_allclose(got.cpu().numpy().astype(np.float32), want.astype(np.float32), rtol=2e-3, atol=2e-2)
    small = pos < 2000
    _ulp_close(_bits(q)[small], wq.view(np.uint16)[small], max_ulp=2, min_exact=0.95)


def test_silu_mul_and_argmax_vs_oracle(native_lib):
    rng = np.random.default_rng(5)
    gate_up = (rng.standard_normal((5, 2 * 13824), dtype=np.float32) * 3).astype(np.float16)
    _ulp_close(_bits(_silu(native_lib, gate_up)), ko.silu_mul(gate_up).view(np.uint16))
    logits = rng.standard_normal((7, 152064), dtype=np.float32).astype(np.float16)
    logits[3, 777] = logits[3].max()          # a tie: the lower index must win
    logits[4, :] = np.float16("nan")
    assert np.array_equal(_argmax(native_lib, logits), ko.argmax(logits))


# ---- (2), (3): the whole step --------------------------------------------------------------------

def _torch_weights(w: so.StepWeights):
    return {"embed": torch.from_numpy(w.embed), "final_norm": torch.from_numpy(w.final_norm),
            "lm_head": torch.from_numpy(w.lm_head),
            "layers": [{k: (None if v is None else torch.from_numpy(v)) for k, v in lw.items()} for lw in w.layers]}


def _config(shape: so.StepShape):
    from jacq_b200.runtime import DecodeModelConfig
    return DecodeModelConfig("test", shape.layers, shape.hidden, shape.nh, shape.nkv, shape.hd, shape.ffn, shape.vocab,
                             rope_base=shape.rope_base, norm_eps=shape.norm_eps, attn_bias=shape.attn_bias,
                             block_size=shape.block, group_size=shape.group, residual=shape.residual)


def _tables(batch, per_seq, seed):
    rng = np.random.default_rng(seed)
    return rng.permutation(batch * per_seq).reshape(batch, per_seq).astype(np.int32)


def test_step_matches_reference_forward_inside_the_residual_window(native_lib, golden):
    """60 tokens through the tiny model: the reference's forward() (fp16 dense cache) against this
    library's step (KIVI cache with R = G = 32, so nothing is quantised before token 64)."""
    from jacq_b200.runtime import DecodeRuntime
    from tests.gpu_utils import DEV
    w = so.random_weights(TINY, int(golden["tiny_seed"]))
    if so.weights_checksum(w) != int(golden["tiny_weights_crc32"]):
        pytest.skip("numpy's generator no longer reproduces the weights the golden run used")
    rt = DecodeRuntime(_config(TINY), _torch_weights(w), batch=1, max_seq_len=128, device=DEV)
    tokens, want = golden["tiny_tokens"], golden["tiny_logits"].astype(np.float32)
    agree = 0
    for i in range(want.shape[0]):
        nxt = rt.step(torch.tensor([int(tokens[i])]))
        got = rt.logits.float().cpu().numpy()[0]
        np.testing.assert_allclose(got, want[i], rtol=1e-2, atol=1e-2, err_msg=f"step {i}")
        agree += int(nxt.item() == tokens[i + 1])
    assert agree >= want.shape[0] - 2   # greedy picks may differ only on near-ties


@pytest.mark.parametrize("batch", [1, 3, 8])
def test_step_matches_oracle_across_quantisation(native_lib, batch):
    """80 steps: the first key group is quantised at token 64; logits stay within the contract's
    tolerance of the CPU oracle, which is fed the same tokens."""
    from jacq_b200.runtime import DecodeRuntime
    from tests.gpu_utils import DEV
    w = so.random_weights(TINY, 11)
    per_seq = 8
    bt = _tables(batch, per_seq, batch)
    oracle = so.StepOracle(TINY, w, bt, batch * per_seq)
    rt = DecodeRuntime(_config(TINY), _torch_weights(w), batch=batch, max_seq_len=per_seq * TINY.block + TINY.residual,
                       device=DEV, block_tables=torch.from_numpy(bt))
    tok = np.arange(batch, dtype=np.int32) * 37 + 3
    worst = 0.0
    for i in range(80):
        want_tok, want_logits = oracle.step(tok)
        got_tok = rt.step(torch.from_numpy(tok)).cpu().numpy()
        got = rt.logits.float().cpu().numpy()
        want = want_logits.astype(np.float32)
        worst = max(worst, float(np.abs(got - want).max()))
        np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-2, err_msg=f"step {i}")
        top2 = np.sort(want, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 0.05
        assert np.array_equal(got_tok[clear], want_tok[clear])
        tok = want_tok.astype(np.int32)
    assert np.array_equal(rt.seq_lens.cpu().numpy(), np.full(batch, 80, np.int32))
    assert worst < 2e-2


Q14B_LAYER = so.StepShape(layers=2, hidden=5120, nh=40, nkv=8, hd=128, ffn=13824, vocab=4096, rope_base=1000000.0,
                          norm_eps=1e-6, attn_bias=True, block=16, group=128, residual=128)


@pytest.mark.parametrize("batch", [1, 8])
def test_step_at_the_qwen25_14b_layer_shape_across_an_age_out(native_lib, batch):
    """Two layers of the full-model configuration's shape (hidden 5120, 40 query / 8 kv heads of 128, FFN 13824,
    block 16 / group 128 / residual 128; a 4096-row vocabulary keeps the CPU side short), 250 tokens of
    synthetic context written into both sides' caches, then 9 steps: the 6th makes the scratch full and quantises
    the first key group. Batch 1 runs the fused GEMV kernels, batch 8 the tensor-core skinny GEMM and the
    stand-alone element-wise kernels. Logits against the CPU step oracle fed the same tokens."""
    from jacq_b200.runtime import DecodeRuntime
    from tests.gpu_utils import DEV, f16_tensor
    shape = Q14B_LAYER
    w = so.random_weights(shape, 77)
    start, steps = 250, 9
    max_len = 512
    per_seq = (max_len - shape.residual) // shape.group * shape.group // shape.block   # the runtime's table width
    bt = _tables(batch, per_seq, 100 + batch)
    oracle = so.StepOracle(shape, w, bt, batch * per_seq, gemv_threads=16)
    rt = DecodeRuntime(_config(shape), _torch_weights(w), batch=batch, max_seq_len=max_len,
                       device=DEV, block_tables=torch.from_numpy(bt))
    rng = np.random.default_rng(5)
    offs = np.arange(batch + 1, dtype=np.int32) * start
    for l in range(shape.layers):
        k = rng.standard_normal((batch * start, shape.nkv, shape.hd), dtype=np.float32)
        k[:, :, :3] *= 10.0
        k = k.astype(np.float16)
        v = rng.standard_normal((batch * start, shape.nkv, shape.hd), dtype=np.float32).astype(np.float16)
        ko.write_batch(oracle.caches[0][l], k, v, bt, np.zeros(batch, np.int32), offs, nthreads=8)
        c = rt.caches[l]
        c.set_block_tables(torch.from_numpy(bt))
        c.write(f16_tensor(k), f16_tensor(v), torch.from_numpy(offs).to(DEV), max_new_per_seq=start, max_start_seq_len=0)
    oracle.seq_lens[:] = start
    rt.set_seq_lens([start] * batch)
    tok = (np.arange(batch, dtype=np.int32) * 311 + 5) % shape.vocab
    worst = 0.0
    for i in range(steps):
        want_tok, want_logits = oracle.step(tok)
        got_tok = rt.step(torch.from_numpy(tok)).cpu().numpy()
        got = rt.logits.float().cpu().numpy()
        want = want_logits.astype(np.float32)
        worst = max(worst, float(np.abs(got - want).max()))
        np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-2, err_msg=f"step {i}")
        top2 = np.sort(want, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 0.05
        assert np.array_equal(got_tok[clear], want_tok[clear])
        tok = want_tok.astype(np.int32)
    assert np.array_equal(rt.seq_lens.cpu().numpy(), np.full(batch, start + steps, np.int32))
    # the quantised group and the live scratch rows of every layer, bit for bit
    torch.cuda.synchronize()
    geom = oracle.geom
    live = [start + steps - geom.split_old(start + steps)] * batch
    assert geom.split_old(start + steps) == shape.group
    from tests import helpers
    for l in range(shape.layers):
        oc = oracle.caches[0][l]
        used = np.unique(bt[:, : shape.group // shape.block])
        for name in helpers.PAGE_FIELDS:
            got_pages = helpers.to_bits(getattr(rt.caches[l].tensors, name))[used]
            want_pages = getattr(oc, helpers.ORACLE_FIELD[name])[used]
            assert np.array_equal(got_pages, want_pages), f"layer {l} {name}"


def test_step_graph_replay_equals_eager(native_lib):
    from jacq_b200.runtime import DecodeRuntime
    from tests.gpu_utils import DEV
    w = so.random_weights(TINY, 3)
    cfg, tw = _config(TINY), _torch_weights(w)
    eager = DecodeRuntime(cfg, tw, batch=4, max_seq_len=160, device=DEV)
    graphed = DecodeRuntime(cfg, tw, batch=4, max_seq_len=160, device=DEV)
    graphed.capture()
    tok = torch.tensor([1, 2, 3, 4], dtype=torch.int32)
    eager.tokens.copy_(tok)
    graphed.tokens.copy_(tok)
    for i in range(100):   # free-running greedy decoding, crossing the first quantisation boundary
        a = eager.step().clone()
        b = graphed.step().clone()
        assert torch.equal(a, b), f"step {i}"
        assert torch.equal(eager.logits, graphed.logits)
    for ce, cg in zip(eager.caches, graphed.caches):
        for name in ce.tensors.names():
            assert torch.equal(getattr(ce.tensors, name), getattr(cg.tensors, name)), name


def test_step_tensor_parallel_two_ranks_on_one_gpu(native_lib):
    """KV-head tensor parallelism of the library step, two ranks as two host threads on one GPU.
    The collective hooks are served on the host (a barrier and torch adds), so no kernel ever waits
    for another; results are compared with the two-rank CPU oracle and the one-rank library run."""
    from jacq_b200 import _native
    from jacq_b200.runtime import DecodeRuntime, shard_layer
    from tests.gpu_utils import DEV
    world, batch, per_seq, steps = 2, 3, 8, 70
    w = so.random_weights(TINY, 21)
    cfg, tw = _config(TINY), _torch_weights(w)
    bt = _tables(batch, per_seq, 9)
    max_len = per_seq * TINY.block + TINY.residual
    single = DecodeRuntime(cfg, tw, batch=batch, max_seq_len=max_len, device=DEV, block_tables=torch.from_numpy(bt))
    oracle = so.StepOracle(TINY, w, bt, batch * per_seq, world=world)

    class HostGroup:
        """All-reduce / all-gather between threads: rendezvous on the host, arithmetic by torch."""
        def __init__(self):
            self.barrier = threading.Barrier(world)
            self.slots = [None] * world

        def exchange(self, rank, tensor):
            torch.cuda.synchronize()
            self.slots[rank] = tensor
            self.barrier.wait()
            parts = list(self.slots)
            self.barrier.wait()
            return parts

    group = HostGroup()
    ranks = []
    for r in range(world):
        shard = {"embed": tw["embed"], "final_norm": tw["final_norm"],
                 "lm_head": tw["lm_head"][r * (TINY.vocab // world): (r + 1) * (TINY.vocab // world)],
                 "layers": [shard_layer(cfg, lw, r, world) for lw in tw["layers"]]}
        rt = DecodeRuntime.__new__(DecodeRuntime)
        rt_group = object()   # stands in for a process group; the hooks below replace the NCCL ones

        def make_comm(self, r=r):
            def allreduce(_u, buf, count, _s):
                mine = self._view(buf, count * 2).view(torch.float16)
                parts = group.exchange(r, mine.clone())
                acc = torch.zeros_like(mine, dtype=torch.float32)
                for p in parts:
                    acc += p.float()
                mine.copy_(acc.half())
                torch.cuda.synchronize()
                return 0

            def allgather(_u, send, recv, nbytes, _s):
                parts = group.exchange(r, self._view(send, nbytes).clone())
                self._view(recv, nbytes * world).copy_(torch.cat(parts))
                torch.cuda.synchronize()
                return 0

            self._callbacks = (_native.ALLREDUCE_F16_FN(allreduce), _native.ALLGATHER_FN(allgather))
            return _native.KiviStepComm(self._callbacks[0], self._callbacks[1], None)

        rt._make_comm = make_comm.__get__(rt)
        DecodeRuntime.__init__(rt, cfg, shard, batch=batch, max_seq_len=max_len, device=DEV, rank=r, world=world,
                               group=rt_group, block_tables=torch.from_numpy(bt))
        ranks.append(rt)

    tok = np.array([4, 99, 512], np.int32)
    torch.cuda.synchronize()
    for i in range(steps):
        want_tok, want_logits = oracle.step(tok)
        single_tok = single.step(torch.from_numpy(tok)).cpu().numpy()
        results, errors = [None] * world, []

        def run(r):
            try:
                with torch.cuda.stream(torch.cuda.Stream(DEV)):
                    results[r] = ranks[r].step(torch.from_numpy(tok)).cpu().numpy()
            except Exception as exc:   # surface a failure instead of leaving the peer at the barrier
                errors.append(exc)
                group.barrier.abort()

        threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        assert not errors, errors
        logits = torch.cat([rt.logits for rt in ranks], dim=1).float().cpu().numpy()
        want = want_logits.astype(np.float32)
        np.testing.assert_allclose(logits, want, rtol=2e-2, atol=2e-2, err_msg=f"step {i} vs two-rank oracle")
        np.testing.assert_allclose(logits, single.logits.float().cpu().numpy(), rtol=2e-2, atol=2e-2)
        assert np.array_equal(results[0], results[1])           # every rank ends with the same tokens
        top2 = np.sort(want, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 0.05
        assert np.array_equal(results[0][clear], want_tok[clear])
        assert np.array_equal(single_tok[clear], want_tok[clear])
        tok = want_tok.astype(np.int32)


def test_peer_exchange_wait_is_bounded(native_lib):
    """Rank 0 of a two-rank peer-memory step whose peer never delivers: every wait runs out of its
    (shortened) poll budget, the step returns, and the status word names the missing rank. Both
    regions live on this GPU and nothing ever writes the second rank's flags."""
    import ctypes
    from jacq_b200 import _native
    from jacq_b200.runtime import DecodeRuntime, shard_layer
    from tests.gpu_utils import DEV
    world, batch = 2, 2
    w = so.random_weights(TINY, 31)
    cfg, tw = _config(TINY), _torch_weights(w)
    shard = {"embed": tw["embed"], "final_norm": tw["final_norm"], "lm_head": tw["lm_head"][: TINY.vocab // world],
             "layers": [shard_layer(cfg, lw, 0, world) for lw in tw["layers"]]}
    rt = DecodeRuntime.__new__(DecodeRuntime)
    rt._make_comm = lambda: None                      # built by hand below
    DecodeRuntime.__init__(rt, cfg, shard, batch=batch, max_seq_len=160, device=DEV, rank=0, world=world, group=object())
    lib = native_lib
    nbytes = int(lib.kivi_b200_p2p_region_bytes(ctypes.byref(rt._cfg_struct), batch))
    assert nbytes > 0
    regions = []
    for _ in range(world):
        region = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * _native.P2P_HANDLE_BYTES)()
        _native.check(lib.kivi_b200_p2p_region_create(nbytes, ctypes.byref(region), handle), "region_create")
        regions.append(region.value)
    ptrs = (ctypes.c_void_p * world)(*regions)
    rt._region = regions[0]
    rt._comm = _native.KiviStepComm(ctypes.cast(None, _native.ALLREDUCE_F16_FN), ctypes.cast(None, _native.ALLGATHER_FN),
                                    None, ptrs, nbytes, 2000)
    assert rt.exchange_status() == 0
    rt.step(torch.tensor([1, 2]))
    torch.cuda.synchronize()
    assert rt.exchange_status() == 0b10              # rank 1 never delivered; rank 0's own pushes were seen
    rt.step(torch.tensor([3, 4]))                    # the error is sticky: later waits do not poll again
    torch.cuda.synchronize()
    assert rt.exchange_status() == 0b10
    assert torch.equal(rt.seq_lens.cpu(), torch.tensor([2, 2], dtype=torch.int32))
    # a region that is too small is refused before anything is launched
    rt._comm.region_bytes = nbytes - 256
    with pytest.raises(_native.KiviStatusError):
        rt.step(torch.tensor([1, 2]))
    for r in regions:
        lib.kivi_b200_p2p_region_destroy(r)
    rt._region = None
