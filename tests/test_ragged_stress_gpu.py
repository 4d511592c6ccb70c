"""Ragged stress (the batch-256 / context 1..32768 configuration): interleaved chunked-prefill
writes of 512 tokens and single-token decode writes that cross group and residual boundaries.

* reduced size (24 sequences up to 3000 tokens): packed cache compared BIT-EXACTLY with the CPU
  oracle after every step;
* full size (256 sequences, lengths uniform in 1..32768, head_dim 128, 32 q / 8 kv heads, block 16,
  group 128, residual 128): size-independent properties -- two different write schedules leave
  bit-identical caches; a constant V comes back from the attention exactly (softmax weights sum
  to one, the constant is representable in int4); a sample of sequences matches the oracle."""
import numpy as np
import pytest
import torch

from oracle import kivi_oracle as ko
from tests import helpers

pytestmark = pytest.mark.gpu


def _schedule(rng, target, chunk=512):
    """Per-step token counts for one sequence: a mix of chunks and single tokens up to target."""
    out, done = [], 0
    while done < target:
        n = chunk if rng.random() < 0.5 else 1
        n = min(n, target - done)
        out.append(n)
        done += n
    return out


def test_ragged_interleaved_writes_bit_exact_reduced(native_lib):
    from jacq_b200.cache import KiviCache
    from tests.gpu_utils import DEV, f16_tensor
    case = helpers.CONFIGS["mistral7b"]
    geom = helpers.oracle_geometry(case)
    rng = np.random.default_rng(20261125)
    n = 24
    targets = rng.integers(1, 3001, n)
    targets[:4] = [1, case.r, case.r + case.g, case.r + 2 * case.g + 1]
    scheds = [_schedule(rng, int(t)) for t in targets]
    steps = max(len(s) for s in scheds)
    pages = (int(targets.max()) + 600) // case.b + 1
    tables = helpers.shuffled_block_tables(n, pages, n * pages + 7)
    oc = ko.OracleCache(geom, n * pages + 7, n, fill=0x77)
    cache = KiviCache(helpers.layout_of(case), n * pages + 7, n, pages, DEV, fill=0x77)
    cache.set_block_tables(torch.from_numpy(tables))
    kv = [helpers.make_kv(case, int(targets[i]), stream=i) for i in range(n)]
    lens = np.zeros(n, np.int32)
    for step in range(steps):
        counts = np.array([s[step] if step < len(s) else 0 for s in scheds], np.int32)
        offs = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        nk = np.concatenate([kv[i][0][lens[i]:lens[i] + counts[i]] for i in range(n)])
        nv = np.concatenate([kv[i][1][lens[i]:lens[i] + counts[i]] for i in range(n)])
        ko.write_batch(oc, nk, nv, tables, lens, offs, nthreads=8)
        cache.write(f16_tensor(nk), f16_tensor(nv), torch.from_numpy(offs).to(DEV),
                    max_new_per_seq=int(counts.max()), max_start_seq_len=int(lens.max()))
        lens = lens + counts
        torch.cuda.synchronize()
        live = [int(t - geom.split_old(int(t))) for t in lens]
        helpers.assert_cache_equal(cache.tensors, oc, live_rows=live, what=f"step {step}: ")
    assert np.array_equal(lens, targets)
    q = helpers.make_q(case, n)
    got = cache.decode(f16_tensor(q), max_seq_len=int(lens.max())).cpu().numpy()
    want = ko.decode_batch(oc, q, tables, lens, mode=1, nthreads=8)
    assert (np.abs(got - want) <= 1e-2 + 1e-2 * np.abs(want)).all()


def _fill_full_size(cache, case, targets, chunk, const_v, seed):
    """Write every sequence up to its target: `chunk`-token chunks while they fit, one odd-sized
    chunk for the remainder, and the last (target % chunk) % 7 tokens one at a time."""
    import torch
    dev = cache.device
    n = len(targets)
    gen = torch.Generator(device=dev)
    done = torch.zeros(n, dtype=torch.int64)
    tgt = torch.from_numpy(targets.astype(np.int64))
    step = 0
    while bool((done < tgt).any()):
        left = tgt - done
        tail = (tgt % chunk) % 7                      # the last few tokens go in one at a time
        body = torch.clamp(left - tail, min=0)        # what is still to be written in chunks
        counts = torch.where(body > 0, torch.minimum(body, torch.full_like(body, chunk)),
                             torch.where(left > 0, torch.ones_like(left), torch.zeros_like(left)))
        total = int(counts.sum())
        offs = torch.zeros(n + 1, dtype=torch.int32)
        offs[1:] = torch.cumsum(counts, 0).to(torch.int32)
        # token content depends only on (sequence, position): generate per sequence streams
        pos = torch.cat([torch.arange(int(done[i]), int(done[i] + counts[i])) + (i << 20) for i in range(n)]).to(dev)
        gen.manual_seed(seed)
        base = torch.randn((4096, case.nkv, case.d), device=dev, dtype=torch.float16, generator=gen)
        k = base[(pos * 2654435761 % 4096)] * (1.0 + (pos % 13).to(torch.float16)[:, None, None] * 0.1)
        v = torch.full_like(k, const_v) if const_v is not None else base[(pos * 40503 % 4096)]
        cache.write(k.contiguous(), v.contiguous(), offs.to(dev), max_new_per_seq=int(counts.max()),
                    max_start_seq_len=int(done.max()))
        done += counts
        step += 1
    return step


def test_ragged_full_size_properties(native_lib):
    from jacq_b200.cache import KiviCache
    from tests.gpu_utils import DEV, f16_tensor, oracle_copy
    case = helpers.CONFIGS["mistral7b"]
    lay = helpers.layout_of(case)
    rng = np.random.default_rng(5)
    n = 256
    targets = rng.integers(1, 32769, n)
    targets[:3] = [1, 32768, case.r + case.g]
    pages = lay.old_pages(32768) + 1
    perm = torch.from_numpy(helpers.shuffled_block_tables(n, pages, n * pages))
    a = KiviCache(lay, n * pages, n, pages, DEV)
    b = KiviCache(lay, n * pages, n, pages, DEV)
    a.set_block_tables(perm)
    b.set_block_tables(perm)
    _fill_full_size(a, case, targets, 512, 0.75, seed=3)
    _fill_full_size(b, case, targets, 384, 0.75, seed=3)
    torch.cuda.synchronize()
    tl = torch.from_numpy(targets.astype(np.int32)).to(DEV)
    assert torch.equal(a.seq_lens, tl) and torch.equal(b.seq_lens, tl)
    for name in helpers.PAGE_FIELDS:
        assert torch.equal(getattr(a.tensors, name), getattr(b.tensors, name)), f"{name}: schedules disagree"
    live = targets - np.maximum(0, targets - case.r) // case.g * case.g
    rows = torch.arange(lay.scratch_rows, device=DEV)[None, None, :, None] < torch.from_numpy(live).to(DEV)[:, None, None, None]
    for name in ("K_RESIDUAL_SCRATCH", "V_RESIDUAL_SCRATCH"):
        x, y = getattr(a.tensors, name), getattr(b.tensors, name)
        assert torch.equal(torch.where(rows, x, torch.zeros_like(x)), torch.where(rows, y, torch.zeros_like(y))), name
    # attention over a constant V returns the constant
    q = f16_tensor(helpers.make_q(case, n))
    out = a.decode(q, max_seq_len=32768)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
    assert float((out - 0.75).abs().max()) < 2e-3
    # a sample of sequences against the oracle (pages copied to the host)
    sample = [0, 1, 2, 17, 200]
    oc, tables = oracle_copy(a, case, sample)
    lens = targets[sample].astype(np.int32)
    want = ko.decode_batch(oc, helpers.to_bits(q[sample]), tables, lens, mode=1, nthreads=8)
    got = out[sample].cpu().numpy()
    assert (np.abs(got - want) <= 1e-2 + 1e-2 * np.abs(want)).all()
    # the same sample, bit for bit: the CPU oracle's token-by-token writer over the sequences' own K/V rows
    # (regenerated from their positions) must leave the pages and live scratch rows the device holds
    gen = torch.Generator(device=DEV)
    gen.manual_seed(3)
    base = torch.randn((4096, case.nkv, case.d), device=DEV, dtype=torch.float16, generator=gen)
    ks, vs = [], []
    for i in sample:
        pos = (torch.arange(int(targets[i])) + (i << 20)).to(DEV)
        k = base[(pos * 2654435761 % 4096)] * (1.0 + (pos % 13).to(torch.float16)[:, None, None] * 0.1)
        ks.append(helpers.to_bits(k))
        vs.append(helpers.to_bits(torch.full_like(k, 0.75)))
    ref = ko.OracleCache(oc.geom, oc.num_blocks, oc.num_slots)
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ko.write_batch(ref, np.concatenate(ks), np.concatenate(vs), tables, np.zeros(len(sample), np.int32), offs, nthreads=8)
    for i, t in enumerate(lens):
        used = oc.geom.split_old(int(t)) // case.b
        for name in ko.OracleCache.PAGE_FIELDS:
            a_, b_ = getattr(oc, name)[tables[i, :used]], getattr(ref, name)[tables[i, :used]]
            assert np.array_equal(a_, b_), f"sequence {sample[i]}: {name} differs from the oracle writer"
        rows_live = int(t) - oc.geom.split_old(int(t))
        assert np.array_equal(oc.k_scratch[i][:, :rows_live], ref.k_scratch[i][:, :rows_live])
        assert np.array_equal(oc.v_scratch[i][:, :rows_live], ref.v_scratch[i][:, :rows_live])
