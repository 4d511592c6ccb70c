"""The N > 1 path on CPU: two gloo ranks shard a ragged batch by decode bytes, each works only on its
own sequences (own pages, tables, scratch: no data-path collective), results are gathered and must
equal the single-process result; step time is the maximum over ranks, as bench.py reports it.
The per-rank arithmetic here is the CPU oracle (no GPU in this test)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jacq_b200 import sharding
from oracle import kivi_oracle as ko
from tests import helpers

SEQ_LENS = [1, 700, 33, 2050, 64, 1500, 65, 900]


def _problem():
    case = helpers.CONFIGS["tinyllama"]
    geom = helpers.oracle_geometry(case)
    n = len(SEQ_LENS)
    pages = max(geom.split_old(t) for t in SEQ_LENS) // case.b + 1
    tables = helpers.shuffled_block_tables(n, pages, n * pages)
    q = helpers.make_q(case, n)
    return case, geom, tables, q


def _decode_subset(case, geom, tables, q, idx):
    """What one rank does: build and decode only its own sequences, in a pool of its own."""
    pages = tables.shape[1]
    oc = ko.OracleCache(geom, len(idx) * pages, len(idx))
    local_tables = np.arange(len(idx) * pages, dtype=np.int32).reshape(len(idx), pages)
    for j, i in enumerate(idx):
        k, v = helpers.make_kv(case, SEQ_LENS[i], stream=i)
        ko.write_tokens(oc, k, v, local_tables[j], 0, slot=j)
    lens = np.array([SEQ_LENS[i] for i in idx], np.int32)
    return ko.decode_batch(oc, q[idx], local_tables, lens, mode=0)


def _rank_main(rank, world, port, out_queue):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case, geom, tables, q = _problem()
        lay = helpers.layout_of(case)
        costs = [lay.decode_algorithmic_bytes(t) for t in SEQ_LENS]
        shards = sharding.balanced_shards(costs, world)
        mine = shards[rank]
        out = _decode_subset(case, geom, tables, q, mine) if mine else np.zeros((0, case.nh, case.d), np.float32)
        gathered = [None] * world
        dist.all_gather_object(gathered, (mine, out))
        t = torch.tensor([float(rank + 1)], dtype=torch.float64)   # stand-in for this rank's step time
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        if rank == 0:
            full = np.zeros((len(SEQ_LENS), case.nh, case.d), np.float32)
            seen = []
            for idx, part in gathered:
                full[idx] = part
                seen += idx
            out_queue.put((sorted(seen), full, float(t.item()), sharding.shard_imbalance(costs, shards)))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.timeout(300)
def test_two_ranks_shard_sequences_without_a_collective():
    world = 2
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    seen, full, max_time, imbalance = queue.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert seen == list(range(len(SEQ_LENS))), "every sequence is owned by exactly one rank"
    assert max_time == float(world), "step time is the maximum over ranks"
    assert imbalance < 1.15
    case, geom, tables, q = _problem()
    want = _decode_subset(case, geom, tables, q, list(range(len(SEQ_LENS))))
    assert np.array_equal(full, want), "sharded result differs from the single-process result"
