"""One rank of the tensor-parallel decode-step test (launched by tests/test_step_tp_gpu.py through
torch.distributed.run, one process per GPU, NCCL). Each rank runs the library step on its shard with
the collectives on NCCL hooks ("nccl") or on the library's peer-memory exchange ("p2p") and checks its slice of the logits against the two-rank
CPU oracle; half-way through it switches to CUDA-graph replay."""
import datetime
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from oracle import step_oracle as so  # noqa: E402
from jacq_b200.runtime import DecodeModelConfig, DecodeRuntime, shard_layer  # noqa: E402

TINY = so.StepShape(layers=2, hidden=256, nh=4, nkv=2, hd=64, ffn=512, vocab=1024, rope_base=10000.0,
                    norm_eps=1e-5, attn_bias=True, block=16, group=32, residual=32)


def main():
    comm = sys.argv[1] if len(sys.argv) > 1 else "nccl"
    batch = int(sys.argv[2]) if len(sys.argv) > 2 else 3   # <= 4: GEMV with fused prologues; above: skinny GEMM path
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    device = torch.device(f"cuda:{int(os.environ['LOCAL_RANK'])}")
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=90))
    s = TINY
    cfg = DecodeModelConfig("test", s.layers, s.hidden, s.nh, s.nkv, s.hd, s.ffn, s.vocab, rope_base=s.rope_base,
                            norm_eps=s.norm_eps, attn_bias=s.attn_bias, block_size=s.block, group_size=s.group,
                            residual=s.residual)
    w = so.random_weights(s, 21)
    per_seq, steps = 8, 80
    bt = np.random.default_rng(9).permutation(batch * per_seq).reshape(batch, per_seq).astype(np.int32)
    oracle = so.StepOracle(s, w, bt, batch * per_seq, world=world)
    vl = s.vocab // world
    shard = {"embed": torch.from_numpy(w.embed), "final_norm": torch.from_numpy(w.final_norm),
             "lm_head": torch.from_numpy(w.lm_head[rank * vl: (rank + 1) * vl]),
             "layers": [shard_layer(cfg, {k: (None if v is None else torch.from_numpy(v)) for k, v in lw.items()},
                                    rank, world) for lw in w.layers]}
    rt = DecodeRuntime(cfg, shard, batch=batch, max_seq_len=per_seq * s.block + s.residual, device=device, rank=rank,
                       world=world, group=dist.group.WORLD, block_tables=torch.from_numpy(bt), comm=comm)
    dist.all_reduce(torch.zeros(8, device=device, dtype=torch.float16))   # communicator up before any capture
    tok = (np.arange(batch, dtype=np.int32) * 101 + 4) % s.vocab
    worst = 0.0
    for i in range(steps):
        if i == steps // 2:
            rt.capture()
        want_tok, want_logits = oracle.step(tok)
        got_tok = rt.step(torch.from_numpy(tok)).cpu().numpy()
        got = rt.logits.float().cpu().numpy()
        want = want_logits.astype(np.float32)[:, rank * vl: (rank + 1) * vl]
        worst = max(worst, float(np.abs(got - want).max()))
        np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-2, err_msg=f"rank {rank} step {i}")
        full = want_logits.astype(np.float32)
        top2 = np.sort(full, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 0.05
        assert np.array_equal(got_tok[clear], want_tok[clear]), f"rank {rank} step {i}"
        tok = want_tok.astype(np.int32)
    assert np.array_equal(rt.seq_lens.cpu().numpy(), np.full(batch, steps, np.int32))
    assert rt.exchange_status() == 0, "a peer-memory wait ran out of polls"
    rt.close()
    dist.barrier()
    torch.cuda.synchronize()
    print(f"TP_WORKER_OK comm={comm} batch={batch} rank={rank} worst_abs_err={worst:.3e}", flush=True)
    # leave without tearing the communicator down: destroying a process group whose collectives sit in a
    # captured CUDA graph has been seen to block for minutes
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
