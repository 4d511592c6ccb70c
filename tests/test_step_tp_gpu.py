"""KV-head tensor parallelism of the decode step on two GPUs, one process per GPU: once with the
collectives on NCCL (torch.distributed hooks), once on the library's own peer-memory exchange
(plain peer stores over NVLink, flags, the sum fused into the consuming kernel). NVLS is off and
no multimem instruction is used, so a rank that fails cannot fault its peer's GPU. Skipped on a
single-GPU box; tests/test_step_gpu.py covers the same library path there with host-side
collectives and the bounded wait of the exchange."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("batch", [3, 6])
@pytest.mark.parametrize("comm", ["nccl", "p2p"])
def test_two_rank_step(native_lib, comm, batch):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(29611 + (comm == "p2p") + 2 * (batch > 4)), str(ROOT / "tests" / "tp_worker.py"), comm,
           str(batch)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    out = proc.stdout + proc.stderr
    assert proc.returncode == 0, out[-4000:]
    assert out.count("TP_WORKER_OK") == 2, out[-4000:]
