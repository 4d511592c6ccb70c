"""The benchmark's command line as the driver uses it, on a machine without a GPU: the reference arm (the CPU
restatement of the reference's kernel math, oracle/) prints the one JSON line with the keys both arms share, and
the product arm refuses to run -- it has no CPU path to fall back to."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def _run(*args, timeout=600):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], cwd=ROOT, capture_output=True, text=True,
                          timeout=timeout)


def test_reference_arm_prints_the_shared_contract_line():
    proc = _run("--impl", "reference", "--steps", "1", "--warmup", "1")
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    assert line["metric"] == "KIVI decode-attn achieved HBM GB/s" and line["unit"] == "GB/s"
    assert line["higher_is_better"] is True and line["vs_baseline"] is None and line["data"] == "synthetic"
    assert line["n_gpus"] == 1 and line["steps"] == 1
    assert line["config"]["workload"] == "mistral7b_decode_attn_b128_t8192"
    assert line["value"] > 0 and line["ms_per_step"] > 0
    base = line["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and base["sample"] and base["value"] == line["value"]
    e2e = line["e2e"]
    assert e2e == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_under_torchrun_prints_once():
    """Launched one process per GPU like the product arm: rank 0 alone does the work and prints, the others leave."""
    proc = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                           "--master-addr", "127.0.0.1", "--master-port", "29631", str(ROOT / "bench.py"), "--impl",
                           "reference", "--gpus", "2", "--steps", "1", "--warmup", "1"],
                          cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["value"] > 0


@pytest.mark.skipif(torch.cuda.is_available(), reason="only meaningful where no GPU is present")
def test_product_arm_has_no_cpu_fallback():
    proc = _run("--steps", "1", "--warmup", "1", "--no-extras", "--no-cpu-baseline", timeout=300)
    assert proc.returncode != 0
    assert not proc.stdout.strip().startswith("{")
