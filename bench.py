"""Benchmark of the int4-KIVI paged decode attention on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

A step is ONE pass of the paged decode attention over one batch of sequences for one layer (the
library's kivi_b200_decode: one kernel launch). Workload at one GPU: the Mistral-7B decode shape
(32 q / 8 kv heads, head_dim 128, batch 128, context 8192, block 16, group 128, residual 128) on
seeded synthetic q/K/V (fp16 N(0,1), 3 of 128 key channels per head x10); the cache is built on
the device by the library's own writer. With N GPUs every rank holds its own 128 sequences
(independent sequences, no collective: weak scaling); the value is the aggregate over ranks.

metric / value  achieved HBM GB/s = algorithmic bytes of the step / device time, inputs resident
                in HBM; tokens/s rides along as `tokens_per_s`
e2e             the same bytes over the time of a full serving step through the public API with
                HOST buffers: pinned q and the step's new K/V rows copied host->device, cache write,
                decode, output copied device->host; the step is captured once as a CUDA graph and
                launched once per step (--no-e2e-graph: separate calls), and its last output is
                checked against a separate decode of the same cache state
roofline        achieved = algorithmic bytes per launch / mean CUDA-event time of the decode launch,
                against the measured HBM copy bandwidth in MEASURED_PEAKS.json
cpu_baseline    the scalar CPU oracle (test infrastructure, a port of the reference's kernel math)
                timed on the host cores on a bounded sample of the same workload
--impl reference  times that CPU port with all host threads (the reference's own implementation of
                this path is CUDA-only and cannot express this geometry)
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (case key in tests.helpers.CONFIGS, batch, context)
    "mistral7b_decode_attn_b128_t8192": ("mistral7b", 128, 8192),
    "qwen05b_decode_attn_b64_t4096": ("qwen05b", 64, 4096),
    "tinyllama_decode_attn_b4_t512": ("tinyllama", 4, 512),
    "reflane_decode_attn_b64_t4096": ("reflane", 64, 4096),
    # same kernel and geometry as the default, a quarter of the batch: 373 MB of pages, still 3x the L2;
    # sized for `ncu --set full` captures
    "mistral7b_decode_attn_b32_t8192": ("mistral7b", 32, 8192),
    # enough (sequence, kv head) units that the context is not split: every CTA walks a whole sequence
    "mistral7b_decode_attn_b48_t8192": ("mistral7b", 48, 8192),
}
# secondary workloads: the other two parts of the path, each against its own HBM roofline
SECONDARY = {
    # one step = the four projections (qkv, o, gate_up, down) of 8 layers of the Qwen2.5-14B shape at
    # batch 1, every GEMV on its own weights: 4.4 GB of fp16 weights streamed once per step
    "gemv_qwen25_14b_8layers_b1": "gemv",
    # the same 32 projections for 8 and 64 sequences: the tensor-core skinny GEMM
    "gemv_qwen25_14b_8layers_b8": "gemv",
    "gemv_qwen25_14b_8layers_b64": "gemv",
    # one step = one 512-token chunk appended to each of 128 sequences (Mistral-7B shape): every
    # sequence ages out four key groups
    "writer_mistral7b_b128_chunk512": "writer",
}
DEFAULT_WORKLOAD = "mistral7b_decode_attn_b128_t8192"
# the whole decode step of the generated runtime around the KIVI cache (Qwen2.5-14B shape, 48 layers,
# random-init fp16 weights, context 32768). With --gpus N the model is split over N ranks by KV heads
# (strong scaling) with an all-reduce after o_proj and down_proj.
STEP_WORKLOADS = {
    # name: (batch, context)
    "qwen25_14b_decode_step_b1_t32768": (1, 32768),
    "qwen25_14b_decode_step_b8_t32768": (8, 32768),
    "qwen25_14b_decode_step_b32_t32768": (32, 32768),
    "qwen25_14b_decode_step_b64_t32768": (64, 32768),   # needs >= 2 GPUs: 132 GB of KV pages + 29.5 GB of weights
}
METRIC = "KIVI decode-attn achieved HBM GB/s"


def _peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def _dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# ------------------------------------------------------------------------------------------------
# synthetic cache, built on the device with the library's writer

def build_cache(case, batch, context, device, spare_tokens=0, seed=20261125):
    import torch
    from jacq_b200.cache import KiviCache
    from tests import helpers
    lay = helpers.layout_of(case)
    pages = lay.old_pages(context + spare_tokens) + 1
    cache = KiviCache(lay, batch * pages, batch, pages, device)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    cache.set_block_tables(torch.randperm(batch * pages, device=device, generator=gen).to(torch.int32)
                           .reshape(batch, pages))
    outl = torch.from_numpy(helpers.outlier_channels(case, seed)).to(device)      # [NKV, n]
    kscale = torch.ones((case.nkv, case.d), device=device, dtype=torch.float16)
    kscale.scatter_(1, outl.long(), 10.0)
    chunk, write_ms, write_bytes = 512, [], 0
    for start in range(0, context, chunk):
        n = min(chunk, context - start)
        k = torch.randn((batch * n, case.nkv, case.d), device=device, dtype=torch.float16, generator=gen) * kscale
        v = torch.randn((batch * n, case.nkv, case.d), device=device, dtype=torch.float16, generator=gen)
        offs = torch.arange(batch + 1, device=device, dtype=torch.int32) * n
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        cache.write(k, v, offs, max_new_per_seq=n, max_start_seq_len=start)
        e1.record()
        torch.cuda.synchronize(device)
        write_ms.append(e0.elapsed_time(e1))
        write_bytes = k.numel() * 2 * 2
    q = torch.randn((batch, case.nh, case.d), device=device, dtype=torch.float16, generator=gen)
    writer = {"ms_per_512_token_chunk": statistics.median(write_ms),
              "input_gbs": write_bytes / statistics.median(write_ms) / 1e6}
    return cache, q, writer


def sample_to_oracle(cache, case, seqs):
    """Host copy (OracleCache) of the chosen sequences, pages renumbered densely."""
    from tests.gpu_utils import oracle_copy
    return oracle_copy(cache, case, seqs)


def cpu_baseline(cache, q, case, context, nthreads, target_seconds=12.0):
    """Time the CPU oracle on a bounded sample of the workload; also checks the GPU output."""
    from oracle import kivi_oracle as ko
    from tests import helpers
    lay = helpers.layout_of(case)
    batch = q.shape[0]
    n = min(batch, 2)
    oc, tables = sample_to_oracle(cache, case, list(range(n)))
    qh = helpers.to_bits(q[:n])
    lens = np.full(n, context, np.int32)
    t0 = time.perf_counter()
    ko.decode_batch(oc, qh, tables, lens, mode=0, nthreads=nthreads)
    probe = time.perf_counter() - t0
    n = int(max(1, min(batch, round(n * target_seconds / max(probe, 1e-6)))))
    n = max(n, min(batch, nthreads // max(1, case.nh) + 1))
    oc, tables = sample_to_oracle(cache, case, list(range(n)))
    qh = helpers.to_bits(q[:n])
    lens = np.full(n, context, np.int32)
    t0 = time.perf_counter()
    want = ko.decode_batch(oc, qh, tables, lens, mode=0, nthreads=nthreads)
    secs = time.perf_counter() - t0
    sample_bytes = lay.decode_algorithmic_bytes(context) * n
    return {"value": sample_bytes / secs / 1e9, "unit": "GB/s", "cores": nthreads, "kind": "port",
            "sample": f"{n} of {batch} sequences of the workload, all heads, {secs:.1f} s",
            "tokens_per_s": n / secs}, want, n


# ------------------------------------------------------------------------------------------------
# clocks

_POLLER = r"""
import sys, time
idx = int(sys.argv[1])
sys.stdout = open(sys.argv[2], "w")
try:
    import pynvml as n
    n.nvmlInit()
    h = n.nvmlDeviceGetHandleByIndex(idx)
    mx = n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM)
    bits = {"hw_slowdown": n.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": n.nvmlClocksEventReasonHwThermalSlowdown,
            "sw_thermal_slowdown": n.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": n.nvmlClocksEventReasonSwPowerCap,
            "hw_power_brake_slowdown": n.nvmlClocksEventReasonHwPowerBrakeSlowdown}
    print("nvml", mx, " ".join(f"{k}={v}" for k, v in bits.items()), flush=True)
    k, power = 0, 0.0
    while True:
        if k % 16 == 0:
            power = n.nvmlDeviceGetPowerUsage(h) / 1000.0
        print(f"{time.time():.6f} {n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)} {power:.1f} {n.nvmlDeviceGetCurrentClocksEventReasons(h)}")
        k += 1
        if k % 64 == 0:
            sys.stdout.flush()
        time.sleep(0.0002)
except Exception as exc:
    print("error", exc, flush=True)
"""


class ClockSampler:
    """SM clock, power and throttle reasons of one GPU, read through NVML (reading only; nothing is set) by a
    child process a few thousand times a second for as long as the benchmark runs; every sample carries the host
    clock, and a timed region asks for the samples that fall inside it. A separate process, because a polling
    thread would contend with the launching thread for the interpreter lock; a few milliseconds of timed region
    still get several samples, which `nvidia-smi -lms` (100 ms at best) would not give."""

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc, self.lines, self.path = None, None, None

    def start(self):
        import tempfile
        try:
            fd, self.path = tempfile.mkstemp(prefix="kivi_clocks_", suffix=".txt")
            os.close(fd)
            self.proc = subprocess.Popen([sys.executable, "-c", _POLLER, str(self.gpu_index), self.path],
                                         stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
            time.sleep(0.5)   # NVML is up and polling before anything is timed
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            self.lines = []
            return
        time.sleep(0.02)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            self.proc.wait()
        try:
            with open(self.path) as fh:
                self.lines = fh.read().splitlines()
            os.unlink(self.path)
        except OSError:
            self.lines = []
        self.proc = None

    def window(self, t0, t1):
        """Statistics of the samples taken between host times t0 and t1 (call after stop())."""
        if not self.lines or not self.lines[0].startswith("nvml"):
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["NVML unavailable: " + (self.lines[0] if self.lines else "no output")]}
        head = self.lines[0].split()
        sm_max = int(head[1])
        names = dict((kv.split("=")[0], int(kv.split("=")[1])) for kv in head[2:])
        sm, power, bits = [], [], 0
        for line in self.lines[1:]:
            parts = line.split()
            if len(parts) != 4:
                continue
            t = float(parts[0])
            if t0 <= t <= t1:
                sm.append(int(parts[1]))
                power.append(float(parts[2]))
                bits |= int(parts[3])
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": sm_max, "samples": 0, "reasons": ["no sample inside the region"]}
        return {"sm_mhz": statistics.median(sm), "sm_min_mhz": min(sm), "sm_max_mhz": sm_max, "power_w_max": max(power),
                "samples": len(sm), "source": "NVML polled by a child process, samples inside the timed region (host clock)",
                "reasons": [name for name, bit in names.items() if bits & bit]}


# ------------------------------------------------------------------------------------------------

def _max_over_ranks(value, device, world):
    import torch
    import torch.distributed as dist
    if world == 1:
        return float(value)
    t = torch.tensor([float(value)], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_decode(cache, q, out, context, steps, warmup, device, rank, world, local_rank):
    """W warm-up launches, then exactly K timed decode launches between a barrier + synchronize on both sides;
    CUDA events on the launching stream (one pair around the K steps, one event after every step). Returns
    (ms of the K steps on this rank, per-step ms, host-clock window of the timed region)."""
    import torch
    import torch.distributed as dist
    for _ in range(max(3, warmup)):
        cache.decode(q, out, max_seq_len=context)
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    t0 = time.time()
    marks[0].record()
    for k in range(steps):
        cache.decode(q, out, max_seq_len=context)
        marks[k + 1].record()
    torch.cuda.synchronize(device)
    t1 = time.time()
    if world > 1:
        dist.barrier()
    per_step = [marks[k].elapsed_time(marks[k + 1]) for k in range(steps)]
    return marks[0].elapsed_time(marks[steps]), per_step, (t0, t1)


def sustained_decode(cache, q, out, context, device, local_rank, seconds=1.0):
    """The same launch back to back for about a second: what the kernel sustains once the GPU sits at its power
    limit (the SM clock drops), reported beside the K-step figure; returns the mean of the last 40 launches and
    the host-clock window of the second half of the run."""
    import torch
    start = time.time()
    t0, ms = time.perf_counter(), []
    while time.perf_counter() - t0 < seconds:
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(41)]
        marks[0].record()
        for k in range(40):
            cache.decode(q, out, max_seq_len=context)
            marks[k + 1].record()
        torch.cuda.synchronize(device)
        ms = [marks[k].elapsed_time(marks[k + 1]) for k in range(40)]
    end = time.time()
    return statistics.mean(ms), ((start + end) / 2, end)


def run_b200(args):
    import torch
    import torch.distributed as dist
    from tests import helpers
    from jacq_b200 import _native
    _native.lib()   # fail loudly when the CUDA library is missing: there is no other path

    rank, local_rank, world = _dist_env()
    if world > 1:
        # the tensor-parallel part below runs its own peer-memory kernels beside NCCL: keep NVLink multicast out of it
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        import datetime
        # a rank that fails must not leave the others waiting for ten minutes: collectives give up after three
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"), timeout=datetime.timedelta(seconds=180))
    device = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(device)

    key, batch, context = WORKLOADS[args.workload]
    case = helpers.CONFIGS[key]
    lay = helpers.layout_of(case)
    e2e_steps = e2e_step_count(args)
    warm = max(3, args.warmup)
    cache, q, writer = build_cache(case, batch, context, device, spare_tokens=e2e_steps + warm + 8,
                                   seed=20261125 + rank)
    out = torch.empty((batch, case.nh, case.d), dtype=torch.float32, device=device)
    step_bytes = lay.decode_algorithmic_bytes(context) * batch

    if args.profile_only:
        # a handful of launches and nothing else: the command line ncu wraps
        for _ in range(args.warmup + args.steps):
            cache.decode(q, out, max_seq_len=context)
        torch.cuda.synchronize(device)
        print(json.dumps({"profile_only": True, "workload": args.workload, "launches": args.warmup + args.steps,
                          "algorithmic_bytes_per_launch": step_bytes}))
        return

    # ---- kernel-resident measurement: `value` and `roofline` --------------------------------
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    total_ms, per_step_ms, timed_window = time_decode(cache, q, out, context, args.steps, args.warmup, device, rank, world,
                                                      local_rank)
    total_ms = _max_over_ranks(total_ms, device, world)
    ms_per_step = total_ms / args.steps
    value = step_bytes * world / (ms_per_step * 1e-3) / 1e9
    plan = (ctypes_plan(cache, batch, context))
    sustained = None
    clocks = None
    if rank == 0 and world == 1:
        sus_ms, sus_window = sustained_decode(cache, q, out, context, device, local_rank)
        sustained = {"value": step_bytes / (sus_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": sus_ms,
                     "what": "the same launch back to back for 1 s (power-limited steady state); clocks over its second half"}
    if sampler:
        sampler.stop()
        clocks = sampler.window(*timed_window)
        if sustained is not None:
            sustained["clocks"] = sampler.window(*sus_window)

    # ---- end to end through the public API with host buffers ---------------------------------
    # Before the CPU leg, which copies gigabytes of pages to the host and keeps all cores busy for half a minute:
    # measured after it the step's copies and launches ran up to a third slower. The step appends tokens, so the
    # residual rows and the lengths are put back afterwards: the CPU leg and the parity check read the cache the
    # timed launches read.
    keep = [t.clone() for t in (cache.tensors.K_RESIDUAL_SCRATCH, cache.tensors.V_RESIDUAL_SCRATCH, cache.seq_lens)]
    e2e = measure_e2e(args, cache, q, case, lay, batch, context, device, rank, world, warm)
    for dst, src in zip((cache.tensors.K_RESIDUAL_SCRATCH, cache.tensors.V_RESIDUAL_SCRATCH, cache.seq_lens), keep):
        dst.copy_(src)
    del keep
    torch.cuda.synchronize(device)

    # ---- CPU baseline on a bounded sample (rank 0, one GPU only); doubles as a parity check ------
    base, parity = None, None
    if args.cpu_baseline and rank == 0:
        nthreads = os.cpu_count() or 1
        base, want, n = cpu_baseline(cache, q, case, context, nthreads)
        got = out[:n].cpu().numpy()
        err = float(np.abs(got - want).max())
        parity = {"sequences": n, "max_abs_err": err, "within_1e-2": bool((np.abs(got - want) <= 1e-2 + 1e-2 * np.abs(want)).all())}
        single = cpu_baseline(cache, q, case, context, 1, target_seconds=6.0)[0]
        base["single_thread"] = {"value": single["value"], "unit": "GB/s", "sample": single["sample"]}

    strong = tp = secondary = None
    if world > 1:
        strong = measure_strong_scaling(args, cache, q, out, case, lay, batch, context, device, rank, world, local_rank)
    del cache, q, out
    torch.cuda.empty_cache()
    if world > 1 and args.extras:
        tp = measure_tp_step(args, device, rank, local_rank, world)
    if world == 1 and args.extras:
        secondary = measure_secondary(args, device)

    if rank == 0:
        peak, peak_kind = _peaks()
        kernel_ms = statistics.mean(per_step_ms)
        achieved = step_bytes / (kernel_ms * 1e-3) / 1e9
        # DRAM bytes per launch: one ncu capture of this kernel on 48 sequences of the same shape read 447.02 MB and
        # wrote 3.91 MB against 447.58 MB of algorithmic bytes; traffic grows with the sequences, so that ratio is
        # applied to this launch
        traffic, traffic_source = None, None
        if key == "mistral7b" and context == 8192:
            traffic = step_bytes * TRAFFIC_RATIO_B48
            traffic_source = "ncu dram__bytes_read+write of a 48-sequence launch, scaled by sequences"
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u4 codes, f16 params/residual, f32 accumulate", "data": "synthetic",
            "config": {"workload": args.workload, "geometry": {"nh": case.nh, "nkv": case.nkv, "head_dim": case.d,
                                                                "block": case.b, "group": case.g, "residual": case.r},
                       "batch_per_gpu": batch, "context": context, "algorithmic_bytes_per_step_per_gpu": step_bytes,
                       "l2": "inputs (1.49 GB of pages per GPU) exceed the 126 MB L2; no flush between iterations",
                       "timing": "W warm-up launches, then K launches timed once with CUDA events between barriers; "
                                 "`sustained` repeats the launch for a second",
                       "launch_plan": plan,
                       "parallelism": f"sequences sharded over {world} GPU(s), no collective"},
            "tokens_per_s": batch * world / (ms_per_step * 1e-3),
            "pct_of_8TBs_nominal": 100.0 * value / world / 8000.0,
            "e2e": e2e,
            "gpu_launches": args.steps * (2 if plan["cut_units"] else 1),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "traffic_source": traffic_source, "peak_source": f"{peak_kind} HBM copy bandwidth",
                         "kernel": "decode_mma_kernel", "ms_per_launch": kernel_ms},
            "sustained": sustained,
            "writer": writer,
            "cpu_baseline": base,
            "parity_vs_cpu_port": parity,
        }
        if strong is not None:
            line["strong"] = strong
        if tp is not None:
            line["tp_step"] = tp
        if secondary is not None:
            line["secondary"] = secondary
        print(json.dumps(line))
        sys.stdout.flush()
    if world > 1:
        # no destroy_process_group(): with NCCL collectives inside a captured graph it can block for minutes
        try:
            dist.barrier()
            torch.cuda.synchronize(device)
        except Exception:   # noqa: BLE001 - the line is out; a rank that failed earlier must not turn the exit into a hang
            pass
        sys.stdout.flush()
        os._exit(0)


# DRAM bytes over algorithmic bytes of decode_mma_kernel, from the ncu capture of the 48-sequence case
TRAFFIC_RATIO_B48 = (447.02 + 3.91) / 447.58


def e2e_step_count(args):
    """Steps of the end-to-end measurement: at least 100. A step is 0.3 ms of host and device work with a
    synchronize in it, and over 20 of them one scheduling hiccup of the host moved the result by 15 %."""
    return max(args.steps, 100)


def ctypes_plan(cache, batch, context):
    """The launch plan the library reports for this batch (kivi_b200_decode_plan)."""
    import ctypes
    from jacq_b200 import _native
    out = (ctypes.c_int32 * 4)()
    _native.check(_native.lib().kivi_b200_decode_plan(ctypes.byref(cache._geom), batch, context, out), "kivi_b200_decode_plan")
    u1, k1, u2, k2 = (int(v) for v in out)
    return {"whole_units": u1 if k1 == 1 else 0, "units_cut": [[u1, k1]] * (k1 > 1) + [[u2, k2]] * (k2 > 1),
            "cut_units": (u1 if k1 > 1 else 0) + (u2 if k2 > 1 else 0), "jobs": u1 * k1 + u2 * k2}


def measure_e2e(args, cache, q, case, lay, batch, context, device, rank, world, warm):
    """One serving step through the public API (KiviCache.write / .decode) with HOST buffers, every step: pinned q,
    the step's new K/V rows and the sequence lengths (host-side metadata, as a serving engine keeps them) copied
    host->device, cache write of one token per sequence, decode with fp16 output, output copied device->host.
    The step is captured once as a CUDA graph and launched once per step (--no-e2e-graph: separate calls); the
    last output is checked against a separate decode of the same cache state."""
    import torch
    import torch.distributed as dist
    e2e_steps = e2e_step_count(args)
    out16 = torch.empty((batch, case.nh, case.d), dtype=torch.float16, device=device)
    # One pinned staging buffer for everything a step sends to the device -- q, the new K and V rows, the
    # sequence lengths before and after the write -- and one device buffer of the same layout: one H2D copy per step.
    nq, nkv_rows = batch * case.nh * case.d, batch * case.nkv * case.d
    halves = nq + 2 * nkv_rows
    stage_bytes = halves * 2 + 2 * batch * 4
    stage_host = torch.empty(stage_bytes, dtype=torch.uint8).pin_memory()
    stage_dev = torch.empty(stage_bytes, dtype=torch.uint8, device=device)

    def views(buf):
        h = buf[: halves * 2].view(torch.float16)
        lens = buf[halves * 2:].view(torch.int32).view(2, batch)      # row 0: before the write, row 1: after
        return (h[:nq].view(batch, case.nh, case.d), h[nq: nq + nkv_rows].view(batch, case.nkv, case.d),
                h[nq + nkv_rows:].view(batch, case.nkv, case.d), lens)

    q_host, nk_host, nv_host, lens_host = views(stage_host)
    q_dev, nk_dev, nv_dev, lens_dev = views(stage_dev)
    out_host = torch.empty(out16.shape, dtype=out16.dtype).pin_memory()
    gen = torch.Generator().manual_seed(7 + rank)
    q_host.copy_(q.cpu())
    nk_host.copy_(torch.randn((batch, case.nkv, case.d), generator=gen).to(torch.float16))
    nv_host.copy_(torch.randn((batch, case.nkv, case.d), generator=gen).to(torch.float16))
    offs = torch.arange(batch + 1, device=device, dtype=torch.int32)
    state = {"len": context}
    # the bounds the launch plan needs are those of the last step of the run
    bound = context + e2e_steps + warm + 4

    def enqueue_step():
        stage_dev.copy_(stage_host, non_blocking=True)
        cache.write(nk_dev, nv_dev, offs, max_new_per_seq=1, max_start_seq_len=bound, start_seq_lens=lens_dev[0], advance=False)
        cache.decode(q_dev, out16, max_seq_len=bound + 1, seq_lens=lens_dev[1])
        out_host.copy_(out16, non_blocking=True)

    lens_np = lens_host.numpy()   # the same pinned bytes: a plain store instead of two tensor operations per step

    def set_lens():
        lens_np[0, :] = state["len"]
        lens_np[1, :] = state["len"] + 1

    set_lens()
    enqueue_step()   # once eagerly: every buffer the calls allocate lazily exists before a capture
    torch.cuda.synchronize(device)
    state["len"] += 1
    graph = None
    if args.e2e_graph:
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):   # other threads (NCCL's watchdog) may call CUDA
                enqueue_step()
            graph = g
        except Exception as exc:   # noqa: BLE001 - the eager path below measures the same step
            print(f"bench: graph capture of the serving step failed ({exc}); timing the eager calls", file=sys.stderr)
            torch.cuda.synchronize(device)

    def serving_step():
        set_lens()
        if graph is not None:
            graph.replay()
        else:
            enqueue_step()
        torch.cuda.synchronize(device)
        state["len"] += 1

    for _ in range(warm):
        serving_step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    e2e_bytes = 0
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        serving_step()
        e2e_bytes += lay.decode_algorithmic_bytes(state["len"]) * batch
    e2e_s = time.perf_counter() - t0
    # what the last replay copied out is what a separate decode call computes from the same cache state
    cache.seq_lens.fill_(state["len"])
    check = torch.empty_like(out16)
    cache.decode(q_dev, check, max_seq_len=bound + 1)
    torch.cuda.synchronize(device)
    if not torch.equal(check.cpu(), out_host):
        raise RuntimeError("bench: the end-to-end step's output differs from a decode of the same cache state")
    e2e_s = _max_over_ranks(e2e_s, device, world)
    h2d = stage_bytes
    d2h = out_host.numel() * 2
    return {"value": e2e_bytes * world / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "ms_per_step": e2e_s / e2e_steps * 1e3, "tokens_per_s": batch * world / (e2e_s / e2e_steps), "steps": e2e_steps,
            "what": "one pinned staging buffer (q, new K/V rows, sequence lengths) H2D, cache write (1 token/sequence), decode (fp16 out), O D2H"
                    + ("; one CUDA graph launch per step" if graph is not None else "; eager calls")}


def measure_strong_scaling(args, cache, q, out, case, lay, batch, context, device, rank, world, local_rank):
    """Strong scaling of the same workload: the `batch` sequences of ONE GPU's workload split over the ranks
    (contiguous shares of equal size; jacq_b200.sharding does the byte-balanced split for ragged batches), each
    rank decoding its share of its own cache. value = bytes of the whole batch / slowest rank's time."""
    from jacq_b200 import sharding
    n = len(sharding.contiguous_shards(batch, world)[rank])
    total_ms, per_step, _ = time_decode(cache, q[:n], out[:n], context, args.steps, args.warmup, device, rank, world,
                                        local_rank)
    total_ms = _max_over_ranks(total_ms, device, world)
    ms = total_ms / args.steps
    value = lay.decode_algorithmic_bytes(context) * batch / (ms * 1e-3) / 1e9
    return {"value": value, "unit": "GB/s", "ms_per_step": ms, "sequences_total": batch, "sequences_per_gpu": n,
            "tokens_per_s": batch / (ms * 1e-3), "launch_plan": ctypes_plan(cache, n, context),
            "what": f"{batch} sequences x {context} tokens in total, split over {world} GPUs; no collective"}


def _timed_steps(fn, steps, warmup, device):
    """W warm-up steps, then K steps enqueued back to back and timed once (an event after every step, one
    synchronize at the end), so that the host's launch latency is not part of a step; per-step ms."""
    import torch
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize(device)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    marks[0].record()
    for k in range(steps):
        fn()
        marks[k + 1].record()
    torch.cuda.synchronize(device)
    return [marks[k].elapsed_time(marks[k + 1]) for k in range(steps)]


def measure_gemv(gbatch, steps, warmup, device):
    """One step = the four projections (qkv, o, gate_up, down) of 8 layers of the Qwen2.5-14B shape for `gbatch`
    sequences, every GEMV on its own weights: 4.4 GB of fp16 weights streamed once per step."""
    import ctypes
    import torch
    from jacq_b200 import _native
    peak, peak_kind = _peaks()
    hidden, ffn, qkv = 5120, 13824, 7168
    shapes = [(qkv, hidden), (hidden, hidden), (2 * ffn, hidden), (hidden, ffn)]
    layers = 8
    gen = torch.Generator(device=device).manual_seed(11)
    weights = [[(torch.randn((o, i), device=device, dtype=torch.float16, generator=gen) * 0.02) for o, i in shapes]
               for _ in range(layers)]
    xs = {i: torch.randn((gbatch, i), device=device, dtype=torch.float16, generator=gen) for i in (hidden, ffn)}
    ys = [[torch.empty((gbatch, o), device=device, dtype=torch.float16) for o, _ in shapes] for _ in range(layers)]
    lib = _native.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)

    def step():
        for lw, ly in zip(weights, ys):
            for w, y in zip(lw, ly):
                rc = lib.kivi_b200_gemv_f16(w.data_ptr(), xs[w.shape[1]].data_ptr(), y.data_ptr(), None,
                                            w.shape[0], w.shape[1], gbatch, stream)
                assert rc == 0
    step_bytes = layers * sum(o * i * 2 + gbatch * (o + i) * 2 for o, i in shapes)
    ms = statistics.mean(_timed_steps(step, steps, warmup, device))
    value = step_bytes / (ms * 1e-3) / 1e9
    kernel = "gemv_kernel" if gbatch <= 4 else "umma_tma_gemm_kernel (tcgen05)"
    return {"metric": "fp16 GEMV achieved HBM GB/s", "value": value, "unit": "GB/s", "ms_per_step": ms,
            "config": {"workload": f"gemv_qwen25_14b_8layers_b{gbatch}", "algorithmic_bytes_per_step": step_bytes,
                       "shapes_out_in": shapes, "layers": layers, "batch": gbatch, "l2": "working set exceeds the 126 MB L2"},
            "gpu_launches": layers * len(shapes) * steps,
            "roofline": {"bound": "hbm", "achieved": value, "peak": peak, "unit": "GB/s", "frac": value / peak,
                         "traffic": None, "peak_source": f"{peak_kind} HBM copy bandwidth", "kernel": kernel}}


def measure_writer(steps, warmup, device):
    """One step = one 512-token chunk appended to each of 128 sequences (Mistral-7B shape): every sequence ages
    out four key groups."""
    import torch
    from tests import helpers
    from jacq_b200.cache import KiviCache
    peak, peak_kind = _peaks()
    case = helpers.CONFIGS["mistral7b"]
    lay = helpers.layout_of(case)
    batch, chunk, start = 128, 512, 512
    pages = lay.old_pages(start + chunk * (steps + max(3, warmup) + 1)) + 1
    cache = KiviCache(lay, batch * pages, batch, pages, device)
    gen = torch.Generator(device=device).manual_seed(5)
    cache.set_block_tables(torch.randperm(batch * pages, device=device, generator=gen).to(torch.int32)
                           .reshape(batch, pages))
    k = torch.randn((batch * chunk, case.nkv, case.d), device=device, dtype=torch.float16, generator=gen)
    v = torch.randn((batch * chunk, case.nkv, case.d), device=device, dtype=torch.float16, generator=gen)
    offs = torch.arange(batch + 1, device=device, dtype=torch.int32) * chunk
    state = {"len": 0}

    def step():
        cache.write(k, v, offs, max_new_per_seq=chunk, max_start_seq_len=state["len"])
        state["len"] += chunk
    step()   # from empty: afterwards every step ages out exactly chunk / group groups per sequence
    g, d, nkv, r, hg = case.g, case.d, case.nkv, case.r, lay.hd_groups
    groups = chunk // g
    per_head = (2 * chunk * d * 2                      # new K and V rows read (by the pack or the append)
                + groups * (g * d + (g // case.b) * d * 4 + g * hg * 4)   # codes, key params per page, value params
                + 2 * 2 * r * d * 2)                   # rows that stay fp16: read once, written once, K and V
    step_bytes = batch * nkv * per_head
    ms = statistics.mean(_timed_steps(step, steps, warmup, device))
    value = step_bytes / (ms * 1e-3) / 1e9
    return {"metric": "KIVI cache-writer achieved HBM GB/s", "value": value, "unit": "GB/s", "ms_per_step": ms,
            "config": {"workload": "writer_mistral7b_b128_chunk512", "algorithmic_bytes_per_step": step_bytes, "batch": batch,
                       "chunk_tokens": chunk, "tokens_per_s": batch * chunk / (ms * 1e-3),
                       "l2": "working set exceeds the 126 MB L2"},
            "gpu_launches": steps,
            "roofline": {"bound": "hbm", "achieved": value, "peak": peak, "unit": "GB/s", "frac": value / peak,
                         "traffic": None, "peak_source": f"{peak_kind} HBM copy bandwidth",
                         "kernel": "pack_groups_kernel (packs the aged-out groups and updates the scratch rows)"}}


def measure_decode_config(name, steps, warmup, device):
    """Decode attention at one of the other attention-only configurations: K timed launches, CUDA events."""
    import torch
    from tests import helpers
    peak, peak_kind = _peaks()
    key, batch, context = WORKLOADS[name]
    case = helpers.CONFIGS[key]
    lay = helpers.layout_of(case)
    cache, q, _ = build_cache(case, batch, context, device)
    out = torch.empty((batch, case.nh, case.d), dtype=torch.float32, device=device)
    step_bytes = lay.decode_algorithmic_bytes(context) * batch
    # The page pools of these configurations fit in the L2: evict them between launches by writing a larger buffer.
    # The fill is also long enough (512 MB, > 100 us) for the host to have enqueued the timed launch before it ends,
    # so that the events bracket the launch on the device and not the host's call overhead.
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=device) if cache.bytes_allocated() < (160 << 20) else None
    for _ in range(max(3, warmup)):
        cache.decode(q, out, max_seq_len=context)
    torch.cuda.synchronize(device)
    ms = []
    for _ in range(steps):
        if flush is not None:
            flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        cache.decode(q, out, max_seq_len=context)
        e1.record()
        torch.cuda.synchronize(device)
        ms.append(e0.elapsed_time(e1))
    med = statistics.median(ms)
    value = step_bytes / (med * 1e-3) / 1e9
    return {"metric": METRIC, "value": value, "unit": "GB/s", "ms_per_step": med, "tokens_per_s": batch / (med * 1e-3),
            "config": {"workload": name, "batch": batch, "context": context, "algorithmic_bytes_per_step": step_bytes,
                       "launch_plan": ctypes_plan(cache, batch, context),
                       "l2": "L2 evicted before every launch (512 MB written; the launch is enqueued behind that fill)" if flush is not None else "inputs exceed the L2"},
            "roofline": {"bound": "hbm (launch-latency bound at this size)" if step_bytes < (100 << 20) else "hbm",
                         "achieved": value, "peak": peak, "unit": "GB/s", "frac": value / peak,
                         "peak_source": f"{peak_kind} HBM copy bandwidth", "kernel": "decode_mma_kernel"}}


def measure_ragged(steps, warmup, device):
    """The ragged stress shape as a throughput case: 256 sequences whose lengths are drawn uniformly from 1..32768
    (32 query / 8 kv heads, head size 128, page 16, group 128), fully shuffled block tables, the cache built by
    interleaved 512-token chunk writes (a sequence drops out of the batch when it is full). One step = one decode
    launch over all 256 sequences; bytes = the sum of every sequence's own algorithmic bytes."""
    import torch
    from tests import helpers
    from jacq_b200.cache import KiviCache
    peak, peak_kind = _peaks()
    case = helpers.CONFIGS["mistral7b"]
    lay = helpers.layout_of(case)
    batch, longest, chunk = 256, 32768, 512
    rng = np.random.default_rng(20261125)
    lens = rng.integers(1, longest + 1, size=batch).astype(np.int64)
    pages = lay.old_pages(longest) + 1
    cache = KiviCache(lay, batch * pages, batch, pages, device)
    gen = torch.Generator(device=device).manual_seed(9)
    cache.set_block_tables(torch.randperm(batch * pages, device=device, generator=gen).to(torch.int32)
                           .reshape(batch, pages))
    # all chunks' rows first (16 GB), then the 64 write calls back to back between two events: the host stays
    # ahead of the device, so the time is the writer's and not the call overhead's
    written, calls = 0, []
    for start in range(0, longest, chunk):
        counts = np.clip(lens - start, 0, chunk)
        total = int(counts.sum())
        if total == 0:
            break
        k = torch.randn((total, case.nkv, case.d), device=device, dtype=torch.float16, generator=gen)
        v = torch.randn((total, case.nkv, case.d), device=device, dtype=torch.float16, generator=gen)
        offs = torch.from_numpy(np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)).to(device)
        calls.append((k, v, offs, start))
        written += total
    # the writer's kernels are loaded by a first call elsewhere (a 2-sequence cache of the same geometry): the first
    # launch of a kernel in a process costs milliseconds of module loading
    small = KiviCache(lay, 2 * (2 * chunk // case.b + 1), 2, 2 * chunk // case.b + 1, device)
    small.set_block_tables(torch.arange(2 * (2 * chunk // case.b + 1), device=device, dtype=torch.int32).reshape(2, -1))
    for first in (0, chunk):
        small.write(calls[0][0][: 2 * chunk], calls[0][1][: 2 * chunk],
                    torch.tensor([0, chunk, 2 * chunk], device=device, dtype=torch.int32), max_new_per_seq=chunk,
                    max_start_seq_len=first)
    del small
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for k, v, offs, start in calls:
        cache.write(k, v, offs, max_new_per_seq=chunk, max_start_seq_len=start)
    e1.record()
    torch.cuda.synchronize(device)
    write_ms = e0.elapsed_time(e1)
    ncalls = len(calls)
    del calls, k, v
    torch.cuda.empty_cache()
    if cache.seq_lens.cpu().numpy().tolist() != lens.tolist():
        raise RuntimeError("bench: the ragged cache's lengths differ from the lengths written")
    q = torch.randn((batch, case.nh, case.d), device=device, dtype=torch.float16, generator=gen)
    out = torch.empty((batch, case.nh, case.d), dtype=torch.float32, device=device)
    step_bytes = int(sum(lay.decode_algorithmic_bytes(int(t)) for t in lens))

    def step():
        cache.decode(q, out, max_seq_len=longest)
    ms = statistics.mean(_timed_steps(step, steps, warmup, device))
    if not bool(torch.isfinite(out).all()):
        raise RuntimeError("bench: the ragged decode produced a non-finite output")
    value = step_bytes / (ms * 1e-3) / 1e9
    return {"metric": METRIC, "value": value, "unit": "GB/s", "ms_per_step": ms, "tokens_per_s": batch / (ms * 1e-3),
            "config": {"workload": "ragged_decode_attn_b256_t1_32768", "batch": batch, "context": "uniform 1..32768",
                       "context_tokens_total": int(lens.sum()), "algorithmic_bytes_per_step": step_bytes,
                       "launch_plan": ctypes_plan(cache, batch, longest),
                       "cache_build": {"tokens": written, "write_calls": ncalls, "ms": write_ms,
                                       "tokens_per_s": written / (write_ms * 1e-3),
                                       "new_rows_gbs": written * case.nkv * case.d * 4 / (write_ms * 1e-3) / 1e9,
                                       "what": "interleaved ragged 512-token chunk writes, all calls back to back "
                                               "between two events; GB/s of the new K and V rows alone"},
                       "l2": "inputs exceed the L2"},
            "gpu_launches": steps,
            "roofline": {"bound": "hbm", "achieved": value, "peak": peak, "unit": "GB/s", "frac": value / peak,
                         "peak_source": f"{peak_kind} HBM copy bandwidth", "kernel": "decode_mma_kernel"}}


def measure_secondary(args, device):
    """The other parts of the path, each against its own HBM roofline (one GPU): the cache writer, the GEMV /
    skinny GEMM of the generated runtime, the whole decode step at batch 1, and the two small attention-only
    configurations. A part that fails is reported as such and does not take the headline down with it."""
    import torch
    out = {}
    jobs = [("writer", lambda: measure_writer(args.steps, args.warmup, device)),
            ("gemv_b1", lambda: measure_gemv(1, args.steps, args.warmup, device)),
            ("gemv_b8", lambda: measure_gemv(8, args.steps, args.warmup, device)),
            ("gemv_b64", lambda: measure_gemv(64, args.steps, args.warmup, device)),
            ("decode_attn_tinyllama_b4_t512", lambda: measure_decode_config("tinyllama_decode_attn_b4_t512", args.steps, args.warmup, device)),
            ("decode_attn_qwen05b_b64_t4096", lambda: measure_decode_config("qwen05b_decode_attn_b64_t4096", args.steps, args.warmup, device)),
            ("decode_attn_ragged_b256_t1_32768", lambda: measure_ragged(args.steps, args.warmup, device)),
            ("decode_step_qwen25_14b_b1_t32768", lambda: measure_step(1, 32768, "p2p", min(args.steps, 10), args.warmup, device, 0, 0, 1, None, sample_clocks=False))]
    for name, fn in jobs:
        try:
            out[name] = fn()
        except Exception as exc:   # noqa: BLE001
            out[name] = {"failed": f"{type(exc).__name__}: {exc}"}
        torch.cuda.synchronize(device)
        torch.cuda.empty_cache()
    return out


def run_secondary(args):
    """GEMV and cache-writer workloads on their own: one GPU, value = algorithmic bytes / CUDA-event time."""
    import torch
    from jacq_b200 import _native
    _native.lib()
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    if SECONDARY[args.workload] == "gemv":
        rec = measure_gemv(int(args.workload.rsplit("_b", 1)[1]), args.steps, args.warmup, device)
    else:
        rec = measure_writer(args.steps, args.warmup, device)
    print(json.dumps({**rec, "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "higher_is_better": True,
                      "scaling": "weak", "vs_baseline": None, "dtype": "f16/u4", "data": "synthetic"}))


def step_weights(cfg, device, rank, world):
    """Random-init fp16 weights of the decode-step workloads, this rank's shard (same seed everywhere, so the
    replicated tensors agree)."""
    import torch
    from jacq_b200.runtime import random_layer
    gen = torch.Generator(device=device).manual_seed(1234)

    def mat(rows, cols):
        return (torch.randn((rows, cols), generator=gen, device=device, dtype=torch.float32) * 0.02).half()

    return {"embed": mat(cfg.vocab, cfg.hidden),
            "final_norm": (1.0 + 0.1 * torch.randn((cfg.hidden,), generator=gen, device=device)).half(),
            "lm_head": mat(cfg.vocab // world, cfg.hidden),
            "layers": [random_layer(cfg, gen, device, rank=rank, world=world) for _ in range(cfg.layers)]}, gen


def measure_step(batch, context, comm, steps, warmup, device, rank, local_rank, world, group, weights=None, gen=None,
                 profile_only=False, sample_clocks=True):
    """Whole decode step (Qwen2.5-14B shape) through jacq_b200.runtime.DecodeRuntime.

    value = tokens/s of the whole job (batch / step time, CUDA-graph replay, device-resident token
    ids); roofline = the bytes one rank must stream per step (its weight shard + the KV bytes of its
    heads) / step time against the measured HBM copy bandwidth; e2e = the same step fed from and
    read back into pinned host memory."""
    import torch
    import torch.distributed as dist
    from jacq_b200.runtime import DecodeModelConfig, DecodeRuntime
    cfg = DecodeModelConfig.qwen25_14b()
    warm = max(3, warmup)
    total_steps = warm + 2 * steps + 2          # warm-up, device-timed steps, end-to-end steps
    start = context - total_steps
    if weights is None:
        weights, gen = step_weights(cfg, device, rank, world)
    tables = torch.randperm(batch * (-(-(context - cfg.residual) // cfg.block_size)), generator=gen, device=device)
    rt = DecodeRuntime(cfg, weights, batch=batch, max_seq_len=context, device=device, rank=rank, world=world,
                       group=group, block_tables=tables.to(torch.int32).reshape(batch, -1), comm=comm)
    # synthetic context: fill layer 0 through the library's writer, then give every layer the same pages
    c0 = rt.caches[0]
    c0.set_block_tables(rt.block_tables)
    nkv_l, d = cfg.num_kv_heads // world, cfg.head_dim
    chunk = 2048
    offs = torch.arange(batch + 1, device=device, dtype=torch.int32)
    done = 0
    while done < start:
        n = min(chunk, start - done)
        k = torch.randn((batch * n, nkv_l, d), generator=gen, device=device, dtype=torch.float16)
        k[:, :, :3] *= 10.0                              # a few outlier key channels, as in the attention workloads
        v = torch.randn((batch * n, nkv_l, d), generator=gen, device=device, dtype=torch.float16)
        c0.write(k, v, offs * n, max_new_per_seq=n, max_start_seq_len=done)
        done += n
    del k, v
    for c in rt.caches[1:]:
        for name in c0.tensors.names():
            getattr(c.tensors, name).copy_(getattr(c0.tensors, name))
    rt.set_seq_lens([start] * batch)
    rt.tokens.copy_(torch.arange(batch, dtype=torch.int32) * 997 + 11)
    if world > 1:
        dist.all_reduce(torch.zeros(8, device=device, dtype=torch.float16))   # communicator up before the capture
    torch.cuda.synchronize(device)
    if profile_only:
        # eager steps inside an NVTX range: the command line ncu wraps (--nvtx --nvtx-include "kivi_step/")
        rt.step()
        torch.cuda.synchronize(device)
        torch.cuda.nvtx.range_push("kivi_step")
        for _ in range(steps):
            rt.step()
        torch.cuda.synchronize(device)
        torch.cuda.nvtx.range_pop()
        return {"profile_only": True, "steps": steps, "launches_per_step": cfg.layers * 10 + 6}
    rt.capture()
    for _ in range(warm):
        rt.step()
    torch.cuda.synchronize(device)

    sampler = ClockSampler(local_rank) if (rank == 0 and sample_clocks) else None
    if sampler:
        sampler.start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.time()
    e0.record()
    for _ in range(steps):
        rt.step()
    e1.record()
    torch.cuda.synchronize(device)
    w1 = time.time()
    clocks = None
    if sampler:
        sampler.stop()
        clocks = sampler.window(w0, w1)
    if world > 1:
        dist.barrier()
    ms_per_step = _max_over_ranks(e0.elapsed_time(e1), device, world) / steps

    # end to end: token ids from pinned host memory in, next ids back out, every step
    tok_host = rt.tokens.cpu().pin_memory()
    out_host = torch.empty_like(tok_host).pin_memory()
    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    for _ in range(steps):
        rt.tokens.copy_(tok_host, non_blocking=True)
        rt.step()
        out_host.copy_(rt.tokens, non_blocking=True)
        torch.cuda.synchronize(device)
        tok_host.copy_(out_host)
    e2e_ms = _max_over_ranks((time.perf_counter() - t0) * 1e3 / steps, device, world)
    final_lens = rt.seq_lens.cpu().tolist()
    exchange_ok = rt.exchange_status() == 0
    weight_bytes = cfg.weight_bytes(world)
    kv_bytes = rt.kv_bytes_per_step(context)
    rt.close()
    del rt
    torch.cuda.empty_cache()

    peak, peak_kind = _peaks()
    rank_bytes = weight_bytes + kv_bytes
    achieved = rank_bytes / (ms_per_step * 1e-3) / 1e9
    launches_per_step = cfg.layers * 10 + 6
    return {
        "metric": "decode-step tokens/s", "value": batch / (ms_per_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f16/u4", "data": "synthetic",
        "config": {"workload": f"qwen25_14b_decode_step_b{batch}_t{context}", "model_shape": cfg.name, "layers": cfg.layers,
                   "batch": batch, "context": context, "block": cfg.block_size, "group": cfg.group_size, "residual": cfg.residual,
                   "parallelism": f"tp{world} over kv heads, {comm} exchange" if world > 1 else "1 gpu",
                   "weights": "random-init fp16 N(0, 0.02)", "step": "CUDA-graph replay of kivi_b200_decode_step",
                   "l2": "29.5 GB of weights and the KV pages exceed the 126 MB L2",
                   "final_seq_lens_ok": final_lens == [context - 2] * batch, "exchange_ok": exchange_ok},
        "e2e": {"value": batch / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 4 * batch,
                "d2h_bytes_per_step": 4 * batch, "ms_per_step": e2e_ms},
        "gpu_launches": launches_per_step * (warm + 2 * steps),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": f"{peak_kind} HBM copy bandwidth",
                     "bytes_per_rank_per_step": {"weights": weight_bytes, "kv_cache": kv_bytes},
                     "kernel": "whole step: gemv / skinny GEMM, decode_mma_kernel, writer, element-wise"},
        "cpu_baseline": None,
        "clocks": clocks,
    }


def tp_parity_check(device, rank, world, comm, batch):
    """A short tensor-parallel run of a small model on all ranks, checked against the CPU step oracle (test
    infrastructure, used here as the checker only): 70 steps across the first quantisation boundary, logits of
    this rank's vocabulary slice within rtol = atol = 2e-2 and the exchange's status word clean."""
    import torch
    import torch.distributed as dist
    from oracle import step_oracle as so
    from jacq_b200.runtime import DecodeModelConfig, DecodeRuntime, shard_layer
    s = so.StepShape(layers=2, hidden=512, nh=16, nkv=8, hd=64, ffn=1024, vocab=2048, rope_base=10000.0,
                     norm_eps=1e-5, attn_bias=True, block=16, group=32, residual=32)
    cfg = DecodeModelConfig("parity", s.layers, s.hidden, s.nh, s.nkv, s.hd, s.ffn, s.vocab, rope_base=s.rope_base,
                            norm_eps=s.norm_eps, attn_bias=s.attn_bias, block_size=s.block, group_size=s.group,
                            residual=s.residual)
    w = so.random_weights(s, 21)
    per_seq, steps = 8, 70
    bt = np.random.default_rng(9).permutation(batch * per_seq).reshape(batch, per_seq).astype(np.int32)
    oracle = so.StepOracle(s, w, bt, batch * per_seq, world=world)
    vl = s.vocab // world
    shard = {"embed": torch.from_numpy(w.embed), "final_norm": torch.from_numpy(w.final_norm),
             "lm_head": torch.from_numpy(w.lm_head[rank * vl: (rank + 1) * vl]),
             "layers": [shard_layer(cfg, {k: (None if v is None else torch.from_numpy(v)) for k, v in lw.items()},
                                    rank, world) for lw in w.layers]}
    rt = DecodeRuntime(cfg, shard, batch=batch, max_seq_len=per_seq * s.block + s.residual, device=device, rank=rank,
                       world=world, group=dist.group.WORLD, block_tables=torch.from_numpy(bt), comm=comm)
    tok = (np.arange(batch, dtype=np.int32) * 101 + 4) % s.vocab
    worst, ok = 0.0, True
    for i in range(steps):
        if i == steps // 2:
            rt.capture()
        want_tok, want_logits = oracle.step(tok)
        rt.step(torch.from_numpy(tok))
        got = rt.logits.float().cpu().numpy()
        want = want_logits.astype(np.float32)[:, rank * vl: (rank + 1) * vl]
        err = np.abs(got - want)
        worst = max(worst, float(err.max()))
        ok = ok and bool((err <= 2e-2 + 2e-2 * np.abs(want)).all())
        tok = want_tok.astype(np.int32)
    ok = ok and rt.exchange_status() == 0 and bool((rt.seq_lens.cpu().numpy() == steps).all())
    rt.close()
    flag = torch.tensor([0.0 if ok else 1.0, worst], device=device, dtype=torch.float64)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    return {"comm": comm, "batch": batch, "ranks": world, "steps": steps, "ok": bool(flag[0].item() == 0.0),
            "max_abs_err_logits": float(flag[1].item()), "checked_against": "CPU step oracle, every rank its vocabulary slice"}


def measure_tp_step(args, device, rank, local_rank, world):
    """The one part of the path with an exchange, on the ranks of this run: KV-head tensor parallelism of the
    Qwen2.5-14B-shaped decode step (strong scaling: the model is split, the batch is not), with the library's
    peer-memory exchange and with NCCL hooks, batch 1 and 8, after a parity run of a small model on the same
    ranks. NVLS is off and no multimem instruction is used."""
    import torch
    import torch.distributed as dist
    from jacq_b200.runtime import DecodeModelConfig
    out = {"parity": [], "runs": []}
    try:
        for comm, b in (("p2p", 3), ("p2p", 6), ("nccl", 3)):
            out["parity"].append(tp_parity_check(device, rank, world, comm, b))
        cfg = DecodeModelConfig.qwen25_14b()
        weights, gen = step_weights(cfg, device, rank, world)
        steps = min(args.steps, 10)
        for batch in (1, 8):
            for comm in ("p2p", "nccl"):
                rec = measure_step(batch, 32768, comm, steps, args.warmup, device, rank, local_rank, world, dist.group.WORLD,
                                   weights=weights, gen=gen, sample_clocks=False)
                out["runs"].append({"batch": batch, "comm": comm, "ms_per_step": rec["ms_per_step"], "tokens_per_s": rec["value"],
                                    "e2e_ms_per_step": rec["e2e"]["ms_per_step"], "roofline_frac_of_rank_bytes": rec["roofline"]["frac"],
                                    "bytes_per_rank_per_step": rec["roofline"]["bytes_per_rank_per_step"],
                                    "exchange_ok": rec["config"]["exchange_ok"], "final_seq_lens_ok": rec["config"]["final_seq_lens_ok"]})
    except Exception as exc:   # noqa: BLE001 - report, keep the headline
        out["failed"] = f"{type(exc).__name__}: {exc}"
    out["what"] = (f"Qwen2.5-14B-shaped decode step, 48 layers, context 32768, tp{world} over kv heads; all-reduce after o_proj "
                   "and down_proj, arg-max gather; CUDA-graph replay; max over ranks")
    return out


def run_step(args):
    """A decode-step workload on its own (`--workload qwen25_14b_decode_step_*`)."""
    import torch
    import torch.distributed as dist
    from jacq_b200 import _native
    _native.lib()
    rank, local_rank, world = _dist_env()
    device = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(device)
    group = None
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD
    batch, context = STEP_WORKLOADS[args.workload]
    rec = measure_step(batch, context, args.comm, args.steps, args.warmup, device, rank, local_rank, world, group,
                       profile_only=args.profile_only)
    if rank == 0:
        print(json.dumps(rec))
    if world > 1:
        # no destroy_process_group(): with NCCL collectives inside a captured graph it can block for minutes
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


def run_reference_cuda_lane(args):
    """Reference arm at the reference's own lane (40/8 heads, head_dim 128, block = group = 32,
    context 4096): the reference's emitted CUDA kernel, compiled unmodified into oracle/_ref, timed on
    this GPU the way the reference serves it -- one jac_launch per sequence (it has no batch form)."""
    import ctypes
    import torch
    from tests import helpers
    from oracle import kivi_oracle as ko
    key, batch, context = WORKLOADS[args.workload]
    case = helpers.CONFIGS[key]
    lib_path = ROOT / "oracle" / "_ref" / "libjacq_ref.so"
    if not lib_path.exists():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libjacq_ref.so was not built "
                          "(needs the reference checkout at build time)"}))
        return
    ref = ctypes.CDLL(str(lib_path))
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    geom = helpers.oracle_geometry(case)
    lay = helpers.layout_of(case)
    pages = lay.old_pages(context)
    nthreads = os.cpu_count() or 1
    tables = helpers.shuffled_block_tables(batch, pages, batch * pages)
    oc = ko.OracleCache(geom, batch * pages, batch)
    kv = [helpers.make_kv(case, context, stream=i) for i in range(batch)]
    ko.write_batch(oc, np.concatenate([k for k, _ in kv]), np.concatenate([v for _, v in kv]), tables,
                   np.zeros(batch, np.int32), np.arange(batch + 1, dtype=np.int32) * context, nthreads=nthreads)

    def dev(a):
        t = torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).to(device)
        return t.view(torch.float16) if a.dtype == np.uint16 else t
    pools = [dev(getattr(oc, n)) for n in ("k_code", "k_scale", "k_zero", "v_code", "v_scale", "v_zero")]
    ks, vs = dev(oc.k_scratch), dev(oc.v_scratch)
    bt = torch.from_numpy(tables).to(device)
    q = dev(helpers.make_q(case, batch).view(np.uint16))
    out = torch.zeros((batch, case.nh, case.d), dtype=torch.float32, device=device)
    P = ctypes.c_void_p
    stream = P(torch.cuda.current_stream(device).cuda_stream)

    def step():
        for i in range(batch):
            ref.jac_launch(P(q[i].data_ptr()), P(bt[i].data_ptr()), *[P(t.data_ptr()) for t in pools],
                           P(ks[i].data_ptr()), P(vs[i].data_ptr()), ctypes.c_int(context), P(out[i].data_ptr()), stream)
    # the reference harness's method (crates/jac-codegen-cuda/src/templates/harness.cu:66-103): warm-up, then every
    # timed iteration behind an L2 eviction (a buffer larger than the L2 is written), cudaEvent timing, min / median / p90
    evict = torch.empty(192 << 20, dtype=torch.uint8, device=device)
    for _ in range(max(1, args.warmup)):
        step()
    torch.cuda.synchronize(device)
    ms = []
    for _ in range(args.steps):
        evict.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        torch.cuda.synchronize(device)
        ms.append(e0.elapsed_time(e1))
    ms.sort()
    mean_ms = statistics.median(ms)
    spread = {"min_ms": ms[0], "median_ms": mean_ms, "p90_ms": ms[min(len(ms) - 1, int(0.9 * len(ms)))]}
    step_bytes = lay.decode_algorithmic_bytes(context) * batch
    value = step_bytes / (mean_ms * 1e-3) / 1e9
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "timing": spread,
        "warmup": max(3, args.warmup), "ms_per_step": mean_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 SIMT", "data": "synthetic",
        "config": {"workload": args.workload, "note": "the reference's own CUDA (decode_attention_kivi_paged snapshot, "
                   "nvcc -O3 for sm_100a), one launch per sequence as in its serving loop"},
        "tokens_per_s": batch / (mean_ms * 1e-3),
        "cpu_baseline": None,
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_reference_step(args):
    """Reference arm of the decode-step workloads. The reference's generated runtime is CUDA only, so
    two things are timed: (1) the CPU port of the step (oracle/step_oracle.py, all host threads) on
    a bounded sample -- 2 of the 48 layers at batch 1 and a 4096-token context, scaled to a whole step;
    (2) where oracle/_ref holds it, the reference's own forward() (templates/runtime.cu, fp16 dense
    KV cache, cuBLAS GEMVs, one token per call) compiled unmodified for the same model shape, at
    the workload's context; it has no batch form, so a batch costs that many calls."""
    import ctypes
    from oracle import step_oracle as so
    batch, context = STEP_WORKLOADS[args.workload]
    _, _, world = _dist_env()
    nthreads = os.cpu_count() or 1
    layers_sampled, ctx_sampled = 2, 4096
    shape = so.StepShape(layers=layers_sampled, hidden=5120, nh=40, nkv=8, hd=128, ffn=13824, vocab=8192,
                         rope_base=1000000.0, norm_eps=1e-6, attn_bias=True, block=16, group=128, residual=128)
    w = so.random_weights(shape, 1)
    pages = (ctx_sampled - shape.residual) // shape.block + 2
    oracle = so.StepOracle(shape, w, np.arange(pages, dtype=np.int32).reshape(1, pages), pages, gemv_threads=nthreads)
    rng = np.random.default_rng(2)
    from oracle import kivi_oracle as ko
    for cache in oracle.caches[0]:       # synthetic context through the oracle writer
        k = rng.standard_normal((ctx_sampled, shape.nkv, shape.hd), dtype=np.float32).astype(np.float16)
        v = rng.standard_normal((ctx_sampled, shape.nkv, shape.hd), dtype=np.float32).astype(np.float16)
        ko.write_batch(cache, k, v, oracle.block_tables, np.zeros(1, np.int32), np.array([0, ctx_sampled], np.int32),
                       nthreads=nthreads)
    oracle.seq_lens[:] = ctx_sampled
    tok = np.array([11])
    oracle.step(tok)
    t0 = time.perf_counter()
    steps = max(1, min(args.steps, 3))
    for _ in range(steps):
        oracle.step(tok)
    sample_s = (time.perf_counter() - t0) / steps
    cpu_step_s = sample_s * 48 / layers_sampled           # layers dominate; the 8192-row lm_head sample rides along
    cpu_value = 1.0 / cpu_step_s
    sample = (f"{layers_sampled} of 48 layers, batch 1, context {ctx_sampled}, vocab 8192, scaled by 48/{layers_sampled}; "
              "scalar C + OpenMP")
    ref_cuda = None
    lib_path = ROOT / "oracle" / "_ref" / "libjacq_ref.so"
    import torch
    if lib_path.exists() and torch.cuda.is_available():
        from jacq_b200.runtime import DecodeModelConfig, random_layer
        ref = ctypes.CDLL(str(lib_path))
        ref.ref_q14b_time_steps.restype = ctypes.c_float
        ref.ref_q14b_set_weights.restype = ctypes.c_int
        device = torch.device("cuda:0")
        torch.cuda.set_device(device)
        cfg = DecodeModelConfig.qwen25_14b()
        gen = torch.Generator(device=device).manual_seed(1234)
        big = lambda r, c: (torch.randn((r, c), generator=gen, device=device, dtype=torch.float32) * 0.02).half()
        keep = [big(cfg.vocab, cfg.hidden), (1.0 + 0.1 * torch.randn((cfg.hidden,), generator=gen, device=device)).half(),
                big(cfg.vocab, cfg.hidden)]
        ptrs = (ctypes.c_void_p * (7 * cfg.layers))()
        for l in range(cfg.layers):
            lw = random_layer(cfg, gen, device)
            for j, kname in enumerate(("attn_norm", "qkv", "qkv_bias", "o", "ffn_norm", "gate_up", "down")):
                keep.append(lw[kname])
                ptrs[7 * l + j] = lw[kname].data_ptr()
        torch.cuda.synchronize()
        if ref.ref_q14b_set_weights(ctypes.c_void_p(keep[0].data_ptr()), ctypes.c_void_p(keep[1].data_ptr()),
                                    ctypes.c_void_p(keep[2].data_ptr()), ptrs) == 0:
            warm = max(1, min(args.warmup, 3))
            k_steps = max(1, min(args.steps, 20))
            pos = context - warm - k_steps - 1
            ref.ref_q14b_time_steps(ctypes.c_int(11), ctypes.c_int(pos), ctypes.c_int(warm))
            ms = float(ref.ref_q14b_time_steps(ctypes.c_int(11), ctypes.c_int(pos + warm), ctypes.c_int(k_steps))) / k_steps
            ref_cuda = {"ms_per_token": ms, "tokens_per_s": 1000.0 / ms, "context": context,
                        "what": "reference forward() + argmax_kernel, fp16 dense KV cache, cuBLAS GEMVs, one token per call"}
    value = ref_cuda["tokens_per_s"] if ref_cuda else cpu_value
    print(json.dumps({
        "impl": "reference", "metric": "decode-step tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": batch * 1000.0 / value, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16" if ref_cuda else "f32 scalar", "data": "synthetic",
        "config": {"workload": args.workload, "note": "value = the reference's own CUDA forward() on this GPU when "
                   "oracle/_ref is present (it serves one sequence per call, so a batch is served at the same tokens/s), "
                   "else the CPU port"},
        "reference_cuda": ref_cuda,
        "cpu_baseline": {"value": cpu_value, "unit": "tokens/s", "cores": nthreads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_reference(args):
    """Reference arm: the CPU port of the reference's writer + decode math, all host threads, no GPU.
    At the reference's own lane the reference's CUDA itself is timed instead."""
    rank, local_rank, world = _dist_env()
    if rank != 0:
        return
    if args.workload in STEP_WORKLOADS:
        return run_reference_step(args)
    if WORKLOADS[args.workload][0] == "reflane":
        return run_reference_cuda_lane(args)
    from tests import helpers
    from oracle import kivi_oracle as ko
    key, batch, context = WORKLOADS[args.workload]
    case = helpers.CONFIGS[key]
    geom = helpers.oracle_geometry(case)
    lay = helpers.layout_of(case)
    nthreads = os.cpu_count() or 1
    n = min(batch, max(1, nthreads))      # one sequence per host thread and step: about half a second of CPU work
    pages = lay.old_pages(context) + 1
    tables = helpers.shuffled_block_tables(n, pages, n * pages)
    oc = ko.OracleCache(geom, n * pages, n)
    kv = [helpers.make_kv(case, context, stream=i) for i in range(n)]
    ko.write_batch(oc, np.concatenate([k for k, _ in kv]), np.concatenate([v for _, v in kv]), tables,
                   np.zeros(n, np.int32), np.arange(n + 1, dtype=np.int32) * context, nthreads=nthreads)
    qh = helpers.make_q(case, n)
    lens = np.full(n, context, np.int32)
    step_bytes = lay.decode_algorithmic_bytes(context) * n
    warm = args.warmup
    for _ in range(warm):
        ko.decode_batch(oc, qh, tables, lens, mode=0, nthreads=nthreads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ko.decode_batch(oc, qh, tables, lens, mode=0, nthreads=nthreads)
    secs = (time.perf_counter() - t0) / args.steps
    value = step_bytes / secs / 1e9
    sample = f"each step = {n} of {batch} sequences of the workload, all heads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": secs * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 scalar", "data": "synthetic",
        "config": {"workload": args.workload, "note": "the reference's own implementation of this path is CUDA "
                   "only and is compiled for block = group = 32 / head_dim 128 / context <= 4096, so it cannot run "
                   "this geometry; this arm times the CPU port of its kernel math (oracle/) on the host cores"},
        "tokens_per_s": n / secs,
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": nthreads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + sorted(SECONDARY) + sorted(STEP_WORKLOADS))
    ap.add_argument("--comm", default="p2p", choices=["p2p", "nccl"],
                    help="decode-step workloads on several GPUs: the library's peer-memory exchange or NCCL hooks")
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false")
    ap.add_argument("--no-e2e-graph", dest="e2e_graph", action="store_false",
                    help="attention workloads: issue the end-to-end serving step as separate calls instead of one CUDA graph")
    ap.add_argument("--no-extras", dest="extras", action="store_false",
                    help="default workload: only the headline measurement (no secondary / tensor-parallel records)")
    ap.add_argument("--profile-only", action="store_true",
                    help="build the cache, run warmup+steps decode launches and exit (for ncu)")
    args = ap.parse_args()
    _, _, world = _dist_env()
    if args.gpus != world and world == 1 and args.gpus > 1:
        # launched without torchrun: spawn the ranks ourselves
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29571", __file__] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    if world > 1:
        args.cpu_baseline = False   # rank 0 at N = 1 only
    if args.workload in STEP_WORKLOADS and args.impl != "reference":
        run_step(args)
    elif args.workload in SECONDARY:
        run_secondary(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
