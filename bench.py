#!/usr/bin/env python
"""Benchmark of the logits -> per-token log-prob path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--skip-extra]

One JSON line on stdout (rank 0).  Headline workload: selective log-softmax over bf16 logits
[20480 x 151936] (4 prompts x group 8 x 640 tokens), one step = one pass of the kernel over
that matrix.  With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank
scores its own 20480 rows: the path has no exchange step, so scaling is weak and there is
no collective.  The "extra" object carries the other workloads: fp32 selective, fused LM
head + log-prob (tensor cores), the vocab-parallel head over the N ranks (one all-reduce),
and GRPO dual scoring.

``--impl reference`` times the CPU restatement of the reference's MLX arithmetic
(oracle/oracle.py; MLX itself is not installable here and its Metal kernel is Apple-only)
on the host cores, on a bounded row sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ROWS = 20480
VOCAB = 151936
METRIC = "selective_logprob_rows_per_s"
UNIT = "rows/s"

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the headline kernel: an ncu
# capture of the same kernel on 2048 rows (a full-size capture is too large to profile
# safely) read 622.46 MB and wrote 3.41 MB; traffic grows with the row count, so x10.
NCU_TRAFFIC_BYTES = 6_258_690_560
CHECK_TOL = 2e-3  # max-abs on log-probs: the bar of the bf16 paths


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
                "source": "fallback"}


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


# ---------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period, self.samples, self.reasons = index, period_s, [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nvml = None

    def _reasons(self):
        n = self.nvml
        try:
            bits = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
        except Exception:
            try:
                bits = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
            except Exception:
                return
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                 0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}
        for bit, name in names.items():
            if bits & bit:
                self.reasons.add(name)

    def _sample(self):
        try:
            self.samples.append(int(self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM)))
            self._reasons()
        except Exception:
            pass

    def _loop(self):
        while not self._stop.is_set():
            self._sample()
            time.sleep(self.period)

    def __enter__(self):
        if self.nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            if not self.samples:
                self._sample()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


# ---------------------------------------------------------------------------- timing
def timed_steps(fn, steps, warmup, barrier, sampler=None):
    """W untimed steps, then K steps between barrier+synchronize, one CUDA-event pair per
    step on the launching stream.  Returns (total ms, per-launch ms list)."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
          for _ in range(steps)]
    t_begin = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    ctx = sampler if sampler is not None else _Null()
    with ctx:
        t_begin.record()
        for a, b in ev:
            a.record()
            fn()
            b.record()
        t_end.record()
        torch.cuda.synchronize()
    barrier()
    total = t_begin.elapsed_time(t_end)
    return total, [a.elapsed_time(b) for a, b in ev]


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def max_over_ranks(x: float, dist_on: bool, device) -> float:
    if not dist_on:
        return x
    import torch
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ---------------------------------------------------------------------------- CPU legs
def cpu_selective(rows_sample: int, threads: int, seed: int = 1002, repeats: int = 1):
    """Times the CPU oracle on ``rows_sample`` rows of the headline workload; rows/s."""
    import torch
    from oracle import oracle
    from tome_b200 import synthetic
    torch.set_num_threads(threads)
    x, ids = synthetic.cfg2_rollout_bf16(rows=rows_sample, device="cpu", seed=seed)
    oracle.selective_logprob(x[:64], ids[:64], 1.0)
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.selective_logprob(x, ids, 1.0)
        best = min(best, time.perf_counter() - t0)
    return rows_sample / best, best


def run_reference(args, rank: int):
    """CPU implementation of the path on the host cores; same metric, config and unit."""
    if rank != 0:
        return
    import torch
    from oracle import oracle
    from tome_b200 import synthetic
    threads = host_cores()
    torch.set_num_threads(threads)
    sample = 1024
    x, ids = synthetic.cfg2_rollout_bf16(rows=sample, device="cpu")
    for _ in range(max(1, args.warmup)):
        oracle.selective_logprob(x, ids, 1.0)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.selective_logprob(x, ids, 1.0)
    dt = time.perf_counter() - t0
    value = sample * args.steps / dt
    desc = f"{sample} rows x {VOCAB} bf16 per step (of {ROWS}), same distribution"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "cfg2: selective log-softmax, bf16 logits [20480 x 151936]",
                   "rows": ROWS, "vocab": VOCAB, "sample": desc},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of mlx-impl/node.py:400-404 (MLX is not installable offline; "
                "the Metal kernel is Apple-only)",
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------- GPU legs
def run_ours(args):
    # stdout must carry exactly one JSON line: libraries that print to file descriptor 1 (NCCL's
    # version banner, for one) are sent to stderr for the duration of the run
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    try:
        line = _run_ours(args)
    finally:
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        os.close(real_stdout)
    if line is not None:
        print(json.dumps(line), flush=True)


def _run_ours(args):
    import torch
    import tome_b200
    from tome_b200 import synthetic

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist_on = world > 1
    if dist_on:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep NCCL's version banner off stdout
        dist.init_process_group("nccl", device_id=device)
        barrier = lambda: dist.barrier(device_ids=[local])  # noqa: E731
    else:
        barrier = lambda: None  # noqa: E731
    peaks = measured_peaks()
    # at least three untimed warm-up steps, whatever was asked for (timing hygiene)
    steps, warmup = max(1, args.steps), max(args.warmup, 3)

    # ---------------- headline: cfg2 selective log-softmax, bf16 [20480 x 151936] per GPU
    logits, targets = synthetic.cfg2_rollout_bf16(ROWS, VOCAB, device, seed=1002 + rank)
    out_box = {}

    def step():
        out_box["lp"] = tome_b200.local_compute_logprobs(logits, targets, 1.0)

    sampler = ClockSampler(physical_gpu_index(local)) if rank == 0 else None
    total_ms, per_launch = timed_steps(step, steps, warmup, barrier, sampler)
    total_ms = max_over_ranks(total_ms, dist_on, device)
    tome_b200.check_device_status(device)
    ms_per_step = total_ms / steps
    value = world * ROWS * steps / (total_ms * 1e-3)
    launch_ms = sum(per_launch) / len(per_launch)
    algo_bytes = ROWS * VOCAB * 2 + ROWS * 8
    achieved = algo_bytes / (launch_ms * 1e-3) / 1e9
    # independent check that the timed kernel did the work: torch reduction on a row sample
    sample = torch.arange(0, ROWS, 320, device=device)
    ref = torch.log_softmax(logits[sample].float(), dim=-1).gather(
        1, targets[sample].long()[:, None]).squeeze(1)
    check_err = float((out_box["lp"][sample] - ref).abs().max())

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "cfg2: selective log-softmax, bf16 logits [20480 x 151936] per GPU "
                               "(4 prompts x group 8 x 640 tokens), fp32 accumulate",
                   "rows_per_gpu": ROWS, "vocab": VOCAB, "temperature": 1.0,
                   "l2": "inputs (6.2 GB per step) are larger than L2; no flush needed",
                   "parallelism": "row-sharded replicas, no collective"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                     "traffic": NCU_TRAFFIC_BYTES, "peak_source": peaks["source"],
                     "algorithmic_bytes_per_launch": algo_bytes,
                     "launch_ms": launch_ms, "frac_of_nominal_8TBps": achieved / 8000.0},
        "gpu_launches": steps,
        "warmup_requested": args.warmup,
        "check": {"max_abs_vs_torch_log_softmax": check_err, "rows_checked": int(sample.numel())},
    }
    if sampler is not None:
        line["clocks"] = sampler.summary()

    # ---------------- end to end through the public host-buffer call (rank-local)
    e2e_steps = max(2, min(steps, 3))
    host_logits = torch.empty((ROWS, VOCAB), dtype=torch.bfloat16).pin_memory()
    host_logits.copy_(logits)
    host_ids = targets.cpu().pin_memory()
    staging = {"key": (tuple(logits.shape), logits.dtype), "logits": logits,
               "ids": torch.empty_like(targets),
               "out": torch.empty((ROWS,), dtype=torch.float32).pin_memory()}
    tome_b200.local_compute_logprobs_host(host_logits, host_ids, 1.0, device, staging)
    barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        tome_b200.local_compute_logprobs_host(host_logits, host_ids, 1.0, device, staging)
    torch.cuda.synchronize()
    e2e_local = time.perf_counter() - t0
    e2e_s = max_over_ranks(e2e_local, dist_on, device)
    h2d_bytes = ROWS * VOCAB * 2 + ROWS * 4
    # the step is the host->device copy: say how fast each rank's copy ran, so that a drop at
    # N > 1 names the host link (PCIe switch / root complex shared between GPUs, NUMA)
    h2d_rate = h2d_bytes * e2e_steps / e2e_local / 1e9
    if dist_on:
        rates = torch.zeros(world, dtype=torch.float64, device=device)
        rates[rank] = h2d_rate
        dist.all_reduce(rates)
        h2d_rates = [round(float(v), 2) for v in rates.tolist()]
    else:
        h2d_rates = [round(h2d_rate, 2)]
    line["e2e"] = {"value": world * ROWS * e2e_steps / e2e_s, "unit": UNIT,
                   "h2d_bytes_per_step": h2d_bytes,
                   "d2h_bytes_per_step": ROWS * 4, "steps": e2e_steps,
                   "ms_per_step": 1e3 * e2e_s / e2e_steps,
                   "h2d_GBps_per_rank": h2d_rates,
                   "h2d_GBps_aggregate": round(sum(h2d_rates), 2),
                   "bound": "host->device copy of the logits (pinned memory); the kernel is "
                            "under 1 ms of each step",
                   "call": "tome_b200.local_compute_logprobs_host (pinned host logits -> host fp32)"}
    del host_logits, staging, logits, targets
    torch.cuda.empty_cache()

    extra, failures = {}, []
    if check_err > CHECK_TOL:
        failures.append(f"headline: max_abs {check_err:.3g}")
    if not args.skip_extra:
        extra, more = run_extra(args, device, rank, world, dist_on, barrier, peaks)
        failures += more
    line["extra"] = extra
    line["checks_failed"] = failures

    # ---------------- CPU baseline beside the GPU number (rank 0, N = 1 only)
    if rank == 0 and world == 1 and not args.skip_cpu:
        threads = host_cores()
        probe_rps, _ = cpu_selective(256, threads)
        n = int(min(8192, max(512, probe_rps * 12.0)))  # about 12 s of CPU work
        rps, secs = cpu_selective(n, threads)
        line["cpu_baseline"] = {
            "value": rps, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{n} rows x {VOCAB} bf16 of the same distribution, {secs:.1f} s, "
                      "oracle/oracle.py (torch CPU restatement of mlx-impl/node.py:400-404)"}
    elif rank == 0:
        line["cpu_baseline"] = None

    if dist_on:
        import torch.distributed as dist
        dist.barrier(device_ids=[local])
        dist.destroy_process_group()
    if failures:  # a timed kernel whose result is wrong is not a measurement
        if rank == 0:
            print(json.dumps(line), file=sys.stderr, flush=True)
        raise SystemExit("bench.py: result checks failed: " + "; ".join(failures))
    return line if rank == 0 else None


def run_extra(args, device, rank, world, dist_on, barrier, peaks):
    """The other workloads: reported under "extra", each timed like the headline and each
    compared, after its timed loop, with an independent torch computation on a sample of its
    rows ("check").  Returns (extra, list of failed checks)."""
    import torch
    import tome_b200
    from tome_b200 import synthetic
    extra, failures = {}, []
    steps = max(3, min(args.steps, 20))
    warm = max(3, min(args.warmup, 5))

    def timed(fn, k=steps, w=warm):
        total, per = timed_steps(fn, k, w, barrier)
        return max_over_ranks(total, dist_on, device) / k, sum(per) / len(per)

    def verdict(name, errors, tol=CHECK_TOL):
        """Records {metric: max_abs} under extra[name]["check"]; every rank must pass."""
        worst = max(errors.values()) if errors else 0.0
        worst = float("inf") if worst != worst else worst
        worst = max_over_ranks(worst, dist_on, device)
        extra[name]["check"] = dict({k: float(v) for k, v in errors.items()}, tol=tol,
                                    ranks_checked=world)
        if not worst <= tol:
            failures.append(f"{name}: {worst:.3g} > {tol:g}")

    def torch_logprob(x, ids, temp):
        lsm = torch.log_softmax(x.float() / temp, dim=-1)
        return lsm.gather(1, ids.long()[:, None]).squeeze(1)

    # cfg1: fp32 selective [1024 x 151936]; L2 (126 MB) is flushed before every launch by
    # writing a 256 MB buffer and then reading another one (the read pushes the dirty lines of
    # the write out, so their write-back does not land inside the timed launch)
    x, ids = synthetic.cfg1_selective_fp32(1024, VOCAB, device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    flush_rd = torch.zeros(64 << 20, dtype=torch.float32, device=device)
    evs = []
    box = {}

    def cfg1_step():
        flush.zero_()
        flush_rd.sum()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        box["lp"] = tome_b200.local_compute_logprobs(x, ids, 1.0)
        b.record()
        evs.append((a, b))

    for _ in range(warm + steps):
        cfg1_step()
    torch.cuda.synchronize()
    ms = sum(a.elapsed_time(b) for a, b in evs[warm:]) / steps
    nbytes = 1024 * VOCAB * 4 + 1024 * 8
    extra["cfg1_selective_fp32"] = {"rows": 1024, "ms": ms, "rows_per_s": 1024 / (ms * 1e-3),
                                    "GBps": nbytes / ms / 1e6,
                                    "frac_of_measured_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"],
                                    "l2": "flushed by a 256 MB write + 256 MB read before each launch"}
    # the same launch repeated without the flush (the 622 MB of logits are five times L2, so a
    # launch finds nothing of them there): launch latency overlaps the launch before
    lp_out = torch.empty(1024, dtype=torch.float32, device=device)
    for _ in range(warm):
        tome_b200.local_compute_logprobs(x, ids, 1.0, out=lp_out)
    ev_a, ev_b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev_a.record()
    for _ in range(steps):
        tome_b200.local_compute_logprobs(x, ids, 1.0, out=lp_out)
    ev_b.record()
    torch.cuda.synchronize()
    ms_b2b = max_over_ranks(ev_a.elapsed_time(ev_b) / steps, dist_on, device)
    extra["cfg1_selective_fp32"]["back_to_back"] = {
        "ms": ms_b2b, "GBps": nbytes / ms_b2b / 1e6,
        "frac_of_measured_hbm": nbytes / ms_b2b / 1e6 / peaks["hbm_gbs"],
        "l2": "no flush: inputs (622 MB) are larger than L2"}
    sel = torch.arange(0, 1024, 16, device=device)
    verdict("cfg1_selective_fp32",
            {"max_abs_logprob": (box["lp"][sel] - torch_logprob(x[sel], ids[sel], 1.0)).abs().max()},
            tol=1e-4)
    del x, ids, flush, flush_rd

    # cfg5: dual scoring + k3 KL, bf16 [32 x 768 x 151936] x 2, ragged lengths, temperature 0.7
    pol, ref, tg, lengths, temp = synthetic.cfg5_dual(32, 768, VOCAB, device)
    active = int(lengths.sum().item())

    def dual_step():
        box["dual"] = tome_b200.grpo_dual_logprob_kl(pol, ref, tg, lengths, temp)

    ms, launch = timed(dual_step)
    nbytes = 2 * active * VOCAB * 2
    extra["cfg5_dual_kl"] = {"active_rows": active, "dense_rows": 32 * 768, "ms": ms,
                             "active_rows_per_s": active / (ms * 1e-3),
                             "GBps": nbytes / launch / 1e6,
                             "frac_of_measured_hbm": nbytes / launch / 1e6 / peaks["hbm_gbs"]}
    # sample: the first, a middle and the last active position of every fourth sequence; every
    # position outside the windows must be zero
    seqs = torch.arange(0, 32, 4, device=device)
    lens = lengths[seqs].long()
    pos = torch.stack([torch.zeros_like(lens), lens // 2, lens - 1], 1)          # [8, 3]
    sq = seqs[:, None].expand_as(pos)
    lp_p, lp_r, kl = box["dual"]
    want_p = torch_logprob(pol[sq, pos].reshape(-1, VOCAB), tg[sq, pos].reshape(-1), temp)
    want_r = torch_logprob(ref[sq, pos].reshape(-1, VOCAB), tg[sq, pos].reshape(-1), temp)
    d = want_r - want_p
    outside = torch.arange(768, device=device)[None, :] >= lengths[:, None]
    masked = lp_p[outside].abs().sum() + lp_r[outside].abs().sum() + kl[outside].abs().sum()
    verdict("cfg5_dual_kl",
            {"max_abs_policy": (lp_p[sq, pos].reshape(-1) - want_p).abs().max(),
             "max_abs_reference": (lp_r[sq, pos].reshape(-1) - want_r).abs().max(),
             "max_abs_kl": (kl[sq, pos].reshape(-1) - (torch.exp(d) - d - 1.0)).abs().max(),
             "masked_positions_abs_sum": masked})
    # ragged single-model scoring packed to the wire layout (node.py:446-458), same logits
    starts = torch.zeros_like(lengths)
    packed_targets = torch.cat([tg[i, : int(lengths[i])] for i in range(tg.shape[0])])

    def ragged_step():
        box["ragged"] = tome_b200.ragged_logprobs(ref, packed_targets, lengths, temp, starts=starts)

    ms_r, launch_r = timed(ragged_step)
    extra["ragged_ref_logprobs"] = {"active_rows": active, "ms": ms_r,
                                    "active_rows_per_s": active / (ms_r * 1e-3),
                                    "GBps": active * VOCAB * 2 / launch_r / 1e6}
    packed, offsets = box["ragged"]
    dense_ref = torch.cat([lp_r[i, : int(lengths[i])] for i in range(lp_r.shape[0])])
    verdict("ragged_ref_logprobs",
            {"max_abs_vs_dual_reference_logprob": (packed - dense_ref).abs().max(),
             "offsets_mismatch": float(int(offsets[-1]) != active)})
    del pol, ref, tg, lengths, packed_targets, starts, lp_p, lp_r, kl, packed, dense_ref
    box.clear()
    torch.cuda.empty_cache()

    # fused top-k sampling + log-prob: one decode step of 64 sequences (the reference's
    # batch), mid-size batches, and large ones
    for name, rows_s in (("sample_topk_64rows", 64), ("sample_topk_128rows", 128),
                         ("sample_topk_256rows", 256), ("sample_topk_4096rows", 4096),
                         ("sample_topk_20480rows", 20480)):
        xs = (torch.randn((rows_s, VOCAB), device=device, dtype=torch.float32) * 3.0).to(
            torch.bfloat16)
        step_no = [0]
        # outputs and scratch are the caller's to reuse from step to step (a decode loop does)
        s_out = (torch.empty(rows_s, dtype=torch.int32, device=device),
                 torch.empty(rows_s, dtype=torch.float32, device=device))
        s_ws = torch.empty(max(16, tome_b200.sample_workspace_bytes(rows_s, VOCAB)),
                           dtype=torch.uint8, device=device)

        def sample_step():
            step_no[0] += 1
            tome_b200.sample_topk_logprob(xs, 0.7, 20, seed=7, offset=step_no[0], out=s_out,
                                          workspace=s_ws)

        ms_s, launch_s = timed(sample_step)
        extra[name] = {"rows": rows_s, "ms": ms_s, "rows_per_s": rows_s / (ms_s * 1e-3),
                       "GBps": rows_s * VOCAB * 2 / launch_s / 1e6,
                       "frac_of_measured_hbm": rows_s * VOCAB * 2 / launch_s / 1e6 / peaks["hbm_gbs"]}
        if rows_s <= 256 and not dist_on:
            # what a decode loop sees per call: back-to-back eager calls, wall clock ("ms" above
            # also carries two event records per call, several microseconds at this size)
            best = float("inf")
            for _ in range(3):
                for _ in range(20):
                    sample_step()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for _ in range(200):
                    sample_step()
                torch.cuda.synchronize()
                best = min(best, (time.perf_counter() - t0) / 200 * 1e6)
            extra[name]["eager_us"] = best
            # at this size the event records bracketing every call cost as much as the call:
            # the leg's headline figures are the back-to-back ones
            extra[name]["ms_with_event_records"] = extra[name]["ms"]
            extra[name]["ms"] = best * 1e-3
            extra[name]["rows_per_s"] = rows_s / (best * 1e-6)
            extra[name]["GBps"] = rows_s * VOCAB * 2 / best / 1e3
            extra[name]["frac_of_measured_hbm"] = extra[name]["GBps"] / peaks["hbm_gbs"]
            extra[name]["l2"] = ("the logits stay in L2 between calls, as they do behind the GEMM "
                                 "that writes them in a decode loop")
            # the kernels' own time, replayed from a CUDA graph; logits of this size stay in L2
            # between replays, as they do behind the GEMM that wrote them in a decode loop
            bound = tome_b200.bind_sample(xs, 0.7, 20, seed=7, out=s_out, workspace=s_ws)
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for _ in range(3):
                    bound(1)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for i in range(20):
                        bound(i)
            torch.cuda.synchronize()
            ms_g, _ = timed(graph.replay, k=20, w=3)
            extra[name]["graph_us"] = ms_g / 20 * 1e3
            extra[name]["graph_GBps"] = rows_s * VOCAB * 2 / (ms_g / 20) / 1e6
            del graph, bound
        tok, lp, tk_i, tk_v = tome_b200.sample_topk_logprob(xs, 0.7, 20, seed=7, offset=1,
                                                            return_topk=True)
        sel = torch.arange(0, rows_s, max(1, rows_s // 32), device=device)
        want_v, _ = torch.topk(xs[sel].float(), 20, dim=-1)
        in_topk = (tk_i[sel] == tok[sel, None]).any(dim=1)
        verdict(name, {"max_abs_logprob": (lp[sel] - torch_logprob(xs[sel], tok[sel], 0.7)).abs().max(),
                       "topk_values_max_abs": (tk_v[sel] - want_v).abs().max(),
                       "token_outside_topk": float((~in_topk).sum())})
        del xs, tok, lp, tk_i, tk_v, s_out, s_ws
    torch.cuda.empty_cache()

    # a vocabulary off the 16-byte grid (50257 bf16 logits per row, contiguous: every row starts
    # at another place of the grid): the same kernels, each row copied from its first 16-byte
    # boundary to its last
    rows_o, vocab_o = 8192, 50257
    xo = (torch.randn((rows_o, vocab_o), device=device, dtype=torch.float32) * 3.0).to(torch.bfloat16)
    ido = torch.randint(0, vocab_o, (rows_o,), device=device, dtype=torch.int32)
    lp_o = torch.empty(rows_o, dtype=torch.float32, device=device)
    full_o = torch.empty_like(xo)
    tok_o = (torch.empty(rows_o, dtype=torch.int32, device=device),
             torch.empty(rows_o, dtype=torch.float32, device=device))
    ws_o = torch.empty(max(16, tome_b200.sample_workspace_bytes(rows_o, vocab_o)),
                       dtype=torch.uint8, device=device)
    nb_o = rows_o * vocab_o * 2
    _, t_sel = timed(lambda: tome_b200.local_compute_logprobs(xo, ido, 1.0, out=lp_o))
    _, t_full = timed(lambda: tome_b200.fused_log_softmax(xo, 1.0, out=full_o))
    _, t_smp = timed(lambda: tome_b200.sample_topk_logprob(xo, 0.7, 20, seed=7, offset=1, out=tok_o,
                                                           workspace=ws_o))
    extra["odd_vocab_50257_bf16"] = {
        "rows": rows_o, "vocab": vocab_o, "selective_ms": t_sel, "selective_GBps": nb_o / t_sel / 1e6,
        "full_ms": t_full, "full_GBps": 2 * nb_o / t_full / 1e6,
        "sample_ms": t_smp, "sample_GBps": nb_o / t_smp / 1e6,
        "l2": "inputs (823 MB) are larger than L2"}
    sel = torch.arange(0, rows_o, rows_o // 32, device=device)
    want_full = xo[sel] - torch.logsumexp(xo[sel].float(), dim=-1, keepdim=True).to(torch.bfloat16)
    verdict("odd_vocab_50257_bf16",
            {"max_abs_logprob": (lp_o[sel] - torch_logprob(xo[sel], ido[sel], 1.0)).abs().max(),
             "max_abs_sampled_logprob": (tok_o[1][sel] - torch_logprob(xo[sel], tok_o[0][sel], 0.7)).abs().max()})
    full_err = float((full_o[sel].float() - want_full.float()).abs().max())
    extra["odd_vocab_50257_bf16"]["check"]["max_abs_full_bf16_ulp_0.0625"] = full_err
    if not full_err <= 0.0625 + 1e-3:
        failures.append(f"odd_vocab_50257_bf16 full: {full_err:.3g}")
    del xo, ido, lp_o, full_o, tok_o, ws_o, want_full
    torch.cuda.empty_cache()

    # paged KV gather / update: 64 sequences x 2048 tokens, 8 KV heads x 128, blocks of 16
    n_blk, Hkv, bs_kv, Dh, Bkv, Lkv = 64 * 128, 8, 16, 128, 64, 2048
    k_pool = torch.randn((n_blk, Hkv, bs_kv, Dh), device=device, dtype=torch.bfloat16)
    v_pool = torch.randn_like(k_pool)
    tables = torch.randperm(n_blk, device=device)[: Bkv * (Lkv // bs_kv)].reshape(Bkv, -1).to(torch.int32)
    offs = torch.full((Bkv,), Lkv, dtype=torch.int32, device=device)
    kv_bytes = 2 * 2 * Bkv * Hkv * Lkv * Dh * 2   # K and V, read + write
    ms_g, launch_g = timed(lambda: tome_b200.gather_paged_kv(tables, offs, k_pool, v_pool, Lkv))
    k_dense, v_dense = tome_b200.gather_paged_kv(tables, offs, k_pool, v_pool, Lkv)
    zero_off = torch.zeros_like(offs)
    k_before = k_pool.clone()
    ms_u, launch_u = timed(lambda: tome_b200.update_paged_kv(k_dense, v_dense, tables, zero_off,
                                                             k_pool, v_pool))
    extra["paged_kv"] = {"shape": "64 seq x 2048 tok x 8 heads x 128, bf16, block 16",
                         "gather_ms": ms_g, "gather_GBps": kv_bytes / launch_g / 1e6,
                         "update_ms": ms_u, "update_GBps": kv_bytes / launch_u / 1e6,
                         "note": "gather time includes torch's allocation of the outputs"}
    # gather: sequence b, token s lives in block tables[b, s // 16] at slot s % 16 (byte-exact);
    # update wrote the gathered tokens back where they came from, so the pool is unchanged
    bsel = torch.tensor([0, 17, 63], device=device)
    want_k = k_pool[tables[bsel].long()].permute(0, 2, 1, 3, 4).reshape(3, Hkv, Lkv, Dh)
    want_v = v_pool[tables[bsel].long()].permute(0, 2, 1, 3, 4).reshape(3, Hkv, Lkv, Dh)
    verdict("paged_kv", {"gather_mismatches": float((k_dense[bsel] != want_k).sum() +
                                                    (v_dense[bsel] != want_v).sum()),
                         "update_mismatches": float((k_pool != k_before).sum())}, tol=0.0)
    del k_pool, v_pool, tables, k_dense, v_dense, k_before, want_k, want_v
    torch.cuda.empty_cache()

    # full-matrix compatibility kernel: the reference's decode-loop shape (64 x V fp32) and
    # larger cases; algorithmic bytes = read + write of the matrix
    for name, rows_f, dt in (("full_fp32_64rows", 64, torch.float32),
                             ("full_bf16_4096rows", 4096, torch.bfloat16),
                             ("full_fp32_2048rows", 2048, torch.float32)):
        xf = (torch.randn((rows_f, VOCAB), device=device, dtype=torch.float32) * 2.0).to(dt)
        of = torch.empty_like(xf)
        ms_f, launch_f = timed(lambda: tome_b200.fused_log_softmax(xf, 1.0, out=of))
        nbytes = 2 * rows_f * VOCAB * xf.element_size()
        extra[name] = {"rows": rows_f, "ms": ms_f, "GBps": nbytes / launch_f / 1e6,
                       "frac_of_measured_hbm": nbytes / launch_f / 1e6 / peaks["hbm_gbs"]}
        if rows_f <= 256 and not dist_on:
            # a decode-step batch: the event records around every call cost as much as the
            # call, so the leg's figures are those of back-to-back eager calls (wall clock)
            best = float("inf")
            for _ in range(3):
                for _ in range(20):
                    tome_b200.fused_log_softmax(xf, 1.0, out=of)
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for _ in range(200):
                    tome_b200.fused_log_softmax(xf, 1.0, out=of)
                torch.cuda.synchronize()
                best = min(best, (time.perf_counter() - t0) / 200 * 1e3)
            extra[name].update({"ms_with_event_records": ms_f, "ms": best,
                                "GBps": nbytes / best / 1e6,
                                "frac_of_measured_hbm": nbytes / best / 1e6 / peaks["hbm_gbs"],
                                "l2": "the logits stay in L2 between calls, as they do behind "
                                      "the GEMM that writes them in a decode loop"})
        sel = torch.arange(0, rows_f, max(1, rows_f // 16), device=device)
        # the Metal kernel's order of operations (mlx-impl/model.py:57-60): the lse is rounded
        # to the logits' dtype and subtracted in that dtype; bf16 outputs sit near -12, where
        # one bf16 ulp is 0.0625 (a flip of the lse's rounding moves a whole row by one ulp)
        want = xf[sel] - torch.logsumexp(xf[sel].float(), dim=-1, keepdim=True).to(dt)
        verdict(name, {"max_abs": (of[sel].float() - want.float()).abs().max()},
                tol=1e-4 if dt == torch.float32 else 0.0625 + 1e-3)
        del xf, of, want
    torch.cuda.empty_cache()

    # one decode step of the reference's rollout (64 sequences x V fp32 logits, node.py:590-605):
    # (a) replayed from a CUDA graph, so the numbers are the kernels' own time without the host
    # cost of the Python call; (b) called eagerly in a loop, which is what a decode loop sees
    # (the larger of host time per call and kernel time), through the plain functions with
    # preallocated outputs and through bound calls.  Single process only: a process group's
    # watchdog thread must not meet a stream capture.
    if not dist_on:
        xd = torch.randn((64, VOCAB), device=device, dtype=torch.float32) * 3.0
        idd = torch.randint(0, VOCAB, (64,), device=device, dtype=torch.int32)
        calls = {"selective_us": lambda: tome_b200.local_compute_logprobs(xd, idd, 0.7),
                 "sample_topk_us": lambda: tome_b200.sample_topk_logprob(xd, 0.7, 20, seed=7,
                                                                         offset=1),
                 "full_matrix_us": lambda: tome_b200.fused_log_softmax(xd, 0.7)}
        step = {"shape": "64 x 151936 fp32", "how": "20 calls per CUDA graph, 20 replays"}
        side = torch.cuda.Stream()
        for key, call in calls.items():
            with torch.cuda.stream(side):
                for _ in range(3):
                    call()
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(20):
                        call()
            torch.cuda.synchronize()
            ms_g, _ = timed(graph.replay, k=20, w=3)
            step[key] = ms_g / 20 * 1e3
            del graph
        extra["decode_step_64rows_graph"] = step

        out_lp = torch.empty(64, dtype=torch.float32, device=device)
        out_tok = torch.empty(64, dtype=torch.int32, device=device)
        out_full = torch.empty_like(xd)
        b_sel = tome_b200.bind_selective(xd, idd, 0.7, out=out_lp)
        b_smp = tome_b200.bind_sample(xd, 0.7, 20, seed=7, out=(out_tok, out_lp))
        b_full = tome_b200.bind_log_softmax(xd, 0.7, out=out_full)
        eager = {
            "selective_us": lambda: tome_b200.local_compute_logprobs(xd, idd, 0.7, out=out_lp),
            "sample_topk_us": lambda: tome_b200.sample_topk_logprob(xd, 0.7, 20, seed=7, offset=1,
                                                                    out=(out_tok, out_lp)),
            "full_matrix_us": lambda: tome_b200.fused_log_softmax(xd, 0.7, out=out_full),
            "selective_bound_us": b_sel,
            "sample_topk_bound_us": lambda: b_smp(1),
            "full_matrix_bound_us": b_full,
        }
        per_call = {"shape": "64 x 151936 fp32",
                    "how": "500 back-to-back eager calls, wall clock / 500, best of 3; plain "
                           "functions with out= and bound calls (tome_b200.bind_*)"}
        for key, call in eager.items():
            best = float("inf")
            for _ in range(3):
                for _ in range(50):
                    call()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for _ in range(500):
                    call()
                torch.cuda.synchronize()
                best = min(best, (time.perf_counter() - t0) / 500 * 1e6)
            per_call[key] = best
        extra["decode_step_64rows_eager"] = per_call
        verdict("decode_step_64rows_eager",
                {"max_abs_selective": (b_sel()[0] - torch_logprob(xd, idd, 0.7)).abs().max(),
                 "max_abs_full": (b_full()[0] - torch.log_softmax(xd / 0.7, -1)).abs().max()},
                tol=1e-4)
        del xd, idd, out_full
    torch.cuda.empty_cache()

    def head_reference(hidden, weight, ids, temp, sel):
        """Unsharded log-probs of the rows `sel`: fp32 matmul on the device + logsumexp."""
        logits = hidden[sel].float() @ weight.float().t()
        lsm_lse = torch.logsumexp(logits / temp, dim=-1)
        return logits.gather(1, ids[sel].long()[:, None]).squeeze(1) / temp - lsm_lse, lsm_lse

    # cfg3: fused LM head + log-prob, Qwen3-0.6B head shape
    hidden, weight, ids = synthetic.cfg3_lm_head(16384, 1024, VOCAB, device)
    ws = torch.empty(tome_b200.lm_head_workspace_bytes(16384, 1024, VOCAB), dtype=torch.uint8,
                     device=device)
    sampler3 = ClockSampler(physical_gpu_index(device.index)) if rank == 0 else None

    def head_step():
        box["head"] = tome_b200.lm_head_logprob(hidden, weight, ids, 1.0, workspace=ws)

    total, per = timed_steps(head_step, steps, warm, barrier, sampler3)
    ms, launch = max_over_ranks(total, dist_on, device) / steps, sum(per) / len(per)
    flops = 2.0 * 16384 * VOCAB * 1024
    extra["cfg3_lm_head"] = {"rows": 16384, "hidden": 1024, "ms": ms,
                             "rows_per_s": 16384 / (ms * 1e-3), "TFLOPs": flops / ms / 1e9,
                             "frac_of_measured_bf16": flops / ms / 1e9 / peaks["bf16_tflops"],
                             "frac_of_measured_bf16_sustained":
                                 flops / ms / 1e9 / peaks["bf16_tflops_sustained"],
                             "frac_of_nominal_2250": flops / ms / 1e9 / 2250.0,
                             "launches_per_step": 2,
                             "clocks": sampler3.summary() if sampler3 is not None else None}
    sel = torch.arange(0, 16384, 256, device=device)
    want_lp, want_lse = head_reference(hidden, weight, ids, 1.0, sel)
    verdict("cfg3_lm_head", {"max_abs_logprob": (box["head"][0][sel] - want_lp).abs().max(),
                             "max_abs_lse": (box["head"][1][sel] - want_lse).abs().max()})
    # the unfused pipeline on the same inputs, for context: cuBLAS GEMM that materialises the
    # bf16 logits (4.98 GB), then the streaming selective kernel over them
    if rank == 0 or dist_on:
        logits_buf = torch.empty((16384, VOCAB), dtype=torch.bfloat16, device=device)
        ms_gemm, _ = timed(lambda: torch.matmul(hidden, weight.t(), out=logits_buf))

        def unfused():
            torch.matmul(hidden, weight.t(), out=logits_buf)
            tome_b200.local_compute_logprobs(logits_buf, ids, 1.0)

        ms_unfused, _ = timed(unfused)
        extra["cfg3_lm_head"]["context_cublas_gemm_only_ms"] = ms_gemm
        extra["cfg3_lm_head"]["context_cublas_gemm_only_TFLOPs"] = flops / ms_gemm / 1e9
        extra["cfg3_lm_head"]["context_unfused_gemm_then_selective_ms"] = ms_unfused
        del logits_buf
    # one or two row tiles: the kernel is bound by reading the weight matrix once
    for rows_small in (128, 256):
        hs = hidden[:rows_small].contiguous()
        ids_s = ids[:rows_small].contiguous()
        ms_s, launch_s = timed(lambda: tome_b200.lm_head_logprob(hs, weight, ids_s, 1.0, workspace=ws))
        extra[f"lm_head_{rows_small}rows"] = {
            "rows": rows_small, "hidden": 1024, "us": launch_s * 1e3,
            "weight_GBps": VOCAB * 1024 * 2 / launch_s / 1e6}
    del hidden, weight, ids, ws
    box.clear()
    torch.cuda.empty_cache()

    # cfg4: vocab-parallel head over the N ranks, strong scaling (total work fixed)
    hidden, weight, ids = synthetic.cfg4_vocab_parallel(32768, 4096, VOCAB, device)
    b, e = synthetic.shard_bounds(VOCAB, rank, world)
    shard = weight[b:e].contiguous()
    ws = torch.empty(tome_b200.lm_head_workspace_bytes(32768, 4096, e - b), dtype=torch.uint8,
                     device=device)
    packed = torch.zeros((2 * world + 1, 32768), dtype=torch.float32, device=device)
    k4 = max(3, min(args.steps, 5))

    def vp_step():
        box["vp"] = tome_b200.lm_head_logprob_vocab_parallel(
            hidden, shard, b, ids, 1.0, workspace=ws, packed=packed)

    ms, launch = timed(vp_step, k=k4, w=3)
    flops = 2.0 * 32768 * VOCAB * 4096
    extra["cfg4_vocab_parallel"] = {"rows": 32768, "hidden": 4096, "shards": world,
                                    "vocab_per_gpu": e - b, "ms": ms, "scaling": "strong",
                                    "TFLOPs_total": flops / ms / 1e9,
                                    "TFLOPs_per_gpu": flops / ms / 1e9 / world,
                                    "frac_of_measured_bf16_sustained":
                                        flops / ms / 1e9 / world / peaks["bf16_tflops_sustained"],
                                    "collective": "one all_reduce of [2N+1, rows] fp32"}
    # every rank compares what it got for a 64-row sample with the UNSHARDED head (the full
    # weight matrix is the same on every rank: same seed), fp32 matmul + logsumexp in torch
    sel = torch.arange(0, 32768, 512, device=device)
    want_lp, want_lse = head_reference(hidden, weight, ids, 1.0, sel)
    verdict("cfg4_vocab_parallel", {"max_abs_logprob": (box["vp"][0][sel] - want_lp).abs().max(),
                                    "max_abs_lse": (box["vp"][1][sel] - want_lse).abs().max()})
    tome_b200.check_device_status(device)
    return extra, failures


def run_only(args):
    """One kernel in a loop on one GPU, at a chosen row count: the command ncu captures."""
    import torch
    import tome_b200
    from tome_b200 import synthetic
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    if args.only == "selective":
        rows = args.rows or ROWS
        if args.fp32:
            x, ids = synthetic.cfg1_selective_fp32(rows, VOCAB, device)
        else:
            x, ids = synthetic.cfg2_rollout_bf16(rows, VOCAB, device)
        fn = lambda: tome_b200.local_compute_logprobs(x, ids, 1.0)  # noqa: E731
        work, unit = rows * VOCAB * x.element_size() + rows * 8, "GB/s"
    elif args.only in ("full", "sample"):
        rows = args.rows or 2048
        x = torch.randn((rows, args.vocab), device=device, dtype=torch.float32) * 3.0
        if not args.fp32:
            x = x.to(torch.bfloat16)
        if args.only == "full":  # algorithmic bytes: the matrix in and out
            fn = lambda: tome_b200.fused_log_softmax(x, 1.0)  # noqa: E731
            work, unit = 2 * rows * args.vocab * x.element_size(), "GB/s"
        else:
            draws = [0]

            def fn():
                draws[0] += 1
                return tome_b200.sample_topk_logprob(x, 0.7, 20, seed=7, offset=draws[0])

            work, unit = rows * args.vocab * x.element_size(), "GB/s"
    else:
        rows = args.rows or 16384
        hidden, weight, ids = synthetic.cfg3_lm_head(rows, args.hidden, args.vocab, device)
        ws = torch.empty(tome_b200.lm_head_workspace_bytes(rows, args.hidden, args.vocab),
                         dtype=torch.uint8, device=device)
        fn = lambda: tome_b200.lm_head_logprob(hidden, weight, ids, 1.0, workspace=ws)  # noqa: E731
        work, unit = 2.0 * rows * args.vocab * args.hidden, "TFLOP/s"
    sampler = ClockSampler(physical_gpu_index(0))
    total, per = timed_steps(fn, args.steps, args.warmup, lambda: None, sampler)
    tome_b200.check_device_status(device)
    ms = sum(per) / len(per)
    rate = work / ms / (1e6 if unit == "GB/s" else 1e9)
    sp = sorted(per)
    out = {"only": args.only, "rows": rows, "ms": ms, "rate": rate, "unit": unit,
           "ms_first": per[0], "ms_last": per[-1], "ms_min": sp[0], "ms_median": sp[len(sp) // 2],
           "clocks": sampler.summary()}
    if args.only == "selective":  # the timed kernel's result against a torch reduction
        sample = torch.arange(0, rows, max(1, rows // 256), device=device)
        ref = torch.log_softmax(x[sample].float(), dim=-1).gather(
            1, ids[sample].long()[:, None]).squeeze(1)
        out["max_abs_vs_torch"] = float((fn()[sample] - ref).abs().max())
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--skip-extra", action="store_true", help="headline workload only")
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline leg")
    ap.add_argument("--only", choices=["selective", "lmhead", "full", "sample"], default=None,
                    help="profiling aid: run just one kernel's loop (no e2e, extras or CPU leg)")
    ap.add_argument("--rows", type=int, default=None, help="row count for --only (small cases)")
    ap.add_argument("--hidden", type=int, default=1024, help="hidden size for --only lmhead")
    ap.add_argument("--vocab", type=int, default=VOCAB, help="vocabulary (shard) size for --only")
    ap.add_argument("--fp32", action="store_true", help="fp32 logits for --only selective / full / sample")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args, int(os.environ.get("RANK", "0")))
        return
    if args.only is not None:
        run_only(args)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus != world and world == 1 and args.gpus > 1:
        # launched without torchrun: re-launch one rank per GPU on this node
        import subprocess
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port",
               os.environ.get("MASTER_PORT", "29531"), os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    run_ours(args)


if __name__ == "__main__":
    main()
