#!/usr/bin/env python
"""Headline benchmark: bf16 -> f32 pg_gemm_ex at M = N = K = 8192 on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one pass of the hot path over the whole 8192^3 product.  With N > 1 the product
is partitioned by N-column shards of B and C (rank r owns columns [r*8192/N, (r+1)*8192/N)),
A is replicated, and there is no collective in the timed path: total work is fixed, so the
scaling is "strong".  Rank 0 prints ONE JSON line.

Inputs are synthetic (seeded N(0,1) rounded to bf16, as the configuration specifies); A, B and
C together are 512 MiB, larger than the 126 MB L2, so consecutive timed launches cannot be
served from cache.

Timing: regions of --steps launches each run back to back, without a host synchronisation between them, for
--window seconds (default 3).  Every region is timed on the device with CUDA events (maximum over ranks);
`ms_per_step` and `value` are the MEDIAN region — the rate the kernel holds under the power cap — while the best
region (the first ones, on a cool GPU) is reported beside it as `burst`.  The SM clock, power and throttle reasons
are sampled through NVML over the same window, so that the line separates tensor-pipe utilisation from clock.

`--impl reference` times picograd's own CPU implementation of the same call (the unmodified
library compiled into oracle/_ref when that build travelled with the repository, else the C
restatement in oracle/) on the host cores, each step a bounded row-slab of the same product.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

M = N = K = 8192
FLOPS = 2.0 * M * N * K
NOMINAL_BF16_TFLOPS = 2250.0


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
        except Exception:
            pass
    return 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples the SM clock and the clock-event (throttle) reasons through NVML from a background
    thread while the timed region runs (read-only queries, about one per millisecond)."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.index = index
        self.samples = []          # (time, sm_mhz, reasons bitmask)
        self.stop_flag = False
        self.thread = None
        self.max_mhz = None
        self.err = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
        except Exception as e:      # no NVML: report that instead of clocks
            self.err = f"NVML unavailable: {e}"

    def _poll(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    why = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    why = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                try:
                    watts = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                except Exception:
                    watts = None
                self.samples.append((time.time(), float(mhz), int(why), watts))
            except Exception as e:
                self.err = str(e)
                break
            time.sleep(0.0005)

    def stop(self, t0, t1):
        self.stop_flag = True
        if self.thread:
            self.thread.join(timeout=1)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [self.err or "no samples"]}
        rows = [x for x in self.samples if t0 <= x[0] <= t1] or self.samples
        mask = 0
        for x in rows:
            mask |= x[2]
        mhz = sorted(x[1] for x in rows)
        watts = [x[3] for x in rows if x[3] is not None]
        pick = lambda q: mhz[min(len(mhz) - 1, int(q * len(mhz)))]
        return {"sm_mhz": statistics.median(mhz), "sm_min_mhz": mhz[0], "sm_p10_mhz": pick(0.1), "sm_p90_mhz": pick(0.9),
                "sm_max_mhz": self.max_mhz, "power_w": statistics.median(watts) if watts else None,
                "reasons": sorted(n for b, n in self.REASONS.items() if mask & b), "samples": len(rows),
                "window_s": round(t1 - t0, 3)}


# ------------------------------------------------------------------------------------------
# CPU arm (reference implementation on the host cores)
# ------------------------------------------------------------------------------------------
def cpu_gemm_fn():
    """(callable(a_bits, b_bits) -> C, kind, threads)."""
    import oracle_lib
    ref = oracle_lib.reference()
    if ref is not None:
        return (lambda a, b: ref.gemm_ex(oracle_lib.BF16, a, b)), "reference", ref.threads()
    if not os.path.exists(oracle_lib.oracle_path()):
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "oracle"], stdout=subprocess.DEVNULL)
    o = oracle_lib.oracle()
    return (lambda a, b: o.gemm_ex(oracle_lib.BF16, a, b)), "port", o.threads()


def cpu_time_rows(fn, a, b, rows):
    t = time.perf_counter()
    fn(a[:rows], b)
    return time.perf_counter() - t


def cpu_baseline(a, b, budget_s=15.0):
    """Times the CPU implementation on a row-slab of the same product sized for ~budget_s."""
    fn, kind, threads = cpu_gemm_fn()
    # size the slab in two steps (small slabs run at a lower rate per row: thread start-up, cold caches)
    rows, t = 64, cpu_time_rows(fn, a, b, 64)
    for _ in range(2):
        want = int(min(M, max(rows, rows * budget_s / max(t, 1e-3)))) // 8 * 8
        if want <= rows * 1.5:
            break
        rows = max(8, want)
        t = cpu_time_rows(fn, a, b, rows)
    tf = 2.0 * rows * N * K / t / 1e12
    return {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": kind,
            "sample": f"rows [0,{rows}) of the 8192^3 bf16 product ({rows}x8192x8192), one run, {t:.2f} s"}


def run_reference_arm(args, rank):
    if rank != 0:
        return
    import workloads as wl
    a, b = wl.config2(M, N, K)
    fn, kind, threads = cpu_gemm_fn()
    t = cpu_time_rows(fn, a, b, 64)
    rows = int(min(M, max(8, 64 * 2.0 / max(t, 1e-3))))     # ~2 s per step
    rows = max(8, rows // 8 * 8)
    for _ in range(args.warmup):
        cpu_time_rows(fn, a, b, rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn(a[:rows], b)
    dt = (time.perf_counter() - t0) / args.steps
    tf = 2.0 * rows * N * K / dt / 1e12
    line = {
        "impl": "reference", "metric": "bf16->f32 GEMM TFLOP/s at M=N=K=8192", "value": tf, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "pg_gemm_ex(PG_DTYPE_BF16) M=N=K=8192, A,B~N(0,1) rounded to bf16, seed 1, C f32",
                   "step": f"row-slab [0,{rows}) of the product per step on the host cores"},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": kind,
                         "sample": f"{rows}x8192x8192 per step, {args.steps} steps"},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
FLOP_PER_CLK_PER_SM = 8192.0      # dense bf16/f16 multiply-adds x 2 per SM per clock (2.25 PFLOP/s = 148 SMs x 8192 x 1.855 GHz)


def hbm_peak_gbs():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def profile_traffic(name, key="dram_bytes_per_launch"):
    """DRAM bytes of one launch as recorded in the committed ncu summary profiles/<name> (a line `<key> = <number>`);
    (None, None) when the summary does not hold one."""
    path = os.path.join(ROOT, "profiles", name)
    try:
        for line in open(path):
            if line.strip().startswith(key):
                return float(line.split("=")[1].split()[0]), f"ncu capture summarised in profiles/{name}"
    except Exception:
        pass
    return None, None


def timed_regions(torch, dist, step, steps, window_s, max_regions=3000):
    """Runs regions of `steps` calls of step() back to back for about window_s seconds.  Returns the per-region
    times in ms (max over ranks), and the wall-clock interval of the window on this rank."""
    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def reduce_max(vals):
        if dist is None:
            return [float(v) for v in vals]
        t = torch.tensor(vals, device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    # one calibration region (also a warm-up) to choose the number of regions
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    c0.record()
    for _ in range(steps):
        step()
    c1.record()
    torch.cuda.synchronize()
    t_cal = reduce_max([c0.elapsed_time(c1)])[0]
    regions = int(min(max_regions, max(3, math.ceil(window_s * 1e3 / max(t_cal, 1e-3)))))
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(regions + 1)]
    barrier()
    w0 = time.time()
    evs[0].record()
    for r in range(regions):
        for _ in range(steps):
            step()
        evs[r + 1].record()
    torch.cuda.synchronize()
    w1 = time.time()
    ms = reduce_max([evs[r].elapsed_time(evs[r + 1]) for r in range(regions)])
    barrier()
    return ms, (w0, w1)


def summarise(ms, steps, work_per_step, unit_scale):
    """Median / best / whole-window rates from per-region times; work_per_step in flops (or bytes), unit_scale
    1e12 for TFLOP/s (1e9 for GB/s)."""
    med, best = statistics.median(ms), min(ms)
    srt = sorted(ms)
    rate = lambda t_ms: work_per_step * steps / (t_ms * 1e-3) / unit_scale
    return {"median_ms_per_step": med / steps, "best_ms_per_step": best / steps, "first_ms_per_step": ms[0] / steps,
            "p10_ms_per_step": srt[int(0.1 * len(srt))] / steps, "p90_ms_per_step": srt[min(len(srt) - 1, int(0.9 * len(srt)))] / steps,
            "regions": len(ms), "steps_per_region": steps, "window_ms": sum(ms),
            "median_rate": rate(med), "best_rate": rate(best), "window_rate": work_per_step * steps * len(ms) / (sum(ms) * 1e-3) / unit_scale}


def tensor_records(summary, clocks, flops_per_gpu_step, world, burst_peak, sustained_peak, src):
    """`roofline` (median region against the sustained peak: both are seconds-long loops under the power cap),
    `burst` (best region against the burst peak) and `sustained` (whole window with the sampled clock)."""
    per_gpu = lambda r: r / world
    roof = {"bound": "tensor", "achieved": per_gpu(summary["median_rate"]), "peak": sustained_peak, "unit": "TFLOP/s",
            "frac": per_gpu(summary["median_rate"]) / sustained_peak,
            "peak_source": f"{src} sustained bf16 (seconds-long loop under the power cap, like the timed window)"}
    burst = {"achieved": per_gpu(summary["best_rate"]), "peak": burst_peak, "unit": "TFLOP/s",
             "frac": per_gpu(summary["best_rate"]) / burst_peak, "ms_per_step": summary["best_ms_per_step"],
             "peak_source": f"{src} burst bf16 (best of a few launches on a cool GPU, like the best region)"}
    sus = {"achieved": per_gpu(summary["window_rate"]), "peak": sustained_peak, "unit": "TFLOP/s",
           "frac": per_gpu(summary["window_rate"]) / sustained_peak, "seconds": summary["window_ms"] * 1e-3}
    mhz = clocks.get("sm_mhz") if clocks else None
    if mhz:
        cyc = summary["median_ms_per_step"] * 1e-3 * mhz * 1e6
        floor = flops_per_gpu_step / (148 * FLOP_PER_CLK_PER_SM)
        sus.update({"sm_mhz_median": mhz, "cycles_per_step": cyc, "tensor_pipe_floor_cycles": floor,
                    "pipe_utilisation_at_sampled_clock": floor / cyc,
                    "note": "rate = pipe utilisation x clock: time x median sampled SM clock against 148 SMs x 8192 flop/clk"})
    return roof, burst, sus


def apply_options(pg, args):
    for o in args.opt:
        name, _, val = o.partition("=")
        pg.set_option(name, int(val))


def run_ours(args, rank, world):
    import torch
    import workloads as wl
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import picograd_b200 as pg
    from picograd_b200 import sharding
    pg.pg_set_device(local)
    apply_options(pg, args)

    if N % world or M % world:
        raise SystemExit(f"--gpus {world} does not divide N={N}")
    n_loc = N // world
    c0 = rank * n_loc
    m_loc, r0 = M // world, rank * (M // world)
    # every rank draws the same seeded matrices and keeps its column shard of B
    a_bits, b_bits = wl.config2(M, N, K)
    b_loc = np.ascontiguousarray(b_bits[:, c0:c0 + n_loc])
    a_host = torch.from_numpy(a_bits.view(np.int16)).pin_memory()
    b_host = torch.from_numpy(b_loc.view(np.int16)).pin_memory()
    c_host = torch.empty((M, n_loc), dtype=torch.float32).pin_memory()
    a_dev = a_host.cuda().view(torch.bfloat16)
    b_dev = b_host.cuda().view(torch.bfloat16)
    c_dev = torch.empty((M, n_loc), dtype=torch.float32, device="cuda")

    def step():
        pg.pg_gemm_ex(pg.PG_DTYPE_BF16, M, n_loc, K, a_dev, K, b_dev, n_loc, c_dev, n_loc)

    for _ in range(max(args.warmup, 3)):
        step()
    pg.pg_dev_sync()
    kernel_path = pg.last_path()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.02)
    launches0 = pg.launch_count()
    ms, (w0, w1) = timed_regions(torch, dist, step, args.steps, args.window)
    launches = pg.launch_count() - launches0          # includes the calibration region
    pg.pg_dev_sync()                                   # surfaces a kernel-side failure, if any
    clocks = sampler.stop(w0, w1) if rank == 0 else None
    summ = summarise(ms, args.steps, FLOPS, 1e12)

    # ---- end to end through the reference-facing call with HOST buffers, every step: H2D of the operands, the
    # product, D2H of C.  One GPU: pg_gemm_ex with host pointers (staged and pipelined inside the call).  N GPUs:
    # each rank uploads 1/N of A's rows and its column shard of B, the ranks all-gather A over NVLink, each
    # multiplies its shard and sends its C shard back.
    e2e_steps = max(2, min(args.steps, 5))
    if world == 1:
        e2e_call = lambda: pg.pg_gemm_ex_host(pg.PG_DTYPE_BF16, M, n_loc, K, a_host, K, b_host, n_loc, c_host, n_loc)
        h2d, d2h = int((M * K + K * n_loc) * 2), int(M * n_loc * 4)
    else:
        a_rows_host = torch.from_numpy(np.ascontiguousarray(a_bits[r0:r0 + m_loc]).view(np.int16)).pin_memory()
        sharded = sharding.HostShardedGemm(pg.PG_DTYPE_BF16, M, N, K)
        e2e_call = lambda: sharded(a_rows_host, b_host, c_host)
        h2d, d2h = int(sharded.h2d_bytes), int(sharded.d2h_bytes)
    e2e_call()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_call()
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if dist is not None:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_tflops = FLOPS / e2e_s / 1e12
    # the host-buffer result against the device-resident one: same bits when both products take the same K order
    # per element (option k_serpentine = 0), else the normwise difference (the strips of the staged product and
    # the resident product each sum K up or down by their own tile walk: rounding only)
    step()
    torch.cuda.synchronize()
    same = bool(torch.equal(c_dev[:64].cpu(), c_host[:64]))
    diff = float((c_dev[:64].cpu().double() - c_host[:64].double()).norm() / c_host[:64].double().norm())

    # ---- the exchange a caller pays only when it wants all of C on every device (excluded from `value`)
    collective = None
    if world > 1:
        full = torch.empty((M, N), dtype=torch.float32, device="cuda")
        staging = torch.empty((world, M, n_loc), dtype=torch.float32, device="cuda")
        for _ in range(3):
            sharding.gather_columns(c_dev, N, out=full, staging=staging)
        torch.cuda.synchronize()
        dist.barrier()
        iters = 10
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3 * iters)]
        for i in range(iters):
            ev[3 * i].record()
            dist.all_gather_into_tensor(staging, c_dev)
            ev[3 * i + 1].record()
            pg.pg_gather_relayout(staging, full, world, M, n_loc, N)
            ev[3 * i + 2].record()
        torch.cuda.synchronize()
        t_ag = statistics.median(ev[3 * i].elapsed_time(ev[3 * i + 1]) for i in range(iters))
        t_rl = statistics.median(ev[3 * i + 1].elapsed_time(ev[3 * i + 2]) for i in range(iters))
        t = torch.tensor([t_ag, t_rl], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_ag, t_rl = (float(x) for x in t.tolist())
        ok = bool(torch.equal(full[:, c0:c0 + n_loc], c_dev))
        hbm, hsrc = hbm_peak_gbs()
        # The same result without a collective: the GEMM kernel stores every finished tile of its shard into the full
        # C of every rank (peer memory mapped over CUDA IPC), the NVLink transfer overlapping the product.
        fused = None
        try:
            peers = sharding.PeerMatrix(M, N)
            for _ in range(3):
                sharding.scatter_gemm(pg.PG_DTYPE_BF16, a_dev, b_dev, peers, c0)
            scatter_path = pg.last_path()
            sharding.finish_scatter(peers)
            same_as_gather = bool(torch.equal(peers.local, full))
            times = []
            for _ in range(iters):
                dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                sharding.scatter_gemm(pg.PG_DTYPE_BF16, a_dev, b_dev, peers, c0)
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
            t = torch.tensor([statistics.median(times)], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_sc = float(t.item())
            peers.close()
            out_bytes = M * n_loc * 4 * (world - 1)
            fused = {"op": "pg_b200_gemm_ex_scatter: product + stores of the shard into every rank's row-major C, one kernel",
                     "ms": t_sc, "kernel": scatter_path, "nvlink_out_bytes_per_gpu": int(out_bytes),
                     "nvlink_out_GBps_per_gpu": out_bytes / (t_sc * 1e-3) / 1e9,
                     "floor_ms": max(out_bytes / 770e9 * 1e3, summ["median_ms_per_step"]),
                     "floor": "the slower of the product alone and the shard's bytes to the other ranks at the measured "
                              "770 GB/s per direction",
                     "equals_gathered_result": same_as_gather}
        except Exception as e:                      # e.g. no peer access between the GPUs of this box
            fused = {"unavailable": str(e)[:200]}
        collective = {
            "op": "NCCL all-gather of the C column shards into [G][M][N/G] + re-layout kernel to row-major [M][N]",
            "all_gather_ms": t_ag, "relayout_ms": t_rl, "bytes_per_gpu": int(M * N * 4),
            "all_gather_busbw_GBps": M * N * 4 * (world - 1) / world / (t_ag * 1e-3) / 1e9,
            "nvlink_reference_GBps": {"peer_copy_per_direction": 770.0, "allreduce_busbw_8_ranks_1GiB": 725.0},
            "relayout_GBps": 2.0 * M * N * 4 / (t_rl * 1e-3) / 1e9, "relayout_frac_of_hbm": 2.0 * M * N * 4 / (t_rl * 1e-3) / 1e9 / hbm,
            "hbm_peak_source": hsrc, "own_shard_intact": ok, "included_in_value": False,
            "product_plus_gather_ms": summ["median_ms_per_step"] + t_ag + t_rl, "fused_scatter": fused}

    if rank == 0:
        burst_peak, sustained_peak, src = measured_peaks()
        roof, burst, sus = tensor_records(summ, clocks, FLOPS / world, world, burst_peak, sustained_peak, src)
        traffic, tsrc = profile_traffic("tc_gemm_kernel_bf16_8192.md") if world == 1 else (None, None)
        roof.update({"traffic": traffic, "traffic_source": tsrc, "algorithmic_bytes": 536870912})
        line = {
            "metric": "bf16->f32 GEMM TFLOP/s at M=N=K=8192", "value": summ["median_rate"], "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": summ["median_ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "pg_gemm_ex(PG_DTYPE_BF16) M=N=K=8192, A,B~N(0,1) rounded to bf16, seed 1, C f32",
                       "partition": f"N-column shards of B and C, {n_loc} columns per GPU, A replicated, no collective",
                       "l2": "A+B+C = 512 MiB per step > 126 MB L2 (inputs larger than L2, no flush needed)",
                       "kernel": kernel_path, "options": args.opt,
                       "timing": f"median of {summ['regions']} back-to-back regions of {args.steps} launches "
                                 f"({summ['window_ms'] / 1e3:.2f} s of GPU time), CUDA events, max over ranks"},
            "timing": summ,
            "pct_of_nominal_peak": 100.0 * summ["median_rate"] / (NOMINAL_BF16_TFLOPS * world),
            "pct_of_nominal_peak_burst": 100.0 * summ["best_rate"] / (NOMINAL_BF16_TFLOPS * world),
            "roofline": roof, "burst": burst, "sustained": sus,
            "e2e": {"value": e2e_tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
                    "path": "pg_gemm_ex with host pointers" if world == 1 else
                            "per rank: H2D of M/N rows of A + its B shard, NCCL all-gather of A, product, D2H of its C shard"},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "staged_equals_resident": same, "staged_vs_resident_relerr": diff,
        }
        if collective:
            line["collective"] = collective
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(a_bits, b_bits)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_other_config(args, rank, world):
    """Configurations 1, 3a, 3b, 4, 5 (and the Linear / square helpers), device-resident: one JSON line with the
    median region time of a whole pass, its rate against the roofline that bounds it, and the sampled clocks.
    Configuration 4 shards by batch over --gpus N (no collective: every rank owns whole outputs); the others run on
    one GPU."""
    import torch
    import workloads as wl
    from gpu_util import to_dev
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        if args.config not in ("4", "4-fused"):
            raise SystemExit("--gpus N > 1 is for the headline configuration and for configuration 4 (batch shards)")
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import picograd_b200 as pg
    from picograd_b200 import ops, sharding
    pg.pg_set_device(local)
    apply_options(pg, args)
    hbm_peak, hbm_src = hbm_peak_gbs()
    burst, sustained, src = measured_peaks()
    cfg = args.config
    bound, profile = "tensor", None
    if cfg == "1":
        a, b = wl.config1(512)
        ad, bd = to_dev(a, wl.F32), to_dev(b, wl.F32)
        fn = lambda: pg.pg_matmul(ad, bd)
        # the same call as a C caller makes it: descriptors built once, the output allocated once
        from picograd_b200 import _lib, backend as _be
        import ctypes as _C
        c1 = torch.empty((512, 512), dtype=torch.float32, device="cuda")
        _da, _db, _do = _be._desc(ad), _be._desc(bd), _be._desc(c1)
        c_fn = lambda: _lib.lib.pg_b200_matmul(_C.byref(_da), _C.byref(_db), _C.byref(_do))
        flops, byts, name, dt = 2.0 * 512 ** 3, 3 * 512 * 512 * 4, "pg_matmul f32 512^3", "f32"
        bound, profile = "launch", "sgemm_nn_pipe_kernel_f32_512.md"
    elif cfg == "square":
        n = args.size
        a, b = wl.config2(n, n, n)
        ad, bd = to_dev(a, wl.BF16), to_dev(b, wl.BF16)
        c = torch.empty((n, n), dtype=torch.float32, device="cuda")
        fn = lambda: pg.pg_gemm_ex(wl.BF16, n, n, n, ad, n, bd, n, c, n)
        flops, byts, name, dt = 2.0 * n ** 3, 2 * n * n * 2 + n * n * 4, f"pg_gemm_ex bf16 {n}^3", "bf16"
    elif cfg in ("3a", "3b", "shard8"):
        m, n, k = {"3a": (4096, 14336, 4096), "3b": (16, 4096, 4096), "shard8": (8192, 1024, 8192)}[cfg]
        mk = wl.config3 if cfg != "shard8" else wl.config2
        code = wl.F16 if cfg != "shard8" else wl.BF16
        a, b = mk(m, n, k)
        ad, bd = to_dev(a, code), to_dev(b, code)
        c = torch.empty((m, n), dtype=torch.float32, device="cuda")
        fn = lambda: pg.pg_gemm_ex(code, m, n, k, ad, k, bd, n, c, n)
        from picograd_b200 import _lib
        _pa, _pb, _pc = ad.data_ptr(), bd.data_ptr(), c.data_ptr()
        c_fn = lambda: _lib.lib.pg_b200_gemm_ex(code, m, n, k, _pa, k, _pb, n, _pc, n)
        dt = "f16" if code == wl.F16 else "bf16"
        flops, byts, name = 2.0 * m * n * k, (m * k + k * n) * 2 + m * n * 4, f"pg_gemm_ex {dt} {m}x{n}x{k}"
        if cfg == "3b":
            bound, profile = "hbm", "tc_gemm_kernel_f16_16x4096x4096.md"
        if cfg == "shard8":
            profile = "tc_gemm_kernel_bf16_8192x1024x8192.md"
    elif cfg in ("4", "4-fused"):
        q, kt, v = wl.config4()
        b0, bc = sharding.batch_shards(64, world)[rank]
        qd, ktd, vd = (to_dev(x[b0:b0 + bc], wl.BF16) for x in (q, kt, v))
        if cfg == "4-fused":
            # the chain pg_bmm -> softmax -> cast -> pg_bmm in one kernel; the f32 scores and the bf16 probabilities
            # never reach HBM, so the algorithmic bytes are Q, Kt, V in and O out
            fn = lambda: pg.pg_attention_bmm(qd, ktd, vd)
            byts = 3 * 64 * 2048 * 128 * 2 + 64 * 2048 * 128 * 4
            name = "pg_attention_bmm (QK^T -> softmax -> PV in one kernel), bf16 [64,2048,128]"
            profile = "attn_fused_kernel_bf16_64x2048x128.md"
        else:
            def fn():
                s = pg.pg_bmm(qd, ktd)
                p16 = ops.softmax_rows(s, out16=torch.bfloat16, want_f32=False)[1]
                pg.pg_bmm(p16, vd)
            byts = 1140850688 + 637534208
            name = "pg_bmm QK^T -> softmax -> PV, bf16 [64,2048,128]"
            bound, profile = "hbm", "bmm_attention_shaped_bf16.md"
        flops, dt = 2 * 2.0 * 64 * 2048 * 2048 * 128, "bf16"
        if world > 1:
            name += f", batch shards of {bc} per GPU, no collective"
    elif cfg in ("linear", "linear-unfused"):
        # nn/nn.c:46-96 (Linear forward) at the first layer of configuration 5, GELU instead of ReLU,
        # a bf16 copy of the output for the next layer: one kernel, or GEMM + a separate GELU/cast pass
        m, k, n = 8192, 4096, 16384
        x, w1, _ = wl.config5()
        xd, w1d = to_dev(x, wl.BF16), to_dev(w1, wl.BF16)
        bias = torch.linspace(-1, 1, n, device="cuda")
        c = torch.empty((m, n), dtype=torch.float32, device="cuda")
        c16 = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        if cfg == "linear":
            fn = lambda: pg.pg_gemm_fused_ex(wl.BF16, m, n, k, xd, k, w1d, n, c, n, bias, pg.PG_ACT_GELU, c16, n)
        else:
            def fn():
                pg.pg_gemm_fused_ex(wl.BF16, m, n, k, xd, k, w1d, n, c, n, bias, pg.PG_ACT_NONE)
                ops.gelu(c, out16=torch.bfloat16, want_f32=True)
        flops, byts = 2.0 * m * n * k, (m * k + k * n) * 2 + m * n * 6 + n * 4
        name, dt = f"Linear forward bf16 {m}x{k} -> {n}, bias + GELU + bf16 copy ({cfg})", "bf16"
    else:
        x, w1, w2 = wl.config5()
        xd, w1d, w2d = (to_dev(t, wl.BF16) for t in (x, w1, w2))
        dy = torch.ones((8192, 4096), dtype=torch.float32, device="cuda")     # loss = sum(y): its gradient, made once
        h = torch.empty((8192, 16384), dtype=torch.float32, device="cuda")
        a16 = torch.empty((8192, 16384), dtype=torch.bfloat16, device="cuda")
        fn = lambda: mlp_step(pg, ops, wl, xd, w1d, w2d, dy, h, a16)
        flops = 6 * 2.0 * 8192 * 4096 * 16384
        byts = None
        name, dt = "MLP step 8192x4096 -> 16384 -> 4096, forward + backward", "bf16"
        profile = "config5_mlp_step_launches.md"
    for _ in range(max(args.warmup, 3)):
        fn()
    pg.pg_dev_sync()
    kernel_path = pg.last_path()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.02)
    l0 = pg.launch_count()
    ms, (w0, w1) = timed_regions(torch, dist, fn, args.steps, args.window)
    per_step_launches = (pg.launch_count() - l0) / ((len(ms) + 1) * args.steps)
    pg.pg_dev_sync()
    clocks = sampler.stop(w0, w1) if rank == 0 else None
    summ = summarise(ms, args.steps, flops, 1e12)
    if rank != 0:
        dist.barrier()
        dist.destroy_process_group()
        return
    line = {"metric": "time of one pass", "config": {"workload": name, "config": cfg, "kernel": kernel_path, "options": args.opt},
            "ms_per_step": summ["median_ms_per_step"], "value": summ["median_rate"], "unit": "TFLOP/s", "dtype": dt,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "data": "synthetic", "higher_is_better": True,
            "scaling": "strong", "gpu_launches_per_step": per_step_launches, "timing": summ, "clocks": clocks}
    if bound == "tensor":
        roof, bst, sus = tensor_records(summ, clocks, flops / world, world, burst, sustained, src)
        line.update({"roofline": roof, "burst": bst, "sustained": sus})
    elif byts:
        gbs = byts / summ["median_ms_per_step"] / 1e6 / world
        line["roofline"] = {"bound": "hbm" if bound == "hbm" else "hbm (launch-bound shape)", "achieved": gbs, "peak": hbm_peak,
                            "unit": "GB/s", "frac": gbs / hbm_peak, "peak_source": f"{hbm_src} copy bandwidth",
                            "best_GBps": byts / summ["best_ms_per_step"] / 1e6 / world}
    if "roofline" in line:
        traffic, tsrc = profile_traffic(profile) if profile else (None, None)
        line["roofline"].update({"traffic": traffic, "traffic_source": tsrc, "algorithmic_bytes": byts})
    if cfg in ("1", "3b"):
        # launch-bound shapes: the same step replayed from a CUDA graph (20 launches per replay) — device time
        # without the CPU side of the calls
        from picograd_b200 import _lib
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            _lib.lib.pg_b200_set_stream(side.cuda_stream)
            fn(); side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(20):
                    fn()
            graph.replay(); side.synchronize()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record(side)
            for _ in range(50):
                graph.replay()
            g1.record(side); side.synchronize()
            # the bare C-ABI call in a loop (no Python wrapper around it): what a C caller's eager loop costs
            for _ in range(200):
                c_fn()
            side.synchronize()
            n_c = 5000
            c0e, c1e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            c0e.record(side)
            for _ in range(n_c):
                c_fn()
            c1e.record(side); side.synchronize()
            line["c_abi_eager_ms_per_step"] = c0e.elapsed_time(c1e) / n_c
        _lib.lib.pg_b200_set_stream(None)
        gms = g0.elapsed_time(g1) / 1000
        line["graph_replay_ms_per_step"] = gms
        line["graph_replay_GBps"] = byts / gms / 1e6
        line["graph_replay_frac_of_measured_hbm"] = byts / gms / 1e6 / hbm_peak
        line["graph_replay_TFLOPs"] = flops / gms / 1e9
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def mlp_step(pg, ops, wl, xd, w1d, w2d, dy, h, a16):
    """Configuration 5, one step: forward (first layer fused: h = x W1 in f32, which the backward pass reads, and
    a16 = bf16(gelu(h)) from the same kernel), then the backward pass of loss = sum(y)."""
    import torch  # noqa: F401
    pg.pg_gemm_fused_ex(wl.BF16, 8192, 16384, 4096, xd, 4096, w1d, 16384, h, 16384, None,
                        pg.PG_ACT_GELU | pg.PG_ACT_COPY_ONLY, a16, 16384)
    y = pg.pg_matmul(a16, w2d)
    da, dw2 = pg.pg_matmul_backward(a16, w2d, dy)
    # the GELU node's backward (dh = da * gelu'(h)) happens inside the split that feeds the first layer's backward
    dx, dw1, _ = pg.pg_matmul_backward_act(xd, w1d, da, pg.PG_ACT_GELU, h)
    return y, da, dw2, dx, dw1


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20, help="launches per timed region")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--window", type=float, default=3.0,
                    help="seconds of GPU time the back-to-back timed regions should add up to")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--config", default="2",
                    choices=["1", "2", "3a", "3b", "4", "4-fused", "5", "linear", "linear-unfused", "square", "shard8"],
                    help="2 (default) is the headline metric; the others time the remaining configurations "
                         "(device-resident) and print one JSON line each; square = bf16 pg_gemm_ex of --size cubed, "
                         "shard8 = the per-GPU shard of the headline at 8 GPUs (8192x1024x8192) on one GPU")
    ap.add_argument("--size", type=int, default=4096, help="edge of --config square")
    ap.add_argument("--opt", action="append", default=[], metavar="NAME=VALUE",
                    help="library option for an A/B run (pg_b200_set_option), e.g. --opt stream_k=0 --opt pdl=0")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1 and args.gpus > 1:
        # launched without torchrun: re-launch ourselves with one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 1000), os.path.abspath(__file__),
               "--gpus", str(args.gpus), "--steps", str(args.steps), "--warmup", str(args.warmup), "--impl", args.impl,
               "--window", str(args.window), "--config", args.config, "--size", str(args.size)]
        for o in args.opt:
            cmd += ["--opt", o]
        if args.no_cpu_baseline:
            cmd.append("--no-cpu-baseline")
        sys.exit(subprocess.call(cmd))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.config != "2":
        run_other_config(args, rank, world)
        return
    run_ours(args, rank, world)


if __name__ == "__main__":
    main()
