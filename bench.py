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

`--impl reference` times picograd's own CPU implementation of the same call (the unmodified
library compiled into oracle/_ref when that build travelled with the repository, else the C
restatement in oracle/) on the host cores, each step a bounded row-slab of the same product.
"""
import argparse
import json
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
                self.samples.append((time.time(), float(mhz), int(why)))
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
        for _, _, why in rows:
            mask |= why
        return {"sm_mhz": statistics.median(m for _, m, _ in rows), "sm_min_mhz": min(m for _, m, _ in rows),
                "sm_max_mhz": self.max_mhz, "reasons": sorted(n for b, n in self.REASONS.items() if mask & b),
                "samples": len(rows)}


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
    pg.pg_set_device(local)

    if N % world:
        raise SystemExit(f"--gpus {world} does not divide N={N}")
    n_loc = N // world
    c0 = rank * n_loc
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

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    pg.pg_dev_sync()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.02)
    barrier()
    launches0 = pg.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.time()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    t_wall1 = time.time()
    launches = pg.launch_count() - launches0
    ms = e0.elapsed_time(e1)
    pg.pg_dev_sync()                                   # surfaces a kernel-side failure, if any
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    ms_per_step = ms / args.steps
    tflops = FLOPS / (ms_per_step * 1e-3) / 1e12

    # end to end through the reference-facing call with HOST buffers: H2D of A and the B shard,
    # the GEMM, D2H of the C shard, every step
    e2e_steps = max(2, min(args.steps, 5))
    pg.pg_gemm_ex_host(pg.PG_DTYPE_BF16, M, n_loc, K, a_host, K, b_host, n_loc, c_host, n_loc)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        pg.pg_gemm_ex_host(pg.PG_DTYPE_BF16, M, n_loc, K, a_host, K, b_host, n_loc, c_host, n_loc)
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if dist is not None:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_tflops = FLOPS / e2e_s / 1e12

    # spot-check the timed result against the device result of the staged call (same bytes)
    same = bool(torch.equal(c_dev[:64].cpu(), c_host[:64]))

    if rank == 0:
        burst, sustained, src = measured_peaks()
        line = {
            "metric": "bf16->f32 GEMM TFLOP/s at M=N=K=8192", "value": tflops, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "pg_gemm_ex(PG_DTYPE_BF16) M=N=K=8192, A,B~N(0,1) rounded to bf16, seed 1, C f32",
                       "partition": f"N-column shards of B and C, {n_loc} columns per GPU, A replicated, no collective",
                       "l2": "A+B+C = 512 MiB per step > 126 MB L2 (inputs larger than L2, no flush needed)",
                       "kernel": pg.last_path()},
            "pct_of_nominal_peak": 100.0 * tflops / (NOMINAL_BF16_TFLOPS * world),
            "roofline": {"bound": "tensor", "achieved": tflops / world, "peak": burst, "unit": "TFLOP/s",
                         "frac": tflops / world / burst,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at this
                         # size, from the ncu capture summarised in profiles/tc_gemm_kernel_bf16_8192.md
                         "traffic": 1.305e9 if world == 1 else None, "algorithmic_bytes": 536870912 // 1,
                         "peak_source": f"{src} burst bf16 (kernel timed alone, back to back)",
                         "frac_of_sustained": tflops / world / sustained},
            "e2e": {"value": e2e_tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": int((M * K + K * n_loc) * 2),
                    "d2h_bytes_per_step": int(M * n_loc * 4), "ms_per_step": e2e_s * 1e3, "steps": e2e_steps},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "staged_equals_resident": same,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(a_bits, b_bits)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_other_config(args):
    """Configurations 1, 3a, 3b, 4, 5 on one GPU, device-resident: one JSON line with the time of a
    whole pass, the flop rate, and the HBM rate for the HBM-bound ones."""
    import torch
    import workloads as wl
    from gpu_util import to_dev
    import picograd_b200 as pg
    from picograd_b200 import ops
    torch.cuda.set_device(0)
    pg.pg_set_device(0)
    hbm_peak = 6549.1
    try:
        hbm_peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        pass
    burst, sustained, src = measured_peaks()
    cfg = args.config
    if cfg == "1":
        a, b = wl.config1(512)
        ad, bd = to_dev(a, wl.F32), to_dev(b, wl.F32)
        fn = lambda: pg.pg_matmul(ad, bd)
        flops, byts, name, dt = 2.0 * 512 ** 3, 3 * 512 * 512 * 4, "pg_matmul f32 512^3", "f32"
    elif cfg in ("3a", "3b"):
        m, n, k = (4096, 14336, 4096) if cfg == "3a" else (16, 4096, 4096)
        a, b = wl.config3(m, n, k)
        ad, bd = to_dev(a, wl.F16), to_dev(b, wl.F16)
        c = torch.empty((m, n), dtype=torch.float32, device="cuda")
        fn = lambda: pg.pg_gemm_ex(wl.F16, m, n, k, ad, k, bd, n, c, n)
        flops, byts, name, dt = 2.0 * m * n * k, (m * k + k * n) * 2 + m * n * 4, f"pg_gemm_ex f16 {m}x{n}x{k}", "f16"
    elif cfg == "4-fused":
        # configuration 4 as one call: the chain pg_bmm -> softmax -> cast -> pg_bmm in one kernel; the f32
        # scores and the bf16 probabilities never reach HBM, so the algorithmic bytes are Q, Kt, V in and O out
        q, kt, v = wl.config4()
        qd, ktd, vd = (to_dev(x, wl.BF16) for x in (q, kt, v))
        fn = lambda: pg.pg_attention_bmm(qd, ktd, vd)
        flops = 2 * 2.0 * 64 * 2048 * 2048 * 128
        byts = 3 * 64 * 2048 * 128 * 2 + 64 * 2048 * 128 * 4
        name, dt = "pg_attention_bmm (QK^T -> softmax -> PV in one kernel), bf16 [64,2048,128]", "bf16"
    elif cfg == "4":
        q, kt, v = wl.config4()
        qd, ktd, vd = (to_dev(x, wl.BF16) for x in (q, kt, v))
        state = {}

        def fn():
            s = pg.pg_bmm(qd, ktd)
            p16 = ops.softmax_rows(s, out16=torch.bfloat16, want_f32=False)[1]
            state["o"] = pg.pg_bmm(p16, vd)
        flops = 2 * 2.0 * 64 * 2048 * 2048 * 128
        byts = 1140850688 + 637534208
        name, dt = "pg_bmm QK^T -> softmax -> PV, bf16 [64,2048,128]", "bf16"
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

        def fn():
            # first layer in one kernel: h = x W1 in f32 (the backward pass reads it) and a16 = bf16(gelu(h))
            pg.pg_gemm_fused_ex(wl.BF16, 8192, 16384, 4096, xd, 4096, w1d, 16384, h, 16384, None,
                                pg.PG_ACT_GELU | pg.PG_ACT_COPY_ONLY, a16, 16384)
            y = pg.pg_matmul(a16, w2d)
            da, dw2 = pg.pg_matmul_backward(a16, w2d, dy)
            dh = ops.gelu_grad(h, da)
            pg.pg_matmul_backward(xd, w1d, dh)
        flops = 6 * 2.0 * 8192 * 4096 * 16384
        byts = None
        name, dt = "MLP step 8192x4096 -> 16384 -> 4096, forward + backward", "bf16"
    for _ in range(max(args.warmup, 3)):
        fn()
    pg.pg_dev_sync()
    l0 = pg.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    pg.pg_dev_sync()
    ms = e0.elapsed_time(e1) / args.steps
    line = {"metric": "time of one pass", "config": {"workload": name, "config": cfg, "kernel": pg.last_path()},
            "ms_per_step": ms, "value": flops / ms / 1e9, "unit": "TFLOP/s", "dtype": dt, "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "data": "synthetic", "higher_is_better": True,
            "gpu_launches": pg.launch_count() - l0,
            "frac_of_measured_bf16_burst": flops / ms / 1e9 / burst}
    if byts:
        line["algorithmic_GBps"] = byts / ms / 1e6
        line["frac_of_measured_hbm"] = byts / ms / 1e6 / hbm_peak
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
            for _ in range(10):
                graph.replay()
            g1.record(side); side.synchronize()
        _lib.lib.pg_b200_set_stream(None)
        gms = g0.elapsed_time(g1) / 200
        line["graph_replay_ms_per_step"] = gms
        if byts:
            line["graph_replay_GBps"] = byts / gms / 1e6
            line["graph_replay_frac_of_measured_hbm"] = byts / gms / 1e6 / hbm_peak
        line["graph_replay_TFLOPs"] = flops / gms / 1e9
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--config", default="2", choices=["1", "2", "3a", "3b", "4", "4-fused", "5", "linear", "linear-unfused"],
                    help="2 (default) is the headline metric; the others time the remaining configurations "
                         "(single GPU, device-resident) and print one JSON line each")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1 and args.gpus > 1:
        # launched without torchrun: re-launch ourselves with one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 1000), os.path.abspath(__file__),
               "--gpus", str(args.gpus), "--steps", str(args.steps), "--warmup", str(args.warmup), "--impl", args.impl]
        if args.no_cpu_baseline:
            cmd.append("--no-cpu-baseline")
        sys.exit(subprocess.call(cmd))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.config != "2":
        run_other_config(args)
        return
    run_ours(args, rank, world)


if __name__ == "__main__":
    main()
