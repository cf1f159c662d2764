#!/usr/bin/env python
"""Benchmark of the quantized GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c1|c3|c5]

One "step" is one pass of the fused NEGEMMLowpMatrixMultiplyCore (+ QUANTIZE_DOWN_FIXEDPOINT output stage)
over one batch of seeded synthetic input.  The default workload is the configuration the headline metric is
quoted on: the square QASYMM8_SIGNED x QSYMM8_PER_CHANNEL GEMMLowp with M = N = K = 4096, bias, per-channel
fixed-point requantisation to QASYMM8_SIGNED.  With N > 1 GPUs (one process per GPU under torchrun) every
rank owns one 4096-row block of A / dst of an (N*4096) x 4096 x 4096 problem (M-sharding, B replicated, no
collective): weak scaling.

Prints ONE JSON line (rank 0).  `value` is device-timed with inputs resident in HBM; `e2e` is the same metric
through the host-buffer C-ABI call (pinned host memory in, pinned host memory out, copies inside the timed
region); `roofline` is the tensor-core roofline of the GEMM kernel; `cpu_baseline` times the reference's own
scalar implementation on a bounded row sample on the host cores.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "gemmlowp_int8_tops"
UNIT = "TOPS"
NOMINAL_INT8_TOPS = 4500.0
# DRAM bytes (read + write) ncu counted for one launch of the fused GEMM, keyed by (M, N, K); see profiles/
NCU_TRAFFIC_BYTES = {(4096, 4096, 4096): 33.7e6}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=2000)
    p.add_argument("--warmup", type=int, default=200)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5", "bw", "tcgen05_rates"])
    p.add_argument("--only", default="", help="bw: run only the kernels whose name contains this text")
    p.add_argument("--small", action="store_true", help="bw: the reduced sizes used for ncu captures (a few hundred MB)")
    p.add_argument("--batch", type=int, default=256, help="global batch of c4 (split over the ranks)")
    p.add_argument("--weak", action="store_true",
                   help="c4: every rank runs a whole --batch (weak scaling) instead of its share of one global batch")
    p.add_argument("--layers", action="store_true", help="c4: print the per-layer time table to stderr")
    p.add_argument("--no-graph", action="store_true", help="c4: launch every layer eagerly instead of one CUDA graph")
    p.add_argument("--size", type=int, default=0, help="override M=N=K of c2 (profiling on a small case)")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--one-cta", action="store_true", help="keep to the one-CTA tensor-core kernel (comparison runs)")
    p.add_argument("--headline-only", action="store_true",
                   help="c2: skip the ResNet-50 and sharded-linear-layer blocks that follow the headline measurement")
    p.add_argument("--net-steps", type=int, default=20,
                   help="cap on the timed steps of the ResNet-50 / sharded-linear blocks (each step is milliseconds)")
    return p.parse_args()


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(gpu_index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self, t_begin=None, t_end=None):
        """Summarises the samples taken between the two wall-clock instants (time.time()); when fewer than
        three fall inside that window every sample of the run (warm-up included) is used and said so."""
        import datetime
        out = {"sm_mhz": None, "sm_max_mhz": None, "power_w_max": None, "reasons": [], "samples": 0,
               "window": "timed region"}
        if self.proc is not None:
            self.proc.terminate()  # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for line in self.file.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(parts[1]), float(parts[2]), float(parts[3]),
                             [n for n, f in zip(names, parts[4:8]) if f.lower().startswith("active")]))
            except ValueError:
                continue
        self.file.close()
        os.unlink(self.file.name)
        sel = [r for r in rows if t_begin is None or (t_begin <= r[0] <= t_end)]
        if len(sel) < 3:
            sel, out["window"] = rows, "whole run incl. warm-up (timed region shorter than three samples)"
        if sel:
            busy = sorted(r[1] for r in sel)[len(sel) // 2:]  # upper half = samples taken under load
            out.update(sm_mhz=statistics.median(busy), sm_max_mhz=max(r[2] for r in sel),
                       power_w_max=max(r[3] for r in sel), reasons=sorted({n for r in sel for n in r[4]}),
                       samples=len(sel))
        return out


# ---------------------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------------------
def _product_multipliers():
    from computelibrary_b200 import capi
    return capi.calculate_quantized_multiplier, capi.calculate_quantized_multipliers


def _reference_multipliers():
    """The reference arm derives its output stage with the reference's own AsymmHelpers (oracle/_ref, else the C
    restatement), so that its process never maps the library under test."""
    import oracle
    impl = oracle.ref() or oracle.port()

    def many(i_scale, w_scales, o_scale):
        w = np.asarray(w_scales, np.float32)
        if hasattr(impl, "calculate_quantized_multipliers"):
            return impl.calculate_quantized_multipliers(np.float32(i_scale), w, np.float32(o_scale))
        pairs = [impl.calculate_quantized_multiplier(float(np.float32(i_scale) * ws / np.float32(o_scale))) for ws in w]
        return np.array([p[0] for p in pairs], np.int32), np.array([p[1] for p in pairs], np.int32)
    return impl.calculate_quantized_multiplier, many


def make_gemm_workload(name, size, derive=None):
    from computelibrary_b200 import workloads as wl
    one, many = derive or _product_multipliers()
    if name == "c1":
        c = wl.config1()
        qm, sh = one(c["real_multiplier"])
        mult, shift = np.array([qm], np.int32), np.array([sh], np.int32)
        label = "config1: QASYMM8 GEMMLowp M=64 N=128 K=256, bias, per-tensor fixed-point requant to QASYMM8"
    elif name == "c5":
        c = wl.config5()
        mult, shift = many(c["i_scale"], c["w_scales"], c["o_scale"])
        label = "config5: s8 linear M=8192 K=4096 N=14336, per-channel requant to s8, no bias"
    else:
        n = size or 4096
        c = wl.config2(M=n, N=n, K=n)
        mult, shift = many(c["i_scale"], c["w_scales"], c["o_scale"])
        label = (f"config2: QASYMM8_SIGNED x QSYMM8_PER_CHANNEL GEMMLowp M=N=K={n}, bias, per-channel "
                 "fixed-point requant to QASYMM8_SIGNED")
    c["mult"], c["shift"], c["label"] = mult, shift, label
    return c


def build_plan(ctx, c):
    import torch
    from computelibrary_b200 import capi
    code = {np.dtype(np.uint8): capi.U8, np.dtype(np.int8): capi.S8}
    a, b = c["a"], c["b"]
    M, K = a.shape
    N = b.shape[1]
    pc = c["mult"].size > 1
    desc, keep = capi.make_gemm_desc(
        M, N, K, code[a.dtype], code[b.dtype], code[np.dtype(c["out_dtype"])], c["a_off"], c["b_off"],
        multiplier=int(c["mult"][0]), shift=int(c["shift"][0]), multipliers=c["mult"] if pc else None,
        shifts=c["shift"] if pc else None, offset=c["offset"], min_bound=c["lo"], max_bound=c["hi"],
        has_bias=c["bias"] is not None)
    plan = capi.GemmPlan(ctx, desc, keep)
    d_b = torch.from_numpy(b.view(np.uint8)).cuda()
    plan.prepare(d_b)
    ctx.sync()
    del d_b  # B may be released after prepare()
    return plan, (M, N, K)


def init_dist(args):
    """One process per GPU (torchrun); NCCL carries the barriers and the max-reduce of the timings only."""
    import torch
    import torch.distributed as dist
    rank, world, local = dist_env()
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def run_ours(args):
    """The headline line: config 2 (or c1 / c5 on one GPU).  Returns the JSON line as a dict on rank 0, else None."""
    import torch
    import torch.distributed as dist

    import computelibrary_b200 as cl

    rank, world, local = init_dist(args)
    sampler = ClockSampler(local) if rank == 0 else None  # started early: nvidia-smi takes a while to come up

    ctx = cl.Context(local, torch.cuda.current_stream().cuda_stream)
    c = make_gemm_workload(args.workload, args.size)
    if world > 1:
        # M-sharding: this rank's rows of A are its own seeded block; B / bias / multipliers are replicated
        from computelibrary_b200 import workloads as wl
        c["a"] = wl.q8_uniform(np.random.default_rng(1000 + rank), c["a"].shape, c["a"].dtype)
    plan, (M, N, K) = build_plan(ctx, c)
    if args.one_cta:
        plan.allow_pair_kernel(False)
    ops = 2.0 * M * N * K

    d_a = torch.from_numpy(c["a"].view(np.uint8)).cuda()
    d_bias = torch.from_numpy(c["bias"]).cuda() if c["bias"] is not None else None
    d_dst = torch.empty((M, N), dtype=torch.uint8, device="cuda")
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")  # > 126 MB L2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: per-step CUDA events on the launching stream, L2 flushed in between ----
    for _ in range(args.warmup):
        flush.zero_()
        plan.run(d_a, None, d_bias, d_dst)
    barrier()
    t_begin = time.time()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    t_wall0 = time.perf_counter()
    for i in range(args.steps):
        flush.zero_()
        starts[i].record()
        plan.run(d_a, None, d_bias, d_dst)
        stops[i].record()
    barrier()
    t_wall = time.perf_counter() - t_wall0
    t_end = time.time()
    ctx.sync()  # raises if a device-side bounded wait ran out
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, stops)]
    total_ms = float(sum(step_ms))
    clocks = sampler.stop(t_begin, t_end) if sampler is not None else None

    # ---- end to end: pinned host A -> device, run, dst -> pinned host, every step ----
    e2e = None
    if not args.no_e2e:
        a_bytes, d_bytes = M * K, M * N
        h_a, h_d = ctx.host_alloc(a_bytes), ctx.host_alloc(d_bytes)
        h_bias = ctx.host_alloc(4 * N) if c["bias"] is not None else 0
        C.memmove(h_a, c["a"].ctypes.data, a_bytes)
        if h_bias:
            C.memmove(h_bias, c["bias"].ctypes.data, 4 * N)
        for _ in range(max(3, args.warmup)):
            plan.run_host(h_a, h_bias, h_d)
        barrier()
        e2e_steps = min(args.steps, 200)
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            plan.run_host(h_a, h_bias, h_d)  # blocks until dst is valid on the host
        torch.cuda.synchronize()
        e2e_s = (time.perf_counter() - t0) * args.steps / e2e_steps  # scaled to the same step count
        got = np.ctypeslib.as_array((C.c_uint8 * d_bytes).from_address(h_d)).reshape(M, N)
        assert np.array_equal(got, d_dst.cpu().numpy()), "host-buffer path and device path disagree"
        e2e_ms = e2e_s * 1e3
        for p in (h_a, h_d, h_bias):
            if p:
                ctx.host_free(p)
    else:
        e2e_ms = None

    # ---- reduce over ranks: the slowest rank defines the step time ----
    if world > 1:
        t = torch.tensor([total_ms, e2e_ms or 0.0], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_max = float(t[0]), float(t[1])
        e2e_ms = e2e_max if e2e_ms is not None else None
    ms_per_step = total_ms / args.steps
    value = world * ops / (ms_per_step * 1e-3) / 1e12
    if e2e_ms is not None:
        e2e = {"value": world * ops / (e2e_ms / args.steps * 1e-3) / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": M * K + (4 * N if c["bias"] is not None else 0), "d2h_bytes_per_step": M * N,
               "ms_per_step": e2e_ms / args.steps}

    # per-rank copy rates of the end-to-end call: what the host side sustains while every rank copies at once
    if e2e is not None:
        e2e["h2d_gbs_per_rank"] = e2e["h2d_bytes_per_step"] / (e2e["ms_per_step"] * 1e-3) / 1e9
        e2e["d2h_gbs_per_rank"] = e2e["d2h_bytes_per_step"] / (e2e["ms_per_step"] * 1e-3) / 1e9
        e2e["note"] = ("copies in and out overlap the GEMM in row blocks (small at both ends, large in the middle); the step costs about the longer copy, "
                       "so the rate above is what one rank's PCIe / host-memory path delivered with all ranks active")
    if rank != 0:
        plan.close()
        ctx.close()
        return None

    peaks = load_peaks()
    kernel_ms = statistics.mean(step_ms)  # the fused GEMM kernel is the only kernel of a step here
    achieved = ops / (kernel_ms * 1e-3) / 1e12
    peak = 2.0 * peaks["bf16_tflops"]
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOPS", "frac": achieved / peak,
        "peak_source": f"2 x {peaks['source']} bf16 cuBLAS burst ({peaks['bf16_tflops']} TFLOP/s): int8 tensor "
                       "rate is twice the bf16 rate; no int8 figure is recorded in MEASURED_PEAKS.json",
        "frac_of_nominal_4500": achieved / NOMINAL_INT8_TOPS,
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the committed ncu capture of this kernel
        # (profiles/): the 4096^3 operands are read once, the 16.8 MB output stays in L2 within the capture window
        "traffic": NCU_TRAFFIC_BYTES.get((M, N, K)),
        "traffic_source": "ncu capture summarised under profiles/" if (M, N, K) in NCU_TRAFFIC_BYTES else None,
        "algorithmic_bytes": M * K + N * K + M * N + 16 * N,
        "kernel": {"tcgen05_2cta": "gemmlowp_tcgen05_2cta_kernel", "tcgen05": "gemmlowp_tcgen05_kernel"}.get(
            plan.kernel, "gemmlowp_simt_kernel"),
        "kernel_ms": kernel_ms,
    }
    try:  # library int8 GEMM as a yardstick only (never on the product path)
        ya = torch.from_numpy(c["a"]).cuda()
        yb = torch.from_numpy(np.ascontiguousarray(c["b"])).cuda().t().contiguous().t()
        for _ in range(3):
            torch._int_mm(ya, yb)
        ts = []
        for _ in range(10):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            torch._int_mm(ya, yb)
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        roofline["yardstick_torch_int_mm_tops"] = ops / (min(ts) * 1e-3) / 1e12
    except Exception as ex:  # noqa: BLE001
        roofline["yardstick_torch_int_mm_tops"] = None
        roofline["yardstick_error"] = str(ex)[:120]

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "s8*s8->s32->s8" if c["a"].dtype == np.int8 else "u8*u8->s32->u8", "data": "synthetic",
        "config": {"workload": c["label"], "per_gpu_shape": [M, N, K], "l2": "flushed between timed steps "
                   "(256 MB write)", "sharding": "M-sharded, B replicated, no collective" if world > 1 else "single GPU"},
        "e2e": e2e, "gpu_launches": args.steps * plan.launches, "roofline": roofline, "clocks": clocks,
        "wall_s_timed_loop": t_wall,
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(c, ops)
    plan.close()
    ctx.close()
    return line


# ---------------------------------------------------------------------------------------------------------
# CPU baseline / reference arm: the reference's own scalar implementation on the host cores
# ---------------------------------------------------------------------------------------------------------
def cpu_reference_step(c, rows, threads):
    """One pass of the reference's CPU implementation over `rows` rows of A: its scalar GEMMLowp core
    (tests/validation/reference/GEMMLowp.cpp:202-255, a serial triple loop) + fixed-point output stage.  The
    rows are split over `threads` host threads the way the NE scheduler splits a window over DimY."""
    import oracle
    from concurrent.futures import ThreadPoolExecutor
    ref = oracle.ref()
    kind = "reference" if ref is not None else "port"
    a = c["a"][:rows]
    pc = c["mult"].size > 1

    if ref is not None:
        def work(blk):
            acc = ref.gemmlowp_core(a[blk], c["b"], c["a_off"], c["b_off"])
            return ref.output_stage(acc, c["bias"], c["mult"] if pc else c["mult"][:1],
                                    c["shift"] if pc else c["shift"][:1], c["offset"], c["lo"], c["hi"],
                                    c["out_dtype"])
        blocks = [slice(i * rows // threads, (i + 1) * rows // threads) for i in range(threads)]
        blocks = [b for b in blocks if b.stop > b.start]
        t0 = time.perf_counter()
        with ThreadPoolExecutor(max_workers=threads) as ex:  # ctypes releases the GIL during the C++ call
            list(ex.map(work, blocks))
        return time.perf_counter() - t0, kind, threads
    port = oracle.port()
    t0 = time.perf_counter()
    port.gemmlowp_fused(a, c["b"], c["bias"], c["a_off"], c["b_off"], c["mult"], c["shift"], c["offset"], c["lo"],
                        c["hi"], c["out_dtype"])
    return time.perf_counter() - t0, kind, port.num_threads()


def cpu_sample_rows(c, threads):
    M, K = c["a"].shape
    N = c["b"].shape[1]
    # the scalar reference sustains roughly 1-2.5 GOP/s per core: aim at about 10 s of work
    target_ops = 1.5e9 * threads * 10
    rows = int(max(threads, min(M, target_ops / (2.0 * N * K))))
    return rows


def cpu_baseline(c, ops_full):
    threads = os.cpu_count() or 1
    rows = cpu_sample_rows(c, threads)
    M, K = c["a"].shape
    N = c["b"].shape[1]
    secs, kind, used = cpu_reference_step(c, rows, threads)
    return {"value": 2.0 * rows * N * K / secs / 1e12, "unit": UNIT, "cores": used, "kind": kind,
            "sample": f"{rows} of {M} rows of A (all of B): {rows}x{N}x{K}, {secs:.2f} s, "
                      f"{'reference scalar oracle compiled in place, rows split over host threads' if kind == 'reference' else 'C restatement with OpenMP'}"}


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    c = make_gemm_workload(args.workload if args.workload in ("c1", "c2", "c5") else "c2", args.size,
                           derive=_reference_multipliers())
    M, K = c["a"].shape
    N = c["b"].shape[1]
    threads = os.cpu_count() or 1
    # keep the whole --steps/--warmup run within a few minutes: a short calibration pass gives this machine's
    # rate, each step then takes as many rows of A as fit its share of about 150 s -- all of them when they fit
    per_step_budget = 150.0 / max(1, args.steps + args.warmup)
    cal_rows = min(M, 16 * threads)
    cal_s, kind, used = cpu_reference_step(c, cal_rows, threads)
    rows = int(max(threads, min(M, cal_rows * per_step_budget / max(cal_s, 1e-6) * 0.8)))
    for _ in range(args.warmup):
        _, kind, used = cpu_reference_step(c, rows, threads)
    t = 0.0
    for _ in range(args.steps):
        s, kind, used = cpu_reference_step(c, rows, threads)
        t += s
    ms = t / args.steps * 1e3
    value = 2.0 * rows * N * K / (ms * 1e-3) / 1e12
    sample = (f"each step = {rows} of {M} rows of A against all of B ({rows}x{N}x{K})" +
              (": the whole problem" if rows == M else ""))
    with open("/proc/self/maps") as f:
        native = sorted({ln.split()[-1] for ln in f if ".so" in ln and ("/oracle/" in ln or "computelibrary_b200" in ln)})
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "s8*s8->s32->s8" if c["a"].dtype == np.int8 else "u8*u8->s32->u8", "data": "synthetic",
        "config": {"workload": c["label"], "per_gpu_shape": [M, N, K], "note": "CPU arm: the NE (Arm) kernels cannot "
                   "be built on x86_64; this times the reference's own scalar implementation of the path"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": used, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "same_config": rows == M, "native_libraries_mapped": native,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------
# further workloads (not the headline line): config 3 convolution, config 5 column-sharded linear layer
# ---------------------------------------------------------------------------------------------------------
def _timed_steps(step, steps, warmup, flush, barrier):
    import torch
    for _ in range(warmup):
        flush.zero_()
        step()
    barrier()
    st = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    en = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        flush.zero_()
        st[i].record()
        step()
        en[i].record()
    barrier()
    return [a.elapsed_time(b) for a, b in zip(st, en)]


def run_conv(args):
    """Config 3: 3x3 s1 p1 NHWC convolution, batch 32 (split over the ranks: strong scaling) through cugl_conv2d_run
    (implicit GEMM: the patches are gathered inside the tensor-core kernel).  HBM roofline on the compulsory bytes."""
    import torch
    import torch.distributed as dist
    import computelibrary_b200 as cl
    from computelibrary_b200 import capi, sharding
    from computelibrary_b200 import workloads as wl
    rank, world, local = init_dist(args)
    ctx = cl.Context(local, torch.cuda.current_stream().cuda_stream)
    c = wl.config3()
    b0, b1 = sharding.batch_shard(c["src"].shape[0], world, rank)
    src = np.ascontiguousarray(c["src"][b0:b1])
    B, H, W, Cc = src.shape
    OFM, kh, kw, _ = c["weights"].shape
    mult, shift = capi.calculate_quantized_multipliers(c["i_scale"], c["w_scales"], c["o_scale"])
    desc, keep = capi.make_conv_desc(B, H, W, Cc, OFM, kh, kw, c["stride"], c["pad"], (1, 1), capi.U8, capi.S8,
                                     c["in_zp"], 0, multipliers=mult, shifts=shift, dst_zp=c["out_zp"],
                                     min_bound=c["lo"], max_bound=c["hi"])
    plan = capi.ConvPlan(ctx, desc, keep)
    wo, ho = plan.out_dims()
    d_src = torch.from_numpy(src).cuda()
    d_w = torch.from_numpy(c["weights"].view(np.uint8)).cuda()
    d_b = torch.from_numpy(c["bias"]).cuda()
    d_dst = torch.empty((B, ho, wo, OFM), dtype=torch.uint8, device="cuda")
    plan.prepare(d_w)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    step_ms = _timed_steps(lambda: plan.run(d_src, d_b, d_dst), args.steps, args.warmup, flush, barrier)
    ctx.sync()
    total_ms = float(sum(step_ms))
    if world > 1:
        t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t[0])
    if rank == 0:
        Bt = c["src"].shape[0]
        M, K = Bt * ho * wo, kh * kw * Cc
        ops = 2.0 * M * OFM * K
        ms = total_ms / args.steps
        implicit = plan.kernel == "implicit"
        # compulsory bytes per rank: input + weights + output; the explicit lowering also writes and reads the patch matrix
        per_rank_bytes = B * H * W * Cc + OFM * K + B * ho * wo * OFM + (0.0 if implicit else 2.0 * B * ho * wo * K)
        peaks = load_peaks()
        ach = per_rank_bytes / (statistics.mean(step_ms) * 1e-3) / 1e9
        print(json.dumps({
            "metric": METRIC, "value": ops / (ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "u8*s8->s32->u8", "data": "synthetic",
            "images_per_s": Bt / (ms * 1e-3),
            "config": {"workload": "config3: 3x3 s1 p1 NHWC conv, batch 32, 56x56x64 -> 64, per-channel weights, "
                       "fused ReLU (NEGEMMConvolutionLayer: im2col + GEMMLowp)", "per_gpu_batch": B,
                       "l2": "flushed between timed steps (256 MB write)",
                       "sharding": "batch split over ranks, weights replicated, no collective"},
            "gpu_launches": args.steps * plan.launches,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": ach / peaks["hbm_gbs"], "traffic": None,
                         "bytes_counted": ("input + weights + output per rank (implicit GEMM: the patch matrix is never "
                                           "materialised)" if implicit else
                                           "input + weights + output + patch matrix written and read once, per rank"),
                         "kernel": "gemmlowp_conv_tcgen05_kernel" if implicit else
                                   "im2col_nhwc_kernel + gemmlowp_tcgen05_kernel",
                         "lowering": plan.kernel}}), flush=True)
    plan.close()
    ctx.close()


def measure_resnet(args, weak):
    """Config 4: QASYMM8 ResNet-50 v1 (examples/graph_resnet50.cpp topology, batch norm folded, ReLU fused), batch split
    over the ranks (strong scaling: one global batch of --batch; weak: --batch per rank), weights replicated, no
    collective.  Every rank takes part; rank 0 gets the result, the others None."""
    import torch
    import torch.distributed as dist
    import computelibrary_b200 as cl
    from computelibrary_b200 import resnet50 as rn
    from computelibrary_b200 import sharding
    rank, world, local = init_dist(args)
    # a stream of its own: the node list is captured into a CUDA graph on it; torch's current stream is set to
    # it so that the bench's events, copies and L2 flush are ordered with the network
    prev_stream = torch.cuda.current_stream()
    work = torch.cuda.Stream()
    torch.cuda.set_stream(work)
    ctx = cl.Context(local, work.cuda_stream)
    global_batch = args.batch * world if weak else args.batch
    b0, b1 = sharding.batch_shard(global_batch, world, rank)
    B = b1 - b0
    net = rn.ResNet50(ctx, B, seed=1)
    rng = np.random.default_rng(100 + rank)
    h_in = torch.from_numpy(rng.integers(0, 256, (B, 224, 224, 3), dtype=np.uint8)).pin_memory()
    d_in = h_in.cuda()
    h_out = torch.empty((B, 1, 1, 1000), dtype=torch.uint8).pin_memory()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    steps, warmup = min(args.steps, args.net_steps), max(3, min(args.warmup, 5))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    for _ in range(2):  # first-use costs (lazy workspaces) stay outside the sampled window
        net.run(d_in)
    barrier()
    graph = None if args.no_graph else net.capture(d_in, work)
    run_net = (lambda: net.run(d_in)) if graph is None else graph.replay
    barrier()
    t_begin = time.time()
    step_ms = _timed_steps(run_net, steps, warmup, flush, barrier)
    clocks = sampler.stop(t_begin, time.time()) if sampler else None
    ctx.sync()

    def e2e_step():
        d_in.copy_(h_in, non_blocking=True)
        run_net()
        h_out.copy_(net.bufs["softmax"], non_blocking=True)

    e2e_ms = [] if args.no_e2e else _timed_steps(e2e_step, max(3, steps // 2), 3, flush, barrier)

    def e2e_pipelined(n):
        """The same work per step -- this step's images in from pinned host memory, the network, the class bytes out --
        as a serving loop runs it: the images of step i + 1 travel on a copy stream into one of two staging buffers
        while step i computes; the work stream takes them over with a device-to-device copy (38.5 MB, about 12 us).
        Returns milliseconds per step over n back-to-back steps (the first step's copy is not hidden and counts)."""
        copy = torch.cuda.Stream()
        stage = [torch.empty_like(d_in), torch.empty_like(d_in)]
        landed = [torch.cuda.Event(), torch.cuda.Event()]
        taken = [torch.cuda.Event(), torch.cuda.Event()]
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        copy.wait_stream(work)
        t0.record(work)
        copy.wait_event(t0)
        for i in range(n):
            b = i & 1
            with torch.cuda.stream(copy):
                if i >= 2:
                    copy.wait_event(taken[b])
                stage[b].copy_(h_in, non_blocking=True)
                landed[b].record(copy)
            work.wait_event(landed[b])
            d_in.copy_(stage[b], non_blocking=True)
            taken[b].record(work)
            run_net()
            h_out.copy_(net.bufs["softmax"], non_blocking=True)
        t1.record(work)
        barrier()
        return t0.elapsed_time(t1) / n

    e2e_pipe_ms = 0.0
    if not args.no_e2e:
        e2e_pipelined(3)
        e2e_pipe_ms = e2e_pipelined(max(6, steps // 2))
    if args.layers and rank == 0:
        rows = net.run_timed(d_in)
        tot = sum(r[3] for r in rows)
        for name, op, kern, ms in rows:
            print(f"{name:34s} {op:15s} {kern:10s} {ms * 1e3:9.1f} us {100 * ms / tot:5.1f} %", file=sys.stderr)
        print(f"sum {tot:.3f} ms", file=sys.stderr)
    t = torch.tensor([float(sum(step_ms)) / steps, float(sum(e2e_ms)) / max(1, len(e2e_ms)), e2e_pipe_ms], device="cuda",
                     dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out = None
    if rank == 0:
        ms, e2e_serial, e2e = float(t[0]), float(t[1]), float(t[2])
        ops_img, bytes_img = rn.graph_ops(net.nodes), rn.graph_bytes(net.nodes)
        peaks = load_peaks()
        # one rank's rates over its own step time: tensor-core rate against 2 x the measured dense bf16 peak, and the
        # bytes a layer-by-layer run must move at least against the measured copy bandwidth
        own_s = statistics.mean(step_ms) * 1e-3
        ach = ops_img * B / own_s / 1e12
        peak = 2.0 * peaks["bf16_tflops"]
        gbs = bytes_img * B / own_s / 1e9
        out = {
            "metric": "resnet50_qasymm8_images_per_s", "value": global_batch / (ms * 1e-3), "unit": "img/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak" if weak else "strong", "dtype": "u8*s8->s32->u8", "data": "synthetic",
            "config": {"workload": f"config4: QASYMM8 ResNet-50 v1, 224x224, global batch {global_batch}, per-channel s8 "
                       "weights, batch norm folded, ReLU fused", "per_gpu_batch": B,
                       "l2": "flushed between timed steps (256 MB write)",
                       "sharding": "batch split over ranks, weights replicated, no collective",
                       "launch": "eager, one C-ABI call per layer" if graph is None else
                                 "one CUDA graph of the layer calls per step"},
            "int8_tops": ops_img * global_batch / (ms * 1e-3) / 1e12,
            "gpu_launches": steps * net.launches,
            "roofline": {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TOP/s", "frac": ach / peak,
                         "traffic": None, "peak_source": "2 x " + peaks["source"] + " dense bf16 cuBLAS rate",
                         "kernel": "whole network (54 convolutions + pooling / addition / softmax kernels)",
                         "hbm": {"achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                                 "bytes_counted": "inputs read + output written once per layer, 8-bit activations "
                                                  f"({bytes_img / 1e6:.1f} MB per image unfused)"}},
            "clocks": clocks}
        if e2e_ms:
            out["e2e"] = {"value": global_batch / (e2e * 1e-3), "unit": "img/s", "ms_per_step": e2e,
                          "h2d_bytes_per_step": int(global_batch * 224 * 224 * 3),   # all ranks together
                          "d2h_bytes_per_step": int(global_batch * 1000),
                          "schedule": "every step copies its own images in from pinned host memory and its class bytes "
                                      "out; the copy of step i + 1 runs on a second stream while step i computes "
                                      "(two staging buffers), back-to-back steps, time per step over the whole run",
                          "unpipelined": {"value": global_batch / (e2e_serial * 1e-3), "ms_per_step": e2e_serial,
                                          "schedule": "copy in, network, copy out on one stream, L2 flushed between steps"}}
    net.close()
    ctx.close()
    torch.cuda.set_stream(prev_stream)
    return out


def run_resnet(args):
    line = measure_resnet(args, args.weak)
    if line is not None:
        line["vs_baseline"] = None
        print(json.dumps(line), flush=True)


def measure_linear_sharded(args):
    """Config 5 on N > 1 GPUs: B is split by columns (multiples of the 256-column tile), every rank computes
    dst[:, n0:n1]; the int8 column blocks reach every rank either through ncclAllGather (baseline) or by the fused
    kernel's epilogue storing each tile into all ranks' buffers (push all-gather).  Rank 0 gets the result."""
    import torch
    import torch.distributed as dist
    import computelibrary_b200 as cl
    from computelibrary_b200 import capi, sharding
    rank, world, local = init_dist(args)
    ctx = cl.Context(local, torch.cuda.current_stream().cuda_stream)
    c = make_gemm_workload("c5", 0)
    M, K = c["a"].shape
    N = c["b"].shape[1]
    n0, n1 = sharding.column_shard(N, world, rank)
    cs = dict(c)
    cs["b"] = np.ascontiguousarray(c["b"][:, n0:n1])
    cs["mult"], cs["shift"] = c["mult"][n0:n1], c["shift"][n0:n1]
    plan, _ = build_plan(ctx, cs)
    d_a = torch.from_numpy(c["a"].view(np.uint8)).cuda()
    d_local = torch.empty((M, n1 - n0), dtype=torch.uint8, device="cuda")
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    full = [None]
    steps, warmup = min(args.steps, args.net_steps), max(3, min(args.warmup, 5))

    def step():
        plan.run(d_a, None, None, d_local)
        full[0] = sharding.allgather_columns(d_local, N, world, rank)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    step_ms = _timed_steps(step, steps, warmup, flush, barrier)
    gemm_ms = _timed_steps(lambda: plan.run(d_a, None, None, d_local), steps, warmup, flush, barrier)

    # ---- fused push all-gather: the epilogue stores each tile into every rank's [M, N] buffer over NVLink ----
    desc_push, keep_push = capi.make_gemm_desc(
        M, n1 - n0, K, capi.S8, capi.S8, capi.S8, c["a_off"], c["b_off"], multipliers=cs["mult"],
        shifts=cs["shift"], offset=c["offset"], min_bound=c["lo"], max_bound=c["hi"], has_bias=False, ldd=N)
    plan_push = capi.GemmPlan(ctx, desc_push, keep_push)
    d_bs = torch.from_numpy(cs["b"].view(np.uint8)).cuda()
    plan_push.prepare(d_bs)
    ctx.sync()
    full_ptr = ctx.malloc(M * N)                       # cudaMalloc'ed so that it can be exported
    handles = [None] * world
    dist.all_gather_object(handles, ctx.ipc_get_handle(full_ptr))
    peers = {r: ctx.ipc_open_handle(handles[r]) for r in range(world) if r != rank}
    dsts = [full_ptr + n0] + [peers[r] + n0 for r in sorted(peers)]
    push_ms = _timed_steps(lambda: plan_push.run_multi(d_a, None, dsts), steps, warmup, flush, barrier)
    ctx.sync()
    barrier()
    # wall time of push steps including the completion barrier a consumer needs
    t0 = time.perf_counter()
    for _ in range(steps):
        plan_push.run_multi(d_a, None, dsts)
        torch.cuda.synchronize()
        dist.barrier()
    push_wall_ms = (time.perf_counter() - t0) * 1e3 / steps
    host = np.empty((M, N), np.uint8)
    ctx.d2h(host.ctypes.data, full_ptr, M * N)
    ctx.sync()
    push_equal = bool(np.array_equal(host, full[0].cpu().numpy()))
    t = torch.tensor([float(sum(step_ms)), float(sum(gemm_ms)), float(sum(push_ms)), push_wall_ms,
                      0.0 if push_equal else 1.0], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    chk = full[0].to(torch.int64).sum().reshape(1)
    lo, hi = chk.clone(), chk.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    out = None
    if rank == 0:
        ops = 2.0 * M * N * K
        ms = float(t[2]) / steps
        nccl_ms = float(t[0]) / steps
        gemm_only = float(t[1]) / steps
        sent = (world - 1) * M * (n1 - n0)
        peaks = load_peaks()
        # the step cannot be faster than its GEMM share on the tensor cores nor than its bytes over one direction of
        # this GPU's NVLink ports (measured peer-copy rate of this pool: 770 GB/s)
        floor_ms = max(ops / world / (2.0 * peaks["bf16_tflops"] * 1e12), sent / 770e9) * 1e3
        out = {
            "metric": METRIC, "value": ops / (ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "dtype": "s8*s8->s32->s8", "data": "synthetic",
            "config": {"workload": c["label"], "sharding": f"columns of B split over {world} ranks "
                       f"({n1 - n0} per rank); fused kernel stores every tile into all ranks' [M,N] buffers "
                       "(push all-gather over NVLink peer stores)",
                       "l2": "flushed between timed steps (256 MB write)"},
            "push_ms": ms, "nccl_ms": nccl_ms, "gemm_only_ms": gemm_only,
            "push_wall_ms_per_step_incl_sync_and_barrier": float(t[3]),
            "nccl_baseline": {"ms_per_step": nccl_ms, "value": ops / (nccl_ms * 1e-3) / 1e12,
                              "what": "same GEMM + ncclAllGather of the column blocks + re-tile copy"},
            "nvlink": {"bytes_sent_per_rank": sent, "achieved_gbs_per_direction": sent / (ms * 1e-3) / 1e9,
                       "measured_peer_copy_gbs": 770.0},
            "roofline": {"bound": "max(tensor, nvlink)", "floor_ms": floor_ms, "frac": floor_ms / ms},
            "push_equals_nccl": bool(float(t[4]) == 0.0),
            "ranks_agree": bool(int(lo) == int(hi)),
            "gpu_launches": steps * plan_push.launches}
    barrier()
    for pptr in peers.values():
        ctx.ipc_close_handle(pptr)
    barrier()
    ctx.free(full_ptr)
    plan_push.close()
    plan.close()
    ctx.close()
    return out


def run_linear_sharded(args):
    line = measure_linear_sharded(args)
    if line is not None:
        line["vs_baseline"] = None
        print(json.dumps(line), flush=True)


def run_bandwidth(args):
    """The HBM-bound kernels of the path, each on one shape, timed alone with the L2 flushed before every launch.
    One JSON line: per kernel the algorithmic bytes, the time and the achieved GB/s against the measured copy peak."""
    import torch
    import computelibrary_b200 as cl
    from computelibrary_b200 import capi
    torch.cuda.set_device(0)
    ctx = cl.Context(0, torch.cuda.current_stream().cuda_stream)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    peaks = load_peaks()
    g = torch.Generator(device="cuda").manual_seed(1)
    sc = 4 if args.small else 1  # divisor of the leading dimension

    def rnd8(*shape):
        return torch.randint(0, 256, shape, dtype=torch.uint8, device="cuda", generator=g)

    cases = []

    def case(name, nbytes, fn, note):
        if args.only and args.only not in name:
            return
        ms = _timed_steps(fn, args.steps, args.warmup, flush, torch.cuda.synchronize)
        ctx.sync()
        t = statistics.mean(ms)
        cases.append({"kernel": name, "case": note, "bytes": int(nbytes), "us": t * 1e3,
                      "gbs": nbytes / (t * 1e-3) / 1e9, "frac_of_measured_copy": nbytes / (t * 1e-3) / 1e9 / peaks["hbm_gbs"]})

    M, K = 32768 // sc, 8192
    a, out = rnd8(M, K), torch.empty(M, dtype=torch.int32, device="cuda")
    case("reduce_rows_kernel", M * K + 4 * M, lambda: ctx.reduce_rows(a, capi.S8, M, K, K, out), f"A s8 [{M}][{K}]")
    K, N = 16384 // sc, 14336
    b, out = rnd8(K, N), torch.empty(N, dtype=torch.int32, device="cuda")
    case("reduce_cols_kernel", K * N + 4 * N, lambda: ctx.reduce_cols(b, capi.S8, K, N, N, out), f"B s8 [{K}][{N}]")
    del a, b
    K, N = 4096, 14336 // sc
    desc, keep = capi.make_gemm_desc(128, N, K, capi.S8, capi.S8, capi.S8, 5, 0, multiplier=2 ** 30, shift=8,
                                     min_bound=-128, max_bound=127)
    plan, b = capi.GemmPlan(ctx, desc, keep), rnd8(K, N)
    case("transpose_colsum_kernel", 2 * K * N + 4 * N, lambda: plan.prepare(b), f"B s8 [{K}][{N}] -> Bt + column sums")
    plan.close()
    del b
    M, N = 8192 // sc, 8192
    acc = torch.randint(-2 ** 20, 2 ** 20, (M, N), dtype=torch.int32, device="cuda", generator=g)
    bias = torch.randint(-5000, 5000, (N,), dtype=torch.int32, device="cuda", generator=g)
    o8 = torch.empty((M, N), dtype=torch.uint8, device="cuda")
    case("output_stage_kernel", 5 * M * N + 4 * N,
         lambda: ctx.output_stage(acc, 4 * N, bias, o8, N, capi.U8, M, N, None, None, 1099511552, 8, 1, 10, 0, 255),
         f"S32 [{M}][{N}] + bias -> u8, per-tensor")
    cs, rs = bias, torch.randint(-5000, 5000, (M,), dtype=torch.int32, device="cuda", generator=g)
    case("offset_contribution_kernel", 8 * M * N + 4 * (M + N),
         lambda: ctx.offset_contribution(acc, M, N, 4096, 4 * N, cs, rs, 3, -7), f"S32 [{M}][{N}] in place, both offsets")
    del acc, o8
    for B in ([32] if args.small else [32, 256]):
        H = W = 56
        Cc, Kp = 64, 576
        src, dst = rnd8(B, H, W, Cc), torch.empty((B * H * W, Kp), dtype=torch.uint8, device="cuda")
        case("im2col_nhwc_kernel", B * H * W * (Cc + Kp),
             lambda: ctx.im2col_nhwc(src, dst, Cc, W, H, B, 3, 3, 1, 1, 1, 1, 1, 1, W, H, 128, Kp),
             f"batch {B}, 56x56x64, 3x3 s1 p1")
        del src, dst
    B = 256 // sc
    pd = capi.make_pool_desc(B, 112, 112, 64, capi.POOL_MAX, (3, 3), (2, 2), (0, 1, 0, 1), (0.05, 0), (0.05, 0))
    wo, ho = capi.pool_out_dims(pd)
    src, dst = rnd8(B, 112, 112, 64), torch.empty((B, ho, wo, 64), dtype=torch.uint8, device="cuda")
    case("maxpool_window_kernel", B * 64 * (112 * 112 + ho * wo), lambda: ctx.pool2d_nhwc(pd, src, dst),
         f"batch {B}, 112x112x64, 3x3 s2")
    del src, dst
    n = (256 // sc) * 56 * 56 * 256
    x, y, z = rnd8(n), rnd8(n), torch.empty(n, dtype=torch.uint8, device="cuda")
    case("add_saturating_kernel", 3 * n, lambda: ctx.add_qasymm8(x, y, z, n, (0.05, 0), (0.05, 0), (0.05, 0), capi.ACT_RELU),
         f"{n} elements, equal quantizations + ReLU")
    print(json.dumps({"metric": "hbm_kernel_gbs", "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                      "peak_measured_copy_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"],
                      "l2": "flushed before every timed launch (256 MB write)", "kernels": cases}), flush=True)
    ctx.close()


def run_issue_rate_probe(args):
    """What the thread that issues tensor-core work pays per instruction on an otherwise idle SM (clocks per tcgen05.mma
    for N = 16 .. 256, per commit, per barrier operation): the stand-alone program built beside the library.  These
    figures are the tile-shape rooflines the design notes quote; nothing of the library runs here."""
    from computelibrary_b200 import build as cuda_build
    exe = cuda_build.PROBE_PATH
    if not os.path.exists(exe):
        raise SystemExit(f"{exe} is missing: run __graft_entry__.build() first")
    out = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    if out.returncode != 0:
        raise SystemExit(f"probe failed: {out.stderr.strip()}")
    line = {"metric": "tcgen05_issue_rates", "n_gpus": 1, "data": "none", "config": {"workload": "one CTA, one issuing thread"}}
    line.update(json.loads(out.stdout))
    print(json.dumps(line), flush=True)


def measure_linear_single(args):
    """Config 5 on one GPU, device resident: the 8192 x 14336 x 4096 s8 linear layer, per-step CUDA events with the L2
    flushed in between -- the same kernel as the headline on a shape with 28 waves of tiles instead of 3.5."""
    import torch
    import computelibrary_b200 as cl
    ctx = cl.Context(torch.cuda.current_device(), torch.cuda.current_stream().cuda_stream)
    c = make_gemm_workload("c5", 0)
    plan, (M, N, K) = build_plan(ctx, c)
    d_a = torch.from_numpy(c["a"].view(np.uint8)).cuda()
    d_bias = torch.from_numpy(c["bias"]).cuda() if c["bias"] is not None else None
    d_dst = torch.empty((M, N), dtype=torch.uint8, device="cuda")
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    steps, warmup = min(args.steps, 20), max(3, min(args.warmup, 5))
    for _ in range(warmup):
        flush.zero_()
        plan.run(d_a, None, d_bias, d_dst)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for s, e in ev:
        flush.zero_()
        s.record()
        plan.run(d_a, None, d_bias, d_dst)
        e.record()
    torch.cuda.synchronize()
    ctx.sync()
    ms = float(np.mean([s.elapsed_time(e) for s, e in ev]))
    tops = 2.0 * M * N * K / (ms * 1e-3) / 1e12
    peaks = load_peaks()
    peak, src = 2.0 * peaks["bf16_tflops"], "2 x " + peaks["source"] + " dense bf16 cuBLAS rate"
    out = {"value": tops, "unit": "TOPS", "ms_per_step": ms, "steps": steps, "warmup": warmup, "kernel": plan.kernel,
           "workload": "config5: s8 linear M=8192 K=4096 N=14336, per-channel requant to s8, no bias (one GPU, unsharded)",
           "roofline": {"bound": "tensor", "achieved": tops, "peak": peak, "unit": "TOPS", "frac": tops / peak, "peak_source": src}}
    plan.close()
    del d_a, d_dst, flush
    return out


def json_only_stdout():
    """Keeps stdout for the JSON line alone: file descriptor 1 is pointed at stderr, where native libraries that print
    there end up (NCCL's version banner on several GPUs), and Python's sys.stdout keeps the original descriptor."""
    sys.stdout.flush()
    keep = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(keep, "w")


def main():
    args = parse_args()
    json_only_stdout()
    _, world, _ = dist_env()
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload == "tcgen05_rates":
        run_issue_rate_probe(args)
    elif args.workload == "bw":
        run_bandwidth(args)
    elif args.workload == "c3":
        run_conv(args)
    elif args.workload == "c4":
        run_resnet(args)
    elif args.workload == "c5" and world > 1:
        run_linear_sharded(args)
    else:
        line = run_ours(args)
        if args.workload == "c2" and not args.headline_only and not args.size:
            # the second half of the metric and the one configuration with a collective, measured in the same
            # process after the headline: ResNet-50 images/s (strong and weak scaling) and, on several GPUs, the
            # column-sharded linear layer with its all-gather
            strong = measure_resnet(args, weak=False)
            weak = measure_resnet(args, weak=True) if world > 1 else strong
            linear = measure_linear_sharded(args) if world > 1 else None
            if line is not None:
                def brief(r):
                    return {k: r[k] for k in ("value", "unit", "ms_per_step", "scaling", "int8_tops", "roofline", "e2e",
                                              "clocks", "gpu_launches", "steps", "warmup") if k in r} | {
                                                  "batch_per_gpu": r["config"]["per_gpu_batch"], "launch": r["config"]["launch"]}
                line["resnet50"] = {"metric": "resnet50_qasymm8_images_per_s",
                                    "workload": strong["config"]["workload"].replace(f"global batch {args.batch}", "batch 256"),
                                    "strong": brief(strong), "weak": brief(weak),
                                    "img_per_s": strong["value"], "img_per_s_weak": weak["value"]}
                if linear is None:
                    line["linear_c5"] = measure_linear_single(args)
                else:
                    line["linear_c5"] = {k: linear[k] for k in ("value", "unit", "push_ms", "nccl_ms", "gemm_only_ms",
                                                                "nvlink", "roofline", "push_equals_nccl", "ranks_agree",
                                                                "push_wall_ms_per_step_incl_sync_and_barrier")}
                    line["linear_c5"]["workload"] = linear["config"]["workload"]
        if line is not None:
            print(json.dumps(line), flush=True)
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
