"""Benchmark of the tt.dot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the hot path over one batch of synthetic input: one tt.dot GEMM launched
through the C-ABI (tx_dot_run). Workloads (BASELINE.json `configs`):

    cfg2         bf16 4096x4096x4160, LoopSplit tail (BLOCK_K 128: main [0,4096) + 64-wide remainder).
                 Default. At N GPUs each rank runs its own column panel of a 4096 x (4096*N) x 4160
                 GEMM (N-sharded, no collective): weak scaling.
    cfg3         bf16 16x14336x4096 decode shape; HBM-bound, roofline in GB/s.
    cfg4         fp8 e4m3 8192^3 with per-row / per-column fp32 scales -> bf16.
    cfg5_nshard  bf16 16384x28672x8192, columns of B and C split over the ranks: strong scaling.
    cfg5_kshard  same GEMM, K split over the ranks, fp32 partials, NCCL reduce-scatter.
    cfg5_kshard_fused[_bf16]  K split over the ranks, the GEMM epilogue stores partial tiles into the owning
                 rank's memory over NVLink (fp32 or bf16 partials), then one local slot reduction.
    attn_d64[_causal], attn_d128[_causal], attn_d64_16k_causal
                 the next row after the GEMM: fused attention forward (two chained tt.dot + online softmax)
                 on the reference benchmark's shapes (batch 4, 32 heads, fp16); metric "attention fwd TFLOP/s".
                 At N GPUs every rank runs its own batch: weak scaling, no collective.

One JSON line is printed by rank 0. `--impl reference` times the reference's CPU path for the same
workload (the same tt.dot run by Triton's interpreter on the host cores) on a bounded tile sample.
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

L2_BYTES = 126 * 1024 * 1024

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed ncu captures
# (profiles/*.md name the command); None where no capture exists.
NCU_TRAFFIC_BYTES = {"cfg2": 110.2e6, "cfg3": 122.2e6, "cfg4": 462.9e6, "cfg5_nshard": None, "cfg5_kshard": None,
                     "attn_d64": 254.7e6}   # attn_d64: 201.4 MB read + 53.3 MB written at the bench shape (one-pass capture)


def measured_peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "_source": "fallback"}


WORKLOADS = {
    #  name         m      n      k     dtype  seed dist       scales  k_split  metric unit
    "cfg2": dict(m=4096, n=4096, k=4160, dtype="bf16", seed=1, dist="uniform", scales=False, k_split=4096, block=(128, 128, 128)),
    # cfg2 launched as a @triton.jit K-loop kernel through the package's Triton backend (same library kernel underneath)
    "cfg2_jit": dict(m=4096, n=4096, k=4160, dtype="bf16", seed=1, dist="uniform", scales=False, k_split=4096, block=(128, 128, 128), jit=True),
    "cfg3": dict(m=16, n=14336, k=4096, dtype="bf16", seed=2, dist="mlp", scales=False, k_split=0, block=(16, 128, 128)),
    "cfg4": dict(m=8192, n=8192, k=8192, dtype="fp8", seed=3, dist="normal", scales=True, k_split=0, block=(128, 128, 128)),
    "cfg5_nshard": dict(m=16384, n=28672, k=8192, dtype="bf16", seed=4, dist="mlp", scales=False, k_split=0, block=(128, 128, 128)),
    "cfg5_kshard": dict(m=16384, n=28672, k=8192, dtype="bf16", seed=4, dist="mlp", scales=False, k_split=0, block=(128, 128, 128)),
    "cfg5_kshard_fused": dict(m=16384, n=28672, k=8192, dtype="bf16", seed=4, dist="mlp", scales=False, k_split=0, block=(128, 128, 128)),
    "cfg5_kshard_fused_bf16": dict(m=16384, n=28672, k=8192, dtype="bf16", seed=4, dist="mlp", scales=False, k_split=0, block=(128, 128, 128)),
    # fused attention forward, the reference's benchmark shapes (06-fused-attention.py:737-763): BATCH 4, 32 heads, fp16
    "attn_d64": dict(attn=True, z=4, h=32, n_ctx=4096, d=64, causal=False, dtype="f16", seed=6),
    "attn_d64_causal": dict(attn=True, z=4, h=32, n_ctx=4096, d=64, causal=True, dtype="f16", seed=6),
    "attn_d128": dict(attn=True, z=4, h=32, n_ctx=4096, d=128, causal=False, dtype="f16", seed=6),
    "attn_d128_causal": dict(attn=True, z=4, h=32, n_ctx=4096, d=128, causal=True, dtype="f16", seed=6),
    "attn_d64_16k_causal": dict(attn=True, z=4, h=32, n_ctx=16384, d=64, causal=True, dtype="f16", seed=6),
    # backward of the same (the reference benchmarks it causal only, :742-744); FLOPs = 2.5 x forward (:799-800)
    "attn_bwd_d64_causal": dict(attn=True, bwd=True, z=4, h=32, n_ctx=4096, d=64, causal=True, dtype="f16", seed=6),
}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int, period_s: float = 0.005):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self) -> dict:
        self._halt.set()
        if self.is_alive():
            self.join(1.0)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ------------------------------------------------------------------------------------------------------
# synthetic inputs (seeded on the CPU; shapes, dtypes and value distributions of BASELINE.json)
# ------------------------------------------------------------------------------------------------------
def torch_dtype(name: str):
    import torch
    return {"bf16": torch.bfloat16, "fp16": torch.float16, "fp8": torch.float8_e4m3fn}[name]


def draw(rows, cols, dist, gen, std=1.0):
    import torch
    if dist == "uniform":
        return torch.rand(rows, cols, generator=gen) * 2 - 1
    return torch.randn(rows, cols, generator=gen) * std


def shard_shape(name: str, w: dict, rank: int, world: int) -> dict:
    """Per-rank problem: (m, n, k), which operand is sharded, and how the job's FLOPs are counted."""
    from triton_ext_b200.parallel import split_range
    m, n, k = w["m"], w["n"], w["k"]
    if name == "cfg5_nshard":
        n0, n1 = split_range(n, world, rank, align=256)
        return dict(m=m, n=n1 - n0, k=k, scaling="strong", job_flops=2.0 * m * n * k, parallelism=f"n-sharded x{world}")
    if name.startswith("cfg5_kshard"):
        k0, k1 = split_range(k, world, rank, align=128)
        return dict(m=m, n=n, k=k1 - k0, scaling="strong", job_flops=2.0 * m * n * k, parallelism=f"k-sharded x{world} + reduce-scatter")
    # every rank runs one full-size problem: its own column panel of an N-times-wider GEMM
    return dict(m=m, n=n, k=k, scaling="weak", job_flops=2.0 * m * n * k * world,
                parallelism="single GPU" if world == 1 else f"n-sharded x{world} (one {n}-column panel per rank)")


def make_host_inputs(w: dict, shp: dict, rank: int):
    import torch
    gen = torch.Generator().manual_seed(w["seed"] + 1000 * rank)
    dt = torch_dtype(w["dtype"])
    a = draw(shp["m"], shp["k"], w["dist"], gen).to(dt)
    b = draw(shp["k"], shp["n"], w["dist"], gen, 0.02 if w["dist"] == "mlp" else 1.0).to(dt)
    rs = cs = None
    if w["scales"]:
        rs = torch.rand(shp["m"], generator=gen) * 1.5 + 0.5
        cs = torch.rand(shp["n"], generator=gen) * 1.5 + 0.5
    return a, b, rs, cs


# ------------------------------------------------------------------------------------------------------
# CPU legs: the same tt.dot through Triton's interpreter (oracle/interp_dot.py) on a bounded tile sample
# ------------------------------------------------------------------------------------------------------
def cpu_baseline_single_core(name: str, w: dict, budget_s: float = 12.0) -> dict:
    import torch
    from oracle.interp_dot import interp_dot, sample_tiles
    shp = shard_shape(name, w, 0, 1)
    bm, bn, bk = w["block"]
    m, n, k = (min(shp["m"], 1024), min(shp["n"], 2048), shp["k"]) if name.startswith("cfg5") or name == "cfg4" else (shp["m"], shp["n"], shp["k"])
    sub = dict(shp, m=m, n=n)
    a, b, rs, cs = make_host_inputs(w, sub, 0)
    out_dtype = torch.bfloat16
    ids = sample_tiles(m, n, bm, bn, 4096, seed=w["seed"])
    done, t0 = 0, time.perf_counter()
    batch = 2
    while done < len(ids) and time.perf_counter() - t0 < budget_s:
        interp_dot(a, b, out_dtype=out_dtype, block_m=bm, block_n=bn, block_k=bk, row_scale=rs, col_scale=cs,
                   tile_ids=ids[done:done + batch])
        done += min(batch, len(ids) - done)
    dt = time.perf_counter() - t0
    flops = 2.0 * min(bm, m) * bn * k * done
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": "port",
            "sample": f"{done} output tiles of {bm}x{bn} (BLOCK_K {bk}, full K={k}) through Triton's CPU interpreter, {dt:.1f} s",
            "seconds": dt}


_REF = {}


def _ref_init(a, b, rs, cs, block):
    os.environ["OMP_NUM_THREADS"] = "1"
    import torch
    torch.set_num_threads(1)
    _REF.update(a=a, b=b, rs=rs, cs=cs, block=block)


def _ref_tiles(ids):
    import torch
    from oracle.interp_dot import interp_dot
    bm, bn, bk = _REF["block"]
    interp_dot(_REF["a"], _REF["b"], out_dtype=torch.bfloat16, block_m=bm, block_n=bn, block_k=bk,
               row_scale=_REF["rs"], col_scale=_REF["cs"], tile_ids=ids)
    return len(ids)


def run_reference_arm(args, name: str, w: dict) -> dict:
    """The reference's CPU implementation of the path on all host cores: a process pool of interpreter
    workers, each step a bounded sample of output tiles."""
    import torch
    import torch.multiprocessing as mp
    from oracle.interp_dot import sample_tiles
    cores = len(os.sched_getaffinity(0))
    shp = shard_shape(name, w, 0, 1)
    bm, bn, bk = w["block"]
    m, n, k = shp["m"], shp["n"], shp["k"]
    if m * k + k * n > 200e6:  # cfg5: draw only the rows / columns the sample touches
        m, n = min(m, 2048), min(n, 4096)
    a, b, rs, cs = make_host_inputs(w, dict(shp, m=m, n=n), 0)
    for t in (a, b, rs, cs):
        if t is not None:
            t.share_memory_()
    # One tile per worker per step (a few tenths of a second) keeps a --steps 200 run within minutes.
    per_worker = {"cfg3": 4}.get(name, 1)
    tiles_per_step = cores * per_worker
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[var] = "1"  # inherited by the workers: one BLAS thread per interpreter process
    all_ids = sample_tiles(m, n, bm, bn, 1 << 20, seed=w["seed"])
    ctx = mp.get_context("spawn")
    with ctx.Pool(cores, initializer=_ref_init, initargs=(a, b, rs, cs, w["block"])) as pool:
        def step(i):
            lo = (i * tiles_per_step) % max(1, len(all_ids) - tiles_per_step + 1)
            ids = all_ids[lo:lo + tiles_per_step]
            chunks = [ids[j::cores] for j in range(cores) if len(ids[j::cores])]
            return sum(pool.map(_ref_tiles, chunks))
        for i in range(args.warmup):
            step(i)
        t0 = time.perf_counter()
        tiles = 0
        for i in range(args.steps):
            tiles += step(args.warmup + i)
        dt = time.perf_counter() - t0
    flops = 2.0 * min(bm, m) * bn * k * tiles
    value = flops / dt / 1e12
    unit = "TFLOP/s"
    sample = (f"{tiles_per_step} output tiles of {bm}x{bn} per step (BLOCK_K {bk}, full K={k}) through Triton's CPU "
              f"interpreter, {cores} worker processes")
    return {"metric": "tt.dot TFLOP/s", "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt / max(1, args.steps) * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic", "impl": "reference",
            "config": {"workload": name, "m": shp["m"], "n": shp["n"], "k": shp["k"]},
            "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


# ------------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------------
def run_gpu_arm(args, name: str, w: dict) -> dict | None:
    import torch
    import torch.distributed as dist
    from triton_ext_b200 import backend as B
    from triton_ext_b200 import parallel as par

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the b200_dot backend has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    shp = shard_shape(name, w, rank, world)
    m, n, k = shp["m"], shp["n"], shp["k"]
    in_dt = torch_dtype(w["dtype"])
    out_dt = torch.bfloat16
    fused = name.startswith("cfg5_kshard_fused") and world > 1
    kshard = name.startswith("cfg5_kshard") and world > 1 and not fused
    a_h, b_h, rs_h, cs_h = make_host_inputs(w, shp, rank)
    a_h, b_h = a_h.pin_memory(), b_h.pin_memory()
    step_out_dt = torch.float32 if kshard else out_dt
    c_h = torch.empty((m, n), dtype=step_out_dt).pin_memory() if not kshard else None

    es = a_h.element_size()
    set_bytes = (m * k + k * n) * es + m * n * (4 if kshard else 2)
    n_sets = 1 if set_bytes > L2_BYTES else min(8, L2_BYTES // set_bytes + 2)
    sets = []
    for _ in range(n_sets):
        sets.append((a_h.to(dev), b_h.to(dev), torch.empty((m, n), dtype=step_out_dt, device=dev)))
    rs_d = rs_h.to(dev) if rs_h is not None else None
    cs_d = cs_h.to(dev) if cs_h is not None else None

    fused_op = None
    if fused:
        pdt = torch.bfloat16 if name.endswith("_bf16") else torch.float32
        fused_op = par.FusedKShardedDot(m, n, k, in_dt, out_dt, partial_dtype=pdt, device=dev)
    cfg = B.make_config(k_split_point=w["k_split"]) if w["k_split"] else None
    pr = B.make_problem(m, n, k, in_dt, step_out_dt, row_scale=rs_h is not None and not kshard,
                        col_scale=cs_h is not None and not kshard)
    plan = B.DotPlan(pr, cfg)
    info = plan.info
    stream = torch.cuda.current_stream(dev)

    def gemm(i):
        a_d, b_d, c_d = sets[i % n_sets]
        plan.run(a_d, b_d, c_d, None if kshard else rs_d, None if kshard else cs_d, stream)
        return c_d

    if w.get("jit"):
        # The user-facing call is kernel[grid](...) of a Triton kernel; Triton's front end, the K-loop proof and
        # the pass pipeline run once, then every launch is tx_dot_run behind Triton's launcher interface.
        from triton.runtime.driver import driver as triton_driver
        from triton_ext_b200 import triton_backend as tbk
        from triton_ext_b200.triton_backend import driver as tb_driver, kernels as tb_kernels

        tbk.install()
        triton_driver.set_active(tb_driver.B200DotDriver())

        def gemm(i):  # noqa: F811
            a_d, b_d, c_d = sets[i % n_sets]
            tb_kernels.launch_dot_kloop(a_d, b_d, c_d, block=w["block"], k_main=w["k_split"])
            return c_d

    if kshard:
        rows = m // world
        scat = torch.empty((rows, n), dtype=torch.float32, device=dev)
        final = torch.empty((rows, n), dtype=out_dt, device=dev)

        def step(i):
            part = gemm(i)
            dist.reduce_scatter_tensor(scat, part, op=dist.ReduceOp.SUM)
            final.copy_(scat)  # cast epilogue after the reduction
    elif fused:
        def step(i):
            a_d, b_d, _ = sets[i % n_sets]
            return fused_op(a_d, b_d)
    else:
        step = gemm

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    sampler = ClockSampler(local_rank)
    sampler.start()
    for i in range(args.warmup):
        step(i)
    barrier()
    launches0 = B.kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    barrier()
    launches = B.kernel_launches() - launches0
    clocks = sampler.stop()
    plan.check(stream)
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        lt = torch.tensor([float(launches)], device=dev)
        dist.all_reduce(lt, op=dist.ReduceOp.SUM)
        launches = int(lt.item())
    ms_per_step = ms / args.steps
    job_flops = shp["job_flops"]
    value = job_flops / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the host-buffer entry point (H2D + kernel + D2H every step) -------------------
    e2e_steps = max(1, min(args.steps, 10))
    if kshard or fused:
        def e2e_step(i):
            a_d, b_d, c_d = sets[0]
            a_d.copy_(a_h, non_blocking=True)
            b_d.copy_(b_h, non_blocking=True)
            r = step(0)
            return (r if fused else final).cpu()
        h2d, d2h = (m * k + k * n) * es, (m // world) * n * 2
    elif w.get("jit"):
        def e2e_step(i):
            a_d, b_d, c_d = sets[0]
            a_d.copy_(a_h, non_blocking=True)
            b_d.copy_(b_h, non_blocking=True)
            gemm(0)
            c_h.copy_(c_d, non_blocking=True)
            torch.cuda.synchronize(dev)
        h2d, d2h = (m * k + k * n) * es, m * n * c_h.element_size()
    else:
        def e2e_step(i):
            plan.run_host(a_h, b_h, c_h, rs_h, cs_h)
        h2d = (m * k + k * n) * es + (4 * (m + n) if rs_h is not None else 0)
        d2h = m * n * c_h.element_size()
    e2e_step(0)
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = job_flops / e2e_s / 1e12

    peaks = measured_peaks()
    algo_bytes = info["algorithmic_bytes"]
    launch_s = ms_per_step * 1e-3  # one kernel launch of this library per step
    hbm_bound = name == "cfg3"
    if hbm_bound:
        achieved = algo_bytes / launch_s / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES.get(name),
                "peak_source": f"hbm_gbs of {peaks['_source']}"}
    else:
        per_gpu_flops = info["flops"]
        achieved = per_gpu_flops / launch_s / 1e12
        peak = peaks["bf16_tflops"] * (2.0 if w["dtype"] == "fp8" else 1.0)
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_BYTES.get(name),
                "peak_source": f"bf16_tflops (burst) of {peaks['_source']}" + (" x2 for fp8 (no measured fp8 figure)" if w["dtype"] == "fp8" else "")}
        if kshard or fused:
            roof["note"] = "step time includes the reduce-scatter; achieved is per-GPU GEMM FLOPs over the whole step"

    line = {
        "metric": "tt.dot TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": shp["scaling"],
        "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic (seeded CPU draw, shapes and distributions of BASELINE.json)",
        "config": {"workload": name, "m": w["m"], "n": w["n"] * (world if shp["scaling"] == "weak" and world > 1 else 1), "k": w["k"],
                   "per_gpu": [m, n, k], "parallelism": shp["parallelism"],
                   "kernel": f"{info['block_m']}x{info['block_n']}x{info['block_k']} stages={info['stages']} pair={info['cta_pair']} "
                             f"swap={info['swap_ab']} sched={info['schedule']} grid={info['grid']}",
                   "loop_split": {"main_iters": info["k_main_iters"], "tail_iters": info["k_tail_iters"], "tail_mmas": info["k_tail_mmas"]},
                   "l2": (f"{n_sets} rotating buffer sets, {n_sets * set_bytes / 1e6:.0f} MB > 126 MB L2" if n_sets > 1
                          else f"one buffer set of {set_bytes / 1e6:.0f} MB > 126 MB L2")},
        "roofline": roof,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "steps": e2e_steps},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    if hbm_bound:
        line["gbps"] = roof["achieved"]
    if world > 1:
        dist.destroy_process_group()
    return line if rank == 0 else None


# ---- fused attention forward (the two chained tt.dot of the reference's demo kernel) ------------------------------
ATTN_SM_SCALE = 1.3   # the reference benchmark's value (06-fused-attention.py:785)


def attn_flops(w: dict, z: int) -> float:
    f = 4.0 * z * w["h"] * w["n_ctx"] * w["n_ctx"] * w["d"]
    f = 0.5 * f if w["causal"] else f
    return 2.5 * f if w.get("bwd") else f


def attn_host_inputs(w: dict, rank: int):
    import torch
    g = torch.Generator().manual_seed(w["seed"] + 1000 * rank)
    return [torch.randn((w["z"], w["h"], w["n_ctx"], w["d"]), generator=g).to(torch.float16) for _ in range(3)]


def attn_cpu_sample(w: dict, budget_s: float = 10.0) -> dict:
    """The oracle's blockwise restatement of the reference kernel on (batch 1, head 1) slices of the workload,
    one core; the sequence is cut to 1024 rows so that a slice takes seconds."""
    import torch
    from oracle import attn_oracle as AO
    n = min(w["n_ctx"], 1024)
    g = torch.Generator().manual_seed(w["seed"])
    q, k, v = (torch.randn((1, 1, n, w["d"]), generator=g).to(torch.float16) for _ in range(3))
    torch.set_num_threads(1)
    done, t0 = 0, time.perf_counter()
    d_o = torch.randn(q.shape, generator=g).to(torch.float16)
    while True:
        if w.get("bwd"):
            AO.attention_grads_eager(q, k, v, d_o, w["causal"], ATTN_SM_SCALE)
        else:
            AO.attention_blockwise(q, k, v, w["causal"], ATTN_SM_SCALE, 128, 64)
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    secs = time.perf_counter() - t0
    fl = 4.0 * n * n * w["d"] * (0.5 if w["causal"] else 1.0) * (2.5 if w.get("bwd") else 1.0) * done
    return {"value": fl / secs / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": "port",
            "sample": f"{done} x (1 batch, 1 head, n_ctx {n}, head_dim {w['d']}) of the workload through oracle/attn_oracle.py "
                      + ("(fp32 autograd through the eager formula)" if w.get("bwd") else
                         "(numpy restatement of the reference kernel, BLOCK_M 128, BLOCK_N 64)") + f", {secs:.1f} s"}


def run_attention_reference_arm(args, name: str, w: dict) -> dict:
    """CPU arm: the eager formula of the reference's own test (matmul, softmax, matmul) on all host threads, one
    (batch, head) slice per step."""
    import torch
    from oracle import attn_oracle as AO
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    n = min(w["n_ctx"], 2048)
    g = torch.Generator().manual_seed(w["seed"])
    q, k, v = (torch.randn((1, 1, n, w["d"]), generator=g).to(torch.float16) for _ in range(3))
    d_o = torch.randn(q.shape, generator=g).to(torch.float16)

    def one():
        if w.get("bwd"):
            AO.attention_grads_eager(q, k, v, d_o, w["causal"], ATTN_SM_SCALE)   # forward + backward; FLOPs count the backward
        else:
            AO.attention_eager(q, k, v, w["causal"], ATTN_SM_SCALE)
    for _ in range(args.warmup):
        one()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one()
    secs = (time.perf_counter() - t0) / max(args.steps, 1)
    fl = 4.0 * n * n * w["d"] * (0.5 if w["causal"] else 1.0) * (2.5 if w.get("bwd") else 1.0)
    val = fl / secs / 1e12
    sample = f"one (batch, head) slice per step, n_ctx cut to {n}, eager matmul-softmax-matmul in fp32 on {cores} threads"
    return {"impl": "reference", "metric": "attention bwd TFLOP/s" if w.get("bwd") else "attention fwd TFLOP/s", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded randn)",
            "config": {"workload": name, "z": w["z"], "h": w["h"], "n_ctx": w["n_ctx"], "head_dim": w["d"], "causal": w["causal"]},
            "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def run_attention_gpu_arm(args, name: str, w: dict) -> dict | None:
    """Every rank runs its own batch of `z` sequences (independent (batch, head) pairs: no collective)."""
    import torch
    import torch.distributed as dist
    from triton_ext_b200 import attention as A

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the attention kernel has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    q_h, k_h, v_h = (t.pin_memory() for t in attn_host_inputs(w, rank))
    o_h = torch.empty_like(q_h).pin_memory()
    q, k, v = q_h.to(dev), k_h.to(dev), v_h.to(dev)
    out = torch.empty_like(q)
    set_bytes = 4 * q.numel() * 2
    if set_bytes <= L2_BYTES:
        raise RuntimeError("attention workload smaller than L2: add rotating buffers before timing it")

    bwd = bool(w.get("bwd"))
    if bwd:
        g = torch.Generator().manual_seed(w["seed"] + 7)
        do_h = torch.randn(q_h.shape, generator=g).to(torch.float16).pin_memory()
        d_o = do_h.to(dev)
        o_fwd, m_fwd = A.attention_forward(q, k, v, w["causal"], ATTN_SM_SCALE, return_m=True, check=True)

        def step(i):
            return A.attention_backward(q, k, v, o_fwd, m_fwd, d_o, w["causal"], ATTN_SM_SCALE)
    else:
        def step(i):
            A.attention_forward(q, k, v, w["causal"], ATTN_SM_SCALE, out=out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    stream = torch.cuda.current_stream(dev)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for i in range(args.warmup):
        step(i)
    barrier()
    launches0 = A.kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    barrier()
    launches = A.kernel_launches() - launches0
    clocks = sampler.stop()
    A.check(dev)
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms, float(launches)], device=dev)
        dist.all_reduce(t[:1], op=dist.ReduceOp.MAX)
        dist.all_reduce(t[1:], op=dist.ReduceOp.SUM)
        ms, launches = float(t[0].item()), int(t[1].item())
    ms_per_step = ms / args.steps
    per_gpu_flops = attn_flops(w, w["z"])
    value = per_gpu_flops * world / (ms_per_step * 1e-3) / 1e12

    e2e_steps = max(1, min(args.steps, 10))
    if bwd:
        oh, mh = o_fwd.cpu().pin_memory(), m_fwd.cpu().pin_memory()
        grads_h = [torch.empty_like(q_h).pin_memory() for _ in range(3)]

        def e2e_step():
            # inputs of the backward from pinned host memory, the three gradients back to it
            dev_in = [t.to(dev, non_blocking=True) for t in (q_h, k_h, v_h, oh, do_h)]
            grads = A.attention_backward(*dev_in[:4], mh.to(dev, non_blocking=True), dev_in[4], w["causal"], ATTN_SM_SCALE)
            for dst, src in zip(grads_h, grads):
                dst.copy_(src, non_blocking=True)
            torch.cuda.synchronize(dev)
        h2d_bytes, d2h_bytes = 5 * q.numel() * 2 + m_fwd.numel() * 4, 3 * q.numel() * 2
    else:
        def e2e_step():
            A.attention_forward_host(q_h, k_h, v_h, w["causal"], ATTN_SM_SCALE, out=o_h)
        h2d_bytes, d2h_bytes = 3 * q.numel() * 2, q.numel() * 2
    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())

    peaks = measured_peaks()
    achieved = per_gpu_flops / (ms_per_step * 1e-3) / 1e12
    sm_mhz = clocks.get("sm_mhz") or 1965
    sfu_bound = 4.0 * w["d"] * 16 * 148 * sm_mhz * 1e6 / 1e12   # one exp2 per score, 16 per clock per SM
    algo_bytes = 4 * q.numel() * 2 + q.numel() // w["d"] * 4
    line = {
        "metric": "attention bwd TFLOP/s" if bwd else "attention fwd TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": w["dtype"], "data": "synthetic (seeded randn, the reference benchmark's shapes and sm_scale)",
        "config": {"workload": name, "z": w["z"] * world, "h": w["h"], "n_ctx": w["n_ctx"], "head_dim": w["d"],
                   "causal": w["causal"], "per_gpu": [w["z"], w["h"], w["n_ctx"], w["d"]],
                   "parallelism": "batch-sharded, no collective" if world > 1 else "single GPU",
                   "kernel": ("per head: 5 tt.dot GEMMs + 3 element-wise kernels, 4 heads in flight" if bwd else
                              "256 query rows per CTA (2 x 128), KV blocks of 128, tcgen05 + TMEM"),
                   "l2": f"one buffer set of {set_bytes / 1e6:.0f} MB > 126 MB L2"},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["bf16_tflops"], "traffic": NCU_TRAFFIC_BYTES.get(name),
                     "peak_source": f"bf16_tflops (burst) of {peaks['_source']}",
                     "note": f"exp2 on the SFU (16 per clock per SM) bounds this shape at {sfu_bound:.0f} TFLOP/s; "
                             f"algorithmic bytes {algo_bytes / 1e6:.0f} MB"},
        "e2e": {"value": per_gpu_flops * world / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d_bytes),
                "d2h_bytes_per_step": int(d2h_bytes), "steps": e2e_steps},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    if world > 1:
        dist.destroy_process_group()
    return line if rank == 0 else None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-baseline-only", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.cpu_baseline_only:
        cb = cpu_baseline_single_core(args.workload, w)
        cb.pop("seconds", None)
        print(json.dumps(cb), flush=True)
        return

    if args.impl == "reference":
        if rank != 0:
            return  # the CPU arm runs once, on rank 0
        arm = run_attention_reference_arm if w.get("attn") else run_reference_arm
        print(json.dumps(arm(args, args.workload, w)), flush=True)
        return

    if w.get("attn"):
        line = run_attention_gpu_arm(args, args.workload, w)
        if line is None:
            return
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = attn_cpu_sample(w)
        print(json.dumps(line), flush=True)
        return

    line = run_gpu_arm(args, args.workload, w)
    if line is None:
        return
    if world == 1 and not args.no_cpu_baseline:
        if w.get("jit"):
            # The interpreter oracle needs TRITON_INTERPRET=1 from before Triton is imported; this process has
            # imported Triton's compiler for the timed arm, so the CPU leg runs in a process of its own.
            import subprocess
            out = subprocess.run([sys.executable, os.path.abspath(__file__), "--workload", args.workload, "--cpu-baseline-only"],
                                 capture_output=True, text=True, check=True)
            cb = json.loads(out.stdout.strip().splitlines()[-1])
        else:
            cb = cpu_baseline_single_core(args.workload, w)
            cb.pop("seconds", None)
        line["cpu_baseline"] = cb
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
