"""Benchmark of the tt.dot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference] [--no-also]

A step is one pass of the hot path over one batch of synthetic input: one tt.dot GEMM launched
through the C-ABI (tx_dot_run), plus its exchange where the K dimension is sharded.
Workloads (BASELINE.json `configs`):

    cfg5         bf16 16384x28672x8192, the multi-GPU configuration. Default. One GPU computes the whole GEMM;
                 N GPUs split the columns of B and C (N-sharded, no collective): strong scaling.
                 (`cfg5_nshard` is the same workload.)
    cfg5_kshard  same GEMM, K split over the ranks, fp32 partials, NCCL reduce-scatter, cast.
    cfg5_kshard_fused[_bf16]  K split over the ranks, the GEMM epilogue stores partial tiles into the owning
                 rank's memory over NVLink (fp32 or bf16 partials), then one local slot reduction.
    cfg2         bf16 4096x4096x4160, LoopSplit tail (BLOCK_K 128: main [0,4096) + 64-wide remainder).
                 At N GPUs each rank runs its own column panel of a 4096 x (4096*N) x 4160 GEMM: weak scaling.
    cfg2_jit     cfg2 launched as a @triton.jit kernel through the package's Triton backend.
    cfg3         bf16 16x14336x4096 decode shape; HBM-bound, roofline in GB/s.
    cfg4         fp8 e4m3 8192^3 with per-row / per-column fp32 scales -> bf16.
    attn_d64[_causal], attn_d128[_causal], attn_d64_16k_causal, attn_bwd_d64_causal, attn_d64_fp8, attn_d128_fp8[_causal]
                 the next row after the GEMM: fused attention (two chained tt.dot + online softmax)
                 on the reference benchmark's shapes (batch 4, 32 heads, fp16).

One JSON line is printed by rank 0. The line of the default run carries, under "also", one compact record per
further workload run in the same process: cfg2, cfg3, cfg4 at one GPU; the three K-sharded forms at N > 1.
Every GEMM record carries a "check": the rank's output against an fp32 matmul of the same (upcast) operands on
sampled rows and columns plus the edges; a failed check makes the process exit non-zero after printing.
`--impl reference` times the reference's CPU path for the same workload (the same tt.dot run by Triton's
interpreter on the host cores) on a bounded tile sample.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024

# dram__bytes_read.sum + dram__bytes_write.sum per launch, copied from the committed ncu captures (the file named
# beside each figure gives the command); None where no capture exists. These are citations of a profile, not
# measurements of the run that prints them.
NCU_TRAFFIC = {
    "cfg5": (7.99e9, "profiles/dot_umma_pair_kernel_cfg5_bf16_16384x28672x8192_dram_traffic.md"),
    "cfg2": (107.9e6, "profiles/dot_umma_pair_kernel_cfg2_bf16_4096x4096x4160.md"),
    "cfg3": (122.0e6, "profiles/dot_umma_kernel_cfg3_bf16_16x14336x4096.md"),
    "cfg4": (365.9e6, "profiles/dot_umma_pair_f8_kernel_cfg4_fp8_8192x8192x8192.md"),
    "attn_d64": (386.4e6, "profiles/attn_fwd_kernel_f16_batch4_heads32_nctx4096_d64.md"),
}


def measured_peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "_source": "fallback"}


CFG5 = dict(m=16384, n=28672, k=8192, dtype="bf16", seed=4, dist="mlp", scales=False, k_split=0, block=(128, 128, 128))
WORKLOADS = {
    "cfg5": dict(CFG5),
    "cfg5_nshard": dict(CFG5),
    "cfg5_kshard": dict(CFG5),
    "cfg5_kshard_fused": dict(CFG5),
    "cfg5_kshard_fused_bf16": dict(CFG5),
    "cfg2": dict(m=4096, n=4096, k=4160, dtype="bf16", seed=1, dist="uniform", scales=False, k_split=4096, block=(128, 128, 128)),
    # cfg2 launched as a @triton.jit K-loop kernel through the package's Triton backend (same library kernel underneath)
    "cfg2_jit": dict(m=4096, n=4096, k=4160, dtype="bf16", seed=1, dist="uniform", scales=False, k_split=4096, block=(128, 128, 128), jit=True),
    "cfg3": dict(m=16, n=14336, k=4096, dtype="bf16", seed=2, dist="mlp", scales=False, k_split=0, block=(16, 128, 128)),
    "cfg4": dict(m=8192, n=8192, k=8192, dtype="fp8", seed=3, dist="normal", scales=True, k_split=0, block=(128, 128, 128)),
    # fused attention forward, the reference's benchmark shapes (06-fused-attention.py:737-763): BATCH 4, 32 heads, fp16
    "attn_d64": dict(attn=True, z=4, h=32, n_ctx=4096, d=64, causal=False, dtype="f16", seed=6),
    "attn_d64_causal": dict(attn=True, z=4, h=32, n_ctx=4096, d=64, causal=True, dtype="f16", seed=6),
    "attn_d128": dict(attn=True, z=4, h=32, n_ctx=4096, d=128, causal=False, dtype="f16", seed=6),
    "attn_d128_causal": dict(attn=True, z=4, h=32, n_ctx=4096, d=128, causal=True, dtype="f16", seed=6),
    "attn_d64_16k_causal": dict(attn=True, z=4, h=32, n_ctx=16384, d=64, causal=True, dtype="f16", seed=6),
    # backward of the same (the reference benchmarks it causal only, :742-744); FLOPs = 2.5 x forward (:799-800)
    # the reference benchmark's fp8 forward (q, k, v, out float8_e5m2, V with n_ctx contiguous; 06-fused-attention.py:774-779)
    "attn_d64_fp8": dict(attn=True, z=4, h=32, n_ctx=4096, d=64, causal=False, dtype="fp8e5m2", seed=6),
    "attn_d128_fp8": dict(attn=True, z=4, h=32, n_ctx=4096, d=128, causal=False, dtype="fp8e5m2", seed=6),
    "attn_d128_fp8_causal": dict(attn=True, z=4, h=32, n_ctx=4096, d=128, causal=True, dtype="fp8e5m2", seed=6),
    "attn_bwd_d64_causal": dict(attn=True, bwd=True, z=4, h=32, n_ctx=4096, d=64, causal=True, dtype="f16", seed=6),
}
DEFAULT_WORKLOAD = "cfg5"
ALSO_ONE_GPU = ["cfg2", "cfg3", "cfg4"]
ALSO_MULTI_GPU = ["cfg5_kshard", "cfg5_kshard_fused", "cfg5_kshard_fused_bf16"]


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int, period_s: float = 0.001):
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
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_min_mhz": s[0] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def sample_clocks(local_rank: int):
    s = ClockSampler(local_rank)
    s.start()
    return s


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


def partition(name: str, world: int) -> str:
    """How a workload is cut over `world` ranks: "n" (columns of B and C), "k" (K blocks + exchange),
    "panel" (every rank its own full-size problem: weak scaling)."""
    if world == 1:
        return "none"
    if name in ("cfg5", "cfg5_nshard"):
        return "n"
    if name.startswith("cfg5_kshard"):
        return "k"
    return "panel"


def shard_shape(name: str, w: dict, rank: int, world: int) -> dict:
    """Per-rank problem: (m, n, k), and how the job's FLOPs are counted."""
    from triton_ext_b200.parallel import split_range
    m, n, k = w["m"], w["n"], w["k"]
    part = partition(name, world)
    if part == "n":
        n0, n1 = split_range(n, world, rank, align=256)
        return dict(m=m, n=n1 - n0, k=k, lo=n0, scaling="strong", job_flops=2.0 * m * n * k, parallelism=f"n-sharded x{world}, no collective")
    if part == "k":
        k0, k1 = split_range(k, world, rank, align=128)
        how = {"cfg5_kshard": "NCCL reduce-scatter of fp32 partials",
               "cfg5_kshard_fused": "partial tiles stored into the owner's memory by the GEMM epilogue (fp32 slots)",
               "cfg5_kshard_fused_bf16": "partial tiles stored into the owner's memory by the GEMM epilogue (bf16 slots)"}[name]
        return dict(m=m, n=n, k=k1 - k0, lo=k0, scaling="strong", job_flops=2.0 * m * n * k, parallelism=f"k-sharded x{world}, {how}")
    if part == "panel":
        return dict(m=m, n=n, k=k, lo=0, scaling="weak", job_flops=2.0 * m * n * k * world,
                    parallelism=f"n-sharded x{world} (one {n}-column panel per rank), no collective")
    # a K-sharded name on one GPU degenerates to the plain GEMM
    return dict(m=m, n=n, k=k, lo=0, scaling="strong" if name.startswith("cfg5") else "weak", job_flops=2.0 * m * n * k,
                parallelism="single GPU")


def make_host_inputs(name: str, w: dict, shp: dict, rank: int, world: int):
    """This rank's operands of one global problem. The replicated operand comes from the workload's seed on every
    rank; a sharded operand is drawn per shard (seed + 1000 * (rank + 1)), so the global matrix is the concatenation
    of the shards and no rank draws more than it holds."""
    import torch
    dt = torch_dtype(w["dtype"])
    std_b = 0.02 if w["dist"] == "mlp" else 1.0
    part = partition(name, world)
    g_all = torch.Generator().manual_seed(w["seed"])
    g_own = torch.Generator().manual_seed(w["seed"] + 1000 * (rank + 1))
    if part == "none":
        a = draw(shp["m"], shp["k"], w["dist"], g_all)
        b = draw(shp["k"], shp["n"], w["dist"], g_all, std_b)
        g_scale = g_all
    elif part in ("n", "panel"):
        a = draw(shp["m"], shp["k"], w["dist"], g_all)          # replicated
        b = draw(shp["k"], shp["n"], w["dist"], g_own, std_b)   # this rank's columns
        g_scale = g_own
    else:
        a = draw(shp["m"], shp["k"], w["dist"], g_own)          # this rank's K columns of A
        b = draw(shp["k"], shp["n"], w["dist"], g_own, std_b)   # this rank's K rows of B
        g_scale = g_all
    a, b = a.to(dt), b.to(dt)
    rs = cs = None
    if w["scales"]:
        rs = torch.rand(shp["m"], generator=g_scale) * 1.5 + 0.5
        cs = torch.rand(shp["n"], generator=g_scale) * 1.5 + 0.5
    return a, b, rs, cs


def plan_config_kw(w: dict) -> dict:
    return dict(k_split_point=w["k_split"]) if w["k_split"] else {}


def buffer_sets(m: int, n: int, k: int, es: int, out_bytes: int):
    set_bytes = (m * k + k * n) * es + m * n * out_bytes
    n_sets = 1 if set_bytes > L2_BYTES else min(8, L2_BYTES // set_bytes + 2)
    return set_bytes, n_sets


def config_dict(name: str, w: dict, world: int) -> dict:
    """The `config` object of the JSON line. Computed without a GPU (the tile choice comes from
    tx_dot_plan_preview), so the b200 arm and the reference arm print the same object."""
    import torch
    from triton_ext_b200 import backend as B
    shp = shard_shape(name, w, 0, world)
    m, n, k = shp["m"], shp["n"], shp["k"]
    part = partition(name, world)
    out_dt = torch.float32 if (part == "k" and name == "cfg5_kshard") else torch.bfloat16
    if part == "k" and name == "cfg5_kshard_fused":
        out_dt = torch.float32
    kw = plan_config_kw(w)
    if part == "k" and name != "cfg5_kshard":
        kw.update(schedule=B.TXD_SCHED_DATA_PARALLEL, swap_ab=2)
    pr = B.make_problem(m, n, k, torch_dtype(w["dtype"]), out_dt, row_scale=w["scales"] and part != "k",
                        col_scale=w["scales"] and part != "k")
    info = B.preview(pr, B.make_config(**kw) if kw else None)
    es = 1 if w["dtype"] == "fp8" else 2
    set_bytes, n_sets = buffer_sets(m, n, k, es, 4 if out_dt == torch.float32 else 2)
    return {"workload": name, "m": w["m"], "n": w["n"] * (world if shp["scaling"] == "weak" and world > 1 else 1), "k": w["k"],
            "per_gpu": [m, n, k], "parallelism": shp["parallelism"],
            "kernel": f"{info['block_m']}x{info['block_n']}x{info['block_k']} stages={info['stages']} pair={info['cta_pair']} "
                      f"swap={info['swap_ab']} sched={info['schedule']} grid={info['grid']}",
            "loop_split": {"main_iters": info["k_main_iters"], "tail_iters": info["k_tail_iters"], "tail_mmas": info["k_tail_mmas"]},
            "l2": (f"{n_sets} rotating buffer sets, {n_sets * set_bytes / 1e6:.0f} MB > 126 MB L2" if n_sets > 1
                   else f"one buffer set of {set_bytes / 1e6:.0f} MB > 126 MB L2")}


# ------------------------------------------------------------------------------------------------------
# CPU legs: the same tt.dot through Triton's interpreter (oracle/interp_dot.py) on a bounded tile sample
# ------------------------------------------------------------------------------------------------------
def cpu_sample_inputs(name: str, w: dict, m_cap: int, n_cap: int):
    shp = shard_shape(name, w, 0, 1)
    big = name.startswith("cfg5") or name == "cfg4"
    m, n = (min(shp["m"], m_cap), min(shp["n"], n_cap)) if big else (shp["m"], shp["n"])
    sub = dict(shp, m=m, n=n)
    return sub, make_host_inputs(name, w, sub, 0, 1)


def cpu_baseline_single_core(name: str, w: dict, budget_s: float = 12.0) -> dict:
    import torch
    from oracle.interp_dot import interp_dot, sample_tiles
    bm, bn, bk = w["block"]
    sub, (a, b, rs, cs) = cpu_sample_inputs(name, w, 1024, 2048)
    m, n, k = sub["m"], sub["n"], sub["k"]
    ids = sample_tiles(m, n, bm, bn, 4096, seed=w["seed"])
    done, t0 = 0, time.perf_counter()
    batch = 2
    while done < len(ids) and time.perf_counter() - t0 < budget_s:
        interp_dot(a, b, out_dtype=torch.bfloat16, block_m=bm, block_n=bn, block_k=bk, row_scale=rs, col_scale=cs,
                   tile_ids=ids[done:done + batch])
        done += min(batch, len(ids) - done)
    dt = time.perf_counter() - t0
    flops = 2.0 * min(bm, m) * bn * k * done
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": "port",
            "sample": f"{done} output tiles of {bm}x{bn} (BLOCK_K {bk}, full K={k}) through Triton's CPU interpreter, {dt:.1f} s"}


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
    workers, each step a bounded sample of output tiles of the workload's whole (unsharded) GEMM."""
    import torch.multiprocessing as mp
    from oracle.interp_dot import sample_tiles
    cores = len(os.sched_getaffinity(0))
    bm, bn, bk = w["block"]
    sub, (a, b, rs, cs) = cpu_sample_inputs(name, w, 2048, 4096)
    m, n, k = sub["m"], sub["n"], sub["k"]
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
    shp = shard_shape(name, w, 0, max(1, args.gpus))
    return {"metric": "tt.dot TFLOP/s", "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt / max(1, args.steps) * 1e3, "higher_is_better": True,
            "scaling": shp["scaling"], "vs_baseline": None, "dtype": w["dtype"],
            "data": "synthetic (seeded CPU draw, shapes and distributions of BASELINE.json)", "impl": "reference",
            "config": config_dict(name, w, max(1, args.gpus)),
            "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


# ------------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------------
class Ctx:
    def __init__(self):
        import torch
        import torch.distributed as dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise RuntimeError("bench.py needs a CUDA device: the b200_dot backend has no CPU path")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.dist = dist
        self.torch = torch

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return float(x)
        t = self.torch.tensor([float(x)], device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return float(x)
        t = self.torch.tensor([float(x)], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def timed_window(ctx: Ctx, step, steps: int, stream, first: int = 0) -> float:
    """Device time of exactly `steps` steps in ms: barrier + synchronize on both sides, CUDA events on the launching
    stream, max over ranks."""
    torch = ctx.torch
    ctx.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        step(first + i)
    e1.record(stream)
    ctx.barrier()
    return ctx.max_over_ranks(e0.elapsed_time(e1))


def rows_to_check(m: int, tile_rows: int, count: int, seed: int):
    """First and last row, both sides of the first tile-row boundary and of the middle one, plus a seeded sample."""
    import torch
    g = torch.Generator().manual_seed(seed)
    fixed = [0, m - 1, min(tile_rows - 1, m - 1), min(tile_rows, m - 1), (m // 2 // tile_rows) * tile_rows, max((m // 2 // tile_rows) * tile_rows - 1, 0)]
    extra = torch.randint(0, m, (max(count - len(fixed), 0),), generator=g).tolist()
    return sorted(set(fixed + extra))


def check_against_fp32(got, ref, extra_bound=None, rtol=1e-2, atol=1e-2) -> dict:
    """|got - ref| <= atol + rtol * |ref| (+ extra_bound) element-wise; ref is an fp32 matmul of the upcast operands."""
    diff = (got.float() - ref).abs()
    bound = atol + rtol * ref.abs()
    if extra_bound is not None:
        bound = bound + extra_bound
    bad = int((diff > bound).sum().item())
    return {"max_err": float(diff.max().item()), "max_ref": float(ref.abs().max().item()), "elements": int(diff.numel()), "bad": bad}


def merge_checks(parts: list, tol_text: str) -> dict:
    out = {"max_err": max(p["max_err"] for p in parts), "max_ref": max(p["max_ref"] for p in parts),
           "elements": sum(p["elements"] for p in parts), "bad": sum(p["bad"] for p in parts), "tol": tol_text}
    out["ok"] = out["bad"] == 0 and math.isfinite(out["max_err"])
    return out


def run_dot_workload(ctx: Ctx, args, name: str, w: dict, headline: bool) -> dict:
    """Times one GEMM workload on this rank's GPU and returns its record (rank 0's view; times are max over ranks)."""
    torch, dist = ctx.torch, ctx.dist
    from triton_ext_b200 import backend as B
    from triton_ext_b200 import parallel as par

    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    shp = shard_shape(name, w, rank, world)
    part = partition(name, world)
    m, n, k = shp["m"], shp["n"], shp["k"]
    in_dt, out_dt = torch_dtype(w["dtype"]), torch.bfloat16
    fused = part == "k" and name.startswith("cfg5_kshard_fused")
    kshard = part == "k" and not fused
    slot_dt = torch.bfloat16 if name.endswith("_bf16") else torch.float32
    steps = args.steps if headline else max(3, min(args.steps, 50))
    warmup = args.warmup

    a_h, b_h, rs_h, cs_h = make_host_inputs(name, w, shp, rank, world)
    step_out_dt = torch.float32 if kshard else out_dt
    es = a_h.element_size()
    set_bytes, n_sets = buffer_sets(m, n, k, es, 4 if kshard else 2)
    sets = []
    for _ in range(n_sets):
        c_d = None if fused else torch.empty((m, n), dtype=step_out_dt, device=dev)
        sets.append((a_h.to(dev), b_h.to(dev), c_d))
    use_scales = rs_h is not None and part != "k"
    rs_d = rs_h.to(dev) if use_scales else None
    cs_d = cs_h.to(dev) if use_scales else None

    fused_op = None
    plan = None
    if fused:
        fused_op = par.FusedKShardedDot(m, n, k, in_dt, out_dt, partial_dtype=slot_dt, device=dev, config_kw=plan_config_kw(w),
                                        parts=args.exchange_pieces)
        info = fused_op.plan.info
    else:
        kw = plan_config_kw(w)
        pr = B.make_problem(m, n, k, in_dt, step_out_dt, row_scale=use_scales, col_scale=use_scales)
        plan = B.DotPlan(pr, B.make_config(**kw) if kw else None)
        info = plan.info
    stream = torch.cuda.current_stream(dev)

    def gemm(i):
        a_d, b_d, c_d = sets[i % n_sets]
        plan.run(a_d, b_d, c_d, rs_d, cs_d, stream)
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

    rows = m // world if part == "k" else m
    if kshard:
        scat = torch.empty((rows, n), dtype=torch.float32, device=dev)
        final = torch.empty((rows, n), dtype=out_dt, device=dev)

        def step(i):
            part_c = gemm(i)
            dist.reduce_scatter_tensor(scat, part_c, op=dist.ReduceOp.SUM)
            final.copy_(scat)  # cast epilogue after the reduction
            return final
    elif fused:
        def step(i):
            a_d, b_d, _ = sets[i % n_sets]
            return fused_op(a_d, b_d)
    else:
        step = gemm

    def check_plan():
        (fused_op.plan if fused else plan).check(stream)

    # ---- the timed region: W warm-up steps, then exactly K steps ------------------------------------------
    sampler = sample_clocks(ctx.local_rank)
    for i in range(warmup):
        step(i)
    ctx.barrier()
    launches0 = B.kernel_launches()
    ms = timed_window(ctx, step, steps, stream)
    launches = int(ctx.sum_over_ranks(B.kernel_launches() - launches0))
    check_plan()
    ms_per_step = ms / steps
    # The same window again until half a second has been timed: a single window of a short kernel holds too few
    # clock samples to say anything about the clocks.
    windows = [ms_per_step]
    spent = ms
    while spent < 500.0 and len(windows) < 200 and not args.kernel_only:
        t = timed_window(ctx, step, steps, stream)
        windows.append(t / steps)
        spent += t
    clocks = sampler.stop()
    sw = sorted(windows)
    job_flops = shp["job_flops"]
    value = job_flops / (ms_per_step * 1e-3) / 1e12

    # ---- sustained regime: at least two seconds of back-to-back steps -------------------------------------
    sust = None
    if not args.no_sustained:
        iters = int(max(steps, math.ceil(2000.0 / max(sw[len(sw) // 2], 1e-3))))
        sampler2 = sample_clocks(ctx.local_rank)
        half = iters // 2
        timed_window(ctx, step, half, stream)                       # first second: lets the power limiter settle
        sust_ms = timed_window(ctx, step, iters - half, stream, first=half) / (iters - half)
        sust = {"seconds": (ms_per_step * iters) / 1e3, "steps": iters, "ms_per_step": sust_ms, "clocks": sampler2.stop()}
        check_plan()

    # ---- result check (outside every timed region) -----------------------------------------------------------
    if args.kernel_only:
        check = {"ok": True, "skipped": "--kernel-only"}
    else:
        check = check_result(ctx, name, w, shp, part, sets[0], step, rs_d, cs_d, info, slot_dt if fused else None, rows)

    # ---- the library GEMM of the same per-GPU problem, same run (context, not part of any timed step) ------
    lib_ms = library_gemm_ms(ctx, args, w, sets, rs_d, cs_d, n_sets, out_dt, steps) if not (w.get("jit") or args.kernel_only) else None

    peaks = measured_peaks()
    per_gpu_flops = info["flops"]
    algo_bytes = info["algorithmic_bytes"]
    launch_s = ms_per_step * 1e-3  # one GEMM launch of this library per step
    # the captures are of the unsharded problem: a shard's launch has no figure
    whole = (m, n, k) == (w["m"], w["n"], w["k"])
    traffic, traffic_src = NCU_TRAFFIC.get(name, (None, None)) if whole else (None, None)
    if name == "cfg3":
        achieved = algo_bytes / launch_s / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": traffic, "traffic_source": traffic_src,
                "peak_source": f"hbm_gbs of {peaks['_source']}"}
        if sust:
            sa = algo_bytes / (sust["ms_per_step"] * 1e-3) / 1e9
            sust.update(achieved=sa, peak=peaks["hbm_gbs"], frac=sa / peaks["hbm_gbs"], unit="GB/s")
    else:
        achieved = per_gpu_flops / launch_s / 1e12
        peak, peak_src = peaks["bf16_tflops"], f"bf16_tflops (burst) of {peaks['_source']}"
        speak, speak_src = peaks.get("bf16_tflops_sustained", peak), f"bf16_tflops_sustained of {peaks['_source']}"
        if w["dtype"] == "fp8":
            f8 = None if args.kernel_only else fp8_peak(ctx)
            if f8:
                peak, peak_src = f8["burst_tflops"], "torch._scaled_mm e4m3 8192^3 (tensor-wide scales) measured in this run: best of 10 single launches and a 20-launch window after an idle second"
                speak, speak_src = f8["sustained_tflops"], "torch._scaled_mm e4m3 8192^3 measured in this run, 2 s back to back"
            else:
                peak, peak_src = 2 * peak, peak_src + " x2 for fp8 (torch._scaled_mm unavailable)"
                speak, speak_src = 2 * speak, speak_src + " x2 for fp8"
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": traffic, "traffic_source": traffic_src, "peak_source": peak_src}
        if part == "k":
            roof["note"] = "the step includes the exchange of the partial sums; achieved is per-GPU GEMM FLOPs over the whole step"
        if sust:
            sa = per_gpu_flops / (sust["ms_per_step"] * 1e-3) / 1e12
            sust.update(achieved=sa, peak=speak, frac=sa / speak, unit="TFLOP/s", peak_source=speak_src)

    rec = {
        "workload": name, "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
        "value": value, "unit": "TFLOP/s", "scaling": shp["scaling"], "dtype": w["dtype"],
        "windows": {"n": len(sw), "median_ms_per_step": sw[len(sw) // 2], "min_ms_per_step": sw[0], "max_ms_per_step": sw[-1]},
        "roofline": roof, "sustained": sust, "check": check, "clocks": clocks, "gpu_launches": launches,
        "config": config_dict(name, w, world),
    }
    if lib_ms:
        rec.update(lib_ms)
    if name == "cfg3":
        rec["gbps"] = roof["achieved"]
    if fused and not args.kernel_only:
        rec["exchange"] = exchange_phases(ctx, fused_op, sets, n_sets, slot_dt, m, n)

    # ---- end to end through the host-buffer entry point (H2D + kernel + D2H every step) -------------------
    if headline and not args.kernel_only:
        a_p, b_p = a_h.pin_memory(), b_h.pin_memory()
        c_p = torch.empty((rows, n), dtype=out_dt).pin_memory()
        e2e_steps = max(1, min(steps, 10))
        if part == "k" or w.get("jit"):
            def e2e_step(i):
                a_d, b_d, _ = sets[0]
                a_d.copy_(a_p, non_blocking=True)
                b_d.copy_(b_p, non_blocking=True)
                c_p.copy_(step(0), non_blocking=True)
                torch.cuda.synchronize(dev)
            h2d, d2h = (m * k + k * n) * es, rows * n * 2
        else:
            def e2e_step(i):
                plan.run_host(a_p, b_p, c_p, rs_h if use_scales else None, cs_h if use_scales else None)
            h2d = (m * k + k * n) * es + (4 * (m + n) if use_scales else 0)
            d2h = m * n * 2
        e2e_step(0)
        ctx.barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            e2e_step(i)
        ctx.barrier()
        e2e_s = ctx.max_over_ranks((time.perf_counter() - t0) / e2e_steps)
        rec["e2e"] = {"value": job_flops / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d),
                      "d2h_bytes_per_step": int(d2h), "steps": e2e_steps}
        del a_p, b_p, c_p
    if plan is not None:
        plan.close()
    del sets
    torch.cuda.empty_cache()
    return rec


def check_result(ctx: Ctx, name, w, shp, part, bufs, step, rs_d, cs_d, info, slot_dt, rows_owned) -> dict:
    """This rank's output of one more step against an fp32 matmul of the same operands, upcast: sampled rows over every
    column, and (where the operands are local) sampled columns over every row, edges of the tile raster included."""
    torch, dist = ctx.torch, ctx.dist
    world, rank = ctx.world, ctx.rank
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        a_d, b_d, _ = bufs
        got_full = step(0)
        torch.cuda.synchronize(ctx.dev)
        m, n, k = shp["m"], shp["n"], shp["k"]
        tile_rows = info["block_m"]
        parts = []
        tol = "rtol 1e-2, atol 1e-2 against fp32" if w["dtype"] != "fp8" else "rtol 3e-2, atol 3e-2 against fp32"
        rtol = atol = 3e-2 if w["dtype"] == "fp8" else 1e-2
        if part == "k":
            # rows this rank owns after the exchange; every rank contributes its K columns of those rows and its K rows of B
            r0 = rank * rows_owned
            rows = ctx.torch.tensor(rows_to_check(rows_owned, tile_rows, 48, 17), device=ctx.dev)
            refs, mags = [], []
            for owner in range(world):
                idx = rows + owner * rows_owned
                refs.append(a_d[idx].float() @ b_d.float())              # this rank's partial of owner's sampled rows
            stacked = torch.stack(refs)
            out_sum = torch.empty_like(refs[0])
            dist.reduce_scatter_tensor(out_sum, stacked, op=dist.ReduceOp.SUM)   # fp32 sum of the partials: the reference
            extra = None
            if slot_dt == torch.bfloat16:
                mag = torch.empty_like(refs[0])
                dist.reduce_scatter_tensor(mag, stacked.abs(), op=dist.ReduceOp.SUM)
                extra = mag * 2.0 ** -8      # every partial is rounded to bf16 once before the sum
                tol += " + 2^-8 of the sum of |partials| (bf16 slots)"
            parts.append(check_against_fp32(got_full[rows], out_sum, extra, rtol, atol))
        else:
            rows = torch.tensor(rows_to_check(m, tile_rows, 64, 17), device=ctx.dev)
            ref = a_d[rows].float() @ b_d.float()
            if rs_d is not None:
                ref = ref * rs_d[rows, None] * cs_d[None, :]
            parts.append(check_against_fp32(got_full[rows], ref, None, rtol, atol))
            cols = torch.tensor(rows_to_check(n, info["block_n"], 32, 19), device=ctx.dev)
            ref = a_d.float() @ b_d[:, cols].float()
            if rs_d is not None:
                ref = ref * rs_d[:, None] * cs_d[None, cols]
            parts.append(check_against_fp32(got_full[:, cols], ref, None, rtol, atol))
        res = merge_checks(parts, tol)
        # every rank checks its own shard; the record holds the worst
        res["bad"] = int(ctx.sum_over_ranks(res["bad"]))
        res["max_err"] = ctx.max_over_ranks(res["max_err"])
        res["ok"] = res["bad"] == 0 and math.isfinite(res["max_err"])
        res["ranks_checked"] = world
        return res
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def library_gemm_ms(ctx: Ctx, args, w, sets, rs_d, cs_d, n_sets, out_dt, steps: int):
    """torch.matmul (cuBLAS) on this rank's problem in both regimes this bench reports for its own kernel: `steps`
    launches after an idle second and the same warm-up (the burst window), and a loop of about two seconds (sustained).
    fp8: torch._scaled_mm with the same row and column scales. Never part of a timed step of this library."""
    torch = ctx.torch
    try:
        if w["dtype"] == "fp8":
            bt = [s[1].t().contiguous().t() for s in sets]   # _scaled_mm wants a column-major B
            sa, sb = rs_d.reshape(-1, 1).contiguous(), cs_d.reshape(1, -1).contiguous()

            def lib(i):
                torch._scaled_mm(sets[i % n_sets][0], bt[i % n_sets], scale_a=sa, scale_b=sb, out_dtype=out_dt)
            key = "scaled_mm"
        else:
            def lib(i):
                torch.matmul(sets[i % n_sets][0], sets[i % n_sets][1])
            key = "cublas"
        stream = torch.cuda.current_stream(ctx.dev)
        lib(0)
        ctx.barrier()
        time.sleep(1.0)   # the bench's own first window also starts from an idle GPU
        for i in range(args.warmup):
            lib(i)
        ms = timed_window(ctx, lib, steps, stream) / steps
        out = {key + "_ms": ms}
        if not args.no_sustained:
            iters = int(max(steps, math.ceil(2000.0 / max(ms, 1e-3))))
            half = iters // 2
            timed_window(ctx, lib, half, stream)
            out[key + "_sustained_ms"] = timed_window(ctx, lib, iters - half, stream, first=half) / (iters - half)
        return out
    except Exception as e:  # a library that refuses the shape is not this bench's failure
        return {"cublas_ms": None, "cublas_error": str(e)[:200]}


_FP8_PEAK = {}


def fp8_peak(ctx: Ctx):
    """Dense e4m3 throughput of the library GEMM on this GPU: torch._scaled_mm 8192^3 with tensor-wide unit scales.
    Burst: the better of 10 single launches and of a 20-launch window after an idle second and five warm-up launches
    (the regime of this bench's own first window: on a box that has just run the sustained loops, single launches
    with a synchronise after each were measured 15 % below that window). Sustained: two seconds back to back."""
    if "v" in _FP8_PEAK:
        return _FP8_PEAK["v"]
    torch = ctx.torch
    try:
        nn = 8192
        a = torch.randn(nn, nn, device=ctx.dev).to(torch.float8_e4m3fn)
        b = torch.randn(nn, nn, device=ctx.dev).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=ctx.dev)
        fl = 2.0 * nn ** 3

        def run():
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        for _ in range(3):
            run()
        torch.cuda.synchronize(ctx.dev)
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run()
            e1.record()
            torch.cuda.synchronize(ctx.dev)
            best = min(best, e0.elapsed_time(e1))
        time.sleep(1.0)
        for _ in range(5):
            run()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            run()
        e1.record()
        torch.cuda.synchronize(ctx.dev)
        best = min(best, e0.elapsed_time(e1) / 20)
        iters = int(math.ceil(2000.0 / best))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(iters // 2):
            run()
        e0.record()
        for _ in range(iters - iters // 2):
            run()
        e1.record()
        torch.cuda.synchronize(ctx.dev)
        sust = e0.elapsed_time(e1) / (iters - iters // 2)
        _FP8_PEAK["v"] = {"burst_tflops": fl / best / 1e9, "sustained_tflops": fl / sust / 1e9}
    except Exception:
        _FP8_PEAK["v"] = None
    return _FP8_PEAK["v"]


def exchange_phases(ctx: Ctx, fused_op, sets, n_sets, slot_dt, m, n) -> dict:
    """Where a fused K-sharded step spends its time: CUDA events between its four phases (median over 10 steps, max
    over ranks), the bytes every rank sends, and what a plain peer copy of that many bytes achieves in this run."""
    torch = ctx.torch
    world = ctx.world
    stream = torch.cuda.current_stream(ctx.dev)
    per_phase = [[] for _ in range(4)]
    for i in range(10):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        a_d, b_d, _ = sets[i % n_sets]
        ctx.barrier()
        fused_op(a_d, b_d, events=ev)
        torch.cuda.synchronize(ctx.dev)
        for j in range(4):
            per_phase[j].append(ev[j].elapsed_time(ev[j + 1]))
    med = [ctx.max_over_ranks(sorted(p)[len(p) // 2]) for p in per_phase]
    es = 2 if slot_dt == torch.bfloat16 else 4
    sent = (world - 1) * (m // world) * n * es
    # plain copy engine figure: this rank's slot 0 into the next rank's slot buffer, all ranks at once (a ring)
    peer = fused_op.handle.get_buffer((ctx.rank + 1) % world, fused_op.slots.shape, fused_op.slots.dtype)
    src = torch.empty_like(fused_op.slots)
    for _ in range(2):
        peer.copy_(src)
    ctx.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(3):
        peer.copy_(src)
    e1.record(stream)
    ctx.barrier()
    copy_ms = ctx.max_over_ranks(e0.elapsed_time(e1) / 3)
    copy_gbs = src.numel() * es / copy_ms / 1e6
    gemm_ms = med[1]
    return {"pieces": fused_op.parts,
            "note": ("phases timed with the exchange in one piece, one after the other"
                     + ("; the timed steps run it in `pieces` pieces with each piece's slot reduction on a second stream "
                        "under the next piece's GEMM" if fused_op.parts > 1 else "")),
            "phase_ms": {"barrier_before": med[0], "gemm_with_remote_stores": med[1], "barrier_after": med[2], "slot_reduction": med[3]},
            "bytes_sent_per_rank": int(sent), "nvlink_gbs_during_gemm": sent / gemm_ms / 1e6,
            "peer_copy_gbs_same_run": copy_gbs, "frac_of_peer_copy": (sent / gemm_ms / 1e6) / copy_gbs}


def headline_line(args, rec: dict, w: dict) -> dict:
    line = {
        "metric": "tt.dot TFLOP/s", "value": rec["value"], "unit": "TFLOP/s", "n_gpus": rec["n_gpus"], "steps": rec["steps"],
        "warmup": rec["warmup"], "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": rec["scaling"],
        "vs_baseline": None, "dtype": w["dtype"],
        "data": "synthetic (seeded CPU draw, shapes and distributions of BASELINE.json)",
        "config": rec["config"], "roofline": rec["roofline"], "e2e": rec.get("e2e"), "gpu_launches": rec["gpu_launches"],
        "clocks": rec["clocks"], "windows": rec["windows"], "sustained": rec["sustained"], "check": rec["check"],
    }
    for key in ("cublas_ms", "cublas_sustained_ms", "scaled_mm_ms", "scaled_mm_sustained_ms", "cublas_error", "gbps", "exchange"):
        if key in rec:
            line[key] = rec[key]
    return line


def compact(rec: dict) -> dict:
    out = {"workload": rec["workload"], "ms_per_step": rec["ms_per_step"], "value": rec["value"], "unit": rec["unit"],
           "achieved": rec["roofline"]["achieved"], "achieved_unit": rec["roofline"]["unit"], "peak": rec["roofline"]["peak"],
           "frac": rec["roofline"]["frac"], "peak_source": rec["roofline"]["peak_source"], "steps": rec["steps"],
           "windows": rec["windows"], "sustained": rec["sustained"], "check": rec["check"], "clocks": rec["clocks"],
           "kernel": rec["config"]["kernel"], "per_gpu": rec["config"]["per_gpu"], "parallelism": rec["config"]["parallelism"]}
    for key in ("cublas_ms", "cublas_sustained_ms", "scaled_mm_ms", "scaled_mm_sustained_ms", "exchange"):
        if key in rec:
            out[key] = rec[key]
    return out


# ---- fused attention forward (the two chained tt.dot of the reference's demo kernel) ------------------------------
ATTN_SM_SCALE = 1.3   # the reference benchmark's value (06-fused-attention.py:785)


def attn_flops(w: dict, z: int) -> float:
    f = 4.0 * z * w["h"] * w["n_ctx"] * w["n_ctx"] * w["d"]
    f = 0.5 * f if w["causal"] else f
    return 2.5 * f if w.get("bwd") else f


def attn_host_inputs(w: dict, rank: int):
    import torch
    g = torch.Generator().manual_seed(w["seed"] + 1000 * rank)
    q, k, v = (torch.randn((w["z"], w["h"], w["n_ctx"], w["d"]), generator=g).to(torch.float16) for _ in range(3))
    if w["dtype"] == "fp8e5m2":   # as the reference's benchmark casts them; V keeps n_ctx contiguous
        q, k = q.to(torch.float8_e5m2), k.to(torch.float8_e5m2)
        v = v.permute(0, 1, 3, 2).contiguous().permute(0, 1, 3, 2).to(torch.float8_e5m2)
    return [q, k, v]


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


def attn_config(name: str, w: dict, world: int, set_bytes: int) -> dict:
    bwd = bool(w.get("bwd"))
    return {"workload": name, "z": w["z"] * world, "h": w["h"], "n_ctx": w["n_ctx"], "head_dim": w["d"],
            "causal": w["causal"], "per_gpu": [w["z"], w["h"], w["n_ctx"], w["d"]],
            "parallelism": "batch-sharded, no collective" if world > 1 else "single GPU",
            "kernel": ("one fused kernel per KV block of 128 rows (five tt.dot per block pair, all accumulators in TMEM) "
                       "+ delta pre-pass + dq cast" if bwd else
                       "256 query rows per CTA (2 x 128), KV blocks of 128, tcgen05 + TMEM"),
            "l2": f"one buffer set of {set_bytes / 1e6:.0f} MB > 126 MB L2"}


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
    world = max(1, args.gpus)
    set_bytes = 4 * w["z"] * w["h"] * w["n_ctx"] * w["d"] * 2
    return {"impl": "reference", "metric": "attention bwd TFLOP/s" if w.get("bwd") else "attention fwd TFLOP/s", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic (seeded randn, the reference benchmark's shapes and sm_scale)",
            "config": attn_config(name, w, world, set_bytes),
            "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def run_attention_gpu_arm(ctx: Ctx, args, name: str, w: dict) -> dict | None:
    """Every rank runs its own batch of `z` sequences (independent (batch, head) pairs: no collective)."""
    torch = ctx.torch
    from triton_ext_b200 import attention as A

    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    q_h, k_h, v_h = (t.pin_memory() for t in attn_host_inputs(w, rank))
    o_h = torch.empty_like(q_h).pin_memory()
    q, k, v = q_h.to(dev), k_h.to(dev), v_h.to(dev)
    out = torch.empty_like(q)
    es = q.element_size()
    set_bytes = 4 * q.numel() * es
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

    stream = torch.cuda.current_stream(dev)
    sampler = sample_clocks(ctx.local_rank)
    for i in range(args.warmup):
        step(i)
    ctx.barrier()
    launches0 = A.kernel_launches()
    ms = timed_window(ctx, step, args.steps, stream)
    launches = int(ctx.sum_over_ranks(A.kernel_launches() - launches0))
    ms_per_step = ms / args.steps
    windows, spent = [ms_per_step], ms
    while spent < 500.0 and len(windows) < 200 and not args.kernel_only:
        t = timed_window(ctx, step, args.steps, stream)
        windows.append(t / args.steps)
        spent += t
    clocks = sampler.stop()
    A.check(dev)
    sw = sorted(windows)
    per_gpu_flops = attn_flops(w, w["z"])
    value = per_gpu_flops * world / (ms_per_step * 1e-3) / 1e12

    # torch's fused attention (a library kernel) on the same tensors, same warm-up and window: context, never part of
    # a timed step of this library
    sdpa_ms = None
    if not args.kernel_only and w["dtype"] != "fp8e5m2":
        try:
            import torch.nn.functional as F
            if bwd:
                qg, kg, vg = (t.detach().clone().requires_grad_() for t in (q, k, v))
                o_lib = F.scaled_dot_product_attention(qg, kg, vg, is_causal=w["causal"], scale=ATTN_SM_SCALE)

                def lib(i):
                    torch.autograd.grad(o_lib, (qg, kg, vg), d_o, retain_graph=True)
            else:
                def lib(i):
                    F.scaled_dot_product_attention(q, k, v, is_causal=w["causal"], scale=ATTN_SM_SCALE)
            for i in range(args.warmup):
                lib(i)
            sdpa_ms = timed_window(ctx, lib, args.steps, stream) / args.steps
        except Exception:
            sdpa_ms = None

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
        h2d_bytes, d2h_bytes = 3 * q.numel() * es, q.numel() * es
    if args.kernel_only:
        e2e_steps = 0
    else:
        e2e_step()
    ctx.barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step()
    ctx.barrier()
    e2e_s = ctx.max_over_ranks((time.perf_counter() - t0) / max(e2e_steps, 1))
    if args.kernel_only:
        e2e_s = float("inf")

    peaks = measured_peaks()
    achieved = per_gpu_flops / (ms_per_step * 1e-3) / 1e12
    sm_mhz = clocks.get("sm_mhz") or 1965
    sfu_bound = 4.0 * w["d"] * 16 * 148 * sm_mhz * 1e6 / 1e12   # one exp2 per score, 16 per clock per SM
    algo_bytes = 4 * q.numel() * es + q.numel() // w["d"] * 4
    traffic, traffic_src = NCU_TRAFFIC.get(name, (None, None))
    line = {
        "metric": "attention bwd TFLOP/s" if bwd else "attention fwd TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": w["dtype"], "data": "synthetic (seeded randn, the reference benchmark's shapes and sm_scale)",
        "config": attn_config(name, w, world, set_bytes),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["bf16_tflops"], "traffic": traffic, "traffic_source": traffic_src,
                     "peak_source": f"bf16_tflops (burst) of {peaks['_source']}",
                     "note": f"exp2 on the SFU (16 per clock per SM) bounds this shape at {sfu_bound:.0f} TFLOP/s; "
                             f"algorithmic bytes {algo_bytes / 1e6:.0f} MB"},
        "e2e": {"value": per_gpu_flops * world / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d_bytes),
                "d2h_bytes_per_step": int(d2h_bytes), "steps": e2e_steps},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "windows": {"n": len(sw), "median_ms_per_step": sw[len(sw) // 2], "min_ms_per_step": sw[0], "max_ms_per_step": sw[-1]},
        "sdpa_ms": sdpa_ms,
    }
    return line if rank == 0 else None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="time the named workload only")
    ap.add_argument("--exchange-pieces", type=int, default=None,
                    help="pieces of the fused K-shard exchange (default: chosen by the library from the problem size)")
    ap.add_argument("--no-sustained", action="store_true", help="skip the two-second back-to-back window")
    ap.add_argument("--kernel-only", action="store_true",
                    help="for profilers: warm-up and the one timed window of the named workload, nothing else "
                         "(no further windows, sustained loop, result check, library GEMM, end-to-end or CPU leg)")
    ap.add_argument("--cpu-baseline-only", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    default_run = args.workload is None and not args.kernel_only
    if args.kernel_only:
        args.no_also = args.no_sustained = args.no_cpu_baseline = True
    name = args.workload or DEFAULT_WORKLOAD
    w = WORKLOADS[name]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.cpu_baseline_only:
        print(json.dumps(cpu_baseline_single_core(name, w)), flush=True)
        return

    if args.impl == "reference":
        if rank != 0:
            return  # the CPU arm runs once, on rank 0
        arm = run_attention_reference_arm if w.get("attn") else run_reference_arm
        print(json.dumps(arm(args, name, w)), flush=True)
        return

    ctx = Ctx()
    if w.get("attn"):
        line = run_attention_gpu_arm(ctx, args, name, w)
        ctx.close()
        if line is None:
            return
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = attn_cpu_sample(w)
        print(json.dumps(line), flush=True)
        return

    rec = run_dot_workload(ctx, args, name, w, headline=True)
    line = headline_line(args, rec, w)
    failed = [name] if not rec["check"]["ok"] else []
    if default_run and not args.no_also:
        also = []
        for other in (ALSO_ONE_GPU if world == 1 else ALSO_MULTI_GPU):
            try:
                r = run_dot_workload(ctx, args, other, WORKLOADS[other], headline=False)
                also.append(compact(r))
                if not r["check"]["ok"]:
                    failed.append(other)
            except Exception as e:  # one workload's failure must not lose the others' records
                also.append({"workload": other, "error": f"{type(e).__name__}: {str(e)[:300]}"})
                failed.append(other)
        line["also"] = also
    ctx.close()
    if rank != 0:
        return
    if world == 1 and not args.no_cpu_baseline:
        if w.get("jit"):
            # The interpreter oracle needs TRITON_INTERPRET=1 from before Triton is imported; this process has
            # imported Triton's compiler for the timed arm, so the CPU leg runs in a process of its own.
            import subprocess
            out = subprocess.run([sys.executable, os.path.abspath(__file__), "--workload", name, "--cpu-baseline-only"],
                                 capture_output=True, text=True, check=True)
            cb = json.loads(out.stdout.strip().splitlines()[-1])
        else:
            cb = cpu_baseline_single_core(name, w)
        line["cpu_baseline"] = cb
    print(json.dumps(line), flush=True)
    if failed:
        sys.stderr.write(f"result check failed or workload raised: {failed}\n")
        sys.exit(1)


if __name__ == "__main__":
    main()
