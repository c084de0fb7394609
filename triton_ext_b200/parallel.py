"""Multi-GPU partitioning of one tt.dot GEMM: one process per GPU, `torch.distributed` for plumbing.

Two partitions, as the path's two natural cuts:

  N-sharded (column-parallel)  rank r owns B[:, n0:n1] and produces C[:, n0:n1]; A is replicated.
                               Independent output panels: no data-path collective at all.
  K-sharded                    rank r owns A[:, k0:k1] and B[k0:k1, :], produces a full-size fp32
                               partial of C, and one NCCL reduce-scatter (sum) over NVLink leaves
                               rank r with rows [m0:m1) of C, which it casts to the output type.

The reference has no multi-GPU code; these follow the partitioning its tt.dot tiles allow
(independent output tiles; K blocks summed into one accumulator,
pass/LoopSplit/06-fused-attention.py:85).

`local_dot` is the per-rank GEMM. It defaults to the CUDA kernels (triton_ext_b200.backend.dot);
the CPU tests of the partition logic pass the oracle instead. Nothing here falls back by itself.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def split_range(extent: int, parts: int, index: int, align: int = 1) -> tuple[int, int]:
    """[lo, hi) of part `index` when `extent` is cut into `parts` pieces whose boundaries are multiples
    of `align` (the last piece takes the remainder). Pieces differ by at most one aligned unit."""
    if parts <= 0 or not (0 <= index < parts):
        raise ValueError("bad partition index")
    units = (extent + align - 1) // align
    base, extra = divmod(units, parts)
    lo_u = index * base + min(index, extra)
    hi_u = lo_u + base + (1 if index < extra else 0)
    return min(lo_u * align, extent), min(hi_u * align, extent)


def _default_local_dot():
    from . import backend
    return backend.dot


def n_sharded_dot(a: torch.Tensor, b_shard: torch.Tensor, *, out_dtype: torch.dtype,
                  row_scale: Optional[torch.Tensor] = None, col_scale_shard: Optional[torch.Tensor] = None,
                  alpha: float = 1.0, local_dot: Optional[Callable] = None, **kw) -> torch.Tensor:
    """This rank's panel C[:, n0:n1] = A @ B[:, n0:n1]. No communication."""
    fn = local_dot or _default_local_dot()
    return fn(a, b_shard, out_dtype=out_dtype, row_scale=row_scale, col_scale=col_scale_shard, alpha=alpha, **kw)


def k_sharded_dot(a_shard: torch.Tensor, b_shard: torch.Tensor, *, out_dtype: torch.dtype,
                  row_scale: Optional[torch.Tensor] = None, col_scale: Optional[torch.Tensor] = None,
                  alpha: float = 1.0, group=None, local_dot: Optional[Callable] = None,
                  partial_dtype: torch.dtype = torch.float32, chunks: int = 1,
                  partial: Optional[torch.Tensor] = None, **kw) -> torch.Tensor:
    """Rows [m0:m1) of C = sum over ranks of A[:, k_r] @ B[k_r, :], with the scale/cast epilogue applied
    after the reduction.

    The local GEMM writes an unscaled partial in `partial_dtype` (fp32 keeps the accumulator's
    precision across ranks; bf16 halves the NVLink bytes at a documented cost in accuracy). The partial
    is reduce-scattered along M: rank r receives the sum of rows split_range(M, world, r).
    With chunks > 1 the M range of every rank is cut into `chunks` panels and the reduce-scatter of
    panel i is issued while the GEMM of panel i+1 runs (two streams on a GPU).
    M must be divisible by world * chunks.
    """
    fn = local_dot or _default_local_dot()
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    m, n = a_shard.shape[0], b_shard.shape[1]
    if m % (world * chunks) != 0:
        raise ValueError(f"M={m} must be divisible by world*chunks={world * chunks}")
    rows = m // world
    out_part = torch.empty((rows, n), dtype=partial_dtype, device=a_shard.device)
    if chunks == 1:
        if partial is None:
            partial = torch.empty((m, n), dtype=partial_dtype, device=a_shard.device)
        fn(a_shard, b_shard, out=partial, out_dtype=partial_dtype, **kw)
        dist.reduce_scatter_tensor(out_part, partial, op=dist.ReduceOp.SUM, group=group)
    else:
        # Panel p holds, for every destination rank d, rows [d*rows + p*pr, d*rows + (p+1)*pr).
        pr = rows // chunks
        on_gpu = a_shard.is_cuda
        comm_stream = torch.cuda.Stream(device=a_shard.device) if on_gpu else None
        works = []
        for pidx in range(chunks):
            idx = torch.cat([torch.arange(d * rows + pidx * pr, d * rows + (pidx + 1) * pr, device=a_shard.device)
                             for d in range(world)])
            a_panel = a_shard.index_select(0, idx)
            panel = fn(a_panel, b_shard, out_dtype=partial_dtype, **kw)
            dst = out_part[pidx * pr:(pidx + 1) * pr]
            if on_gpu:
                ev = torch.cuda.Event()
                ev.record()
                with torch.cuda.stream(comm_stream):
                    comm_stream.wait_event(ev)
                    dist.reduce_scatter_tensor(dst, panel, op=dist.ReduceOp.SUM, group=group)
                panel.record_stream(comm_stream)
            else:
                dist.reduce_scatter_tensor(dst, panel, op=dist.ReduceOp.SUM, group=group)
        if on_gpu:
            torch.cuda.current_stream(a_shard.device).wait_stream(comm_stream)
    # Epilogue after the reduction: alpha, row scale (this rank's rows), column scale, cast.
    m0, _ = rank * rows, (rank + 1) * rows
    acc = out_part.float()
    if alpha != 1.0:
        acc = acc * alpha
    if row_scale is not None:
        acc = acc * row_scale[m0:m0 + rows, None]
    if col_scale is not None:
        acc = acc * col_scale[None, :]
    return acc.to(out_dtype)


class FusedKShardedDot:
    """K-sharded GEMM whose epilogue performs the exchange: every rank's kernel stores its partial tiles
    straight into the owning rank's memory over NVLink (peer-mapped symmetric memory, ordinary TMA tensor
    stores, no multicast); after a stream-ordered barrier each rank sums the `world` slots of its own rows
    with one pass over local HBM and applies the scale / cast epilogue. Compared with "GEMM, then NCCL
    reduce-scatter" the NVLink transfer overlaps the GEMM tile by tile and the result is summed in a fixed
    order (deterministic). `partial_dtype` bf16 halves the NVLink bytes at the cost of rounding each partial.

    One instance per (m, n, k_shard, dtype) and process group; buffers are allocated once.
    """

    def __init__(self, m: int, n: int, k_shard: int, ab_dtype: torch.dtype, out_dtype: torch.dtype, *,
                 partial_dtype: torch.dtype = torch.float32, group=None, device=None, config_kw: Optional[dict] = None,
                 parts: Optional[int] = None):
        import torch.distributed._symmetric_memory as symm_mem
        from . import backend as B
        self.B = B
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if m % self.world:
            raise ValueError(f"M={m} must be divisible by the world size {self.world}")
        self.m, self.n, self.rows = m, n, m // self.world
        self.out_dtype = out_dtype
        dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        kw = dict(schedule=B.TXD_SCHED_DATA_PARALLEL, swap_ab=2)
        kw.update(config_kw or {})
        self.plan = B.DotPlan(B.make_problem(m, n, k_shard, ab_dtype, partial_dtype), B.make_config(**kw))
        block_m = self.plan.info["block_m"]
        if self.rows % block_m:
            raise ValueError(f"M / world = {self.rows} must be a multiple of the tile height {block_m}")
        # Pieces of the exchange: with parts > 1 the sum of piece j runs on a second stream while piece j + 1's GEMM is
        # storing. Measured on B200s (bf16 16384 x 28672 x 8192): no gain at 2 ranks (3.27 against 3.24 ms; the GEMM is
        # power-bound there and the sum draws on the same power limit) and none worth having at 4 (fp32 slots 2.61
        # against 2.66 ms, bf16 slots 1.73 against 1.67 ms: every piece is a launch of its own with a partial last wave
        # and a barrier) or 8 (2.79 against 2.80 ms, 1.51 against 1.49 ms), so the default is one piece.
        tile_rows = self.rows // block_m
        if parts is None:
            parts = 1
        if parts < 1 or tile_rows % parts:
            raise ValueError(f"the {tile_rows} tile rows of a rank do not divide into {parts} parts")
        self.parts = parts
        # [world, rows, n] slots in symmetric memory: slot s of this buffer is written by rank s
        self.slots = symm_mem.empty((self.world, self.rows, n), dtype=partial_dtype, device=dev)
        self.handle = symm_mem.rendezvous(self.slots, self.group)
        self.slot_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.out = torch.empty((self.rows, n), dtype=out_dtype, device=dev)
        self.side = torch.cuda.Stream(device=dev) if parts > 1 else None
        self._piece_done = [torch.cuda.Event() for _ in range(parts)] if parts > 1 else []
        self._side_done = torch.cuda.Event() if parts > 1 else None

    def __call__(self, a_shard: torch.Tensor, b_shard: torch.Tensor, *, row_scale: Optional[torch.Tensor] = None,
                 col_scale: Optional[torch.Tensor] = None, alpha: float = 1.0, events: Optional[list] = None) -> torch.Tensor:
        """One K-sharded GEMM + exchange. `events`, if given, is a list of five CUDA events recorded on the current
        stream before the first phase and after each of the four phases (for per-phase timing); the call then runs
        the exchange in one piece, phase after phase, whatever `parts` is."""
        rs = row_scale[self.rank * self.rows:(self.rank + 1) * self.rows] if row_scale is not None else None
        if events is None and self.parts > 1:
            return self._call_in_pieces(a_shard, b_shard, rs, col_scale, alpha)

        def mark(i):
            if events is not None:
                events[i].record()
        mark(0)
        # 1. nobody may still be reading the slots of the previous call
        self.handle.barrier(channel=0)
        mark(1)
        # 2. GEMM with the exchange in its epilogue
        self.plan.run_to_slots(a_shard, b_shard, self.slot_ptrs, self.rank)
        mark(2)
        # 3. every rank's stores have landed
        self.handle.barrier(channel=1)
        mark(3)
        # 4. local sum of the slots + scale + cast
        self.B.reduce_slots(self.slots, self.out, row_scale=rs, col_scale=col_scale, alpha=alpha)
        mark(4)
        return self.out

    def _call_in_pieces(self, a_shard, b_shard, rs, col_scale, alpha) -> torch.Tensor:
        main = torch.cuda.current_stream(self.out.device)
        rows = self.rows // self.parts
        self.handle.barrier(channel=0)          # nobody may still be reading the slots of the previous call
        for j in range(self.parts):
            self.plan.run_to_slots(a_shard, b_shard, self.slot_ptrs, self.rank, part=j, parts=self.parts)
            self._piece_done[j].record(main)
            with torch.cuda.stream(self.side):
                self.side.wait_event(self._piece_done[j])
                self.handle.barrier(channel=1)  # every rank's stores of piece j have landed
                self.B.reduce_slots(self.slots, self.out, row_scale=rs, col_scale=col_scale, alpha=alpha,
                                    row0=j * rows, rows=rows)
        self._side_done.record(self.side)
        main.wait_event(self._side_done)
        return self.out
