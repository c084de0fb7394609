// The tt.dot K-loop as one persistent, warp-specialised sm_100a kernel.
//
//   warp 0 (one lane)  : TMA producer — fills a ring of shared-memory stages, one K block per stage
//   warp 1 (one lane)  : tcgen05.mma issuer — accumulates in TMEM (fp32), two accumulators so the
//                        epilogue of segment i overlaps the main loop of segment i+1
//   warps 2..5         : epilogue — tcgen05.ld TMEM -> registers, fused scale + cast, global store
//
// The K loop is executed the way the LoopSplit pass leaves it (reference:
// pass/LoopSplit/LoopSplit.cpp:179-193): an unpredicated main loop over [0, k_main_blocks) and a
// remainder loop over [k_main_blocks, k_blocks) in which the operand tiles are zero-filled past K
// and only the tcgen05.mma instructions that cover real data are issued.
//
// Operand roles: "P" is the MMA A operand (128 rows per tile, TMEM lanes), "Q" the MMA B operand
// (block_n rows per tile, TMEM columns). The host maps tt.dot's A/B onto P/Q (swapped for skinny m).
//
// Every wait on an mbarrier is bounded in time. A wait that runs out raises an abort flag in shared
// memory and a status word in global memory; all roles then leave their loops, outstanding TMA
// copies are drained, TMEM is released and the CTA returns normally.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace txd {

constexpr int kBlockM = 128;          // MMA M = TMEM lanes
constexpr int kStageRowBytes = 128;   // one K block = 128 bytes of K per row (one SWIZZLE_128B atom)
constexpr int kMmasPerBlock = 4;      // 128 B / 32 B per tcgen05.mma
constexpr int kMaxStages = 12;
constexpr int kNumThreads = 192;
constexpr int kEpilogueThreads = 128;

enum DeviceStatus : uint32_t {
  kDevOk = 0,
  kDevTimeoutProducer = 1,  // producer waited on an "empty" stage barrier
  kDevTimeoutMmaFull = 2,   // MMA issuer waited on a "full" stage barrier
  kDevTimeoutMmaTmem = 3,   // MMA issuer waited for an accumulator to be drained
  kDevTimeoutEpilogue = 4,  // epilogue waited for an accumulator to be complete
  kDevTimeoutDrain = 5      // teardown waited for copies / MMAs in flight
};

struct alignas(64) DotParams {
  CUtensorMap tmap_p;
  CUtensorMap tmap_q;
  void *out;
  const float *scale_row;  // indexed by the P (lane) index, or null
  const float *scale_col;  // indexed by the Q (column) index, or null
  float *partials;         // stream-K scratch: [2*grid][block_n][128] fp32
  uint32_t *tile_counters; // stream-K scratch: [tiles], zero between launches
  uint32_t *status;        // device status word (0 = ok)
  long long ldo;           // leading dimension of out, elements
  unsigned long long wait_limit_ns;
  float alpha;
  int32_t p_extent, q_extent, k_extent;  // rows of P, rows of Q, K (elements)
  int32_t trans_out;       // 0: out[p*ldo+q]   1: out[q*ldo+p]
  int32_t out_dtype;       // 0 f16, 1 bf16, 3 f32
  int32_t block_n;
  int32_t bk_elems;        // K elements per stage: 64 (16-bit) or 128 (8-bit)
  int32_t stages;
  int32_t k_blocks;        // ceil(K / bk_elems)
  int32_t k_main_blocks;   // LoopSplit mid point / bk_elems
  int32_t tail_mmas;       // MMAs issued by the last remainder block (1..4)
  int32_t tiles_p, tiles_q;
  int32_t group_p;         // raster group height in tiles
  int32_t stream_k;        // 0 = whole tiles round-robin, 1 = equal (tile,k-block) shares
  int32_t kind_f8;         // 0: kind::f16, 1: kind::f8f6f4
  uint32_t idesc;          // tcgen05 instruction descriptor
  // shared-memory matrix descriptors: upper 32 bits, and start-address step (16-byte units) per MMA
  uint32_t p_desc_hi, q_desc_hi;
  uint32_t p_desc_lbo, q_desc_lbo;   // already shifted: (bytes >> 4) << 16
  uint32_t p_kstep, q_kstep;
  int32_t p_mn_major, q_mn_major;    // 1 = rows contiguous in memory (MN-major), 0 = K contiguous
  int32_t chunk_elems;               // 128 B / element size: MN-major box width
  int32_t p_stage_bytes, q_stage_bytes;
  int32_t tmem_cols;
};

// ----------------------------------------------------------------------------------------------
// PTX wrappers
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled TMA load global -> shared, completion counted on an mbarrier (no multicast).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *m, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread t of the warp receives lane (base+t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void epilogue_bar_sync() {
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

// ----------------------------------------------------------------------------------------------
// Bounded waits
// ----------------------------------------------------------------------------------------------
struct AbortCtl {
  volatile uint32_t *flag;  // shared memory
  uint32_t *status;         // global memory
  unsigned long long limit_ns;
};

__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, const AbortCtl &ac,
                                            uint32_t code) {
  const unsigned long long t0 = global_timer_ns();
  uint32_t it = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 63u) == 0) {
      if (*ac.flag) return false;
      if (global_timer_ns() - t0 > ac.limit_ns) {
        *ac.flag = 1;
        atomicCAS(ac.status, 0u, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const AbortCtl &ac,
                                          uint32_t code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, ac, code);
}

// ----------------------------------------------------------------------------------------------
// Work iteration: every role walks the same sequence of segments (tile, [kb0, kb1)).
// ----------------------------------------------------------------------------------------------
struct Segment {
  int tile;
  int kb0, kb1;
};

struct WorkIter {
  // data-parallel
  int next_tile, tile_stride, tiles;
  // stream-K
  long long unit, unit_end;
  int k_blocks;
  bool stream_k;

  __device__ __forceinline__ WorkIter(const DotParams &p) {
    tiles = p.tiles_p * p.tiles_q;
    k_blocks = p.k_blocks;
    stream_k = p.stream_k != 0;
    next_tile = blockIdx.x;
    tile_stride = gridDim.x;
    const long long total = static_cast<long long>(tiles) * k_blocks;
    unit = total * blockIdx.x / gridDim.x;
    unit_end = total * (blockIdx.x + 1) / gridDim.x;
  }
  __device__ __forceinline__ bool next(Segment &s) {
    if (!stream_k) {
      if (next_tile >= tiles) return false;
      s.tile = next_tile;
      s.kb0 = 0;
      s.kb1 = k_blocks;
      next_tile += tile_stride;
      return true;
    }
    if (unit >= unit_end) return false;
    s.tile = static_cast<int>(unit / k_blocks);
    s.kb0 = static_cast<int>(unit - static_cast<long long>(s.tile) * k_blocks);
    const long long tile_end = static_cast<long long>(s.tile + 1) * k_blocks;
    const long long e = tile_end < unit_end ? tile_end : unit_end;
    s.kb1 = s.kb0 + static_cast<int>(e - unit);
    unit = e;
    return true;
  }
};

// First CTA whose stream-K share contains `unit`.
__device__ __forceinline__ int stream_k_owner(long long unit, long long total, int grid) {
  // share c = [total*c/grid, total*(c+1)/grid)
  int c = static_cast<int>((unit * grid) / total);
  while (c + 1 < grid && total * (c + 1) / grid <= unit) ++c;
  while (c > 0 && total * c / grid > unit) --c;
  return c;
}

__device__ __forceinline__ void tile_coords(const DotParams &p, int tile, int &tp, int &tq) {
  const int per_group = p.group_p * p.tiles_q;
  const int g = tile / per_group;
  const int first = g * p.group_p;
  const int gsize = min(p.tiles_p - first, p.group_p);
  const int r = tile - g * per_group;
  tp = first + r % gsize;
  tq = r / gsize;
}

// ----------------------------------------------------------------------------------------------
// Epilogue store of one 32-column (or 16-column) chunk held by one thread
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack2(float a, float b, int out_dtype) {
  if (out_dtype == 1) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}

template <int kCols>
__device__ __forceinline__ void store_chunk(const DotParams &p, float (&f)[32], int prow, int qcol0) {
  // prow: global P index of this thread's accumulator row; qcol0: global Q index of f[0]
  const bool row_ok = prow < p.p_extent;
  const float rs = (p.scale_row && row_ok) ? __ldg(p.scale_row + prow) * p.alpha : p.alpha;
#pragma unroll
  for (int j = 0; j < kCols; ++j) {
    float cs = 1.0f;
    if (p.scale_col && (qcol0 + j) < p.q_extent) cs = __ldg(p.scale_col + qcol0 + j);
    f[j] = f[j] * rs * cs;
  }
  if (!row_ok) return;
  if (p.trans_out) {
    // out[q*ldo + p]: lanes of a warp hold consecutive p -> coalesced per column
    if (p.out_dtype == 3) {
      float *o = reinterpret_cast<float *>(p.out);
#pragma unroll
      for (int j = 0; j < kCols; ++j)
        if (qcol0 + j < p.q_extent) o[static_cast<long long>(qcol0 + j) * p.ldo + prow] = f[j];
    } else if (p.out_dtype == 1) {
      __nv_bfloat16 *o = reinterpret_cast<__nv_bfloat16 *>(p.out);
#pragma unroll
      for (int j = 0; j < kCols; ++j)
        if (qcol0 + j < p.q_extent)
          o[static_cast<long long>(qcol0 + j) * p.ldo + prow] = __float2bfloat16_rn(f[j]);
    } else {
      __half *o = reinterpret_cast<__half *>(p.out);
#pragma unroll
      for (int j = 0; j < kCols; ++j)
        if (qcol0 + j < p.q_extent)
          o[static_cast<long long>(qcol0 + j) * p.ldo + prow] = __float2half_rn(f[j]);
    }
    return;
  }
  const long long base = static_cast<long long>(prow) * p.ldo + qcol0;
  const bool full = (qcol0 + kCols) <= p.q_extent;
  if (p.out_dtype == 3) {
    float *o = reinterpret_cast<float *>(p.out) + base;
    if (full && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < kCols; j += 4)
        *reinterpret_cast<float4 *>(o + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < kCols; ++j)
        if (qcol0 + j < p.q_extent) o[j] = f[j];
    }
    return;
  }
  uint16_t *o = reinterpret_cast<uint16_t *>(p.out) + base;
  if (full && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
    for (int j = 0; j < kCols; j += 8) {
      uint4 w;
      w.x = pack2(f[j], f[j + 1], p.out_dtype);
      w.y = pack2(f[j + 2], f[j + 3], p.out_dtype);
      w.z = pack2(f[j + 4], f[j + 5], p.out_dtype);
      w.w = pack2(f[j + 6], f[j + 7], p.out_dtype);
      *reinterpret_cast<uint4 *>(o + j) = w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < kCols; ++j) {
      if (qcol0 + j < p.q_extent) {
        const uint32_t w = pack2(f[j], 0.0f, p.out_dtype);
        o[j] = static_cast<uint16_t>(w & 0xFFFFu);
      }
    }
  }
}

// ----------------------------------------------------------------------------------------------
// The kernel
// ----------------------------------------------------------------------------------------------
struct SharedCtl {
  unsigned long long full_bar[kMaxStages];
  unsigned long long empty_bar[kMaxStages];
  unsigned long long tmem_full_bar[2];
  unsigned long long tmem_empty_bar[2];
  unsigned long long drain_bar;
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t fixup_last;
  uint32_t epi_ok;
};

template <int kChunk>  // TMEM columns per tcgen05.ld: 32, or 16 when block_n == 16
__device__ __forceinline__ void epilogue_role(const DotParams &p, SharedCtl *ctl,
                                              const AbortCtl &ac, int warp, int lane) {
  const int quarter = warp & 3;                 // TMEM lane quarter this warp may read
  const int row_in_tile = quarter * 32 + lane;  // accumulator row held by this thread
  const int epi_tid = (warp - 2) * 32 + lane;
  const uint32_t tmem_base = ctl->tmem_base;
  const long long total_units = static_cast<long long>(p.tiles_p) * p.tiles_q * p.k_blocks;
  WorkIter it(p);
  Segment s;
  uint32_t seg_i = 0;
  int cta_first_tile = -1;
  while (it.next(s)) {
    const uint32_t acc = seg_i & 1u;
    const uint32_t acc_phase = (seg_i >> 1) & 1u;
    if (cta_first_tile < 0) cta_first_tile = s.tile;
    // One thread watches the barrier and publishes the outcome, so that all 128 epilogue threads
    // take the same branch (they meet again at named barrier 1 below).
    if (epi_tid == 0)
      ctl->epi_ok = mbar_wait(smem_u32(&ctl->tmem_full_bar[acc]), acc_phase, ac, kDevTimeoutEpilogue) ? 1u : 0u;
    epilogue_bar_sync();
    const bool seg_ok = ctl->epi_ok != 0;
    epilogue_bar_sync();
    if (!seg_ok) return;
    tc_fence_after();
    int tp, tq;
    tile_coords(p, s.tile, tp, tq);
    const int prow = tp * kBlockM + row_in_tile;
    const uint32_t taddr =
        tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * static_cast<uint32_t>(p.block_n);
    const bool whole = (s.kb1 - s.kb0) == p.k_blocks;
    if (whole) {
      for (int c0 = 0; c0 < p.block_n; c0 += kChunk) {
        uint32_t v[32];
        if (kChunk == 32) tmem_ld_32x32(taddr + c0, v); else tmem_ld_32x16(taddr + c0, v);
        tmem_ld_wait();
        float f[32];
#pragma unroll
        for (int j = 0; j < kChunk; ++j) f[j] = __uint_as_float(v[j]);
        store_chunk<kChunk>(p, f, prow, tq * p.block_n + c0);
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&ctl->tmem_empty_bar[acc]));
    } else {
      // Partial tile: park the fp32 partial in scratch, column-major inside the tile so that the
      // 32 lanes of a warp write 128 consecutive bytes.
      const int slot = blockIdx.x * 2 + (s.tile == cta_first_tile ? 0 : 1);
      float *mine = p.partials + static_cast<long long>(slot) * p.block_n * kBlockM;
      for (int c0 = 0; c0 < p.block_n; c0 += kChunk) {
        uint32_t v[32];
        if (kChunk == 32) tmem_ld_32x32(taddr + c0, v); else tmem_ld_32x16(taddr + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < kChunk; ++j)
          __stcg(mine + static_cast<long long>(c0 + j) * kBlockM + row_in_tile, __uint_as_float(v[j]));
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&ctl->tmem_empty_bar[acc]));
      // Contributors of this tile are the CTAs whose shares intersect its k-block range.
      const long long u0 = static_cast<long long>(s.tile) * p.k_blocks;
      const int c_first = stream_k_owner(u0, total_units, gridDim.x);
      const int c_last = stream_k_owner(u0 + p.k_blocks - 1, total_units, gridDim.x);
      __threadfence();
      epilogue_bar_sync();
      if (epi_tid == 0) {
        const uint32_t old = atomicAdd(p.tile_counters + s.tile, 1u);
        const uint32_t last = (old == static_cast<uint32_t>(c_last - c_first)) ? 1u : 0u;
        if (last) p.tile_counters[s.tile] = 0;  // ready for the next launch
        ctl->fixup_last = last;
      }
      epilogue_bar_sync();
      const bool last = ctl->fixup_last != 0;
      epilogue_bar_sync();  // fixup_last may be rewritten by the next partial segment
      if (last) {
        __threadfence();
        for (int c0 = 0; c0 < p.block_n; c0 += kChunk) {
          float f[32];
#pragma unroll
          for (int j = 0; j < kChunk; ++j) f[j] = 0.0f;
          // Sum in ascending k order: deterministic regardless of arrival order.
          for (int c = c_first; c <= c_last; ++c) {
            const long long cb = total_units * c / gridDim.x;
            const int c_first_tile = static_cast<int>(cb / p.k_blocks);
            const int cslot = c * 2 + (s.tile == c_first_tile ? 0 : 1);
            const float *src = p.partials + static_cast<long long>(cslot) * p.block_n * kBlockM;
#pragma unroll
            for (int j = 0; j < kChunk; ++j)
              f[j] += __ldcg(src + static_cast<long long>(c0 + j) * kBlockM + row_in_tile);
          }
          store_chunk<kChunk>(p, f, prow, tq * p.block_n + c0);
        }
      }
    }
    ++seg_i;
  }
}

__global__ void __launch_bounds__(kNumThreads, 1) dot_umma_kernel(const __grid_constant__ DotParams p) {
  extern __shared__ uint8_t smem_raw[];
  // Stage buffers need 1024-byte alignment (SWIZZLE_128B atoms); the launch asks for 1 KiB of slack.
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t *smem = smem_raw + pad;
  const uint32_t stage_bytes = static_cast<uint32_t>(p.p_stage_bytes + p.q_stage_bytes);
  SharedCtl *ctl = reinterpret_cast<SharedCtl *>(smem + static_cast<size_t>(p.stages) * stage_bytes);
  const uint32_t stage_base = smem_u32(smem);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  AbortCtl ac;
  ac.flag = &ctl->abort_flag;
  ac.status = p.status;
  ac.limit_ns = p.wait_limit_ns;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&ctl->full_bar[s]), 1);
      mbar_init(smem_u32(&ctl->empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&ctl->tmem_empty_bar[a]), kEpilogueThreads);
    }
    mbar_init(smem_u32(&ctl->drain_bar), 1);
    ctl->abort_flag = 0;
    ctl->fixup_last = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.tmap_p);
    tma_prefetch_desc(&p.tmap_q);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      WorkIter it(p);
      Segment s;
      uint32_t stage = 0, phase = 0;
      uint32_t issued = 0;
      bool ok = true;
      while (ok && it.next(s)) {
        int tp, tq;
        tile_coords(p, s.tile, tp, tq);
        const int p0 = tp * kBlockM;
        const int q0 = tq * p.block_n;
        for (int kb = s.kb0; kb < s.kb1; ++kb) {
          if (!mbar_wait(smem_u32(&ctl->empty_bar[stage]), phase ^ 1u, ac, kDevTimeoutProducer)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&ctl->full_bar[stage]);
          mbar_arrive_expect_tx(full, stage_bytes);
          const uint32_t p_dst = stage_base + stage * stage_bytes;
          const uint32_t q_dst = p_dst + static_cast<uint32_t>(p.p_stage_bytes);
          const int k0 = kb * p.bk_elems;
          if (!p.p_mn_major) {
            tma_load_2d(p_dst, &p.tmap_p, k0, p0, full);
          } else {
            const uint32_t box_bytes = static_cast<uint32_t>(p.bk_elems) * kStageRowBytes;
            for (int c = 0; c * p.chunk_elems < kBlockM; ++c)
              tma_load_2d(p_dst + c * box_bytes, &p.tmap_p, p0 + c * p.chunk_elems, k0, full);
          }
          if (!p.q_mn_major) {
            tma_load_2d(q_dst, &p.tmap_q, k0, q0, full);
          } else {
            const uint32_t box_bytes = static_cast<uint32_t>(p.bk_elems) * kStageRowBytes;
            for (int c = 0; c * p.chunk_elems < p.block_n; ++c)
              tma_load_2d(q_dst + c * box_bytes, &p.tmap_q, q0 + c * p.chunk_elems, k0, full);
          }
          ++issued;
          if (++stage == static_cast<uint32_t>(p.stages)) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *ac.flag) {
        // Abort path: wait (bounded) until every copy this thread started has landed, so that no
        // TMA write is in flight when the CTA's shared memory is released.
        const uint32_t n = issued < static_cast<uint32_t>(p.stages) ? issued : static_cast<uint32_t>(p.stages);
        uint32_t st = stage, ph = phase;
        for (uint32_t i = 0; i < n; ++i) {
          if (st == 0) {
            st = static_cast<uint32_t>(p.stages);
            ph ^= 1u;
          }
          --st;
          const unsigned long long t0 = global_timer_ns();
          while (!mbar_try_wait(smem_u32(&ctl->full_bar[st]), ph)) {
            if (global_timer_ns() - t0 > ac.limit_ns) {
              atomicCAS(ac.status, 0u, static_cast<uint32_t>(kDevTimeoutDrain));
              break;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      WorkIter it(p);
      Segment s;
      uint32_t stage = 0, phase = 0, seg_i = 0;
      bool ok = true;
      while (ok && it.next(s)) {
        const uint32_t acc = seg_i & 1u;
        const uint32_t acc_phase = (seg_i >> 1) & 1u;
        if (!mbar_wait(smem_u32(&ctl->tmem_empty_bar[acc]), acc_phase ^ 1u, ac, kDevTimeoutMmaTmem)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * static_cast<uint32_t>(p.block_n);
        uint32_t accumulate = 0;
        // One K block: wait for its stage, issue `n_mma` MMAs, hand the stage back.
        auto k_block = [&](int n_mma) -> bool {
          if (!mbar_wait(smem_u32(&ctl->full_bar[stage]), phase, ac, kDevTimeoutMmaFull)) return false;
          tc_fence_after();
          const uint32_t p_addr = stage_base + stage * stage_bytes;
          const uint32_t q_addr = p_addr + static_cast<uint32_t>(p.p_stage_bytes);
          const uint64_t pdesc = (static_cast<uint64_t>(p.p_desc_hi) << 32) |
                                 static_cast<uint64_t>(p.p_desc_lbo | ((p_addr & 0x3FFFFu) >> 4));
          const uint64_t qdesc = (static_cast<uint64_t>(p.q_desc_hi) << 32) |
                                 static_cast<uint64_t>(p.q_desc_lbo | ((q_addr & 0x3FFFFu) >> 4));
          if (p.kind_f8) {
#pragma unroll 1
            for (int j = 0; j < n_mma; ++j) {
              umma_f8(d_tmem, pdesc + static_cast<uint64_t>(j * p.p_kstep),
                      qdesc + static_cast<uint64_t>(j * p.q_kstep), p.idesc, accumulate);
              accumulate = 1;
            }
          } else {
#pragma unroll 1
            for (int j = 0; j < n_mma; ++j) {
              umma_f16(d_tmem, pdesc + static_cast<uint64_t>(j * p.p_kstep),
                       qdesc + static_cast<uint64_t>(j * p.q_kstep), p.idesc, accumulate);
              accumulate = 1;
            }
          }
          tc_commit(smem_u32(&ctl->empty_bar[stage]));  // frees the stage when these MMAs retire
          if (++stage == static_cast<uint32_t>(p.stages)) {
            stage = 0;
            phase ^= 1u;
          }
          return true;
        };
        // LoopSplit main loop [lo, mid): every block is full, no predication of any kind.
        const int mid = s.kb1 < p.k_main_blocks ? s.kb1 : p.k_main_blocks;
        int kb = s.kb0;
        for (; ok && kb < mid; ++kb) ok = k_block(kMmasPerBlock);
        // LoopSplit remainder loop [mid, hi): TMA zero-filled the stage past K; the last block
        // issues only the MMAs that cover real columns.
        for (; ok && kb < s.kb1; ++kb)
          ok = k_block(kb == p.k_blocks - 1 ? p.tail_mmas : kMmasPerBlock);
        if (ok) tc_commit(smem_u32(&ctl->tmem_full_bar[acc]));
        ++seg_i;
      }
      if (!ok || *ac.flag) {
        // Abort path: make sure no MMA is still reading shared memory / writing TMEM.
        tc_commit(smem_u32(&ctl->drain_bar));
        const unsigned long long t0 = global_timer_ns();
        while (!mbar_try_wait(smem_u32(&ctl->drain_bar), 0)) {
          if (global_timer_ns() - t0 > ac.limit_ns) {
            atomicCAS(ac.status, 0u, static_cast<uint32_t>(kDevTimeoutDrain));
            break;
          }
        }
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    if (p.block_n >= 32)
      epilogue_role<32>(p, ctl, ac, warp, lane);
    else
      epilogue_role<16>(p, ctl, ac, warp, lane);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}

}  // namespace txd
