// The tt.dot K-loop as one persistent, warp-specialised sm_100a kernel.
//
//   warp 0 (one lane)  : TMA producer of the P operand — fills a ring of shared-memory stages, one K block
//                        per stage, and arms the stage's "full" barrier with the byte count of both operands
//   warp 2 (one lane)  : TMA producer of the Q operand (issuing a TMA copy occupies the issuing thread for
//                        over a hundred nanoseconds; two issuing warps halve the time to fill a stage)
//   warp 1 (one lane)  : tcgen05.mma issuer — accumulates in TMEM (fp32), two accumulators so the
//                        epilogue of segment i overlaps the main loop of segment i+1
//   warps 3..6         : epilogue — tcgen05.ld TMEM -> registers, fused scale + cast, global store; a warp may read
//                        the 32 TMEM lanes of its quarter (warp index mod 4)
//
// The K loop is executed the way the LoopSplit pass leaves it (reference:
// pass/LoopSplit/LoopSplit.cpp:179-193): an unpredicated main loop over [0, k_main_blocks) and a
// remainder loop over [k_main_blocks, k_blocks) in which the operand tiles are zero-filled past K
// and only the tcgen05.mma instructions that cover real data are issued.
//
// Operand roles: "P" is the MMA A operand (128 rows per CTA, TMEM lanes), "Q" the MMA B operand
// (block_n rows per tile, TMEM columns). The host maps tt.dot's A/B onto P/Q (swapped for skinny m).
//
// Two instantiations of one template:
//   single : one CTA per 128 x block_n tile (tcgen05 cta_group::1); also runs the stream-K schedule.
//   pair   : a cluster of two CTAs per 256 x block_n tile (cta_group::2). Each CTA loads its own 128
//            rows of P and its own half of Q; the leader CTA issues MMAs that read both CTAs' shared
//            memory and write both CTAs' TMEM. A CTA then ingests 2/3 of the bytes per FLOP of the
//            single variant, which is what the SM's shared-memory fill rate asks for.
//            No TMA load here uses multicast.
//   wide pair : the pair variant with a 256 x 512 tile: every K block feeds two 256-column MMA halves
//            from one P stage, so a CTA ingests 48 KiB per 1024 tensor cycles instead of 32 KiB per 512.
//            Both TMEM accumulators belong to the tile, so a half's epilogue overlaps only the
//            other half's MMAs of the neighbouring K blocks, not a whole main loop.
//
// Epilogue stores go through a swizzled shared-memory slab and a TMA tensor store (full 128-byte
// lines) when C allows it, else straight from registers.
//
// Every wait on an mbarrier is bounded in time. A wait that runs out raises an abort flag in shared
// memory and a status word in global memory; all roles then leave their loops, outstanding TMA
// copies are drained, TMEM is released and the CTA returns normally.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

// Measurement switches (bits 1, 2, 4, 8 of DotParams::debug_flags) make results wrong by design; they
// exist only in builds made with -DTXD_MEASURE. The shipped library compiles them out.
#ifdef TXD_MEASURE
#define TXD_DBG(p, bit) (((p).debug_flags & (bit)) != 0)
#else
#define TXD_DBG(p, bit) false
#endif

namespace txd {

constexpr int kBlockM = 128;          // MMA M = TMEM lanes
constexpr int kStageRowBytes = 128;   // one K atom = 128 bytes of K per row (one SWIZZLE_128B span);
                                      // a stage (K block) holds 1 or 2 atoms
constexpr int kMmasPerAtom = 4;       // 128 B / 32 B per tcgen05.mma
constexpr int kMaxStages = 12;
// One epilogue warp per TMEM lane quarter. Eight (two per quarter, columns split) were measured: the epilogue got
// shorter, but the MMA warp shares its scheduler with the quarter-1 epilogue warps and its issue loop slowed from 525
// to 562 cycles per K block, a net loss on every shape.
constexpr int kEpilogueWarps = 4;
constexpr int kNumThreads = 96 + kEpilogueWarps * 32;
constexpr int kEpilogueThreads = kEpilogueWarps * 32;
constexpr int kStoreSlabBytes = 32 * 128;  // one epilogue warp's staging slab: 32 rows x 128 bytes
constexpr int kStoreStagingBytes = kEpilogueWarps * 2 * kStoreSlabBytes;  // double-buffered

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
  CUtensorMap tmap_out;    // valid when tma_store != 0
  CUtensorMap tmap_remote[8];  // valid when remote_world > 0: rank r's partial-tile slots (peer memory)
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
  int32_t bk_elems;        // K elements per stage (K block): atoms * chunk_elems
  int32_t stages;
  int32_t k_blocks;        // ceil(K / bk_elems)
  int32_t k_main_blocks;   // LoopSplit mid point / bk_elems
  int32_t tail_mmas;       // MMAs issued by the last remainder block (1 .. 4 * atoms)
  int32_t tiles_p, tiles_q;
  int32_t group_p;         // raster group height in tiles
  int32_t stream_k;        // 0 = whole tiles round-robin only; 1 = tiles from sk_first_tile on are cut into
                           // equal (tile, k-block) shares, one per worker (0: all tiles = pure stream-K)
  int32_t sk_first_tile;   // first tile of the stream-K region; tiles below it run whole, round-robin
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
  int32_t tma_store;                 // 1 = epilogue stores through shared memory + TMA
  int32_t atoms;                     // 128-byte K atoms per stage: 1, 2 or 4 (0 reads as 1)
  int32_t wide;                      // pair kernel only: 1 = a tile is 256 x (2 * block_n): two MMA column halves
                                     // share each P stage and each fill one of the two TMEM accumulators
  // K-sharded GEMM fused with its exchange: instead of C, a tile is stored into the slot this rank owns
  // inside the memory of the rank that owns the tile's rows (plain TMA stores over NVLink, no multicast):
  // slot buffer of rank o = [remote_world][rows_per_rank][n], this rank writes slot `remote_rank`.
  int32_t remote_world;              // 0 = store to `out` as usual
  int32_t remote_rank;
  int32_t rows_per_rank;             // m / remote_world, a multiple of the tile height
  int32_t tp_interleave;             // > 1: consecutive tile rows of the raster belong to consecutive owners (this many
                                     // ranks), starting with the rank after this one
  int32_t tp_begin, tiles_p_all;     // with tp_interleave: this launch covers tile rows [tp_begin, tp_begin + tiles_p)
                                     // of the interleaved order, out of tiles_p_all (a part of the exchange)
  int32_t debug_flags;               // 128 = producer stops after its first K block (host-side fault
                                     // injection: exercises the bounded waits). Builds with -DTXD_MEASURE
                                     // also honour 1 = do not refill stages (tensor-pipe-only timing),
                                     // 2 = one MMA per tile (load-only timing), 4 = skip C stores,
                                     // 8 = one tcgen05.commit per CTA of a pair instead of one for both;
                                     // results are wrong with 1, 2 or 4 set
};

// ----------------------------------------------------------------------------------------------
// Work iteration: every role walks the same sequence of segments (tile, [kb0, kb1)).
// A "worker" is a CTA (single) or a CTA pair (pair).
// ----------------------------------------------------------------------------------------------
struct Segment {
  int tile;
  int kb0, kb1;
};

struct WorkIter {
  int next_tile, tile_stride, dp_end;  // whole tiles, round-robin, below dp_end
  long long unit, unit_end;            // this worker's share of the stream-K region's (tile, k-block) units
  int k_blocks, sk_tile0;

  __device__ __forceinline__ WorkIter(const DotParams &p, int worker, int workers) {
    const int tiles = p.tiles_p * p.tiles_q;
    k_blocks = p.k_blocks;
    sk_tile0 = p.stream_k ? p.sk_first_tile : tiles;
    dp_end = sk_tile0;
    next_tile = worker;
    tile_stride = workers;
    const long long total = static_cast<long long>(tiles - sk_tile0) * k_blocks;
    unit = total * worker / workers;
    unit_end = total * (worker + 1) / workers;
  }
  __device__ __forceinline__ bool next(Segment &s) {
    if (next_tile < dp_end) {
      s.tile = next_tile;
      s.kb0 = 0;
      s.kb1 = k_blocks;
      next_tile += tile_stride;
      return true;
    }
    if (unit >= unit_end) return false;
    const int t = static_cast<int>(unit / k_blocks);
    s.tile = sk_tile0 + t;
    s.kb0 = static_cast<int>(unit - static_cast<long long>(t) * k_blocks);
    const long long tile_end = static_cast<long long>(t + 1) * k_blocks;
    const long long e = tile_end < unit_end ? tile_end : unit_end;
    s.kb1 = s.kb0 + static_cast<int>(e - unit);
    unit = e;
    return true;
  }
};

// The worker whose stream-K share [total*c/n, total*(c+1)/n) contains `unit`.
__device__ __forceinline__ int stream_k_owner(long long unit, long long total, int workers) {
  int c = static_cast<int>((unit * workers) / total);
  while (c + 1 < workers && total * (c + 1) / workers <= unit) ++c;
  while (c > 0 && total * c / workers > unit) --c;
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
  if (p.tp_interleave > 1) {
    const int w = p.tp_interleave;
    tp += p.tp_begin;
    int owner = tp % w + p.remote_rank + 1;
    if (owner >= w) owner -= w;
    tp = owner * (p.tiles_p_all / w) + tp / w;
  }
}

// ----------------------------------------------------------------------------------------------
// Epilogue helpers
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack2(float a, float b, int out_dtype) {
  if (out_dtype == 1) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}

// acc * alpha * row_scale[p] * col_scale[q] for one thread's chunk of kCols consecutive columns.
template <int kCols>
__device__ __forceinline__ void scale_chunk(const DotParams &p, float (&f)[32], int prow, int qcol0) {
  const bool row_ok = prow < p.p_extent;
  const float rs = (p.scale_row && row_ok) ? __ldg(p.scale_row + prow) * p.alpha : p.alpha;
  if (p.scale_col) {
#pragma unroll
    for (int j = 0; j < kCols; ++j) {
      const float cs = (qcol0 + j) < p.q_extent ? __ldg(p.scale_col + qcol0 + j) : 1.0f;
      f[j] = f[j] * rs * cs;
    }
  } else {
#pragma unroll
    for (int j = 0; j < kCols; ++j) f[j] *= rs;
  }
}

// Store straight from registers (any alignment, either orientation).
template <int kCols>
__device__ __forceinline__ void store_chunk_direct(const DotParams &p, float (&f)[32], int prow, int qcol0) {
  if (prow >= p.p_extent || TXD_DBG(p, 4)) return;
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

// Write 32 consecutive columns of this thread's row into a SWIZZLE_128B staging slab.
// `byte0` is the byte offset of f[0] inside the 128-byte slab row (a multiple of 16).
__device__ __forceinline__ void stage_chunk(uint32_t slab, int row_in_slab, int byte0, const float (&f)[32],
                                            int out_dtype) {
  const uint32_t row_addr = slab + static_cast<uint32_t>(row_in_slab) * 128u;
  const uint32_t sw = static_cast<uint32_t>(row_in_slab & 7);
  if (out_dtype == 3) {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint32_t chunk = (static_cast<uint32_t>(byte0 >> 4) + c) ^ sw;
      st_shared_v4(row_addr + chunk * 16u, __float_as_uint(f[4 * c]), __float_as_uint(f[4 * c + 1]),
                   __float_as_uint(f[4 * c + 2]), __float_as_uint(f[4 * c + 3]));
    }
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t chunk = (static_cast<uint32_t>(byte0 >> 4) + c) ^ sw;
      st_shared_v4(row_addr + chunk * 16u, pack2(f[8 * c], f[8 * c + 1], out_dtype),
                   pack2(f[8 * c + 2], f[8 * c + 3], out_dtype), pack2(f[8 * c + 4], f[8 * c + 5], out_dtype),
                   pack2(f[8 * c + 6], f[8 * c + 7], out_dtype));
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

template <int kChunk, bool kPair>  // kChunk: TMEM columns per tcgen05.ld (32, or 16 when block_n == 16)
__device__ __forceinline__ void epilogue_role(const DotParams &p, SharedCtl *ctl, const AbortCtl &ac,
                                              uint32_t staging, int warp, int lane, int worker, int workers,
                                              uint32_t cta_rank) {
  const int quarter = warp & 3;                 // TMEM lane quarter this warp may read
  constexpr int kGroups = kEpilogueWarps / 4;   // warps per TMEM lane quarter; they take alternate column slabs
  const int group = (warp - 3) >> 2;
  const int row_in_tile = quarter * 32 + lane;  // accumulator row held by this thread
  const int epi_tid = (warp - 3) * 32 + lane;
  const uint32_t tmem_base = ctl->tmem_base;
  const int sk_tile0 = p.stream_k ? p.sk_first_tile : p.tiles_p * p.tiles_q;
  const long long total_units = static_cast<long long>(p.tiles_p * p.tiles_q - sk_tile0) * p.k_blocks;
  const int ranks = kPair ? 2 : 1;  // each CTA of a pair parks and combines its own 128 rows
  const int rows_per_tile = kPair ? 2 * kBlockM : kBlockM;
  const uint32_t my_slabs = staging + static_cast<uint32_t>(warp - 3) * 2u * kStoreSlabBytes;
  uint32_t stores = 0;                               // TMA stores issued by this warp (slab parity)
  const int slab_cols = p.out_dtype == 3 ? 32 : 64;  // 128 bytes of output per slab row
  const bool scaled = p.scale_row != nullptr || p.scale_col != nullptr || p.alpha != 1.0f;
  // A wide tile is drained as two 256-column halves, one per TMEM accumulator: to this role they are
  // two consecutive segments, so accumulator index and barrier phase follow the same arithmetic.
  const int halves = (kPair && p.wide) ? 2 : 1;
  WorkIter it(p, worker, workers);
  Segment s;
  uint32_t seg_i = 0;
  bool alive = true;
  while (alive && it.next(s)) {
   int tp, tq_tile;
   tile_coords(p, s.tile, tp, tq_tile);
   for (int half = 0; half < halves; ++half) {
    const uint32_t acc = seg_i & 1u;
    const uint32_t acc_phase = (seg_i >> 1) & 1u;
    // One thread watches the barrier and publishes the outcome, so that all 128 epilogue threads
    // take the same branch (they meet again at named barrier 1 below).
    // (mbarrier.try_wait parks the thread in hardware between probes: this wait lasts a whole main loop, and a
    // thread spinning through it costs power that the tensor pipe's clock then lacks)
    if (epi_tid == 0)
      ctl->epi_ok = mbar_wait_timed(smem_u32(&ctl->tmem_full_bar[acc]), acc_phase, ac, kDevTimeoutEpilogue) ? 1u : 0u;
    epilogue_bar_sync();
    const bool seg_ok = ctl->epi_ok != 0;
    epilogue_bar_sync();
    if (!seg_ok) {
      alive = false;
      break;
    }
    tc_fence_after();
    const int tq = tq_tile * halves + half;
    const int prow0 = tp * rows_per_tile + static_cast<int>(cta_rank) * kBlockM;  // first row of this CTA
    const int prow = prow0 + row_in_tile;
    const int qcol_tile = tq * p.block_n;
    const uint32_t taddr =
        tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * static_cast<uint32_t>(p.block_n);
    const uint32_t empty_bar = smem_u32(&ctl->tmem_empty_bar[acc]);
    auto release_accumulator = [&]() {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (kPair) mbar_arrive_cluster(map_to_cta(empty_bar, 0));
        else mbar_arrive(empty_bar);
      }
    };
    const bool whole = (s.kb1 - s.kb0) == p.k_blocks;
    if (whole && p.tma_store && kChunk == 32) {
      // TMEM -> registers -> swizzled slab -> TMA store; a warp owns 32 rows and two staging slabs. Both 32-column
      // loads of a slab are in flight before one wait, and the values are scaled before the wait for the store that
      // last read the slab, so that wait overlaps the register work.
      for (int c0 = group * slab_cols; c0 < p.block_n; c0 += kGroups * slab_cols) {
        const uint32_t slab = my_slabs + (stores & 1u) * kStoreSlabBytes;
        uint32_t v[2][32];
        tmem_ld_32x32(taddr + c0, v[0]);
        if (slab_cols == 64) tmem_ld_32x32(taddr + c0 + 32, v[1]);
        tmem_ld_wait();
        float f[2][32];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (h == 1 && slab_cols != 64) break;
#pragma unroll
          for (int j = 0; j < 32; ++j) f[h][j] = __uint_as_float(v[h][j]);
          if (scaled) scale_chunk<32>(p, f[h], prow, qcol_tile + c0 + 32 * h);
        }
        if (lane == 0) bulk_wait_group_read<1>();  // the store that last read this slab has drained
        __syncwarp();
        stage_chunk(slab, lane, 0, f[0], p.out_dtype);
        if (slab_cols == 64) stage_chunk(slab, lane, 64, f[1], p.out_dtype);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0 && !TXD_DBG(p, 4)) {
          if (p.remote_world > 0) {
            const int owner = prow0 / p.rows_per_rank;
            const int y = (p.remote_rank - owner) * p.rows_per_rank + prow0 + quarter * 32;
            tma_store_2d(&p.tmap_remote[owner], slab, qcol_tile + c0, y);
          } else {
            tma_store_2d(&p.tmap_out, slab, qcol_tile + c0, prow0 + quarter * 32);
          }
          bulk_commit_group();
        }
        ++stores;
      }
      release_accumulator();
    } else if (whole) {
      for (int c0 = group * kChunk; c0 < p.block_n; c0 += kGroups * kChunk) {
        uint32_t v[32];
        if (kChunk == 32) tmem_ld_32x32(taddr + c0, v); else tmem_ld_32x16(taddr + c0, v);
        tmem_ld_wait();
        float f[32];
#pragma unroll
        for (int j = 0; j < kChunk; ++j) f[j] = __uint_as_float(v[j]);
        if (scaled) scale_chunk<kChunk>(p, f, prow, qcol_tile + c0);
        store_chunk_direct<kChunk>(p, f, prow, qcol_tile + c0);
      }
      release_accumulator();
    } else {
      // Partial tile (stream-K region): park the fp32 partial in scratch, column-major
      // inside the tile so that the 32 lanes of a warp write 128 consecutive bytes.
      // A share touches at most two partial tiles: the one it starts in (slot 0) and the one it ends in.
      const int my_first_tile = sk_tile0 + static_cast<int>((total_units * worker / workers) / p.k_blocks);
      const int slot = (worker * 2 + (s.tile == my_first_tile ? 0 : 1)) * ranks + static_cast<int>(cta_rank);
      float *mine = p.partials + static_cast<long long>(slot) * p.block_n * kBlockM;
      for (int c0 = group * kChunk; c0 < p.block_n; c0 += kGroups * kChunk) {
        uint32_t v[32];
        if (kChunk == 32) tmem_ld_32x32(taddr + c0, v); else tmem_ld_32x16(taddr + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < kChunk; ++j)
          __stcg(mine + static_cast<long long>(c0 + j) * kBlockM + row_in_tile, __uint_as_float(v[j]));
      }
      release_accumulator();
      // Contributors of this tile are the workers whose shares intersect its k-block range.
      const long long u0 = static_cast<long long>(s.tile - sk_tile0) * p.k_blocks;
      const int c_first = stream_k_owner(u0, total_units, workers);
      const int c_last = stream_k_owner(u0 + p.k_blocks - 1, total_units, workers);
      __threadfence();
      epilogue_bar_sync();
      if (epi_tid == 0) {
        uint32_t *counter = p.tile_counters + s.tile * ranks + static_cast<int>(cta_rank);
        const uint32_t old = atomicAdd(counter, 1u);
        const uint32_t last = (old == static_cast<uint32_t>(c_last - c_first)) ? 1u : 0u;
        if (last) *counter = 0;  // ready for the next launch
        ctl->fixup_last = last;
      }
      epilogue_bar_sync();
      const bool last = ctl->fixup_last != 0;
      epilogue_bar_sync();  // fixup_last may be rewritten by the next partial segment
      if (last) {
        __threadfence();
        for (int c0 = group * kChunk; c0 < p.block_n; c0 += kGroups * kChunk) {
          float f[32];
#pragma unroll
          for (int j = 0; j < kChunk; ++j) f[j] = 0.0f;
          // Sum in ascending k order: deterministic regardless of arrival order.
          for (int c = c_first; c <= c_last; ++c) {
            const long long cb = total_units * c / workers;
            const int c_first_tile = sk_tile0 + static_cast<int>(cb / p.k_blocks);
            const int cslot = (c * 2 + (s.tile == c_first_tile ? 0 : 1)) * ranks + static_cast<int>(cta_rank);
            const float *src = p.partials + static_cast<long long>(cslot) * p.block_n * kBlockM;
#pragma unroll
            for (int j = 0; j < kChunk; ++j)
              f[j] += __ldcg(src + static_cast<long long>(c0 + j) * kBlockM + row_in_tile);
          }
          scale_chunk<kChunk>(p, f, prow, qcol_tile + c0);
          store_chunk_direct<kChunk>(p, f, prow, qcol_tile + c0);
        }
      }
    }
    ++seg_i;
   }
  }
  // Shared memory must stay valid until every TMA store has read it.
  if (lane == 0) bulk_wait_group_all();
}

template <bool kPair, bool kF8>
__device__ __forceinline__ void dot_umma_body(const DotParams &p) {
#ifdef TXD_MEASURE
  // Measurement builds: SM cycles and wall time of CTA 0 from kernel entry to exit, so that cycles per K block and
  // the effective SM clock of a launch can be told apart (and the set-up cost read off).
  unsigned long long stamp_c0 = 0, stamp_n0 = 0;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    stamp_c0 = clock64();
    stamp_n0 = global_timer_ns();
  }
#endif
  extern __shared__ uint8_t smem_raw[];
  // Stage buffers need 1024-byte alignment (SWIZZLE_128B atoms); the launch asks for 1 KiB of slack.
  // The pad is the same in every CTA of the grid, so both CTAs of a pair use the same offsets.
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t *smem = smem_raw + pad;
  const uint32_t stage_bytes = static_cast<uint32_t>(p.p_stage_bytes + p.q_stage_bytes);
  const uint32_t ring_bytes = static_cast<uint32_t>(p.stages) * stage_bytes;
  const uint32_t staging_bytes = p.tma_store ? static_cast<uint32_t>(kStoreStagingBytes) : 0u;
  SharedCtl *ctl = reinterpret_cast<SharedCtl *>(smem + ring_bytes + staging_bytes);
  const uint32_t stage_base = smem_u32(smem);
  const uint32_t staging = stage_base + ring_bytes;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = kPair ? cluster_cta_rank() : 0u;
  const bool leader = cta_rank == 0;
  const int worker = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int workers = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int rows_per_tile = kPair ? 2 * kBlockM : kBlockM;
  const int q_rows_per_cta = kPair ? p.block_n / 2 : p.block_n;  // Q rows this CTA loads per tile
  const int atoms = p.atoms > 1 ? p.atoms : 1;
  const int mmas_per_block = kMmasPerAtom * atoms;
  const int halves = (kPair && p.wide) ? 2 : 1;       // MMA column halves per tile
  const int tile_n = p.block_n * halves;               // Q rows (C columns) per tile
  const uint32_t q_half_bytes = static_cast<uint32_t>(p.q_stage_bytes) / static_cast<uint32_t>(halves);

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
      mbar_init(smem_u32(&ctl->tmem_empty_bar[a]), (kPair ? 2 : 1) * kEpilogueWarps);  // one arrival per epilogue warp
    }
    mbar_init(smem_u32(&ctl->drain_bar), 1);
    ctl->abort_flag = 0;
    ctl->fixup_last = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.tmap_p);
    tma_prefetch_desc(&p.tmap_q);
    if (p.tma_store) tma_prefetch_desc(&p.tmap_out);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  if (kPair) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  // Everything above touched only this CTA's shared and tensor memory and the kernel's parameters. From here on
  // global memory is read and written, so a launch that was allowed to start before its predecessor in the stream
  // had finished (programmatic dependent launch) waits for it here; and the launch behind this one may start its
  // own set-up now. Back-to-back launches of short GEMMs then pay their launch and set-up latency once.
  grid_dep_launch();
  grid_dep_wait();
#ifdef TXD_MEASURE
  if (blockIdx.x == 0 && threadIdx.x == 0) {   // set-up (barriers, TMEM, cluster sync) is over
    reinterpret_cast<unsigned long long *>(p.status)[12] = clock64();
    reinterpret_cast<unsigned long long *>(p.status)[13] = global_timer_ns();
  }
#endif

  // ------------------------------ TMA producer (one warp per operand) ------------------------------
  // The whole warp walks the loop; one elected lane arms the barrier (P side) and issues the copies.
  // `q_halves`: bit h set = this warp loads the Q rows of MMA column half h.
  auto producer_role = [&](const bool load_p, const int q_halves) {
    {
      WorkIter it(p, worker, workers);
      Segment s;
      uint32_t stage = 0, phase = 0;
      uint32_t issued = 0;
      bool ok = true;
      const bool issuer = elect_one();
      bool have_slot = false;
      while (ok && it.next(s)) {
        int tp, tq;
        tile_coords(p, s.tile, tp, tq);
        const int p0 = tp * rows_per_tile + static_cast<int>(cta_rank) * kBlockM;
        const int q0 = tq * tile_n + static_cast<int>(cta_rank) * q_rows_per_cta;
        for (int kb = s.kb0; kb < s.kb1; ++kb) {
          // `have_slot`: the probe issued at the end of the previous block already saw this stage free.
          if (!have_slot && !warp_mbar_wait(smem_u32(&ctl->empty_bar[stage]), phase ^ 1u, ac, kDevTimeoutProducer, lane)) {
            ok = false;
            break;
          }
          if ((p.debug_flags & 128) && issued >= 1) {  // injected stall: nothing arrives any more
            ok = false;
            break;
          }
          const uint32_t full_local = smem_u32(&ctl->full_bar[stage]);
          // Pair: every byte of both CTAs is counted on the leader's barrier.
          const uint32_t full = kPair ? map_to_cta(full_local, 0) : full_local;
          if (TXD_DBG(p, 1) && issued >= static_cast<uint32_t>(p.stages)) {
            if (leader && issuer && load_p) mbar_arrive(full_local);
            ++issued;
            if (++stage == static_cast<uint32_t>(p.stages)) { stage = 0; phase ^= 1u; }
            have_slot = false;
            continue;
          }
          if (issuer) {
          if (leader && load_p) mbar_arrive_expect_tx(full_local, kPair ? 2u * stage_bytes : stage_bytes);
          const uint32_t p_dst = stage_base + stage * stage_bytes;
          const uint32_t q_dst = p_dst + static_cast<uint32_t>(p.p_stage_bytes);
          const int k0 = kb * p.bk_elems;
          // MN-major: one box per 128-byte-wide row chunk, bk_elems K slices tall.
          // K-major: one box per K atom (its rows x 128 bytes), atoms side by side in the stage.
          const uint32_t box_bytes = static_cast<uint32_t>(p.bk_elems) * kStageRowBytes;
          const uint32_t p_atom_bytes = static_cast<uint32_t>(kBlockM) * kStageRowBytes;
          const uint32_t q_atom_bytes = static_cast<uint32_t>(q_rows_per_cta) * kStageRowBytes;
          auto load = [&](uint32_t dst, const CUtensorMap *m, int x, int y) {
            if (kPair) tma_load_2d_pair(dst, m, x, y, full);
            else tma_load_2d(dst, m, x, y, full);
          };
          if (!load_p) {
          } else if (!p.p_mn_major) {
            for (int at = 0; at < atoms; ++at) load(p_dst + at * p_atom_bytes, &p.tmap_p, k0 + at * p.chunk_elems, p0);
          } else {
            for (int c = 0; c * p.chunk_elems < kBlockM; ++c)
              load(p_dst + c * box_bytes, &p.tmap_p, p0 + c * p.chunk_elems, k0);
          }
          for (int h = 0; h < halves; ++h) {
            if (!((q_halves >> h) & 1)) continue;
            const uint32_t qh_dst = q_dst + static_cast<uint32_t>(h) * q_half_bytes;
            const int qh0 = q0 + h * p.block_n;
            if (!p.q_mn_major) {
              for (int at = 0; at < atoms; ++at) load(qh_dst + at * q_atom_bytes, &p.tmap_q, k0 + at * p.chunk_elems, qh0);
            } else {
              for (int c = 0; c * p.chunk_elems < q_rows_per_cta; ++c)
                load(qh_dst + c * box_bytes, &p.tmap_q, qh0 + c * p.chunk_elems, k0);
            }
          }
          }
          __syncwarp();
          ++issued;
          if (++stage == static_cast<uint32_t>(p.stages)) {
            stage = 0;
            phase ^= 1u;
          }
          // Probe the next stage's "empty" barrier now; the answer is used at the top of the next block.
          have_slot = __all_sync(0xffffffffu, mbar_test_wait(smem_u32(&ctl->empty_bar[stage]), phase ^ 1u));
        }
      }
      if ((!ok || *ac.flag) && issuer && load_p) {
        // Abort path: wait (bounded) until every copy this thread started has landed, so that no
        // TMA write is in flight when the CTA's shared memory is released. (Single variant and the
        // pair's leader; the follower's copies are counted on the leader's barriers.)
        const uint32_t n = issued < static_cast<uint32_t>(p.stages) ? issued : static_cast<uint32_t>(p.stages);
        uint32_t st = stage, ph = phase;
        for (uint32_t i = 0; i < n && leader; ++i) {
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
  };
  if (warp == 0) {
    producer_role(true, halves == 2 ? 2 : 0);  // P, and the second Q half of a wide tile
  } else if (warp == 2) {
    producer_role(false, 1);
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only in a pair) ------------------------------
    // The whole warp walks the loop; one elected lane issues tcgen05 instructions.
    //
    // This loop is one thread's instruction stream, and that stream, not the tensor pipe, is what bounds the
    // kernel when it is long: a K block of four 256x256x16 MMAs occupies the pipe for 512 cycles, and every
    // instruction the issuing thread executes per block (several cycles each, nothing to overlap them with in a
    // one-warp dependency chain) comes out of those 512 cycles. Measured on this part: a loop of about 80 instructions
    // per block ran at 780 cycles per block whatever the MMA's N, a loop of about 30 runs at the pipe's 512, and a
    // tcgen05.commit per block costs nothing by itself. So the main loop below is branch-free apart from its trip
    // count, its descriptors are two multiply-adds per block, the operand kind is a template parameter, and
    // everything a block may need besides (a partial last block, the hand-over between the column halves of a wide
    // tile, measurement modes) lives in the generic path, which the unpredicated main loop never enters.
    if (leader) {
      WorkIter it(p, worker, workers);
      Segment s;
      uint32_t stage = 0, phase = 0, seg_i = 0;
      bool ok = true;
      const bool issuer = elect_one();
      auto commit_to = [&](uint32_t local_bar) {
        if (kPair) {
          // The same barrier in both CTAs (the follower's producer / epilogue wait on their own copy),
          // signalled by one commit.
          if (TXD_DBG(p, 8)) {
            tc_commit_pair(map_to_cta(local_bar, 0));
            tc_commit_pair(map_to_cta(local_bar, 1));
          } else {
            tc_commit_pair_mask(local_bar, 3);
          }
        } else {
          tc_commit(local_bar);
        }
      };
      // Descriptor pieces that do not change during the kernel.
      auto desc64 = [](uint32_t hi, uint32_t lo) { return (static_cast<uint64_t>(hi) << 32) | static_cast<uint64_t>(lo); };
      const uint32_t p_lo_base = p.p_desc_lbo | ((stage_base & 0x3FFFFu) >> 4);
      const uint32_t q_lo_base = p.q_desc_lbo | (((stage_base + static_cast<uint32_t>(p.p_stage_bytes)) & 0x3FFFFu) >> 4);
      const uint32_t stage16 = stage_bytes >> 4;
      const uint32_t q_half16 = q_half_bytes >> 4;  // second MMA column half of a wide tile inside the Q stage
      const uint32_t full0 = smem_u32(&ctl->full_bar[0]), empty0 = smem_u32(&ctl->empty_bar[0]);
      const uint32_t n_stages = static_cast<uint32_t>(p.stages);
      const uint32_t idesc = p.idesc;
      const uint32_t p_hi = p.p_desc_hi, q_hi = p.q_desc_hi, p_kstep = p.p_kstep, q_kstep = p.q_kstep;
      const uint32_t pk2 = 2u * p_kstep, pk3 = 3u * p_kstep, qk2 = 2u * q_kstep, qk3 = 3u * q_kstep;
      const bool slow_mode = TXD_DBG(p, 2);
      // Start-address step (16-byte units) from one K atom of a stage to the next: K-major atoms lie side
      // by side (rows x 128 bytes each); MN-major stages are linear in K.
      const uint32_t p_atom_step = p.p_mn_major ? 4u * p.p_kstep : static_cast<uint32_t>(kBlockM) * kStageRowBytes / 16u;
      const uint32_t q_atom_step = p.q_mn_major ? 4u * p.q_kstep : static_cast<uint32_t>(q_rows_per_cta) * kStageRowBytes / 16u;
      auto wait_full = [&](uint32_t st, uint32_t ph) -> bool {
        if (!warp_mbar_wait(full0 + st * 8u, ph, ac, kDevTimeoutMmaFull, lane)) return false;
        tc_fence_after();
        return true;
      };
      // The four MMAs of one K atom into accumulator `d`; `first` is the accumulate flag of the first of them.
      auto atom_mmas = [&](uint32_t d, uint32_t plo, uint32_t qlo, uint32_t first) {
        umma<kPair, kF8>(d, desc64(p_hi, plo), desc64(q_hi, qlo), idesc, first);
        umma_acc<kPair, kF8>(d, desc64(p_hi, plo + p_kstep), desc64(q_hi, qlo + q_kstep), idesc);
        umma_acc<kPair, kF8>(d, desc64(p_hi, plo + pk2), desc64(q_hi, qlo + qk2), idesc);
        umma_acc<kPair, kF8>(d, desc64(p_hi, plo + pk3), desc64(q_hi, qlo + qk3), idesc);
      };
      bool ready = false;  // the "full" barrier of `stage` has already been seen complete (warp-uniform)
      auto advance = [&]() {
        if (++stage == n_stages) {
          stage = 0;
          phase ^= 1u;
        }
        // Look at the next stage now: the issuing thread is ahead of the pipe here, and a stage that has landed
        // needs no wait at the top of the next block.
        ready = __all_sync(0xffffffffu, mbar_test_wait(full0 + stage * 8u, phase));
      };
      while (ok && it.next(s)) {
        // Accumulator of the tile (of its first column half when the tile is wide; the second half then
        // uses the other accumulator, in the same barrier phase).
        const uint32_t vseg = seg_i * static_cast<uint32_t>(halves);
        const uint32_t acc = vseg & 1u;
        const uint32_t acc_phase = (vseg >> 1) & 1u;
        ok = warp_mbar_wait(smem_u32(&ctl->tmem_empty_bar[acc]), acc_phase ^ 1u, ac, kDevTimeoutMmaTmem, lane);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * static_cast<uint32_t>(p.block_n);
        const uint32_t d_tmem1 = tmem_base + static_cast<uint32_t>(p.block_n);  // wide: second half
        uint32_t accumulate = 0;
        // Wide tile, between the two column halves of a block. First block of the tile: the second
        // accumulator must have been drained (the epilogue hands the halves back one after the other, so
        // the first half's MMAs of this block run while the second half is still being read out).
        // Last block: the first half is complete, publish it before the second half's MMAs.
        auto between_halves = [&](bool first, bool last) -> bool {
          if (first) {
            if (!warp_mbar_wait(smem_u32(&ctl->tmem_empty_bar[1]), acc_phase ^ 1u, ac, kDevTimeoutMmaTmem, lane)) return false;
            tc_fence_after();
          }
          if (last && issuer) commit_to(smem_u32(&ctl->tmem_full_bar[0]));
          return true;
        };
        // Generic block: any MMA count (the remainder's last block, measurement modes), the first and the last
        // block of a wide tile.
        auto generic_block = [&](int n_mma, bool first, bool last) {
          if (!ready && !wait_full(stage, phase)) {
            ok = false;
            return;
          }
          // Low descriptor words (start address in 16-byte units | leading-dimension field); shared
          // memory ends below 256 KiB, so adding offsets never carries out of the 14-bit address field.
          const uint32_t plo = p_lo_base + stage * stage16;
          const uint32_t qlo = q_lo_base + stage * stage16;
          if (TXD_DBG(p, 2)) n_mma = (accumulate == 0) ? 1 : 0;
          for (int h = 0; h < halves; ++h) {
            if (h == 1 && !between_halves(first, last)) {
              ok = false;
              return;
            }
            if (issuer) {
#pragma unroll 1
              for (int j = 0; j < n_mma; ++j)
                umma<kPair, kF8>(h ? d_tmem1 : d_tmem, desc64(p_hi, plo + (j >> 2) * p_atom_step + (j & 3) * p_kstep),
                                 desc64(q_hi, qlo + h * q_half16 + (j >> 2) * q_atom_step + (j & 3) * q_kstep), idesc,
                                 (accumulate | static_cast<uint32_t>(j)) != 0 ? 1u : 0u);
            }
          }
          if (issuer) commit_to(empty0 + stage * 8u);  // frees the stage when its MMAs retire
          __syncwarp();
          if (n_mma > 0) accumulate = 1;
          advance();
        };
        // LoopSplit: blocks below `mid` belong to the main loop [lo, mid) — full, unpredicated; blocks
        // from `mid` on are the remainder loop [mid, hi), whose stages TMA zero-filled past K and whose
        // last block issues only the MMAs that cover real columns.
        const int mid = s.kb1 < p.k_main_blocks ? s.kb1 : p.k_main_blocks;
        const int last_kb = s.kb1 - 1;
        int kb = s.kb0;
        auto remainder_mmas = [&](int b) { return b == p.k_blocks - 1 ? p.tail_mmas : mmas_per_block; };
        if (halves == 2 && kb < s.kb1) {  // first block of a wide tile: waits for the second accumulator
          generic_block(remainder_mmas(kb), true, kb == last_kb);
          ++kb;
        }
        // ---- main loop ----
        int main_end = slow_mode ? kb : mid;
        if (halves == 2 && main_end > last_kb) main_end = last_kb;  // a wide tile's last block publishes its first half early
        for (; ok && kb < main_end; ++kb) {
          if (!ready && !wait_full(stage, phase)) {
            ok = false;
            break;
          }
          const uint32_t plo = p_lo_base + stage * stage16;
          const uint32_t qlo = q_lo_base + stage * stage16;
          if (issuer) {
            atom_mmas(d_tmem, plo, qlo, accumulate);
            for (int at = 1; at < atoms; ++at) atom_mmas(d_tmem, plo + at * p_atom_step, qlo + at * q_atom_step, 1u);
            if (halves == 2) {
              atom_mmas(d_tmem1, plo, qlo + q_half16, accumulate);
              for (int at = 1; at < atoms; ++at) atom_mmas(d_tmem1, plo + at * p_atom_step, qlo + q_half16 + at * q_atom_step, 1u);
            }
            commit_to(empty0 + stage * 8u);  // frees the stage when its MMAs retire
          }
          accumulate = 1;
          advance();
        }
        // ---- remainder loop (and the last block of a wide tile) ----
        for (; ok && kb < s.kb1; ++kb) generic_block(remainder_mmas(kb), false, kb == last_kb);
        if (ok && issuer) commit_to(smem_u32(&ctl->tmem_full_bar[halves == 2 ? 1u : acc]));
        __syncwarp();
        ++seg_i;
      }
      if ((!ok || *ac.flag) && issuer) {
        // Abort path: make sure no MMA is still reading shared memory / writing TMEM.
        if (kPair) tc_commit_pair(map_to_cta(smem_u32(&ctl->drain_bar), 0));
        else tc_commit(smem_u32(&ctl->drain_bar));
        const unsigned long long t0 = global_timer_ns();
        while (!mbar_try_wait(smem_u32(&ctl->drain_bar), 0)) {
          if (global_timer_ns() - t0 > ac.limit_ns) {
            atomicCAS(ac.status, 0u, static_cast<uint32_t>(kDevTimeoutDrain));
            break;
          }
        }
      }
      __syncwarp();
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    if (p.block_n >= 32)
      epilogue_role<32, kPair>(p, ctl, ac, staging, warp, lane, worker, workers, cta_rank);
    else
      epilogue_role<16, kPair>(p, ctl, ac, staging, warp, lane, worker, workers, cta_rank);
  }

  tc_fence_before();
  __syncthreads();
#ifdef TXD_MEASURE
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long *st = reinterpret_cast<unsigned long long *>(p.status) + 8;
    st[0] = stamp_c0;
    st[1] = clock64();
    st[2] = stamp_n0;
    st[3] = global_timer_ns();
  }
#endif
  // Pair: neither CTA may leave while the other can still signal its barriers, read its shared
  // memory (MMA) or write its TMEM.
  if (kPair) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}

// A translation unit that instantiates dot_umma_body under its own kernel name defines
// TXD_NO_KERNEL_ENTRY_POINTS so that these two are emitted once per library.
#ifndef TXD_NO_KERNEL_ENTRY_POINTS
// One entry point per (single | pair) x (16-bit | 8-bit operands): the operand kind is part of the MMA instruction,
// and a run-time choice of it would sit in the issuing thread's instruction stream once per MMA.
__global__ void __launch_bounds__(kNumThreads, 1) dot_umma_kernel(const __grid_constant__ DotParams p) {
  dot_umma_body<false, false>(p);
}
__global__ void __launch_bounds__(kNumThreads, 1) dot_umma_f8_kernel(const __grid_constant__ DotParams p) {
  dot_umma_body<false, true>(p);
}
__global__ void __launch_bounds__(kNumThreads, 1) dot_umma_pair_kernel(const __grid_constant__ DotParams p) {
  dot_umma_body<true, false>(p);
}
__global__ void __launch_bounds__(kNumThreads, 1) dot_umma_pair_f8_kernel(const __grid_constant__ DotParams p) {
  dot_umma_body<true, true>(p);
}
#endif  // TXD_NO_KERNEL_ENTRY_POINTS

}  // namespace txd
