// Fused attention forward for sm_100a: the two chained tt.dot of the reference's demo kernel
// (pass/LoopSplit/06-fused-attention.py:43-90 inner loop, :164-240 outer kernel) with its online softmax,
// written directly on tcgen05 / TMEM / TMA.
//
// One CTA owns 256 query rows of one (batch, head): two 128-row sub-tiles, each with its own softmax
// warpgroup, its own S accumulator and its own O accumulator in TMEM. K and V tiles of 128 rows are
// streamed once per CTA through a shared-memory ring and used by both sub-tiles.
//
//   warps 0-3 / 4-7 : softmax warpgroup of sub-tile 0 / 1 (one query row per thread): tcgen05.ld of S into
//                     registers (S is then handed back at once, so the next Q K^T overlaps this softmax),
//                     running max and sum in base 2, P = exp2(S*scale - m) rounded to the input type and
//                     written to shared memory as the A operand of the second dot, rescaling of O in TMEM
//                     (tcgen05.ld / tcgen05.st) only when the running max moved by more than 2^8, final
//                     O / l and TMA store
//   warp 8          : TMA producer (Q once; K0, K1, V0, K2, V1, ... through the ring)
//   warp 9          : tcgen05.mma issuer. Per KV block j and sub-tile t in turn: S_t(j+1) = Q_t K_{j+1}^T as soon
//                     as S_t(j) has been read, then O_t += P_t(j) V_j as soon as P_t(j) is complete; K_{j+1} is
//                     released after the second S, V_j after the second O update. Serving the sub-tiles in turn
//                     holds their softmax warpgroups half a block apart, so that one is in its exponentials
//                     while the tensor pipe and the other warpgroup's loads and row maxima run.
//
// Barriers wait by polling mbarrier.test_wait (mbarrier.try_wait was measured to return hundreds of cycles
// late even for phases completed long before, and every hop of this pipeline is on the critical path).
//
// The KV loop is executed the way LoopSplit leaves it (reference LoopSplit.cpp:179-193 applied to the
// compare at 06-fused-attention.py:64): an off-band loop over the blocks that need no mask and an
// on-band loop over the block on the diagonal (and the ragged last block when N_CTX is not a multiple of
// 128). Blocks above the diagonal, which the reference visits with every element masked (each contributes
// p == 0 and alpha == 1 exactly), are not visited.
//
// The fp8 form (kElt == 2: q, k, v and out in e5m2, the reference's `fp8_v` path, 06-fused-attention.py:81-82,191,586)
// is the same pipeline in bytes: a Q or K row of up to 128 e5m2 values is one 128-byte swizzle span (zero-filled by
// TMA past head_dim), V arrives transposed ([head_dim, n_ctx] per head, as the reference lays it out for fp8) and
// is the K-major B operand of the second dot, P is rounded to e5m2 (one span per row), both dots are
// kind::f8f6f4 MMAs of 32 bytes of K, and O is cast to e5m2 and stored straight from registers.
//
// Every wait on an mbarrier is bounded in time; a wait that runs out raises the abort flag, all roles
// leave their loops, copies in flight are drained, TMEM is released and the CTA returns.
#pragma once

#include "sm100_ptx.cuh"

namespace txa {

using namespace txd;

constexpr int kTileRows = 128;        // query rows per sub-tile == KV rows per block
constexpr int kAttnThreads = 320;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kMaxKvStages = 6;
constexpr int kAtomBytes = 128 * 128;  // 128 rows x one 128-byte swizzle span
constexpr int kPBytes = 2 * kAtomBytes;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
constexpr uint32_t kTmemCols = 512;    // S0 | S1 | O0 | O1, 128 columns each

enum AttnDeviceStatus : uint32_t {
  kAttnOk = 0,
  kAttnTimeoutProducer = 1,
  kAttnTimeoutMmaOperand = 2,
  kAttnTimeoutMmaP = 3,
  kAttnTimeoutSoftmaxS = 4,
  kAttnTimeoutSoftmaxO = 5,
  kAttnTimeoutDrain = 6
};

struct AttnParams {
  CUtensorMap tmap_q, tmap_k, tmap_v;  // 3-D {head_dim, n_ctx, batch*heads}, box {64, 128, 1}, SWIZZLE_128B
  CUtensorMap tmap_o;                  // same tensor shape, box {64, 32, 1}; unused by the fp8 form
  void *out;                           // fp8 form: [batch*heads, n_ctx, head_dim] e5m2, stored from registers
  float *m_out;                        // [batch*heads, n_ctx]: m + log2(l), as the reference stores it
  uint32_t *status;
  unsigned long long wait_limit_ns;
  float qk_scale;                      // sm_scale * log2(e)
  int32_t n_ctx, head_dim, heads_total, q_tiles;
  int32_t head_group;                  // heads per launch-order group (their K and V share L2)
  int32_t causal, is_bf16, kv_stages;
  uint32_t idesc_qk, idesc_pv;
  int32_t inject_stall;                // host-side fault injection: the producer stops after Q
};

struct AttnCtl {
  uint64_t q_full;
  uint64_t kv_full[kMaxKvStages], kv_empty[kMaxKvStages];
  uint64_t s_full[2], p_full[2], o_done[2];
  uint64_t s_free[2];     // S_t has been read into registers: the next Q K^T may overwrite it
  uint64_t drain;
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

// Four floats to four e5m2 bytes, element 0 in the lowest byte (round to nearest even, saturating).
__device__ __forceinline__ uint32_t pack_e5m2x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

template <int kElt>  // 0 f16, 1 bf16
__device__ __forceinline__ uint32_t pack_pair(float a, float b) {
  if (kElt == 1) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}

// Byte offset of the 16-byte chunk `chunk16` (0..7) of row `r` inside one K-major SWIZZLE_128B atom
// (128 rows x 128 bytes; groups of 8 rows form 1024-byte swizzle blocks).
__device__ __forceinline__ uint32_t swz_off(int r, int chunk16) {
  return static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128 + ((chunk16 ^ (r & 7)) << 4));
}

// One softmax step of one query row over a 128-column block of S held in registers.
// kMasked = false: the off-band loop (no element masked); true: the on-band loop, where `lim` is the last
// column the row may attend to.
template <bool kMasked>
__device__ __forceinline__ float row_block_max(const uint32_t (&s)[128], int col0, int lim) {
  float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 128; i += 8) {
    float x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      x[u] = __uint_as_float(s[i + u]);
      if (kMasked) x[u] = col0 + i + u <= lim ? x[u] : -INFINITY;
    }
    m0 = fmaxf(m0, fmaxf(x[0], x[1]));
    m1 = fmaxf(m1, fmaxf(x[2], x[3]));
    m2 = fmaxf(m2, fmaxf(x[4], x[5]));
    m3 = fmaxf(m3, fmaxf(x[6], x[7]));
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// P = exp2(S * qk_scale - m) for one row: written to shared memory in the input type (swizzled K-major A
// operand of the second dot); returns the fp32 row sum of the unrounded values, as the reference sums them.
// The exponentials of group g+1 are issued before group g is summed, packed and stored, so that the SFU
// pipeline does not drain between groups (a single warp per scheduler has nobody else to hide its latency).
template <bool kMasked>
__device__ __forceinline__ void exp_group(const uint32_t (&s)[128], int g, float qk_scale, float neg_m, int col0, int lim,
                                          float (&e)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    e[i] = fast_exp2(fmaf(__uint_as_float(s[g * 8 + i]), qk_scale, neg_m));
    if (kMasked) e[i] = col0 + g * 8 + i <= lim ? e[i] : 0.f;
  }
}

template <bool kMasked, int kElt>
__device__ __forceinline__ float row_block_exp_store(const uint32_t (&s)[128], float qk_scale, float neg_m, int col0,
                                                     int lim, uint32_t p_row, int row_xor) {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  float cur[8], nxt[8];
  exp_group<kMasked>(s, 0, qk_scale, neg_m, col0, lim, cur);
#pragma unroll
  for (int g = 0; g < 16; ++g) {  // 8 columns = one 16-byte chunk of P
    if (g + 1 < 16) exp_group<kMasked>(s, g + 1, qk_scale, neg_m, col0, lim, nxt);
    s0 += cur[0] + cur[1];
    s1 += cur[2] + cur[3];
    s2 += cur[4] + cur[5];
    s3 += cur[6] + cur[7];
    if (kElt == 2)  // 8 columns = 8 bytes: half of a 16-byte chunk of the row's one span
      st_shared_v2(p_row + ((((g >> 1) & 7) ^ row_xor) << 4) + (g & 1) * 8, pack_e5m2x4(cur[0], cur[1], cur[2], cur[3]),
                   pack_e5m2x4(cur[4], cur[5], cur[6], cur[7]));
    else
      st_shared_v4(p_row + (g >> 3) * kAtomBytes + (((g & 7) ^ row_xor) << 4), pack_pair<kElt>(cur[0], cur[1]),
                   pack_pair<kElt>(cur[2], cur[3]), pack_pair<kElt>(cur[4], cur[5]), pack_pair<kElt>(cur[6], cur[7]));
#pragma unroll
    for (int i = 0; i < 8; ++i) cur[i] = nxt[i];
  }
  return (s0 + s1) + (s2 + s3);
}

template <int kElt, int kD>  // kElt: 0 f16, 1 bf16, 2 e5m2
__global__ void __launch_bounds__(kAttnThreads, 1) attn_fwd_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t attn_smem_raw[];
  const uint32_t raw = smem_u32(attn_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  constexpr int D = kD;
  constexpr bool kF8 = kElt == 2;
  // One Q / K tile = one ring slot: 128 rows of D 16-bit values, or of one 128-byte span of e5m2 values.
  constexpr uint32_t tile_bytes = kF8 ? static_cast<uint32_t>(kAtomBytes) : static_cast<uint32_t>(kTileRows * D * 2);
  constexpr uint32_t v_bytes = kF8 ? static_cast<uint32_t>(D * 128) : tile_bytes;  // fp8: V^T, D rows of 128 KV bytes
  constexpr uint32_t p_bytes = kF8 ? static_cast<uint32_t>(kAtomBytes) : static_cast<uint32_t>(kPBytes);
  constexpr int d_atoms = kF8 ? 1 : D / 64;
  constexpr uint32_t kStages = (!kF8 && kD == 128) ? 3u : 6u;  // ring slots of one K or V tile each
  const uint32_t q_addr0 = base;
  const uint32_t p_addr0 = base + 2 * tile_bytes;
  const uint32_t kv_addr0 = p_addr0 + 2 * p_bytes;
  AttnCtl *ctl = reinterpret_cast<AttnCtl *>(attn_smem_raw + (kv_addr0 - raw) + kStages * tile_bytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- work: one (head, 256-row query tile). Launch order: groups of `head_group` heads whose K and V fit L2
  // together; inside a group the query tile index is the slow one, late (heavy, when causal) tiles first. The CTAs
  // that run at the same time then share one group's K and V through L2 (with all heads in one group every wave
  // of CTAs streamed every head's K and V from HBM again: 2.6 x the algorithmic bytes were measured), and the
  // last CTAs of the launch are the lightest ones. ----
  const int per_group = p.head_group * p.q_tiles;
  const int g = static_cast<int>(blockIdx.x) / per_group;
  const int r = static_cast<int>(blockIdx.x) - g * per_group;
  const int heads_here = min(p.head_group, p.heads_total - g * p.head_group);
  const int head = g * p.head_group + r % heads_here;
  const int qt = p.q_tiles - 1 - r / heads_here;
  const int q0 = qt * 2 * kTileRows;
  const int kv_blocks_all = (p.n_ctx + kTileRows - 1) / kTileRows;
  const bool ragged = (p.n_ctx % kTileRows) != 0;
  int n_blk[2], n_full[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qs = q0 + t * kTileRows;
    int n = 0;
    if (qs < p.n_ctx) n = p.causal ? min(kv_blocks_all, qs / kTileRows + 1) : kv_blocks_all;
    n_blk[t] = n;
    // LoopSplit: [0, n_full) runs unmasked, [n_full, n) masked. The masked block is the one on the diagonal
    // (causal) or the ragged last one; both can only be the last block of the loop.
    const bool last_masked = n > 0 && (p.causal || (ragged && n == kv_blocks_all));
    n_full[t] = last_masked ? n - 1 : n;
  }
  const int nmax = max(n_blk[0], n_blk[1]);

  AbortCtl ac;
  ac.flag = &ctl->abort_flag;
  ac.status = p.status;
  ac.limit_ns = p.wait_limit_ns;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&ctl->q_full), 1);
    for (int s = 0; s < static_cast<int>(kStages); ++s) {
      mbar_init(smem_u32(&ctl->kv_full[s]), 1);
      mbar_init(smem_u32(&ctl->kv_empty[s]), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(smem_u32(&ctl->s_full[t]), 1);
      mbar_init(smem_u32(&ctl->p_full[t]), kTileRows);  // every softmax thread arrives
      mbar_init(smem_u32(&ctl->o_done[t]), 1);
      mbar_init(smem_u32(&ctl->s_free[t]), kTileRows);
    }
    mbar_init(smem_u32(&ctl->drain), 1);
    ctl->abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.tmap_q);
    tma_prefetch_desc(&p.tmap_k);
    tma_prefetch_desc(&p.tmap_v);
    tma_prefetch_desc(&p.tmap_o);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;


  if (warp == kProducerWarp) {
    // ------------------------------ TMA producer ------------------------------
    const bool issuer = elect_one();
    uint32_t issued = 0;  // ring items issued
    bool ok = true;
    if (nmax > 0) {
      if (issuer) {
        const int active = (n_blk[0] > 0 ? 1 : 0) + (n_blk[1] > 0 ? 1 : 0);
        mbar_arrive_expect_tx(smem_u32(&ctl->q_full), active * tile_bytes);
        for (int t = 0; t < 2; ++t)
          if (n_blk[t] > 0)
            for (int a = 0; a < d_atoms; ++a)
              tma_load_3d(q_addr0 + t * tile_bytes + a * kAtomBytes, &p.tmap_q, a * 64, q0 + t * kTileRows, head,
                          smem_u32(&ctl->q_full));
      }
      __syncwarp();
      auto load_tile = [&](const CUtensorMap *map, int kv_block, bool is_v) {
        const uint32_t slot = issued % kStages;
        const uint32_t phase = (issued / kStages) & 1u;
        if (!warp_mbar_poll(smem_u32(&ctl->kv_empty[slot]), phase ^ 1u, ac, kAttnTimeoutProducer, lane)) {
          ok = false;
          return;
        }
        if (issuer) {
          const uint32_t bar = smem_u32(&ctl->kv_full[slot]);
          if (kF8 && is_v) {  // V^T: the KV index is the contiguous one
            mbar_arrive_expect_tx(bar, v_bytes);
            tma_load_3d(kv_addr0 + slot * tile_bytes, map, kv_block * kTileRows, 0, head, bar);
          } else {
            mbar_arrive_expect_tx(bar, tile_bytes);
            for (int a = 0; a < d_atoms; ++a)
              tma_load_3d(kv_addr0 + slot * tile_bytes + a * kAtomBytes, map, a * 64, kv_block * kTileRows, head, bar);
          }
        }
        __syncwarp();
        ++issued;
      };
      if (!p.inject_stall) {
        load_tile(&p.tmap_k, 0, false);
        for (int j = 0; ok && j < nmax; ++j) {
          if (j + 1 < nmax) load_tile(&p.tmap_k, j + 1, false);
          if (ok) load_tile(&p.tmap_v, j, true);
        }
      }
      // Copies still in flight must land before the CTA's shared memory goes away. On the normal path the
      // MMA warp has waited for every one of them; after an abort, wait for the ones of the last ring pass.
      if (ctl->abort_flag) {
        if (lane == 0) {
          mbar_wait_timed(smem_u32(&ctl->q_full), 0u, ac, kAttnTimeoutDrain);
          const uint32_t first = issued > kStages ? issued - kStages : 0u;
          for (uint32_t i = first; i < issued; ++i) {
            const unsigned long long t0 = global_timer_ns();
            const uint32_t bar = smem_u32(&ctl->kv_full[i % kStages]);
            const uint32_t ph = (i / kStages) & 1u;
            while (!mbar_try_wait(bar, ph))
              if (global_timer_ns() - t0 > ac.limit_ns) break;
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ tcgen05.mma issuer ------------------------------
    const bool issuer = elect_one();
    if (nmax > 0) {
      auto desc64 = [](uint32_t hi, uint32_t lo) { return (static_cast<uint64_t>(hi) << 32) | lo; };
      const uint32_t desc_hi = ((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);  // SBO 1024, sm_100, SWIZZLE_128B
      const uint32_t kmajor_lbo = 1u << 16;                                        // unused for swizzled K-major
      const uint32_t v_lbo = ((static_cast<uint32_t>(kAtomBytes) >> 4) & 0x3FFFu) << 16;  // between 64-column chunks
      auto lo_of = [](uint32_t addr) { return (addr & 0x3FFFFu) >> 4; };
      uint32_t taken = 0;
      bool ok = true;
      auto take = [&]() -> uint32_t {  // next ring item, in the producer's order
        const uint32_t slot = taken % kStages;
        const uint32_t phase = (taken / kStages) & 1u;
        if (!warp_mbar_poll(smem_u32(&ctl->kv_full[slot]), phase, ac, kAttnTimeoutMmaOperand, lane)) ok = false;
        ++taken;
        return slot;
      };
      // The whole warp walks these (addresses and descriptors stay warp-uniform); the elected lane issues.
      const uint32_t idesc_qk = p.idesc_qk, idesc_pv = p.idesc_pv;
      auto issue_qk = [&](int t, uint32_t k_slot) {  // S_t = Q_t K^T : head_dim / 16 MMAs of 128 x 128 x 16
        const uint32_t qa = lo_of(q_addr0 + t * tile_bytes) | kmajor_lbo;
        const uint32_t ka = lo_of(kv_addr0 + k_slot * tile_bytes) | kmajor_lbo;
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(t) * 128u;
        // One divergent region for the whole batch: the issuing lane's instruction stream is what paces the tensor
        // pipe (about 43 cycles per MMA when lean, 60 with a branch and a reconvergence around every MMA).
        if (issuer) {
#pragma unroll
          for (int i = 0; i < (kF8 ? D / 32 : D / 16); ++i) {  // 32 bytes of the head dimension per MMA
            const uint32_t step = static_cast<uint32_t>(i >> 2) * (kAtomBytes >> 4) + static_cast<uint32_t>(i & 3) * 2u;
            if (i == 0) umma<false, kF8>(d_tmem, desc64(desc_hi, qa + step), desc64(desc_hi, ka + step), idesc_qk, 0u);
            else umma_acc<false, kF8>(d_tmem, desc64(desc_hi, qa + step), desc64(desc_hi, ka + step), idesc_qk);
          }
          tc_commit(smem_u32(&ctl->s_full[t]));
        }
        __syncwarp();
      };
      auto issue_pv = [&](int t, uint32_t v_slot, bool accumulate) {  // O_t += P_t V : 8 MMAs of 128 x head_dim x 16
        const uint32_t pa = lo_of(p_addr0 + t * p_bytes) | kmajor_lbo;
        const uint32_t va = lo_of(kv_addr0 + v_slot * tile_bytes) | (kF8 ? kmajor_lbo : v_lbo);
        const uint32_t d_tmem = tmem_base + 256u + static_cast<uint32_t>(t) * 128u;
        if (issuer && kF8) {
          // P (128 rows x 128 KV bytes) and V^T (D rows x 128 KV bytes) are both K-major: 4 MMAs of 32 KV bytes
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t step = static_cast<uint32_t>(i) * 2u;
            if (i == 0) umma<false, true>(d_tmem, desc64(desc_hi, pa + step), desc64(desc_hi, va + step), idesc_pv, accumulate ? 1u : 0u);
            else umma_acc<false, true>(d_tmem, desc64(desc_hi, pa + step), desc64(desc_hi, va + step), idesc_pv);
          }
          tc_commit(smem_u32(&ctl->o_done[t]));
        } else if (issuer) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t pstep = static_cast<uint32_t>(i >> 2) * (kAtomBytes >> 4) + static_cast<uint32_t>(i & 3) * 2u;
            const uint32_t vstep = static_cast<uint32_t>(i) * (16u * 128u >> 4);  // 16 KV rows of 128 bytes
            if (i == 0) umma<false, false>(d_tmem, desc64(desc_hi, pa + pstep), desc64(desc_hi, va + vstep), idesc_pv, accumulate ? 1u : 0u);
            else umma_acc<false, false>(d_tmem, desc64(desc_hi, pa + pstep), desc64(desc_hi, va + vstep), idesc_pv);
          }
          tc_commit(smem_u32(&ctl->o_done[t]));
        }
        __syncwarp();
      };
      auto release = [&](uint32_t slot) {
        if (issuer) tc_commit(smem_u32(&ctl->kv_empty[slot]));
        __syncwarp();
      };

      ok = warp_mbar_poll(smem_u32(&ctl->q_full), 0u, ac, kAttnTimeoutMmaOperand, lane);
      uint32_t k_slot = 0;
      if (ok) k_slot = take();
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (n_blk[t] > 0) issue_qk(t, k_slot);
        release(k_slot);
      }
      // Order of a block's four batches of MMAs: per sub-tile the next S (as soon as its softmax warps hold S(j) in
      // registers), then O_t += P_t(j) V_j (once P_t(j) is in shared memory and O_t is rescaled); K_{j+1} goes back to
      // the producer as soon as both next-S dots are issued. Sub-tile 1's next S is then issued only after sub-tile 0
      // has finished its block, which keeps the two softmax warpgroups half a block apart: one is in its exponentials
      // while the other waits, loads and takes its row maxima. With both next-S dots first, [S0, S1, O0, O1], the
      // warpgroups ran in step, in their exponentials at the same time and idle at the same time. Measured, batch
      // 4 x 32 heads, N_CTX 4096: HEAD_DIM 64 0.916 -> 0.812 ms, causal 0.528 -> 0.496 ms, HEAD_DIM 128 1.064 -> 1.011 ms,
      // causal 0.607 -> 0.587 ms, fp8 HEAD_DIM 128 1.078 -> 1.011 ms.
      // K_{j+1} is taken off the ring one block early, while the warp would otherwise wait for P_1 (a take costs this
      // warp about 250 cycles even when the tile arrived long ago, and this warp's program paces the block).
      // With six ring slots V_{j+1} is in shared memory by then as well and is taken early too; with three its copy
      // only starts when K_{j+1} has just been handed back.
      constexpr bool kVAhead = kStages >= 6;
      uint32_t k_ahead = 0, v_ahead = 0;
      if (ok && nmax > 1) k_ahead = take();
      if (ok && kVAhead) v_ahead = take();
      for (int j = 0; ok && j < nmax; ++j) {
        const bool have_next = j + 1 < nmax;
        const uint32_t kn_slot = k_ahead;
        const uint32_t v_slot = kVAhead ? v_ahead : take();
        if (!ok) break;
        auto next_s = [&](int t) {
          if (!(have_next && j + 1 < n_blk[t])) return;
          if (!warp_mbar_poll(smem_u32(&ctl->s_free[t]), static_cast<uint32_t>(j) & 1u, ac, kAttnTimeoutMmaP, lane)) {
            ok = false;
            return;
          }
          tc_fence_after();
          issue_qk(t, kn_slot);
        };
        auto update_o = [&](int t) {
          if (j >= n_blk[t]) return;
          if (!warp_mbar_poll(smem_u32(&ctl->p_full[t]), static_cast<uint32_t>(j) & 1u, ac, kAttnTimeoutMmaP, lane)) {
            ok = false;
            return;
          }
          tc_fence_after();
          issue_pv(t, v_slot, j > 0);
        };
        next_s(0);
        if (ok) update_o(0);
        if (ok) next_s(1);
        if (!ok) break;
        if (have_next) release(kn_slot);
        if (j + 2 < nmax) {
          k_ahead = take();
          if (!ok) break;
        }
        if (kVAhead && have_next) {
          v_ahead = take();
          if (!ok) break;
        }
        update_o(1);
        if (!ok) break;
        release(v_slot);
      }
      // every MMA issued above has completed before TMEM and shared memory are given back
      if (issuer) tc_commit(smem_u32(&ctl->drain));
      __syncwarp();
      if (lane == 0) {
        const unsigned long long t0 = global_timer_ns();
        while (!mbar_try_wait(smem_u32(&ctl->drain), 0u)) {
          if (global_timer_ns() - t0 > ac.limit_ns) {
            ctl->abort_flag = 1;
            atomicCAS(ac.status, 0u, static_cast<uint32_t>(kAttnTimeoutDrain));
            break;
          }
        }
      }
      __syncwarp();
    }
  } else {
    // ------------------------------ softmax warpgroups ------------------------------
    const int t = warp >> 2;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int row = q0 + t * kTileRows + row_in_tile;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_tmem = lane_base + static_cast<uint32_t>(t) * 128u;
    const uint32_t o_tmem = lane_base + 256u + static_cast<uint32_t>(t) * 128u;
    const uint32_t p_tile = p_addr0 + t * p_bytes;
    const uint32_t p_row = p_tile + static_cast<uint32_t>((row_in_tile >> 3) * 1024 + (row_in_tile & 7) * 128);
    const int row_xor = row_in_tile & 7;
    const int lim = p.causal ? min(row, p.n_ctx - 1) : p.n_ctx - 1;  // last column this row may attend to
    const int n = n_blk[t];
    float m_i = -INFINITY, l_i = 0.f;
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      if (!warp_mbar_poll(smem_u32(&ctl->s_full[t]), static_cast<uint32_t>(j) & 1u, ac, kAttnTimeoutSoftmaxS, lane)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t s[128];
      tmem_ld_32x32(s_tmem, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_ld_32x32(s_tmem + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      tmem_ld_32x32(s_tmem + 64, *reinterpret_cast<uint32_t(*)[32]>(&s[64]));
      tmem_ld_32x32(s_tmem + 96, *reinterpret_cast<uint32_t(*)[32]>(&s[96]));
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(smem_u32(&ctl->s_free[t]));
      const bool masked = j >= n_full[t];
      const int col0 = j * kTileRows;
      const float mx = masked ? row_block_max<true>(s, col0, lim) : row_block_max<false>(s, col0, lim);
      // The running max is only moved when the block's max exceeds it by more than 2^8: until then
      // exponentials are taken against the older, smaller reference (values up to 256, exact to the same
      // relative precision), alpha is exactly 1 and O needs no rescaling. O / l and m + log2(l) do not
      // depend on which reference was used.
      const float m_cand = fmaxf(m_i, mx * p.qk_scale);
      float m_new = (m_cand - m_i > kRescaleThreshold) ? m_cand : m_i;
      if (m_new == -INFINITY) m_new = 0.f;  // a row with nothing to attend to yet
      const float alpha = fast_exp2(m_i - m_new);
      if (j > 0) {
        // O_t += P_t(j-1) V has completed: P_t may be overwritten and O_t rescaled
        if (!warp_mbar_poll(smem_u32(&ctl->o_done[t]), static_cast<uint32_t>(j - 1) & 1u, ac, kAttnTimeoutSoftmaxO,
                            lane)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(o_tmem + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(o_tmem + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      const float sum = masked ? row_block_exp_store<true, kElt>(s, p.qk_scale, -m_new, col0, lim, p_row, row_xor)
                               : row_block_exp_store<false, kElt>(s, p.qk_scale, -m_new, col0, lim, p_row, row_xor);
      l_i = l_i * alpha + sum;
      m_i = m_new;
      fence_proxy_async();  // P is read by the tensor core through the async proxy
      tc_fence_before();
      mbar_arrive(smem_u32(&ctl->p_full[t]));
    }
    if (ok && n > 0) {
      // ---- epilogue of the sub-tile: O / l, cast, store; M = m + log2(l) ----
      ok = warp_mbar_poll(smem_u32(&ctl->o_done[t]), static_cast<uint32_t>(n - 1) & 1u, ac, kAttnTimeoutSoftmaxO, lane);
      if (ok) {
        tc_fence_after();
        const float inv_l = 1.0f / l_i;
        if (kF8) {
          // O / l as e5m2, 32 columns = 32 bytes at a time, straight from this thread's registers to its row
          uint8_t *o_row = static_cast<uint8_t *>(p.out) + (static_cast<long long>(head) * p.n_ctx + row) * p.head_dim;
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(o_tmem + c * 32, o);
            tmem_ld_wait();
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              w[i] = pack_e5m2x4(__uint_as_float(o[4 * i]) * inv_l, __uint_as_float(o[4 * i + 1]) * inv_l,
                                 __uint_as_float(o[4 * i + 2]) * inv_l, __uint_as_float(o[4 * i + 3]) * inv_l);
            if (row < p.n_ctx) {
              if (c * 32 < p.head_dim) *reinterpret_cast<uint4 *>(o_row + c * 32) = make_uint4(w[0], w[1], w[2], w[3]);
              if (c * 32 + 16 < p.head_dim) *reinterpret_cast<uint4 *>(o_row + c * 32 + 16) = make_uint4(w[4], w[5], w[6], w[7]);
            }
          }
        } else {
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(o_tmem + c * 32, o);
          tmem_ld_wait();
          // 32 columns = 64 bytes = chunks (c&1)*4 .. +3 of this row in atom c/2 (P_t's buffer is free now)
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              w[i] = pack_pair<kElt>(__uint_as_float(o[q * 8 + 2 * i]) * inv_l, __uint_as_float(o[q * 8 + 2 * i + 1]) * inv_l);
            st_shared_v4(p_tile + (c >> 1) * kAtomBytes + swz_off(row_in_tile, (c & 1) * 4 + q), w[0], w[1], w[2], w[3]);
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0 && q0 + t * kTileRows + quarter * 32 < p.n_ctx) {  // rows past n_ctx are clipped by the copy
          for (int a = 0; a < d_atoms; ++a)
            tma_store_3d(&p.tmap_o, p_tile + a * kAtomBytes + quarter * 32 * 128, a * 64, q0 + t * kTileRows + quarter * 32,
                         head);
          bulk_commit_group();
          bulk_wait_group_all();
        }
        __syncwarp();
        }
        if (row < p.n_ctx) p.m_out[static_cast<long long>(head) * p.n_ctx + row] = m_i + log2f(l_i);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace txa
