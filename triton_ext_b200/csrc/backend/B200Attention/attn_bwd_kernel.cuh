// Fused attention backward for sm_100a. head_dim 64: dK, dV and dQ in one kernel, five tt.dot per (KV block,
// query block) pair with all accumulators in tensor memory; head_dim 128: the same kernel without the dQ dot, and a
// second kernel for dQ (tensor memory holds four 128-column accumulators, not five). The mathematics is the reference's
// (pass/LoopSplit/06-fused-attention.py: _attn_bwd_dkdv :351-400, _attn_bwd_dq :404-448):
//
//   S^T  = K Q^T                    P^T = exp2(S^T * scale - M[q])      (M = the forward's m + log2 l)
//   dV  += P^T dO                   dP^T = V dO^T
//   dS^T = P^T * (dP^T - delta[q])  dK  += dS^T Q                       dQ[q block] += dS K
//
// with P^T and dS^T rounded to the input type before their dots, as the reference rounds them (:386,:392,:436).
//
// One CTA owns one KV block of 128 rows of one (batch, head) and walks the query blocks that see it (all of
// them, or those at and below the diagonal when causal: the split LoopSplit makes of the reference's loops, the
// diagonal block being the masked one). K and V stay in shared memory; Q and dO tiles stream through a ring.
//
//   warps 0-7 : two threads per TMEM lane (= KV row for S^T, dP^T, dV, dK; = query row for the dQ partial), each
//               with half of the columns:
//               P^T and dS^T into shared memory (the A operands of the next dots), the dQ partial from TMEM
//               through shared memory and a TMA reduce-add into an fp32 accumulator, dV and dK at the end
//   warp 8    : TMA producer (K, V once; Q, dO per query block) and the M / delta vectors of the block
//   warp 9    : tcgen05.mma issuer. Order per query block i: dV(i), S^T(i+1) as soon as P^T(i) is written;
//               dK(i), dQ(i), dP^T(i+1) as soon as dS^T(i) is written: the next block's scores are ready when the
//               compute warps come back for them
//
// dS^T lies in shared memory as [KV row][query] (K-major for dK += dS^T Q); dQ += dS K reads the same bytes
// as an MN-major A operand, so dS is never transposed or stored twice. Every wait is bounded.
#pragma once

#include "attn_fwd_kernel.cuh"

namespace txa {

constexpr int kBwdComputeWarps = 8;   // two threads per TMEM lane, 64 columns each
constexpr int kBwdProducerWarp = 8;
constexpr int kBwdMmaWarp = 9;
constexpr int kBwdThreads = 10 * 32;
constexpr int kBwdStages = 2;  // ring slots at head_dim 64; head_dim 128 has shared memory for one
constexpr int kDqSlabBytes = 32 * 128;  // one compute warp's dQ staging: 32 query rows x 32 fp32 columns

struct AttnBwdParams {
  CUtensorMap tmap_q, tmap_k, tmap_v, tmap_do;  // 3-D {head_dim, n_ctx, batch*heads}, box {64, 128, 1}, SWIZZLE_128B
  CUtensorMap tmap_dq;  // head_dim 64: the fp32 dq accumulator, 3-D {64, n_ctx, batch*heads}, box {32, 32, 1}
  const float *m;       // [batch*heads, n_ctx] from the forward
  const float *delta;   // [batch*heads, n_ctx] rowsum(o * do)
  float *dq_acc;        // [batch*heads, n_ctx, 64] fp32, zero on entry
  void *dk, *dv;        // [batch*heads, n_ctx, 64] in the input type
  uint32_t *status;
  unsigned long long wait_limit_ns;
  float qk_scale, sm_scale;
  int32_t n_ctx, heads_total, kv_blocks;
  int32_t head_dim;     // columns of q, k, v, do, dk, dv in memory (16 or 32 on the 64-wide kernel: the rest is zero fill)
  int32_t causal;
  uint32_t idesc_st;    // 128 x 128, A and B K-major          (S^T, dP^T)
  uint32_t idesc_acc;   // 128 x 64, A K-major, B MN-major      (dV, dK)
  uint32_t idesc_dq;    // 128 x 64, A MN-major, B MN-major     (dQ partial)
  int32_t inject_stall;
};

struct AttnBwdCtl {
  uint64_t kv_full;
  uint64_t full[kBwdStages], empty[kBwdStages];
  uint64_t s_full, dp_full, pt_full, ds_full, dq_full, dq_free, drain;
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  alignas(16) float m_s[kBwdStages][kTileRows];
  alignas(16) float delta_s[kBwdStages][kTileRows];
};

// P^T[kv row][query] = exp2(S^T * scale - M[query]) for 64 queries of one KV row: the fp32 values stay in `s` (dS
// needs them), the rounded ones go to shared memory (one atom of the A operand of dV += P^T dO).
// kMasked: diagonal and ragged blocks; q0 is the first query of these 64 columns.
template <bool kMasked, bool kBf16>
__device__ __forceinline__ void bwd_row_p(uint32_t (&s)[64], const float *m_s, float qk_scale, int q0, int kv_row, int n_ctx,
                                          int causal, uint32_t pt_row, int row_xor) {
  const float4 *m4 = reinterpret_cast<const float4 *>(m_s);
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const float4 ma = m4[g * 2], mb = m4[g * 2 + 1];
    const float mm[8] = {ma.x, ma.y, ma.z, ma.w, mb.x, mb.y, mb.z, mb.w};
    float e[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = g * 8 + i;
      float x = fast_exp2(fmaf(__uint_as_float(s[c]), qk_scale, -mm[i]));
      if (kMasked) {
        const int qrow = q0 + c;
        const bool valid = qrow < n_ctx && kv_row < n_ctx && (!causal || qrow >= kv_row);
        x = valid ? x : 0.f;
      }
      e[i] = x;
      s[c] = __float_as_uint(x);
    }
    st_shared_v4(pt_row + ((g ^ row_xor) << 4), pack_pair<kBf16>(e[0], e[1]), pack_pair<kBf16>(e[2], e[3]),
                 pack_pair<kBf16>(e[4], e[5]), pack_pair<kBf16>(e[6], e[7]));
  }
}

// kD = 64: dK, dV and dQ. kD = 128: dK and dV only (tensor memory has no room for the fifth accumulator); dQ comes from
// attn_bwd_dq_kernel below, as in the reference's two passes.
template <bool kBf16, int kD>
__global__ void __launch_bounds__(kBwdThreads, 1) attn_bwd_kernel(const __grid_constant__ AttnBwdParams p) {
  constexpr bool kWithDq = kD == 64;
  constexpr int kStagesT = kD == 64 ? kBwdStages : 1;
  constexpr int kAtoms = kD / 64;
  constexpr uint32_t kBwdTileBytes = kTileRows * kD * 2;  // one K / V / Q / dO tile, kAtoms swizzle atoms wide
  extern __shared__ uint8_t attn_bwd_smem_raw[];
  const uint32_t raw = smem_u32(attn_bwd_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t k_addr = base, v_addr = base + kBwdTileBytes;
  const uint32_t ring_addr = base + 2 * kBwdTileBytes;             // per stage: Q tile, dO tile
  const uint32_t pt_addr = ring_addr + kStagesT * 2 * kBwdTileBytes;  // P^T  [128 KV rows][128 queries], 2 atoms
  const uint32_t ds_addr = pt_addr + kPBytes;                      // dS^T, same layout
  const uint32_t dqs_addr = ds_addr + kPBytes;                     // (kD 64) dQ staging, one slab per compute warp
  const uint32_t ctl_addr = dqs_addr + (kWithDq ? kBwdComputeWarps * kDqSlabBytes : 0);
  AttnBwdCtl *ctl = reinterpret_cast<AttnBwdCtl *>(attn_bwd_smem_raw + (ctl_addr - raw));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- work: (head, KV block); the KV block index is the fast one, early (heavy, when causal) blocks first ----
  const int head = static_cast<int>(blockIdx.x) / p.kv_blocks;
  const int j = static_cast<int>(blockIdx.x) % p.kv_blocks;
  const int kv0 = j * kTileRows;
  const int q_blocks = (p.n_ctx + kTileRows - 1) / kTileRows;
  const int i_lo = p.causal ? j : 0;
  const int n_it = q_blocks - i_lo;
  const bool kv_ragged = kv0 + kTileRows > p.n_ctx;

  AbortCtl ac;
  ac.flag = &ctl->abort_flag;
  ac.status = p.status;
  ac.limit_ns = p.wait_limit_ns;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&ctl->kv_full), 1);
    for (int s = 0; s < kStagesT; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 2);  // the TMA transaction and the M / delta vectors
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    mbar_init(smem_u32(&ctl->s_full), 1);
    mbar_init(smem_u32(&ctl->dp_full), 1);
    mbar_init(smem_u32(&ctl->pt_full), 2 * kTileRows);
    mbar_init(smem_u32(&ctl->ds_full), 2 * kTileRows);
    mbar_init(smem_u32(&ctl->dq_full), 1);
    mbar_init(smem_u32(&ctl->dq_free), 2 * kTileRows);
    mbar_init(smem_u32(&ctl->drain), 1);
    ctl->abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.tmap_q);
    tma_prefetch_desc(&p.tmap_k);
    tma_prefetch_desc(&p.tmap_v);
    tma_prefetch_desc(&p.tmap_do);
    if (kWithDq) tma_prefetch_desc(&p.tmap_dq);
  }
  if (warp == kBwdMmaWarp) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  // TMEM columns: S^T 0..127 | dP^T 128..255 | dV 256.. | dK 256+kD.. | (kD 64) dQ partial 384..447
  constexpr uint32_t kColSt = 0, kColDp = 128, kColDv = 256, kColDk = 256 + kD, kColDq = 384;

  if (warp == kBwdProducerWarp) {
    // ------------------------------ producer ------------------------------
    const bool issuer = elect_one();
    if (issuer) {
      const uint32_t bar = smem_u32(&ctl->kv_full);
      mbar_arrive_expect_tx(bar, 2 * kBwdTileBytes);
      for (int a = 0; a < kAtoms; ++a) {
        tma_load_3d(k_addr + a * kAtomBytes, &p.tmap_k, a * 64, kv0, head, bar);
        tma_load_3d(v_addr + a * kAtomBytes, &p.tmap_v, a * 64, kv0, head, bar);
      }
    }
    __syncwarp();
    int issued = 0;
    bool ok = true;
    for (int it = 0; ok && it < n_it && !p.inject_stall; ++it) {
      const int slot = it % kStagesT;
      const uint32_t phase = static_cast<uint32_t>(it / kStagesT) & 1u;
      if (!warp_mbar_poll(smem_u32(&ctl->empty[slot]), phase ^ 1u, ac, kAttnTimeoutProducer, lane)) {
        ok = false;
        break;
      }
      const int q0 = (i_lo + it) * kTileRows;
      const uint32_t bar = smem_u32(&ctl->full[slot]);
      if (issuer) {
        mbar_arrive_expect_tx(bar, 2 * kBwdTileBytes);
        for (int a = 0; a < kAtoms; ++a) {
          tma_load_3d(ring_addr + slot * 2 * kBwdTileBytes + a * kAtomBytes, &p.tmap_q, a * 64, q0, head, bar);
          tma_load_3d(ring_addr + slot * 2 * kBwdTileBytes + kBwdTileBytes + a * kAtomBytes, &p.tmap_do, a * 64, q0, head, bar);
        }
      }
      // M and delta of the 128 query rows (rows past n_ctx are masked later; give them harmless values)
      for (int r = lane; r < kTileRows; r += 32) {
        const int row = q0 + r;
        const long long g = static_cast<long long>(head) * p.n_ctx + row;
        ctl->m_s[slot][r] = row < p.n_ctx ? p.m[g] : 0.f;
        ctl->delta_s[slot][r] = row < p.n_ctx ? p.delta[g] : 0.f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar);
      __syncwarp();
      ++issued;
    }
    if (ctl->abort_flag) {  // copies in flight must land before shared memory goes away
      if (lane == 0) {
        mbar_wait_timed(smem_u32(&ctl->kv_full), 0u, ac, kAttnTimeoutDrain);
        const int first = issued > kStagesT ? issued - kStagesT : 0;
        for (int it = first; it < issued; ++it) {
          const unsigned long long t0 = global_timer_ns();
          const uint32_t bar = smem_u32(&ctl->full[it % kStagesT]);
          const uint32_t ph = static_cast<uint32_t>(it / kStagesT) & 1u;
          while (!mbar_try_wait(bar, ph))
            if (global_timer_ns() - t0 > ac.limit_ns) break;
        }
      }
      __syncwarp();
    }
  } else if (warp == kBwdMmaWarp) {
    // ------------------------------ tcgen05.mma issuer ------------------------------
    const bool issuer = elect_one();
    auto desc64 = [](uint32_t hi, uint32_t lo) { return (static_cast<uint64_t>(hi) << 32) | lo; };
    const uint32_t desc_hi = ((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);  // SBO 1024, sm_100, SWIZZLE_128B
    const uint32_t lbo_unused = 1u << 16;
    const uint32_t lbo_atom = ((static_cast<uint32_t>(kAtomBytes) >> 4) & 0x3FFFu) << 16;  // between 64-element chunks
    auto lo_of = [](uint32_t addr) { return (addr & 0x3FFFFu) >> 4; };
    // K-major operand, one atom (head_dim 64): 4 MMAs, +32 bytes per MMA
    // K-major operand, two atoms (128 queries): 8 MMAs, atom step after 4
    // MN-major operand [K rows][64 or 128 contiguous]: 16 K rows = 2048 bytes per MMA
    auto kmajor_step = [](int i) { return static_cast<uint32_t>(i >> 2) * (kAtomBytes >> 4) + static_cast<uint32_t>(i & 3) * 2u; };
    auto mn_step = [](int i) { return static_cast<uint32_t>(i) * (16u * 128u >> 4); };
    bool ok = warp_mbar_poll(smem_u32(&ctl->kv_full), 0u, ac, kAttnTimeoutMmaOperand, lane);
    auto stage_q = [&](int it) { return ring_addr + static_cast<uint32_t>(it % kStagesT) * 2 * kBwdTileBytes; };
    auto wait_stage = [&](int it) {
      return warp_mbar_poll(smem_u32(&ctl->full[it % kStagesT]), static_cast<uint32_t>(it / kStagesT) & 1u, ac,
                            kAttnTimeoutMmaOperand, lane);
    };
    auto issue_st = [&](int it) {  // S^T = K Q^T
      const uint32_t q_addr = stage_q(it);
      if (issuer) {
#pragma unroll
        for (int i = 0; i < kD / 16; ++i)
          umma_f16(tmem_base + kColSt, desc64(desc_hi, (lo_of(k_addr) | lbo_unused) + kmajor_step(i)),
                   desc64(desc_hi, (lo_of(q_addr) | lbo_unused) + kmajor_step(i)), p.idesc_st, i > 0 ? 1u : 0u);
      }
      if (issuer) tc_commit(smem_u32(&ctl->s_full));
      __syncwarp();
    };
    auto issue_dp = [&](int it) {  // dP^T = V dO^T
      const uint32_t do_addr = stage_q(it) + kBwdTileBytes;
      if (issuer) {
#pragma unroll
        for (int i = 0; i < kD / 16; ++i)
          umma_f16(tmem_base + kColDp, desc64(desc_hi, (lo_of(v_addr) | lbo_unused) + kmajor_step(i)),
                   desc64(desc_hi, (lo_of(do_addr) | lbo_unused) + kmajor_step(i)), p.idesc_st, i > 0 ? 1u : 0u);
      }
      if (issuer) tc_commit(smem_u32(&ctl->dp_full));
      __syncwarp();
    };
    if (ok && n_it > 0) ok = wait_stage(0);
    if (ok && n_it > 0) {
      tc_fence_after();
      issue_st(0);
      issue_dp(0);
    }
    for (int it = 0; ok && it < n_it; ++it) {
      const int slot = it % kStagesT;
      const uint32_t ph = static_cast<uint32_t>(it) & 1u;
      const uint32_t q_addr = stage_q(it), do_addr = q_addr + kBwdTileBytes;
      // dV += P^T dO, then the next block's scores (the compute warps hold S^T(it) in registers by now)
      if (!warp_mbar_poll(smem_u32(&ctl->pt_full), ph, ac, kAttnTimeoutMmaP, lane)) break;
      tc_fence_after();
      if (issuer) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          umma_f16(tmem_base + kColDv, desc64(desc_hi, (lo_of(pt_addr) | lbo_unused) + kmajor_step(i)),
                   desc64(desc_hi, (lo_of(do_addr) | lbo_atom) + mn_step(i)), p.idesc_acc, (it > 0 || i > 0) ? 1u : 0u);
      }
      __syncwarp();
      if (kStagesT > 1 && it + 1 < n_it) {
        if (!wait_stage(it + 1)) break;
        issue_st(it + 1);
      }
      // dK += dS^T Q, dQ partial = dS K, then the next block's dP^T
      if (!warp_mbar_poll(smem_u32(&ctl->ds_full), ph, ac, kAttnTimeoutMmaP, lane)) break;
      if (kWithDq && it > 0 && !warp_mbar_poll(smem_u32(&ctl->dq_free), ph ^ 1u, ac, kAttnTimeoutMmaP, lane)) break;
      tc_fence_after();
      if (issuer) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          umma_f16(tmem_base + kColDk, desc64(desc_hi, (lo_of(ds_addr) | lbo_unused) + kmajor_step(i)),
                   desc64(desc_hi, (lo_of(q_addr) | lbo_atom) + mn_step(i)), p.idesc_acc, (it > 0 || i > 0) ? 1u : 0u);
      }
      if (issuer) {
#pragma unroll
        for (int i = 0; i < (kWithDq ? 8 : 0); ++i)
          umma_f16(tmem_base + kColDq, desc64(desc_hi, (lo_of(ds_addr) | lbo_atom) + mn_step(i)),
                   desc64(desc_hi, (lo_of(k_addr) | lbo_atom) + mn_step(i)), p.idesc_dq, i > 0 ? 1u : 0u);
      }
      if (issuer) {
        tc_commit(smem_u32(&ctl->dq_full));
        tc_commit(smem_u32(&ctl->empty[slot]));
      }
      __syncwarp();
      if (it + 1 < n_it) {
        if (kStagesT == 1) {  // one ring slot: the next tiles can only arrive once this block's dots are through
          if (!wait_stage(it + 1)) break;
          tc_fence_after();
          issue_st(it + 1);
        }
        issue_dp(it + 1);
      }
    }
    // every MMA issued above has completed before TMEM and shared memory are given back (also after an abort)
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
  } else {
    // ------------------------------ compute warps ------------------------------
    const int quarter = warp & 3;
    const int half = warp >> 2;         // which 64 of the 128 columns of S^T / dP^T, which 32 of dV / dK / dQ
    const int r = quarter * 32 + lane;  // TMEM lane
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t row_off = static_cast<uint32_t>(half * kAtomBytes + (r >> 3) * 1024 + (r & 7) * 128);
    const int row_xor = r & 7;
    const int kv_row = kv0 + r;
    bool ok = true;
    // The dQ partial of a query block (lane = query row): this warp's 32 rows x 32 columns go through a swizzled
    // shared-memory slab and one TMA reduce-add into the fp32 accumulator (full-line transactions in the copy
    // engine; 2048 scattered 16-byte reductions per block from the threads took 2000 cycles). Rows past n_ctx
    // are clipped by the copy.
    const uint32_t dq_slab = dqs_addr + static_cast<uint32_t>(warp) * kDqSlabBytes;
    auto dq_readout = [&](int it_done) -> bool {
      if (!warp_mbar_poll(smem_u32(&ctl->dq_full), static_cast<uint32_t>(it_done) & 1u, ac, kAttnTimeoutSoftmaxO, lane)) return false;
      tc_fence_after();
      uint32_t v[32];
      tmem_ld_32x32(lane_base + kColDq + half * 32, v);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(smem_u32(&ctl->dq_free));
      if (lane == 0) bulk_wait_group_read<0>();  // the slab's previous reduction has been read
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 8; ++c)
        st_shared_v4(dq_slab + lane * 128 + ((c ^ (lane & 7)) << 4), v[c * 4], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
      fence_proxy_async();
      __syncwarp();
      const int row0 = (i_lo + it_done) * kTileRows + quarter * 32;
      if (lane == 0 && row0 < p.n_ctx) {
        tma_reduce_add_3d(&p.tmap_dq, dq_slab, half * 32, row0, head);
        bulk_commit_group();
      }
      return true;
    };
    for (int it = 0; it < n_it; ++it) {
      const int slot = it % kStagesT;
      const uint32_t ring_phase = static_cast<uint32_t>(it / kStagesT) & 1u;
      const uint32_t ph = static_cast<uint32_t>(it) & 1u;
      const int q0 = (i_lo + it) * kTileRows;
      const bool masked = (p.causal && i_lo + it == j) || kv_ragged || q0 + kTileRows > p.n_ctx;
      // the block's M and delta are in shared memory once its stage is full
      if (!warp_mbar_poll(smem_u32(&ctl->full[slot]), ring_phase, ac, kAttnTimeoutSoftmaxS, lane) ||
          !warp_mbar_poll(smem_u32(&ctl->s_full), ph, ac, kAttnTimeoutSoftmaxS, lane)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t s[64];
      tmem_ld_32x32(lane_base + kColSt + half * 64, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_ld_32x32(lane_base + kColSt + half * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      tmem_ld_wait();
      const float *m_s = ctl->m_s[slot] + half * 64;
      const float *delta_s = ctl->delta_s[slot] + half * 64;
      if (masked) bwd_row_p<true, kBf16>(s, m_s, p.qk_scale, q0 + half * 64, kv_row, p.n_ctx, p.causal, pt_addr + row_off, row_xor);
      else bwd_row_p<false, kBf16>(s, m_s, p.qk_scale, q0 + half * 64, kv_row, p.n_ctx, p.causal, pt_addr + row_off, row_xor);
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(smem_u32(&ctl->pt_full));
      // the previous block's dQ partial, while the tensor pipe works on dV and the next scores
      if (kWithDq && it > 0 && !dq_readout(it - 1)) {
        ok = false;
        break;
      }
      // dS^T = P^T * (dP^T - delta[query])
      if (!warp_mbar_poll(smem_u32(&ctl->dp_full), ph, ac, kAttnTimeoutSoftmaxS, lane)) {
        ok = false;
        break;
      }
      tc_fence_after();
#pragma unroll
      for (int c4 = 0; c4 < 2; ++c4) {
        uint32_t dp[32];
        tmem_ld_32x32(lane_base + kColDp + half * 64 + c4 * 32, dp);
        tmem_ld_wait();
#pragma unroll
        for (int gg = 0; gg < 4; ++gg) {
          const float4 da = reinterpret_cast<const float4 *>(delta_s)[c4 * 8 + gg * 2];
          const float4 db = reinterpret_cast<const float4 *>(delta_s)[c4 * 8 + gg * 2 + 1];
          const float dd[8] = {da.x, da.y, da.z, da.w, db.x, db.y, db.z, db.w};
          float e[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int c = c4 * 32 + gg * 8 + i;
            e[i] = __uint_as_float(s[c]) * (__uint_as_float(dp[gg * 8 + i]) - dd[i]);
          }
          const int g = c4 * 4 + gg;
          st_shared_v4(ds_addr + row_off + ((g ^ row_xor) << 4), pack_pair<kBf16>(e[0], e[1]), pack_pair<kBf16>(e[2], e[3]),
                       pack_pair<kBf16>(e[4], e[5]), pack_pair<kBf16>(e[6], e[7]));
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(smem_u32(&ctl->ds_full));
    }
    if (ok && n_it > 0) {
      if (kWithDq) ok = dq_readout(n_it - 1);
      else ok = warp_mbar_poll(smem_u32(&ctl->dq_full), static_cast<uint32_t>(n_it - 1) & 1u, ac, kAttnTimeoutSoftmaxO, lane);
    }
    if (ok && n_it > 0) {
      // every MMA has completed (the last dq_full was committed after them): dV and dK of this KV block, this
      // thread's 32 columns. The TMEM loads are warp-wide; rows past n_ctx take part in them and store nothing.
      tc_fence_after();
      const int col0 = half * (kD / 2);  // first of this thread's columns
      const long long g = (static_cast<long long>(head) * p.n_ctx + kv_row) * p.head_dim + col0;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const float scale = which == 0 ? 1.0f : p.sm_scale;
        uint4 *dst = reinterpret_cast<uint4 *>(static_cast<char *>(which == 0 ? p.dv : p.dk) + g * 2);
#pragma unroll
        for (int c = 0; c < kD / 64; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(lane_base + (which == 0 ? kColDv : kColDk) + half * (kD / 2) + c * 32, v);
          tmem_ld_wait();
          if (kv_row < p.n_ctx) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (col0 + c * 32 + q * 8 >= p.head_dim) continue;  // zero-fill columns of a narrow head: not in memory
              uint4 w;
              w.x = pack_pair<kBf16>(__uint_as_float(v[q * 8 + 0]) * scale, __uint_as_float(v[q * 8 + 1]) * scale);
              w.y = pack_pair<kBf16>(__uint_as_float(v[q * 8 + 2]) * scale, __uint_as_float(v[q * 8 + 3]) * scale);
              w.z = pack_pair<kBf16>(__uint_as_float(v[q * 8 + 4]) * scale, __uint_as_float(v[q * 8 + 5]) * scale);
              w.w = pack_pair<kBf16>(__uint_as_float(v[q * 8 + 6]) * scale, __uint_as_float(v[q * 8 + 7]) * scale);
              dst[c * 4 + q] = w;
            }
          }
        }
      }
    }
    if (kWithDq && lane == 0) bulk_wait_group_all();  // shared memory stays valid until the reductions have read it
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kBwdMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// dS[query][kv] = P * (dP - delta) for 64 KV columns of one query row, from the scores and dP in registers; written
// rounded to shared memory (one atom of the A operand of dQ += dS K). kMasked: diagonal and ragged blocks.
template <bool kMasked, bool kBf16>
__device__ __forceinline__ void bwd_row_ds(const uint32_t (&sv)[64], const uint32_t (&dp)[64], float qk_scale, float m_row,
                                           float delta_row, int kv0, int qrow, int n_ctx, int causal, uint32_t ds_row,
                                           int row_xor) {
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    float e[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = g * 8 + u;
      float pv = fast_exp2(fmaf(__uint_as_float(sv[c]), qk_scale, -m_row));
      if (kMasked) {
        const int kvc = kv0 + c;
        const bool valid = kvc < n_ctx && qrow < n_ctx && (!causal || qrow >= kvc);
        pv = valid ? pv : 0.f;
      }
      e[u] = pv * (__uint_as_float(dp[c]) - delta_row);
    }
    st_shared_v4(ds_row + ((g ^ row_xor) << 4), pack_pair<kBf16>(e[0], e[1]), pack_pair<kBf16>(e[2], e[3]),
                 pack_pair<kBf16>(e[4], e[5]), pack_pair<kBf16>(e[6], e[7]));
  }
}

// ---------------------------------------------------------------------------------------------------------------
// dQ for head_dim 128 (reference _attn_bwd_dq, :404-448): one CTA per query block of 128 rows walks the KV blocks it
// sees. S = Q K^T and dP = dO V^T in tensor memory, dS = P * (dP - delta) with the row's own M and delta, written to
// shared memory as the A operand of dQ += dS K (K read MN-major from the tile that S used K-major).
// ---------------------------------------------------------------------------------------------------------------
struct AttnBwdDqParams {
  CUtensorMap tmap_q, tmap_k, tmap_v, tmap_do;  // 3-D {128, n_ctx, batch*heads}, box {64, 128, 1}, SWIZZLE_128B
  const float *m, *delta;
  void *dq;
  uint32_t *status;
  unsigned long long wait_limit_ns;
  float qk_scale, sm_scale;
  int32_t n_ctx, heads_total, q_blocks, causal;
  uint32_t idesc_s;    // 128 x 128, A and B K-major
  uint32_t idesc_dq;   // 128 x 128, A K-major, B MN-major
};

struct AttnBwdDqCtl {
  uint64_t q_full, full[2], empty[2], sdp_full, sdp_free, ds_full, done;
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

template <bool kBf16>
__global__ void __launch_bounds__(kBwdThreads, 1) attn_bwd_dq_kernel(const __grid_constant__ AttnBwdDqParams p) {
  constexpr int kD = 128;
  constexpr int kStg = 2;
  constexpr uint32_t kTile = kTileRows * kD * 2;  // 32 KB, two atoms
  extern __shared__ uint8_t attn_bwd_smem_raw[];
  const uint32_t raw = smem_u32(attn_bwd_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t q_addr = base, do_addr = base + kTile;
  const uint32_t ring_addr = base + 2 * kTile;        // per stage: K tile, V tile
  const uint32_t ds_addr = ring_addr + kStg * 2 * kTile;  // dS [128 queries][128 KV], 2 atoms
  AttnBwdDqCtl *ctl = reinterpret_cast<AttnBwdDqCtl *>(attn_bwd_smem_raw + (ds_addr + kPBytes - raw));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // late (heavy, when causal) query blocks first inside a head
  const int head = static_cast<int>(blockIdx.x) / p.q_blocks;
  const int i = p.q_blocks - 1 - static_cast<int>(blockIdx.x) % p.q_blocks;
  const int q0 = i * kTileRows;
  const int kv_blocks = (p.n_ctx + kTileRows - 1) / kTileRows;
  const int n_it = p.causal ? min(kv_blocks, i + 1) : kv_blocks;

  AbortCtl ac;
  ac.flag = &ctl->abort_flag;
  ac.status = p.status;
  ac.limit_ns = p.wait_limit_ns;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&ctl->q_full), 1);
    for (int s = 0; s < kStg; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    mbar_init(smem_u32(&ctl->sdp_full), 1);
    mbar_init(smem_u32(&ctl->sdp_free), 2 * kTileRows);
    mbar_init(smem_u32(&ctl->ds_full), 2 * kTileRows);
    mbar_init(smem_u32(&ctl->done), 1);
    ctl->abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.tmap_q);
    tma_prefetch_desc(&p.tmap_k);
    tma_prefetch_desc(&p.tmap_v);
    tma_prefetch_desc(&p.tmap_do);
  }
  if (warp == kBwdMmaWarp) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  constexpr uint32_t kColS = 0, kColDp = 128, kColDq = 256;

  if (warp == kBwdProducerWarp) {
    const bool issuer = elect_one();
    if (issuer) {
      const uint32_t bar = smem_u32(&ctl->q_full);
      mbar_arrive_expect_tx(bar, 2 * kTile);
      for (int a = 0; a < 2; ++a) {
        tma_load_3d(q_addr + a * kAtomBytes, &p.tmap_q, a * 64, q0, head, bar);
        tma_load_3d(do_addr + a * kAtomBytes, &p.tmap_do, a * 64, q0, head, bar);
      }
    }
    __syncwarp();
    int issued = 0;
    for (int it = 0; it < n_it; ++it) {
      const int slot = it % kStg;
      const uint32_t phase = static_cast<uint32_t>(it / kStg) & 1u;
      if (!warp_mbar_poll(smem_u32(&ctl->empty[slot]), phase ^ 1u, ac, kAttnTimeoutProducer, lane)) break;
      if (issuer) {
        const uint32_t bar = smem_u32(&ctl->full[slot]);
        mbar_arrive_expect_tx(bar, 2 * kTile);
        for (int a = 0; a < 2; ++a) {
          tma_load_3d(ring_addr + slot * 2 * kTile + a * kAtomBytes, &p.tmap_k, a * 64, it * kTileRows, head, bar);
          tma_load_3d(ring_addr + slot * 2 * kTile + kTile + a * kAtomBytes, &p.tmap_v, a * 64, it * kTileRows, head, bar);
        }
      }
      __syncwarp();
      ++issued;
    }
    if (ctl->abort_flag) {
      if (lane == 0) {
        mbar_wait_timed(smem_u32(&ctl->q_full), 0u, ac, kAttnTimeoutDrain);
        const int first = issued > kStg ? issued - kStg : 0;
        for (int it = first; it < issued; ++it) {
          const unsigned long long t0 = global_timer_ns();
          const uint32_t bar = smem_u32(&ctl->full[it % kStg]);
          const uint32_t ph = static_cast<uint32_t>(it / kStg) & 1u;
          while (!mbar_try_wait(bar, ph))
            if (global_timer_ns() - t0 > ac.limit_ns) break;
        }
      }
      __syncwarp();
    }
  } else if (warp == kBwdMmaWarp) {
    const bool issuer = elect_one();
    auto desc64 = [](uint32_t hi, uint32_t lo) { return (static_cast<uint64_t>(hi) << 32) | lo; };
    const uint32_t desc_hi = ((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
    const uint32_t lbo_unused = 1u << 16;
    const uint32_t lbo_atom = ((static_cast<uint32_t>(kAtomBytes) >> 4) & 0x3FFFu) << 16;
    auto lo_of = [](uint32_t addr) { return (addr & 0x3FFFFu) >> 4; };
    auto kmajor_step = [](int s) { return static_cast<uint32_t>(s >> 2) * (kAtomBytes >> 4) + static_cast<uint32_t>(s & 3) * 2u; };
    auto mn_step = [](int s) { return static_cast<uint32_t>(s) * (16u * 128u >> 4); };
    auto issue_sdp = [&](int it) {  // S = Q K^T, dP = dO V^T
      const uint32_t k_addr = ring_addr + static_cast<uint32_t>(it % kStg) * 2 * kTile, v_addr = k_addr + kTile;
#pragma unroll
      for (int s = 0; s < kD / 16; ++s)
        if (issuer)
          umma_f16(tmem_base + kColS, desc64(desc_hi, (lo_of(q_addr) | lbo_unused) + kmajor_step(s)),
                   desc64(desc_hi, (lo_of(k_addr) | lbo_unused) + kmajor_step(s)), p.idesc_s, s > 0 ? 1u : 0u);
#pragma unroll
      for (int s = 0; s < kD / 16; ++s)
        if (issuer)
          umma_f16(tmem_base + kColDp, desc64(desc_hi, (lo_of(do_addr) | lbo_unused) + kmajor_step(s)),
                   desc64(desc_hi, (lo_of(v_addr) | lbo_unused) + kmajor_step(s)), p.idesc_s, s > 0 ? 1u : 0u);
      if (issuer) tc_commit(smem_u32(&ctl->sdp_full));
      __syncwarp();
    };
    auto wait_stage = [&](int it) {
      return warp_mbar_poll(smem_u32(&ctl->full[it % kStg]), static_cast<uint32_t>(it / kStg) & 1u, ac, kAttnTimeoutMmaOperand,
                            lane);
    };
    bool ok = warp_mbar_poll(smem_u32(&ctl->q_full), 0u, ac, kAttnTimeoutMmaOperand, lane);
    if (ok && n_it > 0) ok = wait_stage(0);
    if (ok && n_it > 0) {
      tc_fence_after();
      issue_sdp(0);
    }
    for (int it = 0; ok && it < n_it; ++it) {
      const uint32_t k_addr = ring_addr + static_cast<uint32_t>(it % kStg) * 2 * kTile;
      // the next block's S and dP as soon as this block's are in the compute warps' registers: the tensor pipe works
      // on them while the compute warps turn this block into dS
      if (it + 1 < n_it) {
        if (!wait_stage(it + 1)) break;
        if (!warp_mbar_poll(smem_u32(&ctl->sdp_free), static_cast<uint32_t>(it) & 1u, ac, kAttnTimeoutMmaP, lane)) break;
        tc_fence_after();
        issue_sdp(it + 1);
      }
      if (!warp_mbar_poll(smem_u32(&ctl->ds_full), static_cast<uint32_t>(it) & 1u, ac, kAttnTimeoutMmaP, lane)) break;
      tc_fence_after();
#pragma unroll
      for (int s = 0; s < 8; ++s)  // dQ += dS K : 128 x 128 x 16 each
        if (issuer)
          umma_f16(tmem_base + kColDq, desc64(desc_hi, (lo_of(ds_addr) | lbo_unused) + kmajor_step(s)),
                   desc64(desc_hi, (lo_of(k_addr) | lbo_atom) + mn_step(s)), p.idesc_dq, (it > 0 || s > 0) ? 1u : 0u);
      if (issuer) tc_commit(smem_u32(&ctl->empty[it % kStg]));
      __syncwarp();
    }
    if (issuer) tc_commit(smem_u32(&ctl->done));
    __syncwarp();
    if (lane == 0) {
      const unsigned long long t0 = global_timer_ns();
      while (!mbar_try_wait(smem_u32(&ctl->done), 0u)) {
        if (global_timer_ns() - t0 > ac.limit_ns) {
          ctl->abort_flag = 1;
          atomicCAS(ac.status, 0u, static_cast<uint32_t>(kAttnTimeoutDrain));
          break;
        }
      }
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    const int half = warp >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t row_off = static_cast<uint32_t>(half * kAtomBytes + (r >> 3) * 1024 + (r & 7) * 128);
    const int row_xor = r & 7;
    const int qrow = q0 + r;
    const long long grow = static_cast<long long>(head) * p.n_ctx + qrow;
    const float m_row = qrow < p.n_ctx ? p.m[grow] : 0.f;
    const float delta_row = qrow < p.n_ctx ? p.delta[grow] : 0.f;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      if (!warp_mbar_poll(smem_u32(&ctl->sdp_full), static_cast<uint32_t>(it) & 1u, ac, kAttnTimeoutSoftmaxS, lane)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int c0 = it * kTileRows + half * 64;
      const bool masked = (p.causal && it == i) || (it + 1) * kTileRows > p.n_ctx || q0 + kTileRows > p.n_ctx;
      uint32_t sall[64], dpall[64];
      tmem_ld_32x32(lane_base + kColS + half * 64, *reinterpret_cast<uint32_t(*)[32]>(&sall[0]));
      tmem_ld_32x32(lane_base + kColS + half * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&sall[32]));
      tmem_ld_32x32(lane_base + kColDp + half * 64, *reinterpret_cast<uint32_t(*)[32]>(&dpall[0]));
      tmem_ld_32x32(lane_base + kColDp + half * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&dpall[32]));
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(smem_u32(&ctl->sdp_free));
      // dQ += dS K of the previous block is queued behind this block's S and dP: its commit (the ring slot's
      // "empty" barrier) says when the dS buffer may be overwritten
      if (it > 0 && !warp_mbar_poll(smem_u32(&ctl->empty[(it - 1) % kStg]), static_cast<uint32_t>((it - 1) / kStg) & 1u, ac,
                                    kAttnTimeoutSoftmaxO, lane)) {
        ok = false;
        break;
      }
      if (masked) bwd_row_ds<true, kBf16>(sall, dpall, p.qk_scale, m_row, delta_row, c0, qrow, p.n_ctx, p.causal, ds_addr + row_off, row_xor);
      else bwd_row_ds<false, kBf16>(sall, dpall, p.qk_scale, m_row, delta_row, c0, qrow, p.n_ctx, p.causal, ds_addr + row_off, row_xor);
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(smem_u32(&ctl->ds_full));
    }
    if (ok && n_it > 0) ok = warp_mbar_poll(smem_u32(&ctl->done), 0u, ac, kAttnTimeoutSoftmaxO, lane);
    if (ok && n_it > 0) {
      tc_fence_after();
      uint4 *dst = reinterpret_cast<uint4 *>(static_cast<char *>(p.dq) + (grow * kD + half * 64) * 2);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(lane_base + kColDq + half * 64 + c * 32, v);
        tmem_ld_wait();
        if (qrow < p.n_ctx) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 w;
            w.x = pack_pair<kBf16>(__uint_as_float(v[q * 8 + 0]) * p.sm_scale, __uint_as_float(v[q * 8 + 1]) * p.sm_scale);
            w.y = pack_pair<kBf16>(__uint_as_float(v[q * 8 + 2]) * p.sm_scale, __uint_as_float(v[q * 8 + 3]) * p.sm_scale);
            w.z = pack_pair<kBf16>(__uint_as_float(v[q * 8 + 4]) * p.sm_scale, __uint_as_float(v[q * 8 + 5]) * p.sm_scale);
            w.w = pack_pair<kBf16>(__uint_as_float(v[q * 8 + 6]) * p.sm_scale, __uint_as_float(v[q * 8 + 7]) * p.sm_scale);
            dst[c * 4 + q] = w;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kBwdMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace txa
