// Arithmetic-intensity model that picks tile shape, pipeline depth, operand roles and schedule for one
// tt.dot K-loop on a B200. Pure host C++ (no CUDA): shared by the `dot_tile_select` pass extension and
// by the `b200_dot` backend's plan creation, so both always agree.
//
// The reference has no counterpart: its only analysis is LoopSplit's compare scan
// (pass/LoopSplit/LoopSplit.cpp:107-123). The quantities modelled here are the ones that decide a
// tcgen05 kernel's speed: tensor-pipe cycles per K block, shared-memory feed bytes per K block, wave
// quantisation of the persistent grid, and HBM bytes.
#pragma once

#include <algorithm>
#include <cstdint>
#include <cstring>

#include "b200_dot.h"

namespace txd {

struct MachineModel {
  int sm_count = 148;
  double sm_clock_ghz = 1.9;            // tensor work runs power-capped; only ratios matter here
  double mma_flops_per_clk_16bit = 8192;  // dense bf16/fp16 FLOP per SM per clock
  double mma_flops_per_clk_8bit = 16384;
  double smem_bytes_per_clk = 128;      // shared-memory read bandwidth per SM
  double ingest_bytes_per_clk = 60;     // what TMA can deliver into one SM's shared memory (measured:
                                        // a loads-only run of the ring moved 56 B/clk/SM)
  double hbm_bytes_per_s = 6.4596e12;   // measured copy bandwidth of this pool's B200
  double block_overhead_clk = 0;        // per K block handshake cost not hidden behind the MMAs (measured: none)
  double hbm_bytes_per_s_per_cta = 60e9; // what one persistent CTA's TMA ring sustains from HBM
  double tma_issue_ns = 90;             // time one TMA copy occupies the thread that issues it
  double stage_issue_ns = 60;           // per-stage cost of a producer warp besides the copies
  int smem_budget = 227 * 1024 - 2048;  // dynamic shared memory per CTA minus control block + slack
};

inline int elem_bytes(int dtype) {
  switch (dtype) {
    case TXD_F16:
    case TXD_BF16:
      return 2;
    case TXD_F8E4M3:
    case TXD_F8E5M2:
      return 1;
    case TXD_F32:
      return 4;
    default:
      return 0;
  }
}

struct TileChoice {
  int block_m = 128, block_n = 0, block_k = 0;
  int mma_n = 0;         // N extent of one tcgen05.mma: block_n, or 256 for the 512-column wide pair tile
  int stages = 0;
  int swap_ab = 0;       // 0/1 (resolved)
  int cta_pair = 0;      // 0/1 (resolved): two-CTA clusters, 256-row tiles
  int atoms = 1;         // 128-byte K atoms per stage (block_k = atoms * 128 / element size)
  int tma_store = 0;     // epilogue goes through shared memory + TMA store
  int schedule = 0;      // TXD_SCHED_DATA_PARALLEL, TXD_SCHED_STREAM_K or TXD_SCHED_HYBRID (resolved)
  int sk_first_tile = 0; // first tile of the stream-K region (0 for pure stream-K)
  int group_m = 0;
  int grid = 0;
  int k_blocks = 0, k_main_blocks = 0, tail_mmas = 0;
  int p_extent = 0, q_extent = 0;   // MMA-M side and MMA-N side extents after role assignment
  int tiles_p = 0, tiles_q = 0;
  int p_stage_bytes = 0, q_stage_bytes = 0;
  int smem_bytes = 0, tmem_cols = 0;
  int64_t scratch_bytes = 0;
  double arithmetic_intensity = 0;  // FLOP per algorithmic byte
  double ridge_intensity = 0;       // machine balance: FLOP per byte at which HBM and tensor time meet
  double est_seconds = 0;
  bool hbm_bound = false;
};

inline int round_up(int x, int m) { return (x + m - 1) / m * m; }
inline int cdiv(int x, int m) { return (x + m - 1) / m; }

inline double algorithmic_bytes(const tx_dot_problem &pr) {
  const double es = elem_bytes(pr.ab_dtype), os = elem_bytes(pr.out_dtype);
  double b = (double)pr.m * pr.k * es + (double)pr.k * pr.n * es + (double)pr.m * pr.n * os;
  if (pr.has_row_scale) b += 4.0 * pr.m;
  if (pr.has_col_scale) b += 4.0 * pr.n;
  return b;
}

// Modelled time of one (role assignment, block_n, pairing, schedule) candidate.
inline double model_seconds(const MachineModel &mm, int es, int p_extent, int q_extent, int k,
                            int block_n, bool p_mn_major, bool q_mn_major, bool pair, int atoms, int schedule,
                            int workers, double algo_bytes) {
  const int bk_atom = 128 / es;
  const int bk = atoms * bk_atom;
  const int k_blocks = cdiv(k, bk);
  const int tile_rows = pair ? 256 : 128;
  const int tiles = cdiv(p_extent, tile_rows) * cdiv(q_extent, block_n);
  const double flops_per_clk = es == 1 ? mm.mma_flops_per_clk_8bit : mm.mma_flops_per_clk_16bit;
  // Per SM and K block: a 128 x block_n x bk MMA either way (a pair splits a 256-row tile).
  const double mma_clk = 2.0 * 128 * block_n * bk / flops_per_clk;
  const int q_rows_cta = pair ? block_n / 2 : block_n;
  const int q_rows = q_mn_major ? round_up(q_rows_cta, bk_atom) : q_rows_cta;  // MN-major boxes are 128 B wide
  const double stage_bytes = atoms * (128.0 * 128 + q_rows * 128.0);
  // The tensor pipe reads every stage byte once (a pair reads the peer's Q half as well) ...
  const double read_clk = atoms * (128.0 * 128 + (pair ? 2 : 1) * q_rows * 128.0) / mm.smem_bytes_per_clk;
  // ... and TMA has to deliver the CTA's own stage bytes.
  const double ingest_clk = stage_bytes / mm.ingest_bytes_per_clk;
  const double blk_clk = std::max(mma_clk, std::max(read_clk, ingest_clk)) + mm.block_overhead_clk;
  const long long total = (long long)tiles * k_blocks;
  double blocks_per_worker;  // the busiest worker's share
  if (schedule == TXD_SCHED_STREAM_K) {
    blocks_per_worker = (double)((total + workers - 1) / workers);
  } else if (schedule == TXD_SCHED_HYBRID) {
    const long long dp_tiles = (long long)(tiles / workers) * workers;
    blocks_per_worker = (double)(dp_tiles / workers) * k_blocks +
                        (double)(((long long)(tiles - dp_tiles) * k_blocks + workers - 1) / workers);
  } else {
    blocks_per_worker = (double)cdiv(tiles, workers) * k_blocks;
  }
  const double balance = ((double)total / workers) / blocks_per_worker;  // 1 = equally loaded
  double busy_clk = blocks_per_worker * blk_clk;
  if (schedule != TXD_SCHED_DATA_PARALLEL) {
    // Up to two partial tiles per CTA go through scratch: fp32 write + read, ~64 B/clk through L2.
    busy_clk += 2.0 * (128.0 * block_n * 4 * 2) / 64.0;
  }
  // The last tile's epilogue is not hidden behind a main loop.
  busy_clk += 128.0 * block_n * 4 / 64.0;
  const double t_tensor = busy_clk / (mm.sm_clock_ghz * 1e9);
  // A CTA keeps only its own ring of loads in flight, so few CTAs cannot pull the whole HBM rate,
  // and an unbalanced grid leaves HBM idle while the last CTAs finish.
  const int ctas = pair ? 2 * workers : workers;
  const double t_hbm =
      algo_bytes / std::min(mm.hbm_bytes_per_s, ctas * mm.hbm_bytes_per_s_per_cta) / balance;
  // One warp per operand issues the stage's TMA copies: K-major operands take one copy per atom,
  // MN-major operands one per 128-byte-wide chunk of rows.
  const int p_copies = p_mn_major ? 128 / bk_atom : atoms;
  const int q_copies = q_mn_major ? cdiv(q_rows_cta, bk_atom) : atoms;
  const double t_issue = blocks_per_worker * (mm.stage_issue_ns + mm.tma_issue_ns * std::max(p_copies, q_copies)) * 1e-9;
  return std::max(std::max(t_tensor, t_hbm), t_issue) + 3e-6;  // + launch and pipeline fill
}

// Fill every unset field of `cfg`. Returns 0, or a negative value with *why set.
inline int select_tiles(const tx_dot_problem &pr, const tx_dot_config *cfg_in, const MachineModel &mm,
                        TileChoice &out, const char **why) {
  static const char *kNoWhy = "";
  if (why) *why = kNoWhy;
  tx_dot_config cfg = {};
  if (cfg_in) cfg = *cfg_in;
  const int es = elem_bytes(pr.ab_dtype);
  if (es != 1 && es != 2) {
    if (why) *why = "operand dtype must be f16, bf16, f8e4m3 or f8e5m2";
    return -1;
  }
  const int bk = 128 / es;
  const double algo = algorithmic_bytes(pr);
  const double flops = 2.0 * pr.m * pr.n * pr.k;
  const double flops_per_clk = es == 1 ? mm.mma_flops_per_clk_8bit : mm.mma_flops_per_clk_16bit;
  out.arithmetic_intensity = flops / algo;
  out.ridge_intensity = flops_per_clk * mm.sm_count * mm.sm_clock_ghz * 1e9 / mm.hbm_bytes_per_s;
  out.hbm_bound = out.arithmetic_intensity < out.ridge_intensity;
  const int max_grid = cfg.max_ctas > 0 ? std::min(cfg.max_ctas, mm.sm_count) : mm.sm_count;

  double best = 1e30;
  bool found = false;
  static const int kBlockNs[] = {512, 256, 128, 64, 32, 16};
  for (int swap = 0; swap <= 1; ++swap) {
    if (cfg.swap_ab == 1 && !swap) continue;
    if (cfg.swap_ab == 2 && swap) continue;
    // Swapping only pays when m is the short side; do not consider it otherwise.
    if (cfg.swap_ab == 0 && swap && !(pr.m < 128 && pr.n > pr.m)) continue;
    const int p_extent = swap ? pr.n : pr.m;
    const int q_extent = swap ? pr.m : pr.n;
    // Q is MN-major when its rows (the Q index) are contiguous in memory.
    const bool q_mn = swap ? (pr.a_layout == TXD_COL_MAJOR) : (pr.b_layout == TXD_ROW_MAJOR);
    const bool p_mn_c = swap ? (pr.b_layout == TXD_ROW_MAJOR) : (pr.a_layout == TXD_COL_MAJOR);
    for (int bn : kBlockNs) {
      if (cfg.block_n && bn != cfg.block_n) continue;
      // Do not pad the Q side by more than one tile's worth beyond need.
      if (!cfg.block_n && bn > 16 && bn / 2 >= q_extent) continue;
      for (int pair = 0; pair <= 1; ++pair) {
        if (cfg.cta_pair == 1 && !pair) continue;
        if (cfg.cta_pair == 2 && pair) continue;
        // 512 columns = the wide pair tile: two 256-column MMA halves per K block sharing one P stage.
        if (bn == 512 && !pair) continue;
        // Unasked, the wide tile is taken only where it was measured to win: tensor-bound problems that it tiles
        // without padding and in no more machine time than 256-column tiles do (one wave of wide tiles lasts two
        // waves of narrow ones). There it runs 2.4 % faster (4096 x 4096 x 4160, 8192^3); half a narrow wave of extra
        // quantisation (the column panels of a sharded GEMM) costs it that gain.
        bool wide_auto = false;
        if (bn == 512 && cfg.block_n != 512) {
          if (cfg.atoms > 1 || (cfg.schedule && cfg.schedule != TXD_SCHED_DATA_PARALLEL)) continue;
          if (es != 2) continue;  // 8-bit operands: measured slower than 256-column tiles with two atoms per stage (8192^3 e4m3)
          if (out.hbm_bound || q_extent % 512 != 0 || p_extent % 256 != 0) continue;
          const int pairs = max_grid / 2;
          if (pairs < 1) continue;
          const int tiles_w = (p_extent / 256) * (q_extent / 512), tiles_n = 2 * tiles_w;
          const int waves_w = cdiv(tiles_w, std::min(pairs, tiles_w)), waves_n = cdiv(tiles_n, std::min(pairs, tiles_n));
          if (2 * waves_w > waves_n) continue;
          wide_auto = true;
        }
        const int mma_n = bn == 512 ? 256 : bn;
        if (pair) {
          // Each CTA of a pair holds half of the Q tile, in whole 128-byte-wide boxes when Q is
          // MN-major; pairs are for big problems in the natural orientation only.
          if (swap || bn < 128 || (q_mn && (mma_n / 2) % bk != 0)) continue;
          if (cfg.cta_pair == 0 && p_extent < 512) continue;
        }
        for (int atoms = 1; atoms <= 4; atoms *= 2) {
        if (cfg.atoms && atoms != cfg.atoms) continue;
        if (bn == 512 && atoms != 1) continue;  // a wide stage is 48 KiB; deeper blocks leave too few stages
        // An MN-major operand is loaded as boxes atoms*bk K-slices tall; a TMA box dimension is at most 256.
        if ((p_mn_c || q_mn) && atoms * bk > 256) continue;
        {
          // Two atoms per stage halve the per-block handshakes but also the ring depth: keep >= 3 stages.
          const int q_rows_cta = pair ? bn / 2 : bn;
          const int stage = atoms * (128 * 128 + round_up((q_mn ? round_up(q_rows_cta, bk) : q_rows_cta) * 128, 1024));
          const int staging = (!swap && bn >= 64) ? 4 * 2 * 32 * 128 /* two 4 KiB staging slabs per epilogue warp */ : 0;
          if (atoms >= 2 && (mm.smem_budget - staging) / stage < 3) continue;
          if (atoms >= 2 && pr.k < 4 * atoms * bk) continue;
        }
        const int tiles = cdiv(p_extent, pair ? 256 : 128) * cdiv(q_extent, bn);
        const int k_blocks = cdiv(pr.k, bk * atoms);
        for (int sched = TXD_SCHED_DATA_PARALLEL; sched <= TXD_SCHED_HYBRID; ++sched) {
          if (cfg.schedule && sched != cfg.schedule) continue;
          if (bn == 512 && sched != TXD_SCHED_DATA_PARALLEL) continue;  // both accumulators belong to one tile
          long long units = (long long)tiles * (sched == TXD_SCHED_STREAM_K ? k_blocks : 1);
          if (units < 1) units = 1;
          const int max_workers = pair ? max_grid / 2 : max_grid;
          if (max_workers < 1) continue;
          int workers = (int)std::min<long long>(max_workers, units);
          // HBM-bound whole tiles: as many workers as give every one the same number of tiles. A worker streams at its
          // own SM's rate, so a last round in which half of them have no tile left runs at half the bandwidth
          // (bf16 16 x 28672 x 8192, 224 tiles: 148 workers 77.8 us, 112 workers 71.8 us). Tensor-bound shapes measured
          // no better with the smaller grid (4096 x 4096 x 4160: 110 against 99.5 us), so they keep every SM.
          if (out.hbm_bound && sched == TXD_SCHED_DATA_PARALLEL && tiles > workers)
            workers = cdiv(tiles, cdiv(tiles, workers));
          if (sched == TXD_SCHED_HYBRID) {
            // Needs at least one full wave, a partial last wave, and a K block for every worker in it.
            const int tail = tiles % workers;
            if (tiles < workers || tail == 0 || (long long)tail * k_blocks < workers) continue;
          }
          double t = model_seconds(mm, es, p_extent, q_extent, pr.k, bn, p_mn_c, q_mn, pair != 0, atoms, sched, workers, algo);
          if (wide_auto)  // priced from the measurement: the two-atom 256-column tile's time, less 2.4 %
            t = model_seconds(mm, es, p_extent, q_extent, pr.k, 256, p_mn_c, q_mn, true, 2, sched, std::min(max_workers, 2 * tiles), algo) * 0.93 * 0.976;
          // Prefer the simpler schedule on near-ties, and the role assignment that pads less: zero
          // rows still cost shared-memory fill and tensor cycles even when HBM time hides them.
          // Pure stream-K also spreads concurrently running tiles over the whole matrix (worse L2 reuse).
          // K-block depth: tensor-bound problems ran fastest with one atom per stage (deepest ring);
          // HBM-bound ones with deep blocks (fewer TMA copies and handshakes per byte). Both measured.
          {
            int lg = atoms == 4 ? 2 : (atoms == 2 ? 1 : 0);
            // Measured (8192 x 8192 x 4160 bf16, CTA pairs): one atom per stage is bound by the load path at 690
            // cycles per K block of four MMAs (512 of tensor work), two atoms per stage run at 1 100 cycles per
            // eight MMAs: bigger TMA boxes and half the barrier traffic per byte. Deeper still leaves too few stages.
            t *= out.hbm_bound ? 1.0 - (lg >= 1 ? 0.02 : 0.0) + (lg == 2 ? 0.005 : 0.0) : (lg == 1 ? 0.93 : (lg == 2 ? 1.04 : 1.0));
          }
          if (sched == TXD_SCHED_STREAM_K) t = t * 1.10 + 6e-6;  // + fix-up of the partial tiles (measured on 16x14336x4096)
          // Measured on 4096x4096x4160 (3.46 waves): the partial-tile fix-up of the last wave costs more than
          // the idle SMs it saves, so whole tiles win unless the partial wave is nearly empty.
          if (sched == TXD_SCHED_HYBRID) t *= 1.20;
          const double tile_rows = pair ? 256.0 : 128.0;
          const double padded = (double)cdiv(p_extent, (int)tile_rows) * tile_rows * cdiv(q_extent, bn) * bn;
          t *= 1.0 + 0.25 * (1.0 - (double)p_extent * q_extent / padded);
          if (t < best) {
            best = t;
            found = true;
            out.swap_ab = swap;
            out.block_n = bn;
            out.mma_n = mma_n;
            out.cta_pair = pair;
            out.atoms = atoms;
            out.schedule = sched;
            out.grid = pair ? 2 * workers : workers;
          }
        }
        }
      }
    }
  }
  if (!found) {
    if (why) *why = "no tile configuration satisfies the given constraints";
    return -1;
  }
  out.est_seconds = best;
  const int bks = bk * out.atoms;  // K elements per stage (the kernels' physical K block)
  out.block_k = bks;
  out.p_extent = out.swap_ab ? pr.n : pr.m;
  out.q_extent = out.swap_ab ? pr.m : pr.n;
  out.block_m = out.cta_pair ? 256 : 128;
  out.tiles_p = cdiv(out.p_extent, out.block_m);
  out.tiles_q = cdiv(out.q_extent, out.block_n);
  out.k_blocks = cdiv(pr.k, bks);
  // LoopSplit mid point: first K index of the masked remainder.
  int mid = cfg.k_split_point > 0 ? cfg.k_split_point : (cfg.k_split_point < 0 ? 0 : (pr.k / bks) * bks);
  if (mid > (pr.k / bk) * bk || mid < 0) {
    if (why) *why = "k_split_point lies past the last full K block: a partial block would run unmasked";
    return -1;
  }
  mid = (mid / bks) * bks;  // a split inside a physical block moves down: the remainder only adds masking
  out.k_main_blocks = mid / bks;
  const int rem = pr.k - (out.k_blocks - 1) * bks;  // columns in the last block: 1..bks
  const int umma_k = 32 / es;
  out.tail_mmas = pr.k > 0 ? cdiv(rem, umma_k) : 0;
  const bool p_mn = out.swap_ab ? (pr.b_layout == TXD_ROW_MAJOR) : (pr.a_layout == TXD_COL_MAJOR);
  const bool q_mn = out.swap_ab ? (pr.a_layout == TXD_COL_MAJOR) : (pr.b_layout == TXD_ROW_MAJOR);
  (void)p_mn;
  out.p_stage_bytes = out.atoms * 128 * 128;
  const int q_rows_cta = out.cta_pair ? out.block_n / 2 : out.block_n;
  // The Q stage must keep the next P stage 1024-byte aligned.
  out.q_stage_bytes = out.atoms * round_up((q_mn ? round_up(q_rows_cta, bk) : q_rows_cta) * 128, 1024);
  const int stage_bytes = out.p_stage_bytes + out.q_stage_bytes;
  // C goes out through a shared-memory slab + TMA store when its rows are 16-byte aligned.
  const int os = elem_bytes(pr.out_dtype);
  out.tma_store = (!out.swap_ab && out.block_n >= 64 && (pr.ldc * os) % 16 == 0) ? 1 : 0;  // whole 128-byte slabs
  const int staging = out.tma_store ? 4 * 2 * 32 * 128 /* two 4 KiB staging slabs per epilogue warp */ : 0;
  int stages = cfg.stages ? cfg.stages : std::min(12, (mm.smem_budget - staging) / stage_bytes);
  // A ring above 200 KiB was measured slower than one stage less (bf16 16 x 14336 x 4096, 36 KiB stages: six stages
  // 23.1 us, five and four 22.1 us; 16 x 4096 x 14336: 30.5 against 30.2 us), while rings of 192-200 KiB are the best of
  // their shapes (five 40 KiB stages at m = 32 and m = 64, three 64 KiB stages for the tensor-bound pairs).
  if (!cfg.stages)
    while (stages > 3 && stages * stage_bytes > 200 * 1024) --stages;
  if (stages < 2 || stages > 12 || stages * stage_bytes + staging > mm.smem_budget) {
    if (why) *why = "stages out of range for this tile (2..12, ring must fit shared memory)";
    return -1;
  }
  out.stages = stages;
  out.smem_bytes = stages * stage_bytes + staging + 1024 /*alignment slack*/ + 512 /*control block*/;
  int cols = 32;
  while (cols < 2 * out.block_n) cols *= 2;
  if (out.cta_pair) cols = 512;  // both CTAs of a pair must get the same (whole) allocation
  out.tmem_cols = cols;
  if (cfg.group_m > 0) {
    out.group_m = cfg.group_m;
  } else {
    // Shape one wave of tiles as close to square (in elements) as the grid allows.
    int g = 1;
    double best_g = 1e30;
    for (int cand = 1; cand <= 32; cand *= 2) {
      const double rows = cand * (double)out.block_m, cols_e = (double)(out.cta_pair ? out.grid / 2 : out.grid) / cand * out.block_n;
      const double cost = rows + cols_e;
      if (cost < best_g) {
        best_g = cost;
        g = cand;
      }
    }
    // A group's P panels (group_m x block_m rows x K) are what consecutive waves read again while Q panels stream past
    // once per group, so a taller group means fewer passes over Q from DRAM, as long as its panels stay in L2 under
    // that stream: twice the height when the group then still holds at most 32 MiB (measured on fp8 8192^3: 16 tile rows
    // instead of 8 read 240 MB instead of 342 MB and ran 2 % faster; 32 rows, 64 MiB, read 651 MB; on bf16
    // 16384 x 28672 x 8192, where 8 rows already hold 32 MiB, 16 rows were slower and read more).
    const double panel_bytes = (double)out.block_m * pr.k * es;
    if (2 * g <= 32 && 2.0 * g * panel_bytes <= 32.0 * 1024 * 1024) g *= 2;
    out.group_m = std::max(1, std::min(g, out.tiles_p));
  }
  out.scratch_bytes = 0;
  out.sk_first_tile = 0;
  if (out.schedule != TXD_SCHED_DATA_PARALLEL) {
    // Two partial-tile slots (128 rows x block_n fp32) per CTA, one counter per (tile, CTA of the pair).
    const int ranks = out.cta_pair ? 2 : 1;
    const int workers = out.grid / ranks;
    const int tiles = out.tiles_p * out.tiles_q;
    if (out.schedule == TXD_SCHED_HYBRID) out.sk_first_tile = (tiles / workers) * workers;
    out.scratch_bytes = (int64_t)out.grid * 2 * out.block_n * 128 * 4 + (int64_t)tiles * ranks * 4;
  }
  return 0;
}

inline void fill_plan_info(const tx_dot_problem &pr, const TileChoice &tc, tx_dot_plan_info *info) {
  memset(info, 0, sizeof *info);
  info->block_m = tc.block_m;
  info->block_n = tc.block_n;
  info->block_k = tc.block_k;
  info->stages = tc.stages;
  info->swap_ab = tc.swap_ab;
  info->schedule = tc.schedule;
  info->group_m = tc.group_m;
  info->grid = tc.grid;
  info->k_main_iters = tc.k_main_blocks;
  info->k_tail_iters = tc.k_blocks - tc.k_main_blocks;
  info->k_tail_mmas = tc.tail_mmas;
  info->smem_bytes = tc.smem_bytes;
  info->tmem_columns = tc.tmem_cols;
  info->cta_pair = tc.cta_pair;
  info->scratch_bytes = tc.scratch_bytes;
  info->flops = 2.0 * pr.m * pr.n * pr.k;
  info->algorithmic_bytes = algorithmic_bytes(pr);
}


}  // namespace txd
