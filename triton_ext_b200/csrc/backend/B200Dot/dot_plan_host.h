// Host-side pieces shared by every translation unit that launches dot_umma_body: argument validation,
// the tcgen05 instruction / shared-memory descriptors, the TMA tensor maps and the part of DotParams that
// follows from (problem, tile choice) alone. Include after dot_umma_kernel.cuh.
//
// Functions return a tx_dot_status and write the message into `err`; the including file turns that into
// its own thread-local error text.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "b200_dot.h"
#include "dot_tile_model.h"

namespace txd {
namespace host {

inline int set_error(std::string *err, int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (err) *err = buf;
  return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// What every entry point checks before it looks at a device.
inline int validate_problem(const tx_dot_problem &pr, std::string *err) {
  if (pr.m < 0 || pr.n < 0 || pr.k < 0) return set_error(err, TXD_ERR_INVALID, "negative extent m=%d n=%d k=%d", pr.m, pr.n, pr.k);
  const int es = elem_bytes(pr.ab_dtype);
  if (pr.ab_dtype == TXD_F32 || (es != 1 && es != 2))
    return set_error(err, TXD_ERR_UNSUPPORTED, "operand dtype %d: tt.dot operands must be f16, bf16, f8e4m3 or f8e5m2", pr.ab_dtype);
  if (pr.out_dtype != TXD_F16 && pr.out_dtype != TXD_BF16 && pr.out_dtype != TXD_F32)
    return set_error(err, TXD_ERR_UNSUPPORTED, "output dtype %d: must be f16, bf16 or f32", pr.out_dtype);
  if ((pr.a_layout != TXD_ROW_MAJOR && pr.a_layout != TXD_COL_MAJOR) ||
      (pr.b_layout != TXD_ROW_MAJOR && pr.b_layout != TXD_COL_MAJOR))
    return set_error(err, TXD_ERR_INVALID, "layout must be TXD_ROW_MAJOR or TXD_COL_MAJOR");
  const long long a_min = pr.a_layout == TXD_ROW_MAJOR ? pr.k : pr.m;
  const long long b_min = pr.b_layout == TXD_ROW_MAJOR ? pr.n : pr.k;
  if (pr.lda < a_min || pr.ldb < b_min || pr.ldc < pr.n)
    return set_error(err, TXD_ERR_INVALID, "leading dimension smaller than the row length (lda=%lld ldb=%lld ldc=%lld)",
                     (long long)pr.lda, (long long)pr.ldb, (long long)pr.ldc);
  // TMA: every global stride is a multiple of 16 bytes (no operand is read when an extent is zero).
  const bool empty = pr.m == 0 || pr.n == 0 || pr.k == 0;
  if (!empty && ((pr.lda * es) % 16 != 0 || (pr.ldb * es) % 16 != 0))
    return set_error(err, TXD_ERR_UNSUPPORTED,
                     "lda and ldb must be multiples of %d elements (TMA needs 16-byte row strides); pad the operands", 16 / es);
  return TXD_OK;
}

// tcgen05 instruction descriptor: fp32 accumulator, both operands of `ab_dtype`, MMA shape block_m x mma_n.
inline uint32_t make_idesc(int ab_dtype, bool p_mn, bool q_mn, int block_m, int mma_n) {
  uint32_t fmt = 0;
  if (ab_dtype == TXD_BF16) fmt = 1;        // kind::f16: 0 = f16, 1 = bf16
  if (ab_dtype == TXD_F8E4M3) fmt = 0;      // kind::f8f6f4: 0 = e4m3, 1 = e5m2
  if (ab_dtype == TXD_F8E5M2) fmt = 1;
  uint32_t d = 0;
  d |= 1u << 4;                              // accumulator format: f32
  d |= fmt << 7;                             // A format
  d |= fmt << 10;                            // B format
  d |= (p_mn ? 1u : 0u) << 15;               // A is MN-major
  d |= (q_mn ? 1u : 0u) << 16;               // B is MN-major
  d |= static_cast<uint32_t>(mma_n >> 3) << 17;
  d |= static_cast<uint32_t>(block_m >> 4) << 24;  // 128, or 256 across a CTA pair
  return d;
}

// Shared-memory matrix descriptor pieces for a SWIZZLE_128B operand stage.
inline void make_smem_desc(bool mn_major, int bk_elems, int umma_k, uint32_t *hi, uint32_t *lbo, uint32_t *kstep) {
  // 8 rows (K-major) or 8 K-slices (MN-major) of 128 bytes form one 1024-byte swizzle atom.
  const uint32_t sbo_bytes = 1024;
  // MN-major: consecutive 128-byte-wide boxes along the row index are bk_elems*128 bytes apart.
  const uint32_t lbo_bytes = mn_major ? static_cast<uint32_t>(bk_elems) * 128u : 16u;
  *hi = ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) /* descriptor version for sm_100 */ | (2u << 29) /* SWIZZLE_128B */;
  *lbo = ((lbo_bytes >> 4) & 0x3FFFu) << 16;
  // Start-address step per MMA: 32 bytes along K (K-major) or umma_k 128-byte slices (MN-major).
  *kstep = mn_major ? static_cast<uint32_t>(umma_k) * 128u / 16u : 2u;
}

// SWIZZLE_128B tensor map of one operand: K-major boxes are 128 bytes of K x tile_rows rows (a stage takes
// one per K atom), MN-major boxes 128 bytes of rows x bk_elems K slices.
inline int encode_operand_map(CUtensorMap *map, const void *ptr, int dtype, bool mn_major, long long rows, long long k,
                              long long ld, int tile_rows, int bk_elems, std::string *err) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return set_error(err, TXD_ERR_NO_DEVICE, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return set_error(err, TXD_ERR_INVALID, "operand pointer %p is not 16-byte aligned", ptr);
  const int es = elem_bytes(dtype);
  const CUtensorMapDataType dt = es == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                         : (dtype == TXD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(mn_major ? rows : k), static_cast<cuuint64_t>(mn_major ? k : rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * es};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / es), static_cast<cuuint32_t>(mn_major ? bk_elems : tile_rows)};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, dt, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(err, TXD_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (dims %llu x %llu, stride %llu, box %u x %u)",
                     (int)r, (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)strides[0], box[0], box[1]);
  return TXD_OK;
}

// Tensor map for the epilogue's TMA store: C is row-major [m, n]; one box is 32 rows x 128 bytes.
inline int encode_store_map(CUtensorMap *map, void *ptr, int out_dtype, long long m, long long n, long long ldc, std::string *err) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return set_error(err, TXD_ERR_NO_DEVICE, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  const int os = elem_bytes(out_dtype);
  const CUtensorMapDataType dt = out_dtype == TXD_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                       : (out_dtype == TXD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                                : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(m)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldc) * os};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / os), 32};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, dt, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(err, TXD_ERR_CUDA, "cuTensorMapEncodeTiled (store map) failed with CUresult %d", (int)r);
  return TXD_OK;
}

inline bool p_is_mn_major(const tx_dot_problem &pr, const TileChoice &tc) {
  return tc.swap_ab ? (pr.b_layout == TXD_ROW_MAJOR) : (pr.a_layout == TXD_COL_MAJOR);
}
inline bool q_is_mn_major(const tx_dot_problem &pr, const TileChoice &tc) {
  return tc.swap_ab ? (pr.a_layout == TXD_COL_MAJOR) : (pr.b_layout == TXD_ROW_MAJOR);
}
// Rows of Q one TMA box of a K-major Q stage holds: one CTA's share of one MMA column half.
inline int q_box_rows(const TileChoice &tc) { return tc.cta_pair ? tc.mma_n / 2 : tc.mma_n; }

// Everything in DotParams that follows from the problem and the tile choice: no pointers, no tensor maps,
// no scratch. The wait limit honours TXD_WAIT_LIMIT_MS; TXD_INJECT_STALL != 0 makes the producer stop after
// its first K block (host-side fault injection for the bounded waits).
inline void fill_params(const tx_dot_problem &pr, const TileChoice &tc, DotParams *out) {
  DotParams &bp = *out;
  memset(&bp, 0, sizeof bp);
  const int es = elem_bytes(pr.ab_dtype);
  const bool p_mn = p_is_mn_major(pr, tc), q_mn = q_is_mn_major(pr, tc);
  bp.ldo = pr.ldc;
  bp.wait_limit_ns = 2000000000ull;  // 2 s per wait; a healthy kernel waits microseconds
  if (const char *e = getenv("TXD_WAIT_LIMIT_MS")) {
    const long v = atol(e);
    if (v > 0) bp.wait_limit_ns = static_cast<unsigned long long>(v) * 1000000ull;
  }
  bp.alpha = pr.alpha;
  bp.p_extent = tc.p_extent;
  bp.q_extent = tc.q_extent;
  bp.k_extent = pr.k;
  bp.trans_out = tc.swap_ab ? 1 : 0;
  bp.out_dtype = pr.out_dtype;
  bp.block_n = tc.mma_n;
  bp.wide = tc.block_n > tc.mma_n ? 1 : 0;
  bp.bk_elems = tc.block_k;
  bp.stages = tc.stages;
  bp.k_blocks = tc.k_blocks;
  bp.k_main_blocks = tc.k_main_blocks;
  bp.tail_mmas = tc.tail_mmas;
  bp.tiles_p = tc.tiles_p;
  bp.tiles_q = tc.tiles_q;
  bp.group_p = tc.group_m;
  bp.stream_k = tc.schedule != TXD_SCHED_DATA_PARALLEL ? 1 : 0;
  bp.sk_first_tile = tc.sk_first_tile;
  bp.kind_f8 = es == 1 ? 1 : 0;
  bp.idesc = make_idesc(pr.ab_dtype, p_mn, q_mn, tc.block_m, tc.mma_n);
  bp.tma_store = tc.tma_store;
  bp.atoms = tc.atoms;
  const int umma_k = 32 / es;
  make_smem_desc(p_mn, tc.block_k, umma_k, &bp.p_desc_hi, &bp.p_desc_lbo, &bp.p_kstep);
  make_smem_desc(q_mn, tc.block_k, umma_k, &bp.q_desc_hi, &bp.q_desc_lbo, &bp.q_kstep);
  bp.p_mn_major = p_mn;
  bp.q_mn_major = q_mn;
  bp.chunk_elems = 128 / es;
  bp.p_stage_bytes = tc.p_stage_bytes;
  bp.q_stage_bytes = tc.q_stage_bytes;
  bp.tmem_cols = tc.tmem_cols;
#ifdef TXD_MEASURE
  if (const char *e = getenv("TXD_DEBUG_FLAGS")) bp.debug_flags = atoi(e) & 15;  // measurement builds only
#endif
  if (const char *e = getenv("TXD_INJECT_STALL")) {
    if (atoi(e) != 0) bp.debug_flags |= 128;
  }
}

}  // namespace host
}  // namespace txd
