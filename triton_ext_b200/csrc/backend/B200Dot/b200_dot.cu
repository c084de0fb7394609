// Host side of the `b200_dot` backend extension: plan creation (tile selection, TMA descriptors,
// tcgen05 descriptors, scratch) and launch of the sm_100a kernel, behind the C-ABI of b200_dot.h.
//
// There is no CPU path in this file: without a CUDA device every compute entry point fails with
// TXD_ERR_NO_DEVICE.
#include "b200_dot.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>

#include "dot_tile_model.h"
#include "dot_umma_kernel.cuh"
#include "dot_plan_host.h"

namespace {

thread_local std::string g_last_error;
std::atomic<uint64_t> g_launches{0};

int fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

#define TXD_CUDA(expr)                                                                     \
  do {                                                                                     \
    cudaError_t e_ = (expr);                                                               \
    if (e_ != cudaSuccess)                                                                 \
      return fail(TXD_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_));           \
  } while (0)

__global__ void dot_zero_fill_kernel(void *out, long long ldo, int rows, int cols, int elem_bytes) {
  // K == 0: the accumulator of an empty K loop is zero, and so is every scaled/cast result.
  const long long n = static_cast<long long>(rows) * cols;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols, c = i - r * cols;
    unsigned char *dst = static_cast<unsigned char *>(out) + (r * ldo + c) * elem_bytes;
    for (int b = 0; b < elem_bytes; ++b) dst[b] = 0;
  }
}

struct MapKey {
  const void *ptr = nullptr;
  CUtensorMap map;
};

}  // namespace

struct tx_dot_plan {
  tx_dot_problem problem;
  txd::TileChoice tc;
  txd::DotParams base;  // everything except pointers and tensor maps
  int device = 0;
  int sm_count = 0;
  void *scratch = nullptr;      // partials, then counters
  uint32_t *status = nullptr;   // device status word
  MapKey p_cache, q_cache, out_cache;
  // store maps of the K-sharded exchange, one per destination rank, kept while the slot bases stay the same
  MapKey remote_cache[8];
  int remote_cached_world = 0;
  // host-buffer path
  cudaStream_t host_stream = nullptr;
  void *dev_a = nullptr, *dev_b = nullptr, *dev_c = nullptr;
  float *dev_rs = nullptr, *dev_cs = nullptr;
  size_t a_bytes = 0, b_bytes = 0, c_bytes = 0;
  // pipelined host-buffer path: column panels of B and C; copies in, kernels and copies out on three streams
  tx_dot_config user_cfg = {};
  bool has_user_cfg = false;
  cudaStream_t compute_stream = nullptr, d2h_stream = nullptr;
  tx_dot_plan *panel_plan[2] = {nullptr, nullptr};  // regular panel width, last panel width
  int panel_cols[2] = {0, 0};
  cudaEvent_t ev_in[9] = {}, ev_done[8] = {};
  bool events_made = false;
};

namespace {

int validate(const tx_dot_problem &pr) {
  std::string msg;
  const int rc = txd::host::validate_problem(pr, &msg);
  if (rc) g_last_error = msg;
  return rc;
}

int encode_operand_map(CUtensorMap *map, const void *ptr, int dtype, bool mn_major, long long rows, long long k,
                       long long ld, int tile_rows, int bk_elems) {
  std::string msg;
  const int rc = txd::host::encode_operand_map(map, ptr, dtype, mn_major, rows, k, ld, tile_rows, bk_elems, &msg);
  if (rc) g_last_error = msg;
  return rc;
}

int encode_store_map(CUtensorMap *map, void *ptr, int out_dtype, long long m, long long n, long long ldc) {
  std::string msg;
  const int rc = txd::host::encode_store_map(map, ptr, out_dtype, m, n, ldc, &msg);
  if (rc) g_last_error = msg;
  return rc;
}

int build_plan_tiles(const tx_dot_problem &pr, const tx_dot_config *cfg, int sm_count, txd::TileChoice &tc) {
  txd::MachineModel mm;
  mm.sm_count = sm_count;
  const char *why = "";
  if (txd::select_tiles(pr, cfg, mm, tc, &why) != 0) return fail(TXD_ERR_INVALID, "tile selection: %s", why);
  return TXD_OK;
}

}  // namespace

extern "C" {

int tx_dot_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

const char *tx_dot_last_error(void) { return g_last_error.c_str(); }

uint64_t tx_dot_kernel_launches(void) { return g_launches.load(); }

int tx_dot_plan_preview(const tx_dot_problem *problem, const tx_dot_config *cfg, int32_t sm_count,
                        tx_dot_plan_info *info) {
  if (!problem || !info) return fail(TXD_ERR_INVALID, "null argument");
  int rc = validate(*problem);
  if (rc) return rc;
  if (sm_count <= 0) sm_count = 148;
  txd::TileChoice tc;
  if (problem->m == 0 || problem->n == 0 || problem->k == 0) {
    memset(info, 0, sizeof *info);
    return TXD_OK;
  }
  rc = build_plan_tiles(*problem, cfg, sm_count, tc);
  if (rc) return rc;
  txd::fill_plan_info(*problem, tc, info);
  return TXD_OK;
}

int tx_dot_plan_create(const tx_dot_problem *problem, const tx_dot_config *cfg, tx_dot_plan **out_plan) {
  if (!problem || !out_plan) return fail(TXD_ERR_INVALID, "null argument");
  *out_plan = nullptr;
  int rc = validate(*problem);
  if (rc) return rc;
  if (tx_dot_device_count() <= 0) return fail(TXD_ERR_NO_DEVICE, "no CUDA device: the b200_dot backend has no CPU path");
  int dev = 0;
  TXD_CUDA(cudaGetDevice(&dev));
  cudaDeviceProp prop;
  TXD_CUDA(cudaGetDeviceProperties(&prop, dev));
  if (prop.major != 10)
    return fail(TXD_ERR_UNSUPPORTED, "device %d is sm_%d%d; these kernels are built for sm_100a only", dev, prop.major, prop.minor);

  tx_dot_plan *pl = new (std::nothrow) tx_dot_plan();
  if (!pl) return fail(TXD_ERR_INVALID, "out of host memory");
  pl->problem = *problem;
  if (cfg) {
    pl->user_cfg = *cfg;
    pl->has_user_cfg = true;
  }
  pl->device = dev;
  pl->sm_count = prop.multiProcessorCount;
  const tx_dot_problem &pr = pl->problem;
  // From here on every failure releases the plan before it returns.
  auto cuda_step = [&](cudaError_t e, const char *what) -> int {
    if (e == cudaSuccess) return TXD_OK;
    tx_dot_plan_destroy(pl);
    return fail(TXD_ERR_CUDA, "%s failed: %s", what, cudaGetErrorString(e));
  };
  if ((rc = cuda_step(cudaMalloc(&pl->status, 256), "cudaMalloc (status word)"))) return rc;
  if ((rc = cuda_step(cudaMemset(pl->status, 0, 256), "cudaMemset (status word)"))) return rc;
  if (pr.m == 0 || pr.n == 0 || pr.k == 0) {  // nothing for the tensor pipe to do
    *out_plan = pl;
    return TXD_OK;
  }
  rc = build_plan_tiles(pr, cfg, pl->sm_count, pl->tc);
  if (rc) {
    tx_dot_plan_destroy(pl);
    return rc;
  }
  const txd::TileChoice &tc = pl->tc;
  txd::DotParams &bp = pl->base;
  txd::host::fill_params(pr, tc, &bp);
  bp.status = pl->status;

  if (tc.scratch_bytes > 0) {
    if ((rc = cuda_step(cudaMalloc(&pl->scratch, static_cast<size_t>(tc.scratch_bytes)), "cudaMalloc (stream-K scratch)"))) return rc;
    if ((rc = cuda_step(cudaMemset(pl->scratch, 0, static_cast<size_t>(tc.scratch_bytes)), "cudaMemset (stream-K scratch)"))) return rc;
    bp.partials = static_cast<float *>(pl->scratch);
    bp.tile_counters = reinterpret_cast<uint32_t *>(static_cast<char *>(pl->scratch) +
                                                    static_cast<size_t>(tc.grid) * 2 * tc.block_n * 128 * 4);
  }
  cudaError_t e = cudaSuccess;
  for (auto kernel : {txd::dot_umma_kernel, txd::dot_umma_f8_kernel, txd::dot_umma_pair_kernel, txd::dot_umma_pair_f8_kernel})
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e != cudaSuccess) {
    tx_dot_plan_destroy(pl);
    return fail(TXD_ERR_CUDA, "cannot reserve %d bytes of dynamic shared memory: %s", tc.smem_bytes, cudaGetErrorString(e));
  }
  *out_plan = pl;
  return TXD_OK;
}

int tx_dot_plan_query(const tx_dot_plan *plan, tx_dot_plan_info *info) {
  if (!plan || !info) return fail(TXD_ERR_INVALID, "null argument");
  txd::fill_plan_info(plan->problem, plan->tc, info);
  return TXD_OK;
}

}  // extern "C"

namespace {
struct RemoteTarget {
  void *const *slot_bases = nullptr;
  int world = 0, rank = 0;
  int part = 0, parts = 1;  // this launch computes tile rows [part, part + 1) * tiles_p / parts of the interleaved order
};
int launch_dot(tx_dot_plan *pl, const void *a, const void *b, void *c, const float *row_scale, const float *col_scale,
               void *stream_v, const RemoteTarget *remote);

// One thread per 16 bytes of a slot row (4 fp32 or 8 bf16 columns); slots (slot_elems apart) are summed in slot order in
// fp32. kWorld > 0: the slot count is a compile-time constant, so that all `world` loads of a thread are in flight before
// the first add (the sum is HBM-bound: bytes in flight per SM are what sets its rate); kWorld == 0: any count.
template <int kWorld, bool kF32Slots>
__global__ void __launch_bounds__(256) reduce_slots_kernel(const void *slots, int world_rt, long long slot_elems, long long rows,
                                                           long long n, void *out, int out_dtype, long long ldc,
                                                           const float *row_scale, const float *col_scale, float alpha) {
  constexpr int kCols = kF32Slots ? 4 : 8;
  constexpr int kMaxWorld = kWorld > 0 ? kWorld : 1;
  const int world = kWorld > 0 ? kWorld : world_rt;
  const long long groups = (n + kCols - 1) / kCols;
  const long long total = rows * groups;
  const bool rows_vec = n % kCols == 0;  // every group is whole and 16-byte aligned inside its slot
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / groups, c0 = (i - r * groups) * kCols;
    float acc[kCols];
#pragma unroll
    for (int j = 0; j < kCols; ++j) acc[j] = 0.f;
    auto add = [&](const uint4 &v) {
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      if constexpr (kF32Slots) {
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[q] += __uint_as_float(w[q]);
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162 *>(&w[q]);
          acc[2 * q] += __low2float(h);
          acc[2 * q + 1] += __high2float(h);
        }
      }
    };
    const size_t es = kF32Slots ? 4 : 2;
    const char *base = static_cast<const char *>(slots) + static_cast<size_t>(r * n + c0) * es;
    if (rows_vec && kWorld > 0) {
      uint4 v[kMaxWorld];
#pragma unroll
      for (int s = 0; s < kMaxWorld; ++s)
        v[s] = __ldcs(reinterpret_cast<const uint4 *>(base + static_cast<size_t>(s) * slot_elems * es));
#pragma unroll
      for (int s = 0; s < kMaxWorld; ++s) add(v[s]);
    } else if (rows_vec) {
      for (int s = 0; s < world; ++s) add(__ldcs(reinterpret_cast<const uint4 *>(base + static_cast<size_t>(s) * slot_elems * es)));
    } else {
      for (int s = 0; s < world; ++s)
        for (int j = 0; j < kCols && c0 + j < n; ++j) {
          const char *e = base + (static_cast<size_t>(s) * slot_elems + j) * es;
          acc[j] += kF32Slots ? *reinterpret_cast<const float *>(e) : __bfloat162float(*reinterpret_cast<const __nv_bfloat16 *>(e));
        }
    }
    const float rs = (row_scale ? row_scale[r] : 1.0f) * alpha;
    float o[kCols];
#pragma unroll
    for (int j = 0; j < kCols; ++j) o[j] = acc[j] * rs * ((col_scale && c0 + j < n) ? col_scale[c0 + j] : 1.0f);
    if (rows_vec && out_dtype == TXD_BF16) {
      __nv_bfloat16 *dst = static_cast<__nv_bfloat16 *>(out) + r * ldc + c0;
      if ((reinterpret_cast<uintptr_t>(dst) & (kCols * 2 - 1)) == 0) {
        uint32_t w[kCols / 2];
#pragma unroll
        for (int q = 0; q < kCols / 2; ++q) {
          __nv_bfloat162 h = __floats2bfloat162_rn(o[2 * q], o[2 * q + 1]);
          w[q] = *reinterpret_cast<uint32_t *>(&h);
        }
        if constexpr (kCols == 8) *reinterpret_cast<uint4 *>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
        else *reinterpret_cast<uint2 *>(dst) = make_uint2(w[0], w[1]);
        continue;
      }
    }
    for (int j = 0; j < kCols && c0 + j < n; ++j) {
      const long long at = r * ldc + c0 + j;
      if (out_dtype == TXD_F32) static_cast<float *>(out)[at] = o[j];
      else if (out_dtype == TXD_BF16) static_cast<__nv_bfloat16 *>(out)[at] = __float2bfloat16_rn(o[j]);
      else static_cast<__half *>(out)[at] = __float2half_rn(o[j]);
    }
  }
}

template <bool kF32Slots>
void (*pick_reduce_kernel(int world))(const void *, int, long long, long long, long long, void *, int, long long, const float *,
                                      const float *, float) {
  switch (world) {
    case 2: return reduce_slots_kernel<2, kF32Slots>;
    case 4: return reduce_slots_kernel<4, kF32Slots>;
    case 8: return reduce_slots_kernel<8, kF32Slots>;
    default: return reduce_slots_kernel<0, kF32Slots>;
  }
}
}  // namespace

extern "C" {

int tx_dot_run(tx_dot_plan *pl, const void *a, const void *b, void *c, const float *row_scale,
               const float *col_scale, void *stream_v) {
  return launch_dot(pl, a, b, c, row_scale, col_scale, stream_v, nullptr);
}

int tx_dot_run_to_slots_part(tx_dot_plan *pl, const void *a, const void *b, void *const *slot_bases, int32_t world,
                             int32_t rank, int32_t part, int32_t parts, void *stream_v) {
  if (!pl || !slot_bases) return fail(TXD_ERR_INVALID, "null argument");
  const tx_dot_problem &pr = pl->problem;
  const txd::TileChoice &tc = pl->tc;
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(TXD_ERR_INVALID, "world must be 1..8 and rank inside it");
  if (parts < 1 || part < 0 || part >= parts) return fail(TXD_ERR_INVALID, "part must lie in [0, parts)");
  if (pr.m == 0 || pr.n == 0 || pr.k == 0) return fail(TXD_ERR_UNSUPPORTED, "empty problems have no slot form");
  if (pr.has_row_scale || pr.has_col_scale || pr.alpha != 1.0f)
    return fail(TXD_ERR_INVALID, "partials are exchanged unscaled: create the plan without scales; tx_dot_reduce_slots applies them");
  if (pr.out_dtype != TXD_F32 && pr.out_dtype != TXD_BF16) return fail(TXD_ERR_UNSUPPORTED, "slots are f32 or bf16");
  if (!tc.tma_store || tc.swap_ab || tc.schedule != TXD_SCHED_DATA_PARALLEL || pr.ldc != pr.n)
    return fail(TXD_ERR_UNSUPPORTED, "slot stores need the whole-tile schedule, the TMA-store epilogue and ldc == n "
                                     "(create the plan with schedule = TXD_SCHED_DATA_PARALLEL, swap_ab = 2)");
  if (pr.m % world != 0 || (pr.m / world) % tc.block_m != 0)
    return fail(TXD_ERR_UNSUPPORTED, "m / world = %d must be a multiple of the tile height %d", pr.m / world, tc.block_m);
  if ((pr.m / world / tc.block_m) % parts != 0)
    return fail(TXD_ERR_UNSUPPORTED, "the %d tile rows of a rank do not divide into %d parts", pr.m / world / tc.block_m, parts);
  for (int r = 0; r < world; ++r)
    if (!slot_bases[r] || (reinterpret_cast<uintptr_t>(slot_bases[r]) & 15))
      return fail(TXD_ERR_INVALID, "slot base %d is null or not 16-byte aligned", r);
  RemoteTarget rt;
  rt.slot_bases = slot_bases;
  rt.world = world;
  rt.rank = rank;
  rt.part = part;
  rt.parts = parts;
  return launch_dot(pl, a, b, nullptr, nullptr, nullptr, stream_v, &rt);
}

int tx_dot_run_to_slots(tx_dot_plan *pl, const void *a, const void *b, void *const *slot_bases, int32_t world,
                        int32_t rank, void *stream_v) {
  return tx_dot_run_to_slots_part(pl, a, b, slot_bases, world, rank, 0, 1, stream_v);
}

int tx_dot_reduce_slots_part(const void *slots, int32_t world, int32_t rows_per_rank, int32_t row0, int32_t rows, int32_t n,
                             int32_t slot_dtype, void *out, int32_t out_dtype, int64_t ldc, const float *row_scale,
                             const float *col_scale, float alpha, void *stream_v) {
  if (!slots || !out || world < 1 || rows_per_rank < 0 || n < 0 || ldc < n) return fail(TXD_ERR_INVALID, "bad argument");
  if (row0 < 0 || rows < 0 || row0 + static_cast<long long>(rows) > rows_per_rank)
    return fail(TXD_ERR_INVALID, "rows [%d, %d + %d) are not inside a slot of %d rows", row0, row0, rows, rows_per_rank);
  if (slot_dtype != TXD_F32 && slot_dtype != TXD_BF16) return fail(TXD_ERR_UNSUPPORTED, "slots are f32 or bf16");
  if (out_dtype != TXD_F32 && out_dtype != TXD_BF16 && out_dtype != TXD_F16) return fail(TXD_ERR_UNSUPPORTED, "output dtype must be f16, bf16 or f32");
  if (rows == 0 || n == 0) return TXD_OK;
  const bool f32_slots = slot_dtype == TXD_F32;
  const int cols = f32_slots ? 4 : 8;
  const long long total = static_cast<long long>(rows) * ((n + cols - 1) / cols);
  const int threads = 256;
  const int blocks = static_cast<int>(std::min<long long>((total + threads - 1) / threads, 148LL * 16));
  const size_t slot_es = f32_slots ? 4 : 2;
  const size_t out_es = out_dtype == TXD_F32 ? 4 : 2;
  auto kernel = f32_slots ? pick_reduce_kernel<true>(world) : pick_reduce_kernel<false>(world);
  kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream_v)>>>(
      static_cast<const char *>(slots) + static_cast<size_t>(row0) * n * slot_es, world,
      static_cast<long long>(rows_per_rank) * n, rows, n, static_cast<char *>(out) + static_cast<size_t>(row0) * ldc * out_es,
      out_dtype, ldc, row_scale ? row_scale + row0 : nullptr, col_scale, alpha);
  TXD_CUDA(cudaGetLastError());
  g_launches.fetch_add(1);
  return TXD_OK;
}

int tx_dot_reduce_slots(const void *slots, int32_t world, int32_t rows, int32_t n, int32_t slot_dtype, void *out,
                        int32_t out_dtype, int64_t ldc, const float *row_scale, const float *col_scale, float alpha,
                        void *stream_v) {
  return tx_dot_reduce_slots_part(slots, world, rows, 0, rows, n, slot_dtype, out, out_dtype, ldc, row_scale, col_scale,
                                  alpha, stream_v);
}

}  // extern "C"

namespace {
int launch_dot(tx_dot_plan *pl, const void *a, const void *b, void *c, const float *row_scale, const float *col_scale,
               void *stream_v, const RemoteTarget *remote) {
  if (!pl) return fail(TXD_ERR_INVALID, "null plan");
  const tx_dot_problem &pr = pl->problem;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (pr.m == 0 || pr.n == 0) return TXD_OK;
  if (!c && !remote) return fail(TXD_ERR_INVALID, "null output pointer");
  if (pr.k == 0) {
    dot_zero_fill_kernel<<<pl->sm_count, 256, 0, stream>>>(c, pr.ldc, pr.m, pr.n, txd::elem_bytes(pr.out_dtype));
    TXD_CUDA(cudaGetLastError());
    g_launches.fetch_add(1);
    return TXD_OK;
  }
  if (!a || !b) return fail(TXD_ERR_INVALID, "null operand pointer");
  if ((pr.has_row_scale != 0) != (row_scale != nullptr) || (pr.has_col_scale != 0) != (col_scale != nullptr))
    return fail(TXD_ERR_INVALID, "scale pointers must be given exactly when the plan was created with them");
  const txd::TileChoice &tc = pl->tc;
  const bool swap = tc.swap_ab != 0;
  const void *p_ptr = swap ? b : a;
  const void *q_ptr = swap ? a : b;
  const long long p_ld = swap ? pr.ldb : pr.lda;
  const long long q_ld = swap ? pr.lda : pr.ldb;
  if (pl->p_cache.ptr != p_ptr) {
    int rc = encode_operand_map(&pl->p_cache.map, p_ptr, pr.ab_dtype, pl->base.p_mn_major != 0, tc.p_extent, pr.k, p_ld,
                                txd::kBlockM, tc.block_k);
    if (rc) return rc;
    pl->p_cache.ptr = p_ptr;
  }
  if (pl->q_cache.ptr != q_ptr) {
    int rc = encode_operand_map(&pl->q_cache.map, q_ptr, pr.ab_dtype, pl->base.q_mn_major != 0, tc.q_extent, pr.k, q_ld,
                                txd::host::q_box_rows(tc), tc.block_k);
    if (rc) return rc;
    pl->q_cache.ptr = q_ptr;
  }
  // TMA store needs a 16-byte aligned C; otherwise this launch stores straight from registers.
  const bool tma_store = tc.tma_store && (remote || (reinterpret_cast<uintptr_t>(c) & 15) == 0);
  if (tma_store && !remote && pl->out_cache.ptr != c) {
    int rc = encode_store_map(&pl->out_cache.map, c, pr.out_dtype, pr.m, pr.n, pr.ldc);
    if (rc) return rc;
    pl->out_cache.ptr = c;
  }
  txd::DotParams prm = pl->base;
  prm.tmap_p = pl->p_cache.map;
  prm.tmap_q = pl->q_cache.map;
  prm.out = c;
  // Scales follow their matrix: after the role swap, rows of C are the Q index.
  prm.scale_row = swap ? col_scale : row_scale;
  prm.scale_col = swap ? row_scale : col_scale;
  prm.tma_store = tma_store ? 1 : 0;
  if (tma_store && !remote) prm.tmap_out = pl->out_cache.map;
  if (remote) {
    // One store map per destination rank: its slot buffer seen as a [world * rows_per_rank, n] matrix.
    prm.remote_world = remote->world;
    prm.remote_rank = remote->rank;
    prm.rows_per_rank = pr.m / remote->world;
    // Consecutive tile rows of the raster go to consecutive owners (rank + 1, rank + 2, ..., rank): every wave of tiles
    // stores to all owners at once, so each NVLink pair carries an even share all the time and the tiles whose rows this
    // rank owns (no NVLink bytes) are spread over the run instead of forming a phase of their own.
    prm.tp_interleave = remote->world;
    prm.tiles_p_all = tc.tiles_p;
    prm.tiles_p = tc.tiles_p / remote->parts;
    prm.tp_begin = remote->part * prm.tiles_p;
    if (pl->remote_cached_world != remote->world) {
      for (auto &mk : pl->remote_cache) mk.ptr = nullptr;
      pl->remote_cached_world = remote->world;
    }
    for (int r = 0; r < remote->world; ++r) {
      MapKey &mk = pl->remote_cache[r];
      if (mk.ptr != remote->slot_bases[r]) {
        int rc = encode_store_map(&mk.map, remote->slot_bases[r], pr.out_dtype, pr.m, pr.n, pr.n);
        if (rc) return rc;
        mk.ptr = remote->slot_bases[r];
      }
      prm.tmap_remote[r] = mk.map;
    }
  }
  {
    // Programmatic stream serialization: this launch may be scheduled while the kernel before it in the stream is
    // still running (as SMs become free); the kernel waits for that predecessor before it touches global memory.
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(tc.grid);
    lc.blockDim = dim3(txd::kNumThreads);
    lc.dynamicSmemBytes = tc.smem_bytes;
    lc.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
    if (tc.cta_pair) {
      attr[n_attr].id = cudaLaunchAttributeClusterDimension;
      attr[n_attr].val.clusterDim.x = 2;
      attr[n_attr].val.clusterDim.y = 1;
      attr[n_attr].val.clusterDim.z = 1;
      ++n_attr;
    }
    lc.attrs = attr;
    lc.numAttrs = n_attr;
    auto kernel = tc.cta_pair ? (prm.kind_f8 ? txd::dot_umma_pair_f8_kernel : txd::dot_umma_pair_kernel)
                              : (prm.kind_f8 ? txd::dot_umma_f8_kernel : txd::dot_umma_kernel);
    TXD_CUDA(cudaLaunchKernelEx(&lc, kernel, prm));
  }
  TXD_CUDA(cudaGetLastError());
  g_launches.fetch_add(1);
  return TXD_OK;
}
}  // namespace

extern "C" {

int tx_dot_plan_check(tx_dot_plan *pl, void *stream_v) {
  if (!pl) return fail(TXD_ERR_INVALID, "null plan");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  TXD_CUDA(cudaStreamSynchronize(stream));
  uint32_t st = 0;
  TXD_CUDA(cudaMemcpy(&st, pl->status, sizeof st, cudaMemcpyDeviceToHost));
  if (st != 0) {
    cudaMemset(pl->status, 0, sizeof st);
    if (pl->scratch) cudaMemset(pl->scratch, 0, static_cast<size_t>(pl->tc.scratch_bytes));
    static const char *kWho[] = {"", "TMA producer (stage never freed)", "MMA issuer (stage never filled)",
                                 "MMA issuer (accumulator never drained)", "epilogue (accumulator never completed)",
                                 "teardown (copies or MMAs still in flight)"};
    return fail(TXD_ERR_DEVICE_TIMEOUT, "device-side wait ran out in the %s; output is undefined", kWho[st < 6 ? st : 0]);
  }
  return TXD_OK;
}

}  // extern "C"

namespace {

constexpr int kMaxHostPanels = 8;

// The host-buffer path is dominated by its copies (PCIe), so above 32 MB they are overlapped with the kernels:
// one operand goes to the device whole, the other one and C are cut into panels; panel j+1 travels to the device
// while panel j is multiplied and panel j-1 travels back.
// The operand that travels whole comes first and delays the first kernel, so it should be the smaller one: rows of A
// and C are the panels when A is row-major (contiguous panels) and B is not the bigger operand; otherwise columns of B and
// C (contiguous for a column-major B, strided 2-D copies for a row-major one).
bool host_panels_by_rows(const tx_dot_problem &pr) {
  const long long a_elems = static_cast<long long>(pr.m) * pr.k, b_elems = static_cast<long long>(pr.k) * pr.n;
  return pr.a_layout == TXD_ROW_MAJOR && b_elems <= a_elems;
}

int host_panels(const tx_dot_problem &pr) {
  const long long es = txd::elem_bytes(pr.ab_dtype), os = txd::elem_bytes(pr.out_dtype);
  const long long bytes = (static_cast<long long>(pr.m) * pr.k + static_cast<long long>(pr.k) * pr.n) * es +
                          static_cast<long long>(pr.m) * pr.n * os;
  const int extent = host_panels_by_rows(pr) ? pr.m : pr.n;
  if (pr.k == 0 || bytes < (32LL << 20) || extent < 2 * 512) return 1;
  int panels = extent / 512;  // at least two tile rows / columns per panel
  if (panels > kMaxHostPanels) panels = kMaxHostPanels;
  return panels < 2 ? 1 : panels;
}

int run_host_pipelined(tx_dot_plan *pl, const void *a_host, const void *b_host, void *c_host,
                       const float *row_scale_host, const float *col_scale_host) {
  const tx_dot_problem &pr = pl->problem;
  const size_t es = txd::elem_bytes(pr.ab_dtype), os = txd::elem_bytes(pr.out_dtype);
  const int panels = host_panels(pr);
  const bool by_rows = host_panels_by_rows(pr);
  const int extent = by_rows ? pr.m : pr.n;
  // panel boundaries on multiples of 256 (tile size; keeps every sub-pointer 16-byte aligned)
  const int step = ((extent / panels + 255) / 256) * 256;
  if (!pl->compute_stream) {
    TXD_CUDA(cudaStreamCreateWithFlags(&pl->compute_stream, cudaStreamNonBlocking));
    TXD_CUDA(cudaStreamCreateWithFlags(&pl->d2h_stream, cudaStreamNonBlocking));
  }
  if (!pl->events_made) {
    for (auto &e : pl->ev_in) TXD_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    for (auto &e : pl->ev_done) TXD_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    pl->events_made = true;
  }
  cudaStream_t in = pl->host_stream, run = pl->compute_stream, out = pl->d2h_stream;
  // the whole operand and the scales first
  if (by_rows) TXD_CUDA(cudaMemcpyAsync(pl->dev_b, b_host, pl->b_bytes, cudaMemcpyHostToDevice, in));
  else TXD_CUDA(cudaMemcpyAsync(pl->dev_a, a_host, pl->a_bytes, cudaMemcpyHostToDevice, in));
  if (pr.has_row_scale) {
    if (!row_scale_host) return fail(TXD_ERR_INVALID, "row scale expected");
    TXD_CUDA(cudaMemcpyAsync(pl->dev_rs, row_scale_host, sizeof(float) * pr.m, cudaMemcpyHostToDevice, in));
  }
  if (pr.has_col_scale) {
    if (!col_scale_host) return fail(TXD_ERR_INVALID, "column scale expected");
    TXD_CUDA(cudaMemcpyAsync(pl->dev_cs, col_scale_host, sizeof(float) * pr.n, cudaMemcpyHostToDevice, in));
  }
  for (int j = 0; j < panels; ++j) {
    const int i0 = j * step;
    if (i0 >= extent) break;
    const int i1 = (i0 + step < extent && j + 1 < panels) ? i0 + step : extent;
    const int w = i1 - i0;
    const char *a_dev = static_cast<const char *>(pl->dev_a);
    const char *b_dev = static_cast<const char *>(pl->dev_b);
    char *c_dev = static_cast<char *>(pl->dev_c);
    if (by_rows) {
      // rows [i0, i1) of A (row-major: contiguous) and of C
      const size_t a_off = static_cast<size_t>(i0) * pr.lda * es;
      TXD_CUDA(cudaMemcpyAsync(static_cast<char *>(pl->dev_a) + a_off, static_cast<const char *>(a_host) + a_off,
                               static_cast<size_t>(w) * pr.lda * es, cudaMemcpyHostToDevice, in));
      a_dev += a_off;
      c_dev += static_cast<size_t>(i0) * pr.ldc * os;
    } else {
      // columns [i0, i1) of B: a strided block of a row-major [K, N] matrix, or rows of its column-major storage
      const size_t b_off = pr.b_layout == TXD_ROW_MAJOR ? static_cast<size_t>(i0) * es : static_cast<size_t>(i0) * pr.ldb * es;
      const char *b_src = static_cast<const char *>(b_host) + b_off;
      char *b_dst = static_cast<char *>(pl->dev_b) + b_off;
      if (pr.b_layout == TXD_ROW_MAJOR)
        TXD_CUDA(cudaMemcpy2DAsync(b_dst, pr.ldb * es, b_src, pr.ldb * es, static_cast<size_t>(w) * es, pr.k,
                                   cudaMemcpyHostToDevice, in));
      else
        TXD_CUDA(cudaMemcpyAsync(b_dst, b_src, static_cast<size_t>(w) * pr.ldb * es, cudaMemcpyHostToDevice, in));
      b_dev += b_off;
      c_dev += static_cast<size_t>(i0) * os;
    }
    TXD_CUDA(cudaEventRecord(pl->ev_in[j], in));
    // the panel's own plan (same leading dimensions: it works in place inside the full matrices)
    const int which = (w == step) ? 0 : 1;
    if (!pl->panel_plan[which] || pl->panel_cols[which] != w) {
      if (pl->panel_plan[which]) tx_dot_plan_destroy(pl->panel_plan[which]);
      pl->panel_plan[which] = nullptr;
      tx_dot_problem sub = pr;
      if (by_rows) sub.m = w; else sub.n = w;
      int rc = tx_dot_plan_create(&sub, pl->has_user_cfg ? &pl->user_cfg : nullptr, &pl->panel_plan[which]);
      if (rc) return rc;
      pl->panel_cols[which] = w;
    }
    TXD_CUDA(cudaStreamWaitEvent(run, pl->ev_in[j], 0));
    const float *rs = pl->dev_rs ? pl->dev_rs + (by_rows ? i0 : 0) : nullptr;
    const float *cs = pl->dev_cs ? pl->dev_cs + (by_rows ? 0 : i0) : nullptr;
    int rc = tx_dot_run(pl->panel_plan[which], a_dev, b_dev, c_dev, rs, cs, run);
    if (rc) return rc;
    TXD_CUDA(cudaEventRecord(pl->ev_done[j], run));
    TXD_CUDA(cudaStreamWaitEvent(out, pl->ev_done[j], 0));
    char *c_dst = static_cast<char *>(c_host) + (c_dev - static_cast<char *>(pl->dev_c));
    if (by_rows)
      TXD_CUDA(cudaMemcpyAsync(c_dst, c_dev, static_cast<size_t>(w) * pr.ldc * os, cudaMemcpyDeviceToHost, out));
    else
      TXD_CUDA(cudaMemcpy2DAsync(c_dst, pr.ldc * os, c_dev, pr.ldc * os, static_cast<size_t>(w) * os, pr.m,
                                 cudaMemcpyDeviceToHost, out));
  }
  TXD_CUDA(cudaStreamSynchronize(out));
  for (int which = 0; which < 2; ++which)
    if (pl->panel_plan[which]) {
      int rc = tx_dot_plan_check(pl->panel_plan[which], run);
      if (rc) return rc;
    }
  return TXD_OK;
}

}  // namespace

extern "C" {

int tx_dot_run_host(tx_dot_plan *pl, const void *a_host, const void *b_host, void *c_host,
                    const float *row_scale_host, const float *col_scale_host) {
  if (!pl) return fail(TXD_ERR_INVALID, "null plan");
  const tx_dot_problem &pr = pl->problem;
  if (pr.m == 0 || pr.n == 0) return TXD_OK;
  if (!c_host || (pr.k > 0 && (!a_host || !b_host))) return fail(TXD_ERR_INVALID, "null host pointer");
  const size_t es = txd::elem_bytes(pr.ab_dtype), os = txd::elem_bytes(pr.out_dtype);
  const size_t a_rows = pr.a_layout == TXD_ROW_MAJOR ? pr.m : pr.k;
  const size_t b_rows = pr.b_layout == TXD_ROW_MAJOR ? pr.k : pr.n;
  if (!pl->host_stream) {
    TXD_CUDA(cudaStreamCreateWithFlags(&pl->host_stream, cudaStreamNonBlocking));
    pl->a_bytes = a_rows * pr.lda * es;
    pl->b_bytes = b_rows * pr.ldb * es;
    pl->c_bytes = static_cast<size_t>(pr.m) * pr.ldc * os;
    if (pl->a_bytes) TXD_CUDA(cudaMalloc(&pl->dev_a, pl->a_bytes));
    if (pl->b_bytes) TXD_CUDA(cudaMalloc(&pl->dev_b, pl->b_bytes));
    TXD_CUDA(cudaMalloc(&pl->dev_c, pl->c_bytes));
    if (pr.has_row_scale) TXD_CUDA(cudaMalloc(&pl->dev_rs, sizeof(float) * pr.m));
    if (pr.has_col_scale) TXD_CUDA(cudaMalloc(&pl->dev_cs, sizeof(float) * pr.n));
  }
  cudaStream_t s = pl->host_stream;
  if (host_panels(pr) > 1) return run_host_pipelined(pl, a_host, b_host, c_host, row_scale_host, col_scale_host);
  if (pr.k > 0) {
    TXD_CUDA(cudaMemcpyAsync(pl->dev_a, a_host, pl->a_bytes, cudaMemcpyHostToDevice, s));
    TXD_CUDA(cudaMemcpyAsync(pl->dev_b, b_host, pl->b_bytes, cudaMemcpyHostToDevice, s));
  }
  if (pr.has_row_scale) {
    if (!row_scale_host) return fail(TXD_ERR_INVALID, "row scale expected");
    TXD_CUDA(cudaMemcpyAsync(pl->dev_rs, row_scale_host, sizeof(float) * pr.m, cudaMemcpyHostToDevice, s));
  }
  if (pr.has_col_scale) {
    if (!col_scale_host) return fail(TXD_ERR_INVALID, "column scale expected");
    TXD_CUDA(cudaMemcpyAsync(pl->dev_cs, col_scale_host, sizeof(float) * pr.n, cudaMemcpyHostToDevice, s));
  }
  int rc = tx_dot_run(pl, pl->dev_a, pl->dev_b, pl->dev_c, pl->dev_rs, pl->dev_cs, s);
  if (rc) return rc;
  TXD_CUDA(cudaMemcpyAsync(c_host, pl->dev_c, pl->c_bytes, cudaMemcpyDeviceToHost, s));
  return tx_dot_plan_check(pl, s);
}

#ifdef TXD_MEASURE
// Measurement builds only: {cycles at start, cycles at end, ns at start, ns at end} of CTA 0 of the plan's last launch.
__attribute__((visibility("default"))) int tx_dot_debug_stamps(tx_dot_plan *pl, unsigned long long *out4) {
  if (!pl || !out4) return TXD_ERR_INVALID;
  TXD_CUDA(cudaDeviceSynchronize());
  TXD_CUDA(cudaMemcpy(out4, reinterpret_cast<char *>(pl->status) + 64, 48, cudaMemcpyDeviceToHost));  // 6 words
  return TXD_OK;
}
#endif

int tx_dot_plan_destroy(tx_dot_plan *pl) {
  if (!pl) return TXD_OK;
  if (pl->scratch) cudaFree(pl->scratch);
  if (pl->status) cudaFree(pl->status);
  if (pl->dev_a) cudaFree(pl->dev_a);
  if (pl->dev_b) cudaFree(pl->dev_b);
  if (pl->dev_c) cudaFree(pl->dev_c);
  if (pl->dev_rs) cudaFree(pl->dev_rs);
  if (pl->dev_cs) cudaFree(pl->dev_cs);
  if (pl->host_stream) cudaStreamDestroy(pl->host_stream);
  if (pl->compute_stream) cudaStreamDestroy(pl->compute_stream);
  if (pl->d2h_stream) cudaStreamDestroy(pl->d2h_stream);
  if (pl->events_made) {
    for (auto &e : pl->ev_in) cudaEventDestroy(e);
    for (auto &e : pl->ev_done) cudaEventDestroy(e);
  }
  for (tx_dot_plan *sub : pl->panel_plan) tx_dot_plan_destroy(sub);
  delete pl;
  return TXD_OK;
}

}  // extern "C"
