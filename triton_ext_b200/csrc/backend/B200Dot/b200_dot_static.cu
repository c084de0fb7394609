// tx_dot_run_static_scratch — the stream-K tt.dot kernel for callers that must not allocate.
//
// Who needs it: code that runs where a device allocation is impossible or forbidden — a launch made
// while another library owns the whole memory pool of the process, a real-time or interrupt-like host
// thread that may not take the driver's allocator lock, a plug-in host that audits cudaMalloc calls.
// The plan-based entry points (tx_dot_plan_create) allocate a status word and, for the stream-K
// schedule, a scratch buffer for partial tiles. This entry point allocates nothing, on the device or
// through any library: the scratch lives in one fixed-size array that is part of the loaded module.
//
// Limits and rules, all checked or documented here:
//   * the stream-K scratch of the chosen configuration (2 partial tiles per CTA + one counter per output
//     tile) must fit kPartialBytes / kCounterBytes below; a bigger problem is refused with
//     TXD_ERR_UNSUPPORTED and a message giving both sizes;
//   * every GPU that loads the library carries the array (about 4.1 MiB) until the process exits;
//   * all calls share the array. Two calls whose kernels overlap on one GPU (different streams, or
//     different host threads) race on it and produce garbage: serialise them;
//   * the array keeps whatever the last call left. The tile counters must start at zero, so every
//     call clears the ones it uses on `stream` before its launch; partial tiles are always written
//     before they are read and need no clearing;
//   * the first call on a device looks up the array's device address and raises the kernel's
//     shared-memory limit. Make that first call before starting any stream capture.
//
// The kernel is the same dot_umma_body<false> as everywhere else, instantiated here under its own
// name so that the array, the address lookup and the launch sit in one translation unit: in host code
// the array's name is only a host-side handle, never a device address — the address passed to the
// kernel comes from cudaGetSymbolAddress, looked up with the target device current.
#include "b200_dot.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "dot_tile_model.h"
#define TXD_NO_KERNEL_ENTRY_POINTS  // this file launches its own instantiation only
#include "dot_umma_kernel.cuh"

namespace {

constexpr size_t kPartialBytes = 4u << 20;   // fp32 partial tiles: grid * 2 * block_n * 128 * 4 bytes
constexpr size_t kCounterBytes = 64u << 10;  // one uint32 per output tile: up to 16384 tiles
constexpr size_t kStatusBytes = 256;         // device status word of the bounded waits
constexpr size_t kScratchBytes = kPartialBytes + kCounterBytes + kStatusBytes;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

thread_local std::string g_error;

int fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_error = buf;
  return code;
}

#define TXS_CUDA(expr)                                                                   \
  do {                                                                                   \
    cudaError_t e_ = (expr);                                                             \
    if (e_ != cudaSuccess)                                                               \
      return fail(TXD_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_));         \
  } while (0)

__global__ void __launch_bounds__(txd::kNumThreads, 1)
dot_umma_static_scratch_kernel(const __grid_constant__ txd::DotParams p) {
  txd::dot_umma_body<false>(p);
}

struct DeviceSetup {
  bool ready = false;
  unsigned char *scratch = nullptr;  // device address of g_static_scratch on this device
  int sm_count = 0;
};
std::mutex g_setup_mu;
DeviceSetup g_setup[kMaxDevices];

// Once per device, with that device current: resolve the array's device address, raise the kernel's
// dynamic shared-memory limit. Neither call allocates.
int setup_device(int dev, DeviceSetup **out) {
  if (dev < 0 || dev >= kMaxDevices) return fail(TXD_ERR_UNSUPPORTED, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_setup_mu);
  DeviceSetup &s = g_setup[dev];
  if (!s.ready) {
    int major = 0, sms = 0;
    TXS_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    TXS_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (major != 10) return fail(TXD_ERR_UNSUPPORTED, "device %d is not sm_100; these kernels are built for sm_100a only", dev);
    void *ptr = nullptr;
    TXS_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
    if (!ptr) return fail(TXD_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    TXS_CUDA(cudaFuncSetAttribute(dot_umma_static_scratch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    s.scratch = static_cast<unsigned char *>(ptr);
    s.sm_count = sms;
    s.ready = true;
  }
  *out = &s;
  return TXD_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

// SWIZZLE_128B tensor map of one operand: K-major boxes are bk x tile_rows, MN-major boxes 128 bytes x bk.
int encode_operand(CUtensorMap *map, const void *ptr, int dtype, bool mn_major, long long rows, long long k,
                   long long ld, int tile_rows, int bk) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return fail(TXD_ERR_NO_DEVICE, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return fail(TXD_ERR_INVALID, "operand pointer %p is not 16-byte aligned", ptr);
  const int es = txd::elem_bytes(dtype);
  const CUtensorMapDataType dt = es == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                         : (dtype == TXD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(mn_major ? rows : k), static_cast<cuuint64_t>(mn_major ? k : rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * es};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / es), static_cast<cuuint32_t>(mn_major ? bk : tile_rows)};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, dt, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TXD_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return TXD_OK;
}

int encode_store(CUtensorMap *map, void *ptr, int out_dtype, long long m, long long n, long long ldc) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return fail(TXD_ERR_NO_DEVICE, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  const int os = txd::elem_bytes(out_dtype);
  const CUtensorMapDataType dt = out_dtype == TXD_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                       : (out_dtype == TXD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                                : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(m)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldc) * os};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / os), 32};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, dt, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TXD_ERR_CUDA, "cuTensorMapEncodeTiled (store map) failed with CUresult %d", (int)r);
  return TXD_OK;
}

uint32_t smem_desc_hi() { return ((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29); }  // SBO 1024, sm_100, SWIZZLE_128B

}  // namespace

extern "C" {

int64_t tx_dot_static_scratch_capacity(void) { return static_cast<int64_t>(kPartialBytes); }

const char *tx_dot_static_scratch_last_error(void) { return g_error.c_str(); }

int tx_dot_run_static_scratch(const tx_dot_problem *problem, const tx_dot_config *cfg_in, const void *a, const void *b,
                              void *c, const float *row_scale, const float *col_scale, void *stream_v) {
  if (!problem) return fail(TXD_ERR_INVALID, "null problem");
  const tx_dot_problem &pr = *problem;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int es = txd::elem_bytes(pr.ab_dtype), os = txd::elem_bytes(pr.out_dtype);
  if (pr.m < 0 || pr.n < 0 || pr.k < 0) return fail(TXD_ERR_INVALID, "negative extent");
  if (pr.ab_dtype == TXD_F32 || (es != 1 && es != 2)) return fail(TXD_ERR_UNSUPPORTED, "operand dtype must be f16, bf16, f8e4m3 or f8e5m2");
  if (pr.out_dtype != TXD_F16 && pr.out_dtype != TXD_BF16 && pr.out_dtype != TXD_F32)
    return fail(TXD_ERR_UNSUPPORTED, "output dtype must be f16, bf16 or f32");
  if (pr.m == 0 || pr.n == 0) return TXD_OK;
  if (!c) return fail(TXD_ERR_INVALID, "null output pointer");
  if (pr.ldc < pr.n) return fail(TXD_ERR_INVALID, "ldc smaller than n");
  if (pr.k == 0) {  // empty K loop: C = 0
    TXS_CUDA(cudaMemset2DAsync(c, static_cast<size_t>(pr.ldc) * os, 0, static_cast<size_t>(pr.n) * os, pr.m, stream));
    return TXD_OK;
  }
  if (!a || !b) return fail(TXD_ERR_INVALID, "null operand pointer");
  if ((pr.has_row_scale != 0) != (row_scale != nullptr) || (pr.has_col_scale != 0) != (col_scale != nullptr))
    return fail(TXD_ERR_INVALID, "scale pointers must be given exactly when the problem asks for them");
  const long long a_min = pr.a_layout == TXD_ROW_MAJOR ? pr.k : pr.m;
  const long long b_min = pr.b_layout == TXD_ROW_MAJOR ? pr.n : pr.k;
  if (pr.lda < a_min || pr.ldb < b_min) return fail(TXD_ERR_INVALID, "leading dimension smaller than the row length");
  if ((pr.lda * es) % 16 != 0 || (pr.ldb * es) % 16 != 0)
    return fail(TXD_ERR_UNSUPPORTED, "lda and ldb must be multiples of %d elements (TMA needs 16-byte row strides)", 16 / es);

  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return fail(TXD_ERR_NO_DEVICE, "no CUDA device: the b200_dot backend has no CPU path");
  }
  DeviceSetup *setup = nullptr;
  int rc = setup_device(dev, &setup);
  if (rc) return rc;

  // Always the stream-K schedule on single CTAs: that is the variant whose scratch this array replaces.
  tx_dot_config cfg = {};
  if (cfg_in) cfg = *cfg_in;
  cfg.schedule = TXD_SCHED_STREAM_K;
  cfg.cta_pair = 2;
  txd::MachineModel mm;
  mm.sm_count = setup->sm_count;
  txd::TileChoice tc;
  const char *why = "";
  if (txd::select_tiles(pr, &cfg, mm, tc, &why) != 0) return fail(TXD_ERR_INVALID, "tile selection: %s", why);
  const size_t partial_need = static_cast<size_t>(tc.grid) * 2 * tc.block_n * 128 * 4;
  const size_t counter_need = static_cast<size_t>(tc.tiles_p) * tc.tiles_q * 4;
  if (partial_need > kPartialBytes || counter_need > kCounterBytes)
    return fail(TXD_ERR_UNSUPPORTED,
                "stream-K scratch of this configuration (%zu bytes of partial tiles, %zu bytes of counters) exceeds the "
                "static scratch (%zu / %zu bytes); use a smaller block_n or max_ctas, or the plan-based entry points",
                partial_need, counter_need, kPartialBytes, kCounterBytes);

  const bool swap = tc.swap_ab != 0;
  const bool p_mn = swap ? (pr.b_layout == TXD_ROW_MAJOR) : (pr.a_layout == TXD_COL_MAJOR);
  const bool q_mn = swap ? (pr.a_layout == TXD_COL_MAJOR) : (pr.b_layout == TXD_ROW_MAJOR);
  const int umma_k = 32 / es;

  txd::DotParams prm;
  memset(&prm, 0, sizeof prm);
  rc = encode_operand(&prm.tmap_p, swap ? b : a, pr.ab_dtype, p_mn, tc.p_extent, pr.k, swap ? pr.ldb : pr.lda, txd::kBlockM, tc.block_k);
  if (rc) return rc;
  rc = encode_operand(&prm.tmap_q, swap ? a : b, pr.ab_dtype, q_mn, tc.q_extent, pr.k, swap ? pr.lda : pr.ldb, tc.block_n, tc.block_k);
  if (rc) return rc;
  const bool tma_store = tc.tma_store && (reinterpret_cast<uintptr_t>(c) & 15) == 0;
  if (tma_store) {
    rc = encode_store(&prm.tmap_out, c, pr.out_dtype, pr.m, pr.n, pr.ldc);
    if (rc) return rc;
  }
  unsigned char *base = setup->scratch;
  prm.out = c;
  prm.scale_row = swap ? col_scale : row_scale;
  prm.scale_col = swap ? row_scale : col_scale;
  prm.partials = reinterpret_cast<float *>(base);
  prm.tile_counters = reinterpret_cast<uint32_t *>(base + kPartialBytes);
  prm.status = reinterpret_cast<uint32_t *>(base + kPartialBytes + kCounterBytes);
  prm.ldo = pr.ldc;
  prm.wait_limit_ns = 2000000000ull;
  if (const char *e = getenv("TXD_WAIT_LIMIT_MS")) {
    const long v = atol(e);
    if (v > 0) prm.wait_limit_ns = static_cast<unsigned long long>(v) * 1000000ull;
  }
  prm.alpha = pr.alpha;
  prm.p_extent = tc.p_extent;
  prm.q_extent = tc.q_extent;
  prm.k_extent = pr.k;
  prm.trans_out = swap ? 1 : 0;
  prm.out_dtype = pr.out_dtype;
  prm.block_n = tc.block_n;
  prm.bk_elems = tc.block_k;
  prm.stages = tc.stages;
  prm.k_blocks = tc.k_blocks;
  prm.k_main_blocks = tc.k_main_blocks;
  prm.tail_mmas = tc.tail_mmas;
  prm.tiles_p = tc.tiles_p;
  prm.tiles_q = tc.tiles_q;
  prm.group_p = tc.group_m;
  prm.stream_k = 1;
  prm.kind_f8 = es == 1 ? 1 : 0;
  {
    uint32_t fmt = (pr.ab_dtype == TXD_BF16 || pr.ab_dtype == TXD_F8E5M2) ? 1u : 0u;
    prm.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((p_mn ? 1u : 0u) << 15) | ((q_mn ? 1u : 0u) << 16) |
                (static_cast<uint32_t>(tc.block_n >> 3) << 17) | (static_cast<uint32_t>(txd::kBlockM >> 4) << 24);
  }
  prm.p_desc_hi = prm.q_desc_hi = smem_desc_hi();
  prm.p_desc_lbo = (((p_mn ? static_cast<uint32_t>(tc.block_k) * 128u : 16u) >> 4) & 0x3FFFu) << 16;
  prm.q_desc_lbo = (((q_mn ? static_cast<uint32_t>(tc.block_k) * 128u : 16u) >> 4) & 0x3FFFu) << 16;
  prm.p_kstep = p_mn ? static_cast<uint32_t>(umma_k) * 128u / 16u : 2u;
  prm.q_kstep = q_mn ? static_cast<uint32_t>(umma_k) * 128u / 16u : 2u;
  prm.p_mn_major = p_mn;
  prm.q_mn_major = q_mn;
  prm.chunk_elems = 128 / es;
  prm.p_stage_bytes = tc.p_stage_bytes;
  prm.q_stage_bytes = tc.q_stage_bytes;
  prm.tmem_cols = tc.tmem_cols;
  prm.tma_store = tma_store ? 1 : 0;
  prm.atoms = tc.atoms;

  // The counters of the tiles this call touches must be zero when its kernel starts; an earlier call
  // that gave up on a wait may have left some non-zero.
  TXS_CUDA(cudaMemsetAsync(prm.tile_counters, 0, counter_need, stream));
  dot_umma_static_scratch_kernel<<<tc.grid, txd::kNumThreads, tc.smem_bytes, stream>>>(prm);
  TXS_CUDA(cudaGetLastError());
  return TXD_OK;
}

int tx_dot_static_scratch_check(void *stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return fail(TXD_ERR_NO_DEVICE, "no CUDA device");
  }
  DeviceSetup *setup = nullptr;
  int rc = setup_device(dev, &setup);
  if (rc) return rc;
  TXS_CUDA(cudaStreamSynchronize(stream));
  uint32_t st = 0;
  unsigned char *status = setup->scratch + kPartialBytes + kCounterBytes;
  TXS_CUDA(cudaMemcpy(&st, status, sizeof st, cudaMemcpyDeviceToHost));
  if (st != 0) {
    const uint32_t zero = 0;
    cudaMemcpy(status, &zero, sizeof zero, cudaMemcpyHostToDevice);
    return fail(TXD_ERR_DEVICE_TIMEOUT, "a device-side wait ran out (code %u) in a static-scratch launch; output is undefined", st);
  }
  return TXD_OK;
}

}  // extern "C"
