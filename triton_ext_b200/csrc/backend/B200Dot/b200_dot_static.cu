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
#include "dot_plan_host.h"

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
  txd::dot_umma_body<false, false>(p);
}
__global__ void __launch_bounds__(txd::kNumThreads, 1)
dot_umma_static_scratch_f8_kernel(const __grid_constant__ txd::DotParams p) {
  txd::dot_umma_body<false, true>(p);
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
    TXS_CUDA(cudaFuncSetAttribute(dot_umma_static_scratch_f8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    s.scratch = static_cast<unsigned char *>(ptr);
    s.sm_count = sms;
    s.ready = true;
  }
  *out = &s;
  return TXD_OK;
}

}  // namespace

extern "C" {

int64_t tx_dot_static_scratch_capacity(void) { return static_cast<int64_t>(kPartialBytes); }

const char *tx_dot_static_scratch_last_error(void) { return g_error.c_str(); }

int tx_dot_run_static_scratch(const tx_dot_problem *problem, const tx_dot_config *cfg_in, const void *a, const void *b,
                              void *c, const float *row_scale, const float *col_scale, void *stream_v) {
  if (!problem) return fail(TXD_ERR_INVALID, "null problem");
  const tx_dot_problem &pr = *problem;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int os = txd::elem_bytes(pr.out_dtype);
  {
    std::string msg;
    const int vrc = txd::host::validate_problem(pr, &msg);  // the same checks as tx_dot_plan_create
    if (vrc) {
      g_error = msg;
      return vrc;
    }
  }
  if (pr.m == 0 || pr.n == 0) return TXD_OK;
  if (!c) return fail(TXD_ERR_INVALID, "null output pointer");
  if (pr.k == 0) {  // empty K loop: C = 0
    TXS_CUDA(cudaMemset2DAsync(c, static_cast<size_t>(pr.ldc) * os, 0, static_cast<size_t>(pr.n) * os, pr.m, stream));
    return TXD_OK;
  }
  if (!a || !b) return fail(TXD_ERR_INVALID, "null operand pointer");
  if ((pr.has_row_scale != 0) != (row_scale != nullptr) || (pr.has_col_scale != 0) != (col_scale != nullptr))
    return fail(TXD_ERR_INVALID, "scale pointers must be given exactly when the problem asks for them");
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
  txd::DotParams prm;
  txd::host::fill_params(pr, tc, &prm);  // honours TXD_WAIT_LIMIT_MS and TXD_INJECT_STALL like the plan path
  std::string msg;
  rc = txd::host::encode_operand_map(&prm.tmap_p, swap ? b : a, pr.ab_dtype, prm.p_mn_major != 0, tc.p_extent, pr.k,
                                     swap ? pr.ldb : pr.lda, txd::kBlockM, tc.block_k, &msg);
  if (!rc)
    rc = txd::host::encode_operand_map(&prm.tmap_q, swap ? a : b, pr.ab_dtype, prm.q_mn_major != 0, tc.q_extent, pr.k,
                                       swap ? pr.lda : pr.ldb, txd::host::q_box_rows(tc), tc.block_k, &msg);
  const bool tma_store = tc.tma_store && (reinterpret_cast<uintptr_t>(c) & 15) == 0;
  if (!rc && tma_store) rc = txd::host::encode_store_map(&prm.tmap_out, c, pr.out_dtype, pr.m, pr.n, pr.ldc, &msg);
  if (rc) {
    g_error = msg;
    return rc;
  }
  unsigned char *base = setup->scratch;
  prm.out = c;
  prm.scale_row = swap ? col_scale : row_scale;
  prm.scale_col = swap ? row_scale : col_scale;
  prm.partials = reinterpret_cast<float *>(base);
  prm.tile_counters = reinterpret_cast<uint32_t *>(base + kPartialBytes);
  prm.status = reinterpret_cast<uint32_t *>(base + kPartialBytes + kCounterBytes);
  prm.tma_store = tma_store ? 1 : 0;

  // The counters of the tiles this call touches must be zero when its kernel starts; an earlier call
  // that gave up on a wait may have left some non-zero.
  TXS_CUDA(cudaMemsetAsync(prm.tile_counters, 0, counter_need, stream));
  if (prm.kind_f8) dot_umma_static_scratch_f8_kernel<<<tc.grid, txd::kNumThreads, tc.smem_bytes, stream>>>(prm);
  else dot_umma_static_scratch_kernel<<<tc.grid, txd::kNumThreads, tc.smem_bytes, stream>>>(prm);
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
