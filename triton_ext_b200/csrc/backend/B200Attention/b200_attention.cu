// Host side of the fused attention forward: argument checks, TMA descriptors, launch, status.
// There is no CPU path here: without an sm_100 device every compute entry point fails.
#include "b200_attention.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <string>

#include "attn_bwd_kernel.cuh"
#include "attn_fwd_kernel.cuh"

namespace {

thread_local std::string g_attn_error;
std::atomic<uint64_t> g_attn_launches{0};

int afail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_attn_error = buf;
  return code;
}

#define TXA_CUDA(expr)                                                                      \
  do {                                                                                      \
    cudaError_t e_ = (expr);                                                                \
    if (e_ != cudaSuccess)                                                                  \
      return afail(TXD_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_));           \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn attn_encode_fn() {
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

// [batch*heads, n_ctx, head_dim] viewed as a 3-D tensor; a box is 64 columns (128 bytes) x box_rows rows.
int encode_head_map(CUtensorMap *map, const void *ptr, bool bf16, long long heads_total, long long n_ctx, int head_dim,
                    int box_rows) {
  EncodeTiledFn enc = attn_encode_fn();
  if (!enc) return afail(TXD_ERR_NO_DEVICE, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(n_ctx),
                        static_cast<cuuint64_t>(heads_total)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_dim) * 2, static_cast<cuuint64_t>(n_ctx) * head_dim * 2};
  cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                   const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return afail(TXD_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
  return TXD_OK;
}

// The fp8 form's operands as byte tensors. Q and K: [batch*heads, n_ctx, head_dim] e5m2, a box is one 128-byte span
// x 128 rows (columns past head_dim are out of bounds and arrive as zeros). V: [batch*heads, head_dim, n_ctx]
// (transposed, as the reference lays V out for fp8), a box is 128 KV bytes x box_rows head-dimension rows.
int encode_byte_map(CUtensorMap *map, const void *ptr, long long heads_total, long long rows, long long cols, int box_rows) {
  EncodeTiledFn enc = attn_encode_fn();
  if (!enc) return afail(TXD_ERR_NO_DEVICE, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(heads_total)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows) * cols};
  cuuint32_t box[3] = {128, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return afail(TXD_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
  return TXD_OK;
}

// Head dimension the kernels are instantiated for. 16 and 32 run on the 64-wide kernels: the tensor maps describe
// the real tensors, every TMA box is 64 columns wide, and the columns past head_dim arrive as zeros (out-of-bounds
// fill) and are clipped from TMA stores. Zero columns of Q and K add nothing to Q K^T, zero columns of V and dO give
// zero columns of O, dQ, dK and dV that are never written.
int kernel_head_dim(int head_dim) { return head_dim <= 64 ? 64 : 128; }

// `fmt`: kind::f16 0 = f16, 1 = bf16; kind::f8f6f4 1 = e5m2
uint32_t attn_idesc(uint32_t fmt, bool b_mn_major, int n) {
  uint32_t d = 0;
  d |= 1u << 4;    // fp32 accumulator
  d |= fmt << 7;   // A type
  d |= fmt << 10;  // B type
  d |= (b_mn_major ? 1u : 0u) << 16;
  d |= static_cast<uint32_t>(n >> 3) << 17;
  d |= static_cast<uint32_t>(128 >> 4) << 24;
  return d;
}

constexpr int kBwdLanes = 4;

struct DeviceState {
  uint32_t *status = nullptr;
  bool attr_set = false;
  // host-buffer path
  cudaStream_t stream = nullptr, run_stream = nullptr, out_stream = nullptr;
  cudaEvent_t ev_in[8] = {}, ev_done[8] = {};
  bool events_made = false;
  void *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr;
  float *m = nullptr;
  size_t tensor_bytes = 0, m_bytes = 0;
  // backward: per-head workspace (scores, probabilities, their gradients) and the GEMM plans of the last shape
  // (kBwdLanes heads are in flight at a time, each on a stream, a workspace slice and a set of plans of its own)
  void *bwd_ws = nullptr;
  size_t bwd_ws_bytes = 0;
  tx_dot_plan *bwd_plan[4 * 4] = {};  // per lane: QK^T / dO V^T, P^T dO, dS K, dS^T Q
  cudaStream_t bwd_stream[4] = {};
  cudaEvent_t bwd_fork = nullptr, bwd_join[4] = {};
  int bwd_n = 0, bwd_d = 0, bwd_dtype = -1;
  float bwd_scale = 0.f;
  // forward as a composition of tt.dot GEMMs (head_dim 256): per lane Q K^T (fp32) and P V with the 1 / l row scale
  tx_dot_plan *fwd_plan[2 * 4] = {};
  int fwd_n = 0, fwd_d = 0, fwd_dtype = -1;
};
std::mutex g_state_mutex;
DeviceState g_state[64];

int device_state(DeviceState **out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return afail(TXD_ERR_NO_DEVICE, "no CUDA device");
  }
  std::lock_guard<std::mutex> lock(g_state_mutex);
  DeviceState &st = g_state[dev];
  if (!st.status) {
    cudaDeviceProp prop;
    TXA_CUDA(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
      return afail(TXD_ERR_NO_DEVICE, "device %d is sm_%d%d; these kernels are built for sm_100a only", dev, prop.major,
                   prop.minor);
    TXA_CUDA(cudaMalloc(&st.status, sizeof(uint32_t)));
    TXA_CUDA(cudaMemset(st.status, 0, sizeof(uint32_t)));
  }
  if (!st.attr_set) {
    TXA_CUDA(cudaFuncSetAttribute(txa::attn_fwd_kernel<0, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    TXA_CUDA(cudaFuncSetAttribute(txa::attn_fwd_kernel<0, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    TXA_CUDA(cudaFuncSetAttribute(txa::attn_fwd_kernel<1, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    TXA_CUDA(cudaFuncSetAttribute(txa::attn_fwd_kernel<1, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    TXA_CUDA(cudaFuncSetAttribute(txa::attn_fwd_kernel<2, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    TXA_CUDA(cudaFuncSetAttribute(txa::attn_fwd_kernel<2, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    TXA_CUDA(cudaFuncSetAttribute(txa::attn_bwd_kernel<false, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    TXA_CUDA(cudaFuncSetAttribute(txa::attn_bwd_kernel<true, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    TXA_CUDA(cudaFuncSetAttribute(txa::attn_bwd_kernel<false, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    TXA_CUDA(cudaFuncSetAttribute(txa::attn_bwd_kernel<true, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    TXA_CUDA(cudaFuncSetAttribute(txa::attn_bwd_dq_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    TXA_CUDA(cudaFuncSetAttribute(txa::attn_bwd_dq_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    st.attr_set = true;
  }
  *out = &st;
  return TXD_OK;
}

int validate(const tx_attn_problem *pr) {
  if (!pr) return afail(TXD_ERR_INVALID, "null problem");
  if (pr->batch < 1 || pr->heads < 1 || pr->n_ctx < 1) return afail(TXD_ERR_INVALID, "batch, heads and n_ctx must be >= 1");
  if (pr->head_dim != 16 && pr->head_dim != 32 && pr->head_dim != 64 && pr->head_dim != 128 && pr->head_dim != 256)
    return afail(TXD_ERR_UNSUPPORTED, "head_dim %d: the reference's 16, 32, 64, 128 and 256 are built", pr->head_dim);
  if (pr->dtype != TXD_F16 && pr->dtype != TXD_BF16 && pr->dtype != TXD_F8E5M2)
    return afail(TXD_ERR_UNSUPPORTED, "dtype must be f16, bf16 or (forward only) f8e5m2");
  if (pr->dtype == TXD_F8E5M2) {
    if (pr->head_dim == 256) return afail(TXD_ERR_UNSUPPORTED, "head_dim 256 is built for f16 and bf16 only");
    if (pr->n_ctx % 16 != 0)
      return afail(TXD_ERR_UNSUPPORTED, "f8e5m2: n_ctx %d must be a multiple of 16 (rows of the transposed V are TMA strides)", pr->n_ctx);
  }
  if (!(pr->sm_scale > 0.f)) return afail(TXD_ERR_INVALID, "sm_scale must be positive");
  if (static_cast<long long>(pr->batch) * pr->heads > 0x7fffffffLL / ((pr->n_ctx + 255) / 256))
    return afail(TXD_ERR_UNSUPPORTED, "too many (head, query tile) pairs for one grid");
  return TXD_OK;
}


// ---- backward: the element-wise steps between the GEMMs (reference _attn_bwd_preprocess,
// pass/LoopSplit/06-fused-attention.py:333-346, and the p / ds lines of _attn_bwd_dkdv :377-393 and _attn_bwd_dq :428-439) ------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// delta[row] = sum_d o[row, d] * do[row, d]: d / 8 lanes per row, 16-byte loads (d is 64 or 128)
template <typename T>
__global__ void attn_bwd_delta_kernel(const T *o, const T *d_o, float *delta, long long rows, int d) {
  const int lanes_per_row = d / 8;                 // 8 or 16
  const int rows_per_warp = 32 / lanes_per_row;    // 4 or 2
  const long long warp_id = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long row = warp_id * rows_per_warp + lane / lanes_per_row;
  float acc = 0.f;
  if (row < rows) {
    const long long off = row * d + (lane % lanes_per_row) * 8;
    const uint4 a = *reinterpret_cast<const uint4 *>(o + off);
    const uint4 b = *reinterpret_cast<const uint4 *>(d_o + off);
    const T *pa = reinterpret_cast<const T *>(&a);
    const T *pb = reinterpret_cast<const T *>(&b);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += to_f32(pa[i]) * to_f32(pb[i]);
  }
  for (int off = lanes_per_row / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (row < rows && lane % lanes_per_row == 0) delta[row] = acc;
}

// p[r, c] = exp2(s[r, c] * qk_scale - m[r]) (m already holds the row's log2-sum), zero above the diagonal
template <typename T>
__global__ void attn_bwd_p_kernel(const float *s, const float *m, T *p, int n, long long ld, float qk_scale, int causal) {
  const long long total = static_cast<long long>(n) * n;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / n), c = static_cast<int>(i - static_cast<long long>(r) * n);
    float v = exp2f(fmaf(s[r * ld + c], qk_scale, -m[r]));
    if (causal && c > r) v = 0.f;
    p[r * ld + c] = from_f32<T>(v);
  }
}

// ds[r, c] = p[r, c] * (dp[r, c] - delta[r]), written over p
template <typename T>
__global__ void attn_bwd_ds_kernel(T *p, const float *dp, const float *delta, int n, long long ld) {
  const long long total = static_cast<long long>(n) * n;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / n), c = static_cast<int>(i - static_cast<long long>(r) * n);
    const float v = to_f32(p[r * ld + c]) * (dp[r * ld + c] - delta[r]);
    p[r * ld + c] = from_f32<T>(v);
  }
}

template <typename T>
int attn_bwd_typed(const tx_attn_problem *pr, DeviceState *st, const T *q, const T *k, const T *v, const T *o, const T *d_o,
                   const float *m, T *dq, T *dk, T *dv, cudaStream_t stream) {
  const int n = pr->n_ctx, d = pr->head_dim;
  const long long ld = (n + 7) / 8 * 8;
  const long long heads_total = static_cast<long long>(pr->batch) * pr->heads;
  const size_t lane_bytes = static_cast<size_t>(n) * ld * (4 + 4 + sizeof(T));
  char *ws = static_cast<char *>(st->bwd_ws);
  float *delta = reinterpret_cast<float *>(ws + kBwdLanes * lane_bytes);
  const float qk_scale = pr->sm_scale * 1.44269504f;
  const long long rows = heads_total * n;
  attn_bwd_delta_kernel<T><<<static_cast<unsigned>((rows * (d / 8) + 255) / 256), 256, 0, stream>>>(o, d_o, delta, rows, d);
  TXA_CUDA(cudaGetLastError());
  // heads are independent: kBwdLanes of them are in flight at a time, so that their small kernels fill the GPU
  TXA_CUDA(cudaEventRecord(st->bwd_fork, stream));
  for (int l = 0; l < kBwdLanes; ++l) TXA_CUDA(cudaStreamWaitEvent(st->bwd_stream[l], st->bwd_fork, 0));
  const unsigned ew_grid = 148 * 4;
  for (long long h = 0; h < heads_total; ++h) {
    const int l = static_cast<int>(h % kBwdLanes);
    cudaStream_t ls = st->bwd_stream[l];
    tx_dot_plan **plan = &st->bwd_plan[4 * l];
    float *s_buf = reinterpret_cast<float *>(ws + l * lane_bytes);
    float *dp_buf = s_buf + static_cast<size_t>(n) * ld;
    T *p_buf = reinterpret_cast<T *>(dp_buf + static_cast<size_t>(n) * ld);
    const size_t off = static_cast<size_t>(h) * n * d;
    int rc;
    // S = Q K^T and dP = dO V^T (fp32)
    if ((rc = tx_dot_run(plan[0], q + off, k + off, s_buf, nullptr, nullptr, ls))) return rc;
    if ((rc = tx_dot_run(plan[0], d_o + off, v + off, dp_buf, nullptr, nullptr, ls))) return rc;
    attn_bwd_p_kernel<T><<<ew_grid, 256, 0, ls>>>(s_buf, m + h * n, p_buf, n, ld, qk_scale, pr->causal);
    // dV = P^T dO
    if ((rc = tx_dot_run(plan[1], p_buf, d_o + off, dv + off, nullptr, nullptr, ls))) return rc;
    attn_bwd_ds_kernel<T><<<ew_grid, 256, 0, ls>>>(p_buf, dp_buf, delta + h * n, n, ld);
    // dQ = sm_scale dS K, dK = sm_scale dS^T Q
    if ((rc = tx_dot_run(plan[2], p_buf, k + off, dq + off, nullptr, nullptr, ls))) return rc;
    if ((rc = tx_dot_run(plan[3], p_buf, q + off, dk + off, nullptr, nullptr, ls))) return rc;
  }
  for (int l = 0; l < kBwdLanes; ++l) {
    TXA_CUDA(cudaEventRecord(st->bwd_join[l], st->bwd_stream[l]));
    TXA_CUDA(cudaStreamWaitEvent(stream, st->bwd_join[l], 0));
  }
  TXA_CUDA(cudaGetLastError());
  g_attn_launches.fetch_add(static_cast<uint64_t>(1 + 2 * heads_total));
  return TXD_OK;
}


// The lanes of the GEMM compositions: kBwdLanes heads in flight, each on a stream of its own.
int ensure_lanes(DeviceState *st) {
  if (st->bwd_fork) return TXD_OK;
  TXA_CUDA(cudaEventCreateWithFlags(&st->bwd_fork, cudaEventDisableTiming));
  for (int l = 0; l < kBwdLanes; ++l) {
    TXA_CUDA(cudaStreamCreateWithFlags(&st->bwd_stream[l], cudaStreamNonBlocking));
    TXA_CUDA(cudaEventCreateWithFlags(&st->bwd_join[l], cudaEventDisableTiming));
  }
  return TXD_OK;
}

// One row of base-2 softmax over fp32 scores, as the reference's forward defines it (06-fused-attention.py:59-89,
// 236-240): m = max_c s[c] * qk_scale over the visible columns, p[c] = exp2(s[c] * qk_scale - m) rounded to the input
// type for the second dot, l = sum of the unrounded p, M = m + log2(l); the division by l is left to the P V GEMM's
// row scale. One block per row.
template <typename T>
__global__ void attn_fwd_softmax_rows_kernel(const float *s, T *p, float *m_out, float *inv_l, int n, long long ld,
                                             float qk_scale, int causal) {
  const int r = blockIdx.x;
  const int visible = causal ? r + 1 : n;
  const float *row = s + static_cast<long long>(r) * ld;
  __shared__ float red[32];
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < visible; c += blockDim.x) mx = fmaxf(mx, row[c] * qk_scale);
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
  for (int w = 1; w < static_cast<int>(blockDim.x >> 5); ++w) mx = fmaxf(mx, red[w]);
  __syncthreads();
  float sum = 0.f;
  T *prow = p + static_cast<long long>(r) * ld;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float e = c < visible ? exp2f(fmaf(row[c], qk_scale, -mx)) : 0.f;
    sum += e;
    prow[c] = from_f32<T>(e);
  }
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    float l = 0.f;
    for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) l += red[w];
    m_out[r] = mx + log2f(l);
    inv_l[r] = 1.0f / l;
  }
}

// Forward for head dimensions the fused kernel has no tensor-memory plan for (256: two 256-column O accumulators and
// two S tiles do not fit 512 TMEM columns): per head S = Q K^T by the tt.dot kernel (fp32), the row softmax above, and
// O = (P V) / l by the tt.dot kernel with its fused row scale. Scores travel through global memory, so this is the slow
// form; it exists so that the reference's whole HEAD_DIM list runs.
template <typename T>
int attn_fwd_composed(const tx_attn_problem *pr, DeviceState *st, const T *q, const T *k, const T *v, T *out, float *m_out,
                      cudaStream_t stream) {
  const int n = pr->n_ctx, d = pr->head_dim;
  const long long ld = (n + 7) / 8 * 8;
  const long long heads_total = static_cast<long long>(pr->batch) * pr->heads;
  // scores (fp32), probabilities (input type), 1 / l per row; every lane starts on a 256-byte boundary
  const size_t lane_bytes = (static_cast<size_t>(n) * ld * (4 + sizeof(T)) + static_cast<size_t>(n) * sizeof(float) + 255) / 256 * 256;
  int rc;
  {
    std::lock_guard<std::mutex> lock(g_state_mutex);
    const size_t need = kBwdLanes * lane_bytes + 256;
    if (st->bwd_ws_bytes < need) {
      if (st->bwd_ws) cudaFree(st->bwd_ws);
      st->bwd_ws = nullptr;
      st->bwd_ws_bytes = 0;
      TXA_CUDA(cudaMalloc(&st->bwd_ws, need));
      st->bwd_ws_bytes = need;
    }
    if ((rc = ensure_lanes(st))) return rc;
    if (st->fwd_n != n || st->fwd_d != d || st->fwd_dtype != pr->dtype) {
      for (tx_dot_plan *&p : st->fwd_plan) {
        if (p) tx_dot_plan_destroy(p);
        p = nullptr;
      }
      for (int l = 0; l < kBwdLanes; ++l) {
        tx_dot_problem g = {};
        // scores [n, n] = Q [n, d] x K^T (K is a row-major [n, d] tensor read transposed), fp32
        g.m = n; g.n = n; g.k = d; g.ab_dtype = pr->dtype; g.out_dtype = TXD_F32;
        g.a_layout = TXD_ROW_MAJOR; g.b_layout = TXD_COL_MAJOR; g.lda = d; g.ldb = d; g.ldc = ld; g.alpha = 1.0f;
        if ((rc = tx_dot_plan_create(&g, nullptr, &st->fwd_plan[2 * l]))) return afail(rc, "forward plan 0: %s", tx_dot_last_error());
        // O [n, d] = (P [n, n] x V [n, d]) * (1 / l)[row]
        g.m = n; g.n = d; g.k = n; g.out_dtype = pr->dtype; g.b_layout = TXD_ROW_MAJOR; g.lda = ld; g.ldb = d; g.ldc = d;
        g.has_row_scale = 1;
        if ((rc = tx_dot_plan_create(&g, nullptr, &st->fwd_plan[2 * l + 1]))) return afail(rc, "forward plan 1: %s", tx_dot_last_error());
      }
      st->fwd_n = n; st->fwd_d = d; st->fwd_dtype = pr->dtype;
    }
  }
  char *ws = static_cast<char *>(st->bwd_ws);
  const float qk_scale = pr->sm_scale * 1.44269504f;
  TXA_CUDA(cudaEventRecord(st->bwd_fork, stream));
  for (int l = 0; l < kBwdLanes; ++l) TXA_CUDA(cudaStreamWaitEvent(st->bwd_stream[l], st->bwd_fork, 0));
  for (long long h = 0; h < heads_total; ++h) {
    const int l = static_cast<int>(h % kBwdLanes);
    cudaStream_t ls = st->bwd_stream[l];
    float *s_buf = reinterpret_cast<float *>(ws + l * lane_bytes);
    T *p_buf = reinterpret_cast<T *>(s_buf + static_cast<size_t>(n) * ld);
    float *inv_l = reinterpret_cast<float *>(p_buf + static_cast<size_t>(n) * ld);
    const size_t off = static_cast<size_t>(h) * n * d;
    if ((rc = tx_dot_run(st->fwd_plan[2 * l], q + off, k + off, s_buf, nullptr, nullptr, ls))) return afail(rc, "%s", tx_dot_last_error());
    attn_fwd_softmax_rows_kernel<T><<<n, 256, 0, ls>>>(s_buf, p_buf, m_out + h * n, inv_l, n, ld, qk_scale, pr->causal ? 1 : 0);
    if ((rc = tx_dot_run(st->fwd_plan[2 * l + 1], p_buf, v + off, out + off, inv_l, nullptr, ls))) return afail(rc, "%s", tx_dot_last_error());
  }
  for (int l = 0; l < kBwdLanes; ++l) {
    TXA_CUDA(cudaEventRecord(st->bwd_join[l], st->bwd_stream[l]));
    TXA_CUDA(cudaStreamWaitEvent(stream, st->bwd_join[l], 0));
  }
  TXA_CUDA(cudaGetLastError());
  g_attn_launches.fetch_add(static_cast<uint64_t>(3 * heads_total));
  return TXD_OK;
}

// dq = cast(sm_scale * dq_acc)
template <typename T>
__global__ void attn_bwd_dq_convert_kernel(const float *acc, T *dq, long long rows, int head_dim, float sm_scale) {
  // acc is [rows, 64] fp32, dq [rows, head_dim] (head_dim <= 64: the accumulator's other columns are zero fill)
  const long long count = rows * head_dim;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / head_dim;
    const int c = static_cast<int>(i - r * head_dim);
    dq[i] = from_f32<T>(acc[r * 64 + c] * sm_scale);
  }
}

// The fused backward (attn_bwd_kernel.cuh) between the delta pre-pass and, at head_dim 64, the dq conversion;
// at head_dim 128 a second kernel computes dq.
template <typename T>
int attn_bwd_fused(const tx_attn_problem *pr, DeviceState *st, const T *q, const T *k, const T *v, const T *o, const T *d_o,
                   const float *m, T *dq, T *dk, T *dv, cudaStream_t stream) {
  const bool bf16 = pr->dtype == TXD_BF16;
  const int hd = pr->head_dim;            // columns of the tensors
  const int d = kernel_head_dim(hd);      // columns the kernels work on (the rest is zero fill)
  const long long heads_total = static_cast<long long>(pr->batch) * pr->heads;
  const long long rows = heads_total * pr->n_ctx;
  float *delta = static_cast<float *>(st->bwd_ws);
  float *dq_acc = delta + ((rows + 63) / 64) * 64;
  attn_bwd_delta_kernel<T><<<static_cast<unsigned>((rows * (hd / 8) + 255) / 256), 256, 0, stream>>>(o, d_o, delta, rows, hd);
  TXA_CUDA(cudaGetLastError());
  if (d == 64) TXA_CUDA(cudaMemsetAsync(dq_acc, 0, static_cast<size_t>(rows) * 64 * sizeof(float), stream));
  unsigned long long wait_limit_ns = 2000ull * 1000 * 1000;
  if (const char *e = getenv("TXD_WAIT_LIMIT_MS")) {
    const long ms = atol(e);
    if (ms > 0) wait_limit_ns = static_cast<unsigned long long>(ms) * 1000 * 1000;
  }
  txa::AttnBwdParams prm = {};
  int rc;
  if ((rc = encode_head_map(&prm.tmap_q, q, bf16, heads_total, pr->n_ctx, hd, 128))) return rc;
  if ((rc = encode_head_map(&prm.tmap_k, k, bf16, heads_total, pr->n_ctx, hd, 128))) return rc;
  if ((rc = encode_head_map(&prm.tmap_v, v, bf16, heads_total, pr->n_ctx, hd, 128))) return rc;
  if ((rc = encode_head_map(&prm.tmap_do, d_o, bf16, heads_total, pr->n_ctx, hd, 128))) return rc;
  if (d == 64) {
    // the fp32 dq accumulator as a 3-D tensor {64, n_ctx, heads}: boxes of 32 columns (128 bytes) x 32 rows
    EncodeTiledFn enc = attn_encode_fn();
    if (!enc) return afail(TXD_ERR_NO_DEVICE, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(pr->n_ctx), static_cast<cuuint64_t>(heads_total)};
    cuuint64_t strides[2] = {64 * sizeof(float), static_cast<cuuint64_t>(pr->n_ctx) * 64 * sizeof(float)};
    cuuint32_t box[3] = {32, 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(&prm.tmap_dq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, dq_acc, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return afail(TXD_ERR_CUDA, "cuTensorMapEncodeTiled (dq accumulator) failed with code %d", static_cast<int>(r));
  }
  prm.m = m;
  prm.delta = delta;
  prm.dq_acc = dq_acc;
  prm.dk = dk;
  prm.dv = dv;
  prm.status = st->status;
  prm.wait_limit_ns = wait_limit_ns;
  if (const char *e = getenv("TXD_INJECT_STALL")) prm.inject_stall = atoi(e) != 0;
  prm.qk_scale = pr->sm_scale * 1.44269504f;
  prm.sm_scale = pr->sm_scale;
  prm.n_ctx = pr->n_ctx;
  prm.head_dim = hd;
  prm.heads_total = static_cast<int32_t>(heads_total);
  prm.kv_blocks = (pr->n_ctx + 127) / 128;
  prm.causal = pr->causal ? 1 : 0;
  prm.idesc_st = attn_idesc(bf16, false, 128);
  prm.idesc_acc = attn_idesc(bf16, true, d);
  prm.idesc_dq = attn_idesc(bf16, true, 64) | (1u << 15);  // A operand MN-major as well
  const size_t tile = static_cast<size_t>(128) * d * 2;
  const size_t stages = d == 64 ? txa::kBwdStages : 1;
  const size_t smem = 2 * tile + stages * 2 * tile + 2 * txa::kPBytes +
                      (d == 64 ? txa::kBwdComputeWarps * txa::kDqSlabBytes : 0) + sizeof(txa::AttnBwdCtl) + 1024;
  const unsigned grid = static_cast<unsigned>(heads_total * prm.kv_blocks);
  if (d == 64) {
    if (bf16) txa::attn_bwd_kernel<true, 64><<<grid, txa::kBwdThreads, smem, stream>>>(prm);
    else txa::attn_bwd_kernel<false, 64><<<grid, txa::kBwdThreads, smem, stream>>>(prm);
    TXA_CUDA(cudaGetLastError());
    attn_bwd_dq_convert_kernel<T><<<148 * 8, 256, 0, stream>>>(dq_acc, dq, rows, hd, pr->sm_scale);
    TXA_CUDA(cudaGetLastError());
  } else {
    if (bf16) txa::attn_bwd_kernel<true, 128><<<grid, txa::kBwdThreads, smem, stream>>>(prm);
    else txa::attn_bwd_kernel<false, 128><<<grid, txa::kBwdThreads, smem, stream>>>(prm);
    TXA_CUDA(cudaGetLastError());
    txa::AttnBwdDqParams dqp = {};
    dqp.tmap_q = prm.tmap_q;
    dqp.tmap_k = prm.tmap_k;
    dqp.tmap_v = prm.tmap_v;
    dqp.tmap_do = prm.tmap_do;
    dqp.m = m;
    dqp.delta = delta;
    dqp.dq = dq;
    dqp.status = st->status;
    dqp.wait_limit_ns = wait_limit_ns;
    dqp.qk_scale = prm.qk_scale;
    dqp.sm_scale = pr->sm_scale;
    dqp.n_ctx = pr->n_ctx;
    dqp.heads_total = prm.heads_total;
    dqp.q_blocks = prm.kv_blocks;
    dqp.causal = prm.causal;
    dqp.idesc_s = attn_idesc(bf16, false, 128);
    dqp.idesc_dq = attn_idesc(bf16, true, 128);
    const size_t dq_smem = 2 * tile + 2 * 2 * tile + txa::kPBytes + sizeof(txa::AttnBwdDqCtl) + 1024;
    if (bf16) txa::attn_bwd_dq_kernel<true><<<grid, txa::kBwdThreads, dq_smem, stream>>>(dqp);
    else txa::attn_bwd_dq_kernel<false><<<grid, txa::kBwdThreads, dq_smem, stream>>>(dqp);
    TXA_CUDA(cudaGetLastError());
  }
  g_attn_launches.fetch_add(3);
  return TXD_OK;
}

}  // namespace

extern "C" {

const char *tx_attn_last_error(void) { return g_attn_error.c_str(); }
uint64_t tx_attn_kernel_launches(void) { return g_attn_launches.load(); }

double tx_attn_flops(const tx_attn_problem *pr) {
  if (!pr) return 0.0;
  double f = 4.0 * pr->batch * pr->heads * static_cast<double>(pr->n_ctx) * pr->n_ctx * pr->head_dim;
  return pr->causal ? 0.5 * f : f;
}

int tx_attn_fwd(const tx_attn_problem *pr, const void *q, const void *k, const void *v, void *out, float *m,
                void *stream_v) {
  int rc = validate(pr);
  if (rc) return rc;
  if (!q || !k || !v || !out) return afail(TXD_ERR_INVALID, "null tensor pointer");
  DeviceState *st = nullptr;
  rc = device_state(&st);
  if (rc) return rc;
  const bool bf16 = pr->dtype == TXD_BF16;
  const bool f8 = pr->dtype == TXD_F8E5M2;
  const long long heads_total = static_cast<long long>(pr->batch) * pr->heads;
  const int kd = kernel_head_dim(pr->head_dim);
  txa::AttnParams prm = {};
  if (f8) {
    if ((rc = encode_byte_map(&prm.tmap_q, q, heads_total, pr->n_ctx, pr->head_dim, 128))) return rc;
    if ((rc = encode_byte_map(&prm.tmap_k, k, heads_total, pr->n_ctx, pr->head_dim, 128))) return rc;
    if ((rc = encode_byte_map(&prm.tmap_v, v, heads_total, pr->head_dim, pr->n_ctx, kd))) return rc;
    prm.out = out;
  } else {
    if ((rc = encode_head_map(&prm.tmap_q, q, bf16, heads_total, pr->n_ctx, pr->head_dim, 128))) return rc;
    if ((rc = encode_head_map(&prm.tmap_k, k, bf16, heads_total, pr->n_ctx, pr->head_dim, 128))) return rc;
    if ((rc = encode_head_map(&prm.tmap_v, v, bf16, heads_total, pr->n_ctx, pr->head_dim, 128))) return rc;
    if ((rc = encode_head_map(&prm.tmap_o, out, bf16, heads_total, pr->n_ctx, pr->head_dim, 32))) return rc;
  }
  prm.m_out = m;
  prm.status = st->status;
  prm.wait_limit_ns = 2000ull * 1000 * 1000;
  if (const char *e = getenv("TXD_WAIT_LIMIT_MS")) {
    const long ms = atol(e);
    if (ms > 0) prm.wait_limit_ns = static_cast<unsigned long long>(ms) * 1000 * 1000;
  }
  if (const char *e = getenv("TXD_INJECT_STALL")) prm.inject_stall = atoi(e) != 0;
  prm.qk_scale = pr->sm_scale * 1.44269504f;  // 1 / ln 2, as the reference writes it
  prm.n_ctx = pr->n_ctx;
  prm.head_dim = pr->head_dim;
  prm.heads_total = static_cast<int32_t>(heads_total);
  prm.q_tiles = (pr->n_ctx + 255) / 256;
  {
    // heads whose K and V (2 tensors x n_ctx x head_dim x 2 bytes each) fit in 48 MB of the 126 MB L2 together
    const long long kv_bytes = (f8 ? 2LL : 4LL) * pr->n_ctx * pr->head_dim;
    long long grp = (48LL << 20) / (kv_bytes > 0 ? kv_bytes : 1);
    if (grp < 1) grp = 1;
    if (grp > heads_total) grp = heads_total;
    const long long groups = (heads_total + grp - 1) / grp;
    grp = (heads_total + groups - 1) / groups;  // equal groups: the last one is not a short tail of heavy tiles
    prm.head_group = static_cast<int32_t>(grp);
  }
  prm.causal = pr->causal ? 1 : 0;
  prm.is_bf16 = bf16 ? 1 : 0;
  prm.kv_stages = (kd == 128 && !f8) ? 3 : 6;  // what the kernel templates use; shared memory is sized from it
  prm.idesc_qk = attn_idesc(f8 || bf16 ? 1u : 0u, false, 128);
  prm.idesc_pv = attn_idesc(f8 || bf16 ? 1u : 0u, !f8, kd);  // fp8: V arrives transposed, K-major
  if (!m) {
    // the kernel always writes M; give it a scratch row vector when the caller does not want it
    std::lock_guard<std::mutex> lock(g_state_mutex);
    const size_t need = static_cast<size_t>(heads_total) * pr->n_ctx * sizeof(float);
    if (st->m_bytes < need) {
      if (st->m) cudaFree(st->m);
      st->m = nullptr;
      st->m_bytes = 0;
      TXA_CUDA(cudaMalloc(&st->m, need));
      st->m_bytes = need;
    }
    prm.m_out = st->m;
  }
  if (pr->head_dim == 256) {
    cudaStream_t cs = static_cast<cudaStream_t>(stream_v);
    if (bf16)
      return attn_fwd_composed<__nv_bfloat16>(pr, st, static_cast<const __nv_bfloat16 *>(q), static_cast<const __nv_bfloat16 *>(k),
                                              static_cast<const __nv_bfloat16 *>(v), static_cast<__nv_bfloat16 *>(out), prm.m_out, cs);
    return attn_fwd_composed<__half>(pr, st, static_cast<const __half *>(q), static_cast<const __half *>(k),
                                     static_cast<const __half *>(v), static_cast<__half *>(out), prm.m_out, cs);
  }
  const size_t tile_bytes = f8 ? static_cast<size_t>(txa::kAtomBytes) : static_cast<size_t>(128) * kd * 2;
  const size_t p_bytes = f8 ? static_cast<size_t>(txa::kAtomBytes) : static_cast<size_t>(txa::kPBytes);
  const size_t smem = 2 * tile_bytes + 2 * p_bytes + prm.kv_stages * tile_bytes + sizeof(txa::AttnCtl) + 1024;
  const unsigned grid = static_cast<unsigned>(heads_total * prm.q_tiles);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (f8 && kd == 64) txa::attn_fwd_kernel<2, 64><<<grid, txa::kAttnThreads, smem, stream>>>(prm);
  else if (f8) txa::attn_fwd_kernel<2, 128><<<grid, txa::kAttnThreads, smem, stream>>>(prm);
  else if (bf16 && kd == 64) txa::attn_fwd_kernel<1, 64><<<grid, txa::kAttnThreads, smem, stream>>>(prm);
  else if (bf16) txa::attn_fwd_kernel<1, 128><<<grid, txa::kAttnThreads, smem, stream>>>(prm);
  else if (kd == 64) txa::attn_fwd_kernel<0, 64><<<grid, txa::kAttnThreads, smem, stream>>>(prm);
  else txa::attn_fwd_kernel<0, 128><<<grid, txa::kAttnThreads, smem, stream>>>(prm);
  TXA_CUDA(cudaGetLastError());
  g_attn_launches.fetch_add(1);
  return TXD_OK;
}

int tx_attn_check(void *stream_v) {
  DeviceState *st = nullptr;
  int rc = device_state(&st);
  if (rc) return rc;
  TXA_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream_v)));
  uint32_t status = 0;
  TXA_CUDA(cudaMemcpy(&status, st->status, sizeof status, cudaMemcpyDeviceToHost));
  if (status != 0) {
    cudaMemset(st->status, 0, sizeof status);
    return afail(TXD_ERR_DEVICE_TIMEOUT, "a bounded wait inside the attention kernel ran out (role code %u)", status);
  }
  for (tx_dot_plan *p : st->bwd_plan)
    if (p && (rc = tx_dot_plan_check(p, stream_v))) return afail(rc, "backward GEMM: %s", tx_dot_last_error());
  return TXD_OK;
}

int tx_attn_fwd_host(const tx_attn_problem *pr, const void *q, const void *k, const void *v, void *out, float *m) {
  int rc = validate(pr);
  if (rc) return rc;
  if (!q || !k || !v || !out) return afail(TXD_ERR_INVALID, "null host pointer");
  DeviceState *st = nullptr;
  rc = device_state(&st);
  if (rc) return rc;
  const size_t heads_total = static_cast<size_t>(pr->batch) * pr->heads;
  const size_t es = pr->dtype == TXD_F8E5M2 ? 1 : 2;
  const size_t bytes = heads_total * pr->n_ctx * pr->head_dim * es;
  const size_t m_bytes = heads_total * pr->n_ctx * sizeof(float);
  {
    std::lock_guard<std::mutex> lock(g_state_mutex);
    if (!st->stream) TXA_CUDA(cudaStreamCreateWithFlags(&st->stream, cudaStreamNonBlocking));
    if (st->tensor_bytes < bytes) {
      void **bufs[4] = {&st->q, &st->k, &st->v, &st->o};
      for (void **b : bufs) {
        if (*b) cudaFree(*b);
        *b = nullptr;
      }
      st->tensor_bytes = 0;
      for (void **b : bufs) TXA_CUDA(cudaMalloc(b, bytes));
      st->tensor_bytes = bytes;
    }
    if (st->m_bytes < m_bytes) {
      if (st->m) cudaFree(st->m);
      st->m = nullptr;
      st->m_bytes = 0;
      TXA_CUDA(cudaMalloc(&st->m, m_bytes));
      st->m_bytes = m_bytes;
    }
  }
  cudaStream_t s = st->stream;
  // (batch, head) pairs are independent and contiguous in memory: above 32 MB they travel in up to 8 groups, and
  // group g+1 is copied in while group g runs and group g-1 is copied out (three streams).
  const size_t groups = (4 * bytes >= (32u << 20) && heads_total >= 2) ? (heads_total < 8 ? heads_total : 8) : 1;
  if (groups == 1) {
    TXA_CUDA(cudaMemcpyAsync(st->q, q, bytes, cudaMemcpyHostToDevice, s));
    TXA_CUDA(cudaMemcpyAsync(st->k, k, bytes, cudaMemcpyHostToDevice, s));
    TXA_CUDA(cudaMemcpyAsync(st->v, v, bytes, cudaMemcpyHostToDevice, s));
    rc = tx_attn_fwd(pr, st->q, st->k, st->v, st->o, st->m, s);
    if (rc) return rc;
    TXA_CUDA(cudaMemcpyAsync(out, st->o, bytes, cudaMemcpyDeviceToHost, s));
    if (m) TXA_CUDA(cudaMemcpyAsync(m, st->m, m_bytes, cudaMemcpyDeviceToHost, s));
    return tx_attn_check(s);
  }
  {
    std::lock_guard<std::mutex> lock(g_state_mutex);
    if (!st->run_stream) {
      TXA_CUDA(cudaStreamCreateWithFlags(&st->run_stream, cudaStreamNonBlocking));
      TXA_CUDA(cudaStreamCreateWithFlags(&st->out_stream, cudaStreamNonBlocking));
    }
    if (!st->events_made) {
      for (auto &e : st->ev_in) TXA_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
      for (auto &e : st->ev_done) TXA_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
      st->events_made = true;
    }
  }
  const size_t head_bytes = static_cast<size_t>(pr->n_ctx) * pr->head_dim * es;
  const size_t head_m_bytes = static_cast<size_t>(pr->n_ctx) * sizeof(float);
  for (size_t g = 0; g < groups; ++g) {
    const size_t h0 = heads_total * g / groups, h1 = heads_total * (g + 1) / groups;
    const size_t off = h0 * head_bytes, len = (h1 - h0) * head_bytes;
    auto at = [&](const void *base) { return static_cast<const char *>(base) + off; };
    auto dev_at = [&](void *base) { return static_cast<char *>(base) + off; };
    TXA_CUDA(cudaMemcpyAsync(dev_at(st->q), at(q), len, cudaMemcpyHostToDevice, s));
    TXA_CUDA(cudaMemcpyAsync(dev_at(st->k), at(k), len, cudaMemcpyHostToDevice, s));
    TXA_CUDA(cudaMemcpyAsync(dev_at(st->v), at(v), len, cudaMemcpyHostToDevice, s));
    TXA_CUDA(cudaEventRecord(st->ev_in[g], s));
    TXA_CUDA(cudaStreamWaitEvent(st->run_stream, st->ev_in[g], 0));
    tx_attn_problem sub = *pr;
    sub.batch = 1;
    sub.heads = static_cast<int32_t>(h1 - h0);
    float *m_dev = st->m + h0 * pr->n_ctx;
    rc = tx_attn_fwd(&sub, dev_at(st->q), dev_at(st->k), dev_at(st->v), dev_at(st->o), m_dev, st->run_stream);
    if (rc) return rc;
    TXA_CUDA(cudaEventRecord(st->ev_done[g], st->run_stream));
    TXA_CUDA(cudaStreamWaitEvent(st->out_stream, st->ev_done[g], 0));
    TXA_CUDA(cudaMemcpyAsync(static_cast<char *>(out) + off, dev_at(st->o), len, cudaMemcpyDeviceToHost, st->out_stream));
    if (m)
      TXA_CUDA(cudaMemcpyAsync(reinterpret_cast<char *>(m) + h0 * head_m_bytes, m_dev, (h1 - h0) * head_m_bytes,
                               cudaMemcpyDeviceToHost, st->out_stream));
  }
  TXA_CUDA(cudaStreamSynchronize(st->out_stream));
  return tx_attn_check(st->run_stream);
}

int tx_attn_bwd(const tx_attn_problem *pr, const void *q, const void *k, const void *v, const void *o, const void *d_o,
                const float *m, void *dq, void *dk, void *dv, void *stream_v) {
  int rc = validate(pr);
  if (rc) return rc;
  if (pr->dtype == TXD_F8E5M2)
    return afail(TXD_ERR_UNSUPPORTED, "the backward takes f16 or bf16 (the reference's backward has no fp8 form)");
  if (!q || !k || !v || !o || !d_o || !m || !dq || !dk || !dv) return afail(TXD_ERR_INVALID, "null tensor pointer");
  DeviceState *st = nullptr;
  rc = device_state(&st);
  if (rc) return rc;
  const int n = pr->n_ctx, d = pr->head_dim;
  const long long ld = (n + 7) / 8 * 8;
  const char *force_unfused = getenv("TXA_BWD_UNFUSED");
  // head_dim 256 has no fused kernel (tensor-memory plan): it takes the composition of tt.dot GEMMs below
  if (d != 256 && !(force_unfused && atoi(force_unfused) != 0)) {
    const size_t rows = static_cast<size_t>(pr->batch) * pr->heads * n;
    const size_t need = ((rows + 63) / 64) * 64 * sizeof(float) + (d <= 64 ? rows * 64 * sizeof(float) : 0) + 256;
    {
      std::lock_guard<std::mutex> lock(g_state_mutex);
      if (st->bwd_ws_bytes < need) {
        if (st->bwd_ws) cudaFree(st->bwd_ws);
        st->bwd_ws = nullptr;
        st->bwd_ws_bytes = 0;
        TXA_CUDA(cudaMalloc(&st->bwd_ws, need));
        st->bwd_ws_bytes = need;
      }
    }
    cudaStream_t fs = static_cast<cudaStream_t>(stream_v);
    if (pr->dtype == TXD_BF16)
      return attn_bwd_fused<__nv_bfloat16>(pr, st, static_cast<const __nv_bfloat16 *>(q), static_cast<const __nv_bfloat16 *>(k),
                                           static_cast<const __nv_bfloat16 *>(v), static_cast<const __nv_bfloat16 *>(o),
                                           static_cast<const __nv_bfloat16 *>(d_o), m, static_cast<__nv_bfloat16 *>(dq),
                                           static_cast<__nv_bfloat16 *>(dk), static_cast<__nv_bfloat16 *>(dv), fs);
    return attn_bwd_fused<__half>(pr, st, static_cast<const __half *>(q), static_cast<const __half *>(k),
                                  static_cast<const __half *>(v), static_cast<const __half *>(o), static_cast<const __half *>(d_o),
                                  m, static_cast<__half *>(dq), static_cast<__half *>(dk), static_cast<__half *>(dv), fs);
  }
  {
    std::lock_guard<std::mutex> lock(g_state_mutex);
    const size_t need = kBwdLanes * static_cast<size_t>(n) * ld * (4 + 4 + 2) +
                        static_cast<size_t>(pr->batch) * pr->heads * n * sizeof(float) + 256;
    if (st->bwd_ws_bytes < need) {
      if (st->bwd_ws) cudaFree(st->bwd_ws);
      st->bwd_ws = nullptr;
      st->bwd_ws_bytes = 0;
      TXA_CUDA(cudaMalloc(&st->bwd_ws, need));
      st->bwd_ws_bytes = need;
    }
    if ((rc = ensure_lanes(st))) return rc;
    if (st->bwd_n != n || st->bwd_d != d || st->bwd_dtype != pr->dtype || st->bwd_scale != pr->sm_scale) {
      for (tx_dot_plan *&p : st->bwd_plan) {
        if (p) tx_dot_plan_destroy(p);
        p = nullptr;
      }
      for (int l = 0; l < kBwdLanes; ++l) {
        tx_dot_plan **plan = &st->bwd_plan[4 * l];
        tx_dot_problem g = {};
        // [n, n] = [n, d] x [d, n]: scores and dP, fp32; the second operand is a row-major [n, d] tensor read transposed
        g.m = n; g.n = n; g.k = d; g.ab_dtype = pr->dtype; g.out_dtype = TXD_F32;
        g.a_layout = TXD_ROW_MAJOR; g.b_layout = TXD_COL_MAJOR; g.lda = d; g.ldb = d; g.ldc = ld; g.alpha = 1.0f;
        if ((rc = tx_dot_plan_create(&g, nullptr, &plan[0]))) return afail(rc, "backward plan 0: %s", tx_dot_last_error());
        // [n, d] = P^T [n, n] x dO [n, d]
        g.m = n; g.n = d; g.k = n; g.out_dtype = pr->dtype;
        g.a_layout = TXD_COL_MAJOR; g.b_layout = TXD_ROW_MAJOR; g.lda = ld; g.ldb = d; g.ldc = d; g.alpha = 1.0f;
        if ((rc = tx_dot_plan_create(&g, nullptr, &plan[1]))) return afail(rc, "backward plan 1: %s", tx_dot_last_error());
        // dQ = sm_scale dS K
        g.a_layout = TXD_ROW_MAJOR; g.alpha = pr->sm_scale;
        if ((rc = tx_dot_plan_create(&g, nullptr, &plan[2]))) return afail(rc, "backward plan 2: %s", tx_dot_last_error());
        // dK = sm_scale dS^T Q
        g.a_layout = TXD_COL_MAJOR;
        if ((rc = tx_dot_plan_create(&g, nullptr, &plan[3]))) return afail(rc, "backward plan 3: %s", tx_dot_last_error());
      }
      st->bwd_n = n; st->bwd_d = d; st->bwd_dtype = pr->dtype; st->bwd_scale = pr->sm_scale;
    }
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (pr->dtype == TXD_BF16)
    return attn_bwd_typed<__nv_bfloat16>(pr, st, static_cast<const __nv_bfloat16 *>(q), static_cast<const __nv_bfloat16 *>(k),
                                         static_cast<const __nv_bfloat16 *>(v), static_cast<const __nv_bfloat16 *>(o),
                                         static_cast<const __nv_bfloat16 *>(d_o), m, static_cast<__nv_bfloat16 *>(dq),
                                         static_cast<__nv_bfloat16 *>(dk), static_cast<__nv_bfloat16 *>(dv), stream);
  return attn_bwd_typed<__half>(pr, st, static_cast<const __half *>(q), static_cast<const __half *>(k),
                                static_cast<const __half *>(v), static_cast<const __half *>(o), static_cast<const __half *>(d_o), m,
                                static_cast<__half *>(dq), static_cast<__half *>(dk), static_cast<__half *>(dv), stream);
}

}  // extern "C"
