/* C-ABI of the fused attention forward kernel for sm_100a (B200).
 *
 * Replaces, for callers that bind a library instead of JIT-compiling Triton, the forward launch of the
 * reference's demo kernel: `_attn_fwd[grid](q, k, v, sm_scale, M, o, strides..., Z, H, N_CTX, HEAD_DIM,
 * BLOCK_M, BLOCK_N, CAUSAL)` in pass/LoopSplit/06-fused-attention.py:626-637 (kernel :164-240, inner loop
 * :43-90). Same operands and results: q, k, v, out are contiguous [batch, heads, n_ctx, head_dim] tensors
 * of one 16-bit type (or float8_e5m2, see `dtype` below); `m` receives, per query row, running max + log2(sum) in base 2 (:236,:239), which
 * the reference keeps for its backward pass.
 *
 * Plain pointers and sizes only; every function returns a tx_dot_status code (b200_dot.h) and
 * tx_attn_last_error() holds the text of this thread's last failure. There is no CPU path: without an
 * sm_100 device every compute entry point returns TXD_ERR_NO_DEVICE.
 */
#ifndef B200_ATTENTION_H_
#define B200_ATTENTION_H_

#include <stdint.h>

#include "b200_dot.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tx_attn_problem {
  int32_t batch, heads; /* Z, H of the reference launch                                             */
  int32_t n_ctx;        /* sequence length; any value >= 1 (the reference asks for multiples of BLOCK_M) */
  int32_t head_dim;     /* 16, 32, 64, 128 or 256 (the reference's list, :589). 64 and 128: fused     */
                        /* kernels; 16 and 32: the 64-wide kernels, zero-filled; 256: a composition of */
                        /* the tt.dot GEMM kernels around a row softmax (slow)                         */
  int32_t dtype;        /* TXD_F16 or TXD_BF16 for q, k, v and out; TXD_F8E5M2 for the forward only    */
                        /* (the reference's fp8 path, :81-82, :191, :774-779): q, k, out as above in    */
                        /* e5m2, v stored [batch, heads, head_dim, n_ctx] (n_ctx contiguous, as the      */
                        /* reference lays it out for fp8), P and out rounded to e5m2 (nearest even);     */
                        /* head_dim 16, 32, 64 or 128, n_ctx a multiple of 16                            */
  int32_t causal;       /* 0 / 1                                                                     */
  float sm_scale;       /* > 0; scores are scaled by sm_scale * log2(e) and exponentiated in base 2   */
  int32_t reserved[5];  /* zero                                                                      */
} tx_attn_problem;

/* Asynchronous launch on `stream` (a cudaStream_t); all pointers are device pointers, 16-byte aligned.
 * `m` may be NULL when the caller does not need it (the library then writes it to a per-device scratch vector, which the
 * first such call of a size allocates: make that call before capturing a CUDA graph). Launches of one device may come from
 * several host threads; the per-device scratch and workspaces are single buffers shared by every stream, so calls that use
 * them (m == NULL, tx_attn_bwd, tx_attn_fwd_host) must not overlap on one device: not from different threads, and not from
 * one thread on different streams either (two backward calls in flight would both accumulate into the one fp32 dq buffer).
 * Order such calls on one stream, or with events. */
TXD_API int tx_attn_fwd(const tx_attn_problem *problem, const void *q, const void *k, const void *v, void *out,
                        float *m, void *stream);

/* Synchronises `stream` and reports a bounded wait that ran out inside the kernel
 * (TXD_ERR_DEVICE_TIMEOUT) or a CUDA error. */
TXD_API int tx_attn_check(void *stream);

/* The same through host buffers: copies q, k, v to the device, runs, copies out (and m) back, synchronises. */
TXD_API int tx_attn_fwd_host(const tx_attn_problem *problem, const void *q, const void *k, const void *v, void *out,
                             float *m);

/* Backward of the same attention: dq, dk, dv from q, k, v, the forward's output `o` and row vector `m`, and the
 * gradient `d_o` of the output (reference `_attention.backward`, pass/LoopSplit/06-fused-attention.py:645-688: kernels
 * `_attn_bwd_preprocess` :333-346, `_attn_bwd_dkdv` :351-400, `_attn_bwd_dq` :404-448, `_attn_bwd` :451-577). All tensors
 * are contiguous [batch, heads, n_ctx, head_dim] device tensors of the problem's type, `m` is [batch, heads, n_ctx]
 * fp32. Same mathematics as the reference (P recomputed from the scores and `m`, delta = rowsum(o * d_o),
 * dS = P * (dP - delta), P and dS rounded to the input type before their dots). head_dim 64 runs one fused kernel (all
 * five dots per block pair on tensor memory, dq through fp32 reductions), head_dim 128 two (dk and dv; dq). Workspaces
 * (row sums, the fp32 dq accumulator) are kept per device. Asynchronous on `stream`; tx_attn_check reports its bounded waits too. */
TXD_API int tx_attn_bwd(const tx_attn_problem *problem, const void *q, const void *k, const void *v, const void *o,
                        const void *d_o, const float *m, void *dq, void *dk, void *dv, void *stream);

/* FLOPs of one forward call as the reference's benchmark counts them (:795-798): 4 * Z * H * N^2 * D, halved
 * when causal. */
TXD_API double tx_attn_flops(const tx_attn_problem *problem);

TXD_API uint64_t tx_attn_kernel_launches(void);
TXD_API const char *tx_attn_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* B200_ATTENTION_H_ */
