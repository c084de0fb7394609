/*
 * b200_dot.h — C-ABI of the `b200_dot` backend extension: the launch interface of the
 * hand-written sm_100a kernels that execute one `tt.dot` tile-GEMM K-loop
 * (main body + LoopSplit-peeled remainder, fp32 accumulate, fused scale/cast epilogue).
 *
 * What it replaces in the reference (triton-lang/triton-ext):
 *   - backend/CMakeLists.txt (0 bytes): the reference's `backend/` extension slot is empty; this
 *     library is what fills it.
 *   - The contraction itself is the `tl.dot` call sites of
 *     pass/LoopSplit/06-fused-attention.py:63,85,115,135 (fp32 accumulator created at :222) and the
 *     scale/cast epilogue idioms of :66,78,237,240 — in the reference they are lowered by upstream
 *     Triton's NVIDIA backend (GPU) or by Triton's interpreter (CPU, `create_dot`).
 *   - The main/tail split of the K loop is the loop pair produced by
 *     pass/LoopSplit/LoopSplit.cpp:179-193; here it is executed inside one kernel.
 *
 * Plain C, plain pointers and sizes; no torch or MLIR types cross this boundary.
 * Every entry point returns a tx_dot_status; tx_dot_last_error() gives the text for the calling thread.
 * There is no CPU fallback: without a CUDA device every compute entry point returns
 * TXD_ERR_NO_DEVICE.
 */
#ifndef B200_DOT_H
#define B200_DOT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define TXD_API
#else
#define TXD_API __attribute__((visibility("default")))
#endif

typedef enum tx_dot_status {
  TXD_OK = 0,
  TXD_ERR_INVALID = 1,        /* bad argument (null pointer, non-positive extent, misaligned pointer) */
  TXD_ERR_UNSUPPORTED = 2,    /* legal tt.dot, but outside what the kernels cover (see message) */
  TXD_ERR_CUDA = 3,           /* a CUDA runtime / driver call failed */
  TXD_ERR_DEVICE_TIMEOUT = 4, /* a bounded device-side wait ran out; output is undefined */
  TXD_ERR_NO_DEVICE = 5       /* no CUDA device / driver available */
} tx_dot_status;

/* Element types. Operands of one tt.dot share a type (Triton's semantic.dot rule). */
typedef enum tx_dot_dtype {
  TXD_F16 = 0,
  TXD_BF16 = 1,
  TXD_F8E4M3 = 2,
  TXD_F32 = 3, /* output only */
  TXD_F8E5M2 = 4
} tx_dot_dtype;

typedef enum tx_dot_layout {
  TXD_ROW_MAJOR = 0, /* A[m,k] at a[m*lda+k];  B[k,n] at b[k*ldb+n] */
  TXD_COL_MAJOR = 1  /* A[m,k] at a[k*lda+m];  B[k,n] at b[n*ldb+k] */
} tx_dot_layout;

typedef enum tx_dot_schedule {
  TXD_SCHED_AUTO = 0,
  TXD_SCHED_DATA_PARALLEL = 1, /* persistent CTAs, whole output tiles */
  TXD_SCHED_STREAM_K = 2,      /* persistent CTAs, equal shares of the (tile, k-block) space; partial
                                  tiles are combined through plan-owned scratch memory */
  TXD_SCHED_HYBRID = 3         /* whole tiles for every full wave of the grid, then the tiles of the last,
                                  partial wave cut into equal (tile, k-block) shares as in stream-K */
} tx_dot_schedule;

/* C[m,n] = cast( alpha * row_scale[m] * col_scale[n] * sum_k A[m,k]*B[k,n] ), fp32 accumulate.
 * C is always row-major with leading dimension ldc. */
typedef struct tx_dot_problem {
  int32_t m, n, k;
  int32_t ab_dtype;      /* tx_dot_dtype of A and B */
  int32_t out_dtype;     /* tx_dot_dtype of C: F16, BF16 or F32 */
  int32_t a_layout;      /* tx_dot_layout */
  int32_t b_layout;      /* tx_dot_layout */
  int32_t has_row_scale; /* run() takes a float[m] multiplied into row m  */
  int32_t has_col_scale; /* run() takes a float[n] multiplied into column n */
  int64_t lda, ldb, ldc; /* leading dimensions in elements */
  float alpha;           /* scalar scale of the accumulator (1.0f for a plain dot) */
} tx_dot_problem;

/* Kernel configuration. Zero in a field = let the arithmetic-intensity analysis choose. */
typedef struct tx_dot_config {
  int32_t block_n;       /* columns of C per tile: 16, 32, 64, 128 or 256 (the MMA's N extent), or 512 = the wide
                            pair tile: two 256-column MMA halves per K block sharing one stage of A (CTA pairs,
                            whole-tile schedule, one K atom per stage) */
  int32_t stages;        /* depth of the TMA shared-memory ring (2..12) */
  int32_t swap_ab;       /* 1 = compute C^T = B^T A^T (skinny m), 2 = never swap, 0 = auto */
  int32_t schedule;      /* tx_dot_schedule */
  int32_t group_m;       /* tile-raster group height (tiles) for L2 reuse */
  int32_t max_ctas;      /* cap on the persistent grid (0 = number of SMs) */
  int32_t k_split_point; /* LoopSplit mid point of the K loop in elements; 0 = floor(K/BK)*BK,
                            negative = split at 0 (the whole loop runs as the masked remainder).
                            Must not exceed floor(K/BK)*BK; a value inside a physical K block is
                            moved down to the block start. Iterations below it run unpredicated;
                            the rest run as the masked remainder. */
  int32_t cta_pair;      /* 1 = two-CTA clusters (tcgen05 cta_group::2, 256 x block_n tiles),
                            2 = single CTAs (128 x block_n tiles), 0 = auto */
  int32_t atoms;         /* 128-byte K atoms per pipeline stage: 1, 2 or 4 (block_k = atoms * 128 B) */
  int32_t reserved;
} tx_dot_config;

/* What a plan decided; filled by tx_dot_plan_query. */
typedef struct tx_dot_plan_info {
  int32_t block_m, block_n, block_k;
  int32_t stages;
  int32_t swap_ab;
  int32_t schedule;
  int32_t group_m;
  int32_t grid;            /* CTAs launched */
  int32_t k_main_iters;    /* unpredicated K iterations: [0, k_split_point) */
  int32_t k_tail_iters;    /* masked remainder iterations: [k_split_point, K) */
  int32_t k_tail_mmas;     /* tcgen05.mma instructions issued by the last remainder iteration */
  int32_t smem_bytes;      /* dynamic shared memory per CTA */
  int32_t tmem_columns;    /* TMEM columns allocated per CTA */
  int32_t cta_pair;        /* 1 when the two-CTA kernel was chosen (block_m is then 256) */
  int64_t scratch_bytes;   /* plan-owned global scratch (stream-K partial tiles + counters) */
  double flops;            /* 2*m*n*k */
  double algorithmic_bytes;/* read A once + read B once + write C once (+ scales) */
} tx_dot_plan_info;

typedef struct tx_dot_plan tx_dot_plan; /* opaque */

/* Number of CUDA devices visible, 0 if none (never fails). */
TXD_API int tx_dot_device_count(void);

/* Text of the last error raised on the calling thread ("" if none). Borrowed pointer. */
TXD_API const char *tx_dot_last_error(void);

/* Validate the problem, run the tile-selection analysis for unset config fields, and allocate
 * plan-owned scratch on the current device. `cfg` may be NULL. Needs a CUDA device. On failure nothing stays allocated.
 * A plan is not thread-safe: it caches the tensor maps of the last operand pointers and rewrites them in
 * tx_dot_run, so one plan serves one host thread at a time (create one plan per thread, or lock around the calls).
 * Launches of one plan that use its scratch (stream-K, hybrid) must not overlap on the device either. */
TXD_API int tx_dot_plan_create(const tx_dot_problem *problem, const tx_dot_config *cfg,
                               tx_dot_plan **out_plan);

/* Same analysis without touching a device: fills `info` for (problem, cfg) assuming `sm_count` SMs.
 * Usable on a machine with no GPU. */
TXD_API int tx_dot_plan_preview(const tx_dot_problem *problem, const tx_dot_config *cfg,
                                int32_t sm_count, tx_dot_plan_info *info);

TXD_API int tx_dot_plan_query(const tx_dot_plan *plan, tx_dot_plan_info *info);

/* Launch on `stream` (a cudaStream_t; NULL = default stream). All pointers are device pointers,
 * 16-byte aligned. row_scale / col_scale must be non-NULL exactly when the plan asked for them.
 * Asynchronous: returns after the launch. Device-side waits are bounded; a wait that runs out is
 * reported by tx_dot_plan_check(). */
TXD_API int tx_dot_run(tx_dot_plan *plan, const void *a, const void *b, void *c,
                       const float *row_scale, const float *col_scale, void *stream);

/* Synchronise `stream` and report TXD_ERR_DEVICE_TIMEOUT if any launch of this plan since the last
 * check gave up on a wait. */
TXD_API int tx_dot_plan_check(tx_dot_plan *plan, void *stream);

/* The same contraction from HOST buffers: copies A, B (and scales) to plan-owned device buffers,
 * launches, copies C back and synchronises. This is the call a host-side user of the extension
 * makes; it is what the end-to-end figure of the benchmark times. Pinned host memory is used as-is. */
TXD_API int tx_dot_run_host(tx_dot_plan *plan, const void *a_host, const void *b_host, void *c_host,
                            const float *row_scale_host, const float *col_scale_host);

/*
 * K-sharded GEMM fused with its partial-sum exchange (one process per GPU, `world` ranks over NVLink).
 * Rank r holds A[:, k_r] and B[k_r, :] and creates a plan for the m x n x |k_r| problem with out_dtype F32
 * or BF16, no scales, alpha 1, whole-tile schedule. Instead of writing C, the kernel's epilogue stores each
 * tile straight into the memory of the rank that owns the tile's rows: slot_bases[o] is the device address
 * (peer-mapped where o != rank) of rank o's slot buffer, laid out [world][m / world][n] in out_dtype, and this
 * rank writes slot `rank` of every buffer. The stores are ordinary TMA tensor stores; no multicast is used.
 * Needs m % world == 0 and (m / world) % block_m == 0, world <= 8.
 * After every rank's launch has completed (a stream-ordered barrier between the ranks is the caller's job),
 * tx_dot_reduce_slots sums the `world` slots of the local buffer in slot order (deterministic), applies
 * alpha / row_scale / col_scale and casts:  out[r, c] = cast(alpha * rs[r] * cs[c] * sum_s slots[s][r][c]).
 * The reference has no multi-GPU code; this is the fused form of "GEMM, then reduce-scatter".
 */
TXD_API int tx_dot_run_to_slots(tx_dot_plan *plan, const void *a, const void *b, void *const *slot_bases,
                                int32_t world, int32_t rank, void *stream);
TXD_API int tx_dot_reduce_slots(const void *slots, int32_t world, int32_t rows, int32_t n, int32_t slot_dtype,
                                void *out, int32_t out_dtype, int64_t ldc, const float *row_scale,
                                const float *col_scale, float alpha, void *stream);

/*
 * The same exchange in `parts` pieces, so that the sum of a finished piece can run (on another stream, after the ranks'
 * barrier for that piece) while the next piece's GEMM is still storing. The tile rows are dealt to the owners in turn,
 * so piece `part` fills rows [part, part + 1) * (m / world / parts) of this rank's slot in every owner's buffer, and
 * tx_dot_reduce_slots_part sums exactly those rows: rows [row0, row0 + rows) of each of the `world` slots (each
 * rows_per_rank x n) into rows [row0, row0 + rows) of `out`; `out` and `row_scale` are the whole result's. Needs
 * (m / world / block_m) % parts == 0. With parts = 1 and row0 = 0, rows = rows_per_rank these are the two calls above.
 */
TXD_API int tx_dot_run_to_slots_part(tx_dot_plan *plan, const void *a, const void *b, void *const *slot_bases,
                                     int32_t world, int32_t rank, int32_t part, int32_t parts, void *stream);
TXD_API int tx_dot_reduce_slots_part(const void *slots, int32_t world, int32_t rows_per_rank, int32_t row0, int32_t rows,
                                     int32_t n, int32_t slot_dtype, void *out, int32_t out_dtype, int64_t ldc,
                                     const float *row_scale, const float *col_scale, float alpha, void *stream);

TXD_API int tx_dot_plan_destroy(tx_dot_plan *plan);

/*
 * No counterpart in the reference (it has no kernels and no allocator policy): a launch for callers
 * that may not allocate — hosts whose memory pool belongs to another library, threads that must not
 * take the driver's allocator lock, plug-in sandboxes that forbid cudaMalloc. It runs the stream-K
 * schedule on single CTAs with the partial-tile scratch, tile counters and status word held in one
 * fixed array inside the library image, and calls no allocating routine of CUDA or of any library.
 *
 *   - `problem` and `cfg` as for tx_dot_plan_create (cfg may be NULL; schedule and cta_pair are
 *     overridden). The configuration's scratch must fit: at most tx_dot_static_scratch_capacity()
 *     bytes of partial tiles (grid * 2 * block_n * 128 * 4) and 16384 output tiles; otherwise
 *     TXD_ERR_UNSUPPORTED with both sizes in the message. Lower block_n or max_ctas to fit.
 *   - All calls on a GPU share the array: launches that overlap in time race and give garbage, so
 *     serialise them (one stream, or events). Each call clears the counters it needs on `stream`.
 *   - The first call on a device resolves the array's device address and raises the kernel's
 *     shared-memory limit; make it before starting any stream capture.
 *   - Every GPU that loads the library holds the array (about 4.1 MiB) until the process exits.
 * tx_dot_static_scratch_check synchronises `stream` and reports a wait that ran out since the last
 * check. Error text: tx_dot_static_scratch_last_error().
 */
TXD_API int tx_dot_run_static_scratch(const tx_dot_problem *problem, const tx_dot_config *cfg,
                                      const void *a, const void *b, void *c, const float *row_scale,
                                      const float *col_scale, void *stream);
TXD_API int tx_dot_static_scratch_check(void *stream);
TXD_API int64_t tx_dot_static_scratch_capacity(void);
TXD_API const char *tx_dot_static_scratch_last_error(void);

/* Kernels this library has launched in this process since load (for launch accounting). */
TXD_API uint64_t tx_dot_kernel_launches(void);

#ifdef __cplusplus
}
#endif
#endif /* B200_DOT_H */
