/*
 * TEST INFRASTRUCTURE — not part of the product path.
 *
 * Plain-C restatement of how a tiled `tt.dot` GEMM is evaluated on the host by Triton's interpreter,
 * which is the CPU path of the reference's only tl.dot call sites
 * (pass/LoopSplit/06-fused-attention.py:63,85 with the fp32 accumulator of :222):
 *
 *   for each output tile (BLOCK_M x BLOCK_N), acc = 0 (fp32)
 *     for k0 in range(0, K, BLOCK_K):                       the K loop LoopSplit rewrites
 *       a = A[tile rows, k0:k0+BLOCK_K]  (zero past K)      masked tt.load
 *       b = B[k0:k0+BLOCK_K, tile cols]  (zero past K)
 *       acc = matmul(a, b) in fp32 + acc                     interpreter `create_dot`:
 *                                                            np.matmul(a, b, dtype=float32) + acc
 *   C[tile] = cast(acc * alpha * row_scale[:,None] * col_scale[None,:])
 *
 * Triton 3.6.0 (third-party; installed wheel, not part of the reference) — runtime/interpreter.py
 * create_dot: fp8 operands are widened exactly, the product of the block is formed in fp32 and added
 * to the accumulator. The order of additions inside one block is numpy's (BLAS); here it is a plain
 * ascending-k loop, so results agree to fp32 rounding, not bit for bit.
 *
 * Output casts: fp16 round-to-nearest-even (numpy astype); bf16 either truncation (what the
 * interpreter's cast does) or round-to-nearest-even (what the GPU kernels do), chosen by the caller.
 *
 * Pinned by tests/test_oracle.py against oracle/interp_dot.py on the committed fixtures.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { DO_F16 = 0, DO_BF16 = 1, DO_F8E4M3 = 2, DO_F32 = 3, DO_F8E5M2 = 4 };

static float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400u));
      man &= 0x3FFu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static uint16_t f32_to_f16_rne(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  int32_t exp = (int32_t)((x >> 23) & 0xFFu) - 127 + 15;
  uint32_t man = x & 0x7FFFFFu;
  if (((x >> 23) & 0xFFu) == 0xFFu) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000u;
    uint32_t shift = (uint32_t)(14 - exp);
    uint32_t half = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1u))) ++half;
    return (uint16_t)(sign | half);
  }
  uint32_t half = ((uint32_t)exp << 10) | (man >> 13);
  uint32_t rem = man & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) ++half;
  return (uint16_t)(sign | half);
}

static float bf16_to_f32(uint16_t h) {
  uint32_t bits = (uint32_t)h << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static uint16_t f32_to_bf16(float f, int truncate) {
  uint32_t x;
  memcpy(&x, &f, 4);
  if (truncate) return (uint16_t)(x >> 16);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
  uint32_t lsb = (x >> 16) & 1u;
  x += 0x7FFFu + lsb;
  return (uint16_t)(x >> 16);
}

static float f8e4m3_to_f32(uint8_t v) {
  int sign = v >> 7, exp = (v >> 3) & 0xF, man = v & 7;
  float r;
  if (exp == 0) r = ldexpf((float)man, -9);
  else if (exp == 15 && man == 7) r = NAN;
  else r = ldexpf((float)(8 + man), exp - 10);
  return sign ? -r : r;
}

static float f8e5m2_to_f32(uint8_t v) {
  return f16_to_f32((uint16_t)((uint16_t)v << 8));
}

static float load_elem(const void *base, int dtype, int64_t idx) {
  switch (dtype) {
    case DO_F16: return f16_to_f32(((const uint16_t *)base)[idx]);
    case DO_BF16: return bf16_to_f32(((const uint16_t *)base)[idx]);
    case DO_F8E4M3: return f8e4m3_to_f32(((const uint8_t *)base)[idx]);
    case DO_F8E5M2: return f8e5m2_to_f32(((const uint8_t *)base)[idx]);
    default: return ((const float *)base)[idx];
  }
}

/*
 * Compute the output tiles listed in tile_ids (NULL = every tile, row-major tile numbering
 * tile = tm * tiles_n + tn). Element strides let A and B be either major. C is row-major, ldc.
 * Returns 0, or -1 on a bad argument.
 */
__attribute__((visibility("default")))
int dot_oracle_tiles(const void *a, const void *b, void *c, const float *row_scale, const float *col_scale,
                     int32_t m, int32_t n, int32_t k, int32_t ab_dtype, int32_t out_dtype,
                     int64_t a_stride_m, int64_t a_stride_k, int64_t b_stride_k, int64_t b_stride_n, int64_t ldc,
                     float alpha, int32_t block_m, int32_t block_n, int32_t block_k, int32_t bf16_truncate,
                     const int32_t *tile_ids, int32_t n_tile_ids) {
  if (!c || m < 0 || n < 0 || k < 0 || block_m <= 0 || block_n <= 0 || block_k <= 0) return -1;
  if (k > 0 && (!a || !b)) return -1;
  const int tiles_m = (m + block_m - 1) / block_m, tiles_n = (n + block_n - 1) / block_n;
  const int total = tile_ids ? n_tile_ids : tiles_m * tiles_n;
  int bad = 0;
#pragma omp parallel for schedule(dynamic, 1)
  for (int t = 0; t < total; ++t) {
    const int tile = tile_ids ? tile_ids[t] : t;
    if (tile < 0 || tile >= tiles_m * tiles_n) { bad = 1; continue; }
    const int tm = tile / tiles_n, tn = tile % tiles_n;
    const int m0 = tm * block_m, n0 = tn * block_n;
    const int mh = (m - m0 < block_m) ? m - m0 : block_m;
    const int nw = (n - n0 < block_n) ? n - n0 : block_n;
    float *acc = (float *)calloc((size_t)block_m * block_n, sizeof(float));
    float *blk = (float *)malloc((size_t)block_m * block_n * sizeof(float));
    float *at = (float *)malloc((size_t)block_m * block_k * sizeof(float));
    float *bt = (float *)malloc((size_t)block_k * block_n * sizeof(float));
    for (int k0 = 0; k0 < k; k0 += block_k) {
      const int kw = (k - k0 < block_k) ? k - k0 : block_k;
      for (int i = 0; i < mh; ++i)
        for (int kk = 0; kk < kw; ++kk)
          at[(size_t)i * block_k + kk] = load_elem(a, ab_dtype, (int64_t)(m0 + i) * a_stride_m + (int64_t)(k0 + kk) * a_stride_k);
      for (int kk = 0; kk < kw; ++kk)
        for (int j = 0; j < nw; ++j)
          bt[(size_t)kk * block_n + j] = load_elem(b, ab_dtype, (int64_t)(k0 + kk) * b_stride_k + (int64_t)(n0 + j) * b_stride_n);
      /* blk = a_tile @ b_tile in fp32, then acc = blk + acc  (create_dot) */
      for (int i = 0; i < mh; ++i) {
        float *row = blk + (size_t)i * block_n;
        for (int j = 0; j < nw; ++j) row[j] = 0.0f;
        for (int kk = 0; kk < kw; ++kk) {
          const float av = at[(size_t)i * block_k + kk];
          const float *brow = bt + (size_t)kk * block_n;
          for (int j = 0; j < nw; ++j) row[j] += av * brow[j];
        }
        float *arow = acc + (size_t)i * block_n;
        for (int j = 0; j < nw; ++j) arow[j] = row[j] + arow[j];
      }
    }
    for (int i = 0; i < mh; ++i) {
      const float rs = row_scale ? row_scale[m0 + i] : 1.0f;
      for (int j = 0; j < nw; ++j) {
        float v = acc[(size_t)i * block_n + j];
        v = v * (alpha * rs);
        if (col_scale) v = v * col_scale[n0 + j];
        const int64_t o = (int64_t)(m0 + i) * ldc + (n0 + j);
        if (out_dtype == DO_F32) ((float *)c)[o] = v;
        else if (out_dtype == DO_BF16) ((uint16_t *)c)[o] = f32_to_bf16(v, bf16_truncate);
        else ((uint16_t *)c)[o] = f32_to_f16_rne(v);
      }
    }
    free(acc); free(blk); free(at); free(bt);
  }
  return bad ? -1 : 0;
}
