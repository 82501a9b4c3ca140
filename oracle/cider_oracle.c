/*
 * CPU oracle for cider's online activation-quantized linear path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of
 * the reference's Metal kernels so that the CUDA kernels can be checked against
 * it.  It is linked by nothing in the product: only the tests, the smoke check
 * and the bench's cpu_baseline / reference arm load it.
 *
 * Parity pinning: the reference's own tests pin only the raw integer GEMM
 * (benchmarks/test_bitexact.py:19-58) and its numpy weight-quant helpers can be
 * imported to pin S8 (cider/ops.py:73-116, cider/nn.py:34-59).  Activation
 * quantization, the fused dequant epilogues, the matrix-vector kernels and W4A8
 * have no test or golden vector in the reference: for those this oracle is a
 * restatement of the Metal source only ("parity unpinned").
 *
 * Floating-point conventions.  The Metal sources are compiled with default
 * options (fast-math on), so `a*b + c` may or may not be contracted there.  This
 * oracle fixes ONE definition: IEEE binary32, round-to-nearest-even, with the
 * multiply-adds of the dequant epilogues contracted into a single fused
 * multiply-add (fmaf).  The file must be compiled with -ffp-contract=off so that
 * nothing else is contracted behind our back.
 *
 * fp16 values cross the boundary as _Float16 (IEEE binary16).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 half_t;

#define CLONES __attribute__((target_clones("arch=skylake-avx512", "avx2", "default")))

int cider_oracle_version(void) { return 1; }

int cider_oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Thread count of the following calls (a launcher such as torchrun exports
 * OMP_NUM_THREADS=1 to its workers; the timed CPU baseline wants the host's cores). */
void cider_oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------ S1 ----
 * Per-token activation quantization.
 * cider/kernels/w8a8_quantize.metal:34-38 (absmax), :64-67 (scale, zero
 * guard), :71 (reciprocal), :82-86 (multiply, round, clamp, cast).
 * round() in Metal is round-half-away-from-zero == C roundf().
 */
CLONES
static float quantize_row(const half_t *row, int64_t K, int8_t *qrow) {
  float amax = 0.0f;
  for (int64_t k = 0; k < K; ++k) {
    float v = fabsf((float)row[k]);
    amax = v > amax ? v : amax;
  }
  float s = amax / 127.0f;
  if (s == 0.0f) s = 1.0f;
  float inv = 1.0f / s;
  for (int64_t k = 0; k < K; ++k) {
    float v = roundf((float)row[k] * inv);
    v = v < -128.0f ? -128.0f : (v > 127.0f ? 127.0f : v);
    qrow[k] = (int8_t)v;
  }
  return s;
}

void cider_oracle_quantize_per_token(const half_t *x, int64_t M, int64_t K,
                                     int64_t ldx, int8_t *q, float *scale) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m)
    scale[m] = quantize_row(x + m * ldx, K, q + m * K);
}

/* ------------------------------------------------------------------ S2 ----
 * Raw integer GEMM, C[m,n] = sum_k A[m,k]*B[n,k], exact int32.
 * cider/kernels/w8a8_matmul.metal:301-453; cider/ops.py:238-255.
 */
CLONES
static int32_t dot_i8(const int8_t *a, const int8_t *b, int64_t K) {
  int32_t acc = 0;
  for (int64_t k = 0; k < K; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
  return acc;
}

void cider_oracle_int8_matmul_int32(const int8_t *a, const int8_t *b,
                                    int32_t *c, int64_t M, int64_t N,
                                    int64_t K) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n)
      c[m * N + n] = dot_i8(a + m * K, b + n * K, K);
}

/* ------------------------------------------------------------- S3 / S5 ----
 * Per-channel linear.
 *  M > 1: quantize (S1) -> integer GEMM (S2) -> fused dequant
 *         half(float(acc)*sa[m]*sw[n] + float(bias[n])),
 *         cider/kernels/w8a8_matmul.metal:63-81 (left to right; the final
 *         multiply-add is fused here).
 *  M == 1: the reference does NOT quantize the activation
 *         (csrc/src/w8a8_primitive.mm:157-178):
 *         y[n] = half(sw[n] * sum_k float(W[n,k])*float(x[k]) + float(bias[n])),
 *         cider/kernels/w8a8_int8_mv.metal:34-69.  The reference's fp32
 *         summation order depends on its SIMD-group layout; the oracle sums in
 *         binary64 and the comparison carries a tolerance.
 * bias may be NULL (zeros, cider/ops.py:143-144).
 */
CLONES
static double dot_i8_f16(const int8_t *w, const half_t *x, int64_t K) {
  double acc = 0.0;
  for (int64_t k = 0; k < K; ++k) acc += (double)w[k] * (double)(float)x[k];
  return acc;
}

void cider_oracle_perchannel_linear(const half_t *x, const int8_t *w,
                                    const float *sw, const half_t *bias,
                                    half_t *y, int64_t M, int64_t N,
                                    int64_t K) {
  if (M == 1) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      float dot = (float)dot_i8_f16(w + n * K, x, K);
      float b = bias ? (float)bias[n] : 0.0f;
      y[n] = (half_t)fmaf(sw[n], dot, b);
    }
    return;
  }
  int8_t *q = (int8_t *)malloc((size_t)M * K);
  float *sa = (float *)malloc(sizeof(float) * (size_t)M);
  cider_oracle_quantize_per_token(x, M, K, K, q, sa);
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      int32_t acc = dot_i8(q + m * K, w + n * K, K);
      float b = bias ? (float)bias[n] : 0.0f;
      float t = (float)acc * sa[m];
      y[m * N + n] = (half_t)fmaf(t, sw[n], b);
    }
  free(q);
  free(sa);
}

/* Same epilogue, but for activations that were quantized elsewhere. */
void cider_oracle_dequant_perchannel(const int32_t *acc, const float *sa,
                                     const float *sw, const half_t *bias,
                                     half_t *y, int64_t M, int64_t N) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      float b = bias ? (float)bias[n] : 0.0f;
      float t = (float)acc[m * N + n] * sa[m];
      y[m * N + n] = (half_t)fmaf(t, sw[n], b);
    }
}

/* ------------------------------------------------------------- S4 / S6 ----
 * Per-group linear.  sw is [K/gs, N] fp32 (physically transposed,
 * cider/nn.py:85-88; kernel index scale_w[g*N+n]).
 *  M > 1: accf = sum_g float(acc_g) * sw[g,n] in ascending g, one fused
 *         multiply-add per group (cider/kernels/pergroup_int8_gemm.metal:99-172,
 *         flush at :164), then half(accf*sa[m] + float(bias[n])) (:184).
 *  M == 1: y[n] = half(sum sw[g,n]*dot + float(bias[n])) with fp activations
 *         (cider/kernels/pergroup_int8_mv.metal:50-103); summed in binary64.
 */
void cider_oracle_pergroup_linear(const half_t *x, const int8_t *w,
                                  const float *sw, const half_t *bias,
                                  half_t *y, int64_t M, int64_t N, int64_t K,
                                  int64_t gs) {
  const int64_t G = K / gs;
  if (M == 1) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      double acc = 0.0;
      for (int64_t g = 0; g < G; ++g)
        acc += (double)sw[g * N + n] * dot_i8_f16(w + n * K + g * gs, x + g * gs, gs);
      float b = bias ? (float)bias[n] : 0.0f;
      y[n] = (half_t)((float)acc + b);
    }
    return;
  }
  int8_t *q = (int8_t *)malloc((size_t)M * K);
  float *sa = (float *)malloc(sizeof(float) * (size_t)M);
  cider_oracle_quantize_per_token(x, M, K, K, q, sa);
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      float accf = 0.0f;
      for (int64_t g = 0; g < G; ++g) {
        int32_t acc = dot_i8(q + m * K + g * gs, w + n * K + g * gs, gs);
        accf = fmaf((float)acc, sw[g * N + n], accf);
      }
      float b = bias ? (float)bias[n] : 0.0f;
      y[m * N + n] = (half_t)fmaf(accf, sa[m], b);
    }
  free(q);
  free(sa);
}

/* ------------------------------------------------------------------ S7 ----
 * W4A8.  packed is [K/2, N] uint8, N contiguous; high nibble = even k, low
 * nibble = odd k, value = nibble - 8 (cider/kernels/w4a8_matmul.metal:47-70).
 *  gs == 0: reference semantics, sw[N] per column, no bias, no M==1 branch:
 *           half(float(acc)*sa[m]*sw[n])   (w4a8_matmul.metal:72-89).
 *  gs  > 0: extension for group-wise int4 scales sw[K/gs, N]: the per-group
 *           accumulation of S4 on top of the same unpack, no bias.
 */
void cider_oracle_unpack_w4(const uint8_t *packed, int8_t *w_nk, int64_t N,
                            int64_t K) {
  /* produces W as [N, K] int8 (the layout of the int8 weight paths) */
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n)
    for (int64_t i = 0; i < K / 2; ++i) {
      uint8_t p = packed[i * N + n];
      w_nk[n * K + 2 * i] = (int8_t)((int)(p >> 4) - 8);
      w_nk[n * K + 2 * i + 1] = (int8_t)((int)(p & 15) - 8);
    }
}

void cider_oracle_w4a8_linear(const half_t *x, const uint8_t *packed,
                              const float *sw, half_t *y, int64_t M, int64_t N,
                              int64_t K, int64_t gs) {
  int8_t *w = (int8_t *)malloc((size_t)N * K);
  int8_t *q = (int8_t *)malloc((size_t)M * K);
  float *sa = (float *)malloc(sizeof(float) * (size_t)M);
  cider_oracle_unpack_w4(packed, w, N, K);
  cider_oracle_quantize_per_token(x, M, K, K, q, sa);
  if (gs == 0) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t m = 0; m < M; ++m)
      for (int64_t n = 0; n < N; ++n) {
        int32_t acc = dot_i8(q + m * K, w + n * K, K);
        float t = (float)acc * sa[m];
        y[m * N + n] = (half_t)(t * sw[n]);
      }
  } else {
    const int64_t G = K / gs;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t m = 0; m < M; ++m)
      for (int64_t n = 0; n < N; ++n) {
        float accf = 0.0f;
        for (int64_t g = 0; g < G; ++g) {
          int32_t acc = dot_i8(q + m * K + g * gs, w + n * K + g * gs, gs);
          accf = fmaf((float)acc, sw[g * N + n], accf);
        }
        y[m * N + n] = (half_t)(accf * sa[m]);
      }
  }
  free(w);
  free(q);
  free(sa);
}

/* --------------------------------------------------------------------------
 * Decoder glue used around the linears (no counterpart inside the reference:
 * RMSNorm and SDPA live in its un-vendored MLX dependencies).  Stated here in
 * the plainest form so the CUDA kernels have a checker.
 */

/* y = half( float(x) * rsqrt(mean(x^2) + eps) * float(w) ), fp32 math with the
 * mean accumulated in binary64 (order-free). */
void cider_oracle_rmsnorm(const half_t *x, const half_t *w, half_t *y,
                          int64_t M, int64_t K, float eps) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    double ss = 0.0;
    for (int64_t k = 0; k < K; ++k) {
      double v = (double)(float)x[m * K + k];
      ss += v * v;
    }
    float r = 1.0f / sqrtf((float)(ss / (double)K) + eps);
    for (int64_t k = 0; k < K; ++k)
      y[m * K + k] = (half_t)(((float)x[m * K + k] * r) * (float)w[k]);
  }
}

/* Single-query attention per (batch, q head): out = softmax(q.K^T*scale) V over
 * T cached positions, GQA (Hq % Hkv == 0), fp16 KV cache laid out
 * [B, Hkv, Tcap, D]; math in binary64. */
void cider_oracle_sdpa_decode(const half_t *q, const half_t *kc,
                              const half_t *vc, half_t *out, int64_t B,
                              int64_t Hq, int64_t Hkv, int64_t D, int64_t T,
                              int64_t Tcap, float scale) {
  const int64_t rep = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < B; ++b)
    for (int64_t h = 0; h < Hq; ++h) {
      const half_t *qv = q + (b * Hq + h) * D;
      const half_t *kb = kc + ((b * Hkv + h / rep) * Tcap) * D;
      const half_t *vb = vc + ((b * Hkv + h / rep) * Tcap) * D;
      double *p = (double *)malloc(sizeof(double) * (size_t)(T > 0 ? T : 1));
      double mx = -INFINITY;
      for (int64_t t = 0; t < T; ++t) {
        double s = 0.0;
        for (int64_t d = 0; d < D; ++d)
          s += (double)(float)qv[d] * (double)(float)kb[t * D + d];
        p[t] = s * (double)scale;
        if (p[t] > mx) mx = p[t];
      }
      double den = 0.0;
      for (int64_t t = 0; t < T; ++t) {
        p[t] = exp(p[t] - mx);
        den += p[t];
      }
      for (int64_t d = 0; d < D; ++d) {
        double o = 0.0;
        for (int64_t t = 0; t < T; ++t) o += p[t] * (double)(float)vb[t * D + d];
        out[(b * Hq + h) * D + d] = (half_t)(float)(T > 0 ? o / den : 0.0);
      }
      free(p);
    }
}
