/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the arithmetic that
 * hqu-little-boy/ncnn-compiler emits for its hot operators.  Nothing in the
 * product may link or call this file; it exists so tests and the bench's
 * cpu_baseline leg can check the CUDA path against the reference's semantics.
 *
 * Parity status: the reference keeps no stored golden outputs for these
 * operators (its tests compute expectations with upstream ncnn at test time,
 * test/Numerical/support/numerical_test_support.cpp:542-699), and its
 * LLVM/MLIR 21 toolchain is not available, so values are "parity unpinned";
 * what is pinned are the order of operations below (each cites the lowering it
 * follows) and hand-derived known answers for the reference's own fixtures.
 *
 * Layout: like the reference, every rank-3 tensor is NHWC with N = 1
 * (lib/Conversion/NCNNToTosa/NCNNToTosa.cpp:48-52,939-987): arrays here are
 * [H][W][C].  Weights arrive in ncnn order [O][I][KH][KW].
 * Build: gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC (no fast-math: the
 * reference's arith ops carry no fast-math flags, tools/ncnn-compile.cpp:1929-1935).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* Convolution, fp32 branch (NCNNToTosa.cpp:1403-1528): the accumulator starts at
 * the bias (zero splat when bias_term = 0, :1319-1323) and the window is walked
 * kh, kw, c as linalg.conv_2d_nhwc_hwcf does; zero padding, cross-correlation. */
int orc_conv2d_f32(const float* x, int H, int W, int C, const float* w, const float* bias, int O,
                   int KH, int KW, int sh, int sw, int pt, int pl, int dh, int dw, int OH, int OW,
                   float* y) {
  float* wt = (float*)malloc(sizeof(float) * (size_t)KH * KW * C * O); /* HWCF */
  if (!wt) return 1;
  for (int o = 0; o < O; ++o)
    for (int c = 0; c < C; ++c)
      for (int kh = 0; kh < KH; ++kh)
        for (int kw = 0; kw < KW; ++kw)
          wt[(((size_t)kh * KW + kw) * C + c) * O + o] = w[(((size_t)o * C + c) * KH + kh) * KW + kw];
#pragma omp parallel for schedule(static)
  for (int oh = 0; oh < OH; ++oh) {
    for (int ow = 0; ow < OW; ++ow) {
      float* acc = y + ((size_t)oh * OW + ow) * O;
      for (int o = 0; o < O; ++o) acc[o] = bias ? bias[o] : 0.0f;
      for (int kh = 0; kh < KH; ++kh) {
        const int ih = oh * sh - pt + kh * dh;
        for (int kw = 0; kw < KW; ++kw) {
          const int iw = ow * sw - pl + kw * dw;
          const int inside = ih >= 0 && ih < H && iw >= 0 && iw < W;
          const float* xp = inside ? x + ((size_t)ih * W + iw) * C : NULL;
          const float* wp = wt + ((size_t)kh * KW + kw) * C * O;
          for (int c = 0; c < C; ++c) {
            const float xv = inside ? xp[c] : 0.0f; /* padded value participates as 0 */
            const float* wr = wp + (size_t)c * O;
            for (int o = 0; o < O; ++o) acc[o] = acc[o] + xv * wr[o];
          }
        }
      }
    }
  }
  free(wt);
  return 0;
}

/* Convolution, int8 branch (NCNNToTosa.cpp:1136-1315): int8 x int8 -> int32, zero
 * points 0, padding value 0 (:1160-1167,1277-1290).  Output is the raw accumulator. */
int orc_conv2d_i8(const int8_t* x, int H, int W, int C, const int8_t* w, int O, int KH, int KW,
                  int sh, int sw, int pt, int pl, int dh, int dw, int OH, int OW, int32_t* y) {
  int8_t* wt = (int8_t*)malloc((size_t)KH * KW * C * O);
  if (!wt) return 1;
  for (int o = 0; o < O; ++o)
    for (int c = 0; c < C; ++c)
      for (int kh = 0; kh < KH; ++kh)
        for (int kw = 0; kw < KW; ++kw)
          wt[(((size_t)kh * KW + kw) * C + c) * O + o] = w[(((size_t)o * C + c) * KH + kh) * KW + kw];
#pragma omp parallel for schedule(static)
  for (int oh = 0; oh < OH; ++oh) {
    for (int ow = 0; ow < OW; ++ow) {
      int32_t* acc = y + ((size_t)oh * OW + ow) * O;
      for (int o = 0; o < O; ++o) acc[o] = 0;
      for (int kh = 0; kh < KH; ++kh) {
        const int ih = oh * sh - pt + kh * dh;
        if (ih < 0 || ih >= H) continue;
        for (int kw = 0; kw < KW; ++kw) {
          const int iw = ow * sw - pl + kw * dw;
          if (iw < 0 || iw >= W) continue;
          const int8_t* xp = x + ((size_t)ih * W + iw) * C;
          const int8_t* wp = wt + ((size_t)kh * KW + kw) * C * O;
          for (int c = 0; c < C; ++c) {
            const int32_t xv = xp[c];
            const int8_t* wr = wp + (size_t)c * O;
            for (int o = 0; o < O; ++o) acc[o] += xv * (int32_t)wr[o];
          }
        }
      }
    }
  }
  free(wt);
  return 0;
}

/* ConvolutionDepthWise (NCNNToTosa.cpp:3074-3503): group == channels, weight
 * [C][1][KH][KW]; out[oh,ow,c] = bias[c] + sum_{kh,kw} in * w. */
int orc_depthwise_f32(const float* x, int H, int W, int C, const float* w, const float* bias,
                      int KH, int KW, int sh, int sw, int pt, int pl, int dh, int dw, int OH,
                      int OW, float* y) {
#pragma omp parallel for schedule(static)
  for (int oh = 0; oh < OH; ++oh)
    for (int ow = 0; ow < OW; ++ow) {
      float* acc = y + ((size_t)oh * OW + ow) * C;
      for (int c = 0; c < C; ++c) acc[c] = bias ? bias[c] : 0.0f;
      for (int kh = 0; kh < KH; ++kh) {
        const int ih = oh * sh - pt + kh * dh;
        for (int kw = 0; kw < KW; ++kw) {
          const int iw = ow * sw - pl + kw * dw;
          const int inside = ih >= 0 && ih < H && iw >= 0 && iw < W;
          for (int c = 0; c < C; ++c) {
            const float xv = inside ? x[((size_t)ih * W + iw) * C + c] : 0.0f;
            acc[c] = acc[c] + xv * w[((size_t)c * KH + kh) * KW + kw];
          }
        }
      }
    }
  return 0;
}

int orc_depthwise_i8(const int8_t* x, int H, int W, int C, const int8_t* w, int KH, int KW,
                     int sh, int sw, int pt, int pl, int dh, int dw, int OH, int OW, int32_t* y) {
#pragma omp parallel for schedule(static)
  for (int oh = 0; oh < OH; ++oh)
    for (int ow = 0; ow < OW; ++ow) {
      int32_t* acc = y + ((size_t)oh * OW + ow) * C;
      for (int c = 0; c < C; ++c) acc[c] = 0;
      for (int kh = 0; kh < KH; ++kh) {
        const int ih = oh * sh - pt + kh * dh;
        if (ih < 0 || ih >= H) continue;
        for (int kw = 0; kw < KW; ++kw) {
          const int iw = ow * sw - pl + kw * dw;
          if (iw < 0 || iw >= W) continue;
          for (int c = 0; c < C; ++c)
            acc[c] += (int32_t)x[((size_t)ih * W + iw) * C + c] *
                      (int32_t)w[((size_t)c * KH + kh) * KW + kw];
        }
      }
    }
  return 0;
}

/* InnerProduct / Gemm contraction (NCNNToTosa.cpp:5254-5392, 4990-5109):
 * y[m][n] = sum_k a[m][k] * b[n][k], accumulator starts at 0 (tosa.matmul); bias,
 * alpha and beta are applied by the caller afterwards, as the lowering does. */
int orc_matmul_f32(const float* a, const float* b, int M, int K, int N, float* y) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float acc = 0.0f;
      const float* ar = a + (size_t)m * K;
      const float* br = b + (size_t)n * K;
      for (int k = 0; k < K; ++k) acc = acc + ar[k] * br[k];
      y[(size_t)m * N + n] = acc;
    }
  return 0;
}

int orc_matmul_i8(const int8_t* a, const int8_t* b, int M, int K, int N, int32_t* y) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      int32_t acc = 0;
      const int8_t* ar = a + (size_t)m * K;
      const int8_t* br = b + (size_t)n * K;
      for (int k = 0; k < K; ++k) acc += (int32_t)ar[k] * (int32_t)br[k];
      y[(size_t)m * N + n] = acc;
    }
  return 0;
}

/* Pooling, static branch (NCNNToTosa.cpp:1879-1994, getPoolPadding :997-1105).
 * kind 0 = max (padding never wins), 1 = average over the in-bounds elements
 * only (sum, then one division by the count).  The caller passes the inferred
 * output extent (NCNNOps.cpp:488-531); windows may run past the input on the
 * trailing side (ncnn "full" mode tail window). */
int orc_pool_f32(const float* x, int H, int W, int C, int kind, int KH, int KW, int sh, int sw,
                 int pt, int pl, int OH, int OW, float* y) {
#pragma omp parallel for schedule(static)
  for (int oh = 0; oh < OH; ++oh)
    for (int ow = 0; ow < OW; ++ow)
      for (int c = 0; c < C; ++c) {
        float acc = kind == 0 ? -INFINITY : 0.0f;
        int count = 0;
        for (int kh = 0; kh < KH; ++kh) {
          const int ih = oh * sh - pt + kh;
          if (ih < 0 || ih >= H) continue;
          for (int kw = 0; kw < KW; ++kw) {
            const int iw = ow * sw - pl + kw;
            if (iw < 0 || iw >= W) continue;
            const float v = x[((size_t)ih * W + iw) * C + c];
            if (kind == 0) {
              acc = v > acc ? v : acc;
            } else {
              acc = acc + v;
            }
            ++count;
          }
        }
        if (kind == 1) acc = acc / (float)count;
        y[((size_t)oh * OW + ow) * C + c] = acc;
      }
  return 0;
}

int orc_pool_max_i8(const int8_t* x, int H, int W, int C, int KH, int KW, int sh, int sw, int pt,
                    int pl, int OH, int OW, int8_t* y) {
  for (int oh = 0; oh < OH; ++oh)
    for (int ow = 0; ow < OW; ++ow)
      for (int c = 0; c < C; ++c) {
        int acc = -128;
        for (int kh = 0; kh < KH; ++kh) {
          const int ih = oh * sh - pt + kh;
          if (ih < 0 || ih >= H) continue;
          for (int kw = 0; kw < KW; ++kw) {
            const int iw = ow * sw - pl + kw;
            if (iw < 0 || iw >= W) continue;
            const int v = x[((size_t)ih * W + iw) * C + c];
            acc = v > acc ? v : acc;
          }
        }
        y[((size_t)oh * OW + ow) * C + c] = (int8_t)acc;
      }
  return 0;
}

/* quantizeSignedI8 (NCNNToTosa.cpp:322-389): v = x*s; r = v >= 0 ? floor(v+0.5f)
 * : ceil(v-0.5f), every step rounded to fp32; clamp max(min(r,127),-127); fptosi. */
int orc_quantize(const float* x, size_t count, size_t inner, const float* scale, size_t nscale,
                 int8_t* y) {
  for (size_t i = 0; i < count; ++i) {
    const float s = nscale == 1 ? scale[0] : scale[(i / inner) % nscale];
    const volatile float v = x[i] * s;
    volatile float t;
    float r;
    if (v >= 0.0f) {
      t = v + 0.5f;
      r = floorf(t);
    } else {
      t = v + -0.5f;
      r = ceilf(t);
    }
    r = r < 127.0f ? r : 127.0f;
    r = r > -127.0f ? r : -127.0f;
    y[i] = (int8_t)r;
  }
  return 0;
}
