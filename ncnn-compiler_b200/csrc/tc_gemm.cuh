// Tensor-core contraction kernel for sm_100a: out[M,N] = epilogue(A[M,K] * B[N,K]^T).
//
// One kernel serves Convolution (A rows are output pixels gathered from an NHWC
// activation tensor by TMA im2col loads, K runs over filter taps x input
// channels), InnerProduct and Gemm (A is a plain row-major matrix loaded by
// tiled TMA).  B is always the packed weight matrix [N][K], K contiguous.
//
// Pipeline per CTA (persistent, one CTA per SM, 224 threads):
//   warps 0,6  TMA producers (A tiles / B tiles): fill a ring of shared-memory stages
//              (A tile 128 x K-block, B tile block_n x K-block, 128B/64B-swizzled rows)
//   warp 1     MMA issuer: tcgen05.mma from shared memory into one of two TMEM
//              accumulators (128 lanes x block_n fp32/int32 columns)
//   warps 2-5  epilogue: tcgen05.ld of the finished accumulator, then bias, residual,
//              activation, dequantise/requantise, store (fp32, fp32 split hi/lo, int8)
// The accumulator is double-buffered so the epilogue of tile i overlaps the
// main loop of tile i+1.
//
// Arithmetic kinds:
//   GEMM_TF32    one kind::tf32 MMA per K step (fast mode, ~1e-3 relative error)
//   GEMM_TF32X3  operands are stored as hi/lo tf32 planes (x = hi + lo exactly);
//                three MMAs lo*hi + hi*lo + hi*hi recover ~fp32 accuracy
//   GEMM_BF16X3  operands are stored as two bf16 planes (x ~ hi + mid, 16 significant bits);
//                three kind::f16 MMAs mid*hi + hi*mid + hi*hi, each at twice the tf32 rate
//                on half the operand bytes, give ~1e-5 relative error
//   GEMM_I8      kind::i8, int32 accumulation, exact
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "ptx_sm100.cuh"

namespace nb {

enum : int { GEMM_TF32 = 0, GEMM_TF32X3 = 1, GEMM_I8 = 2, GEMM_BF16X3 = 3 };

__host__ __device__ constexpr int tc_planes(int kind) { return kind == GEMM_TF32X3 || kind == GEMM_BF16X3 ? 2 : 1; }
__host__ __device__ constexpr int tc_elem_bytes(int kind) { return kind == GEMM_I8 ? 1 : (kind == GEMM_BF16X3 ? 2 : 4); }
// ACT_SIGMOID..ACT_SCALE follow the reference's separate activation ops:
//   SIGMOID      1/(1+exp(-clamp(x, +-88.376...)))            (ConvertSigmoid, NCNNToTosa.cpp:2991-3021)
//   SWISH        x * 1/(1+exp(-x))                            (ConvertSwish, :3702-3720)
//   HARDSIGMOID  clamp(x*alpha + beta, 0, 1), HARDSWISH x * that (ConvertHardActivation, :3023-3072)
//   TANH         tanh(x)                                      (ConvertTanH, :3722-3736)
//   SCALE        x * a                                        (ConvertDropout, :2047-2070)
//   SQUARE       x * x                                        (ConvertUnary, :5225-5252)
enum : int {
  ACT_NONE = 0, ACT_RELU = 1, ACT_LEAKY = 2, ACT_CLIP = 3, ACT_SIGMOID = 4, ACT_SWISH = 5, ACT_HARDSIGMOID = 6,
  ACT_HARDSWISH = 7, ACT_TANH = 8, ACT_SCALE = 9, ACT_SQUARE = 10, ACT_GELU = 11
};
// OUT_F32        plain fp32
// OUT_F32_SPLIT  two fp32 planes: hi = value rounded to tf32, lo = value - hi
// OUT_I8         int8 after requantisation with out_scale
// OUT_F32_TF32   fp32 rounded to tf32 (fast mode keeps operands unbiased)
// OUT_BF16X2     two bf16 planes: hi = bf16(value), mid = bf16(value - hi)
enum : int { OUT_F32 = 0, OUT_F32_SPLIT = 1, OUT_I8 = 2, OUT_F32_TF32 = 3, OUT_BF16X2 = 4 };
// format of the optional residual operand of the epilogue
enum : int { RES_NONE = 0, RES_F32 = 1, RES_SPLIT = 2, RES_BF16X2 = 3 };

enum : int {
  TC_OK = 0,
  TC_TIMEOUT_PRODUCER = 1,
  TC_TIMEOUT_MMA = 2,
  TC_TIMEOUT_EPILOGUE = 3,
};

constexpr int kTcThreads = 224;      // warps: 0 A producer, 1 MMA issuer, 2-5 epilogue, 6 B producer
constexpr int kTcThreadsTwoEpi = 352;  // + warps 7-10: a second epilogue group for shallow contractions
constexpr int kTcBlockM = 128;
constexpr int kTcMaxStages = 8;
constexpr uint32_t kTcTmemCols = 512;           // two accumulators of up to 128 columns, or two pairs of them
constexpr uint64_t kTcWaitLimitNs = 2000000000ull;  // a wait longer than 2 s is a bug

struct TcGemmParams {
  int M, N;
  int tiles_m, tiles_n, block_n;
  int k_blocks;   // K iterations per tile = taps * c_blocks
  int c_blocks;   // channel blocks per filter tap (K blocks for a plain GEMM)
  int k_elems;    // elements per K block
  int row_bytes;  // bytes per shared-memory operand row: 128 or 64
  int stages;
  int stage_bytes;  // bytes of one ring stage: planes * (A tile + B tile rounded to 1 KB)
  int a_im2col;  // A addressing: 0 plain matrix (tiled TMA), 1 im2col TMA
  int OH, OW, KW;
  int stride_h, stride_w, pad_t, pad_l, dil_h, dil_w;
  // epilogue
  const float* bias;   // [N] or null
  const float* scale;  // [N] int8 dequantisation factor 1/(s_w*s_in), GEMM_I8 only
  float* out0;
  float* out1;
  int8_t* outq;
  const float* res0;  // optional residual (same layout as the output), plane hi
  const float* res1;  // optional residual plane lo
  int res_mode;       // RES_*
  long long ldo;      // output row stride in elements
  int out_mode;
  int act;
  float act_a, act_b;  // leaky slope / clip bounds
  float out_scale;     // requantisation scale (OUT_I8)
  int* status;         // device words: [0] stays 0 unless a bounded wait gave up; [1] non-zero injects a stalled
                       // stage into tc_gemm_kernel (host tests of the time-out path), zero in production
  int tma_store;       // fp32 outputs leave through shared-memory staging tiles and TMA stores
  int staging_bytes;   // staging area of one epilogue group (residual + output tiles)
  int epi_groups;      // 1 or 2 epilogue warpgroups (2: accumulator g is drained by group g; shallow layers)
  int wide;            // staged chunks are 32 columns wide (always with bf16 pairs; plain fp32 when it pays)
  int out_bufs;        // staging tiles in flight (2..4), each 8 KB per output plane
  // 1: tiles may be two 128-row halves that share one B tile per K block: the A halves sit side by
  // side in a stage and accumulate into neighbouring column ranges.  The first pair_rows tile rows
  // are such pairs (256 rows each), the remaining tiles_m - pair_rows tile rows are single tiles:
  // whole waves of pairs, then a last wave that is not coarser than it has to be.
  int pair;
  int pair_rows;
  int sub_blocks;  // int8: K blocks per ring stage (one barrier hand-shake for several small copies); 1 elsewhere
  long long* trace;    // optional (bring-up): per-role clock stamps of CTA 0, 8 values per tile
  // CTA pairs (tc_gemm2.cuh): tiles are 256 rows, tiles_m counts those.
  // streamk = 1: every pair gets an equal share of all (tile, K block) units, so a tile may be split
  // between neighbouring pairs; the pair that holds a tile's last K block adds the others' partial
  // accumulators (exchanged through sk_ws) and runs the epilogue.
  int streamk;
  // Quantised copies of an fp32 result for the int8 contractions that read it next (up to two, each with
  // its consumer's input scale): written by the epilogue next to the fp32 tensor, so no Quantize pass
  // re-reads it.  Q(.) is the reference's (NCNNToTosa.cpp:356-385) applied to the value that is stored.
  int side_count;
  int8_t* side_q0;
  int8_t* side_q1;
  float side_scale0, side_scale1;
  long long side_ld;   // row stride of the int8 copies in elements
  int side_staged;     // the copies leave through staging tiles and TMA stores (tc_gemm_kernel, channels in 64s)
  uint32_t* sk_ws;     // one slot of 128 x block_n accumulator words per CTA
  int* sk_flags;       // one word per CTA: 1 while its slot holds a partial that nobody has consumed
};

// round-half-away-from-zero exactly as the reference evaluates it in fp32:
// floor(v + 0.5f) for v >= 0, ceil(v - 0.5f) otherwise, then clamp to [-127, 127].
__device__ __forceinline__ int quantize_rha(float x, float s) {
  const float v = __fmul_rn(x, s);
  const float r = v >= 0.0f ? floorf(__fadd_rn(v, 0.5f)) : ceilf(__fadd_rn(v, -0.5f));
  const float c = fmaxf(fminf(r, 127.0f), -127.0f);
  return static_cast<int>(c);
}

__device__ __forceinline__ float round_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// two floats -> two bf16 (round to nearest even), `a` in the low half
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ float bf16_low(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_high(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
// hi = bf16(x), mid = bf16(x - hi) for two values at once
__device__ __forceinline__ void split_bf16x2(float a, float b, uint32_t& hi, uint32_t& mid) {
  hi = pack_bf16x2(a, b);
  mid = pack_bf16x2(__fadd_rn(a, -bf16_low(hi)), __fadd_rn(b, -bf16_high(hi)));
}

// The activations a network seldom uses live in one function that is called, not inlined: an epilogue applies its
// activation to 16 or 32 values in a row, and a copy of every branch per value made the loops large enough to
// stall on instruction fetch (a 3x3 depthwise block spent 5000 cycles there instead of 400).
static __device__ __noinline__ float apply_act_rare(float y, int act, float a, float b) {
  if (act == ACT_SIGMOID) {
    const float c = fminf(fmaxf(y, -88.3762626647949f), 88.3762626647949f);
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-c)));
  }
  if (act == ACT_SWISH) return __fmul_rn(y, __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-y))));
  if (act == ACT_HARDSIGMOID || act == ACT_HARDSWISH) {
    const float gate = fminf(fmaxf(__fadd_rn(__fmul_rn(y, a), b), 0.0f), 1.0f);
    return act == ACT_HARDSWISH ? __fmul_rn(y, gate) : gate;
  }
  if (act == ACT_TANH) return tanhf(y);
  if (act == ACT_SCALE) return __fmul_rn(y, a);
  if (act == ACT_SQUARE) return __fmul_rn(y, y);
  // (x * erfc(x * -1/sqrt(2))) * 0.5, the order of ConvertGELU (NCNNToTosa.cpp:4670-4738)
  if (act == ACT_GELU) return __fmul_rn(__fmul_rn(y, erfcf(__fmul_rn(y, -0.7071067811865476f))), 0.5f);
  return y;
}

__device__ __forceinline__ float apply_act(float y, int act, float a, float b) {
  if (act == ACT_NONE) return y;
  if (act == ACT_RELU) return fmaxf(y, 0.0f);
  if (act == ACT_CLIP) return fminf(fmaxf(y, a), b);
  if (act == ACT_LEAKY) return y >= 0.0f ? y : __fmul_rn(y, a);
  return apply_act_rare(y, act, a, b);
}

// 16 fp32 results of one row -> 16 int8 with the reference's rounding, one 16-byte store
__device__ __forceinline__ void tc_store_side_quant(int8_t* q, float scale, const float (&y)[16]) {
  uint32_t w[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    w[g] = (static_cast<uint32_t>(quantize_rha(y[4 * g + 0], scale)) & 0xffu) |
           ((static_cast<uint32_t>(quantize_rha(y[4 * g + 1], scale)) & 0xffu) << 8) |
           ((static_cast<uint32_t>(quantize_rha(y[4 * g + 2], scale)) & 0xffu) << 16) |
           ((static_cast<uint32_t>(quantize_rha(y[4 * g + 3], scale)) & 0xffu) << 24);
  }
  *reinterpret_cast<uint4*>(q) = make_uint4(w[0], w[1], w[2], w[3]);
}

// the same 16 bytes into a shared-memory staging tile
__device__ __forceinline__ void tc_stage_side_quant(uint32_t smem_at, float scale, const float (&y)[16]) {
  uint32_t w[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    w[g] = (static_cast<uint32_t>(quantize_rha(y[4 * g + 0], scale)) & 0xffu) |
           ((static_cast<uint32_t>(quantize_rha(y[4 * g + 1], scale)) & 0xffu) << 8) |
           ((static_cast<uint32_t>(quantize_rha(y[4 * g + 2], scale)) & 0xffu) << 16) |
           ((static_cast<uint32_t>(quantize_rha(y[4 * g + 3], scale)) & 0xffu) << 24);
  }
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(smem_at), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
               : "memory");
}

// BF16IO: a bf16-pair tensor takes part (as output or residual); kept out of the other
// instantiation so that the int8 and plain fp32 epilogues stay lean.
template <int KIND, bool BF16IO, bool SIDE = false>
__device__ __forceinline__ void tc_epilogue_chunk(const TcGemmParams& p, const uint32_t (&v)[16],
                                                  long long m, int n_first, const float* tile_bias,
                                                  const float* tile_scale) {
  float y[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int n = n_first + j;
    float t;
    if (n < p.N) {
      if (KIND == GEMM_I8) {
        t = __fmul_rn(static_cast<float>(static_cast<int>(v[j])), tile_scale[j]);
      } else {
        t = __uint_as_float(v[j]);
      }
      if (p.bias != nullptr) t = __fadd_rn(t, tile_bias[j]);
    } else {
      t = 0.0f;
    }
    y[j] = t;
  }
  const long long row = m * p.ldo;
  const bool vec4 = (p.ldo % 4 == 0) && (n_first % 4 == 0);
  if (BF16IO && p.res_mode == RES_BF16X2) {
    const uint16_t* r0 = reinterpret_cast<const uint16_t*>(p.res0);
    const uint16_t* r1 = reinterpret_cast<const uint16_t*>(p.res1);
    if ((p.ldo % 8 == 0) && n_first + 15 < p.N) {
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(r0 + row + n_first + 8 * g));
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(r1 + row + n_first + 8 * g));
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          y[8 * g + 2 * e] = __fadd_rn(y[8 * g + 2 * e], __fadd_rn(bf16_low(aw[e]), bf16_low(bw[e])));
          y[8 * g + 2 * e + 1] = __fadd_rn(y[8 * g + 2 * e + 1], __fadd_rn(bf16_high(aw[e]), bf16_high(bw[e])));
        }
      }
    } else {
      for (int j = 0; j < 16; ++j)
        if (n_first + j < p.N)
          y[j] = __fadd_rn(y[j], __fadd_rn(__uint_as_float(static_cast<uint32_t>(r0[row + n_first + j]) << 16),
                                           __uint_as_float(static_cast<uint32_t>(r1[row + n_first + j]) << 16)));
    }
  } else if (p.res0 != nullptr) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int n = n_first + 4 * g;
      if (vec4 && n + 3 < p.N) {
        float4 r = __ldg(reinterpret_cast<const float4*>(p.res0 + row + n));
        if (p.res1 != nullptr) {
          const float4 l = __ldg(reinterpret_cast<const float4*>(p.res1 + row + n));
          r.x = __fadd_rn(r.x, l.x);
          r.y = __fadd_rn(r.y, l.y);
          r.z = __fadd_rn(r.z, l.z);
          r.w = __fadd_rn(r.w, l.w);
        }
        y[4 * g + 0] = __fadd_rn(y[4 * g + 0], r.x);
        y[4 * g + 1] = __fadd_rn(y[4 * g + 1], r.y);
        y[4 * g + 2] = __fadd_rn(y[4 * g + 2], r.z);
        y[4 * g + 3] = __fadd_rn(y[4 * g + 3], r.w);
      } else {
        for (int e = 0; e < 4; ++e) {
          if (n + e < p.N) {
            float r = __ldg(p.res0 + row + n + e);
            if (p.res1 != nullptr) r = __fadd_rn(r, __ldg(p.res1 + row + n + e));
            y[4 * g + e] = __fadd_rn(y[4 * g + e], r);
          }
        }
      }
    }
  }
  if (p.out_mode == OUT_I8) {
    int q[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      int t = quantize_rha(y[j], p.out_scale);
      if (p.act == ACT_RELU) t = max(t, 0);
      q[j] = t;
    }
    if ((p.ldo % 16 == 0) && (n_first % 16 == 0) && n_first + 15 < p.N) {
      uint32_t w[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        w[g] = (static_cast<uint32_t>(q[4 * g + 0]) & 0xffu) |
               ((static_cast<uint32_t>(q[4 * g + 1]) & 0xffu) << 8) |
               ((static_cast<uint32_t>(q[4 * g + 2]) & 0xffu) << 16) |
               ((static_cast<uint32_t>(q[4 * g + 3]) & 0xffu) << 24);
      }
      *reinterpret_cast<uint4*>(p.outq + row + n_first) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      for (int j = 0; j < 16; ++j)
        if (n_first + j < p.N) p.outq[row + n_first + j] = static_cast<int8_t>(q[j]);
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) y[j] = apply_act(y[j], p.act, p.act_a, p.act_b);
  if (SIDE && p.side_count > 0) {
    tc_store_side_quant(p.side_q0 + m * p.side_ld + n_first, p.side_scale0, y);
    if (p.side_count > 1) tc_store_side_quant(p.side_q1 + m * p.side_ld + n_first, p.side_scale1, y);
  }
  if (BF16IO && p.out_mode == OUT_BF16X2) {
    uint16_t* o0 = reinterpret_cast<uint16_t*>(p.out0);
    uint16_t* o1 = reinterpret_cast<uint16_t*>(p.out1);
    uint32_t hi[8], mid[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) split_bf16x2(y[2 * e], y[2 * e + 1], hi[e], mid[e]);
    if ((p.ldo % 8 == 0) && n_first + 15 < p.N) {
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        *reinterpret_cast<uint4*>(o0 + row + n_first + 8 * g) =
            make_uint4(hi[4 * g], hi[4 * g + 1], hi[4 * g + 2], hi[4 * g + 3]);
        *reinterpret_cast<uint4*>(o1 + row + n_first + 8 * g) =
            make_uint4(mid[4 * g], mid[4 * g + 1], mid[4 * g + 2], mid[4 * g + 3]);
      }
    } else {
      for (int j = 0; j < 16; ++j) {
        if (n_first + j < p.N) {
          o0[row + n_first + j] = static_cast<uint16_t>(j & 1 ? hi[j >> 1] >> 16 : hi[j >> 1] & 0xffffu);
          o1[row + n_first + j] = static_cast<uint16_t>(j & 1 ? mid[j >> 1] >> 16 : mid[j >> 1] & 0xffffu);
        }
      }
    }
    return;
  }
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int n = n_first + 4 * g;
    float hi[4], lo[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float t = y[4 * g + e];
      if (p.out_mode == OUT_F32) {
        hi[e] = t;
        lo[e] = 0.0f;
      } else {
        hi[e] = round_tf32(t);
        lo[e] = __fadd_rn(t, -hi[e]);
      }
    }
    if (vec4 && n + 3 < p.N) {
      *reinterpret_cast<float4*>(p.out0 + row + n) = make_float4(hi[0], hi[1], hi[2], hi[3]);
      if (p.out_mode == OUT_F32_SPLIT)
        *reinterpret_cast<float4*>(p.out1 + row + n) = make_float4(lo[0], lo[1], lo[2], lo[3]);
    } else {
      for (int e = 0; e < 4; ++e) {
        if (n + e < p.N) {
          p.out0[row + n + e] = hi[e];
          if (p.out_mode == OUT_F32_SPLIT) p.out1[row + n + e] = lo[e];
        }
      }
    }
  }
}

// fp32 result of 16 accumulator columns: dequantise / bias, residual, activation.  Every
// scalar arrives by value (a reference to the kernel-parameter struct turns each field
// access into a generic load) and every decision is taken outside the unrolled loops: one
// thread's branches are not hidden by other warps here.  `bias` and `res` hold zeros when
// the layer has none (adding +0 changes at most the sign of a zero).
template <int KIND>
__device__ __forceinline__ void tc_epilogue_values(const uint32_t (&v)[16], const float (&bias)[16],
                                                   const float (&scale)[16], const float (&res)[16],
                                                   int act, float act_a, float act_b,
                                                   float (&y)[16]) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    float t;
    if (KIND == GEMM_I8) {
      t = __fmul_rn(static_cast<float>(static_cast<int>(v[j])), scale[j]);
    } else {
      t = __uint_as_float(v[j]);
    }
    y[j] = __fadd_rn(__fadd_rn(t, bias[j]), res[j]);
  }
  if (act == ACT_RELU) {
#pragma unroll
    for (int j = 0; j < 16; ++j) y[j] = fmaxf(y[j], 0.0f);
  } else if (act == ACT_CLIP) {
#pragma unroll
    for (int j = 0; j < 16; ++j) y[j] = fminf(fmaxf(y[j], act_a), act_b);
  } else if (act == ACT_LEAKY) {
#pragma unroll
    for (int j = 0; j < 16; ++j) y[j] = y[j] >= 0.0f ? y[j] : __fmul_rn(y[j], act_a);
  } else if (act != ACT_NONE) {
#pragma unroll
    for (int j = 0; j < 16; ++j) y[j] = apply_act(y[j], act, act_a, act_b);
  }
}

// Staging tiles are [128 rows][16 fp32] with the 64-byte TMA swizzle: the 16-byte chunk j
// of row r lives at r*64 + ((j ^ ((r >> 1) & 3)) * 16).
__device__ __forceinline__ uint32_t stage_chunk_offset(int row, int j) {
  return static_cast<uint32_t>(row * 64 + ((j ^ ((row >> 1) & 3)) << 4));
}

// ---- staged epilogue shared by the contraction kernels --------------------------------
// Results leave through shared-memory staging tiles and TMA stores.  Shared-memory plan:
// 16 KB of residual tiles at res_stage, then out_bufs output tiles at out_stage.  A chunk is
// 16 accumulator columns, or 32 ("wide") as soon as a bf16-pair tensor takes part, because a
// staging row is 64 bytes: 16 fp32 or 32 bf16.  Tiles per chunk:
//   out  F32            one tile  [128][16 fp32]           (wide: two, columns +0 and +16)
//   out  F32_SPLIT      hi tile, lo tile                   (never wide)
//   out  BF16X2         hi tile, mid tile [128][32 bf16]   (always wide)
//   res  F32 / SPLIT / BF16X2 likewise in the residual area
// One barrier per chunk: all four warps write tile c, barrier, the leader stores it, waits
// until the tile that chunk c+2 will use has been read out, and fetches the residual of
// chunk c+1; the others learn all that at the barrier of chunk c+1.
struct TcStageCfg {
  uint32_t res_stage, out_stage, res_bar;
  int out_bufs, out_mode, res_mode;
  int act;
  float act_a, act_b;
  int N, block_n;
  int wide;      // 32-column chunks
  int bar_base;  // named barriers bar_base and bar_base + 1 belong to this epilogue group
  // partial accumulators of other CTAs to add before the epilogue (split tiles): fix_count slots,
  // the first at fix_ws, each fix_stride words after the one before; laid out [16-column group][row][16]
  const uint32_t* fix_ws;
  long long fix_stride;
  int fix_count;
  // int8 copies of the result (see TcGemmParams::side_q): pointers at this tile's first row and column,
  // rows of the tile that exist
  int side_count;
  int8_t* side_q0;
  int8_t* side_q1;
  float side_scale0, side_scale1;
  long long side_ld;
  int side_rows;
  // staged form of the int8 copies (side_stage != 0): 64 columns of a copy are collected in a [128][64]
  // int8 tile (64-byte swizzle, two tiles per copy used in turn) and leave through one TMA store
  // (io.store_side); otherwise every thread stores its 16 bytes itself
  uint32_t side_stage;
};


// Sum of the partial accumulators of one row over 16 columns.  The slots were written by other SMs
// during this launch: read them from L2, never through L1.
template <int KIND>
__device__ __forceinline__ void tc_load_partials(const TcStageCfg& c, int col, int row, uint32_t (&sum)[16]) {
  const uint32_t* src = c.fix_ws + (static_cast<size_t>(col >> 4) * 128 + row) * 16;
#pragma unroll
  for (int j = 0; j < 16; ++j) sum[j] = 0u;
  for (int i = 0; i < c.fix_count; ++i) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint4 a = __ldcg(reinterpret_cast<const uint4*>(src) + q);
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (KIND == GEMM_I8) sum[4 * q + e] += w[e];
        else sum[4 * q + e] = __float_as_uint(__fadd_rn(__uint_as_float(sum[4 * q + e]), __uint_as_float(w[e])));
      }
    }
    src += c.fix_stride;
  }
}

template <int KIND>
__device__ __forceinline__ void tc_add_partials(uint32_t (&v)[16], const uint32_t (&sum)[16]) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    if (KIND == GEMM_I8) v[j] += sum[j];
    else v[j] = __float_as_uint(__fadd_rn(__uint_as_float(v[j]), __uint_as_float(sum[j])));
  }
}

// IO: load_res(plane, smem_dst, bar, column) and store_out(plane, smem_src, column) issue the
// TMA copies of one staging tile; the caller binds tensor maps and row coordinates.
// EXTRAS: partial sums of split tiles and int8 copies of the result take part.  They are compiled out of
// the plain instantiation: an epilogue warp runs alone on its scheduler, so every instruction and every live
// register of a path that is not taken still costs the layers that never take it.
template <int KIND, class IO, bool EXTRAS = false>
__device__ __forceinline__ bool tc_staged_epilogue(const TcStageCfg c, const IO& io, uint32_t t_row, int n0,
                                                   int row, bool leader, const float* tile_bias,
                                                   const float* tile_scale, uint32_t& res_ph, int& out_slot,
                                                   volatile int* abort_ptr, int* side_slot = nullptr) {
  using namespace ptx;
  const bool has_res = c.res_mode != RES_NONE;
  const bool wide = c.wide != 0;
  const int cw = wide ? 32 : 16;
  const bool two_out = wide || c.out_mode == OUT_F32_SPLIT;
  const uint32_t out_tile_bytes = two_out ? 16384u : 8192u;
  const bool two_res = wide || c.res_mode == RES_SPLIT;
  auto fetch_res = [&](int col) {
    mbar_arrive_expect_tx(c.res_bar, two_res ? 16384u : 8192u);
    io.load_res(0, c.res_stage, c.res_bar, col);
    if (c.res_mode == RES_F32) {
      if (wide) io.load_res(0, c.res_stage + 8192u, c.res_bar, col + 16);
    } else {
      io.load_res(1, c.res_stage + 8192u, c.res_bar, col);
    }
  };
  if (leader && has_res) fetch_res(n0);
  named_barrier_sync(c.bar_base, 128);  // tile constants are in place
  bool ok = true;
  // split tiles: the other CTAs' partial sums, fetched one 16-column group ahead of their use
  uint32_t part[EXTRAS ? 16 : 1];
  if (EXTRAS && c.fix_count > 0) tc_load_partials<KIND>(c, 0, row, reinterpret_cast<uint32_t (&)[16]>(part));
  for (int c0 = 0; c0 < c.block_n && n0 + c0 < c.N; c0 += cw) {
    const uint32_t stage0 = c.out_stage + static_cast<uint32_t>(out_slot) * out_tile_bytes;
    if (has_res) {
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(c.res_bar, res_ph, abort_ptr, kTcWaitLimitNs) ? 1 : 0) != 0;
      res_ph ^= 1u;
      if (!ok) break;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (h == 1 && (!wide || n0 + c0 + 16 >= c.N)) break;  // (columns past N are clipped by the store)
      uint32_t v[16];
      tmem_ld16(t_row + static_cast<uint32_t>(c0 + 16 * h), v);
      tmem_ld_wait();
      if (EXTRAS && c.fix_count > 0) {
        tc_add_partials<KIND>(v, reinterpret_cast<uint32_t (&)[16]>(part));
        const int next = c0 + 16 * h + 16;
        if (next < c.block_n) tc_load_partials<KIND>(c, next, row, reinterpret_cast<uint32_t (&)[16]>(part));
      }
      float r[16];
      if (c.res_mode == RES_BF16X2) {
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const uint32_t off = stage_chunk_offset(row, 2 * h + jj);
          uint32_t a[4], b[4];
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
                       : "r"(c.res_stage + off));
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3])
                       : "r"(c.res_stage + 8192u + off));
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            r[8 * jj + 2 * e] = __fadd_rn(bf16_low(a[e]), bf16_low(b[e]));
            r[8 * jj + 2 * e + 1] = __fadd_rn(bf16_high(a[e]), bf16_high(b[e]));
          }
        }
      } else if (has_res) {
        const uint32_t base = c.res_stage + (wide ? 8192u * h : 0u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t off = stage_chunk_offset(row, j);
          float4 a;
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w)
                       : "r"(base + off));
          if (c.res_mode == RES_SPLIT) {
            float4 b;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(b.x), "=f"(b.y), "=f"(b.z), "=f"(b.w)
                         : "r"(base + 8192u + off));
            a.x = __fadd_rn(a.x, b.x);
            a.y = __fadd_rn(a.y, b.y);
            a.z = __fadd_rn(a.z, b.z);
            a.w = __fadd_rn(a.w, b.w);
          }
          r[4 * j + 0] = a.x;
          r[4 * j + 1] = a.y;
          r[4 * j + 2] = a.z;
          r[4 * j + 3] = a.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = 0.0f;
      }
      float y[16], cb[16], cs[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 b4 = *reinterpret_cast<const float4*>(&tile_bias[c0 + 16 * h + 4 * j]);
        cb[4 * j + 0] = b4.x;
        cb[4 * j + 1] = b4.y;
        cb[4 * j + 2] = b4.z;
        cb[4 * j + 3] = b4.w;
        if (KIND == GEMM_I8) {
          const float4 s4 = *reinterpret_cast<const float4*>(&tile_scale[c0 + 16 * h + 4 * j]);
          cs[4 * j + 0] = s4.x;
          cs[4 * j + 1] = s4.y;
          cs[4 * j + 2] = s4.z;
          cs[4 * j + 3] = s4.w;
        } else {
          cs[4 * j + 0] = cs[4 * j + 1] = cs[4 * j + 2] = cs[4 * j + 3] = 0.0f;
        }
      }
      tc_epilogue_values<KIND>(v, cb, cs, r, c.act, c.act_a, c.act_b, y);
      if (!EXTRAS) {
      } else if (c.side_count > 0 && c.side_stage != 0u) {
        // staged: this row's 16 bytes of the current 64-column group, tile *side_slot of each copy
        const uint32_t at = c.side_stage + static_cast<uint32_t>(*side_slot) * 8192u +
                            stage_chunk_offset(row, ((c0 + 16 * h) >> 4) & 3);
        tc_stage_side_quant(at, c.side_scale0, y);
        if (c.side_count > 1) tc_stage_side_quant(at + 16384u, c.side_scale1, y);
      } else if (c.side_count > 0 && row < c.side_rows && n0 + c0 + 16 * h < c.N) {
        const long long at = static_cast<long long>(row) * c.side_ld + c0 + 16 * h;
        tc_store_side_quant(c.side_q0 + at, c.side_scale0, y);
        if (c.side_count > 1) tc_store_side_quant(c.side_q1 + at, c.side_scale1, y);
      }
      if (c.out_mode == OUT_BF16X2) {
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          uint32_t hi[4], mid[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) split_bf16x2(y[8 * jj + 2 * e], y[8 * jj + 2 * e + 1], hi[e], mid[e]);
          const uint32_t off = stage_chunk_offset(row, 2 * h + jj);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage0 + off), "r"(hi[0]), "r"(hi[1]),
                       "r"(hi[2]), "r"(hi[3])
                       : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage0 + 8192u + off), "r"(mid[0]),
                       "r"(mid[1]), "r"(mid[2]), "r"(mid[3])
                       : "memory");
        }
      } else if (c.out_mode == OUT_F32) {
        const uint32_t base = stage0 + (wide ? 8192u * h : 0u);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(base + stage_chunk_offset(row, j)),
                       "f"(y[4 * j]), "f"(y[4 * j + 1]), "f"(y[4 * j + 2]), "f"(y[4 * j + 3])
                       : "memory");
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float hi[4], lo[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            hi[e] = round_tf32(y[4 * j + e]);
            lo[e] = __fadd_rn(y[4 * j + e], -hi[e]);
          }
          const uint32_t off = stage_chunk_offset(row, j);
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(stage0 + off), "f"(hi[0]), "f"(hi[1]),
                       "f"(hi[2]), "f"(hi[3])
                       : "memory");
          if (c.out_mode == OUT_F32_SPLIT)
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(stage0 + 8192u + off), "f"(lo[0]),
                         "f"(lo[1]), "f"(lo[2]), "f"(lo[3])
                         : "memory");
        }
      }
    }
    fence_proxy_async_smem();
    named_barrier_sync(c.bar_base + 1, 128);
    if (leader) {
      // rows and columns of a tile that fall outside the tensor are clipped by the store
      io.store_out(0, stage0, n0 + c0);
      if (c.out_mode == OUT_F32) {
        if (wide && n0 + c0 + 16 < c.N) io.store_out(0, stage0 + 8192u, n0 + c0 + 16);
      } else if (two_out) {
        io.store_out(1, stage0 + 8192u, n0 + c0);
      }
      if (EXTRAS && c.side_count > 0 && c.side_stage != 0u && (((c0 + cw) & 63) == 0 || c0 + cw >= c.block_n || n0 + c0 + cw >= c.N)) {
        const uint32_t src = c.side_stage + static_cast<uint32_t>(*side_slot) * 8192u;
        io.store_side(0, src, n0 + (c0 & ~63));
        if (c.side_count > 1) io.store_side(1, src + 16384u, n0 + (c0 & ~63));
      }
      tma_store_commit();
      tma_store_wait_read(c.out_bufs >= 2 ? c.out_bufs - 2 : 0);
      const int c1 = c0 + cw;
      if (has_res && c1 < c.block_n && n0 + c1 < c.N) fetch_res(n0 + c1);
    }
    // a single staging tile is written again only after its store has read it
    if (c.out_bufs == 1) named_barrier_sync(c.bar_base, 128);
    if (++out_slot >= c.out_bufs) out_slot = 0;
    // the other tile of each int8 copy for the next 64-column group (every thread keeps the same count)
    if (EXTRAS && c.side_count > 0 && c.side_stage != 0u && (((c0 + cw) & 63) == 0 || c0 + cw >= c.block_n || n0 + c0 + cw >= c.N))
      *side_slot ^= 1;
  }
  return ok;
}

// Staged epilogue for int8 results (no residual): a chunk is 64 accumulator columns, one
// 64-byte staging row of int8 per accumulator row.  Dequantise, add the bias, requantise with
// out_scale, clamp at zero for a fused ReLU (the order of the reference's int8 path), pack, and
// store the [128][64] tile with one TMA store.
template <int KIND, class IO, bool EXTRAS = false>
__device__ __forceinline__ void tc_staged_epilogue_i8(const TcStageCfg c, float out_scale, const IO& io,
                                                      uint32_t t_row, int n0, int row, bool leader,
                                                      const float* tile_bias, const float* tile_scale,
                                                      int& out_slot) {
  using namespace ptx;
  named_barrier_sync(c.bar_base, 128);  // tile constants are in place
  uint32_t part[EXTRAS ? 16 : 1];
  if (EXTRAS && c.fix_count > 0) tc_load_partials<KIND>(c, 0, row, reinterpret_cast<uint32_t (&)[16]>(part));
  for (int c0 = 0; c0 < c.block_n && n0 + c0 < c.N; c0 += 64) {
    const uint32_t stage0 = c.out_stage + static_cast<uint32_t>(out_slot) * 8192u;
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      uint32_t v[16];
      tmem_ld16(t_row + static_cast<uint32_t>(c0 + 16 * h), v);
      tmem_ld_wait();
      if (EXTRAS && c.fix_count > 0) {
        tc_add_partials<KIND>(v, reinterpret_cast<uint32_t (&)[16]>(part));
        const int next = c0 + 16 * h + 16;
        if (next < c.block_n) tc_load_partials<KIND>(c, next, row, reinterpret_cast<uint32_t (&)[16]>(part));
      }
      uint32_t w[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const float4 b4 = *reinterpret_cast<const float4*>(&tile_bias[c0 + 16 * h + 4 * g]);
        const float4 s4 = *reinterpret_cast<const float4*>(&tile_scale[c0 + 16 * h + 4 * g]);
        const float bias[4] = {b4.x, b4.y, b4.z, b4.w}, scale[4] = {s4.x, s4.y, s4.z, s4.w};
        uint32_t word = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float t = KIND == GEMM_I8 ? __fmul_rn(static_cast<float>(static_cast<int>(v[4 * g + e])), scale[e])
                                    : __uint_as_float(v[4 * g + e]);
          t = __fadd_rn(t, bias[e]);
          int q = quantize_rha(t, out_scale);
          if (c.act == ACT_RELU) q = max(q, 0);
          word |= (static_cast<uint32_t>(q) & 0xffu) << (8 * e);
        }
        w[g] = word;
      }
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage0 + stage_chunk_offset(row, h)), "r"(w[0]),
                   "r"(w[1]), "r"(w[2]), "r"(w[3])
                   : "memory");
    }
    fence_proxy_async_smem();
    named_barrier_sync(c.bar_base + 1, 128);
    if (leader) {
      io.store_out(0, stage0, n0 + c0);
      tma_store_commit();
      tma_store_wait_read(c.out_bufs - 2);
    }
    if (++out_slot == c.out_bufs) out_slot = 0;
  }
}

// SIDE: the instantiation that also writes int8 copies of its fp32 result (TcGemmParams::side_q); kept out
// of the plain kernel so that layers without such copies run exactly the code they ran before.
template <int KIND, bool SIDE = false>
__global__ void __launch_bounds__(kTcThreadsTwoEpi, 1)
tc_gemm_kernel(const __grid_constant__ TcGemmParams p, const __grid_constant__ CUtensorMap map_a0,
               const __grid_constant__ CUtensorMap map_a1,
               const __grid_constant__ CUtensorMap map_b0,
               const __grid_constant__ CUtensorMap map_b1,
               const __grid_constant__ CUtensorMap map_o0,
               const __grid_constant__ CUtensorMap map_o1,
               const __grid_constant__ CUtensorMap map_r0,
               const __grid_constant__ CUtensorMap map_r1,
               const __grid_constant__ CUtensorMap map_s0,
               const __grid_constant__ CUtensorMap map_s1) {
  using namespace ptx;
  grid_dependency_trigger();  // the next kernel of the stream may begin its preamble
  constexpr int PLANES = tc_planes(KIND);

  extern __shared__ uint8_t tc_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kTcMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kTcMaxStages];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];
  __shared__ __align__(8) uint64_t res_bar[2];
  __shared__ __align__(16) float tile_bias_all[2][128];
  __shared__ __align__(16) float tile_scale_all[2][128];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(tc_smem_raw) + 1023u) & ~1023u;
  const uint32_t slot = static_cast<uint32_t>(kTcBlockM) * p.row_bytes;
  const uint32_t stage_bytes = static_cast<uint32_t>(p.stage_bytes);
  const int AS = p.pair ? 2 : 1;  // A tiles per stage
  const uint32_t b_slot = (stage_bytes / PLANES) - static_cast<uint32_t>(AS) * slot;  // B tile, rounded to 1 KB
  const uint32_t tx_bytes = PLANES * (slot + static_cast<uint32_t>(p.block_n) * p.row_bytes);
  const int S = p.stages;
  // int8 K blocks are small (two MMAs over 12 KB for 64 channels): a stage holds SUB of them, so that the
  // ~450 cycles of arming and releasing a stage are paid once per SUB blocks
  const int SUB = KIND == GEMM_I8 ? (p.sub_blocks > 1 ? p.sub_blocks : 1) : 1;
  const int k_groups = p.k_blocks / SUB;
  const int total_tiles = p.tiles_m * p.tiles_n;
  volatile int* abort_ptr = &abort_flag;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < S; ++i) {
      mbar_init(smem_u32(&full_bar[i]), 2);  // one arrival per producer warp
      mbar_init(smem_u32(&empty_bar[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&tfull_bar[i]), 1);
      mbar_init(smem_u32(&tempty_bar[i]), 4);
    }
    mbar_init(smem_u32(&res_bar[0]), 1);
    mbar_init(smem_u32(&res_bar[1]), 1);
    fence_mbar_init();
    prefetch_tensormap(&map_a0);
    prefetch_tensormap(&map_b0);
    if (PLANES == 2) {
      prefetch_tensormap(&map_a1);
      prefetch_tensormap(&map_b1);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), kTcTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  // barriers, tensor memory and descriptors are ready: from here on the kernel touches tensors that the
  // kernel before it in the stream may still be writing
  grid_dependency_wait();
  // Fault injection for the time-out path (host tests only; status[1] is zero in production): the first
  // tile's first stage is never armed, so the MMA issuer's bounded wait on it runs out, every role leaves
  // through the abort path, and the host reads status 7.  The limit shrinks to 2 ms for such a run.
  const int test_stall = p.status[1];
  const uint64_t wait_limit = test_stall ? 2000000ull : kTcWaitLimitNs;

  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------ producers
    // Arming a stage and issuing its copies costs the issuing thread several hundred cycles per
    // K block (about 450 for the barrier hand-shake plus about 120 per TMA instruction, whatever
    // the box size), more than the MMAs of a narrow K block take.  So the work is split: warp 0
    // feeds the A tiles, warp 6 the B tiles, each arming the stage for its own bytes (the full
    // barrier counts two arrivals).  Within a warp lane p issues plane p.
    const bool is_b = warp == 6;
    // (paired tiles: lanes PLANES..2*PLANES-1 of the A warp issue the second half's planes)
    // (int8 with several K blocks per stage, never paired: lane b issues the copy of the stage's K block b, so
    // the copies of a stage cost the warp one instruction's time, not one each)
    const bool by_block = KIND == GEMM_I8 && SUB > 1;
    const bool issuer = by_block ? lane < SUB : lane < (is_b ? PLANES : PLANES * AS);
    const int my_sb = by_block ? lane : 0;
    const int my_plane = by_block ? 0 : lane % PLANES;
    const int my_half = is_b || by_block ? 0 : lane / PLANES;
    const CUtensorMap* my_map = is_b ? (my_plane ? &map_b1 : &map_b0) : (my_plane ? &map_a1 : &map_a0);
    const uint32_t my_lane_slot = by_block ? 0u : static_cast<uint32_t>(lane);
    const uint32_t my_off = is_b ? static_cast<uint32_t>(PLANES * AS) * slot + my_lane_slot * b_slot : my_lane_slot * slot;
    const uint32_t b_tx = PLANES * static_cast<uint32_t>(p.block_n) * p.row_bytes;
    int s = 0;
    uint32_t ph = 0;
    long long issued = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int m_blk = tile / p.tiles_n;
      const int n_blk = tile - m_blk * p.tiles_n;
      const bool pair_tile = m_blk < p.pair_rows;
      // a second half that starts past the last row repeats the first (its results are never stored)
      long long m0 = pair_tile ? static_cast<long long>(m_blk) * (2 * kTcBlockM)
                               : static_cast<long long>(p.pair_rows) * (2 * kTcBlockM) +
                                     static_cast<long long>(m_blk - p.pair_rows) * kTcBlockM;
      if (pair_tile && m0 + static_cast<long long>(my_half) * kTcBlockM < p.M) m0 += static_cast<long long>(my_half) * kTcBlockM;
      const bool issues = issuer && (is_b || pair_tile || my_half == 0);
      const uint32_t my_tx = is_b ? b_tx : static_cast<uint32_t>(PLANES * (pair_tile ? 2 : 1)) * slot;
      const int n0 = n_blk * p.block_n;
      int img = 0, h_base = 0, w_base = 0;
      if (p.a_im2col) {
        const long long per_img = static_cast<long long>(p.OH) * p.OW;
        img = static_cast<int>(m0 / per_img);
        const int r = static_cast<int>(m0 - img * per_img);
        const int oh = r / p.OW;
        const int ow = r - oh * p.OW;
        h_base = oh * p.stride_h - p.pad_t;
        w_base = ow * p.stride_w - p.pad_l;
      }
      if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) p.trace[(tile / gridDim.x) * 16 + 0] = clock64();
      // this lane's K block: channel block, filter row and column (lanes that issue by block start at theirs)
      int cb = 0, kh = 0, kw = 0;
      auto next_k_block = [&]() {
        if (++cb == p.c_blocks) {
          cb = 0;
          if (++kw == p.KW) {
            kw = 0;
            ++kh;
          }
        }
      };
      for (int kg = 0; kg < k_groups; ++kg) {
        const uint32_t fb = smem_u32(&full_bar[s]);
        int w = 1;
        if (lane == 0) {
          w = mbar_wait_bounded(smem_u32(&empty_bar[s]), ph ^ 1u, abort_ptr, wait_limit) ? 1 : 0;
          if (w && !(test_stall && kg == 0 && tile == static_cast<int>(blockIdx.x))) mbar_arrive_expect_tx(fb, my_tx * static_cast<uint32_t>(SUB));
        }
        w = __shfl_sync(0xffffffffu, w, 0);
        if (!w) {
          ok = false;
          break;
        }
        const bool tr = p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0 && tile == static_cast<int>(gridDim.x) && kg < 32;
        if (tr) p.trace[1024 + kg * 4 + 0] = clock64();
        {
          const int kb = kg * SUB + my_sb;
          if (by_block) {
            // (computed, not stepped: lanes that step by different amounts would diverge and issue one by one)
            const int tap = kb / p.c_blocks;
            cb = kb - tap * p.c_blocks;
            kh = tap / p.KW;
            kw = tap - kh * p.KW;
          }
          if (issues && !(test_stall && kg == 0 && tile == static_cast<int>(blockIdx.x))) {
            const uint32_t dst = smem_base + static_cast<uint32_t>(s * SUB + my_sb) * stage_bytes + my_off;
            if (is_b) {
              tma_load_2d(dst, my_map, fb, kb * p.k_elems, n0);
            } else if (p.a_im2col) {
              tma_load_im2col_4d(dst, my_map, fb, cb * p.k_elems, w_base, h_base, img,
                                 static_cast<uint16_t>(kw * p.dil_w), static_cast<uint16_t>(kh * p.dil_h));
            } else {
              tma_load_2d(dst, my_map, fb, kb * p.k_elems, static_cast<int>(m0));
            }
          }
          if (!by_block) next_k_block();
        }
        if (tr) p.trace[1024 + kg * 4 + 1] = clock64();
        ++issued;
        if (++s == S) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
    if (lane == 0) {
      if (!ok) {
        if (atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_PRODUCER);
      }
      if (*abort_ptr != 0) {
        // Some role gave up.  Copies this warp issued may still be landing in
        // shared memory: wait (bounded) for each of the last S fills to finish.
        int zero = 0;
        const long long first = issued > S ? issued - S : 0;
        for (long long i = first; i < issued; ++i) {
          const int st = static_cast<int>(i % S);
          const uint32_t par = static_cast<uint32_t>((i / S) & 1);
          mbar_wait_bounded(smem_u32(&full_bar[st]), par, &zero, test_stall ? 2000000ull : 200000000ull);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      // formats: kind::i8 s32 <- s8 (2, 1); kind::tf32 f32 <- tf32 (1, 2); kind::f16 f32 <- bf16 (1, 1)
      const uint32_t idesc = KIND == GEMM_I8
                                 ? instr_desc(2u, 1u, kTcBlockM, static_cast<uint32_t>(p.block_n))
                                 : instr_desc(1u, KIND == GEMM_BF16X3 ? 1u : 2u, kTcBlockM,
                                              static_cast<uint32_t>(p.block_n));
      // One thread issues every MMA, so its instruction stream is the critical path:
      // descriptors are formed by adding small constants to values computed once.
      // (the start-address field counts 16-byte units; a K step is 32 bytes = 2 units)
      const int k_steps = p.row_bytes / 32;
      const int k_blocks = p.k_blocks;
      const uint64_t desc_fixed = smem_desc_kmajor(0u, static_cast<uint32_t>(p.row_bytes));
      const uint64_t a_first = desc_fixed + ((smem_base & 0x3ffffu) >> 4);
      const uint64_t stage_units = stage_bytes >> 4;
      const uint64_t slot_units = slot >> 4;
      const uint64_t b_slot_units = b_slot >> 4;
      const uint64_t a1_from_a = static_cast<uint64_t>(PLANES) * slot_units;  // second half's planes
      const uint64_t b_from_a = static_cast<uint64_t>(PLANES * AS) * slot_units;
      const uint32_t acc_stride = p.pair ? 256u : 128u;
      const int pair_rows = p.pair_rows;
      const int tiles_n = p.tiles_n;
      const bool tracing = p.trace != nullptr && blockIdx.x == 0;
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait_bounded(smem_u32(&tempty_bar[acc]), acc_ph ^ 1u, abort_ptr, wait_limit)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (tracing) p.trace[(tile / gridDim.x) * 16 + 1] = clock64();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * acc_stride;
        const uint32_t d_tmem1 = d_tmem + 128u;
        const bool pair = tile / tiles_n < pair_rows;
        uint32_t accumulate = 0u;
        for (int kb = 0; kb < k_groups; ++kb) {
          if (!mbar_wait_bounded(smem_u32(&full_bar[s]), ph, abort_ptr, wait_limit)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const bool tr = tracing && tile == static_cast<int>(gridDim.x) && kb < 32;
          if (tr) p.trace[1024 + kb * 4 + 2] = clock64();
          for (int sb = 0; sb < SUB; ++sb) {
          const uint64_t a0 = a_first + static_cast<uint64_t>(s * SUB + sb) * stage_units;
          const uint64_t b0 = a0 + b_from_a;
          if (!pair) {
#pragma unroll 4
          for (int k = 0; k < k_steps; ++k) {
            const uint64_t ka = a0 + 2u * k;
            const uint64_t kbd = b0 + 2u * k;
            if (KIND == GEMM_TF32) {
              mma_tf32(d_tmem, ka, kbd, idesc, accumulate);
            } else if (KIND == GEMM_TF32X3) {
              mma_tf32(d_tmem, ka + slot_units, kbd, idesc, accumulate);  // lo * hi
              mma_tf32(d_tmem, ka, kbd + b_slot_units, idesc, 1u);        // hi * lo
              mma_tf32(d_tmem, ka, kbd, idesc, 1u);                       // hi * hi
            } else if (KIND == GEMM_BF16X3) {
              mma_f16(d_tmem, ka + slot_units, kbd, idesc, accumulate);  // mid * hi
              mma_f16(d_tmem, ka, kbd + b_slot_units, idesc, 1u);        // hi * mid
              mma_f16(d_tmem, ka, kbd, idesc, 1u);                       // hi * hi
            } else {
              mma_i8(d_tmem, ka, kbd, idesc, accumulate);
            }
            accumulate = 1u;
          }
          } else {
            // both halves against the same B tile; each half has its own accumulator columns
#pragma unroll 4
            for (int k = 0; k < k_steps; ++k) {
              const uint64_t ka = a0 + 2u * k;
              const uint64_t ka1 = ka + a1_from_a;
              const uint64_t kbd = b0 + 2u * k;
              if (KIND == GEMM_TF32) {
                mma_tf32(d_tmem, ka, kbd, idesc, accumulate);
                mma_tf32(d_tmem1, ka1, kbd, idesc, accumulate);
              } else if (KIND == GEMM_TF32X3) {
                mma_tf32(d_tmem, ka + slot_units, kbd, idesc, accumulate);
                mma_tf32(d_tmem, ka, kbd + b_slot_units, idesc, 1u);
                mma_tf32(d_tmem, ka, kbd, idesc, 1u);
                mma_tf32(d_tmem1, ka1 + slot_units, kbd, idesc, accumulate);
                mma_tf32(d_tmem1, ka1, kbd + b_slot_units, idesc, 1u);
                mma_tf32(d_tmem1, ka1, kbd, idesc, 1u);
              } else if (KIND == GEMM_BF16X3) {
                mma_f16(d_tmem, ka + slot_units, kbd, idesc, accumulate);
                mma_f16(d_tmem, ka, kbd + b_slot_units, idesc, 1u);
                mma_f16(d_tmem, ka, kbd, idesc, 1u);
                mma_f16(d_tmem1, ka1 + slot_units, kbd, idesc, accumulate);
                mma_f16(d_tmem1, ka1, kbd + b_slot_units, idesc, 1u);
                mma_f16(d_tmem1, ka1, kbd, idesc, 1u);
              } else {
                mma_i8(d_tmem, ka, kbd, idesc, accumulate);
                mma_i8(d_tmem1, ka1, kbd, idesc, accumulate);
              }
              accumulate = 1u;
            }
          }
          }
          tc_commit(smem_u32(&empty_bar[s]));
          if (tr) p.trace[1024 + kb * 4 + 3] = clock64();
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit(smem_u32(&tfull_bar[acc]));
        if (tracing) p.trace[(tile / gridDim.x) * 16 + 2] = clock64();
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1u;
      }
      if (!ok) {
        if (atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_MMA);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    // One group (warps 2-5) drains both accumulators in turn; with two groups (shallow
    // contractions, where the epilogue sets the pace) group g = warps 2-5 / 7-10 drains
    // accumulator g only, i.e. every other tile, with its own staging tiles, barrier ids,
    // per-tile constants and residual barrier.
    const int group = warp >= 7 ? 1 : 0;
    const int groups = p.epi_groups;
    const int first_thread = group ? 224 : 64;
    const bool leader = static_cast<int>(threadIdx.x) == first_thread;
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+31] belong to this warp
    float* tile_bias = tile_bias_all[group];
    float* tile_scale = tile_scale_all[group];
    const int bar_base = 1 + 3 * group;
    int acc = groups == 2 ? group : 0;
    uint32_t acc_ph = 0;
    uint32_t res_ph = 0;
    int out_slot = 0;
    int side_slot = 0;
    bool ok = true;
    // a register copy: the helper below takes the struct by reference, and a reference to the
    // kernel parameter itself turns every field access into a generic load
    const TcGemmParams lp = p;
    const int e_act = p.act;
    const float e_act_a = p.act_a, e_act_b = p.act_b;
    const int e_res_mode = p.res_mode;
    const int e_out_mode = p.out_mode, e_N = p.N, e_block_n = p.block_n, e_out_bufs = p.out_bufs;
    const bool tracing = p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 64;
    const int tile_step = static_cast<int>(gridDim.x) * groups;
    for (int tile = blockIdx.x + (groups == 2 ? group * static_cast<int>(gridDim.x) : 0); tile < total_tiles && ok;
         tile += tile_step) {
      const int m_blk = tile / p.tiles_n;
      const int n_blk = tile - m_blk * p.tiles_n;
      const bool pair_tile = m_blk < p.pair_rows;
      const long long m_tile = pair_tile ? static_cast<long long>(m_blk) * (2 * kTcBlockM)
                                         : static_cast<long long>(p.pair_rows) * (2 * kTcBlockM) +
                                               static_cast<long long>(m_blk - p.pair_rows) * kTcBlockM;
      const int n0 = n_blk * p.block_n;
      if (tracing) p.trace[(tile / gridDim.x) * 16 + 3] = clock64();
      // the vote keeps the warp together: tcgen05.ld below needs all 32 lanes
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&tfull_bar[acc]), acc_ph, abort_ptr, wait_limit) ? 1 : 0) != 0;
      if (!ok) break;
      tc_fence_after_sync();
      if (tracing) p.trace[(tile / gridDim.x) * 16 + 4] = clock64();
      const uint32_t t_row0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                              static_cast<uint32_t>(acc) * (p.pair ? 256u : 128u);
      {
        // per-column constants of this tile, fetched once (every warp of the group has left the
        // previous tile's last chunk: it ends with a barrier)
        const int t = static_cast<int>(threadIdx.x) - first_thread;
        const int n = n0 + t;
        tile_bias[t] = (p.bias != nullptr && n < p.N) ? __ldg(p.bias + n) : 0.0f;
        tile_scale[t] = (KIND == GEMM_I8 && n < p.N) ? __ldg(p.scale + n) : 0.0f;
      }
      // a paired tile is drained half by half; a second half past the last row is skipped
      for (int half = 0; half < (pair_tile ? 2 : 1) && ok; ++half) {
      const long long m_half = m_tile + static_cast<long long>(half) * kTcBlockM;
      if (half == 1 && m_half >= lp.M) break;
      const long long m = m_half + quarter * 32 + lane;
      const uint32_t t_row = t_row0 + static_cast<uint32_t>(half) * 128u;
      if (p.tma_store) {
        // staging area behind the ring, one per group: residual tiles (16 KB), then the output tiles
        TcStageCfg cfg{};
        cfg.res_stage = smem_base + static_cast<uint32_t>(S * SUB) * stage_bytes + static_cast<uint32_t>(group) * p.staging_bytes;
        cfg.out_stage = cfg.res_stage + (e_res_mode != RES_NONE ? 16384u : 0u);
        cfg.res_bar = smem_u32(&res_bar[group]);
        cfg.out_bufs = e_out_bufs;
        cfg.out_mode = e_out_mode;
        cfg.res_mode = e_res_mode;
        cfg.act = e_act;
        cfg.act_a = e_act_a;
        cfg.act_b = e_act_b;
        cfg.N = e_N;
        cfg.block_n = e_block_n;
        cfg.wide = p.wide;
        cfg.bar_base = bar_base;
        if (SIDE) {
          cfg.side_count = p.side_count;
          cfg.side_ld = p.side_ld;
          cfg.side_rows = static_cast<int>(lp.M - m_half < kTcBlockM ? lp.M - m_half : kTcBlockM);
          cfg.side_q0 = p.side_q0 != nullptr ? p.side_q0 + m_half * p.side_ld + n0 : nullptr;
          cfg.side_q1 = p.side_q1 != nullptr ? p.side_q1 + m_half * p.side_ld + n0 : nullptr;
          cfg.side_scale0 = p.side_scale0;
          cfg.side_scale1 = p.side_scale1;
        }
        const int m_first = static_cast<int>(m_half);
        // staging tiles of the int8 copies sit behind this group's output tiles
        cfg.side_stage = SIDE && p.side_staged ? cfg.out_stage + static_cast<uint32_t>(e_out_bufs) *
                                                             ((p.wide || e_out_mode == OUT_F32_SPLIT) ? 16384u : 8192u)
                                       : 0u;
        struct {
          const CUtensorMap *o0, *o1, *r0, *r1, *s0, *s1;
          int m_first;
          __device__ __forceinline__ void load_res(int plane, uint32_t dst, uint32_t bar, int col) const {
            ptx::tma_load_2d(dst, plane ? r1 : r0, bar, col, m_first);
          }
          __device__ __forceinline__ void store_out(int plane, uint32_t src, int col) const {
            ptx::tma_store_2d(plane ? o1 : o0, src, col, m_first);
          }
          __device__ __forceinline__ void store_side(int copy, uint32_t src, int col) const {
            ptx::tma_store_2d(copy ? s1 : s0, src, col, m_first);
          }
        } io{&map_o0, &map_o1, &map_r0, &map_r1, &map_s0, &map_s1, m_first};
        if (e_out_mode == OUT_I8) {
          tc_staged_epilogue_i8<KIND>(cfg, p.out_scale, io, t_row, n0, quarter * 32 + lane, leader, tile_bias,
                                      tile_scale, out_slot);
        } else {
          if (SIDE && p.side_count > 0)
            ok = tc_staged_epilogue<KIND, decltype(io), true>(cfg, io, t_row, n0, quarter * 32 + lane, leader, tile_bias,
                                                              tile_scale, res_ph, out_slot, abort_ptr, &side_slot);
          else
            ok = tc_staged_epilogue<KIND>(cfg, io, t_row, n0, quarter * 32 + lane, leader, tile_bias, tile_scale,
                                          res_ph, out_slot, abort_ptr);
          if (!ok) break;
        }
      } else {
        named_barrier_sync(bar_base + 2, 128);
        const bool bf16_io = e_out_mode == OUT_BF16X2 || e_res_mode == RES_BF16X2;
        for (int c0 = 0; c0 < e_block_n; c0 += 16) {
          uint32_t v[16];
          tmem_ld16(t_row + static_cast<uint32_t>(c0), v);
          tmem_ld_wait();
          if (m < lp.M && n0 + c0 < e_N) {
            if (SIDE && lp.side_count > 0) tc_epilogue_chunk<KIND, true, true>(lp, v, m, n0 + c0, tile_bias + c0, tile_scale + c0);
            else if (bf16_io) tc_epilogue_chunk<KIND, true>(lp, v, m, n0 + c0, tile_bias + c0, tile_scale + c0);
            else tc_epilogue_chunk<KIND, false>(lp, v, m, n0 + c0, tile_bias + c0, tile_scale + c0);
          }
        }
        named_barrier_sync(bar_base + 2, 128);  // nobody reads the tile constants any more
      }
      }
      if (!ok) break;
      tc_fence_before_sync();
      __syncwarp();
      if (tracing) p.trace[(tile / gridDim.x) * 16 + 5] = clock64();
      if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
      if (groups == 2) {
        acc_ph ^= 1u;  // this group's accumulator is used by every tile it sees
      } else {
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1u;
      }
    }
    if (!ok && lane == 0) {
      if (atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_EPILOGUE);
    }
    if (p.tma_store && leader) tma_store_wait_all();  // stores still read shared memory
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kTcTmemCols);
}

}  // namespace nb
