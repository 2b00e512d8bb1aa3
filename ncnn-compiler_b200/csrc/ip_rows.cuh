// InnerProduct / Gemm for a handful of rows (M <= 8): one pass over the weights at HBM speed.
//
// With so few rows the contraction is a matrix-vector product: every weight is used M times and the launch is
// bound by reading the weights once.  The tensor-core kernels spend such a call in tile prologues and tails
// (a 128-row tile holds one to eight live rows); here the M input rows sit in shared memory as fp32 (or int8),
// every warp owns COLS output columns at a time and streams their weight rows with 8- or 16-byte loads, all
// lanes side by side along K, and the partial sums meet in a shuffle reduction.  Operands are the ones the
// tensor-core path uses (bf16 hi/mid planes [N][ldw] packed at load time, or int8), so nothing is stored twice:
// fp32 mode: y = sum_k (a_hi + a_mid)[k] * (w_hi + w_mid)[k] in fp32 (no product of the pairs is dropped);
// int8: exact int32 accumulation, then the reference's order float(acc) * scale, + bias, requantise or activate.
#pragma once

#include "tc_gemm.cuh"

namespace nb {

constexpr int kIpRowsMaxM = 8;
constexpr int kIpRowsThreads = 512;
constexpr int kIpRowsCols = 2;  // output columns per warp and pass: shared-memory reads stay below the weight stream

struct IpRowsParams {
  int M, K, N;
  long long lda;          // elements between input rows
  long long ldw;          // elements between weight rows (K padded to the tensor-core K block)
  const void* a0;         // bf16 hi plane, or int8
  const void* a1;         // bf16 mid plane
  const void* w0;
  const void* w1;
  const float* bias;      // [N] or null
  const float* scale;     // int8: dequantisation factor per output column
  float out_scale;        // int8 output: requantisation scale
  int act;
  float act_a, act_b;
  int out_mode;           // OUT_F32, OUT_BF16X2 or (int8) OUT_I8
  float* out0;
  float* out1;
  int8_t* outq;
  long long ldo;
};

inline size_t ip_rows_smem_bytes(int M, int K, bool int8) {
  return static_cast<size_t>(M) * K * (int8 ? 1 : 4);
}

// True when the launch fits: few rows, rows of whole vectors, all rows in shared memory at once, and weights
// large enough (8 MB as stored) for the call to be a pass over them.  Smaller layers stay on the tensor-core path
// at every M, so that their results do not change with the batch size; for the large ones the last bits of a row
// differ between M <= 8 and M > 8 (another order of summation), never between calls of the same M.
inline bool ip_rows_applies(long long M, int K, int N, bool int8, int out_mode, bool has_res, bool has_side) {
  if (M < 1 || M > kIpRowsMaxM || N < 1 || has_res || has_side) return false;
  if (static_cast<long long>(K) * N * (int8 ? 1 : 4) < (8ll << 20)) return false;
  if (K % (int8 ? 16 : 8) != 0) return false;
  if (out_mode != OUT_F32 && out_mode != OUT_BF16X2 && !(int8 && out_mode == OUT_I8)) return false;
  return ip_rows_smem_bytes(static_cast<int>(M), K, int8) <= 160 * 1024;
}

__device__ __forceinline__ void ip_rows_store(const IpRowsParams& p, int m, int n, float y) {
  const long long at = static_cast<long long>(m) * p.ldo + n;
  if (p.out_mode == OUT_BF16X2) {
    uint32_t hi, mid;
    split_bf16x2(y, 0.0f, hi, mid);
    reinterpret_cast<uint16_t*>(p.out0)[at] = static_cast<uint16_t>(hi & 0xffffu);
    reinterpret_cast<uint16_t*>(p.out1)[at] = static_cast<uint16_t>(mid & 0xffffu);
  } else {
    p.out0[at] = y;
  }
}

template <bool INT8>
static __global__ void __launch_bounds__(kIpRowsThreads, 1) k_ip_rows(const IpRowsParams p) {
  extern __shared__ __align__(16) uint8_t ip_rows_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int COLS = kIpRowsCols;
  if (INT8) {
    // rows as they are: [M][K] int8
    const int vecs = p.K / 16;
    for (int i = threadIdx.x; i < p.M * vecs; i += kIpRowsThreads) {
      const int m = i / vecs, v = i - m * vecs;
      reinterpret_cast<uint4*>(ip_rows_smem)[i] =
          __ldg(reinterpret_cast<const uint4*>(static_cast<const int8_t*>(p.a0) + m * p.lda) + v);
    }
  } else {
    // rows as fp32: hi + mid of the bf16 pair, eight values per step
    float* xs = reinterpret_cast<float*>(ip_rows_smem);
    const int vecs = p.K / 8;
    for (int i = threadIdx.x; i < p.M * vecs; i += kIpRowsThreads) {
      const int m = i / vecs, v = i - m * vecs;
      const uint4 h = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.a0) + m * p.lda) + v);
      const uint4 d = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.a1) + m * p.lda) + v);
      float4* dst = reinterpret_cast<float4*>(xs + static_cast<size_t>(m) * p.K + 8 * v);
      dst[0] = make_float4(__fadd_rn(bf16_low(h.x), bf16_low(d.x)), __fadd_rn(bf16_high(h.x), bf16_high(d.x)),
                           __fadd_rn(bf16_low(h.y), bf16_low(d.y)), __fadd_rn(bf16_high(h.y), bf16_high(d.y)));
      dst[1] = make_float4(__fadd_rn(bf16_low(h.z), bf16_low(d.z)), __fadd_rn(bf16_high(h.z), bf16_high(d.z)),
                           __fadd_rn(bf16_low(h.w), bf16_low(d.w)), __fadd_rn(bf16_high(h.w), bf16_high(d.w)));
    }
  }
  __syncthreads();
  const int tasks = (p.N + COLS - 1) / COLS;
  // (column pairs are dealt out CTA by CTA, so that every SM streams weights even when there are fewer pairs than warps)
  for (int task = warp * gridDim.x + blockIdx.x; task < tasks; task += gridDim.x * (kIpRowsThreads / 32)) {
    const int n0 = task * COLS;
    float acc[kIpRowsMaxM][COLS];
    int iacc[kIpRowsMaxM][COLS];
#pragma unroll
    for (int m = 0; m < kIpRowsMaxM; ++m)
#pragma unroll
      for (int c = 0; c < COLS; ++c) {
        acc[m][c] = 0.0f;
        iacc[m][c] = 0;
      }
    // The weight stream is software-pipelined: while the lanes work on two steps that have arrived, the next two
    // are in flight (with 16 warps that is 64 KB per SM, more than the HBM latency x bandwidth product asks for).
    if (INT8) {
      const int8_t* w = static_cast<const int8_t*>(p.w0);
      constexpr int STEP = 32 * 16;  // K elements a warp covers per step
      int4 cur[2][COLS], nxt[2][COLS];
      auto fetch = [&](int4 (&dst)[2][COLS], int k0) {
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
          for (int c = 0; c < COLS; ++c) {
            const int k = k0 + u * STEP + lane * 16;
            dst[u][c] = (k < p.K && n0 + c < p.N) ? __ldg(reinterpret_cast<const int4*>(w + static_cast<long long>(n0 + c) * p.ldw + k))
                                                   : make_int4(0, 0, 0, 0);
          }
      };
      fetch(cur, 0);
      for (int k0 = 0; k0 < p.K; k0 += 2 * STEP) {
        fetch(nxt, k0 + 2 * STEP);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int k = k0 + u * STEP + lane * 16;
          if (k < p.K) {
#pragma unroll
            for (int m = 0; m < kIpRowsMaxM; ++m) {
              if (m < p.M) {
                const int4 x = *reinterpret_cast<const int4*>(ip_rows_smem + static_cast<size_t>(m) * p.K + k);
#pragma unroll
                for (int c = 0; c < COLS; ++c) {
                  int s = iacc[m][c];
                  s = __dp4a(x.x, cur[u][c].x, s);
                  s = __dp4a(x.y, cur[u][c].y, s);
                  s = __dp4a(x.z, cur[u][c].z, s);
                  s = __dp4a(x.w, cur[u][c].w, s);
                  iacc[m][c] = s;
                }
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
          for (int c = 0; c < COLS; ++c) cur[u][c] = nxt[u][c];
      }
    } else {
      const uint16_t* w0 = static_cast<const uint16_t*>(p.w0);
      const uint16_t* w1 = static_cast<const uint16_t*>(p.w1);
      const float* xs = reinterpret_cast<const float*>(ip_rows_smem);
      // A step covers 256 K elements as two halves of 128: a lane takes four consecutive values of each half, so
      // that the 16-byte reads of the input rows from shared memory are side by side across the warp (eight
      // consecutive values per lane would put lanes four apart on the same banks).
      constexpr int STEP = 32 * 8;
      uint2 cur[2][COLS][2][2], nxt[2][COLS][2][2];  // [step][column][half][plane]
      auto fetch = [&](uint2 (&dst)[2][COLS][2][2], int k0) {
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
          for (int c = 0; c < COLS; ++c)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              const int k = k0 + u * STEP + hf * 128 + lane * 4;
              if (k < p.K && n0 + c < p.N) {
                dst[u][c][hf][0] = __ldg(reinterpret_cast<const uint2*>(w0 + static_cast<long long>(n0 + c) * p.ldw + k));
                dst[u][c][hf][1] = __ldg(reinterpret_cast<const uint2*>(w1 + static_cast<long long>(n0 + c) * p.ldw + k));
              } else {
                dst[u][c][hf][0] = dst[u][c][hf][1] = make_uint2(0u, 0u);
              }
            }
      };
      fetch(cur, 0);
      for (int k0 = 0; k0 < p.K; k0 += 2 * STEP) {
        fetch(nxt, k0 + 2 * STEP);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const int k = k0 + u * STEP + hf * 128 + lane * 4;
            if (k < p.K) {
              float wv[COLS][4];
#pragma unroll
              for (int c = 0; c < COLS; ++c) {
                const uint2 h = cur[u][c][hf][0], d = cur[u][c][hf][1];
                wv[c][0] = __fadd_rn(bf16_low(h.x), bf16_low(d.x));
                wv[c][1] = __fadd_rn(bf16_high(h.x), bf16_high(d.x));
                wv[c][2] = __fadd_rn(bf16_low(h.y), bf16_low(d.y));
                wv[c][3] = __fadd_rn(bf16_high(h.y), bf16_high(d.y));
              }
#pragma unroll
              for (int m = 0; m < kIpRowsMaxM; ++m) {
                if (m < p.M) {
                  const float4 x = *reinterpret_cast<const float4*>(xs + static_cast<size_t>(m) * p.K + k);
#pragma unroll
                  for (int c = 0; c < COLS; ++c) {
                    float s = acc[m][c];
                    s = fmaf(x.x, wv[c][0], s);
                    s = fmaf(x.y, wv[c][1], s);
                    s = fmaf(x.z, wv[c][2], s);
                    s = fmaf(x.w, wv[c][3], s);
                    acc[m][c] = s;
                  }
                }
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
          for (int c = 0; c < COLS; ++c)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              cur[u][c][hf][0] = nxt[u][c][hf][0];
              cur[u][c][hf][1] = nxt[u][c][hf][1];
            }
      }
    }
    // the lanes' partial sums meet (a fixed tree: the result does not depend on timing)
#pragma unroll
    for (int m = 0; m < kIpRowsMaxM; ++m) {
      if (m < p.M) {
#pragma unroll
        for (int c = 0; c < COLS; ++c) {
          if (INT8) {
            int s = iacc[m][c];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            iacc[m][c] = s;
          } else {
            float s = acc[m][c];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, o));
            acc[m][c] = s;
          }
        }
      }
    }
    // lane (m * COLS + c) finishes and stores result (m, c)
#pragma unroll
    for (int m = 0; m < kIpRowsMaxM; ++m) {
#pragma unroll
      for (int c = 0; c < COLS; ++c) {
        if (lane == m * COLS + c && m < p.M && n0 + c < p.N) {
          const int n = n0 + c;
          float y = INT8 ? __fmul_rn(static_cast<float>(iacc[m][c]), p.scale[n]) : acc[m][c];
          if (p.bias != nullptr) y = __fadd_rn(y, p.bias[n]);
          if (INT8 && p.out_mode == OUT_I8) {
            int q = quantize_rha(y, p.out_scale);
            if (p.act == ACT_RELU) q = max(q, 0);
            p.outq[static_cast<long long>(m) * p.ldo + n] = static_cast<int8_t>(q);
          } else {
            ip_rows_store(p, m, n, apply_act(y, p.act, p.act_a, p.act_b));
          }
        }
      }
    }
  }
}

}  // namespace nb
