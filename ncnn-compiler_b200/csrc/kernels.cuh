// Memory-bound and CUDA-core kernels of the runtime.  Activations live in HBM as
// channel-last arrays ([image][h][w][c], c contiguous) in one of these formats:
//   FMT_F32    one fp32 plane
//   FMT_SPLIT  two fp32 planes hi/lo with x == hi + lo exactly (hi is x rounded to
//              tf32); feeds the 3xTF32 tensor-core path
//   FMT_I8     one int8 plane
//   FMT_TF32   one fp32 plane whose values are rounded to tf32 when stored
//   FMT_BF16X2 two bf16 planes hi/mid with x ~ hi + mid (16 significant bits); feeds the
//              bf16x3 tensor-core path.  The planes are addressed through p0/p1.
// All kernels index with 64-bit offsets, use 128-bit accesses when the channel
// count allows, and keep the reference's order of operations where it affects
// the result (no FMA in int8 epilogues, sequential window sums).
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#include "tc_gemm.cuh"

namespace nb {

enum : int { FMT_F32 = 0, FMT_SPLIT = 1, FMT_I8 = 2, FMT_TF32 = 3, FMT_BF16X2 = 4 };

struct ActRef {
  float* p0 = nullptr;
  float* p1 = nullptr;
  int8_t* q = nullptr;
  int fmt = FMT_F32;
};

__device__ __forceinline__ float act_load(const ActRef& a, long long i) {
  if (a.fmt == FMT_I8) return static_cast<float>(a.q[i]);
  if (a.fmt == FMT_BF16X2) {
    const uint32_t h = reinterpret_cast<const uint16_t*>(a.p0)[i], m = reinterpret_cast<const uint16_t*>(a.p1)[i];
    return __fadd_rn(__uint_as_float(h << 16), __uint_as_float(m << 16));
  }
  float v = a.p0[i];
  if (a.fmt == FMT_SPLIT) v = __fadd_rn(v, a.p1[i]);
  return v;
}

__device__ __forceinline__ void act_store(const ActRef& a, long long i, float v) {
  if (a.fmt == FMT_I8) {
    a.q[i] = static_cast<int8_t>(static_cast<int>(v));
  } else if (a.fmt == FMT_F32) {
    a.p0[i] = v;
  } else if (a.fmt == FMT_BF16X2) {
    uint32_t hi, mid;
    split_bf16x2(v, 0.0f, hi, mid);
    reinterpret_cast<uint16_t*>(a.p0)[i] = static_cast<uint16_t>(hi & 0xffffu);
    reinterpret_cast<uint16_t*>(a.p1)[i] = static_cast<uint16_t>(mid & 0xffffu);
  } else {
    const float hi = round_tf32(v);
    a.p0[i] = hi;
    if (a.fmt == FMT_SPLIT) a.p1[i] = __fadd_rn(v, -hi);
  }
}

__device__ __forceinline__ float4 act_load4(const ActRef& a, long long i) {
  if (a.fmt == FMT_I8) {
    const char4 c = *reinterpret_cast<const char4*>(a.q + i);
    return make_float4(c.x, c.y, c.z, c.w);
  }
  if (a.fmt == FMT_BF16X2) {
    const uint2 h = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(a.p0) + i);
    const uint2 m = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(a.p1) + i);
    return make_float4(__fadd_rn(bf16_low(h.x), bf16_low(m.x)), __fadd_rn(bf16_high(h.x), bf16_high(m.x)),
                       __fadd_rn(bf16_low(h.y), bf16_low(m.y)), __fadd_rn(bf16_high(h.y), bf16_high(m.y)));
  }
  float4 v = *reinterpret_cast<const float4*>(a.p0 + i);
  if (a.fmt == FMT_SPLIT) {
    const float4 l = *reinterpret_cast<const float4*>(a.p1 + i);
    v.x = __fadd_rn(v.x, l.x);
    v.y = __fadd_rn(v.y, l.y);
    v.z = __fadd_rn(v.z, l.z);
    v.w = __fadd_rn(v.w, l.w);
  }
  return v;
}

__device__ __forceinline__ void act_store4(const ActRef& a, long long i, float4 v) {
  if (a.fmt == FMT_I8) {
    *reinterpret_cast<char4*>(a.q + i) =
        make_char4(static_cast<signed char>(static_cast<int>(v.x)),
                   static_cast<signed char>(static_cast<int>(v.y)),
                   static_cast<signed char>(static_cast<int>(v.z)),
                   static_cast<signed char>(static_cast<int>(v.w)));
  } else if (a.fmt == FMT_F32) {
    *reinterpret_cast<float4*>(a.p0 + i) = v;
  } else if (a.fmt == FMT_BF16X2) {
    uint2 h, m;
    split_bf16x2(v.x, v.y, h.x, m.x);
    split_bf16x2(v.z, v.w, h.y, m.y);
    *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(a.p0) + i) = h;
    *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(a.p1) + i) = m;
  } else {
    const float4 hi = make_float4(round_tf32(v.x), round_tf32(v.y), round_tf32(v.z), round_tf32(v.w));
    *reinterpret_cast<float4*>(a.p0 + i) = hi;
    if (a.fmt == FMT_SPLIT)
      *reinterpret_cast<float4*>(a.p1 + i) =
          make_float4(__fadd_rn(v.x, -hi.x), __fadd_rn(v.y, -hi.y), __fadd_rn(v.z, -hi.z),
                      __fadd_rn(v.w, -hi.w));
  }
}

// ----------------------------------------------------------------- layout edges
// Caller's [image][C][H*W] fp32  ->  channel-last [image][H][Wp][Cp] (pixel (h,w) is
// stored at row offset w + w_off; padding columns/channels stay zero).  With
// quant_scale > 0 the values are quantised to int8 on the way.
struct EdgeParams {
  long long images;
  int C, H, W, Cp, Wp, w_off;
  float quant_scale;
};

static __global__ void k_chw_to_nhwc_tiled(const float* __restrict__ src, ActRef dst, EdgeParams p) {
  __shared__ float tile[32][33];
  const long long img = blockIdx.z;
  const int hw = p.H * p.W;
  const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const float* s = src + img * static_cast<long long>(p.C) * hw;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int c = c0 + r, px = p0 + threadIdx.x;
    tile[r][threadIdx.x] = (c < p.C && px < hw) ? s[static_cast<long long>(c) * hw + px] : 0.0f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int px = p0 + r, c = c0 + threadIdx.x;
    if (px < hw && c < p.C) {
      const int h = px / p.W, w = px - h * p.W;
      const long long o =
          ((img * p.H + h) * static_cast<long long>(p.Wp) + w + p.w_off) * p.Cp + c;
      float v = tile[threadIdx.x][r];
      if (p.quant_scale > 0.0f) v = static_cast<float>(quantize_rha(v, p.quant_scale));
      act_store(dst, o, v);
    }
  }
}

// Few channels (C <= 4): one thread per pixel, one 16-byte store per plane.
static __global__ void k_chw_to_nhwc_small(const float* __restrict__ src, ActRef dst, EdgeParams p) {
  const long long hw = static_cast<long long>(p.H) * p.W;
  const long long total = p.images * hw;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long img = i / hw;
    const long long px = i - img * hw;
    const int h = static_cast<int>(px / p.W), w = static_cast<int>(px - static_cast<long long>(h) * p.W);
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = 0; c < p.C; ++c) v[c] = src[(img * p.C + c) * hw + px];
    const long long o = ((img * p.H + h) * static_cast<long long>(p.Wp) + w + p.w_off) * p.Cp;
    if (dst.fmt == FMT_I8) {
      // Cp == 16 or 8: channels 0..3 carry data, the rest of the 16- or 8-byte pixel is zero
      uint32_t w0 = 0;
      for (int c = 0; c < p.C; ++c)
        w0 |= (static_cast<uint32_t>(quantize_rha(v[c], p.quant_scale)) & 0xffu) << (8 * c);
      if (p.Cp == 8) *reinterpret_cast<uint2*>(dst.q + o) = make_uint2(w0, 0u);
      else *reinterpret_cast<uint4*>(dst.q + o) = make_uint4(w0, 0u, 0u, 0u);
    } else {
      act_store4(dst, o, make_float4(v[0], v[1], v[2], v[3]));
    }
  }
}

// Channel-last [image][HW][Cp] -> caller's [image][C][HW] fp32.
static __global__ void k_nhwc_to_chw_tiled(ActRef src, float* __restrict__ dst, long long images, int C,
                                    int HW, int Cp) {
  __shared__ float tile[32][33];
  const long long img = blockIdx.z;
  const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int px = p0 + r, c = c0 + threadIdx.x;
    tile[r][threadIdx.x] =
        (px < HW && c < C) ? act_load(src, (img * HW + px) * static_cast<long long>(Cp) + c) : 0.0f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int c = c0 + r, px = p0 + threadIdx.x;
    if (c < C && px < HW) dst[(img * C + c) * static_cast<long long>(HW) + px] = tile[threadIdx.x][r];
  }
}

// The same for rows whose width is a multiple of 4 and fp32 / bf16-pair storage with Cp == 4 (or int8 with Cp == 8):
// one thread per 4 consecutive pixels of a row, one 128-bit load per channel plane and 64 or
// 32 contiguous bytes stored per output plane; grid = (row quads, images), 32-bit indices.
static __global__ void k_chw_to_nhwc_small_x4(const float* __restrict__ src, ActRef dst, EdgeParams p) {
  const int hw = p.H * p.W;
  const int quads = hw / 4;
  const long long img = blockIdx.y;
  const float* s = src + img * static_cast<long long>(p.C) * hw;
  for (int q = blockIdx.x * blockDim.x + threadIdx.x; q < quads; q += gridDim.x * blockDim.x) {
    const int px = q * 4;
    const int h = px / p.W, w = px - h * p.W;
    float4 ch[3];
#pragma unroll
    for (int c = 0; c < 3; ++c)
      ch[c] = c < p.C ? __ldg(reinterpret_cast<const float4*>(s + static_cast<long long>(c) * hw + px))
                      : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 c3 = p.C > 3 ? __ldg(reinterpret_cast<const float4*>(s + 3ll * hw + px)) : make_float4(0.f, 0.f, 0.f, 0.f);
    const long long o = ((img * p.H + h) * static_cast<long long>(p.Wp) + w + p.w_off) * p.Cp;
    const float v[4][4] = {{ch[0].x, ch[1].x, ch[2].x, c3.x}, {ch[0].y, ch[1].y, ch[2].y, c3.y},
                           {ch[0].z, ch[1].z, ch[2].z, c3.z}, {ch[0].w, ch[1].w, ch[2].w, c3.w}};
    if (dst.fmt == FMT_I8) {
      // Cp == 8: four quantised channels and four zero bytes per pixel, 32 contiguous bytes per thread
      uint32_t q[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        q[k] = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          q[k] |= (static_cast<uint32_t>(quantize_rha(v[k][c], p.quant_scale)) & 0xffu) << (8 * c);
      }
      uint2* d = reinterpret_cast<uint2*>(dst.q + o);  // (rows start pad_l pixels in: 8-byte alignment only)
#pragma unroll
      for (int k = 0; k < 4; ++k) d[k] = make_uint2(q[k], 0u);
      continue;
    }
    if (dst.fmt == FMT_BF16X2) {
      // four pixels = 32 contiguous bytes per plane, 8-byte aligned (rows start pad_l pixels in): 16-byte stores
      // where the alignment allows, an 8-byte store either side of one 16-byte store where it does not
      uint2 h[4], m[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        split_bf16x2(v[k][0], v[k][1], h[k].x, m[k].x);
        split_bf16x2(v[k][2], v[k][3], h[k].y, m[k].y);
      }
      uint16_t* d0 = reinterpret_cast<uint16_t*>(dst.p0) + o;
      uint16_t* d1 = reinterpret_cast<uint16_t*>(dst.p1) + o;
      if ((o & 7) == 0) {
        reinterpret_cast<uint4*>(d0)[0] = make_uint4(h[0].x, h[0].y, h[1].x, h[1].y);
        reinterpret_cast<uint4*>(d0)[1] = make_uint4(h[2].x, h[2].y, h[3].x, h[3].y);
        reinterpret_cast<uint4*>(d1)[0] = make_uint4(m[0].x, m[0].y, m[1].x, m[1].y);
        reinterpret_cast<uint4*>(d1)[1] = make_uint4(m[2].x, m[2].y, m[3].x, m[3].y);
      } else {
        *reinterpret_cast<uint2*>(d0) = h[0];
        *reinterpret_cast<uint4*>(d0 + 4) = make_uint4(h[1].x, h[1].y, h[2].x, h[2].y);
        *reinterpret_cast<uint2*>(d0 + 12) = h[3];
        *reinterpret_cast<uint2*>(d1) = m[0];
        *reinterpret_cast<uint4*>(d1 + 4) = make_uint4(m[1].x, m[1].y, m[2].x, m[2].y);
        *reinterpret_cast<uint2*>(d1 + 12) = m[3];
      }
      continue;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) act_store4(dst, o + 4 * k, make_float4(v[k][0], v[k][1], v[k][2], v[k][3]));
  }
}

// ----------------------------------------------------------------- element-wise
enum : int { UN_COPY = 0, UN_ACT = 1, UN_AFFINE = 2, UN_QUANT = 3 };
struct UnaryParams {
  int op;
  int act;
  float act_a, act_b;
  const float* scale;   // UN_AFFINE: per-channel scale; UN_QUANT: scale(s)
  const float* offset;  // UN_AFFINE: per-channel offset
  int nscale;           // UN_QUANT: 1 or channels
  int channels = 1;     // channel index of element i = (i / inner) % channels
  int inner = 1;        // 1 for channel-last storage, row length for rank-2 tensors
};

__device__ __forceinline__ float unary_apply(const UnaryParams& u, float v, long long i) {
  if (u.op == UN_ACT) return apply_act(v, u.act, u.act_a, u.act_b);
  if (u.op == UN_AFFINE) {
    const int c = static_cast<int>((i / u.inner) % u.channels);
    return __fadd_rn(__fmul_rn(v, u.scale[c]), u.offset[c]);
  }
  if (u.op == UN_QUANT) {
    const float s = u.nscale == 1 ? u.scale[0] : u.scale[(i / u.inner) % u.channels];
    return static_cast<float>(quantize_rha(v, s));
  }
  return v;
}

template <int VEC>
static __global__ void k_unary(ActRef in, ActRef out, long long count, UnaryParams u) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * VEC;
  for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * VEC;
       i < count; i += stride) {
    if (VEC == 4) {
      float4 v = act_load4(in, i);
      v.x = unary_apply(u, v.x, i);
      v.y = unary_apply(u, v.y, i + 1);
      v.z = unary_apply(u, v.z, i + 2);
      v.w = unary_apply(u, v.w, i + 3);
      act_store4(out, i, v);
    } else {
      act_store(out, i, unary_apply(u, act_load(in, i), i));
    }
  }
}

// Per-tensor Quantize of a plain fp32 plane, 16 elements per thread: four 128-bit loads, one
// 128-bit store of packed int8 (the Quantize steps in front of int8 contractions); optionally a second
// int8 result of the same values with another scale.
__device__ __forceinline__ uint32_t quantize_pack4(const float4& v, float scale) {
  return (static_cast<uint32_t>(quantize_rha(v.x, scale)) & 0xffu) | ((static_cast<uint32_t>(quantize_rha(v.y, scale)) & 0xffu) << 8) |
         ((static_cast<uint32_t>(quantize_rha(v.z, scale)) & 0xffu) << 16) | ((static_cast<uint32_t>(quantize_rha(v.w, scale)) & 0xffu) << 24);
}
static __global__ void k_quantize16(const float* __restrict__ x, int8_t* __restrict__ y, long long count16, float scale,
                                    int8_t* __restrict__ y2, float scale2) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < count16;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4* src = reinterpret_cast<const float4*>(x) + i * 4;
    float4 v[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) v[g] = __ldg(src + g);
    reinterpret_cast<uint4*>(y)[i] = make_uint4(quantize_pack4(v[0], scale), quantize_pack4(v[1], scale), quantize_pack4(v[2], scale),
                                                quantize_pack4(v[3], scale));
    if (y2 != nullptr)
      reinterpret_cast<uint4*>(y2)[i] = make_uint4(quantize_pack4(v[0], scale2), quantize_pack4(v[1], scale2),
                                                   quantize_pack4(v[2], scale2), quantize_pack4(v[3], scale2));
  }
}

// out = act(op(a * ca?, b * cb?)): Eltwise SUM with coefficients (a coefficient of
// exactly 1 is skipped, as the reference does) and BinaryOp add/sub/mul/max.
enum : int { BIN_ADD = 0, BIN_SUB = 1, BIN_MUL = 2, BIN_MAX = 4 };
struct BinaryParams {
  int op;
  int use_scalar;
  float scalar;
  int scale_a, scale_b;
  float ca, cb;
  int act;
  float act_a, act_b;
};

__device__ __forceinline__ float binary_apply(const BinaryParams& b, float x, float y) {
  if (b.scale_a) x = __fmul_rn(x, b.ca);
  if (b.scale_b) y = __fmul_rn(y, b.cb);
  float r;
  switch (b.op) {
    case BIN_ADD: r = __fadd_rn(x, y); break;
    case BIN_SUB: r = __fadd_rn(x, -y); break;
    case BIN_MUL: r = __fmul_rn(x, y); break;
    default: r = fmaxf(x, y); break;
  }
  return apply_act(r, b.act, b.act_a, b.act_b);
}

template <int VEC>
static __global__ void k_binary(ActRef a, ActRef b, ActRef out, long long count, BinaryParams p) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * VEC;
  for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * VEC;
       i < count; i += stride) {
    if (VEC == 4) {
      const float4 x = act_load4(a, i);
      const float4 y = p.use_scalar ? make_float4(p.scalar, p.scalar, p.scalar, p.scalar)
                                    : act_load4(b, i);
      act_store4(out, i, make_float4(binary_apply(p, x.x, y.x), binary_apply(p, x.y, y.y),
                                     binary_apply(p, x.z, y.z), binary_apply(p, x.w, y.w)));
    } else {
      const float x = act_load(a, i);
      const float y = p.use_scalar ? p.scalar : act_load(b, i);
      act_store(out, i, binary_apply(p, x, y));
    }
  }
}

// ----------------------------------------------------------------- pooling
struct PoolParams {
  long long images;
  int H, W, C, OH, OW;
  int kind;  // 0 max, 1 average over in-bounds elements
  int KH, KW, sh, sw, pt, pl;
  // adaptive windows [floor(o*in/out), ceil((o+1)*in/out)) per axis (ConvertPooling's adaptive
  // branch, NCNNToTosa.cpp:1706-1745); an axis whose output extent equals "same as input" has
  // one-element windows, which the same formula yields
  int adaptive;
  // optional int8 copy of the result for an int8 contraction that reads it next: Q(value, side_scale),
  // same layout as the fp32 result
  int8_t* side_q;
  float side_scale;
};

__device__ __forceinline__ void pool_store_side4(const PoolParams& p, long long o, float a, float b, float c, float d) {
  if (p.side_q == nullptr) return;
  *reinterpret_cast<char4*>(p.side_q + o) =
      make_char4(static_cast<signed char>(quantize_rha(a, p.side_scale)), static_cast<signed char>(quantize_rha(b, p.side_scale)),
                 static_cast<signed char>(quantize_rha(c, p.side_scale)), static_cast<signed char>(quantize_rha(d, p.side_scale)));
}

template <int VEC>
static __global__ void k_pool(ActRef in, ActRef out, PoolParams p) {
  const int cv = p.C / VEC;
  const long long total = p.images * p.OH * p.OW * cv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % cv) * VEC;
    long long r = i / cv;
    const int ow = static_cast<int>(r % p.OW);
    r /= p.OW;
    const int oh = static_cast<int>(r % p.OH);
    const long long img = r / p.OH;
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = p.kind == 0 ? -INFINITY : 0.0f;
    int hb, he, wb, we;
    if (p.adaptive) {
      hb = static_cast<int>(static_cast<long long>(oh) * p.H / p.OH);
      he = static_cast<int>((static_cast<long long>(oh + 1) * p.H + p.OH - 1) / p.OH);
      wb = static_cast<int>(static_cast<long long>(ow) * p.W / p.OW);
      we = static_cast<int>((static_cast<long long>(ow + 1) * p.W + p.OW - 1) / p.OW);
    } else {
      hb = max(oh * p.sh - p.pt, 0);
      he = min(oh * p.sh - p.pt + p.KH, p.H);
      wb = max(ow * p.sw - p.pl, 0);
      we = min(ow * p.sw - p.pl + p.KW, p.W);
    }
    int count = 0;
    for (int ih = hb; ih < he; ++ih) {
      for (int iw = wb; iw < we; ++iw) {
        const long long idx = ((img * p.H + ih) * p.W + iw) * p.C + c;
        float v[VEC];
        if (VEC == 4) {
          const float4 t = act_load4(in, idx);
          v[0] = t.x;
          v[1 % VEC] = t.y;
          v[2 % VEC] = t.z;
          v[3 % VEC] = t.w;
        } else {
          v[0] = act_load(in, idx);
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          acc[e] = p.kind == 0 ? fmaxf(acc[e], v[e]) : __fadd_rn(acc[e], v[e]);
        ++count;
      }
    }
    if (p.kind == 1) {
      const float n = static_cast<float>(count);
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = __fdiv_rn(acc[e], n);
    }
    const long long o = ((img * p.OH + oh) * p.OW + ow) * p.C + c;
    if (VEC == 4) {
      act_store4(out, o, make_float4(acc[0], acc[1 % VEC], acc[2 % VEC], acc[3 % VEC]));
      pool_store_side4(p, o, acc[0], acc[1 % VEC], acc[2 % VEC], acc[3 % VEC]);
    } else {
      act_store(out, o, acc[0]);
      if (p.side_q != nullptr) p.side_q[o] = static_cast<int8_t>(quantize_rha(acc[0], p.side_scale));
    }
  }
}

// Global pooling (one window = the whole image) with channels in fours: one thread per four channels of an image
// walks the pixels in the reference's order, seven loads in flight at a time (the generic kernel waits for every
// pixel in turn: 49 memory latencies for a 7 x 7 image).
static __global__ void __launch_bounds__(128) k_global_pool4(ActRef in, ActRef out, PoolParams p) {
  const int c = (blockIdx.x * 128 + threadIdx.x) * 4;
  const long long img = blockIdx.y;
  if (c >= p.C) return;
  const int hw = p.H * p.W;
  const long long base = img * hw * p.C + c;
  float4 acc = p.kind == 0 ? make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY) : make_float4(0.f, 0.f, 0.f, 0.f);
  auto take = [&](const float4& v) {
    if (p.kind == 0) {
      acc = make_float4(fmaxf(acc.x, v.x), fmaxf(acc.y, v.y), fmaxf(acc.z, v.z), fmaxf(acc.w, v.w));
    } else {
      acc = make_float4(__fadd_rn(acc.x, v.x), __fadd_rn(acc.y, v.y), __fadd_rn(acc.z, v.z), __fadd_rn(acc.w, v.w));
    }
  };
  int px = 0;
  for (; px + 7 <= hw; px += 7) {
    float4 v[7];
#pragma unroll
    for (int j = 0; j < 7; ++j) v[j] = act_load4(in, base + static_cast<long long>(px + j) * p.C);
#pragma unroll
    for (int j = 0; j < 7; ++j) take(v[j]);
  }
  for (; px < hw; ++px) take(act_load4(in, base + static_cast<long long>(px) * p.C));
  if (p.kind == 1) {
    const float n = static_cast<float>(hw);
    acc = make_float4(__fdiv_rn(acc.x, n), __fdiv_rn(acc.y, n), __fdiv_rn(acc.z, n), __fdiv_rn(acc.w, n));
  }
  const long long o = img * p.C + c;
  act_store4(out, o, acc);
  pool_store_side4(p, o, acc.x, acc.y, acc.z, acc.w);
}

// ----------------------------------------------------------------- depthwise conv
struct ConvGeom {
  long long images;
  int H, W, C, OH, OW, O;
  int KH, KW, sh, sw, pt, pl, dh, dw;
};

struct ConvEpilogue {
  const float* bias;   // [O] or null
  const float* scale;  // int8: dequantisation factor per output channel
  float out_scale;     // int8 output: requantisation scale
  int act;
  float act_a, act_b;
  ActRef res;          // optional residual
  int has_res;
};

__device__ __forceinline__ float conv_finish_f32(const ConvEpilogue& e, float acc, float res) {
  if (e.has_res) acc = __fadd_rn(acc, res);
  return apply_act(acc, e.act, e.act_a, e.act_b);
}

// int8 epilogue in the reference's order: float(acc) * r, + bias, (+ residual), then
// either requantise (ReLU applied on the int8 value) or activation on fp32.
__device__ __forceinline__ float conv_finish_i8(const ConvEpilogue& e, int acc, int o, float res,
                                                bool out_i8) {
  float y = __fmul_rn(static_cast<float>(acc), e.scale[o]);
  if (e.bias != nullptr) y = __fadd_rn(y, e.bias[o]);
  if (e.has_res) y = __fadd_rn(y, res);
  if (out_i8) {
    int q = quantize_rha(y, e.out_scale);
    if (e.act == ACT_RELU) q = max(q, 0);
    return static_cast<float>(q);
  }
  return apply_act(y, e.act, e.act_a, e.act_b);
}

// Weights are stored [KH*KW][C] so that neighbouring threads (neighbouring channels)
// read neighbouring weights.  One thread computes VEC channels of one output pixel.
template <int VEC, bool INT8>
static __global__ void k_depthwise(ActRef in, ActRef out, const void* __restrict__ weights, ConvGeom g,
                            ConvEpilogue e) {
  const int cv = g.C / VEC;
  const long long total = g.images * g.OH * g.OW * cv;
  const float* wf = static_cast<const float*>(weights);
  const int8_t* wq = static_cast<const int8_t*>(weights);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % cv) * VEC;
    long long r = i / cv;
    const int ow = static_cast<int>(r % g.OW);
    r /= g.OW;
    const int oh = static_cast<int>(r % g.OH);
    const long long img = r / g.OH;
    float acc[VEC];
    int iacc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      acc[v] = (!INT8 && e.bias != nullptr) ? e.bias[c + v] : 0.0f;
      iacc[v] = 0;
    }
    for (int kh = 0; kh < g.KH; ++kh) {
      const int ih = oh * g.sh - g.pt + kh * g.dh;
      if (ih < 0 || ih >= g.H) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        const int iw = ow * g.sw - g.pl + kw * g.dw;
        if (iw < 0 || iw >= g.W) continue;
        const long long idx = ((img * g.H + ih) * g.W + iw) * g.C + c;
        const int widx = (kh * g.KW + kw) * g.C + c;
        float x[VEC];
        if (VEC == 4) {
          const float4 t = act_load4(in, idx);
          x[0] = t.x;
          x[1 % VEC] = t.y;
          x[2 % VEC] = t.z;
          x[3 % VEC] = t.w;
        } else {
          x[0] = act_load(in, idx);
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          if (INT8) {
            iacc[v] += static_cast<int>(x[v]) * static_cast<int>(wq[widx + v]);
          } else {
            acc[v] = fmaf(x[v], wf[widx + v], acc[v]);
          }
        }
      }
    }
    const long long o = ((img * g.OH + oh) * g.OW + ow) * g.C + c;
    float y[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      const float res = e.has_res ? act_load(e.res, o + v) : 0.0f;
      y[v] = INT8 ? conv_finish_i8(e, iacc[v], c + v, res, out.fmt == FMT_I8)
                  : conv_finish_f32(e, acc[v], res);
    }
    if (VEC == 4) {
      act_store4(out, o, make_float4(y[0], y[1 % VEC], y[2 % VEC], y[3 % VEC]));
    } else {
      act_store(out, o, y[0]);
    }
  }
}

// 3x3 depthwise, fp32, dilation 1.  A block stages the input patch of an 8x8 output tile
// for 32 channels in shared memory, then each thread produces two outputs from shared memory.
// The patch is read once per tile (1.6x halo overhead at stride 1) instead of once per filter
// tap.  Plain fp32 inputs (the usual case: the producer is a 1x1 convolution whose result
// feeds only this layer) are copied with cp.async, 16 bytes per request, all requests of the
// block in flight at once and no registers held (zero fill outside the image); split formats
// take the register path, which adds the planes on the way in.
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* src, int src_bytes) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}

template <int STRIDE>
static __global__ void __launch_bounds__(256) k_depthwise3x3_tile(ActRef in, ActRef out,
                                                                  const float* __restrict__ weights,
                                                                  ConvGeom g, ConvEpilogue e) {
  constexpr int TO = 8;                      // output tile edge
  constexpr int TI = (TO - 1) * STRIDE + 3;  // input patch edge
  constexpr int CG = 8;                      // float4 channel groups per block
  constexpr int LOADS = (TI * TI * CG + 255) / 256;
  __shared__ float4 patch[TI * TI * CG];
  __shared__ float4 taps[9 * CG];
  const int tiles_w = (g.OW + TO - 1) / TO;
  const int tile_y = blockIdx.x / tiles_w, tile_x = blockIdx.x - tile_y * tiles_w;
  const int cg0 = blockIdx.y * CG;
  const int cv = g.C / 4;
  const long long img = blockIdx.z;
  const int oy0 = tile_y * TO, ox0 = tile_x * TO;
  const int iy0 = oy0 * STRIDE - g.pt, ix0 = ox0 * STRIDE - g.pl;
  const bool plain = in.fmt == FMT_F32;
#pragma unroll
  for (int k = 0; k < LOADS; ++k) {
    const int idx = threadIdx.x + k * 256;
    if (idx >= TI * TI * CG) break;
    const int cg = idx % CG;
    const int px = idx / CG;
    const int py = px / TI;
    const int iy = iy0 + py, ix = ix0 + (px - py * TI);
    const bool valid = cg0 + cg < cv && iy >= 0 && iy < g.H && ix >= 0 && ix < g.W;
    const long long off = valid ? ((img * g.H + iy) * g.W + ix) * static_cast<long long>(g.C) + (cg0 + cg) * 4 : 0;
    if (plain) {
      cp_async_16(&patch[idx], in.p0 + off, valid ? 16 : 0);
    } else {
      patch[idx] = valid ? act_load4(in, off) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  if (threadIdx.x < 9 * CG) {
    const int cg = threadIdx.x % CG, tap = threadIdx.x / CG;
    taps[threadIdx.x] = cg0 + cg < cv ? __ldg(reinterpret_cast<const float4*>(weights + tap * g.C + (cg0 + cg) * 4))
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  for (int o = threadIdx.x; o < TO * TO * CG; o += 256) {
    const int cg = o % CG;
    const int p = o / CG;
    const int ty = p / TO, tx = p - ty * TO;
    const int oy = oy0 + ty, ox = ox0 + tx;
    if (cg0 + cg >= cv || oy >= g.OH || ox >= g.OW) continue;
    const int c = (cg0 + cg) * 4;
    float4 acc = e.bias != nullptr ? *reinterpret_cast<const float4*>(e.bias + c)
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int kh = 0; kh < 3; ++kh) {
#pragma unroll
      for (int kw = 0; kw < 3; ++kw) {
        const float4 x = patch[((ty * STRIDE + kh) * TI + tx * STRIDE + kw) * CG + cg];
        const float4 k = taps[(kh * 3 + kw) * CG + cg];
        acc.x = fmaf(x.x, k.x, acc.x);
        acc.y = fmaf(x.y, k.y, acc.y);
        acc.z = fmaf(x.z, k.z, acc.z);
        acc.w = fmaf(x.w, k.w, acc.w);
      }
    }
    const long long off = ((img * g.OH + oy) * g.OW + ox) * static_cast<long long>(g.C) + c;
    float4 res = make_float4(0.f, 0.f, 0.f, 0.f);
    if (e.has_res) res = act_load4(e.res, off);
    acc.x = conv_finish_f32(e, acc.x, res.x);
    acc.y = conv_finish_f32(e, acc.y, res.y);
    acc.z = conv_finish_f32(e, acc.z, res.z);
    acc.w = conv_finish_f32(e, acc.w, res.w);
    act_store4(out, off, acc);
  }
}

// 3x3 stride-2 max pooling through the same shared-memory tile as the depthwise kernel: the
// 17x17 input patch of an 8x8 output tile is staged once for 32 channels (cp.async for plain
// fp32 inputs), then every thread takes the maximum over the taps that lie inside the image
// (padding never wins, ConvertPooling, NCNNToTosa.cpp:1913-1954).
static __global__ void __launch_bounds__(256) k_maxpool3x3s2_tile(ActRef in, ActRef out, PoolParams p) {
  constexpr int TO = 8, TI = 17, CG = 8;
  constexpr int LOADS = (TI * TI * CG + 255) / 256;
  __shared__ float4 patch[TI * TI * CG];
  const int tiles_w = (p.OW + TO - 1) / TO;
  const int tile_y = blockIdx.x / tiles_w, tile_x = blockIdx.x - tile_y * tiles_w;
  const int cg0 = blockIdx.y * CG;
  const int cv = p.C / 4;
  const long long img = blockIdx.z;
  const int oy0 = tile_y * TO, ox0 = tile_x * TO;
  const int iy0 = oy0 * 2 - p.pt, ix0 = ox0 * 2 - p.pl;
  const bool plain = in.fmt == FMT_F32;
#pragma unroll
  for (int k = 0; k < LOADS; ++k) {
    const int idx = threadIdx.x + k * 256;
    if (idx >= TI * TI * CG) break;
    const int cg = idx % CG;
    const int px = idx / CG;
    const int py = px / TI;
    const int iy = iy0 + py, ix = ix0 + (px - py * TI);
    const bool valid = cg0 + cg < cv && iy >= 0 && iy < p.H && ix >= 0 && ix < p.W;
    const long long off = valid ? ((img * p.H + iy) * p.W + ix) * static_cast<long long>(p.C) + (cg0 + cg) * 4 : 0;
    if (plain) {
      cp_async_16(&patch[idx], in.p0 + off, valid ? 16 : 0);
    } else {
      patch[idx] = valid ? act_load4(in, off) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  for (int o = threadIdx.x; o < TO * TO * CG; o += 256) {
    const int cg = o % CG;
    const int q = o / CG;
    const int ty = q / TO, tx = q - ty * TO;
    const int oy = oy0 + ty, ox = ox0 + tx;
    if (cg0 + cg >= cv || oy >= p.OH || ox >= p.OW) continue;
    const float ninf = __int_as_float(0xff800000);
    float4 acc = make_float4(ninf, ninf, ninf, ninf);
#pragma unroll
    for (int kh = 0; kh < 3; ++kh) {
      const int iy = oy * 2 - p.pt + kh;
      if (iy < 0 || iy >= p.H) continue;
#pragma unroll
      for (int kw = 0; kw < 3; ++kw) {
        const int ix = ox * 2 - p.pl + kw;
        if (ix < 0 || ix >= p.W) continue;
        const float4 x = patch[((ty * 2 + kh) * TI + tx * 2 + kw) * CG + cg];
        acc.x = fmaxf(acc.x, x.x);
        acc.y = fmaxf(acc.y, x.y);
        acc.z = fmaxf(acc.z, x.z);
        acc.w = fmaxf(acc.w, x.w);
      }
    }
    const long long dst = ((img * p.OH + oy) * p.OW + ox) * static_cast<long long>(p.C) + (cg0 + cg) * 4;
    act_store4(out, dst, acc);
    pool_store_side4(p, dst, acc.x, acc.y, acc.z, acc.w);
  }
}

// ----------------------------------------------------------------- direct conv / matmul
// CUDA-core convolution: exact fp32 accumulation (fused multiply-add), any geometry.
// Weights are stored [KH*KW][C][O].  One thread per (pixel, output channel); threads
// of a warp share the pixel, so activation reads are broadcasts and weight reads coalesce.
template <bool INT8>
static __global__ void k_conv_direct(ActRef in, ActRef out, const void* __restrict__ weights, ConvGeom g,
                              ConvEpilogue e) {
  const long long total = g.images * g.OH * g.OW * g.O;
  const float* wf = static_cast<const float*>(weights);
  const int8_t* wq = static_cast<const int8_t*>(weights);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int o = static_cast<int>(i % g.O);
    long long r = i / g.O;
    const int ow = static_cast<int>(r % g.OW);
    r /= g.OW;
    const int oh = static_cast<int>(r % g.OH);
    const long long img = r / g.OH;
    float acc = (!INT8 && e.bias != nullptr) ? e.bias[o] : 0.0f;
    int iacc = 0;
    for (int kh = 0; kh < g.KH; ++kh) {
      const int ih = oh * g.sh - g.pt + kh * g.dh;
      if (ih < 0 || ih >= g.H) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        const int iw = ow * g.sw - g.pl + kw * g.dw;
        if (iw < 0 || iw >= g.W) continue;
        const long long xb = ((img * g.H + ih) * g.W + iw) * g.C;
        const long long wb = static_cast<long long>(kh * g.KW + kw) * g.C * g.O + o;
        for (int c = 0; c < g.C; ++c) {
          if (INT8) {
            iacc += static_cast<int>(in.q[xb + c]) * static_cast<int>(wq[wb + static_cast<long long>(c) * g.O]);
          } else {
            acc = fmaf(act_load(in, xb + c), wf[wb + static_cast<long long>(c) * g.O], acc);
          }
        }
      }
    }
    const float res = e.has_res ? act_load(e.res, i) : 0.0f;
    const float y = INT8 ? conv_finish_i8(e, iacc, o, res, out.fmt == FMT_I8)
                         : conv_finish_f32(e, acc, res);
    act_store(out, i, y);
  }
}

// InnerProduct / Gemm on CUDA cores: y[m][n] = sum_k a[m][k] * w[k][n] (weights
// stored [K][N]); bias is added after the sum, as the reference's matmul + add does.
template <bool INT8>
static __global__ void k_matmul_direct(ActRef a, ActRef out, const void* __restrict__ weights,
                                long long M, int K, int N, ConvEpilogue e, float gemm_beta_unused) {
  const long long total = M * N;
  const float* wf = static_cast<const float*>(weights);
  const int8_t* wq = static_cast<const int8_t*>(weights);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int n = static_cast<int>(i % N);
    const long long m = i / N;
    float acc = 0.0f;
    int iacc = 0;
    for (int k = 0; k < K; ++k) {
      if (INT8) {
        iacc += static_cast<int>(a.q[m * K + k]) * static_cast<int>(wq[static_cast<long long>(k) * N + n]);
      } else {
        acc = fmaf(act_load(a, m * K + k), wf[static_cast<long long>(k) * N + n], acc);
      }
    }
    float y;
    if (INT8) {
      y = conv_finish_i8(e, iacc, n, 0.0f, out.fmt == FMT_I8);
    } else {
      if (e.bias != nullptr) acc = __fadd_rn(acc, e.bias[n]);
      y = conv_finish_f32(e, acc, 0.0f);
    }
    act_store(out, i, y);
  }
}

// Gemm with int8 weights and per-row dynamic activation scales
// (reference: computeGemmRowScales + dequantizeGemmAccumulator): one block per row.
//   s_m = absmax == 0 ? 1 : 127 / absmax;  a_q = Q(a, s_m);
//   y = float(acc) / (s_m * s_B);  y = (y + beta*c) * alpha
static __global__ void k_gemm_i8_rowscale(ActRef a, ActRef out,
                                   const int8_t* __restrict__ wq /*[N][K]*/, int K, int N,
                                   float s_b, const float* __restrict__ c_bias, float alpha,
                                   float beta, int has_c, int scale_alpha) {
  extern __shared__ int8_t row_q[];
  __shared__ float red[32];
  __shared__ float s_row;
  const long long m = blockIdx.x;
  float mx = 0.0f;
  for (int k = threadIdx.x; k < K; k += blockDim.x) mx = fmaxf(mx, fabsf(act_load(a, m * K + k)));
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.0f;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) t = fmaxf(t, red[w]);
    s_row = t == 0.0f ? 1.0f : __fdiv_rn(127.0f, t);
  }
  __syncthreads();
  const float s = s_row;
  for (int k = threadIdx.x; k < K; k += blockDim.x)
    row_q[k] = static_cast<int8_t>(quantize_rha(act_load(a, m * K + k), s));
  __syncthreads();
  const float combined = __fmul_rn(s, s_b);
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    int acc = 0;
    for (int k = 0; k < K; ++k) acc += static_cast<int>(row_q[k]) * static_cast<int>(wq[static_cast<long long>(n) * K + k]);
    float y = __fdiv_rn(static_cast<float>(acc), combined);
    if (has_c) y = __fadd_rn(y, __fmul_rn(c_bias[n], beta));
    if (scale_alpha) y = __fmul_rn(y, alpha);
    act_store(out, m * N + n, y);
  }
}

// Copy between two logical tensors whose elements correspond by logical (ncnn
// ----------------------------------------------------------------- softmax, concat
// Softmax along one storage axis (ConvertSoftmax, NCNNToTosa.cpp:2072-2112): per line
// m = max, e = exp(x - m), s = sum e, out = e * (1/s).  A line is `len` elements `inner`
// apart; line l of an image starts at (l / inner) * len * inner + l % inner.  One warp per line.
struct SoftmaxParams {
  long long images, image_elems;
  int lines, len, inner;
};

static __global__ void k_softmax(ActRef in, ActRef out, SoftmaxParams p) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long total = p.images * p.lines;
  for (long long l = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5; l < total; l += warps) {
    const long long img = l / p.lines;
    const int line = static_cast<int>(l - img * p.lines);
    const long long base = img * p.image_elems + static_cast<long long>(line / p.inner) * p.len * p.inner + line % p.inner;
    float m = __int_as_float(0xff800000);  // -inf
    for (int k = lane; k < p.len; k += 32) m = fmaxf(m, act_load(in, base + static_cast<long long>(k) * p.inner));
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float s = 0.0f;
    for (int k = lane; k < p.len; k += 32) s = __fadd_rn(s, expf(__fadd_rn(act_load(in, base + static_cast<long long>(k) * p.inner), -m)));
    for (int o = 16; o > 0; o >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, o));
    const float r = __fdiv_rn(1.0f, s);
    for (int k = lane; k < p.len; k += 32) {
      const long long i = base + static_cast<long long>(k) * p.inner;
      act_store(out, i, __fmul_rn(expf(__fadd_rn(act_load(in, i), -m)), r));
    }
  }
}

// One input of a Concat (ConvertConcat, NCNNToTosa.cpp:2012-2045): copies [outer][len_in][inner]
// into [outer][len_out][inner] at position `offset` along the middle axis, per image.
struct ConcatParams {
  long long images, in_image_elems, out_image_elems;
  int outer, len_in, len_out, inner, offset;
  int slice;  // 1: the other direction (ConvertSlice, NCNNToTosa.cpp:5458-5544): `in` is the long
              // tensor [outer][len_out][inner], `out` receives [outer][len_in][inner] from `offset`
};

static __global__ void k_concat_copy(ActRef in, ActRef out, ConcatParams p) {
  const long long per = static_cast<long long>(p.outer) * p.len_in * p.inner;
  const long long total = p.images * per;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long img = i / per;
    long long r = i - img * per;
    const int in_i = static_cast<int>(r % p.inner);
    r /= p.inner;
    const int l = static_cast<int>(r % p.len_in);
    const int o = static_cast<int>(r / p.len_in);
    const long long wide = img * p.out_image_elems + (static_cast<long long>(o) * p.len_out + p.offset + l) * p.inner + in_i;
    const long long narrow = img * p.in_image_elems + (i - img * per);
    if (p.slice) act_store(out, narrow, act_load(in, wide));
    else act_store(out, wide, act_load(in, narrow));
  }
}

// row-major [c][h][w]) index, optionally transposing a rank-2 source: serves
// Flatten/Reshape/Squeeze/ExpandDims and rank-2 Permute.
struct RelayoutParams {
  long long images;
  long long count;            // logical elements per image
  int src_rank, sc, sh, sw;   // logical dims (rank 1: sw; rank 2: sh x sw; rank 3: sc x sh x sw)
  int dst_rank, dc, dh, dw;
  int transpose2d;            // source is read as its rank-2 transpose
  int permute3d;              // rank 3 to rank 3: destination extent i is source extent perm[i]
  int perm[3];
  // rank 4 [c][d][h][w] -> [c][h][w][d] (ncnn order_type 3, import_permute, ImportTensor.cpp:374-383): both sides
  // are stored in their logical order; s4 are the source extents d, h, w
  int permute4d;
  int s4d, s4h, s4w;
};

__device__ __forceinline__ long long storage_offset(int rank, int c_dim, int h_dim, int w_dim,
                                                    long long logical) {
  if (rank != 3) return logical;
  const int w = static_cast<int>(logical % w_dim);
  const long long r = logical / w_dim;
  const int h = static_cast<int>(r % h_dim);
  const int c = static_cast<int>(r / h_dim);
  return (static_cast<long long>(h) * w_dim + w) * c_dim + c;
}

static __global__ void k_relayout(ActRef in, ActRef out, RelayoutParams p) {
  const long long total = p.images * p.count;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long img = i / p.count;
    const long long l = i - img * p.count;
    long long src_l = l;
    if (p.transpose2d) {
      // destination is [dh][dw] = source[sw'][sh'] transposed
      const int col = static_cast<int>(l % p.dw);
      const int row = static_cast<int>(l / p.dw);
      src_l = static_cast<long long>(col) * p.sw + row;
    } else if (p.permute3d) {
      int d[3], sidx[3];
      d[2] = static_cast<int>(l % p.dw);
      const long long r = l / p.dw;
      d[1] = static_cast<int>(r % p.dh);
      d[0] = static_cast<int>(r / p.dh);
#pragma unroll
      for (int k = 0; k < 3; ++k) sidx[p.perm[k]] = d[k];
      src_l = (static_cast<long long>(sidx[0]) * p.sh + sidx[1]) * p.sw + sidx[2];
    } else if (p.permute4d) {
      // destination index (c, h, w, d) reads source (c, d, h, w)
      const int dd = static_cast<int>(l % p.s4d);
      long long r = l / p.s4d;
      const int ww = static_cast<int>(r % p.s4w);
      r /= p.s4w;
      const int hh = static_cast<int>(r % p.s4h);
      const long long cc = r / p.s4h;
      src_l = ((cc * p.s4d + dd) * p.s4h + hh) * p.s4w + ww;
    }
    const long long so = img * p.count + storage_offset(p.src_rank, p.sc, p.sh, p.sw, src_l);
    const long long dof = img * p.count + storage_offset(p.dst_rank, p.dc, p.dh, p.dw, l);
    act_store(out, dof, act_load(in, so));
  }
}

// ----------------------------------------------------------------- 2x2 stride-2 deconvolution
// The only Deconvolution the reference imports (ImportDetection.cpp:349-470): out[2h+a][2w+b][o] =
// bias[o] + sum_c in[h][w][c] * W[o][c][a][b], no kernel flip (ConvertDeconvolution,
// NCNNToTosa.cpp:2737-2990).  Weights arrive repacked [a][b][c][o]; one thread per output value,
// neighbouring threads neighbouring output channels.
struct DeconvParams {
  long long images;
  int H, W, C, O;  // input extents, output channels
  int relu;
};

static __global__ void k_deconv2x2(ActRef in, ActRef out, const float* __restrict__ w,
                                   const float* __restrict__ bias, DeconvParams p) {
  const long long total = p.images * 4ll * p.H * p.W * p.O;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int o = static_cast<int>(i % p.O);
    long long r = i / p.O;
    const int ow = static_cast<int>(r % (2 * p.W));
    r /= 2 * p.W;
    const int oh = static_cast<int>(r % (2 * p.H));
    const long long img = r / (2 * p.H);
    const long long src = ((img * p.H + (oh >> 1)) * p.W + (ow >> 1)) * p.C;
    const float* wk = w + static_cast<long long>((oh & 1) * 2 + (ow & 1)) * p.C * p.O + o;
    float acc = bias != nullptr ? bias[o] : 0.0f;
    for (int c = 0; c < p.C; ++c) acc = __fadd_rn(__fmul_rn(act_load(in, src + c), wk[static_cast<long long>(c) * p.O]), acc);
    act_store(out, i, p.relu ? fmaxf(acc, 0.0f) : acc);
  }
}

// ----------------------------------------------------------------- broadcast, remap
// BinaryOp with numpy-style broadcasting over the logical [c, h, w] dims (computeBinaryResult,
// NCNNOps.cpp:1181-1245; ConvertBinary, NCNNToTosa.cpp:5111-5223).  Every operand is addressed as
// c*sc + h*sh + w*sw in its own storage, with a zero stride where it is broadcast.
struct BroadcastParams {
  long long images;
  int rank, C, H, W;                  // output logical dims (missing leading dims are 1)
  long long a_image, b_image, o_image;  // elements per image
  int a_sc, a_sh, a_sw, b_sc, b_sh, b_sw;
  BinaryParams op;
};

static __global__ void k_binary_broadcast(ActRef a, ActRef b, ActRef out, BroadcastParams p) {
  const long long total = p.images * p.o_image;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long img = i / p.o_image;
    long long r = i - img * p.o_image;
    int c = 0, h = 0, w = 0;
    if (p.rank == 3) {  // storage [h][w][c]
      c = static_cast<int>(r % p.C);
      r /= p.C;
      w = static_cast<int>(r % p.W);
      h = static_cast<int>(r / p.W);
    } else {            // [h][w] or [w]
      w = static_cast<int>(r % p.W);
      h = static_cast<int>(r / p.W);
    }
    const float x = act_load(a, img * p.a_image + static_cast<long long>(c) * p.a_sc + static_cast<long long>(h) * p.a_sh + static_cast<long long>(w) * p.a_sw);
    const float y = act_load(b, img * p.b_image + static_cast<long long>(c) * p.b_sc + static_cast<long long>(h) * p.b_sh + static_cast<long long>(w) * p.b_sw);
    act_store(out, i, binary_apply(p.op, x, y));
  }
}

// Index remapping of rank-3 tensors: out(h, w, c) takes one input element (or a constant, or a
// bilinear blend of four).  REMAP_PAD: constant padding (ConvertPadding, NCNNToTosa.cpp:2114-2250);
// REMAP_SHUFFLE: channel shuffle, [group][C/group] -> [C/group][group] (ConvertShuffleChannel,
// :5394-5456); REMAP_NEAREST / REMAP_BILINEAR: Interp (ConvertInterp, :2252-2572).
enum : int { REMAP_PAD = 0, REMAP_SHUFFLE = 1, REMAP_NEAREST = 2, REMAP_BILINEAR = 3 };
struct RemapParams {
  long long images;
  int mode;
  int C, H, W, OH, OW;      // input and output extents (channels unchanged)
  int top, left;            // REMAP_PAD
  float value;
  int group;                // REMAP_SHUFFLE
  int scale_h, scale_w;     // REMAP_NEAREST without an explicit size
  int explicit_h, explicit_w;
  int align_corner;         // REMAP_BILINEAR
};

// source coordinate of bilinear resize exactly as the reference spells it in f32
__device__ __forceinline__ void bilinear_coordinate(int index, int in, int out, int align, int* base, float* frac) {
  const float in_f = static_cast<float>(in), out_f = static_cast<float>(out), idx = static_cast<float>(index);
  const float in_max = __fadd_rn(in_f, -1.0f);
  float src;
  if (align) src = __fdiv_rn(__fmul_rn(idx, in_max), __fadd_rn(out_f, -1.0f));
  else src = __fadd_rn(__fdiv_rn(__fmul_rn(__fadd_rn(idx, 0.5f), in_f), out_f), -0.5f);
  src = fminf(fmaxf(src, 0.0f), in_max);
  int b = static_cast<int>(floorf(src));
  b = min(b, in - 2);
  *base = b;
  *frac = __fadd_rn(src, -static_cast<float>(b));
}

static __global__ void k_remap(ActRef in, ActRef out, RemapParams p) {
  const long long in_image = static_cast<long long>(p.H) * p.W * p.C;
  const long long out_image = static_cast<long long>(p.OH) * p.OW * p.C;
  const long long total = p.images * out_image;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long img = i / out_image;
    long long r = i - img * out_image;
    const int c = static_cast<int>(r % p.C);
    r /= p.C;
    const int w = static_cast<int>(r % p.OW);
    const int h = static_cast<int>(r / p.OW);
    const long long base = img * in_image;
    auto at = [&](int y, int x, int ch) { return act_load(in, base + (static_cast<long long>(y) * p.W + x) * p.C + ch); };
    float v;
    if (p.mode == REMAP_PAD) {
      const int y = h - p.top, x = w - p.left;
      v = (y >= 0 && y < p.H && x >= 0 && x < p.W) ? at(y, x, c) : p.value;
    } else if (p.mode == REMAP_SHUFFLE) {
      v = at(h, w, (c % p.group) * (p.C / p.group) + c / p.group);
    } else if (p.mode == REMAP_NEAREST) {
      const int y = p.explicit_h ? static_cast<int>((static_cast<long long>(h) * p.H) / p.OH) : h / p.scale_h;
      const int x = p.explicit_w ? static_cast<int>((static_cast<long long>(w) * p.W) / p.OW) : w / p.scale_w;
      v = at(y, x, c);
    } else {
      int y0, x0;
      float fy, fx;
      bilinear_coordinate(h, p.H, p.OH, p.align_corner, &y0, &fy);
      bilinear_coordinate(w, p.W, p.OW, p.align_corner, &x0, &fx);
      const float gx = __fadd_rn(1.0f, -fx), gy = __fadd_rn(1.0f, -fy);
      const float top = __fadd_rn(__fmul_rn(at(y0, x0, c), gx), __fmul_rn(at(y0, x0 + 1, c), fx));
      const float bottom = __fadd_rn(__fmul_rn(at(y0 + 1, x0, c), gx), __fmul_rn(at(y0 + 1, x0 + 1, c), fx));
      v = __fadd_rn(__fmul_rn(top, gy), __fmul_rn(bottom, fy));
    }
    act_store(out, i, v);
  }
}

// Mean over a set of logical axes of a rank-3 tensor (ConvertReduction, NCNNToTosa.cpp:5546-5682):
// reduce_sum axis by axis in storage order (h, then w, then c), then one multiplication by
// coeff / count.  One thread per output element; `red_*` is 1 where the axis is reduced.
struct ReduceParams {
  long long images;
  int C, H, W;
  int red_c, red_h, red_w;
  float factor;
};

static __global__ void k_reduce_mean(ActRef in, ActRef out, ReduceParams p) {
  const int oc = p.red_c ? 1 : p.C, oh = p.red_h ? 1 : p.H, ow = p.red_w ? 1 : p.W;
  const long long per = static_cast<long long>(oc) * oh * ow;
  const long long in_image = static_cast<long long>(p.C) * p.H * p.W;
  const long long total = p.images * per;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long img = i / per;
    long long r = i - img * per;  // output storage order [h][w][c] over the kept extents
    const int c0 = static_cast<int>(r % oc);
    r /= oc;
    const int w0 = static_cast<int>(r % ow);
    const int h0 = static_cast<int>(r / ow);
    const int nc = p.red_c ? p.C : 1, nh = p.red_h ? p.H : 1, nw = p.red_w ? p.W : 1;
    float sc = 0.0f;
    for (int c = 0; c < nc; ++c) {
      float sw = 0.0f;
      for (int w = 0; w < nw; ++w) {
        float sh = 0.0f;
        for (int h = 0; h < nh; ++h)
          sh = __fadd_rn(sh, act_load(in, img * in_image + (static_cast<long long>(h0 + h) * p.W + (w0 + w)) * p.C + c0 + c));
        sw = __fadd_rn(sw, sh);
      }
      sc = __fadd_rn(sc, sw);
    }
    act_store(out, i, __fmul_rn(sc, p.factor));
  }
}

// ----------------------------------------------------------------- standalone int8 boundary ops
// Element i belongs to channel (i / inner) % channels.  Scales/bias hold one value or
// one per channel.
//   quantize:    y = Q(x, s[c])                                   (ConvertQuantize)
//   dequantize:  y = float(v) * s[c] (+ bias[c])                  (dequantizeNcnn)
//   requantize:  t = float(v) * s_in[c] (+ bias[c]); relu?; y = Q(t, s_out[c])
struct QuantOpParams {
  long long count;
  long long inner;
  int channels;
  const float* scale_in;
  int nscale_in;
  const float* scale_out;
  int nscale_out;
  const float* bias;
  int nbias;
  int relu;
};

static __global__ void k_op_quantize(const float* __restrict__ x, int8_t* __restrict__ y, QuantOpParams p) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < p.count;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>((i / p.inner) % p.channels);
    y[i] = static_cast<int8_t>(quantize_rha(x[i], p.scale_in[p.nscale_in == 1 ? 0 : c]));
  }
}

static __global__ void k_op_dequantize(const int* __restrict__ v, float* __restrict__ y, QuantOpParams p) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < p.count;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>((i / p.inner) % p.channels);
    float t = __fmul_rn(static_cast<float>(v[i]), p.scale_in[p.nscale_in == 1 ? 0 : c]);
    if (p.bias != nullptr) t = __fadd_rn(t, p.bias[p.nbias == 1 ? 0 : c]);
    y[i] = t;
  }
}

static __global__ void k_op_requantize(const int* __restrict__ v, int8_t* __restrict__ y, QuantOpParams p) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < p.count;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>((i / p.inner) % p.channels);
    float t = __fmul_rn(static_cast<float>(v[i]), p.scale_in[p.nscale_in == 1 ? 0 : c]);
    if (p.bias != nullptr) t = __fadd_rn(t, p.bias[p.nbias == 1 ? 0 : c]);
    if (p.relu) t = fmaxf(t, 0.0f);
    y[i] = static_cast<int8_t>(quantize_rha(t, p.scale_out[p.nscale_out == 1 ? 0 : c]));
  }
}

}  // namespace nb
