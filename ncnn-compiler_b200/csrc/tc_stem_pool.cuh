// Stem convolution with the 3x3 stride-2 max pooling that follows it, in one kernel (bf16-pair or int8 operands).
//
// tc_stem_kernel writes the stem's result (the largest tensor of a ResNet) to HBM and the pooling kernel reads
// it back.  Here a CTA owns a contiguous range of POOLED rows and walks the convolution rows they need in
// order: 2j-1, 2j, 2j+1 for the first pooled row j of the range (or of an image), then two new rows per pooled
// row, because row 2j+1 is also row 2(j+1)-1.  Every convolution row is computed like a tile of tc_stem_kernel
// (input rows by TMA, windows read in place, three bf16 MMAs or one int8 MMA per K step; two MMA-issuing warps
// take alternate rows).  Eight epilogue warps drain it from TMEM with bias and activation; a thread meets the
// same pixel column and channels in every row, so the maximum over the three rows is kept in registers, and
// the row that completes a pooled row writes it into one row of shared memory, from which the warps take the
// maxima over pixels 2x-1 .. 2x+1, convert them and store the pooled row with TMA.  The stem's own result never
// reaches HBM.  One convolution row per range is computed twice (2 % at 148 ranges over 64 x 56 pooled rows).
// The values are those of the two separate kernels: the same bits.  Results: bf16 pairs (hi and mid planes)
// for the bf16 form; fp32, and optionally an int8 copy Q(value, side_scale) for the int8 convolution that reads
// the pooled tensor next, for the int8 form.
#pragma once

#include "tc_stem.cuh"

namespace nb {

constexpr int kStemPoolThreads = 352;  // warp 0 producer, 1 and 10 MMA, 2-9 epilogue and pooling (two warps per TMEM lane quarter)
constexpr int kStemPoolEpiThreads = 256;

struct TcStemPoolParams {
  TcStemParams s;       // the convolution (tiles, staging and output fields unused)
  int images;
  int POH, POW;         // pooled extent: OH / 2, OW / 2 (3x3 windows, stride 2, one pixel of padding)
  int ring_row_bytes;   // the row of vertical maxima: OW x N fp32, rounded to 1 KB
  int stage_tile_bytes; // one staging tile of the pooled row: POW rows x 64 bytes, rounded to 1 KB
  int row_stages;       // input row stages in shared memory: 4, or 2 where 4 do not fit
  int has_side;         // fp32 results: an int8 copy leaves through the second output map
  float side_scale;
};

// f(img, oh, last) for every convolution row of this CTA, `last` when the row completes a pooled row
template <class F>
__device__ __forceinline__ void stem_pool_rows(const TcStemPoolParams& p, F&& f) {
  const long long total = static_cast<long long>(p.images) * p.POH;  // (fits an int: the planner checks)
  const int q0 = static_cast<int>(total * blockIdx.x / gridDim.x), q1 = static_cast<int>(total * (blockIdx.x + 1) / gridDim.x);
  int img = q0 / p.POH, j = q0 - img * p.POH;
  for (int q = q0; q < q1; ++q) {
    const bool first = q == q0 || j == 0;  // nothing of this pooled row's window has been computed yet
    for (int oh = max(first ? 2 * j - 1 : 2 * j, 0); oh <= 2 * j + 1; ++oh)
      if (!f(img, oh, j, oh == 2 * j + 1, static_cast<long long>(q))) return;
    if (++j == p.POH) {
      j = 0;
      ++img;
    }
  }
}

template <int KIND>
__global__ void __launch_bounds__(kStemPoolThreads, 1)
tc_stem_pool_kernel(const __grid_constant__ TcStemPoolParams pp, const __grid_constant__ CUtensorMap map_a0,
                    const __grid_constant__ CUtensorMap map_a1, const __grid_constant__ CUtensorMap map_b0,
                    const __grid_constant__ CUtensorMap map_b1, const __grid_constant__ CUtensorMap map_o0,
                    const __grid_constant__ CUtensorMap map_o1) {
  using namespace ptx;
  const TcStemParams& p = pp.s;
  constexpr int PLANES = KIND == GEMM_I8 ? 1 : 2;
  grid_dependency_trigger();
  extern __shared__ uint8_t stem_pool_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[4];
  __shared__ __align__(8) uint64_t empty_bar[4];
  __shared__ __align__(8) uint64_t tfull_bar[4];   // four accumulators of 64 columns: two per MMA issuer
  __shared__ __align__(8) uint64_t tempty_bar[4];
  __shared__ __align__(8) uint64_t weights_bar;
  __shared__ __align__(16) float tile_bias[128];
  __shared__ __align__(16) float tile_scale[128];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(stem_pool_smem_raw) + 1023u) & ~1023u;
  const int S = pp.row_stages;  // row stages (a stage holds the KH input rows of one convolution row, both planes)
  const uint32_t b_region = smem_base;  // [KH][plane][b_slot]
  const uint32_t a_region = b_region + static_cast<uint32_t>(p.KH * PLANES) * static_cast<uint32_t>(p.b_slot);
  const uint32_t stage_bytes = static_cast<uint32_t>(PLANES) * static_cast<uint32_t>(p.a_plane_bytes);
  const uint32_t ring = a_region + static_cast<uint32_t>(S) * stage_bytes;      // one row of vertical maxima, fp32
  const uint32_t staging = ring + static_cast<uint32_t>(pp.ring_row_bytes);    // pooled row: tiles of [POW][64 B]
  volatile int* abort_ptr = &abort_flag;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&full_bar[i]), 1);
      mbar_init(smem_u32(&empty_bar[i]), 1);
      mbar_init(smem_u32(&tfull_bar[i]), 1);
      mbar_init(smem_u32(&tempty_bar[i]), kStemPoolEpiThreads / 32);
    }
    mbar_init(smem_u32(&weights_bar), 1);
    fence_mbar_init();
    prefetch_tensormap(&map_a0);
    prefetch_tensormap(&map_b0);
    if (PLANES == 2) {
      prefetch_tensormap(&map_a1);
      prefetch_tensormap(&map_b1);
    }
    prefetch_tensormap(&map_o0);
    if (PLANES == 2 || pp.has_side) prefetch_tensormap(&map_o1);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 256);
    tmem_relinquish();
  }
  if (threadIdx.x >= 64) {
    const int t = static_cast<int>(threadIdx.x) - 64;
    if (t < 128) {
      tile_bias[t] = (p.bias != nullptr && t < p.N) ? __ldg(p.bias + t) : 0.0f;
      tile_scale[t] = (KIND == GEMM_I8 && t < p.N) ? __ldg(p.scale + t) : 0.0f;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ producer: weights once, then rows
    const CUtensorMap* map_a = lane ? &map_a1 : &map_a0;
    const CUtensorMap* map_b = lane ? &map_b1 : &map_b0;
    const uint32_t wb = smem_u32(&weights_bar);
    if (lane == 0) mbar_arrive_expect_tx(wb, static_cast<uint32_t>(p.KH * PLANES) * static_cast<uint32_t>(p.N) * 64u);
    __syncwarp();
    if (lane < PLANES) {
      // (the K coordinate counts elements: 32 bf16 or 64 int8 per filter row)
      for (int kh = 0; kh < p.KH; ++kh)
        tma_load_2d(b_region + static_cast<uint32_t>(kh * PLANES + lane) * p.b_slot, map_b, wb, kh * (KIND == GEMM_I8 ? 64 : 32), 0);
    }
    int s = 0;
    uint32_t ph = 0;
    long long issued = 0;
    bool ok = true;
    stem_pool_rows(pp, [&](int img, int oh, int, bool, long long) {
      const uint32_t fb = smem_u32(&full_bar[s]);
      int w = 1;
      if (lane == 0) {
        w = mbar_wait_bounded(smem_u32(&empty_bar[s]), ph ^ 1u, abort_ptr, kTcWaitLimitNs) ? 1 : 0;
        if (w) mbar_arrive_expect_tx(fb, static_cast<uint32_t>(PLANES * p.KH) * static_cast<uint32_t>(p.row_bytes));
      }
      w = __shfl_sync(0xffffffffu, w, 0);
      if (!w) {
        ok = false;
        return false;
      }
      // rows above or below the image are filled with zeros by the copy
      if (lane < PLANES)
        tma_load_4d(a_region + static_cast<uint32_t>(s) * stage_bytes + static_cast<uint32_t>(lane) * p.a_plane_bytes, map_a, fb,
                    0, 0, oh * p.stride_h - p.pad_t, img);
      ++issued;
      if (++s == S) {
        s = 0;
        ph ^= 1u;
      }
      return true;
    });
    if (lane == 0) {
      if (!ok && atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_PRODUCER);
      if (*abort_ptr != 0) {
        int zero = 0;
        mbar_wait_bounded(wb, 0, &zero, 200000000ull);
        const long long first = issued > S ? issued - S : 0;
        for (long long i = first; i < issued; ++i)
          mbar_wait_bounded(smem_u32(&full_bar[i % S]), static_cast<uint32_t>((i / S) & 1), &zero, 200000000ull);
      }
    }
  } else if (warp == 1 || warp == 10) {
    // ---------------------------------------------------------- MMA issuers (the MMAs of a row as in tc_stem_kernel)
    // A thread issues one of these narrow MMAs every ~75 cycles, the tensor pipe could take one every ~48: two
    // threads in two warps issue alternate rows, each with its own row stage and its own accumulator (MMAs
    // into one accumulator must come from one thread, only then are they ordered).
    const int me = warp == 1 ? 0 : 1;
    if (lane == 0) {
      const uint32_t idesc = KIND == GEMM_I8 ? instr_desc(2u, 1u, kTcBlockM, static_cast<uint32_t>(p.N))
                                             : instr_desc(1u, 1u, kTcBlockM, static_cast<uint32_t>(p.N));
      bool ok = mbar_wait_bounded(smem_u32(&weights_bar), 0, abort_ptr, kTcWaitLimitNs);
      tc_fence_after_sync();
      const uint64_t a_fixed = smem_desc_plain(0u, 16u, 128u);
      const uint64_t b_fixed = smem_desc_kmajor(0u, 64u);
      const uint64_t a_plane_units = static_cast<uint64_t>(p.a_plane_bytes) >> 4;
      const uint64_t row_units = static_cast<uint64_t>(p.row_bytes) >> 4;
      const uint64_t b_slot_units = static_cast<uint64_t>(p.b_slot) >> 4;
      const uint64_t b_first = b_fixed + ((b_region & 0x3ffffu) >> 4);
      // row r of this CTA's sequence: issuer r & 1, stage r % S, accumulator r & 3 (two per issuer, so that the
      // MMAs of its next row run while the epilogue drains the row before)
      int row = 0;
      if (ok) {
        stem_pool_rows(pp, [&](int, int, int, bool, long long) {
          const int r = row++;
          if ((r & 1) != me) return true;
          const int s = r % S, acc = r & 3;
          const uint32_t ph = static_cast<uint32_t>((r / S) & 1), acc_ph = static_cast<uint32_t>((r >> 2) & 1);
          if (!mbar_wait_bounded(smem_u32(&tempty_bar[acc]), acc_ph ^ 1u, abort_ptr, kTcWaitLimitNs) ||
              !mbar_wait_bounded(smem_u32(&full_bar[s]), ph, abort_ptr, kTcWaitLimitNs)) {
            ok = false;
            return false;
          }
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * 64u;
          const uint64_t a_hi0 = a_fixed + (((a_region + static_cast<uint32_t>(s) * stage_bytes) & 0x3ffffu) >> 4);
          uint32_t accumulate = 0u;
          for (int kh = 0; kh < p.KH; ++kh) {
            const uint64_t a_hi = a_hi0 + static_cast<uint64_t>(kh) * row_units;
            const uint64_t b_hi = b_first + static_cast<uint64_t>(PLANES * kh) * b_slot_units;
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
              const uint64_t ka = a_hi + 2u * ks;
              const uint64_t kb = b_hi + 2u * ks;
              if (KIND == GEMM_I8) {
                mma_i8(d_tmem, ka, kb, idesc, accumulate);
              } else {
                mma_f16(d_tmem, ka + a_plane_units, kb, idesc, accumulate);  // mid * hi
                mma_f16(d_tmem, ka, kb + b_slot_units, idesc, 1u);           // hi * mid
                mma_f16(d_tmem, ka, kb, idesc, 1u);                          // hi * hi
              }
              accumulate = 1u;
            }
          }
          tc_commit(smem_u32(&empty_bar[s]));
          tc_commit(smem_u32(&tfull_bar[acc]));
          return true;
        });
      }
      if (!ok && atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_MMA);
    }
  } else {
    // ------------------------------------------------------------ epilogue and pooling (warps 2-9)
    // warps 2-5 drain the first half of the channels, warps 6-9 the second; all 256 threads pool
    const int t = static_cast<int>(threadIdx.x) - 64;
    const int col_half = warp >= 6 ? 1 : 0;
    const int quarter = warp & 3;  // TMEM lanes 32*quarter.. = pixels of the convolution row
    const int px = quarter * 32 + lane;
    const int chunks = p.N / 4;                // 16-byte chunks of a ring row entry (N fp32 per pixel)
    const uint32_t mask = static_cast<uint32_t>(chunks > 16 ? 15 : chunks - 1);  // chunk ^ (pixel & mask): spreads the banks
    const uint32_t entry = static_cast<uint32_t>(p.N) * 4u;
    const int chunk_shift = p.N == 64 ? 4 : 3;
    // none, ReLU and clip as one clamp (the planner admits no other activation): one copy of a many-way
    // activation per value made this loop stall on instruction fetch
    const float act_lo = p.act == ACT_RELU ? 0.0f : (p.act == ACT_CLIP ? p.act_a : -INFINITY);
    const float act_hi = p.act == ACT_CLIP ? p.act_b : INFINITY;
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    // Vertical maxima stay in registers: this thread drains the same pixel column and the same channels of every
    // convolution row, so the maximum over rows 2j-1, 2j, 2j+1 needs no shared memory.  `odd_row` holds this
    // thread's values of the last odd row (row 2j+1 is also row 2(j+1)-1), `upper` the maximum of rows 2j-1 and 2j;
    // the odd row that completes a pooled row writes max(upper, row) into the one row of shared memory from which
    // the horizontal maxima are taken: a third of the shared-memory reads and half of the writes of pooling out
    // of three stored rows, next to MMAs that read their operands from the same memory.
    float odd_row[32], upper[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) odd_row[i] = upper[i] = -INFINITY;
    stem_pool_rows(pp, [&](int img, int oh, int j, bool last, long long q) {
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&tfull_bar[acc]), acc_ph, abort_ptr, kTcWaitLimitNs) ? 1 : 0) != 0;
      if (!ok) return false;
      tc_fence_after_sync();
      // ---- drain: bias and activation as the stand-alone epilogue
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc) * 64u;
      const bool odd = (oh & 1) != 0;
      const bool row_above = oh > 0;  // an even row has row oh - 1 above it in `odd_row` unless it is the image's first
      // this thread's 16 or 32 accumulator columns into registers, then the accumulator is free for the MMAs again
      const int c_first = col_half * (p.N / 2);
      const bool two_chunks = p.N / 2 > 16;
      uint32_t vv[2][16];
      tmem_ld16(t_row + static_cast<uint32_t>(c_first), vv[0]);
      if (two_chunks) tmem_ld16(t_row + static_cast<uint32_t>(c_first + 16), vv[1]);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
      acc = (acc + 1) & 3;
      if (acc == 0) acc_ph ^= 1u;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        if (cc == 0 || two_chunks) {
          const int c0 = c_first + cc * 16;
          const uint32_t (&v)[16] = vv[cc];
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const float4 b4 = *reinterpret_cast<const float4*>(&tile_bias[c0 + 4 * g]);
            float y[4];
            if (KIND == GEMM_I8) {
              // dequantise: float(accumulator) * scale[channel], then bias (the order of the stand-alone epilogue)
              const float4 s4 = *reinterpret_cast<const float4*>(&tile_scale[c0 + 4 * g]);
              y[0] = __fmul_rn(static_cast<float>(static_cast<int>(v[4 * g + 0])), s4.x);
              y[1] = __fmul_rn(static_cast<float>(static_cast<int>(v[4 * g + 1])), s4.y);
              y[2] = __fmul_rn(static_cast<float>(static_cast<int>(v[4 * g + 2])), s4.z);
              y[3] = __fmul_rn(static_cast<float>(static_cast<int>(v[4 * g + 3])), s4.w);
            } else {
              y[0] = __uint_as_float(v[4 * g + 0]);
              y[1] = __uint_as_float(v[4 * g + 1]);
              y[2] = __uint_as_float(v[4 * g + 2]);
              y[3] = __uint_as_float(v[4 * g + 3]);
            }
            y[0] = fminf(fmaxf(__fadd_rn(__fadd_rn(y[0], b4.x), 0.0f), act_lo), act_hi);
            y[1] = fminf(fmaxf(__fadd_rn(__fadd_rn(y[1], b4.y), 0.0f), act_lo), act_hi);
            y[2] = fminf(fmaxf(__fadd_rn(__fadd_rn(y[2], b4.z), 0.0f), act_lo), act_hi);
            y[3] = fminf(fmaxf(__fadd_rn(__fadd_rn(y[3], b4.w), 0.0f), act_lo), act_hi);
            float* up = &upper[cc * 16 + 4 * g];
            float* od = &odd_row[cc * 16 + 4 * g];
            if (!odd) {
#pragma unroll
              for (int e = 0; e < 4; ++e) up[e] = row_above ? fmaxf(od[e], y[e]) : y[e];
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e) od[e] = y[e];
              if (last && px < p.OW) {
                const uint32_t chunk = static_cast<uint32_t>(c0 / 4 + g);
                const uint32_t at = ring + static_cast<uint32_t>(px) * entry + ((chunk ^ (static_cast<uint32_t>(px) & mask)) << 4);
                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(at), "f"(fmaxf(up[0], y[0])), "f"(fmaxf(up[1], y[1])),
                             "f"(fmaxf(up[2], y[2])), "f"(fmaxf(up[3], y[3]))
                             : "memory");
              }
            }
          }
        }
      }
      if (last) {
        // ---- pooled row j: horizontal maxima over pixels 2x-1 .. 2x+1 of the row of vertical maxima
        if (t == 0) tma_store_wait_read(0);  // the staging tiles of the pooled row before have been read out
        named_barrier_sync(1, kStemPoolEpiThreads);  // the row of vertical maxima is complete
        const int items = pp.POW * chunks;
#pragma unroll 1
        for (int item = t; item < items; item += kStemPoolEpiThreads) {
          const int x = item >> chunk_shift, c = item & (chunks - 1);
          // (pixel -1 is replaced by pixel 0: a maximum does not change when an element is taken twice)
          float4 v[3];
#pragma unroll
          for (int dx = 0; dx < 3; ++dx) {
            const int sx = max(2 * x + dx - 1, 0);
            const uint32_t off = static_cast<uint32_t>(sx) * entry + ((static_cast<uint32_t>(c) ^ (static_cast<uint32_t>(sx) & mask)) << 4);
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v[dx].x), "=f"(v[dx].y), "=f"(v[dx].z), "=f"(v[dx].w) : "r"(ring + off));
          }
          float4 m = v[0];
#pragma unroll
          for (int i = 1; i < 3; ++i) m = make_float4(fmaxf(m.x, v[i].x), fmaxf(m.y, v[i].y), fmaxf(m.z, v[i].z), fmaxf(m.w, v[i].w));
          if (KIND == GEMM_I8) {
            // fp32 results: staging [16-channel box][POW rows][64 bytes]; then the int8 copy, one tile of POW rows x N bytes
            const uint32_t at = staging + static_cast<uint32_t>(c >> 2) * static_cast<uint32_t>(pp.stage_tile_bytes) + stage_chunk_offset(x, c & 3);
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(at), "f"(m.x), "f"(m.y), "f"(m.z), "f"(m.w) : "memory");
            if (pp.has_side) {
              const uint32_t word = (static_cast<uint32_t>(quantize_rha(m.x, pp.side_scale)) & 0xffu) |
                                    ((static_cast<uint32_t>(quantize_rha(m.y, pp.side_scale)) & 0xffu) << 8) |
                                    ((static_cast<uint32_t>(quantize_rha(m.z, pp.side_scale)) & 0xffu) << 16) |
                                    ((static_cast<uint32_t>(quantize_rha(m.w, pp.side_scale)) & 0xffu) << 24);
              const uint32_t side_at = staging + static_cast<uint32_t>(p.N / 16) * static_cast<uint32_t>(pp.stage_tile_bytes) +
                                       stage_chunk_offset(x, c >> 2) + static_cast<uint32_t>((c & 3) * 4);
              asm volatile("st.shared.b32 [%0], %1;" ::"r"(side_at), "r"(word) : "memory");
            }
          } else {
            uint32_t hi0, mid0, hi1, mid1;
            split_bf16x2(m.x, m.y, hi0, mid0);
            split_bf16x2(m.z, m.w, hi1, mid1);
            // staging: [plane][32-channel half][POW rows][64 bytes], 64-byte swizzle as the store expects
            const int half = c >> 3, c8 = c & 7;
            const uint32_t at = staging + static_cast<uint32_t>(half) * static_cast<uint32_t>(pp.stage_tile_bytes) +
                                stage_chunk_offset(x, c8 >> 1) + static_cast<uint32_t>((c8 & 1) * 8);
            const uint32_t plane = static_cast<uint32_t>((p.N + 31) / 32) * static_cast<uint32_t>(pp.stage_tile_bytes);
            asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(at), "r"(hi0), "r"(hi1) : "memory");
            asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(at + plane), "r"(mid0), "r"(mid1) : "memory");
          }
        }
        fence_proxy_async_smem();
        named_barrier_sync(1, kStemPoolEpiThreads);  // staged; and every read of the ring for this pooled row is done
        if (t == 0) {
          const int m_first = static_cast<int>(q) * pp.POW;  // pooled pixels before this row
          if (KIND == GEMM_I8) {
            const int boxes = p.N / 16;
            for (int b = 0; b < boxes; ++b) tma_store_2d(&map_o0, staging + static_cast<uint32_t>(b) * pp.stage_tile_bytes, 16 * b, m_first);
            if (pp.has_side) tma_store_2d(&map_o1, staging + static_cast<uint32_t>(boxes) * pp.stage_tile_bytes, 0, m_first);
          } else {
            const int halves = (p.N + 31) / 32;
            for (int h = 0; h < halves; ++h) {
              tma_store_2d(&map_o0, staging + static_cast<uint32_t>(h) * pp.stage_tile_bytes, 32 * h, m_first);
              tma_store_2d(&map_o1, staging + static_cast<uint32_t>(halves + h) * pp.stage_tile_bytes, 32 * h, m_first);
            }
          }
          tma_store_commit();
        }
      }
      (void)img;
      return true;
    });
    if (!ok && lane == 0 && atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_EPILOGUE);
    if (t == 0) tma_store_wait_all();
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, 256);
}

}  // namespace nb
