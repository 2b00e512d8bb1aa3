// The second half, or the whole, of an inverted-residual block in one kernel:
//   [1x1 "expand" convolution + activation ->] 3x3 depthwise convolution + activation -> 1x1 "projection"
//   convolution (+ bias, residual, activation).
//
// Run one after the other these layers write the widest tensors of the network to HBM and read them back, on
// layers that are bound by HBM either way.  Here the expanded tensor and the depthwise result never leave the
// SM.  A tile is a rectangle of output pixels of one image (16 x 8 at stride 1, 8 x 8 at stride 2: up to 128
// rows of the projection's GEMM); per block of 32 (expanded) channels
//   * the fp32 input patch of the depthwise filter ((TH-1)*stride+3 rows x (TW-1)*stride+3 columns x 32 channels)
//     arrives in shared memory: loaded by TMA (coordinates outside the image read as zero: that is the padding),
//     or, with the expand layer fused in (EXPAND), computed on the tensor cores from the block's input patch
//     (<= 32 channels, bf16 pairs, loaded once per tile): the MMA thread multiplies the patch (two or three
//     128-pixel strips) by the block's 32 weight rows into a TMEM accumulator of the depthwise group, two blocks
//     ahead of the group; the group's warps read it back (tcgen05.ld), add the bias, apply the activation, write
//     zero where the pixel lies outside the image, and store the fp32 patch,
//   * four CUDA-core warps (two such groups take alternate blocks) compute the depthwise results from it with
//     the arithmetic of the stand-alone kernel (bias, nine fmaf in filter order, activation), split each value
//     into its bf16 pair (hi = bf16(x), mid = bf16(x - hi)) and write both planes straight into the K-major,
//     64-byte-swizzled operand tile that tcgen05.mma reads,
//   * one thread issues the projection's MMAs (mid*hi + hi*mid + hi*hi, as tc_gemm_kernel does) against
//     that channel block's weights, which TMA streams through a small ring,
// and the usual epilogue warps drain the accumulator (bias, residual, activation, TMA stores).
// Without EXPAND the operands, their order and the accumulation are those of the two separate kernels, so the
// results are the same bits.  With EXPAND the expand layer's products are the same too; only its bias is added
// after the accumulation instead of by the epilogue of a separate kernel, which is the same fp32 addition.
//
// Warps (448 threads): 0 TMA producer, 1 MMA issuer, 2-5 epilogue, 6-13 depthwise.  Every wait is
// bounded and ends in the status word.
#pragma once

#include "tc_gemm.cuh"

namespace nb {

constexpr int kDwpThreads = 448;
constexpr int kDwpChannels = 32;  // channels per block: 64-byte bf16 rows
constexpr int kDwpTileW = 8;
constexpr int kDwpMaxStages = 4;
constexpr int kDwpMaxPatches = 4;

// geometry of a tile by stride
__host__ __device__ constexpr int dwp_tile_h(int stride) { return stride == 1 ? 16 : 8; }
__host__ __device__ constexpr int dwp_patch_h(int stride) { return (dwp_tile_h(stride) - 1) * stride + 3; }
__host__ __device__ constexpr int dwp_patch_w(int stride) { return (kDwpTileW - 1) * stride + 3; }
__host__ __device__ constexpr int dwp_patch_pixels(int stride) { return dwp_patch_h(stride) * dwp_patch_w(stride); }
__host__ __device__ constexpr int dwp_patch_bytes(int stride) {
  return (dwp_patch_pixels(stride) * kDwpChannels * 4 + 1023) / 1024 * 1024;
}
// one bf16 plane of the operand tile: the rows a tile has, 64 bytes each (the MMA reads 128 rows: past a
// stride-2 tile's 64 it reads what follows in shared memory, into accumulator rows that are never stored)
__host__ __device__ constexpr int dwp_a_plane_bytes(int stride) { return dwp_tile_h(stride) * kDwpTileW * 64; }

struct TcDwProjParams {
  int images, H, W, C;  // depthwise OUTPUT extent, channels of the depthwise layer
  int Hin, Win;         // depthwise input extent (= H, W at stride 1)
  int N;                // projection output channels
  int tiles_y, tiles_x, tiles_n, block_n;
  int c_blocks;         // blocks of 32 channels (the last one may be partly past C: zero-filled)
  int pad_t, pad_l;
  int stages;           // weight ring depth
  int patch_bufs;       // input patch ring depth, 2 or 4 (even: a slot then always serves the same depthwise group)
  int b_bytes;          // one plane of a weight stage, rounded to 1 KB
  int out_bufs;
  const float* dw_weights;  // [9][C], tap-major
  const float* dw_bias;     // [C] or null
  int dw_act;
  float dw_act_a, dw_act_b;
  // expand layer (EXPAND): x is [image][Hin][Win][Cin] as bf16 hi / mid planes, weights packed [C][32] bf16 hi / mid
  int Cin;
  int x_row_bytes;          // operand rows of the input patch and of the expand weights: 64 bytes (32 channels), or 32
                            // (16 channels) when the block's input has no more: two patch buffers then fit where one did
  int x_plane_bytes;        // one bf16 plane of an input patch buffer, rounded to 1 KB
  int x_bufs;               // input patch buffers: 2, or 1 when two do not fit
  int ex_ksteps;            // K steps of 16 input channels the expand MMAs run: ceil(Cin / 16)
  const float* ex_bias;     // [C] or null
  int ex_act;
  float ex_act_a, ex_act_b;
  const float* bias;        // projection bias [N] or null
  int res_mode, out_mode, act;
  float act_a, act_b;
  int* status;
};

// (KIND: the projection's arithmetic; bf16 pairs are the only form built)
template <int KIND, int STRIDE, bool EXPAND>
__global__ void __launch_bounds__(kDwpThreads, 1)
tc_dw_project_kernel(const __grid_constant__ TcDwProjParams p, const __grid_constant__ CUtensorMap map_x,
                     const __grid_constant__ CUtensorMap map_x1, const __grid_constant__ CUtensorMap map_e0,
                     const __grid_constant__ CUtensorMap map_e1,
                     const __grid_constant__ CUtensorMap map_b0, const __grid_constant__ CUtensorMap map_b1,
                     const __grid_constant__ CUtensorMap map_o0, const __grid_constant__ CUtensorMap map_o1,
                     const __grid_constant__ CUtensorMap map_r0, const __grid_constant__ CUtensorMap map_r1) {
  using namespace ptx;
  constexpr int TH = dwp_tile_h(STRIDE), TW = kDwpTileW;
  constexpr int PH = dwp_patch_h(STRIDE), PW = dwp_patch_w(STRIDE), NPX = PH * PW;
  constexpr uint32_t kPatchBytes = dwp_patch_bytes(STRIDE);
  constexpr uint32_t kAPlaneBytes = dwp_a_plane_bytes(STRIDE);
  constexpr int MT = (NPX + 127) / 128;        // EXPAND: 128-pixel strips of the patch = MMAs of M = 128
  constexpr uint32_t kExWeightBytes = 2048u;   // EXPAND: one plane of a block's expand weights, 32 rows x 64 bytes
  grid_dependency_trigger();  // the next kernel of the stream may begin its preamble

  extern __shared__ uint8_t dwp_smem_raw[];
  __shared__ __align__(8) uint64_t patch_full[kDwpMaxPatches], patch_empty[kDwpMaxPatches];
  __shared__ __align__(8) uint64_t x_full[2], x_empty[2];
  __shared__ __align__(8) uint64_t e_full[2], e_empty[2];
  __shared__ __align__(8) uint64_t a_full[2], a_empty[2];
  __shared__ __align__(8) uint64_t b_full[kDwpMaxStages], b_empty[kDwpMaxStages];
  __shared__ __align__(8) uint64_t tfull_bar[2], tempty_bar[2];
  __shared__ __align__(8) uint64_t res_bar;
  __shared__ __align__(16) float tile_bias[256];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(dwp_smem_raw) + 1023u) & ~1023u;
  const int P = EXPAND ? 2 : p.patch_bufs;  // EXPAND: one patch per depthwise group, filled by the group itself
  const uint32_t x_base = smem_base;                                      // EXPAND: input patches, hi then mid plane
  const uint32_t x_plane = static_cast<uint32_t>(p.x_plane_bytes);
  const int XB = EXPAND ? p.x_bufs : 1;
  const uint32_t patch_base = x_base + (EXPAND ? static_cast<uint32_t>(XB) * 2u * x_plane : 0u);  // ring of fp32 patches
  const uint32_t a_base = patch_base + static_cast<uint32_t>(P) * kPatchBytes;  // two operand tiles (hi, mid planes)
  const uint32_t a_stage_bytes = 2u * kAPlaneBytes;
  const uint32_t b_base = a_base + 2u * a_stage_bytes;                    // weight ring (hi, mid planes)
  const uint32_t b_bytes = static_cast<uint32_t>(p.b_bytes);
  const uint32_t b_stage_bytes = 2u * b_bytes + (EXPAND ? 2u * kExWeightBytes : 0u);  // (+ the block's expand weights)
  const int S = p.stages;
  const uint32_t res_stage = b_base + static_cast<uint32_t>(S) * b_stage_bytes;
  const uint32_t out_stage = res_stage + (p.res_mode != RES_NONE ? 16384u : 0u);
  const bool wide_out = p.out_mode == OUT_BF16X2 || p.res_mode == RES_BF16X2;
  // the depthwise filter and bias of every channel, [10][c_blocks * 32] fp32 (taps 0..8, then the bias; zero past C)
  const uint32_t table = out_stage + static_cast<uint32_t>(p.out_bufs) * (wide_out ? 16384u : 8192u);
  const int c_pad = p.c_blocks * kDwpChannels;
  // EXPAND: the expand layer's bias [c_pad] (zero past C)
  const uint32_t ex_table = table + static_cast<uint32_t>(10 * c_pad) * 4u;
  // TMEM columns: the projection's two accumulators, then one expand accumulator (MT strips x 32 columns) per group
  const uint32_t acc_stride = p.block_n > 128 ? 256u : 128u;
  const uint32_t e_col0 = 2u * acc_stride;
  const int tiles_per_image = p.tiles_y * p.tiles_x;
  const int total_tiles = p.images * tiles_per_image * p.tiles_n;
  volatile int* abort_ptr = &abort_flag;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < kDwpMaxPatches; ++i) {
      mbar_init(smem_u32(&patch_full[i]), 1);
      mbar_init(smem_u32(&patch_empty[i]), 4);  // one arrival per warp of the depthwise group that read it
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&x_full[i]), 1);
      mbar_init(smem_u32(&x_empty[i]), 1);  // the commit after the tile's last expand MMA
      mbar_init(smem_u32(&e_full[i]), 1);
      mbar_init(smem_u32(&e_empty[i]), 4);  // the four warps of the group that read the accumulator
      mbar_init(smem_u32(&a_full[i]), 4);
      mbar_init(smem_u32(&a_empty[i]), 1);
      mbar_init(smem_u32(&tfull_bar[i]), 1);
      mbar_init(smem_u32(&tempty_bar[i]), 4);
    }
    for (int i = 0; i < S; ++i) {
      mbar_init(smem_u32(&b_full[i]), 1);
      mbar_init(smem_u32(&b_empty[i]), 1);
    }
    mbar_init(smem_u32(&res_bar), 1);
    fence_mbar_init();
    prefetch_tensormap(&map_x);
    prefetch_tensormap(&map_b0);
    prefetch_tensormap(&map_b1);
    prefetch_tensormap(&map_o0);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), kTcTmemCols);
    tmem_relinquish();
  }
  // (constants of the layers, not results of the kernel before: they may be read ahead of the dependency wait)
  for (int i = static_cast<int>(threadIdx.x); i < 10 * c_pad; i += kDwpThreads) {
    const int k = i / c_pad, c = i - k * c_pad;
    float v = 0.0f;
    if (c < p.C) v = k < 9 ? __ldg(p.dw_weights + static_cast<size_t>(k) * p.C + c) : (p.dw_bias != nullptr ? __ldg(p.dw_bias + c) : 0.0f);
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(table + static_cast<uint32_t>(i) * 4u), "f"(v) : "memory");
  }
  if (EXPAND) {
    for (int c = static_cast<int>(threadIdx.x); c < c_pad; c += kDwpThreads) {
      const float v = (c < p.C && p.ex_bias != nullptr) ? __ldg(p.ex_bias + c) : 0.0f;
      asm volatile("st.shared.f32 [%0], %1;" ::"r"(ex_table + static_cast<uint32_t>(c) * 4u), "f"(v) : "memory");
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  grid_dependency_wait();

  // channel blocks of one pixel tile are neighbours, so CTAs working side by side share the patch in L2
  auto decode = [&](int tile, int* img, int* oy0, int* ox0, int* n0) {
    const int n_blk = tile % p.tiles_n;
    int t = tile / p.tiles_n;
    const int tx = t % p.tiles_x;
    t /= p.tiles_x;
    const int ty = t % p.tiles_y;
    *img = t / p.tiles_y;
    *oy0 = ty * TH;
    *ox0 = tx * TW;
    *n0 = n_blk * p.block_n;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    // lane 0: the fp32 patch of a channel block (EXPAND: both planes of the tile's input patch); lanes 1, 2: the
    // two planes of that block's projection weights; lanes 3, 4 (EXPAND): the two planes of its expand weights
    const uint32_t patch_tx = static_cast<uint32_t>(NPX * kDwpChannels * 4);
    const uint32_t x_tx = 2u * static_cast<uint32_t>(NPX) * static_cast<uint32_t>(p.x_row_bytes);
    const uint32_t b_tx = 2u * static_cast<uint32_t>(p.block_n) * 64u + (EXPAND ? 2u * 32u * static_cast<uint32_t>(p.x_row_bytes) : 0u);
    int s = 0, pb = 0;
    uint32_t ph = 0, p_ph = 0;
    long long patches = 0, weights = 0, tiles_done = 0, x_issued = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tiles_done) {
      int img, oy0, ox0, n0;
      decode(tile, &img, &oy0, &ox0, &n0);
      if (EXPAND) {
        // With two buffers the patch of the NEXT tile is requested here (the first tile's before the loop): its
        // buffer was released by the tile before this one, so the wait cannot hold up this tile's weight copies.
        // With one buffer the patch of THIS tile is requested, once the previous tile's expand MMAs have read theirs.
        const long long first = XB == 2 ? (tiles_done == 0 ? 0 : tiles_done + 1) : tiles_done;
        const long long last = XB == 2 ? tiles_done + 1 : tiles_done;
        for (long long tl = first; tl <= last && ok; ++tl) {
          const int t2 = static_cast<int>(blockIdx.x) + static_cast<int>(tl) * static_cast<int>(gridDim.x);
          if (t2 >= total_tiles) break;
          int img2, oy2, ox2, n2;
          decode(t2, &img2, &oy2, &ox2, &n2);
          const int xb = static_cast<int>(tl % XB);
          const uint32_t x_ph = static_cast<uint32_t>((tl / XB) & 1);
          int w = 1;
          if (lane == 0) {
            w = mbar_wait_bounded(smem_u32(&x_empty[xb]), x_ph ^ 1u, abort_ptr, kTcWaitLimitNs) ? 1 : 0;
            if (w) {
              const uint32_t dst = x_base + static_cast<uint32_t>(xb) * 2u * x_plane;
              mbar_arrive_expect_tx(smem_u32(&x_full[xb]), x_tx);
              tma_load_4d(dst, &map_x, smem_u32(&x_full[xb]), 0, ox2 * STRIDE - p.pad_l, oy2 * STRIDE - p.pad_t, img2);
              tma_load_4d(dst + x_plane, &map_x1, smem_u32(&x_full[xb]), 0, ox2 * STRIDE - p.pad_l, oy2 * STRIDE - p.pad_t, img2);
            }
          }
          w = __shfl_sync(0xffffffffu, w, 0);
          if (!w) ok = false;
          else ++x_issued;
        }
        if (!ok) break;
      }
      for (int cb = 0; cb < p.c_blocks && ok; ++cb) {
        int w = 1;
        if (!EXPAND) {
          if (lane == 0) {
            w = mbar_wait_bounded(smem_u32(&patch_empty[pb]), p_ph ^ 1u, abort_ptr, kTcWaitLimitNs) ? 1 : 0;
            if (w) {
              mbar_arrive_expect_tx(smem_u32(&patch_full[pb]), patch_tx);
              tma_load_4d(patch_base + static_cast<uint32_t>(pb) * kPatchBytes, &map_x, smem_u32(&patch_full[pb]),
                          cb * kDwpChannels, ox0 * STRIDE - p.pad_l, oy0 * STRIDE - p.pad_t, img);
            }
          }
          w = __shfl_sync(0xffffffffu, w, 0);
          if (!w) {
            ok = false;
            break;
          }
          ++patches;
          if (++pb == P) {
            pb = 0;
            p_ph ^= 1u;
          }
        }
        if (lane == 0) {
          w = mbar_wait_bounded(smem_u32(&b_empty[s]), ph ^ 1u, abort_ptr, kTcWaitLimitNs) ? 1 : 0;
          if (w) mbar_arrive_expect_tx(smem_u32(&b_full[s]), b_tx);
        }
        w = __shfl_sync(0xffffffffu, w, 0);
        if (!w) {
          ok = false;
          break;
        }
        const uint32_t stage = b_base + static_cast<uint32_t>(s) * b_stage_bytes;
        if (lane == 1 || lane == 2)
          tma_load_2d(stage + (lane - 1) * b_bytes, lane == 1 ? &map_b0 : &map_b1, smem_u32(&b_full[s]), cb * kDwpChannels, n0);
        if (EXPAND && (lane == 3 || lane == 4))
          tma_load_2d(stage + 2u * b_bytes + (lane - 3) * kExWeightBytes, lane == 3 ? &map_e0 : &map_e1, smem_u32(&b_full[s]), 0,
                      cb * kDwpChannels);
        ++weights;
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
        // copies issued by this warp may still be landing: wait (bounded) for the last ones
        int zero = 0;
        for (long long i = weights > S ? weights - S : 0; i < weights; ++i)
          mbar_wait_bounded(smem_u32(&b_full[i % S]), static_cast<uint32_t>((i / S) & 1), &zero, 200000000ull);
        for (long long i = patches > P ? patches - P : 0; i < patches; ++i)
          mbar_wait_bounded(smem_u32(&patch_full[i % P]), static_cast<uint32_t>((i / P) & 1), &zero, 200000000ull);
        for (long long i = x_issued > XB ? x_issued - XB : 0; i < x_issued; ++i)
          mbar_wait_bounded(smem_u32(&x_full[i % XB]), static_cast<uint32_t>((i / XB) & 1), &zero, 200000000ull);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc(1u, 1u, kTcBlockM, static_cast<uint32_t>(p.block_n));
      const uint32_t idesc_ex = instr_desc(1u, 1u, kTcBlockM, 32u);
      const uint64_t fixed = smem_desc_kmajor(0u, 64u);  // 64-byte rows, 64-byte swizzle
      const uint64_t fixed_x = smem_desc_kmajor(0u, EXPAND ? static_cast<uint32_t>(p.x_row_bytes) : 64u);
      const uint64_t a_plane_units = kAPlaneBytes >> 4;
      const uint64_t b_units = b_bytes >> 4;
      const int c_blocks = p.c_blocks;
      const long long my_tiles = blockIdx.x < static_cast<unsigned>(total_tiles) ? (total_tiles - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;
      const long long total_items = my_tiles * c_blocks;
      bool ok = true;
      // EXPAND: the expand layer of item `it` (tile it / c_blocks, channel block it % c_blocks) into the TMEM
      // accumulator of group it & 1: the patch strips (A, 128 pixels x 32 channels each) times the block's 32 weight
      // rows (B), three products per K step.  Issued two items ahead of the projection of the same group.
      auto issue_expand = [&](long long it) -> bool {
        const long long tl = it / c_blocks;
        const int cb = static_cast<int>(it - tl * c_blocks);
        const int g = static_cast<int>(it & 1);
        const int xb = static_cast<int>(tl % XB);
        const int st = static_cast<int>(it % S);
        if (cb == 0 && !mbar_wait_bounded(smem_u32(&x_full[xb]), static_cast<uint32_t>((tl / XB) & 1), abort_ptr, kTcWaitLimitNs)) return false;
        if (!mbar_wait_bounded(smem_u32(&b_full[st]), static_cast<uint32_t>((it / S) & 1), abort_ptr, kTcWaitLimitNs)) return false;
        if (!mbar_wait_bounded(smem_u32(&e_empty[g]), static_cast<uint32_t>(((it >> 1) & 1) ^ 1), abort_ptr, kTcWaitLimitNs)) return false;
        tc_fence_after_sync();
        const uint32_t xa = x_base + static_cast<uint32_t>(xb) * 2u * x_plane;
        const uint32_t wb = b_base + static_cast<uint32_t>(st) * b_stage_bytes + 2u * b_bytes;
        const uint64_t w0 = fixed_x + ((wb & 0x3ffffu) >> 4);
        const uint64_t w_units = kExWeightBytes >> 4;
        const uint64_t x_units = x_plane >> 4;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint32_t d = tmem_base + e_col0 + static_cast<uint32_t>(g * MT + mt) * 32u;
          const uint64_t a0 = fixed_x + (((xa + static_cast<uint32_t>(mt) * 128u * static_cast<uint32_t>(p.x_row_bytes)) & 0x3ffffu) >> 4);
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            if (k >= p.ex_ksteps) break;  // (16 input channels: the second half of the 64-byte rows is zero padding)
            const uint64_t ka = a0 + 2u * k, kb = w0 + 2u * k;
            mma_f16(d, ka + x_units, kb, idesc_ex, k ? 1u : 0u);  // mid * hi
            mma_f16(d, ka, kb + w_units, idesc_ex, 1u);            // hi * mid
            mma_f16(d, ka, kb, idesc_ex, 1u);                      // hi * hi
          }
        }
        tc_commit(smem_u32(&e_full[g]));
        if (cb == c_blocks - 1) tc_commit(smem_u32(&x_empty[xb]));  // the tile's input patch has been read
        return true;
      };
      if (EXPAND) {
        for (long long it = 0; it < 2 && it < total_items && ok; ++it) ok = issue_expand(it);
      }
      int s = 0, as = 0, acc = 0;
      uint32_t ph = 0, a_ph = 0, acc_ph = 0;
      long long item = 0;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait_bounded(smem_u32(&tempty_bar[acc]), acc_ph ^ 1u, abort_ptr, kTcWaitLimitNs)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * acc_stride;
        uint32_t accumulate = 0u;
        for (int cb = 0; cb < c_blocks; ++cb, ++item) {
          if (EXPAND && item + 2 < total_items && !issue_expand(item + 2)) {
            ok = false;
            break;
          }
          // (EXPAND: the stage's copies were awaited when its expand MMAs were issued)
          if (!mbar_wait_bounded(smem_u32(&a_full[as]), a_ph, abort_ptr, kTcWaitLimitNs) ||
              (!EXPAND && !mbar_wait_bounded(smem_u32(&b_full[s]), ph, abort_ptr, kTcWaitLimitNs))) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint64_t a0 = fixed + (((a_base + static_cast<uint32_t>(as) * a_stage_bytes) & 0x3ffffu) >> 4);
          const uint64_t b0 = fixed + (((b_base + static_cast<uint32_t>(s) * b_stage_bytes) & 0x3ffffu) >> 4);
#pragma unroll
          for (int k = 0; k < 2; ++k) {  // two K steps of 16 channels (32 bytes = 2 units) per block
            const uint64_t ka = a0 + 2u * k;
            const uint64_t kb = b0 + 2u * k;
            mma_f16(d_tmem, ka + a_plane_units, kb, idesc, accumulate);  // mid * hi
            mma_f16(d_tmem, ka, kb + b_units, idesc, 1u);                // hi * mid
            mma_f16(d_tmem, ka, kb, idesc, 1u);                          // hi * hi
            accumulate = 1u;
          }
          tc_commit(smem_u32(&a_empty[as]));
          tc_commit(smem_u32(&b_empty[s]));
          as ^= 1;
          if (as == 0) a_ph ^= 1u;
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit(smem_u32(&tfull_bar[acc]));
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1u;
      }
      if (!ok) {
        if (atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_MMA);
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (warps 2-5)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // accumulator row = pixel (row / 8, row % 8) of the tile
    TcStageCfg cfg{};
    cfg.bar_base = 1;
    cfg.res_stage = res_stage;
    cfg.out_stage = out_stage;
    cfg.res_bar = smem_u32(&res_bar);
    cfg.out_bufs = p.out_bufs;
    cfg.out_mode = p.out_mode;
    cfg.res_mode = p.res_mode;
    cfg.act = p.act;
    cfg.act_a = p.act_a;
    cfg.act_b = p.act_b;
    cfg.N = p.N;
    cfg.block_n = p.block_n;
    cfg.wide = wide_out ? 1 : 0;
    int acc = 0, out_slot = 0;
    uint32_t acc_ph = 0, res_ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      int img, oy0, ox0, n0;
      decode(tile, &img, &oy0, &ox0, &n0);
      ok = __all_sync(0xffffffffu,
                      mbar_wait_bounded(smem_u32(&tfull_bar[acc]), acc_ph, abort_ptr, kTcWaitLimitNs) ? 1 : 0) != 0;
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc) * acc_stride;
      for (int t = static_cast<int>(threadIdx.x) - 64; t < p.block_n; t += 128) {
        const int n = n0 + t;
        tile_bias[t] = (p.bias != nullptr && n < p.N) ? __ldg(p.bias + n) : 0.0f;
      }
      // (the boxes of the output and residual maps are TH x TW pixels: of a stride-2 tile only the first 64
      // staging rows leave)
      struct {
        const CUtensorMap *o0, *o1, *r0, *r1;
        int x, y, img;
        __device__ __forceinline__ void load_res(int plane, uint32_t dst, uint32_t bar, int col) const {
          ptx::tma_load_4d(dst, plane ? r1 : r0, bar, col, x, y, img);
        }
        __device__ __forceinline__ void store_out(int plane, uint32_t src, int col) const {
          ptx::tma_store_4d(plane ? o1 : o0, src, col, x, y, img);
        }
        __device__ __forceinline__ void store_side(int, uint32_t, int) const {}
      } io{&map_o0, &map_o1, &map_r0, &map_r1, ox0, oy0, img};
      ok = tc_staged_epilogue<KIND>(cfg, io, t_row, n0, row, threadIdx.x == 64, tile_bias, tile_bias, res_ph,
                                           out_slot, abort_ptr);
      if (!ok) break;
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
      acc ^= 1;
      if (acc == 0) acc_ph ^= 1u;
    }
    if (!ok && lane == 0) {
      if (atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_EPILOGUE);
    }
    if (threadIdx.x == 64) tma_store_wait_all();
  } else {
    // ------------------------------------------------------------ depthwise (warps 6-13, 256 threads)
    // Two groups of four warps take alternate channel blocks (group g: blocks g, g+2, ... of the CTA's sequence,
    // so group g always fills operand tile g): while one group waits for its patch or for its operand tile to be
    // free, the other computes.  In a group a thread owns four channels, one column of the tile and half of its
    // rows below each other: the input rows it needs are read once for all of them.
    constexpr int R = TH / 2;                   // result rows per thread
    constexpr int IR = (R - 1) * STRIDE + 3;    // input rows they need
    const int t = static_cast<int>(threadIdx.x) - 192;
    const int group = t >> 7;
    const int tg = t & 127;
    const int quad = t & 7;                 // channels 4*quad .. 4*quad+3 of the block
    const int col = (t >> 3) & 7;           // column of the tile
    const int row0 = ((t >> 6) & 1) * R;    // first of the thread's rows
    bool ok = true;
    // none / ReLU / clip as one clamp: fminf(fmaxf(y, lo), hi) returns y itself between the bounds
    const float act_lo = p.dw_act == ACT_RELU ? 0.0f : (p.dw_act == ACT_CLIP ? p.dw_act_a : -INFINITY);
    const float act_hi = p.dw_act == ACT_CLIP ? p.dw_act_b : INFINITY;
    const float ex_lo = p.ex_act == ACT_RELU ? 0.0f : (p.ex_act == ACT_CLIP ? p.ex_act_a : -INFINITY);
    const float ex_hi = p.ex_act == ACT_CLIP ? p.ex_act_b : INFINITY;
    const uint32_t a_tile = a_base + static_cast<uint32_t>(group) * a_stage_bytes;
    long long item = 0;   // position in the CTA's sequence of (tile, channel block)
    long long tiles_done = 0;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tiles_done) {
      int img, oy0, ox0, n0;
      decode(tile, &img, &oy0, &ox0, &n0);
      for (int cb = 0; cb < p.c_blocks && ok; ++cb, ++item) {
        if ((item & 1) != group) continue;
        const int pb = EXPAND ? group : static_cast<int>(item % P);
        const uint32_t a_ph = static_cast<uint32_t>((item >> 1) & 1);
        const uint32_t patch = patch_base + static_cast<uint32_t>(pb) * kPatchBytes;
        if (EXPAND) {
          // ---- the expand layer's accumulator of this block (MT strips of 128 patch pixels x 32 channels in
          // TMEM) -> bias, activation, zero outside the image -> the group's fp32 patch.  A warp reads the 32
          // lanes of its TMEM quarter: one pixel per thread and strip, all 32 channels.  The patch is written with
          // its 16-byte chunks permuted by the pixel index (chunk ^ (pixel & 7)), which spreads the 32 rows a
          // warp stores at a time over the banks.
          ok = __all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&e_full[group]), static_cast<uint32_t>((item >> 1) & 1),
                                                         abort_ptr, kTcWaitLimitNs) ? 1 : 0) != 0;
          if (!ok) break;
          tc_fence_after_sync();
          const int q = warp & 3;  // the TMEM lanes this warp may read: 32 q .. 32 q + 31
          const uint32_t bias_at = ex_table + static_cast<uint32_t>(cb * kDwpChannels) * 4u;
#pragma unroll 1  // (one copy of the strip's code: the kernel's roles already compete for the instruction cache)
          for (int mt = 0; mt < MT; ++mt) {
            const int px = mt * 128 + q * 32 + lane;
            if (mt * 128 + q * 32 >= NPX) break;  // (the whole warp is past the patch)
            const int pr = px / PW, pc = px - pr * PW;
            const int iy = oy0 * STRIDE - p.pad_t + pr, ix = ox0 * STRIDE - p.pad_l + pc;
            // outside the image the depthwise filter sees its zero padding, not act(bias)
            const bool inside = px < NPX && iy >= 0 && iy < p.Hin && ix >= 0 && ix < p.Win;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + e_col0 + static_cast<uint32_t>(group * MT + mt) * 32u;
            const uint32_t rowat = patch + static_cast<uint32_t>(px) * 128u;
            const uint32_t sw = static_cast<uint32_t>(px & 7);
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {
              uint32_t v[16];
              tmem_ld16(taddr + 16u * h, v);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float4 b4;
                asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(b4.x), "=f"(b4.y), "=f"(b4.z), "=f"(b4.w) : "r"(bias_at + static_cast<uint32_t>(16 * h + 4 * j) * 4u));
                float4 y;
                y.x = inside ? fminf(fmaxf(__fadd_rn(__uint_as_float(v[4 * j + 0]), b4.x), ex_lo), ex_hi) : 0.0f;
                y.y = inside ? fminf(fmaxf(__fadd_rn(__uint_as_float(v[4 * j + 1]), b4.y), ex_lo), ex_hi) : 0.0f;
                y.z = inside ? fminf(fmaxf(__fadd_rn(__uint_as_float(v[4 * j + 2]), b4.z), ex_lo), ex_hi) : 0.0f;
                y.w = inside ? fminf(fmaxf(__fadd_rn(__uint_as_float(v[4 * j + 3]), b4.w), ex_lo), ex_hi) : 0.0f;
                if (px < NPX)
                  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(rowat + ((static_cast<uint32_t>(4 * h + j) ^ sw) << 4)),
                               "f"(y.x), "f"(y.y), "f"(y.z), "f"(y.w) : "memory");
              }
            }
          }
          // the accumulator has been read: the expand MMAs of the group's next block may overwrite it
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&e_empty[group]));
          named_barrier_sync(3 + group, 128);  // the group's patch is complete
        }
        const uint32_t tc = table + static_cast<uint32_t>(cb * kDwpChannels + quad * 4) * 4u;  // the thread's channels
        float4 tap[9], bias;
#pragma unroll
        for (int k = 0; k < 9; ++k)
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(tap[k].x), "=f"(tap[k].y), "=f"(tap[k].z), "=f"(tap[k].w) : "r"(tc + static_cast<uint32_t>(k * c_pad) * 4u));
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(bias.x), "=f"(bias.y), "=f"(bias.z), "=f"(bias.w) : "r"(tc + static_cast<uint32_t>(9 * c_pad) * 4u));
        if (!EXPAND) {
          // the vote keeps the warp together for the barrier arrivals below
          ok = __all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&patch_full[pb]), static_cast<uint32_t>((item / P) & 1),
                                                         abort_ptr, kTcWaitLimitNs) ? 1 : 0) != 0;
          if (!ok) break;
        }
        float4 acc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = bias;
        // input rows row0*STRIDE .. +IR-1 of the patch; input row i feeds result row r with filter row kh = i - r*STRIDE
#pragma unroll
        for (int i = 0; i < IR; ++i) {
          float4 x[3];
#pragma unroll
          for (int kw = 0; kw < 3; ++kw) {
            const int px = (row0 * STRIDE + i) * PW + col * STRIDE + kw;
            const uint32_t chunk = EXPAND ? static_cast<uint32_t>(quad ^ (px & 7)) : static_cast<uint32_t>(quad);
            const uint32_t at = patch + static_cast<uint32_t>(px) * 128u + (chunk << 4);
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x[kw].x), "=f"(x[kw].y), "=f"(x[kw].z), "=f"(x[kw].w) : "r"(at));
          }
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const int kh = i - r * STRIDE;
            if (kh < 0 || kh > 2) continue;
#pragma unroll
            for (int kw = 0; kw < 3; ++kw) {
              const float4 k = tap[kh * 3 + kw];
              acc[r].x = fmaf(x[kw].x, k.x, acc[r].x);
              acc[r].y = fmaf(x[kw].y, k.y, acc[r].y);
              acc[r].z = fmaf(x[kw].z, k.z, acc[r].z);
              acc[r].w = fmaf(x[kw].w, k.w, acc[r].w);
            }
          }
        }
        // the patch has been read: it may be refilled (by the producer, or by this group's next expand step)
        if (EXPAND) {
          named_barrier_sync(5 + group, 128);
        } else {
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&patch_empty[pb]));
        }
        // the group's operand tile, filled two blocks ago, must have been consumed by its MMAs
        ok = __all_sync(0xffffffffu,
                        mbar_wait_bounded(smem_u32(&a_empty[group]), a_ph ^ 1u, abort_ptr, kTcWaitLimitNs) ? 1 : 0) != 0;
        if (!ok) break;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          float4 y;
          y.x = fminf(fmaxf(acc[r].x, act_lo), act_hi);
          y.y = fminf(fmaxf(acc[r].y, act_lo), act_hi);
          y.z = fminf(fmaxf(acc[r].z, act_lo), act_hi);
          y.w = fminf(fmaxf(acc[r].w, act_lo), act_hi);
          uint32_t hi0, mid0, hi1, mid1;
          split_bf16x2(y.x, y.y, hi0, mid0);
          split_bf16x2(y.z, y.w, hi1, mid1);
          // operand row = pixel (row, col) of the tile; 64-byte rows with the 64-byte swizzle: the
          // 16-byte chunk j of row m lives at m*64 + ((j ^ ((m >> 1) & 3)) * 16)
          const int m = (row0 + r) * TW + col;
          const uint32_t at = a_tile + stage_chunk_offset(m, quad >> 1) + static_cast<uint32_t>((quad & 1) * 8);
          asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(at), "r"(hi0), "r"(hi1) : "memory");
          asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(at + kAPlaneBytes), "r"(mid0), "r"(mid1) : "memory");
        }
        fence_proxy_async_smem();  // the tensor core reads what these stores wrote
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&a_full[group]));
      }
    }
    if (!ok && lane == 0) {
      if (atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_EPILOGUE);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kTcTmemCols);
}

}  // namespace nb
