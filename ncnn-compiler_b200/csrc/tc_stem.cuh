// Stem convolution (few input channels; fp32 accuracy mode or int8) with the input rows resident in
// shared memory: one tile is one output row of one image.
//
// The graph input is stored channel-padded to 4 and width-padded, as bf16 pairs: 8 bytes per pixel
// and plane.  With a horizontal stride of 2 the filter window of output pixel x starts 16 bytes
// after the window of pixel x-1, and 16 bytes is exactly the row pitch inside a core matrix of the
// un-swizzled K-major operand layout.  So the A operand of tcgen05.mma can be read straight out of
// a contiguous input row: a descriptor with a leading-dimension offset of 16 bytes (next 16-byte K
// chunk = next 16 bytes) and a stride offset of 128 bytes (next 8 rows) makes row r of the operand
// the 64-byte window at `row + 16 r`: the windows overlap in shared memory instead of being
// copied out 4x by an im2col load.  One TMA copy per plane brings the KH input rows of a tile
// (13 KB for the 7x7 ResNet stem, against 112 KB of window copies); the weights of all KH filter
// rows stay resident.  Replaces the stem case of ConvertConvolution (lib/Conversion/NCNNToTosa/
// NCNNToTosa.cpp:1403-1528); results are bit-identical to tc_gemm_kernel's (same products, same
// K order).  The int8 form stores 8 channels per pixel (8 bytes), so the same 16-byte pitch holds: 64-byte
// windows of 8 pixels, one plane, kind::i8 with K = 32 per instruction.
#pragma once

#include "tc_gemm.cuh"

namespace nb {

constexpr int kStemThreads = 352;  // warp 0 producer, 1 MMA, 2-5 epilogue group 0, 6 idle, 7-10 group 1
constexpr int kStemMaxStages = 8;

struct TcStemParams {
  int tiles;          // images * OH: one output row each
  int OH, OW, KH;
  int stride_h, pad_t;
  int N;              // output channels = MMA N (multiple of 16, at most 128)
  int M;              // images * OH * OW output pixels
  int row_bytes;      // one padded input row of one plane (multiple of 128)
  int a_plane_bytes;  // KH rows plus what the last window rows overrun, rounded to 1 KB
  int b_slot;         // one weight tile of one plane: N rows x 64 bytes, rounded to 1 KB
  int stages;         // A ring depth
  int accs;           // accumulators in TMEM: 4 of 64 columns (N <= 64) or 2 of 128
  int issuers;        // MMA-issuing warps: 2 (warps 1 and 6 take alternate tiles) with four accumulators, else 1
  const float* bias;
  const float* scale;  // int8: dequantisation factor per output channel
  float out_scale;     // int8 results: requantisation scale
  int out_mode, act;
  float act_a, act_b;
  int wide, out_bufs, staging_bytes, epi_groups;
  int* status;
};

// un-swizzled K-major descriptor: K chunks `lbo` bytes apart, 8-row groups `sbo` bytes apart
__device__ __forceinline__ uint64_t smem_desc_plain(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3fffu) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3fffu) << 32;
  d |= 1ull << 46;
  return d;
}

// KIND is GEMM_BF16X3 (two planes: hi, mid) or GEMM_I8 (one plane)
template <int KIND>
__global__ void __launch_bounds__(kStemThreads, 1)
tc_stem_kernel(const __grid_constant__ TcStemParams p, const __grid_constant__ CUtensorMap map_a0,
               const __grid_constant__ CUtensorMap map_a1, const __grid_constant__ CUtensorMap map_b0,
               const __grid_constant__ CUtensorMap map_b1, const __grid_constant__ CUtensorMap map_o0,
               const __grid_constant__ CUtensorMap map_o1) {
  using namespace ptx;
  grid_dependency_trigger();  // the next kernel of the stream may begin its preamble
  constexpr int PLANES = tc_planes(KIND);
  extern __shared__ uint8_t stem_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStemMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kStemMaxStages];
  __shared__ __align__(8) uint64_t tfull_bar[4];
  __shared__ __align__(8) uint64_t tempty_bar[4];
  __shared__ __align__(8) uint64_t weights_bar;
  __shared__ __align__(8) uint64_t unused_res_bar[2];
  __shared__ __align__(16) float tile_bias_all[2][128];
  __shared__ __align__(16) float tile_scale_all[2][KIND == GEMM_I8 ? 128 : 4];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(stem_smem_raw) + 1023u) & ~1023u;
  const int S = p.stages;
  const uint32_t b_region = smem_base;  // [KH][plane][b_slot]
  const uint32_t a_region = b_region + static_cast<uint32_t>(p.KH * PLANES) * static_cast<uint32_t>(p.b_slot);
  const uint32_t stage_bytes = static_cast<uint32_t>(PLANES) * static_cast<uint32_t>(p.a_plane_bytes);
  const uint32_t staging = a_region + static_cast<uint32_t>(S) * stage_bytes;
  volatile int* abort_ptr = &abort_flag;
  // tile i of this CTA's sequence: stage i % S, accumulator i % accs, issuer i % issuers
  const int accs = p.accs == 4 ? 4 : 2;
  const uint32_t acc_cols = accs == 4 ? 64u : 128u;
  const int issuers = p.issuers == 2 ? 2 : 1;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < S; ++i) {
      mbar_init(smem_u32(&full_bar[i]), 1);
      mbar_init(smem_u32(&empty_bar[i]), 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&tfull_bar[i]), 1);
      mbar_init(smem_u32(&tempty_bar[i]), 4);
    }
    for (int i = 0; i < 2; ++i) mbar_init(smem_u32(&unused_res_bar[i]), 1);
    mbar_init(smem_u32(&weights_bar), 1);
    fence_mbar_init();
    prefetch_tensormap(&map_a0);
    prefetch_tensormap(&map_b0);
    if (PLANES == 2) {
      prefetch_tensormap(&map_a1);
      prefetch_tensormap(&map_b1);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  // barriers, tensor memory and descriptors are ready: from here on the kernel touches tensors that the
  // kernel before it in the stream may still be writing
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
        tma_load_2d(b_region + static_cast<uint32_t>(kh * PLANES + lane) * p.b_slot, map_b, wb,
                    kh * (KIND == GEMM_I8 ? 64 : 32), 0);
    }
    int s = 0;
    uint32_t ph = 0;
    long long issued = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x) {
      const int img = tile / p.OH;
      const int oh = tile - img * p.OH;
      const uint32_t fb = smem_u32(&full_bar[s]);
      int w = 1;
      if (lane == 0) {
        w = mbar_wait_bounded(smem_u32(&empty_bar[s]), ph ^ 1u, abort_ptr, kTcWaitLimitNs) ? 1 : 0;
        if (w) mbar_arrive_expect_tx(fb, static_cast<uint32_t>(PLANES * p.KH) * static_cast<uint32_t>(p.row_bytes));
      }
      w = __shfl_sync(0xffffffffu, w, 0);
      if (!w) {
        ok = false;
        break;
      }
      // rows above or below the image are filled with zeros by the copy
      if (lane < PLANES)
        tma_load_4d(a_region + static_cast<uint32_t>(s) * stage_bytes + static_cast<uint32_t>(lane) * p.a_plane_bytes,
                    map_a, fb, 0, 0, oh * p.stride_h - p.pad_t, img);
      ++issued;
      if (++s == S) {
        s = 0;
        ph ^= 1u;
      }
    }
    if (lane == 0) {
      if (!ok && atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_PRODUCER);
      if (*abort_ptr != 0) {
        // copies this warp issued may still be landing: wait (bounded) for them before the CTA ends
        int zero = 0;
        mbar_wait_bounded(wb, 0, &zero, 200000000ull);
        const long long first = issued > S ? issued - S : 0;
        for (long long i = first; i < issued; ++i)
          mbar_wait_bounded(smem_u32(&full_bar[i % S]), static_cast<uint32_t>((i / S) & 1), &zero, 200000000ull);
      }
    }
  } else if (warp == 1 || (warp == 6 && issuers == 2)) {
    // ---------------------------------------------------------- MMA issuers
    // One thread issues a narrow MMA every 75-150 cycles, the tensor pipe takes one every ~48: with four
    // accumulators warps 1 and 6 issue alternate tiles (MMAs into one accumulator must come from one thread).
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
      int i = me;  // position in this CTA's tile sequence
      for (int tile = blockIdx.x + me * static_cast<int>(gridDim.x); tile < p.tiles && ok; tile += issuers * static_cast<int>(gridDim.x), i += issuers) {
        const int s = i % S, acc = i % accs;
        const uint32_t ph = static_cast<uint32_t>((i / S) & 1), acc_ph = static_cast<uint32_t>((i / accs) & 1);
        if (!mbar_wait_bounded(smem_u32(&tempty_bar[acc]), acc_ph ^ 1u, abort_ptr, kTcWaitLimitNs) ||
            !mbar_wait_bounded(smem_u32(&full_bar[s]), ph, abort_ptr, kTcWaitLimitNs)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * acc_cols;
        const uint64_t a_hi0 = a_fixed + (((a_region + static_cast<uint32_t>(s) * stage_bytes) & 0x3ffffu) >> 4);
        uint32_t accumulate = 0u;
        for (int kh = 0; kh < p.KH; ++kh) {
          const uint64_t a_hi = a_hi0 + static_cast<uint64_t>(kh) * row_units;
          const uint64_t b_hi = b_first + static_cast<uint64_t>(PLANES * kh) * b_slot_units;
#pragma unroll
          for (int ks = 0; ks < 2; ++ks) {  // a 64-byte window = two K steps of 32 bytes (2 units)
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
      }
      if (!ok && atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_MMA);
    }
  } else if (warp != 6) {
    // ------------------------------------------------------------ epilogue (as in tc_gemm_kernel)
    // (with two groups, group g drains the tiles at odd / even positions of the sequence)
    const int group = warp >= 7 ? 1 : 0;
    const int groups = p.epi_groups;
    if (group < groups) {
      const int first_thread = group ? 224 : 64;
      const bool leader = static_cast<int>(threadIdx.x) == first_thread;
      const int quarter = warp & 3;
      float* tile_bias = tile_bias_all[group];
      float* tile_scale = tile_scale_all[group];
      {
        const int t = static_cast<int>(threadIdx.x) - first_thread;
        tile_bias[t] = (p.bias != nullptr && t < p.N) ? __ldg(p.bias + t) : 0.0f;
        if (KIND == GEMM_I8) tile_scale[t] = t < p.N ? __ldg(p.scale + t) : 0.0f;
        else if (t < 4) tile_scale[t] = 0.0f;
      }
      int i = groups == 2 ? group : 0;  // position in this CTA's tile sequence
      uint32_t res_ph = 0;
      int out_slot = 0;
      bool ok = true;
      TcStageCfg cfg{};
      cfg.res_stage = staging + static_cast<uint32_t>(group) * p.staging_bytes;
      cfg.out_stage = cfg.res_stage;
      cfg.res_bar = smem_u32(&unused_res_bar[group]);
      cfg.out_bufs = p.out_bufs;
      cfg.out_mode = p.out_mode;
      cfg.res_mode = RES_NONE;
      cfg.act = p.act;
      cfg.act_a = p.act_a;
      cfg.act_b = p.act_b;
      cfg.N = p.N;
      cfg.block_n = p.N;
      cfg.wide = p.wide;
      cfg.bar_base = 1 + 3 * group;
      const int tile_step = static_cast<int>(gridDim.x) * groups;
      for (int tile = blockIdx.x + (groups == 2 ? group * static_cast<int>(gridDim.x) : 0); tile < p.tiles && ok;
           tile += tile_step, i += groups) {
        const int acc = i % accs;
        const uint32_t acc_ph = static_cast<uint32_t>((i / accs) & 1);
        ok = __all_sync(0xffffffffu,
                        mbar_wait_bounded(smem_u32(&tfull_bar[acc]), acc_ph, abort_ptr, kTcWaitLimitNs) ? 1 : 0) != 0;
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t t_row =
            tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc) * acc_cols;
        // the stores take OW rows of the staging tile (their box is OW rows high); rows beyond hold
        // whatever followed the input row in shared memory and go nowhere
        struct {
          const CUtensorMap *o0, *o1;
          int m_first;
          __device__ __forceinline__ void load_res(int, uint32_t, uint32_t, int) const {}
          __device__ __forceinline__ void store_out(int plane, uint32_t src, int col) const {
            ptx::tma_store_2d(plane ? o1 : o0, src, col, m_first);
          }
          __device__ __forceinline__ void store_side(int, uint32_t, int) const {}
        } io{&map_o0, &map_o1, tile * p.OW};
        if (KIND == GEMM_I8 && p.out_mode == OUT_I8) {
          tc_staged_epilogue_i8<KIND>(cfg, p.out_scale, io, t_row, 0, quarter * 32 + lane, leader, tile_bias, tile_scale,
                                      out_slot);
        } else {
          ok = tc_staged_epilogue<KIND>(cfg, io, t_row, 0, quarter * 32 + lane, leader, tile_bias, tile_scale, res_ph,
                                        out_slot, abort_ptr);
          if (!ok) break;
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
      }
      if (!ok && lane == 0 && atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0)
        atomicCAS(p.status, 0, TC_TIMEOUT_EPILOGUE);
      if (leader) tma_store_wait_all();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, 256);
}

}  // namespace nb
