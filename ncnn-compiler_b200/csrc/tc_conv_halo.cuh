// Stride-1 convolution on the tensor cores with the input patch resident in shared memory.
//
// tc_gemm_kernel fetches the 128 input pixels of a tile once per filter tap (im2col TMA).
// The operand path from L2 into an SM sustains only ~40 bytes/cycle, so for 3x3 filters
// that re-fetch, not the tensor pipe, sets the pace.  Here a tile is a 16 x 8 rectangle
// of output pixels of one image.  For each block of input channels (one 128-byte row: 32
// fp32 or 64 bf16) the
// (16+KH-1) x (8+KW-1) input patch is loaded ONCE by a 4-D tiled TMA (out-of-range
// coordinates read as zero: that is the padding), and every filter tap multiplies straight
// out of it: the A descriptor of tap (kh, kw) starts (kh*patch_w + kw) rows into the patch,
// and its stride between 8-row groups is one patch row.  (The MMA unit and TMA both swizzle
// on absolute shared-memory address bits, so a descriptor may start at any 128-byte row;
// checked on hardware.)  Only the weights stream per tap.
//
// Roles, accumulator double-buffering, bounded waits and the staged TMA-store epilogue are
// those of tc_gemm_kernel; floating-point kinds only (tf32, tf32x3, bf16x3), outputs in rows
// of 16 bytes.
//
// PAIR = true runs two pixel tiles on a cluster of two CTAs: each CTA keeps its own patch, loads HALF of
// the weight rows of a tap, and CTA 0 issues tcgen05.mma.cta_group::2 (M = 256: both patches against the
// whole weight tile).  What an SM must fetch per tile is then one patch per channel block and half a
// weight tile per tap, which is what the operand path can deliver next to running MMAs; every copy still
// writes one CTA's shared memory only.
#pragma once

#include "tc_gemm.cuh"

namespace nb {

constexpr int kHaloTileH = 16;
constexpr int kHaloTileW = 8;
constexpr int kHaloThreads = 192;  // warps: 0 producer, 1 MMA issuer, 2-5 epilogue

struct TcHaloParams {
  int images, OH, OW, N;
  int tiles_y, tiles_x, tiles_n, block_n;
  int c_blocks, k_elems, taps, KW;
  int pad_t, pad_l;
  int patch_h, patch_w;
  int patch_bytes;   // one plane of one patch buffer, rounded to 1 KB
  int b_bytes;       // one plane of one B stage, rounded to 1 KB
  int stages;        // B ring depth
  int out_bufs;      // output staging tiles (>= 2)
  const float* bias;
  int res_mode;      // RES_*
  int out_mode;
  int act;
  float act_a, act_b;
  int* status;
  long long* trace;  // optional (bring-up): clock stamps of the first work item of a worker in the middle of the grid
};

template <int KIND, bool PAIR = false>
__global__ void __launch_bounds__(kHaloThreads, 1)
tc_conv_halo_kernel(const __grid_constant__ TcHaloParams p, const __grid_constant__ CUtensorMap map_a0,
                    const __grid_constant__ CUtensorMap map_a1,
                    const __grid_constant__ CUtensorMap map_b0,
                    const __grid_constant__ CUtensorMap map_b1,
                    const __grid_constant__ CUtensorMap map_o0,
                    const __grid_constant__ CUtensorMap map_o1,
                    const __grid_constant__ CUtensorMap map_r0,
                    const __grid_constant__ CUtensorMap map_r1) {
  using namespace ptx;
  grid_dependency_trigger();  // the next kernel of the stream may begin its preamble
  constexpr int PLANES = tc_planes(KIND);

  extern __shared__ uint8_t halo_smem_raw[];
  __shared__ __align__(8) uint64_t a_full[2];
  __shared__ __align__(8) uint64_t a_empty[2];
  __shared__ __align__(8) uint64_t b_full[kTcMaxStages];
  __shared__ __align__(8) uint64_t b_empty[kTcMaxStages];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];
  __shared__ __align__(8) uint64_t res_bar;
  __shared__ __align__(16) float tile_bias[256];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int CTAS = PAIR ? 2 : 1;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int worker = static_cast<int>(blockIdx.x) / CTAS;   // a CTA, or a pair of them
  const int workers = static_cast<int>(gridDim.x) / CTAS;
  const int b_rows = p.block_n / CTAS;                      // weight rows of a tap that this CTA loads
  const uint32_t smem_base = (smem_u32(halo_smem_raw) + 1023u) & ~1023u;
  const uint32_t patch_bytes = static_cast<uint32_t>(p.patch_bytes);
  const uint32_t a_buf_bytes = PLANES * patch_bytes;
  const uint32_t b_bytes = static_cast<uint32_t>(p.b_bytes);
  const uint32_t b_stage_bytes = PLANES * b_bytes;
  const uint32_t b_ring = smem_base + 2u * a_buf_bytes;
  const int S = p.stages;
  const uint32_t res_stage = b_ring + static_cast<uint32_t>(S) * b_stage_bytes;
  const uint32_t out_stage = res_stage + (p.res_mode != RES_NONE ? 16384u : 0u);
  const int tiles_per_image = p.tiles_y * p.tiles_x;
  const int pixel_tiles = p.images * tiles_per_image;
  // work items: a pixel tile (PAIR: two consecutive pixel tiles) times a channel block
  const int total_tiles = ((pixel_tiles + CTAS - 1) / CTAS) * p.tiles_n;
  volatile int* abort_ptr = &abort_flag;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&a_full[i]), 1);
      mbar_init(smem_u32(&a_empty[i]), 1);
      mbar_init(smem_u32(&tfull_bar[i]), 1);
      mbar_init(smem_u32(&tempty_bar[i]), 4u * CTAS);
    }
    for (int i = 0; i < S; ++i) {
      mbar_init(smem_u32(&b_full[i]), 1);
      mbar_init(smem_u32(&b_empty[i]), 1);
    }
    mbar_init(smem_u32(&res_bar), 1);
    fence_mbar_init();
    prefetch_tensormap(&map_a0);
    prefetch_tensormap(&map_b0);
    prefetch_tensormap(&map_o0);
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(&tmem_slot), kTcTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(&tmem_slot), kTcTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the other CTA's barriers exist before anything is sent to them
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  // barriers, tensor memory and descriptors are ready: from here on the kernel touches tensors that the
  // kernel before it in the stream may still be writing
  grid_dependency_wait();

  // tile -> (image, tile row, tile column, channel block); channel blocks of one pixel tile
  // are neighbours so that CTAs working side by side share the patch in L2
  // (*valid: a pair's second pixel tile may lie past the last one; it then repeats the first and stores nothing)
  auto decode = [&](int tile, int* img, int* oy0, int* ox0, int* n0, bool* valid) {
    const int n_blk = tile % p.tiles_n;
    int t = (tile / p.tiles_n) * CTAS + static_cast<int>(rank);
    *valid = t < pixel_tiles;
    if (!*valid) t -= static_cast<int>(rank);
    const int tx = t % p.tiles_x;
    t /= p.tiles_x;
    const int ty = t % p.tiles_y;
    *img = t / p.tiles_y;
    *oy0 = ty * kHaloTileH;
    *ox0 = tx * kHaloTileW;
    *n0 = n_blk * p.block_n;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    // one lane per TMA copy (issuing is what costs): lanes 0/1 the weight planes of a tap,
    // lanes 2/3 the patch planes of a channel block; lane 0 owns the barrier traffic
    const bool b_issuer = lane < PLANES;
    const bool a_issuer = lane >= 2 && lane < 2 + PLANES;
    const int plane = lane & 1;
    // (PAIR: the bytes of both CTAs are counted on CTA 0's barriers, armed by CTA 0)
    const uint32_t a_tx = CTAS * PLANES * static_cast<uint32_t>(p.patch_h * p.patch_w) * 128u;
    const uint32_t b_tx = CTAS * PLANES * static_cast<uint32_t>(b_rows) * 128u;
    int s = 0, ab = 0;
    uint32_t ph = 0, a_ph = 0;
    long long a_issued = 0, b_issued = 0;
    bool ok = true;
    for (int tile = worker; tile < total_tiles && ok; tile += workers) {
      int img, oy0, ox0, n0;
      bool valid;
      decode(tile, &img, &oy0, &ox0, &n0, &valid);
      n0 += static_cast<int>(rank) * b_rows;
      for (int cb = 0; cb < p.c_blocks && ok; ++cb) {
        const uint32_t ab_bar = PAIR ? map_to_cta(smem_u32(&a_full[ab]), 0u) : smem_u32(&a_full[ab]);
        int w = 1;
        if (lane == 0) {
          w = mbar_wait_bounded(smem_u32(&a_empty[ab]), a_ph ^ 1u, abort_ptr, kTcWaitLimitNs) ? 1 : 0;
          if (w && rank == 0) mbar_arrive_expect_tx(smem_u32(&a_full[ab]), a_tx);
        }
        w = __shfl_sync(0xffffffffu, w, 0);
        if (!w) {
          ok = false;
          break;
        }
        if (a_issuer) {
          const uint32_t dst = smem_base + static_cast<uint32_t>(ab) * a_buf_bytes + plane * patch_bytes;
          if (PAIR) tma_load_4d_pair(dst, plane ? &map_a1 : &map_a0, ab_bar, cb * p.k_elems, ox0 - p.pad_l, oy0 - p.pad_t, img);
          else tma_load_4d(dst, plane ? &map_a1 : &map_a0, ab_bar, cb * p.k_elems, ox0 - p.pad_l, oy0 - p.pad_t, img);
        }
        ++a_issued;
        ab ^= 1;
        if (ab == 0) a_ph ^= 1u;
        for (int tap = 0; tap < p.taps; ++tap) {
          const uint32_t fb = PAIR ? map_to_cta(smem_u32(&b_full[s]), 0u) : smem_u32(&b_full[s]);
          if (lane == 0) {
            w = mbar_wait_bounded(smem_u32(&b_empty[s]), ph ^ 1u, abort_ptr, kTcWaitLimitNs) ? 1 : 0;
            if (w && rank == 0) mbar_arrive_expect_tx(smem_u32(&b_full[s]), b_tx);
          }
          w = __shfl_sync(0xffffffffu, w, 0);
          if (!w) {
            ok = false;
            break;
          }
          const bool ptr_ = p.trace != nullptr && worker == workers / 2 && rank == 0 && tile == worker && cb == 0 && lane == 0 && tap < 16;
          if (ptr_) p.trace[16 + 4 * tap + 2] = clock64();
          if (b_issuer) {
            const uint32_t dst = b_ring + static_cast<uint32_t>(s) * b_stage_bytes + plane * b_bytes;
            if (PAIR) tma_load_2d_pair(dst, plane ? &map_b1 : &map_b0, fb, (tap * p.c_blocks + cb) * p.k_elems, n0);
            else tma_load_2d(dst, plane ? &map_b1 : &map_b0, fb, (tap * p.c_blocks + cb) * p.k_elems, n0);
          }
          ++b_issued;
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
    if (lane == 0) {
      if (!ok) {
        if (atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_PRODUCER);
      }
      if (*abort_ptr != 0 && rank == 0) {
        // copies may still be landing (CTA 0's barriers count both CTAs' bytes): wait (bounded) for the last ones
        int zero = 0;
        for (long long i = b_issued > S ? b_issued - S : 0; i < b_issued; ++i)
          mbar_wait_bounded(smem_u32(&b_full[i % S]), static_cast<uint32_t>((i / S) & 1), &zero, 200000000ull);
        for (long long i = a_issued > 2 ? a_issued - 2 : 0; i < a_issued; ++i)
          mbar_wait_bounded(smem_u32(&a_full[i % 2]), static_cast<uint32_t>((i / 2) & 1), &zero, 200000000ull);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0 && rank == 0) {
      const uint32_t idesc =
          instr_desc(1u, KIND == GEMM_BF16X3 ? 1u : 2u, kTcBlockM * CTAS, static_cast<uint32_t>(p.block_n));
      // A: 128-byte rows, 128B swizzle, 8-row groups one patch row apart
      const uint64_t a_fixed = (static_cast<uint64_t>((static_cast<uint32_t>(p.patch_w) * 128u) >> 4) << 32) |
                               (1ull << 46) | (2ull << 61);
      const uint64_t b_fixed = smem_desc_kmajor(0u, 128u);
      const uint64_t patch_units = patch_bytes >> 4;
      const uint64_t b_units = b_bytes >> 4;
      const int taps = p.taps, KW = p.KW, PW = p.patch_w, c_blocks = p.c_blocks;
      const uint32_t acc_stride = p.block_n > 128 ? 256u : 128u;
      int s = 0, ab = 0, acc = 0;
      uint32_t ph = 0, a_ph = 0, acc_ph = 0;
      bool ok = true;
      for (int tile = worker; tile < total_tiles && ok; tile += workers) {
        if (!mbar_wait_bounded(smem_u32(&tempty_bar[acc]), acc_ph ^ 1u, abort_ptr, kTcWaitLimitNs)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * acc_stride;
        uint32_t accumulate = 0u;
        for (int cb = 0; cb < c_blocks && ok; ++cb) {
          if (!mbar_wait_bounded(smem_u32(&a_full[ab]), a_ph, abort_ptr, kTcWaitLimitNs)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint64_t a_patch =
              a_fixed + (((smem_base + static_cast<uint32_t>(ab) * a_buf_bytes) & 0x3ffffu) >> 4);
          int kh = 0, kw = 0;
          const bool tr = p.trace != nullptr && worker == workers / 2 && tile == worker && cb == 0;
          if (tr) p.trace[0] = clock64();
          for (int tap = 0; tap < taps; ++tap) {
            if (!mbar_wait_bounded(smem_u32(&b_full[s]), ph, abort_ptr, kTcWaitLimitNs)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            if (tr && tap < 16) p.trace[16 + 4 * tap] = clock64();
            const uint64_t a0 = a_patch + static_cast<uint64_t>((kh * PW + kw) * 8);  // 128 B = 8 units
            const uint64_t b0 = b_fixed + (((b_ring + static_cast<uint32_t>(s) * b_stage_bytes) & 0x3ffffu) >> 4);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint64_t ka = a0 + 2u * k;
              const uint64_t kb = b0 + 2u * k;
              if (PAIR) {
                if (KIND == GEMM_TF32) {
                  mma_tf32_pair(d_tmem, ka, kb, idesc, accumulate);
                } else if (KIND == GEMM_BF16X3) {
                  mma_f16_pair(d_tmem, ka + patch_units, kb, idesc, accumulate);  // mid * hi
                  mma_f16_pair(d_tmem, ka, kb + b_units, idesc, 1u);              // hi * mid
                  mma_f16_pair(d_tmem, ka, kb, idesc, 1u);                        // hi * hi
                } else {
                  mma_tf32_pair(d_tmem, ka + patch_units, kb, idesc, accumulate);
                  mma_tf32_pair(d_tmem, ka, kb + b_units, idesc, 1u);
                  mma_tf32_pair(d_tmem, ka, kb, idesc, 1u);
                }
              } else if (KIND == GEMM_TF32) {
                mma_tf32(d_tmem, ka, kb, idesc, accumulate);
              } else if (KIND == GEMM_BF16X3) {
                mma_f16(d_tmem, ka + patch_units, kb, idesc, accumulate);  // mid * hi
                mma_f16(d_tmem, ka, kb + b_units, idesc, 1u);              // hi * mid
                mma_f16(d_tmem, ka, kb, idesc, 1u);                        // hi * hi
              } else {
                mma_tf32(d_tmem, ka + patch_units, kb, idesc, accumulate);  // lo * hi
                mma_tf32(d_tmem, ka, kb + b_units, idesc, 1u);              // hi * lo
                mma_tf32(d_tmem, ka, kb, idesc, 1u);                        // hi * hi
              }
              accumulate = 1u;
            }
            if (PAIR) tc_commit_pair(smem_u32(&b_empty[s]), 3);
            else tc_commit(smem_u32(&b_empty[s]));
            if (tr && tap < 16) p.trace[16 + 4 * tap + 1] = clock64();
            if (++s == S) {
              s = 0;
              ph ^= 1u;
            }
            if (++kw == KW) {
              kw = 0;
              ++kh;
            }
          }
          if (!ok) break;
          if (PAIR) tc_commit_pair(smem_u32(&a_empty[ab]), 3);
          else tc_commit(smem_u32(&a_empty[ab]));
          ab ^= 1;
          if (ab == 0) a_ph ^= 1u;
        }
        if (!ok) break;
        if (PAIR) tc_commit_pair(smem_u32(&tfull_bar[acc]), 3);
        else tc_commit(smem_u32(&tfull_bar[acc]));
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1u;
      }
      if (!ok) {
        if (atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_MMA);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
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
    cfg.wide = (p.out_mode == OUT_BF16X2 || p.res_mode == RES_BF16X2) ? 1 : 0;
    const int e_N = p.N;
    int acc = 0, out_slot = 0;
    uint32_t acc_ph = 0, res_ph = 0;
    bool ok = true;
    const uint32_t acc_stride = p.block_n > 128 ? 256u : 128u;
    const uint32_t tempty0 = PAIR ? map_to_cta(smem_u32(&tempty_bar[0]), 0u) : smem_u32(&tempty_bar[0]);
    const uint32_t tempty1 = PAIR ? map_to_cta(smem_u32(&tempty_bar[1]), 0u) : smem_u32(&tempty_bar[1]);
    for (int tile = worker; tile < total_tiles && ok; tile += workers) {
      int img, oy0, ox0, n0;
      bool valid;
      decode(tile, &img, &oy0, &ox0, &n0, &valid);
      ok = __all_sync(0xffffffffu,
                      mbar_wait_bounded(smem_u32(&tfull_bar[acc]), acc_ph, abort_ptr, kTcWaitLimitNs) ? 1 : 0) != 0;
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_row =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc) * acc_stride;
      for (int t = static_cast<int>(threadIdx.x) - 64; t < p.block_n; t += 128) {
        const int n = n0 + t;
        tile_bias[t] = (p.bias != nullptr && n < e_N) ? __ldg(p.bias + n) : 0.0f;
      }
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
      const bool etr = p.trace != nullptr && worker == workers / 2 && rank == 0 && tile == worker && threadIdx.x == 64;
      if (etr) p.trace[4] = clock64();
      if (valid) {
        ok = tc_staged_epilogue<KIND>(cfg, io, t_row, n0, row, threadIdx.x == 64, tile_bias, tile_bias, res_ph,
                                      out_slot, abort_ptr);
        if (!ok) break;
      }
      if (etr) p.trace[5] = clock64();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(acc ? tempty1 : tempty0);
        else mbar_arrive(acc ? tempty1 : tempty0);
      }
      acc ^= 1;
      if (acc == 0) acc_ph ^= 1u;
    }
    if (!ok && lane == 0) {
      if (atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_EPILOGUE);
    }
    if (threadIdx.x == 64) tma_store_wait_all();
  }

  // (a pair: neither CTA leaves while the other may still signal its barriers or read its shared memory)
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();
  tc_fence_after_sync();
  if (warp == 1) {
    if (PAIR) tmem_dealloc_pair(tmem_base, kTcTmemCols);
    else tmem_dealloc(tmem_base, kTcTmemCols);
  }
}

}  // namespace nb
