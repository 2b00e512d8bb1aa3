// Tensor-core contraction on CTA pairs, with an even split of the K blocks over the pairs.
//
// Same contract as tc_gemm_kernel (out[M,N] = epilogue(A[M,K] * B[N,K]^T), A by im2col or tiled
// TMA, B the packed weights, the staged TMA-store epilogue), different shape of the work:
//
// * A tile is 256 rows x block_n columns (block_n up to 256) and belongs to a cluster of two CTAs
//   on the two SMs of one TPC.  Each CTA loads its own 128 rows of A and HALF of the B rows into
//   its own shared memory, and holds its 128 rows of the accumulator in its own tensor memory;
//   CTA 0 issues one tcgen05.mma.cta_group::2 (M = 256) for both.  Per output row a K block then
//   moves 128 + block_n/2 operand rows into an SM instead of 128 + block_n, and reads as little
//   from shared memory per MMA: the operand path, not the tensor pipe, bounds the one-CTA kernel.
//   Every copy writes one CTA's shared memory only; the barrier that counts a stage's bytes lives
//   in CTA 0, the "stage is free" and "accumulator is ready" signals go to both CTAs as arrivals of
//   tcgen05.commit.
//
// * The pairs are persistent workers.  With streamk = 0 worker w takes tiles w, w + G, ...; with
//   streamk = 1 the (tile, K block) units are cut into G equal ranges, so no SM idles in a ragged
//   last wave (layers with few, deep tiles: 49 tiles of 36 K blocks on 74 pairs).  A range may end
//   inside a tile: that piece is computed FIRST and its raw accumulator goes to the CTA's slot of a
//   workspace in global memory with a flag; the worker that holds the tile's last K block waits for
//   those flags (bounded), adds the partial sums in a fixed order and runs the epilogue.  A worker
//   therefore never waits for anything that itself waits, and sums are reproducible run to run.
//
// The same kernel also runs with one CTA per worker (PAIR = false: tiles of 128 rows, the whole B tile in
// the CTA, cta_group::1 instructions, no cluster): that form serves contractions whose few tiles must be
// split to fill the GPU but whose B operand one SM should stream alone (InnerProduct with a handful of rows:
// a pair's CTA sees only half of the weights per MMA, which halves the rate at which an SM can stream them).
//
// Warps of a CTA: 0 A producer, 1 MMA issuer (CTA 0) / idle (CTA 1), 2-5 epilogue, 6 B producer, and for
// wide tiles 7-10 a second epilogue group that drains the other half of the columns.  All waits are
// bounded and end in the status word.
#pragma once

#include "tc_gemm.cuh"

namespace nb {

constexpr int kTc2Threads = 224;        // warps: 0 A producer, 1 MMA issuer, 2-5 epilogue, 6 B producer
constexpr int kTc2ThreadsTwoEpi = 352;  // + warps 7-10: a second epilogue group for the other half of the columns
constexpr int kTc2TileM = 256;  // rows of a pair's tile
constexpr int kTc2MaxBlockN = 256;
constexpr int kTc2AccStride = 256;  // tensor-memory columns between the two accumulators

// The pieces of work of one pair, in the order in which it runs them.
struct Tc2Work {
  long long u0, u1;  // stream-K: this worker's range of units
  int t_first, t_last;
  int nseg;
  int tail_first;  // the range ends inside a tile: that piece runs first
  int KB, G, worker, streamk;
  long long tiles, U;

  __host__ __device__ __forceinline__ void init(const TcGemmParams& p, int worker_, int G_) {
    KB = p.k_blocks;
    G = G_;
    worker = worker_;
    streamk = p.streamk;
    tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
    U = tiles * KB;
    tail_first = 0;
    t_first = t_last = 0;
    u0 = u1 = 0;
    if (streamk) {
      u0 = U * worker / G;
      u1 = U * (worker + 1) / G;
      if (u1 <= u0) {
        nseg = 0;
        return;
      }
      t_first = static_cast<int>(u0 / KB);
      t_last = static_cast<int>((u1 - 1) / KB);
      nseg = t_last - t_first + 1;
      tail_first = (u1 - static_cast<long long>(t_last) * KB) < KB ? 1 : 0;
    } else {
      nseg = worker < tiles ? static_cast<int>((tiles - worker + G - 1) / G) : 0;
    }
  }

  // piece i: its tile, its K blocks [kb0, kb1), and whether this worker finishes the tile
  __host__ __device__ __forceinline__ void seg(int i, int* tile, int* kb0, int* kb1, int* owned) const {
    if (!streamk) {
      *tile = worker + i * G;
      *kb0 = 0;
      *kb1 = KB;
      *owned = 1;
      return;
    }
    const int j = tail_first ? (i == 0 ? nseg - 1 : i - 1) : i;
    *tile = t_first + j;
    *kb0 = j == 0 ? static_cast<int>(u0 - static_cast<long long>(t_first) * KB) : 0;
    *kb1 = j == nseg - 1 ? static_cast<int>(u1 - static_cast<long long>(t_last) * KB) : KB;
    *owned = *kb1 == KB ? 1 : 0;
  }

  // how many workers before this one computed K blocks [0, kb0) of `tile` (they are w-1, w-2, ...)
  __host__ __device__ __forceinline__ int contributors(int tile, int kb0) const {
    if (!streamk || kb0 == 0) return 0;
    const long long ts = static_cast<long long>(tile) * KB;
    int c = 0;
    for (int w = worker - 1; w >= 0 && U * (w + 1) / G > ts; --w) ++c;
    return c;
  }
};

template <int KIND, bool PAIR>
__global__ void __launch_bounds__(kTc2ThreadsTwoEpi, 1)
tc_gemm2_kernel(const __grid_constant__ TcGemmParams p, const __grid_constant__ CUtensorMap map_a0,
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

  extern __shared__ uint8_t tc2_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kTcMaxStages];   // used in CTA 0: both CTAs' bytes of a stage
  __shared__ __align__(8) uint64_t empty_bar[kTcMaxStages];  // per CTA: the MMAs that read the stage are done
  __shared__ __align__(8) uint64_t tfull_bar[2];             // per CTA: accumulator complete
  __shared__ __align__(8) uint64_t tempty_bar[2];            // used in CTA 0: both CTAs' epilogues have drained it
  __shared__ __align__(8) uint64_t res_bar[2];
  __shared__ __align__(16) float tile_bias[kTc2MaxBlockN];
  __shared__ __align__(16) float tile_scale[KIND == GEMM_I8 ? kTc2MaxBlockN : 4];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  constexpr int CTAS = PAIR ? 2 : 1;               // CTAs per worker
  constexpr int TILE_M = PAIR ? kTc2TileM : kTcBlockM;  // rows of a worker's tile
  const uint32_t smem_base = (smem_u32(tc2_smem_raw) + 1023u) & ~1023u;
  const uint32_t slot = static_cast<uint32_t>(kTcBlockM) * p.row_bytes;
  const uint32_t stage_bytes = static_cast<uint32_t>(p.stage_bytes);
  const uint32_t b_slot = (stage_bytes / PLANES) - slot;  // this CTA's half of the B tile, rounded to 1 KB
  const int b_rows = p.block_n / CTAS;
  const int S = p.stages;
  volatile int* abort_ptr = &abort_flag;

  const unsigned trace_cta = (gridDim.x / 4u) * 2u;  // bring-up stamps come from a pair in the middle of the grid
  Tc2Work work;
  work.init(p, static_cast<int>(blockIdx.x) / CTAS, static_cast<int>(gridDim.x) / CTAS);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < S; ++i) {
      mbar_init(smem_u32(&full_bar[i]), 2);  // CTA 0's two producer warps; the bytes of both CTAs
      mbar_init(smem_u32(&empty_bar[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&tfull_bar[i]), 1);
      mbar_init(smem_u32(&tempty_bar[i]), 4u * CTAS * static_cast<uint32_t>(p.epi_groups));  // every epilogue warp of the worker
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

  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------ producers
    // Warp 0 feeds this CTA's 128 rows of A, warp 6 its half of the B rows; lane p issues plane p.
    // The bytes are counted on CTA 0's full barrier, armed by CTA 0's two producer warps for both CTAs.
    const bool is_b = warp == 6;
    const bool issuer = lane < PLANES;
    const CUtensorMap* my_map = is_b ? (lane ? &map_b1 : &map_b0) : (lane ? &map_a1 : &map_a0);
    const uint32_t my_off = is_b ? static_cast<uint32_t>(PLANES) * slot + lane * b_slot : lane * slot;
    const uint32_t tx_both = static_cast<uint32_t>(CTAS) * PLANES * (is_b ? static_cast<uint32_t>(b_rows) * p.row_bytes : slot);
    int s = 0;
    uint32_t ph = 0;
    long long issued = 0;
    bool ok = true;
    for (int i = 0; i < work.nseg && ok; ++i) {
      int tile, kb0, kb1, owned;
      work.seg(i, &tile, &kb0, &kb1, &owned);
      const int m_blk = tile / p.tiles_n;
      const int n_blk = tile - m_blk * p.tiles_n;
      // a second half that starts past the last row repeats the first (its results are never stored)
      long long m0 = static_cast<long long>(m_blk) * TILE_M;
      if (m0 + static_cast<long long>(rank) * kTcBlockM < p.M) m0 += static_cast<long long>(rank) * kTcBlockM;
      const int n0 = n_blk * p.block_n + static_cast<int>(rank) * b_rows;
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
      const int tap0 = kb0 / p.c_blocks;
      int cb = kb0 - tap0 * p.c_blocks;
      int kh = tap0 / p.KW;
      int kw = tap0 - kh * p.KW;
      for (int kb = kb0; kb < kb1; ++kb) {
        const uint32_t fb = PAIR ? map_to_cta(smem_u32(&full_bar[s]), 0u) : smem_u32(&full_bar[s]);
        int w = 1;
        if (lane == 0) {
          w = mbar_wait_bounded(smem_u32(&empty_bar[s]), ph ^ 1u, abort_ptr, kTcWaitLimitNs) ? 1 : 0;
          if (w && rank == 0) mbar_arrive_expect_tx(smem_u32(&full_bar[s]), tx_both);
        }
        w = __shfl_sync(0xffffffffu, w, 0);
        if (!w) {
          ok = false;
          break;
        }
        const bool tr = p.trace != nullptr && blockIdx.x == trace_cta && threadIdx.x == 0 && i == 0 && kb - kb0 < 40;
        if (tr) p.trace[16 + 4 * (kb - kb0) + 2] = clock64();
        if (issuer) {
          const uint32_t dst = smem_base + s * stage_bytes + my_off;
          if (PAIR) {
            if (is_b) {
              tma_load_2d_pair(dst, my_map, fb, kb * p.k_elems, n0);
            } else if (p.a_im2col) {
              tma_load_im2col_4d_pair(dst, my_map, fb, cb * p.k_elems, w_base, h_base, img,
                                      static_cast<uint16_t>(kw * p.dil_w), static_cast<uint16_t>(kh * p.dil_h));
            } else {
              tma_load_2d_pair(dst, my_map, fb, kb * p.k_elems, static_cast<int>(m0));
            }
          } else {
            if (is_b) {
              tma_load_2d(dst, my_map, fb, kb * p.k_elems, n0);
            } else if (p.a_im2col) {
              tma_load_im2col_4d(dst, my_map, fb, cb * p.k_elems, w_base, h_base, img,
                                 static_cast<uint16_t>(kw * p.dil_w), static_cast<uint16_t>(kh * p.dil_h));
            } else {
              tma_load_2d(dst, my_map, fb, kb * p.k_elems, static_cast<int>(m0));
            }
          }
        }
        if (tr) p.trace[16 + 4 * (kb - kb0) + 3] = clock64();
        ++issued;
        if (++cb == p.c_blocks) {
          cb = 0;
          if (++kw == p.KW) {
            kw = 0;
            ++kh;
          }
        }
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
      if (*abort_ptr != 0 && rank == 0) {
        // Some role gave up.  Copies may still be landing in shared memory: wait (bounded) for the
        // last S fills that were armed (CTA 0's barriers count both CTAs' bytes).
        int zero = 0;
        const long long first = issued > S ? issued - S : 0;
        for (long long i = first; i < issued; ++i) {
          const int st = static_cast<int>(i % S);
          const uint32_t par = static_cast<uint32_t>((i / S) & 1);
          mbar_wait_bounded(smem_u32(&full_bar[st]), par, &zero, 200000000ull);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer (CTA 0 only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = KIND == GEMM_I8
                                 ? instr_desc(2u, 1u, TILE_M, static_cast<uint32_t>(p.block_n))
                                 : instr_desc(1u, KIND == GEMM_BF16X3 ? 1u : 2u, TILE_M,
                                              static_cast<uint32_t>(p.block_n));
      const int k_steps = p.row_bytes / 32;
      const uint64_t desc_fixed = smem_desc_kmajor(0u, static_cast<uint32_t>(p.row_bytes));
      const uint64_t a_first = desc_fixed + ((smem_base & 0x3ffffu) >> 4);
      const uint64_t stage_units = stage_bytes >> 4;
      const uint64_t slot_units = slot >> 4;
      const uint64_t b_slot_units = b_slot >> 4;
      const uint64_t b_from_a = static_cast<uint64_t>(PLANES) * slot_units;
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (int i = 0; i < work.nseg && ok; ++i) {
        int tile, kb0, kb1, owned;
        work.seg(i, &tile, &kb0, &kb1, &owned);
        if (!mbar_wait_bounded(smem_u32(&tempty_bar[acc]), acc_ph ^ 1u, abort_ptr, kTcWaitLimitNs)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * kTc2AccStride;
        uint32_t accumulate = 0u;
        const bool tracing = p.trace != nullptr && blockIdx.x == trace_cta && i == 0;
        if (tracing) {
          p.trace[0] = clock64();
          p.trace[1] = static_cast<long long>(global_timer_ns());
        }
        const bool ptr = p.trace != nullptr && blockIdx.x == trace_cta && i < 6;
        if (ptr) p.trace[512 + 8 * i] = clock64();
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(smem_u32(&full_bar[s]), ph, abort_ptr, kTcWaitLimitNs)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (tracing && kb - kb0 < 40) p.trace[16 + 4 * (kb - kb0)] = clock64();
          const uint64_t a0 = a_first + static_cast<uint64_t>(s) * stage_units;
          const uint64_t b0 = a0 + b_from_a;
#pragma unroll 4
          for (int k = 0; k < k_steps; ++k) {
            const uint64_t ka = a0 + 2u * k;
            const uint64_t kbd = b0 + 2u * k;
            if (PAIR) {
              if (KIND == GEMM_TF32) {
                mma_tf32_pair(d_tmem, ka, kbd, idesc, accumulate);
              } else if (KIND == GEMM_TF32X3) {
                mma_tf32_pair(d_tmem, ka + slot_units, kbd, idesc, accumulate);  // lo * hi
                mma_tf32_pair(d_tmem, ka, kbd + b_slot_units, idesc, 1u);        // hi * lo
                mma_tf32_pair(d_tmem, ka, kbd, idesc, 1u);                       // hi * hi
              } else if (KIND == GEMM_BF16X3) {
                mma_f16_pair(d_tmem, ka + slot_units, kbd, idesc, accumulate);  // mid * hi
                mma_f16_pair(d_tmem, ka, kbd + b_slot_units, idesc, 1u);        // hi * mid
                mma_f16_pair(d_tmem, ka, kbd, idesc, 1u);                       // hi * hi
              } else {
                mma_i8_pair(d_tmem, ka, kbd, idesc, accumulate);
              }
            } else {
              if (KIND == GEMM_TF32) {
                mma_tf32(d_tmem, ka, kbd, idesc, accumulate);
              } else if (KIND == GEMM_TF32X3) {
                mma_tf32(d_tmem, ka + slot_units, kbd, idesc, accumulate);
                mma_tf32(d_tmem, ka, kbd + b_slot_units, idesc, 1u);
                mma_tf32(d_tmem, ka, kbd, idesc, 1u);
              } else if (KIND == GEMM_BF16X3) {
                mma_f16(d_tmem, ka + slot_units, kbd, idesc, accumulate);
                mma_f16(d_tmem, ka, kbd + b_slot_units, idesc, 1u);
                mma_f16(d_tmem, ka, kbd, idesc, 1u);
              } else {
                mma_i8(d_tmem, ka, kbd, idesc, accumulate);
              }
            }
            accumulate = 1u;
          }
          if (PAIR) tc_commit_pair(smem_u32(&empty_bar[s]), 3);  // the stage is free in both CTAs
          else tc_commit(smem_u32(&empty_bar[s]));
          if (tracing && kb - kb0 < 40) p.trace[16 + 4 * (kb - kb0) + 1] = clock64();
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (!ok) break;
        if (PAIR) tc_commit_pair(smem_u32(&tfull_bar[acc]), 3);  // both CTAs' halves of the accumulator are complete
        else tc_commit(smem_u32(&tfull_bar[acc]));
        if (tracing) {
          p.trace[2] = clock64();
          p.trace[3] = static_cast<long long>(global_timer_ns());
        }
        if (ptr) {
          p.trace[512 + 8 * i + 1] = clock64();
          p.trace[512 + 8 * i + 5] = kb1 - kb0;
        }
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1u;
      }
      if (!ok) {
        if (atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_MMA);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    // One group (warps 2-5) drains all block_n columns; with two groups (352 threads) warps 2-5 take
    // the first half of the columns and warps 7-10 the second, each with its own staging tiles,
    // barriers, residual barrier and workspace flags.  An epilogue warp runs alone on its scheduler
    // and pays every instruction's latency, so two groups nearly halve the time of a wide tile.
    const int groups = p.epi_groups;
    const int group = warp >= 7 ? 1 : 0;
    const int first_thread = group ? 224 : 64;
    const bool leader = static_cast<int>(threadIdx.x) == first_thread;
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+31] belong to this warp
    const int row = quarter * 32 + lane;
    const int half = p.block_n / groups;  // columns of this group
    const int col0 = group * half;        // first column of the group inside the tile
    const size_t slot_words = static_cast<size_t>(kTcBlockM) * p.block_n;
    const int bar_base = 1 + 3 * group;   // named barriers bar_base .. bar_base + 2
    const int my_flag = static_cast<int>(blockIdx.x) * 2 + group;
    const int flag_step = 2 * CTAS;  // flag words between this CTA and the same CTA of the worker before
    float* my_bias = tile_bias + col0;
    float* my_scale = tile_scale + (KIND == GEMM_I8 ? col0 : 0);
    int acc = 0;
    uint32_t acc_ph = 0;
    uint32_t res_ph = 0;
    int out_slot = 0;
    bool ok = true;
    TcStageCfg cfg{};
    cfg.res_stage = smem_base + static_cast<uint32_t>(S) * stage_bytes + static_cast<uint32_t>(group) * p.staging_bytes;
    cfg.out_stage = cfg.res_stage + (p.res_mode != RES_NONE ? 16384u : 0u);
    cfg.res_bar = smem_u32(&res_bar[group]);
    cfg.out_bufs = p.out_bufs;
    cfg.out_mode = p.out_mode;
    cfg.res_mode = p.res_mode;
    cfg.act = p.act;
    cfg.act_a = p.act_a;
    cfg.act_b = p.act_b;
    cfg.N = p.N;
    cfg.block_n = half;
    cfg.wide = p.wide;
    cfg.bar_base = bar_base;
    cfg.fix_stride = -static_cast<long long>(CTAS) * static_cast<long long>(slot_words);  // the same CTA of the worker before
    const uint32_t tempty0 = PAIR ? map_to_cta(smem_u32(&tempty_bar[0]), 0u) : smem_u32(&tempty_bar[0]);
    const uint32_t tempty1 = PAIR ? map_to_cta(smem_u32(&tempty_bar[1]), 0u) : smem_u32(&tempty_bar[1]);
    for (int i = 0; i < work.nseg && ok; ++i) {
      int tile, kb0, kb1, owned;
      work.seg(i, &tile, &kb0, &kb1, &owned);
      const int m_blk = tile / p.tiles_n;
      const int n_blk = tile - m_blk * p.tiles_n;
      const long long m_first = static_cast<long long>(m_blk) * TILE_M + static_cast<long long>(rank) * kTcBlockM;
      const bool row_valid = m_first + row < p.M;  // rows past the end hold nothing worth exchanging
      const int n0 = n_blk * p.block_n + col0;
      // the vote keeps the warp together: tcgen05.ld below needs all 32 lanes
      ok = __all_sync(0xffffffffu,
                      mbar_wait_bounded(smem_u32(&tfull_bar[acc]), acc_ph, abort_ptr, kTcWaitLimitNs) ? 1 : 0) != 0;
      if (!ok) break;
      tc_fence_after_sync();
      const bool etr = p.trace != nullptr && blockIdx.x == trace_cta && threadIdx.x == 64 && i == 0;
      if (etr) p.trace[4] = clock64();
      const bool eptr = p.trace != nullptr && blockIdx.x == trace_cta && threadIdx.x == 64 && i < 6;
      if (eptr) {
        p.trace[512 + 8 * i + 2] = clock64();
        p.trace[512 + 8 * i + 6] = owned;
      }
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(acc) * kTc2AccStride + static_cast<uint32_t>(col0);
      // this group's columns of a CTA's workspace slot: [16-column group][row][16]
      const size_t ws_group = static_cast<size_t>(col0 >> 4) * 128 * 16;
      if (!owned) {
        // a piece of a tile that another pair finishes: raw accumulator to this CTA's slot, then the flag
        uint32_t* dst = p.sk_ws + static_cast<size_t>(blockIdx.x) * slot_words + ws_group;
        for (int c0 = 0; c0 < half; c0 += 32) {
          uint32_t v[16], w[16];
          tmem_ld16(t_row + static_cast<uint32_t>(c0), v);
          tmem_ld16(t_row + static_cast<uint32_t>(c0 + 16), w);
          tmem_ld_wait();
          uint4* d4 = reinterpret_cast<uint4*>(dst + (static_cast<size_t>(c0 >> 4) * 128 + row) * 16);
          if (row_valid) {
#pragma unroll
            for (int q = 0; q < 4; ++q) d4[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            if (c0 + 16 < half) {
              d4 += 128 * 4;
#pragma unroll
              for (int q = 0; q < 4; ++q) d4[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
            }
          }
        }
        __threadfence();
        named_barrier_sync(bar_base + 2, 128);
        if (leader) st_release_gpu(p.sk_flags + my_flag, 1);
      } else {
        const int fix = work.contributors(tile, kb0);
        if (fix > 0) {
          // wait (bounded) until every piece of this tile has been published; lane 0 of each warp polls
          int got = 1;
          if (lane == 0) {
            for (int c = 1; c <= fix && got; ++c) {
              const int* flag = p.sk_flags + (my_flag - flag_step * c);
              uint64_t t0 = 0;
              uint32_t polls = 0;
              while (ld_acquire_gpu(flag) == 0) {
                if ((++polls & 0xffu) == 0) {
                  if (*abort_ptr != 0) {
                    got = 0;
                    break;
                  }
                  const uint64_t now = global_timer_ns();
                  if (t0 == 0) t0 = now;
                  else if (now - t0 > kTcWaitLimitNs) {
                    got = 0;
                    break;
                  }
                }
              }
            }
          }
          ok = __all_sync(0xffffffffu, got) != 0;
          if (!ok) break;
          if (eptr) {
            p.trace[512 + 8 * i + 4] = clock64();
            p.trace[512 + 8 * i + 7] = fix;
          }
        }
        if (m_first < p.M) {
          cfg.side_count = p.side_count;
          cfg.side_ld = p.side_ld;
          cfg.side_rows = static_cast<int>(p.M - m_first < kTcBlockM ? p.M - m_first : kTcBlockM);
          cfg.side_q0 = p.side_q0 != nullptr ? p.side_q0 + m_first * p.side_ld + n0 : nullptr;
          cfg.side_q1 = p.side_q1 != nullptr ? p.side_q1 + m_first * p.side_ld + n0 : nullptr;
          cfg.side_scale0 = p.side_scale0;
          cfg.side_scale1 = p.side_scale1;
          cfg.fix_count = row_valid ? fix : 0;  // (a row past the end skips the loads; its results are clipped)
          cfg.fix_ws = fix > 0 ? p.sk_ws + static_cast<size_t>(static_cast<int>(blockIdx.x) - CTAS) * slot_words + ws_group
                               : nullptr;
          // per-column constants of this tile (every warp of the group has left the previous tile's last
          // chunk: it ends with a barrier)
          for (int t = static_cast<int>(threadIdx.x) - first_thread; t < half; t += 128) {
            const int n = n0 + t;
            my_bias[t] = (p.bias != nullptr && n < p.N) ? __ldg(p.bias + n) : 0.0f;
            if (KIND == GEMM_I8) my_scale[t] = n < p.N ? __ldg(p.scale + n) : 0.0f;
          }
          const int m_row = static_cast<int>(m_first);
          struct {
            const CUtensorMap *o0, *o1, *r0, *r1;
            int m_first;
            __device__ __forceinline__ void load_res(int plane, uint32_t dst, uint32_t bar, int col) const {
              ptx::tma_load_2d(dst, plane ? r1 : r0, bar, col, m_first);
            }
            __device__ __forceinline__ void store_out(int plane, uint32_t src, int col) const {
              ptx::tma_store_2d(plane ? o1 : o0, src, col, m_first);
            }
            __device__ __forceinline__ void store_side(int, uint32_t, int) const {}
          } io{&map_o0, &map_o1, &map_r0, &map_r1, m_row};
          const bool extras = fix > 0 || p.side_count > 0;
          if (p.out_mode == OUT_I8) {
            if (extras)
              tc_staged_epilogue_i8<KIND, decltype(io), true>(cfg, p.out_scale, io, t_row, n0, row, leader, my_bias, my_scale,
                                                              out_slot);
            else
              tc_staged_epilogue_i8<KIND>(cfg, p.out_scale, io, t_row, n0, row, leader, my_bias, my_scale, out_slot);
          } else {
            if (extras)
              ok = tc_staged_epilogue<KIND, decltype(io), true>(cfg, io, t_row, n0, row, leader, my_bias, my_scale, res_ph,
                                                                out_slot, abort_ptr);
            else
              ok = tc_staged_epilogue<KIND>(cfg, io, t_row, n0, row, leader, my_bias, my_scale, res_ph, out_slot,
                                            abort_ptr);
            if (!ok) break;
          }
        }
        if (fix > 0) {
          // every warp of the group has read the slots (it passed the chunk barriers, or this one): free them
          named_barrier_sync(bar_base + 2, 128);
          if (leader)
            for (int c = 1; c <= fix; ++c) p.sk_flags[my_flag - flag_step * c] = 0;
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (etr) p.trace[5] = clock64();
      if (eptr) p.trace[512 + 8 * i + 3] = clock64();
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
    if (leader) tma_store_wait_all();  // stores still read shared memory
  }

  // Neither CTA leaves while the other may still signal its barriers or read its shared memory.
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
