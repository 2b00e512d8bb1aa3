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
// Warps of a CTA (224 threads): 0 A producer, 1 MMA issuer (CTA 0) / idle (CTA 1), 2-5 epilogue,
// 6 B producer.  All waits are bounded and end in the status word.
#pragma once

#include "tc_gemm.cuh"

namespace nb {

constexpr int kTc2Threads = 224;
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

template <int KIND>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kTc2Threads, 1)
tc_gemm2_kernel(const __grid_constant__ TcGemmParams p, const __grid_constant__ CUtensorMap map_a0,
                const __grid_constant__ CUtensorMap map_a1,
                const __grid_constant__ CUtensorMap map_b0,
                const __grid_constant__ CUtensorMap map_b1,
                const __grid_constant__ CUtensorMap map_o0,
                const __grid_constant__ CUtensorMap map_o1,
                const __grid_constant__ CUtensorMap map_r0,
                const __grid_constant__ CUtensorMap map_r1) {
  using namespace ptx;
  constexpr int PLANES = tc_planes(KIND);

  extern __shared__ uint8_t tc2_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kTcMaxStages];   // used in CTA 0: both CTAs' bytes of a stage
  __shared__ __align__(8) uint64_t empty_bar[kTcMaxStages];  // per CTA: the MMAs that read the stage are done
  __shared__ __align__(8) uint64_t tfull_bar[2];             // per CTA: accumulator complete
  __shared__ __align__(8) uint64_t tempty_bar[2];            // used in CTA 0: both CTAs' epilogues have drained it
  __shared__ __align__(8) uint64_t res_bar;
  __shared__ __align__(16) float tile_bias[kTc2MaxBlockN];
  __shared__ __align__(16) float tile_scale[KIND == GEMM_I8 ? kTc2MaxBlockN : 4];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const uint32_t smem_base = (smem_u32(tc2_smem_raw) + 1023u) & ~1023u;
  const uint32_t slot = static_cast<uint32_t>(kTcBlockM) * p.row_bytes;
  const uint32_t stage_bytes = static_cast<uint32_t>(p.stage_bytes);
  const uint32_t b_slot = (stage_bytes / PLANES) - slot;  // this CTA's half of the B tile, rounded to 1 KB
  const int b_rows = p.block_n / 2;
  const int S = p.stages;
  volatile int* abort_ptr = &abort_flag;

  Tc2Work work;
  work.init(p, static_cast<int>(blockIdx.x >> 1), static_cast<int>(gridDim.x >> 1));

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < S; ++i) {
      mbar_init(smem_u32(&full_bar[i]), 2);  // CTA 0's two producer warps; the bytes of both CTAs
      mbar_init(smem_u32(&empty_bar[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&tfull_bar[i]), 1);
      mbar_init(smem_u32(&tempty_bar[i]), 8);  // four epilogue warps of each CTA
    }
    mbar_init(smem_u32(&res_bar), 1);
    fence_mbar_init();
    prefetch_tensormap(&map_a0);
    prefetch_tensormap(&map_b0);
    if (PLANES == 2) {
      prefetch_tensormap(&map_a1);
      prefetch_tensormap(&map_b1);
    }
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&tmem_slot), kTcTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the other CTA's barriers exist before anything is sent to them
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------ producers
    // Warp 0 feeds this CTA's 128 rows of A, warp 6 its half of the B rows; lane p issues plane p.
    // The bytes are counted on CTA 0's full barrier, armed by CTA 0's two producer warps for both CTAs.
    const bool is_b = warp == 6;
    const bool issuer = lane < PLANES;
    const CUtensorMap* my_map = is_b ? (lane ? &map_b1 : &map_b0) : (lane ? &map_a1 : &map_a0);
    const uint32_t my_off = is_b ? static_cast<uint32_t>(PLANES) * slot + lane * b_slot : lane * slot;
    const uint32_t tx_both = 2u * PLANES * (is_b ? static_cast<uint32_t>(b_rows) * p.row_bytes : slot);
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
      long long m0 = static_cast<long long>(m_blk) * kTc2TileM;
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
        const uint32_t fb = map_to_cta(smem_u32(&full_bar[s]), 0u);
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
        if (issuer) {
          const uint32_t dst = smem_base + s * stage_bytes + my_off;
          if (is_b) {
            tma_load_2d_pair(dst, my_map, fb, kb * p.k_elems, n0);
          } else if (p.a_im2col) {
            tma_load_im2col_4d_pair(dst, my_map, fb, cb * p.k_elems, w_base, h_base, img,
                                    static_cast<uint16_t>(kw * p.dil_w), static_cast<uint16_t>(kh * p.dil_h));
          } else {
            tma_load_2d_pair(dst, my_map, fb, kb * p.k_elems, static_cast<int>(m0));
          }
        }
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
                                 ? instr_desc(2u, 1u, kTc2TileM, static_cast<uint32_t>(p.block_n))
                                 : instr_desc(1u, KIND == GEMM_BF16X3 ? 1u : 2u, kTc2TileM,
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
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(smem_u32(&full_bar[s]), ph, abort_ptr, kTcWaitLimitNs)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint64_t a0 = a_first + static_cast<uint64_t>(s) * stage_units;
          const uint64_t b0 = a0 + b_from_a;
#pragma unroll 4
          for (int k = 0; k < k_steps; ++k) {
            const uint64_t ka = a0 + 2u * k;
            const uint64_t kbd = b0 + 2u * k;
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
            accumulate = 1u;
          }
          tc_commit_pair(smem_u32(&empty_bar[s]), 3);  // the stage is free in both CTAs
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit_pair(smem_u32(&tfull_bar[acc]), 3);  // both CTAs' halves of the accumulator are complete
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1u;
      }
      if (!ok) {
        if (atomicCAS(const_cast<int*>(abort_ptr), 0, 1) == 0) atomicCAS(p.status, 0, TC_TIMEOUT_MMA);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2-5 of both CTAs)
    const bool leader = threadIdx.x == 64;
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+31] belong to this warp
    const int row = quarter * 32 + lane;
    const size_t slot_words = static_cast<size_t>(kTcBlockM) * p.block_n;
    int acc = 0;
    uint32_t acc_ph = 0;
    uint32_t res_ph = 0;
    int out_slot = 0;
    bool ok = true;
    TcStageCfg cfg{};
    cfg.res_stage = smem_base + static_cast<uint32_t>(S) * stage_bytes;
    cfg.out_stage = cfg.res_stage + (p.res_mode != RES_NONE ? 16384u : 0u);
    cfg.res_bar = smem_u32(&res_bar);
    cfg.out_bufs = p.out_bufs;
    cfg.out_mode = p.out_mode;
    cfg.res_mode = p.res_mode;
    cfg.act = p.act;
    cfg.act_a = p.act_a;
    cfg.act_b = p.act_b;
    cfg.N = p.N;
    cfg.block_n = p.block_n;
    cfg.wide = p.wide;
    cfg.bar_base = 1;
    cfg.fix_stride = -2ll * static_cast<long long>(slot_words);  // the same CTA rank of the pair before
    const uint32_t tempty0 = map_to_cta(smem_u32(&tempty_bar[0]), 0u);
    const uint32_t tempty1 = map_to_cta(smem_u32(&tempty_bar[1]), 0u);
    for (int i = 0; i < work.nseg && ok; ++i) {
      int tile, kb0, kb1, owned;
      work.seg(i, &tile, &kb0, &kb1, &owned);
      const int m_blk = tile / p.tiles_n;
      const int n_blk = tile - m_blk * p.tiles_n;
      const long long m_first = static_cast<long long>(m_blk) * kTc2TileM + static_cast<long long>(rank) * kTcBlockM;
      const int n0 = n_blk * p.block_n;
      // the vote keeps the warp together: tcgen05.ld below needs all 32 lanes
      ok = __all_sync(0xffffffffu,
                      mbar_wait_bounded(smem_u32(&tfull_bar[acc]), acc_ph, abort_ptr, kTcWaitLimitNs) ? 1 : 0) != 0;
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(acc) * kTc2AccStride;
      if (!owned) {
        // a piece of a tile that another pair finishes: raw accumulator to this CTA's slot, then the flag
        uint32_t* dst = p.sk_ws + static_cast<size_t>(blockIdx.x) * slot_words;
        for (int c0 = 0; c0 < p.block_n; c0 += 16) {
          uint32_t v[16];
          tmem_ld16(t_row + static_cast<uint32_t>(c0), v);
          tmem_ld_wait();
          uint4* d4 = reinterpret_cast<uint4*>(dst + (static_cast<size_t>(c0 >> 4) * 128 + row) * 16);
#pragma unroll
          for (int q = 0; q < 4; ++q) d4[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        }
        __threadfence();
        named_barrier_sync(3, 128);
        if (leader) st_release_gpu(p.sk_flags + blockIdx.x, 1);
      } else {
        const int fix = work.contributors(tile, kb0);
        if (fix > 0) {
          // wait (bounded) until every piece of this tile has been published; lane 0 of each warp polls
          int got = 1;
          if (lane == 0) {
            for (int c = 1; c <= fix && got; ++c) {
              const int* flag = p.sk_flags + (static_cast<int>(blockIdx.x) - 2 * c);
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
        }
        if (m_first < p.M) {
          cfg.fix_count = fix;
          cfg.fix_ws = fix > 0 ? p.sk_ws + static_cast<size_t>(static_cast<int>(blockIdx.x) - 2) * slot_words : nullptr;
          // per-column constants of this tile (every warp has left the previous tile's last chunk:
          // it ends with a barrier)
          for (int t = static_cast<int>(threadIdx.x) - 64; t < p.block_n; t += 128) {
            const int n = n0 + t;
            tile_bias[t] = (p.bias != nullptr && n < p.N) ? __ldg(p.bias + n) : 0.0f;
            if (KIND == GEMM_I8) tile_scale[t] = n < p.N ? __ldg(p.scale + n) : 0.0f;
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
          } io{&map_o0, &map_o1, &map_r0, &map_r1, m_row};
          if (p.out_mode == OUT_I8) {
            tc_staged_epilogue_i8<KIND>(cfg, p.out_scale, io, t_row, n0, row, leader, tile_bias, tile_scale, out_slot);
          } else {
            ok = tc_staged_epilogue<KIND>(cfg, io, t_row, n0, row, leader, tile_bias, tile_scale, res_ph, out_slot,
                                          abort_ptr);
            if (!ok) break;
          }
        }
        if (fix > 0) {
          // every warp has read the slots (it passed the chunk barriers, or this one): free them
          named_barrier_sync(3, 128);
          if (leader)
            for (int c = 1; c <= fix; ++c) p.sk_flags[static_cast<int>(blockIdx.x) - 2 * c] = 0;
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc ? tempty1 : tempty0);
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
  cluster_sync_all();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc_pair(tmem_base, kTcTmemCols);
}

}  // namespace nb
