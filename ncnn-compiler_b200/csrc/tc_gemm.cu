#include "tc_gemm.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace nb {
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
using EncodeIm2colFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                    cuuint32_t, cuuint32_t, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn g_encode_tiled = nullptr;
EncodeIm2colFn g_encode_im2col = nullptr;
std::once_flag g_driver_once;
std::string g_driver_error;

void load_driver_entry_points() {
  std::call_once(g_driver_once, [] {
    cudaDriverEntryPointQueryResult query;
    void* fn = nullptr;
    cudaError_t err =
        cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query);
    if (err != cudaSuccess || query != cudaDriverEntryPointSuccess || fn == nullptr) {
      g_driver_error = "cuTensorMapEncodeTiled is not available from this driver";
      return;
    }
    g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    fn = nullptr;
    err = cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &query);
    if (err != cudaSuccess || query != cudaDriverEntryPointSuccess || fn == nullptr) {
      g_driver_error = "cuTensorMapEncodeIm2col is not available from this driver";
      return;
    }
    g_encode_im2col = reinterpret_cast<EncodeIm2colFn>(fn);
  });
}

CUtensorMapSwizzle swizzle_for(int row_bytes) {
  return row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : (row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                             : CU_TENSOR_MAP_SWIZZLE_32B);
}

CUtensorMapDataType dtype_for(int kind) {
  return kind == GEMM_I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                         : (kind == GEMM_BF16X3 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32);
}

int elem_bytes(int kind) { return tc_elem_bytes(kind); }

std::string encode_tiled_2d(CUtensorMap* map, int kind, const void* base, uint64_t inner,
                            uint64_t outer, uint64_t outer_stride_bytes, uint32_t box_inner,
                            uint32_t box_outer, int row_bytes) {
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {outer_stride_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r = g_encode_tiled(map, dtype_for(kind), 2, const_cast<void*>(base), dims,
                                    strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                    swizzle_for(row_bytes), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)) +
           " (inner " + std::to_string(inner) + ", outer " + std::to_string(outer) + ", stride " +
           std::to_string(outer_stride_bytes) + ")";
  }
  return {};
}

std::string encode_im2col(CUtensorMap* map, int kind, const void* base, const TcIm2colView& v,
                          uint32_t channels_per_pixel, int row_bytes) {
  const cuuint64_t dims[4] = {v.C, v.W, v.H, v.N};
  const cuuint64_t strides[3] = {v.stride_w, v.stride_h, v.stride_n};
  // Bounding box of filter-origin positions: the first is -pad, the last is the
  // origin of the last output pixel; TMA wants it relative to the tensor's far edge.
  const int last_w = -v.pad_l + (v.OW - 1) * v.stride_conv_w;
  const int last_h = -v.pad_t + (v.OH - 1) * v.stride_conv_h;
  const int lower[2] = {-v.pad_l, -v.pad_t};
  const int upper[2] = {last_w - (static_cast<int>(v.W) - 1), last_h - (static_cast<int>(v.H) - 1)};
  const cuuint32_t elem_strides[4] = {1, static_cast<cuuint32_t>(v.stride_conv_w),
                                      static_cast<cuuint32_t>(v.stride_conv_h), 1};
  const CUresult r = g_encode_im2col(
      map, dtype_for(kind), 4, const_cast<void*>(base), dims, strides, lower, upper,
      channels_per_pixel, kTcBlockM, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
      swizzle_for(row_bytes), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return "cuTensorMapEncodeIm2col failed with code " + std::to_string(static_cast<int>(r)) +
           " (C " + std::to_string(v.C) + ", W " + std::to_string(v.W) + ", H " +
           std::to_string(v.H) + ", N " + std::to_string(v.N) + ", strides " +
           std::to_string(v.stride_w) + "/" + std::to_string(v.stride_h) + "/" +
           std::to_string(v.stride_n) + ", corners " + std::to_string(lower[0]) + "," +
           std::to_string(lower[1]) + " / " + std::to_string(upper[0]) + "," +
           std::to_string(upper[1]) + ")";
  }
  return {};
}

// Dynamic shared memory a CTA may fill: 227 KB per block, minus the kernel's static shared
// memory (barriers and per-tile constants: 1.2 KB, 2.2 KB for the int8 kernel with its
// dequantisation factors), minus 1 KB of alignment slack.
constexpr int tc_smem_budget(int kind) { return (kind == GEMM_I8 ? 223 : 224) * 1024; }
// From this many K blocks per tile on, the main loop of the next tile hides even the slower
// direct epilogue, and a third ring stage is worth more than the staging tiles.
constexpr int kDirectEpilogueDepth = 32;

// Tile width: every multiple of 16 up to 128 is a legal UMMA N.  Cost model:
// waves over the SMs times (columns computed + a fixed per-tile term for the
// A traffic and pipeline fill, which do not shrink with the tile).
int choose_block_n(long long tiles_m, int N, int sm_count, int step) {
  int best = step;
  double best_cost = 1e300;
  for (int bn = step; bn <= 128; bn += step) {
    const long long tiles = tiles_m * ((N + bn - 1) / bn);
    const long long waves = (tiles + sm_count - 1) / sm_count;
    const double cost = static_cast<double>(waves) * (bn + 24);
    if (cost < best_cost - 1e-9 || (std::fabs(cost - best_cost) <= 1e-9 && bn > best)) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

// NCNN_B200_PAIR=0 in the environment keeps every tile at 128 rows.
bool pair_enabled() {
  const char* f = std::getenv("NCNN_B200_PAIR");
  return f == nullptr || f[0] != '0';
}

int env_int(const char* name, int fallback);

void finish_plan(TcLaunch* L, int kind, long long M, int N, const TcEpilogue& e, int sm_count) {
  TcGemmParams& p = L->p;
  p.M = static_cast<int>(M);
  p.N = N;
  p.tiles_m = static_cast<int>((M + kTcBlockM - 1) / kTcBlockM);
  // a bf16-pair output or residual is staged 32 columns at a time
  const int res_mode = e.res0 == nullptr ? RES_NONE : (e.res_bf16 ? RES_BF16X2 : (e.res1 != nullptr ? RES_SPLIT : RES_F32));
  // Shallow contractions are bound by the epilogue: plain fp32 results then also go out 32 columns
  // at a time (half as many barriers and store rounds per tile).
  const bool shallow_f32 = e.out_mode == OUT_F32 && res_mode != RES_SPLIT && N % 16 == 0 && N >= 32 && p.k_blocks <= 4;
  const bool wide = e.out_mode == OUT_BF16X2 || res_mode == RES_BF16X2 || shallow_f32;
  // int8 results can leave through TMA stores in chunks of 64 columns when every tile is a
  // multiple of 64 wide, rows are 16-byte multiples and nothing is added after requantisation
  const bool i8_staged = e.out_mode == OUT_I8 && N % 64 == 0 && e.ldo % 16 == 0 && e.res0 == nullptr &&
                         (reinterpret_cast<uintptr_t>(e.outq) & 15) == 0;
  // int8 copies of an fp32 result (TcEpilogue::side_q) leave 64 columns at a time through staging tiles of
  // their own (two [128][64] tiles per copy) when rows and tiles come in 64-channel units
  const bool side_staged = e.side_count > 0 && e.out_mode != OUT_I8 && N % 64 == 0 && e.ldo % 16 == 0 &&
                           (reinterpret_cast<uintptr_t>(e.side_q[0]) & 15) == 0 &&
                           (reinterpret_cast<uintptr_t>(e.side_q[1]) & 15) == 0;
  const int side_bytes = side_staged ? e.side_count * 16384 : 0;
  p.block_n = choose_block_n(p.tiles_m, N, sm_count, (i8_staged || side_staged) ? 64 : (wide ? 32 : 16));
  p.tiles_n = (N + p.block_n - 1) / p.block_n;
  const int kTcSmemBudget = tc_smem_budget(kind);
  const int planes = tc_planes(kind);
  // a stage holds the A tile(s) and block_n rows of B, every sub-buffer 1 KB aligned
  const int b_bytes = (p.block_n * p.row_bytes + 1023) / 1024 * 1024;
  p.stage_bytes = planes * (kTcBlockM * p.row_bytes + b_bytes);
  // fp32 results leave through TMA stores when rows are 16-byte multiples; the staging
  // tiles (out hi/lo, residual hi/lo, 8 KB each) sit behind the ring
  const bool f32_out = e.out_mode != OUT_I8;
  const bool aligned = e.ldo % (wide ? 8 : 4) == 0 && (reinterpret_cast<uintptr_t>(e.out0) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(e.out1) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(e.res0) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(e.res1) & 15) == 0;
  // (a wide chunk cannot carry fp32 hi/lo planes: that pairing does not occur, the direct path covers it)
  p.tma_store = f32_out && aligned && !(wide && (e.out_mode == OUT_F32_SPLIT || e.out_mode == OUT_F32_TF32 ||
                                                  res_mode == RES_SPLIT))
                    ? 1
                    : 0;
  if (i8_staged) p.tma_store = 1;
  // residual tiles (16 KB) + two to four output tiles of 8 KB per plane; fewer when the
  // operand ring would drop below three stages
  const int out_tile = (e.out_mode != OUT_I8 && (e.out_mode == OUT_F32_SPLIT || wide) ? 2 : 1) * 8192;
  int staging = 0;
  p.out_bufs = 2;
  if (p.tma_store) {
    for (int bufs : {4, 3, 2}) {
      p.out_bufs = bufs;
      staging = ((res_mode != RES_NONE ? 16384 : 0) + side_bytes) + bufs * out_tile;
      if ((kTcSmemBudget - staging) / p.stage_bytes >= 3 || bufs == 2) break;
    }
    // Deep contractions hide even a slow epilogue behind the next tile's main loop; there a third
    // ring stage is worth more than the staging tiles.  With one tile per CTA nothing hides the
    // epilogue, and the direct one takes several times as long as the staged one.
    const int with = (kTcSmemBudget - staging) / p.stage_bytes;
    const int without = (kTcSmemBudget) / p.stage_bytes;
    const long long tiles_all = static_cast<long long>(p.tiles_m) * p.tiles_n;
    if (with < 3 && without >= 3 && p.k_blocks >= kDirectEpilogueDepth && tiles_all > sm_count) {
      p.tma_store = 0;
      staging = 0;
    }
  }
  // Shallow contractions (a few K blocks per tile) are bound by the epilogue, which runs one warp
  // per scheduler and so pays every instruction's latency in full: a second epilogue group drains
  // every other tile, with a staging area of its own.  Two groups with two staging tiles each beat
  // one group with four, so the tile count per group is reduced before the second group is given up.
  const long long tiles_total = static_cast<long long>(p.tiles_m) * p.tiles_n;
  // The same holds for deeper contractions whose K blocks are cheap (int8: a K block is 128 channels
  // and one or two MMAs): estimate both sides per tile, in cycles, from measured figures -- about 1800
  // cycles per fp32 chunk and 3000 per 64-column int8 chunk in the epilogue; per K block the larger of
  // the MMA issue time and the operand fetch at 45 bytes per cycle.
  const int chunk_cols = e.out_mode == OUT_I8 ? 64 : (wide ? 32 : 16);
  const double epi_cycles = static_cast<double>((p.block_n + chunk_cols - 1) / chunk_cols) * (e.out_mode == OUT_I8 ? 3000.0 : 1800.0);
  const double mma_cycles = (planes == 2 ? 3.0 : 1.0) * (p.row_bytes / 32) * (p.block_n <= 64 ? 48.0 : 64.0 * p.block_n / 128.0);
  const double main_cycles = p.k_blocks * std::max(mma_cycles, p.stage_bytes / 45.0);
  const bool epilogue_bound = env_int("NCNN_B200_EPI2", 1) != 0 && epi_cycles > 1.2 * main_cycles;
  p.epi_groups = 1;
  if (p.tma_store && (p.k_blocks <= 4 || epilogue_bound) && tiles_total >= 2ll * sm_count) {
    const int res_bytes = (res_mode != RES_NONE ? 16384 : 0) + side_bytes;
    for (int bufs : {4, 3, 2}) {
      const int both = 2 * (res_bytes + bufs * out_tile);
      if (bufs > p.out_bufs) continue;
      // (a tile of one or two K blocks needs no more than the next tile's operands in flight)
      if ((kTcSmemBudget - both) / p.stage_bytes >= (bufs == 2 ? (p.k_blocks <= 2 ? 2 : 3) : 4)) {
        p.epi_groups = 2;
        p.out_bufs = bufs;
        staging = both;
        break;
      }
    }
  }
  // Paired tiles: two 128-row halves share every B tile, so a K block moves 256 + block_n operand
  // rows for twice the output instead of 2 x (128 + block_n).  Worth it where the operand fetch sets
  // the pace (deep contractions over full 128-byte rows; the stem's 64-byte window rows ran 9%
  // slower paired) and the coarser tiles still fill the SMs wave by wave; the ring then holds two
  // (larger) stages.
  p.pair = 0;
  p.pair_rows = 0;
  if (pair_enabled() && p.tma_store && p.epi_groups == 1 && p.k_blocks >= 6 && p.block_n <= 128 &&
      p.row_bytes >= 128) {
    const int pair_stage = planes * (2 * kTcBlockM * p.row_bytes + b_bytes);
    // as many output tiles as still leave two stages (the leader waits less for stores to drain)
    int pair_bufs = 2;
    for (int bufs : {4, 3})
      if ((kTcSmemBudget - ((res_mode != RES_NONE ? 16384 : 0) + side_bytes) - bufs * out_tile) / pair_stage >= 2) {
        pair_bufs = bufs;
        break;
      }
    const int pair_staging = ((res_mode != RES_NONE ? 16384 : 0) + side_bytes) + pair_bufs * out_tile;
    const long long waves_single = (tiles_total + sm_count - 1) / sm_count;
    const double cost_single = static_cast<double>(waves_single) * (kTcBlockM + p.block_n);
    // whole waves of pairs first, single tiles for what is left; k waves of pairs cover
    // floor(k * SMs / tiles_n) tile rows of 256
    const int max_pair_rows = p.tiles_m / 2;
    double best = cost_single;
    int best_rows = 0;
    for (int k = 1; k <= 65; ++k) {  // up to 64 waves of pairs, then "all pairs"
      const int rows = k == 65 ? max_pair_rows
                               : static_cast<int>(std::min<long long>(max_pair_rows, static_cast<long long>(k) * sm_count / p.tiles_n));
      const long long pair_tiles = static_cast<long long>(rows) * p.tiles_n;
      const long long single_tiles = static_cast<long long>(p.tiles_m - 2 * rows) * p.tiles_n;
      const double cost = static_cast<double>((pair_tiles + sm_count - 1) / sm_count) * (2 * kTcBlockM + p.block_n) +
                          static_cast<double>((single_tiles + sm_count - 1) / sm_count) * (kTcBlockM + p.block_n);
      if (cost < best - 1e-9) {
        best = cost;
        best_rows = rows;
      }
      if (rows == max_pair_rows) break;
    }
    const long long tiles_mixed = static_cast<long long>(p.tiles_m - best_rows) * p.tiles_n;
    if (best_rows > 0 && best < 0.97 * cost_single && tiles_mixed * 10 >= 9ll * sm_count &&
        (kTcSmemBudget - pair_staging) / pair_stage >= 2) {
      p.pair = 1;
      p.pair_rows = best_rows;
      p.tiles_m = p.tiles_m - best_rows;  // tile rows: best_rows pairs, then singles
      p.stage_bytes = pair_stage;
      p.out_bufs = pair_bufs;
      staging = pair_staging;
    }
  }
  p.staging_bytes = staging / p.epi_groups;
  const int budget = kTcSmemBudget - staging;
  // int8 K blocks are two to four MMAs over 12-32 KB: arming and releasing a ring stage (~450 cycles of barrier
  // hand-shake per block, more than the block's copies and MMAs take) sets the pace.  A stage then holds several
  // K blocks (a divisor of their count, at least three stages deep): one hand-shake for all of them.
  p.sub_blocks = 1;
  if (kind == GEMM_I8 && !p.pair && env_int("NCNN_B200_SUB_BLOCKS", 1) != 0)
    for (int sub : {4, 3, 2})
      if (p.k_blocks % sub == 0 && budget / (sub * p.stage_bytes) >= 3) {
        p.sub_blocks = sub;
        break;
      }
  p.stages = std::max(2, std::min(kTcMaxStages, budget / (p.sub_blocks * p.stage_bytes)));
  L->smem_bytes = p.stages * p.sub_blocks * p.stage_bytes + staging + 1024;
  // never fewer bytes than half an SM's shared memory: two CTAs must not share an
  // SM, each allocates tensor memory for itself
  L->smem_bytes = std::max(L->smem_bytes, 120 * 1024);
  const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
  L->grid = static_cast<int>(std::min<long long>(tiles, sm_count));
  L->kind = kind;
  p.bias = e.bias;
  p.scale = e.scale;
  p.out0 = e.out0;
  p.out1 = e.out1;
  p.outq = e.outq;
  p.res0 = e.res0;
  p.res1 = e.res1;
  p.res_mode = res_mode;
  p.wide = wide ? 1 : 0;
  p.ldo = e.ldo;
  p.out_mode = e.out_mode;
  p.act = e.act;
  p.act_a = e.act_a;
  p.act_b = e.act_b;
  p.out_scale = e.out_scale;
  p.status = e.status;
  p.trace = e.trace;
  p.side_staged = side_staged && p.tma_store ? 1 : 0;
  p.side_count = e.side_count;
  p.side_ld = e.ldo;
  p.side_q0 = e.side_q[0];
  p.side_q1 = e.side_q[1];
  p.side_scale0 = e.side_scale[0];
  p.side_scale1 = e.side_scale[1];
  L->map_o0 = L->map_o1 = L->map_r0 = L->map_r1 = L->map_s0 = L->map_s1 = CUtensorMap{};
}

// ---- CTA pairs (tc_gemm2.cuh)
// NCNN_B200_CTA2=0 keeps every contraction on the one-CTA kernel; NCNN_B200_STREAMK=0 never splits
// a tile between pairs, =1 always does where it can; NCNN_B200_CTA2_MIN_KB sets the shallowest
// contraction (K blocks per tile) that goes to pairs.
int env_int(const char* name, int fallback) {
  const char* f = std::getenv(name);
  return f == nullptr || f[0] == 0 ? fallback : std::atoi(f);
}

int max_pairs_resident(int kind, int smem_bytes, int sm_count);

// Function attributes (the opt-in to more than 48 KB of dynamic shared memory) belong to a device's
// context: they are set once per device, with that device current, not once per process.
struct PerDeviceOnce {
  std::mutex mutex;
  bool done[64] = {};
  cudaError_t result[64] = {};
  template <class F>
  cudaError_t run(F&& setup) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mutex);
    if (!done[device]) {
      result[device] = setup();
      done[device] = true;
    }
    return result[device];
  }
};

// NCNN_B200_PDL=0 launches every contraction kernel fully serialised behind its predecessor.
bool pdl_enabled() {
  static const bool on = env_int("NCNN_B200_PDL", 1) != 0;
  return on;
}

// Launch attributes of the contraction kernels: clusters of two CTAs for the pair form, and programmatic
// stream serialisation: the kernel's preamble (barriers, tensor memory, descriptor prefetch) may run while
// the previous kernel of the stream drains; the kernel itself waits (grid_dependency_wait) before it
// touches any tensor.
struct KernelLaunchConfig {
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attrs[2];
  KernelLaunchConfig(int grid, int threads, int smem_bytes, bool pair, cudaStream_t stream) {
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(static_cast<unsigned>(threads));
    cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
    cfg.stream = stream;
    cfg.attrs = attrs;
    cfg.numAttrs = 0;
    if (pair) {
      attrs[cfg.numAttrs].id = cudaLaunchAttributeClusterDimension;
      attrs[cfg.numAttrs].val.clusterDim.x = 2;
      attrs[cfg.numAttrs].val.clusterDim.y = 1;
      attrs[cfg.numAttrs].val.clusterDim.z = 1;
      ++cfg.numAttrs;
    }
    if (pdl_enabled()) {
      attrs[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attrs[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
      ++cfg.numAttrs;
    }
  }
};

// True when tc_gemm2_kernel takes this contraction (on CTA pairs, or on single CTAs with tiles split
// between them); fills the plan like finish_plan does.
// `half_blocks_ok`: K blocks of half the size (64-byte rows) address the same packed operands, so
// the plan may trade K-block size for staging tiles.
bool finish_plan_workers(TcLaunch* L, int kind, long long M, int N, const TcEpilogue& e, int sm_count,
                         bool half_blocks_ok) {
  TcGemmParams& p = L->p;
  if (env_int("NCNN_B200_CTA2", 1) == 0 || sm_count < 2) return false;
  if (p.k_blocks < env_int("NCNN_B200_CTA2_MIN_KB", 6)) return false;
  const int res_mode = e.res0 == nullptr ? RES_NONE : (e.res_bf16 ? RES_BF16X2 : (e.res1 != nullptr ? RES_SPLIT : RES_F32));
  const bool wide = e.out_mode == OUT_BF16X2 || res_mode == RES_BF16X2;
  const bool i8_staged = e.out_mode == OUT_I8 && N % 64 == 0 && e.ldo % 16 == 0 && e.res0 == nullptr &&
                         (reinterpret_cast<uintptr_t>(e.outq) & 15) == 0;
  const bool f32_out = e.out_mode != OUT_I8;
  const bool aligned = e.ldo % (wide ? 8 : 4) == 0 && (reinterpret_cast<uintptr_t>(e.out0) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(e.out1) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(e.res0) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(e.res1) & 15) == 0;
  const bool staged = i8_staged || (f32_out && aligned &&
                                    !(wide && (e.out_mode == OUT_F32_SPLIT || e.out_mode == OUT_F32_TF32 ||
                                               res_mode == RES_SPLIT)));
  if (!staged) return false;  // this kernel has the staged epilogue only
  if (e.side_count > 0) return false;  // int8 copies of the result: the one-CTA kernel writes those
  const int step = i8_staged ? 64 : (wide ? 32 : 16);
  auto even_width = [&](int widest) {
    const int n_tiles = (N + widest - 1) / widest;
    return ((N + n_tiles - 1) / n_tiles + step - 1) / step * step;
  };
  const int full_kb = p.k_blocks;
  const int forced_split = env_int("NCNN_B200_STREAMK", -1);
  const bool ws_given = e.sk_ws != nullptr && e.sk_flags != nullptr;

  // Form 1, CTA pairs: tiles of 256 rows x up to 256 columns.  Measured on ResNet-18 at batch 64: tiles of
  // 256 columns keep the tensor pipe busy through the whole main loop (the operand path of an SM carries half
  // the bytes per product); narrower pair tiles gain nothing over the one-CTA kernel's paired tiles and pay
  // more barrier hand-shakes per output.  Taken when whole tiles fill at least one wave of pairs.
  const int pair_bn = even_width(kTc2MaxBlockN);
  const long long pair_tiles = ((M + kTc2TileM - 1) / kTc2TileM) * ((N + pair_bn - 1) / pair_bn);
  const bool pair_form = pair_bn >= env_int("NCNN_B200_CTA2_MIN_BN", 192) &&
                         (pair_tiles >= sm_count / 2 || env_int("NCNN_B200_CTA2_ALWAYS", 0) != 0);
  // Form 2, single CTAs with split tiles: tiles of 128 rows x up to 128 columns, every SM an equal share of
  // the K blocks.  Taken when whole tiles would leave SMs idle (few, deep tiles) and the workspace allows.
  const int one_bn = even_width(128);
  const long long one_tiles = ((M + kTcBlockM - 1) / kTcBlockM) * ((N + one_bn - 1) / one_bn);
  const long long one_units = one_tiles * full_kb;
  const int one_workers = static_cast<int>(std::min<long long>(sm_count, one_units / 4));
  bool split_form = false;
  // Where a tile is cut depends on how many tiles there are, so a split layer rounds its fp32 sums
  // differently at different batch sizes.  Convolutions keep whole tiles (splitting them gained nothing
  // on the benchmark networks, and a batch then equals its images run one by one bit for bit);
  // InnerProduct and Gemm, where a handful of rows must stream megabytes of weights, are split.
  const bool may_split = forced_split == 1 || (forced_split != 0 && !p.a_im2col);
  if (!pair_form && ws_given && may_split && one_workers >= 2) {
    // Every worker ends with the tile it finishes, whose partial sums arrive no earlier than the other
    // workers finish theirs: publishing, waiting and adding them is an exposed tail worth about twenty
    // K blocks (measured on 3x3 convolutions of 256 and 512 channels at batch 64, where splitting lost).
    const double cost_whole = static_cast<double>((one_tiles + sm_count - 1) / sm_count) * full_kb;
    const double cost_split = static_cast<double>((one_units + one_workers - 1) / one_workers) + 20.0;
    split_form = forced_split == 1 || cost_split < 0.9 * cost_whole;
  }
  if (!pair_form && !split_form) return false;
  const int ctas = pair_form ? 2 : 1;
  const int tile_m = pair_form ? kTc2TileM : kTcBlockM;

  p.M = static_cast<int>(M);
  p.N = N;
  p.tiles_m = static_cast<int>((M + tile_m - 1) / tile_m);
  p.block_n = pair_form ? pair_bn : one_bn;
  p.tiles_n = (N + p.block_n - 1) / p.block_n;
  const int budget_all = tc_smem_budget(kind);
  const int planes = tc_planes(kind);
  p.tma_store = 1;
  const int out_tile = (e.out_mode != OUT_I8 && (e.out_mode == OUT_F32_SPLIT || wide) ? 2 : 1) * 8192;
  const int res_bytes = res_mode != RES_NONE ? 16384 : 0;
  // Choose epilogue groups, K-block size and staging tiles.  Two groups (each half of the columns) come
  // first: the epilogue of a wide tile is what a worker with one or two tiles cannot hide.  Then full-size
  // K blocks, then as many staging tiles as leave the ring deep enough to cover the copy latency.
  const bool two_groups_ok = env_int("NCNN_B200_CTA2_GROUPS", 2) >= 2 && p.block_n >= 128 && (p.block_n / 2) % step == 0;
  const int full_rb = p.row_bytes, full_cb = p.c_blocks, full_ke = p.k_elems;
  bool chosen = false;
  int staging = 0;
  auto try_config = [&](int groups, bool half_blocks, int bufs, int min_stages) {
    const int rb = half_blocks ? full_rb / 2 : full_rb;
    const int b_bytes = ((p.block_n / ctas) * rb + 1023) / 1024 * 1024;
    const int stage = planes * (kTcBlockM * rb + b_bytes);
    const int stg = groups * (res_bytes + bufs * out_tile);
    const int stages = std::min(kTcMaxStages, (budget_all - stg) / stage);
    if (stages < min_stages) return false;
    p.epi_groups = groups;
    p.out_bufs = bufs;
    p.row_bytes = rb;
    p.k_elems = half_blocks ? full_ke / 2 : full_ke;
    p.c_blocks = half_blocks ? full_cb * 2 : full_cb;
    p.k_blocks = half_blocks ? full_kb * 2 : full_kb;
    p.stage_bytes = stage;
    p.stages = stages;
    staging = stg;
    return true;
  };
  const bool halves = half_blocks_ok && full_rb == 128 && kind == GEMM_BF16X3;
  for (int groups : {2, 1}) {
    if (groups == 2 && !two_groups_ok) continue;
    for (int hb = 0; hb < 2 && !chosen; ++hb) {
      if (hb == 1 && !halves) continue;
      for (int bufs : {4, 3, 2})
        if (!chosen && try_config(groups, hb == 1, bufs, hb ? 4 : 3)) chosen = true;
    }
    if (chosen) break;
  }
  // last resort: one group, one or two staging tiles, two stages
  if (!chosen)
    for (int bufs : {2, 1})
      if (!chosen && (bufs >= 2 || e.out_mode != OUT_I8) && try_config(1, false, bufs, 2)) chosen = true;
  if (!chosen) {
    p.row_bytes = full_rb;
    p.k_elems = full_ke;
    p.c_blocks = full_cb;
    p.k_blocks = full_kb;
    return false;
  }
  p.pair = 0;
  p.pair_rows = 0;
  p.sub_blocks = 1;
  p.staging_bytes = staging / p.epi_groups;
  L->smem_bytes = std::max(p.stages * p.stage_bytes + staging + 1024, 120 * 1024);
  L->kind = kind;
  L->cta2 = ctas;
  // workers: one per TPC (pairs) or per SM, all resident at once
  int workers = pair_form ? std::min(sm_count / 2, max_pairs_resident(kind, L->smem_bytes, sm_count)) : sm_count;
  if (workers < 1) return false;
  const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
  const long long units = tiles * p.k_blocks;
  // Splitting tiles pays when whole tiles leave SMs idle in the last wave; the worker that finishes a
  // split tile spends about three K blocks' time on the partial sums.
  const double cost_whole = static_cast<double>((tiles + workers - 1) / workers) * p.k_blocks;
  const double cost_split = static_cast<double>((units + workers - 1) / workers) + 20.0 * p.k_blocks / full_kb;
  const size_t ws_need = static_cast<size_t>(ctas * workers) * kTcBlockM * p.block_n * 4;
  const bool can_split = ws_given && e.sk_ws_bytes >= ws_need && e.sk_flag_count >= 2 * ctas * workers &&
                         units >= 4ll * workers;
  if (split_form) {
    if (!can_split && units < 4ll * workers) workers = static_cast<int>(std::max<long long>(1, units / 4));
    p.streamk = ws_given && e.sk_ws_bytes >= static_cast<size_t>(workers) * kTcBlockM * p.block_n * 4 &&
                        e.sk_flag_count >= 2 * workers
                    ? 1
                    : 0;
    if (!p.streamk) {
      p.row_bytes = full_rb;
      p.k_elems = full_ke;
      p.c_blocks = full_cb;
      p.k_blocks = full_kb;
      L->cta2 = 0;
      return false;
    }
  } else {
    p.streamk = can_split && may_split && (forced_split == 1 || cost_split < 0.95 * cost_whole) ? 1 : 0;
  }
  if (!p.streamk) workers = static_cast<int>(std::min<long long>(workers, tiles));
  p.sk_ws = e.sk_ws;
  p.sk_flags = e.sk_flags;
  L->grid = ctas * workers;
  p.bias = e.bias;
  p.scale = e.scale;
  p.out0 = e.out0;
  p.out1 = e.out1;
  p.outq = e.outq;
  p.res0 = e.res0;
  p.res1 = e.res1;
  p.res_mode = res_mode;
  p.wide = wide ? 1 : 0;
  p.ldo = e.ldo;
  p.out_mode = e.out_mode;
  p.act = e.act;
  p.act_a = e.act_a;
  p.act_b = e.act_b;
  p.out_scale = e.out_scale;
  p.status = e.status;
  p.trace = e.trace;
  p.side_staged = 0;  // (this kernel stores the int8 copies thread by thread)
  p.side_count = e.side_count;
  p.side_ld = e.ldo;
  p.side_q0 = e.side_q[0];
  p.side_q1 = e.side_q[1];
  p.side_scale0 = e.side_scale[0];
  p.side_scale1 = e.side_scale[1];
  L->map_o0 = L->map_o1 = L->map_r0 = L->map_r1 = CUtensorMap{};
  return true;
}

// [M][N] plane seen as a 2-D tensor (N innermost) with boxes of 64 bytes (16 fp32 or 32 bf16)
// x 128 rows, 64-byte swizzle
std::string encode_plane(CUtensorMap* map, const void* base, long long M, int N, long long ld, bool bf16) {
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(M)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * (bf16 ? 2 : 4)};
  const cuuint32_t box[2] = {bf16 ? 32u : 16u, static_cast<cuuint32_t>(kTcBlockM)};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r = g_encode_tiled(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                                    const_cast<void*>(base),
                                    dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                    CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return "cuTensorMapEncodeTiled failed for an output plane with code " + std::to_string(static_cast<int>(r));
  return {};
}

std::string encode_epilogue_maps(TcLaunch* L, const TcEpilogue& e) {
  if (!L->p.tma_store) return {};
  if (e.out_mode == OUT_I8) {
    // [M][N] int8 plane, boxes of 64 columns x 128 rows, 64-byte swizzle
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(L->p.N), static_cast<cuuint64_t>(L->p.M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(e.ldo)};
    const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(kTcBlockM)};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult r = g_encode_tiled(&L->map_o0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, e.outq, dims, strides, box,
                                      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return "cuTensorMapEncodeTiled failed for an int8 output plane with code " + std::to_string(static_cast<int>(r));
    return {};
  }
  const bool ob = e.out_mode == OUT_BF16X2;
  std::string err = encode_plane(&L->map_o0, e.out0, L->p.M, L->p.N, e.ldo, ob);
  if (err.empty() && (e.out_mode == OUT_F32_SPLIT || ob))
    err = encode_plane(&L->map_o1, e.out1, L->p.M, L->p.N, e.ldo, ob);
  if (err.empty() && e.res0 != nullptr) err = encode_plane(&L->map_r0, e.res0, L->p.M, L->p.N, e.ldo, e.res_bf16);
  if (err.empty() && e.res1 != nullptr) err = encode_plane(&L->map_r1, e.res1, L->p.M, L->p.N, e.ldo, e.res_bf16);
  for (int i = 0; i < e.side_count && err.empty() && L->p.side_staged; ++i) {
    // [M][N] int8 plane, boxes of 64 columns x 128 rows, 64-byte swizzle
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(L->p.N), static_cast<cuuint64_t>(L->p.M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(e.ldo)};
    const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(kTcBlockM)};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult r = g_encode_tiled(i ? &L->map_s1 : &L->map_s0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, e.side_q[i], dims,
                                      strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) err = "cuTensorMapEncodeTiled failed for an int8 copy of the result with code " + std::to_string(static_cast<int>(r));
  }
  return err;
}

}  // namespace

int tc_row_bytes(int kind, int channels) {
  if (kind == GEMM_I8) {
    if (channels % 16 != 0) return 0;
    return channels > 64 ? 128 : (channels > 32 ? 64 : 32);
  }
  // bf16 rows: 64 channels when they divide evenly, else 32 per block; a last block that
  // reaches past the tensor is zero-filled by TMA (pixel rows must stay 16-byte multiples)
  if (kind == GEMM_BF16X3) return channels % 64 == 0 ? 128 : (channels % 8 == 0 ? 64 : 0);
  if (channels % 4 != 0) return 0;
  return 128;
}

int tc_k_elems(int kind, int channels) {
  const int rb = tc_row_bytes(kind, channels);
  if (rb == 0) return 0;
  return rb / tc_elem_bytes(kind);
}

std::string tc_plan_conv(TcLaunch* L, int kind, const TcIm2colView& v, const void* w0,
                         const void* w1, int out_channels, const TcEpilogue& e, int sm_count) {
  load_driver_entry_points();
  if (!g_driver_error.empty()) return g_driver_error;
  const int rb = tc_row_bytes(kind, static_cast<int>(v.C));
  if (rb == 0) return "channel count is not addressable by TMA (row not a multiple of 16 bytes)";
  TcGemmParams& p = L->p;
  std::memset(&p, 0, sizeof(p));
  p.row_bytes = rb;
  p.k_elems = rb / tc_elem_bytes(kind);
  p.c_blocks = static_cast<int>((v.C + p.k_elems - 1) / p.k_elems);
  p.k_blocks = v.KH * v.KW * p.c_blocks;
  p.a_im2col = 1;
  p.OH = v.OH;
  p.OW = v.OW;
  p.KW = v.KW;
  p.stride_h = v.stride_conv_h;
  p.stride_w = v.stride_conv_w;
  p.pad_t = v.pad_t;
  p.pad_l = v.pad_l;
  p.dil_h = v.dil_h;
  p.dil_w = v.dil_w;
  const long long M = static_cast<long long>(v.N) * v.OH * v.OW;
  if (M > 0x7fffffffll) return "too many output pixels for one launch";
  L->cta2 = 0;
  if (!finish_plan_workers(L, kind, M, out_channels, e, sm_count, v.C % 64 == 0))
    finish_plan(L, kind, M, out_channels, e, sm_count);
  const uint32_t b_box_rows = static_cast<uint32_t>(L->cta2 == 2 ? p.block_n / 2 : p.block_n);
  const int prb = p.row_bytes;  // the pair plan may have halved the K blocks

  std::string err = encode_im2col(&L->map_a0, kind, v.plane0, v, p.k_elems, prb);
  if (!err.empty()) return err;
  if (tc_planes(kind) == 2) {
    err = encode_im2col(&L->map_a1, kind, v.plane1, v, p.k_elems, prb);
    if (!err.empty()) return err;
  } else {
    L->map_a1 = L->map_a0;
  }
  const uint64_t k_total = static_cast<uint64_t>(p.k_blocks) * p.k_elems;
  err = encode_tiled_2d(&L->map_b0, kind, w0, k_total, out_channels,
                        k_total * elem_bytes(kind), p.k_elems, b_box_rows, prb);
  if (!err.empty()) return err;
  if (tc_planes(kind) == 2) {
    err = encode_tiled_2d(&L->map_b1, kind, w1, k_total, out_channels,
                          k_total * elem_bytes(kind), p.k_elems, b_box_rows, prb);
    if (!err.empty()) return err;
  } else {
    L->map_b1 = L->map_b0;
  }
  return encode_epilogue_maps(L, e);
}

std::string tc_plan_gemm(TcLaunch* L, int kind, const void* a0, const void* a1, long long M, int K,
                         long long lda, const void* w0, const void* w1, int N,
                         const TcEpilogue& e, int sm_count) {
  load_driver_entry_points();
  if (!g_driver_error.empty()) return g_driver_error;
  const int es = elem_bytes(kind);
  if ((lda * es) % 16 != 0) return "row stride of A is not a multiple of 16 bytes";
  if (M > 0x7fffffffll) return "too many rows for one launch";
  TcGemmParams& p = L->p;
  std::memset(&p, 0, sizeof(p));
  p.row_bytes = 128;
  p.k_elems = 128 / es;
  p.c_blocks = (K + p.k_elems - 1) / p.k_elems;
  p.k_blocks = p.c_blocks;
  p.a_im2col = 0;
  p.OH = p.OW = p.KW = 1;
  p.stride_h = p.stride_w = p.dil_h = p.dil_w = 1;
  L->cta2 = 0;
  if (!finish_plan_workers(L, kind, M, N, e, sm_count, K % 64 == 0)) finish_plan(L, kind, M, N, e, sm_count);
  const uint32_t b_box_rows = static_cast<uint32_t>(L->cta2 == 2 ? p.block_n / 2 : p.block_n);
  const int prb = p.row_bytes;  // the pair plan may have halved the K blocks
  std::string err = encode_tiled_2d(&L->map_a0, kind, a0, K, M, lda * es, p.k_elems, kTcBlockM, prb);
  if (!err.empty()) return err;
  if (tc_planes(kind) == 2) {
    err = encode_tiled_2d(&L->map_a1, kind, a1, K, M, lda * es, p.k_elems, kTcBlockM, prb);
    if (!err.empty()) return err;
  } else {
    L->map_a1 = L->map_a0;
  }
  const uint64_t k_total = static_cast<uint64_t>(p.k_blocks) * p.k_elems;
  err = encode_tiled_2d(&L->map_b0, kind, w0, k_total, N, k_total * es, p.k_elems, b_box_rows, prb);
  if (!err.empty()) return err;
  if (tc_planes(kind) == 2) {
    err = encode_tiled_2d(&L->map_b1, kind, w1, k_total, N, k_total * es, p.k_elems, b_box_rows, prb);
    if (!err.empty()) return err;
  } else {
    L->map_b1 = L->map_b0;
  }
  return encode_epilogue_maps(L, e);
}

namespace {

template <int KIND>
cudaError_t prepare_worker_kernel() {
  cudaError_t e = cudaFuncSetAttribute(tc_gemm2_kernel<KIND, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       tc_smem_budget(KIND) + 1024);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(tc_gemm2_kernel<KIND, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             tc_smem_budget(KIND) + 1024);
  return e;
}

cudaError_t prepare_worker_kernels() {
  static PerDeviceOnce once;
  return once.run([] {
    cudaError_t e = prepare_worker_kernel<GEMM_TF32>();
    if (e == cudaSuccess) e = prepare_worker_kernel<GEMM_TF32X3>();
    if (e == cudaSuccess) e = prepare_worker_kernel<GEMM_I8>();
    if (e == cudaSuccess) e = prepare_worker_kernel<GEMM_BF16X3>();
    return e;
  });
}

template <int KIND>
int pairs_resident(int smem_bytes, int sm_count) {
  KernelLaunchConfig wc(sm_count / 2 * 2, kTc2ThreadsTwoEpi, smem_bytes, true, nullptr);
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, tc_gemm2_kernel<KIND, true>, &wc.cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return clusters;
}

// how many CTA pairs of the kernel the device runs at once (no device: as many as there are TPCs)
int max_pairs_resident(int kind, int smem_bytes, int sm_count) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    cudaGetLastError();
    return sm_count / 2;
  }
  if (prepare_worker_kernels() != cudaSuccess) return 0;
  switch (kind) {
    case GEMM_TF32: return pairs_resident<GEMM_TF32>(smem_bytes, sm_count);
    case GEMM_TF32X3: return pairs_resident<GEMM_TF32X3>(smem_bytes, sm_count);
    case GEMM_BF16X3: return pairs_resident<GEMM_BF16X3>(smem_bytes, sm_count);
    default: return pairs_resident<GEMM_I8>(smem_bytes, sm_count);
  }
}

template <int KIND>
cudaError_t launch_workers(const TcLaunch& L, cudaStream_t stream) {
  const bool pair = L.cta2 == 2;
  KernelLaunchConfig wc(L.grid, L.p.epi_groups == 2 ? kTc2ThreadsTwoEpi : kTc2Threads, L.smem_bytes, pair, stream);
  if (pair)
    return cudaLaunchKernelEx(&wc.cfg, tc_gemm2_kernel<KIND, true>, L.p, L.map_a0, L.map_a1, L.map_b0, L.map_b1,
                              L.map_o0, L.map_o1, L.map_r0, L.map_r1);
  return cudaLaunchKernelEx(&wc.cfg, tc_gemm2_kernel<KIND, false>, L.p, L.map_a0, L.map_a1, L.map_b0, L.map_b1,
                            L.map_o0, L.map_o1, L.map_r0, L.map_r1);
}

cudaError_t tc_launch_workers(const TcLaunch& L, cudaStream_t stream) {
  const cudaError_t prep = prepare_worker_kernels();
  if (prep != cudaSuccess) return prep;
  cudaError_t e;
  switch (L.kind) {
    case GEMM_TF32: e = launch_workers<GEMM_TF32>(L, stream); break;
    case GEMM_TF32X3: e = launch_workers<GEMM_TF32X3>(L, stream); break;
    case GEMM_BF16X3: e = launch_workers<GEMM_BF16X3>(L, stream); break;
    default: e = launch_workers<GEMM_I8>(L, stream); break;
  }
  return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace

cudaError_t tc_launch(const TcLaunch& L, cudaStream_t stream) {
  if (L.cta2) return tc_launch_workers(L, stream);
  static PerDeviceOnce attr_once;
  const cudaError_t attr_err = attr_once.run([] {
    const int max_smem = tc_smem_budget(GEMM_TF32) + 1024;  // contents + alignment slack
    cudaError_t e = cudaFuncSetAttribute(tc_gemm_kernel<GEMM_TF32>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tc_gemm_kernel<GEMM_TF32X3>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tc_gemm_kernel<GEMM_I8>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem_budget(GEMM_I8) + 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tc_gemm_kernel<GEMM_BF16X3>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tc_gemm_kernel<GEMM_I8, true>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem_budget(GEMM_I8) + 1024);
    return e;
  });
  if (attr_err != cudaSuccess) return attr_err;
  KernelLaunchConfig lc(L.grid, L.p.epi_groups == 2 ? kTcThreadsTwoEpi : kTcThreads, L.smem_bytes, false, stream);
  cudaError_t e;
  switch (L.kind) {
    case GEMM_TF32:
      e = cudaLaunchKernelEx(&lc.cfg, tc_gemm_kernel<GEMM_TF32>, L.p, L.map_a0, L.map_a1, L.map_b0, L.map_b1, L.map_o0,
                             L.map_o1, L.map_r0, L.map_r1, L.map_s0, L.map_s1);
      break;
    case GEMM_TF32X3:
      e = cudaLaunchKernelEx(&lc.cfg, tc_gemm_kernel<GEMM_TF32X3>, L.p, L.map_a0, L.map_a1, L.map_b0, L.map_b1, L.map_o0,
                             L.map_o1, L.map_r0, L.map_r1, L.map_s0, L.map_s1);
      break;
    case GEMM_BF16X3:
      e = cudaLaunchKernelEx(&lc.cfg, tc_gemm_kernel<GEMM_BF16X3>, L.p, L.map_a0, L.map_a1, L.map_b0, L.map_b1, L.map_o0,
                             L.map_o1, L.map_r0, L.map_r1, L.map_s0, L.map_s1);
      break;
    default:
      // (int8 copies of an fp32 result are written by an instantiation of its own)
      if (L.p.side_count > 0)
        e = cudaLaunchKernelEx(&lc.cfg, tc_gemm_kernel<GEMM_I8, true>, L.p, L.map_a0, L.map_a1, L.map_b0, L.map_b1, L.map_o0,
                               L.map_o1, L.map_r0, L.map_r1, L.map_s0, L.map_s1);
      else
        e = cudaLaunchKernelEx(&lc.cfg, tc_gemm_kernel<GEMM_I8>, L.p, L.map_a0, L.map_a1, L.map_b0, L.map_b1, L.map_o0,
                               L.map_o1, L.map_r0, L.map_r1, L.map_s0, L.map_s1);
      break;
  }
  return e != cudaSuccess ? e : cudaGetLastError();
}

// ------------------------------------------------------------------ patch-resident convolution
namespace {

std::string encode_tiled_4d(CUtensorMap* map, bool bf16, const void* base, int C, int W, int H, int N, uint32_t box_c,
                            uint32_t box_w, uint32_t box_h, CUtensorMapSwizzle swizzle) {
  const cuuint64_t es = bf16 ? 2 : 4;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(W), static_cast<cuuint64_t>(H),
                              static_cast<cuuint64_t>(N)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(C) * es, static_cast<cuuint64_t>(C) * es * W,
                                 static_cast<cuuint64_t>(C) * es * W * H};
  const cuuint32_t box[4] = {box_c, box_w, box_h, 1};
  const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
  const CUresult r = g_encode_tiled(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4,
                                    const_cast<void*>(base), dims, strides,
                                    box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return "cuTensorMapEncodeTiled (4-D) failed with code " + std::to_string(static_cast<int>(r));
  return {};
}

}  // namespace

bool tc_halo_applies(int kind, int C, int KH, int KW, int stride_h, int stride_w, int dil_h, int dil_w, int OH,
                     int OW, int out_channels, int out_mode) {
  if (kind != GEMM_TF32 && kind != GEMM_TF32X3 && kind != GEMM_BF16X3) return false;
  if (stride_h != 1 || stride_w != 1 || dil_h != 1 || dil_w != 1) return false;
  if (KH * KW < 2 || KH > 7 || KW > 7) return false;  // a 1x1 filter has nothing to reuse
  if (C % (kind == GEMM_BF16X3 ? 64 : 32) != 0 || out_channels % 4 != 0 || out_mode == OUT_I8) return false;
  if (out_mode == OUT_BF16X2 && out_channels % 32 != 0) return false;
  const double covered = static_cast<double>((OH + kHaloTileH - 1) / kHaloTileH * kHaloTileH) *
                         ((OW + kHaloTileW - 1) / kHaloTileW * kHaloTileW);
  return static_cast<double>(OH) * OW / covered >= 0.70;
}

std::string tc_plan_conv_halo(TcHaloLaunch* L, int kind, const TcHaloConv& c, const TcEpilogue& e, int sm_count,
                              bool pair) {
  load_driver_entry_points();
  if (!g_driver_error.empty()) return g_driver_error;
  TcHaloParams& p = L->p;
  std::memset(&p, 0, sizeof(p));
  const int planes = tc_planes(kind);
  const bool a_bf16 = kind == GEMM_BF16X3;
  const int res_mode = e.res0 == nullptr ? RES_NONE : (e.res_bf16 ? RES_BF16X2 : (e.res1 != nullptr ? RES_SPLIT : RES_F32));
  const bool out_bf16 = e.out_mode == OUT_BF16X2;
  const bool wide = out_bf16 || res_mode == RES_BF16X2;
  if (wide && (e.out_mode == OUT_F32_SPLIT || e.out_mode == OUT_F32_TF32 || res_mode == RES_SPLIT))
    return "fp32 hi/lo planes cannot be staged together with a bf16-pair tensor";
  if (e.ldo != c.out_channels) return "the patch-resident kernel writes dense channel-last rows";
  p.images = c.images;
  p.OH = c.OH;
  p.OW = c.OW;
  p.N = c.out_channels;
  p.tiles_y = (c.OH + kHaloTileH - 1) / kHaloTileH;
  p.tiles_x = (c.OW + kHaloTileW - 1) / kHaloTileW;
  // an MMA of any N <= 128 costs the same issue time: take the widest tile
  const int step = wide ? 32 : 16;
  const int widest = pair ? 256 : 128;  // a pair's CTA holds half of the weight rows of a tap
  {
    const int n_tiles = (c.out_channels + widest - 1) / widest;
    p.block_n = ((c.out_channels + n_tiles - 1) / n_tiles + step - 1) / step * step;
  }
  p.tiles_n = (c.out_channels + p.block_n - 1) / p.block_n;
  const int ctas = pair ? 2 : 1;
  L->pair = pair ? 1 : 0;
  if (pair && (p.block_n / 2) % 8 != 0) return "a pair's half of the weight tile must be whole 8-row groups";
  p.k_elems = 128 / tc_elem_bytes(kind);
  p.c_blocks = c.C / p.k_elems;
  p.taps = c.KH * c.KW;
  p.KW = c.KW;
  p.pad_t = c.pad_t;
  p.pad_l = c.pad_l;
  p.patch_h = kHaloTileH + c.KH - 1;
  p.patch_w = kHaloTileW + c.KW - 1;
  p.patch_bytes = (p.patch_h * p.patch_w * 128 + 1023) / 1024 * 1024;
  p.b_bytes = ((p.block_n / ctas) * 128 + 1023) / 1024 * 1024;
  p.bias = e.bias;
  p.res_mode = res_mode;
  p.out_mode = e.out_mode;
  p.act = e.act;
  p.act_a = e.act_a;
  p.act_b = e.act_b;
  p.status = e.status;
  p.trace = e.trace;
  const int out_tile = (e.out_mode == OUT_F32_SPLIT || wide ? 2 : 1) * 8192;
  const int fixed = 2 * planes * p.patch_bytes + (res_mode != RES_NONE ? 16384 : 0);
  p.out_bufs = 4;
  const int kTcSmemBudget = 222 * 1024;  // the halo kernel's own static shared memory is ~2 KB
  p.stages = (kTcSmemBudget - fixed - p.out_bufs * out_tile) / (planes * p.b_bytes);
  if (p.stages < 4) {
    p.out_bufs = 2;
    p.stages = (kTcSmemBudget - fixed - p.out_bufs * out_tile) / (planes * p.b_bytes);
  }
  p.stages = std::min(p.stages, kTcMaxStages);
  if (p.stages < 2) return "shared memory cannot hold the patch buffers and two weight stages";
  L->smem_bytes = fixed + p.out_bufs * out_tile + p.stages * planes * p.b_bytes + 1024;
  L->smem_bytes = std::max(L->smem_bytes, 120 * 1024);
  const long long pixel_tiles = static_cast<long long>(c.images) * p.tiles_y * p.tiles_x;
  const long long tiles = ((pixel_tiles + ctas - 1) / ctas) * p.tiles_n;
  if (pixel_tiles * p.tiles_n > 0x7fffffffll) return "too many tiles for one launch";
  L->grid = ctas * static_cast<int>(std::min<long long>(tiles, sm_count / ctas));
  L->kind = kind;

  std::string err = encode_tiled_4d(&L->map_a0, a_bf16, c.in0, c.C, c.W, c.H, c.images, p.k_elems, p.patch_w,
                                    p.patch_h, CU_TENSOR_MAP_SWIZZLE_128B);
  if (err.empty() && planes == 2)
    err = encode_tiled_4d(&L->map_a1, a_bf16, c.in1, c.C, c.W, c.H, c.images, p.k_elems, p.patch_w, p.patch_h,
                          CU_TENSOR_MAP_SWIZZLE_128B);
  if (!err.empty()) return err;
  const uint64_t k_total = static_cast<uint64_t>(p.taps) * p.c_blocks * p.k_elems;
  err = encode_tiled_2d(&L->map_b0, kind, c.w0, k_total, c.out_channels, k_total * tc_elem_bytes(kind), p.k_elems,
                        p.block_n / ctas, 128);
  if (err.empty() && planes == 2)
    err = encode_tiled_2d(&L->map_b1, kind, c.w1, k_total, c.out_channels, k_total * tc_elem_bytes(kind), p.k_elems,
                          p.block_n / ctas, 128);
  if (!err.empty()) return err;
  // outputs and residuals: [image][OH][OW][N], tiles of 64 bytes of channels x 8 x 16 pixels, 64-byte swizzle
  auto plane = [&](CUtensorMap* map, const void* base, bool bf16) {
    return encode_tiled_4d(map, bf16, base, c.out_channels, c.OW, c.OH, c.images, bf16 ? 32 : 16, kHaloTileW,
                           kHaloTileH, CU_TENSOR_MAP_SWIZZLE_64B);
  };
  err = plane(&L->map_o0, e.out0, out_bf16);
  if (err.empty() && (e.out_mode == OUT_F32_SPLIT || out_bf16)) err = plane(&L->map_o1, e.out1, out_bf16);
  if (err.empty() && e.res0 != nullptr) err = plane(&L->map_r0, e.res0, e.res_bf16);
  if (err.empty() && e.res1 != nullptr) err = plane(&L->map_r1, e.res1, e.res_bf16);
  return err;
}

cudaError_t tc_launch_halo(const TcHaloLaunch& L, cudaStream_t stream) {
  static PerDeviceOnce attr_once;
  const cudaError_t attr_err = attr_once.run([] {
    const int max_smem = 223 * 1024;
    cudaError_t e = cudaFuncSetAttribute(tc_conv_halo_kernel<GEMM_TF32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         max_smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tc_conv_halo_kernel<GEMM_TF32X3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               max_smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tc_conv_halo_kernel<GEMM_BF16X3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               max_smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tc_conv_halo_kernel<GEMM_TF32, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               max_smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tc_conv_halo_kernel<GEMM_TF32X3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               max_smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tc_conv_halo_kernel<GEMM_BF16X3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               max_smem);
    return e;
  });
  if (attr_err != cudaSuccess) return attr_err;
  KernelLaunchConfig lc(L.grid, kHaloThreads, L.smem_bytes, L.pair != 0, stream);
  cudaError_t e;
#define NB_LAUNCH_HALO(KIND, PAIRED)                                                                             \
  e = cudaLaunchKernelEx(&lc.cfg, tc_conv_halo_kernel<KIND, PAIRED>, L.p, L.map_a0, L.map_a1, L.map_b0, L.map_b1, \
                         L.map_o0, L.map_o1, L.map_r0, L.map_r1)
  if (L.kind == GEMM_BF16X3) {
    if (L.pair) NB_LAUNCH_HALO(GEMM_BF16X3, true);
    else NB_LAUNCH_HALO(GEMM_BF16X3, false);
  } else if (L.kind == GEMM_TF32X3) {
    if (L.pair) NB_LAUNCH_HALO(GEMM_TF32X3, true);
    else NB_LAUNCH_HALO(GEMM_TF32X3, false);
  } else {
    if (L.pair) NB_LAUNCH_HALO(GEMM_TF32, true);
    else NB_LAUNCH_HALO(GEMM_TF32, false);
  }
#undef NB_LAUNCH_HALO
  return e != cudaSuccess ? e : cudaGetLastError();
}

// ------------------------------------------------------------------ depthwise + projection
namespace {

struct DwProjShape {
  int block_n = 0, tiles_n = 0, stages = 0, out_bufs = 0, patches = 0, b_bytes = 0, x_plane_bytes = 0, x_row_bytes = 64, x_bufs = 0, smem = 0;
  bool ok = false;
};

// Shared-memory plan of tc_dw_project_kernel.  expand: the expand layer is fused in (input patches as bf16 planes
// of 64-byte rows, one fp32 patch per depthwise group, the block's expand weights beside its projection weights in
// every ring stage, the expand bias beside the depthwise table).
DwProjShape dw_project_shape(int N, int out_mode, int res_mode, int C, int stride, bool expand, int cin = 32) {
  DwProjShape r;
  const bool wide = out_mode == OUT_BF16X2 || res_mode == RES_BF16X2;
  if (out_mode != OUT_BF16X2 && out_mode != OUT_F32) return r;
  if (wide && res_mode == RES_SPLIT) return r;
  if (stride != 1 && stride != 2) return r;
  if (stride == 2 && !expand) return r;  // (patches loaded by TMA are built for stride 1 only)
  const int step = wide ? 32 : 16;
  const int n_tiles = (N + 255) / 256;
  r.block_n = ((N + n_tiles - 1) / n_tiles + step - 1) / step * step;
  if (r.block_n > 256 || r.block_n % 16 != 0) return r;
  if (expand && r.block_n > 128) return r;  // (the expand accumulators take the TMEM columns past two 128-column ones)
  r.tiles_n = (N + r.block_n - 1) / r.block_n;
  r.b_bytes = (r.block_n * 64 + 1023) / 1024 * 1024;
  const int out_tile = wide ? 16384 : 8192;
  const int budget = 222 * 1024;  // the kernel's own static shared memory is ~2 KB
  const int c_pad = (C + kDwpChannels - 1) / kDwpChannels * kDwpChannels;
  const int table = (c_pad * (expand ? 11 : 10) * 4 + 1023) / 1024 * 1024;  // depthwise filter and bias (+ expand bias)
  const int stage = 2 * r.b_bytes + (expand ? 4096 : 0);
  r.x_row_bytes = cin <= 16 ? 32 : 64;
  r.x_plane_bytes = expand ? (dwp_patch_pixels(stride) * r.x_row_bytes + 1023) / 1024 * 1024 : 0;
  // Deep patch ring first (a patch load outlasts one block's arithmetic), then three weight stages, then
  // output staging tiles; the last resort is two of each.  With the expand layer: two input patch buffers if they
  // fit, and never fewer than three stages (the expand MMAs run two blocks ahead of the projection's).
  for (int min_stages : {4, 3, 2}) {
    if (expand ? min_stages < 3 : min_stages > 3) continue;  // (without the expand layer three stages are plenty)
    for (int x_bufs : {2, 1}) {
      if (!expand && x_bufs != 2) continue;
      // (an even ring only: the two depthwise groups take alternate blocks, so with an even depth a slot always
      // belongs to the same group, which waits for its phases in order; with three slots a slot would alternate
      // between the groups, a group would wait for every second phase of it, and a parity wait cannot tell a
      // phase from the one two before it: a load delayed past a whole block's arithmetic let a group read a stale
      // patch, about once in 10^5 loads with the L2 flushed)
      for (int patches : {4, 2}) {
        if (expand && patches != 2) continue;
        for (int bufs : {4, 3, 2}) {
          if (expand && bufs == 4) continue;
          const int fixed = (expand ? x_bufs * 2 * r.x_plane_bytes : 0) + patches * dwp_patch_bytes(stride) +
                            2 * 2 * dwp_a_plane_bytes(stride) + (res_mode != RES_NONE ? 16384 : 0) + table;
          const int stages = std::min(kDwpMaxStages, (budget - fixed - bufs * out_tile) / stage);
          if (stages >= min_stages) {
            r.stages = stages;
            r.out_bufs = bufs;
            r.patches = patches;
            r.x_bufs = expand ? x_bufs : 0;
            r.smem = fixed + bufs * out_tile + stages * stage + 1024;
            r.ok = true;
            return r;
          }
        }
      }
    }
  }
  return r;
}

// an image that fills less than 60 % of its tiles (7 x 7 fills 38 % of a 16 x 8 tile) is faster as separate layers
bool dw_project_fills(int H, int W, int stride) {
  const int th = dwp_tile_h(stride);
  const int tiles = ((H + th - 1) / th) * ((W + kDwpTileW - 1) / kDwpTileW);
  return env_int("NCNN_B200_FUSE_DW", 1) >= 2 || static_cast<long long>(H) * W * 10 >= 6ll * tiles * th * kDwpTileW;
}

}  // namespace

bool tc_dw_project_applies(int C, int N, int H, int W, int out_mode, bool has_res, bool res_bf16) {
  if (C % 4 != 0 || C < 8 || N % 8 != 0 || H < 1 || W < 1) return false;
  if (!dw_project_fills(H, W, 1)) return false;
  const int res_mode = !has_res ? RES_NONE : (res_bf16 ? RES_BF16X2 : RES_F32);
  if (out_mode == OUT_F32 && N % 4 != 0) return false;
  return dw_project_shape(N, out_mode, res_mode, C, 1, false).ok;
}

bool tc_block_applies(int Cin, int C, int N, int OH, int OW, int stride, bool has_res) {
  if (Cin < 8 || Cin > 32 || Cin % 8 != 0 || C % 8 != 0 || C < 32 || N % 8 != 0 || OH < 1 || OW < 1) return false;
  if (has_res && stride != 1) return false;
  if (!dw_project_fills(OH, OW, stride)) return false;
  // whatever formats the planner gives the output and the residual later
  for (int out_mode : {OUT_F32, OUT_BF16X2})
    for (int res_mode : {RES_NONE, RES_F32, RES_BF16X2}) {
      if (!has_res && res_mode != RES_NONE) continue;
      if (has_res && res_mode == RES_NONE) continue;
      if (!dw_project_shape(N, out_mode, res_mode, C, stride, true, Cin).ok) return false;
    }
  return true;
}

std::string tc_plan_dw_project(TcDwProjLaunch* L, const TcDwProjConv& c, const TcEpilogue& e, int sm_count) {
  load_driver_entry_points();
  if (!g_driver_error.empty()) return g_driver_error;
  TcDwProjParams& p = L->p;
  std::memset(&p, 0, sizeof(p));
  const int res_mode = e.res0 == nullptr ? RES_NONE : (e.res_bf16 ? RES_BF16X2 : (e.res1 != nullptr ? RES_SPLIT : RES_F32));
  const bool expand = c.ex_w0 != nullptr;
  const int stride = c.stride;
  const DwProjShape shape = dw_project_shape(c.out_channels, e.out_mode, res_mode, c.C, stride, expand, expand ? c.Cin : 32);
  if (!shape.ok) return "the fused depthwise + projection kernel does not take this output format, width or stride";
  if (e.ldo != c.out_channels) return "the fused depthwise + projection kernel writes dense channel-last rows";
  const int x_channels = expand ? c.Cin : c.C;
  if ((reinterpret_cast<uintptr_t>(c.x) & 15) != 0 || (static_cast<size_t>(x_channels) * (expand ? 2 : 4)) % 16 != 0 ||
      (expand && (c.x1 == nullptr || (reinterpret_cast<uintptr_t>(c.x1) & 15) != 0)))
    return "input rows of the fused kernel must be 16-byte aligned";
  const bool out_bf16 = e.out_mode == OUT_BF16X2;
  const int th = dwp_tile_h(stride);
  p.images = c.images;
  p.H = c.H;
  p.W = c.W;
  p.Hin = c.Hin;
  p.Win = c.Win;
  p.C = c.C;
  p.N = c.out_channels;
  p.tiles_y = (c.H + th - 1) / th;
  p.tiles_x = (c.W + kDwpTileW - 1) / kDwpTileW;
  p.block_n = shape.block_n;
  p.tiles_n = shape.tiles_n;
  p.c_blocks = (c.C + kDwpChannels - 1) / kDwpChannels;
  p.pad_t = c.pad_t;
  p.pad_l = c.pad_l;
  p.stages = shape.stages;
  p.patch_bufs = shape.patches;
  p.b_bytes = shape.b_bytes;
  p.out_bufs = shape.out_bufs;
  p.dw_weights = c.dw_weights;
  p.dw_bias = c.dw_bias;
  p.dw_act = c.dw_act;
  p.dw_act_a = c.dw_act_a;
  p.dw_act_b = c.dw_act_b;
  p.Cin = expand ? c.Cin : 0;
  p.x_plane_bytes = shape.x_plane_bytes;
  p.x_row_bytes = shape.x_row_bytes;
  p.x_bufs = shape.x_bufs;
  p.ex_ksteps = expand ? (shape.x_row_bytes == 32 ? 1 : (c.Cin + 15) / 16) : 0;
  p.ex_bias = c.ex_bias;
  p.ex_act = c.ex_act;
  p.ex_act_a = c.ex_act_a;
  p.ex_act_b = c.ex_act_b;
  p.bias = e.bias;
  p.res_mode = res_mode;
  p.out_mode = e.out_mode;
  p.act = e.act;
  p.act_a = e.act_a;
  p.act_b = e.act_b;
  p.status = e.status;
  L->stride = stride;
  L->expand = expand;
  L->smem_bytes = std::max(shape.smem, 120 * 1024);
  const long long tiles = static_cast<long long>(c.images) * p.tiles_y * p.tiles_x * p.tiles_n;
  if (tiles > 0x7fffffffll) return "too many tiles for one launch";
  L->grid = static_cast<int>(std::min<long long>(tiles, sm_count));
  // input patches, [image][Hin][Win][channels], boxes of 32 channels x patch width x patch height: fp32 and dense
  // in shared memory for the depthwise filter; with the expand layer fused in, the bf16 planes of the block's input
  // as 64-byte-swizzled operand rows (channels past Cin read as zero)
  const uint32_t x_box = expand ? static_cast<uint32_t>(shape.x_row_bytes / 2) : kDwpChannels;
  const CUtensorMapSwizzle x_swizzle = !expand ? CU_TENSOR_MAP_SWIZZLE_NONE
                                               : (shape.x_row_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B);
  std::string err = encode_tiled_4d(&L->map_x, expand, c.x, x_channels, c.Win, c.Hin, c.images, x_box, dwp_patch_w(stride),
                                    dwp_patch_h(stride), x_swizzle);
  if (err.empty() && expand)
    err = encode_tiled_4d(&L->map_x1, true, c.x1, x_channels, c.Win, c.Hin, c.images, x_box, dwp_patch_w(stride),
                          dwp_patch_h(stride), x_swizzle);
  // expand weights: [C][32] bf16 per plane (64-byte pitch), one block of 32 rows per copy, as many K columns as the rows hold
  if (err.empty() && expand) err = encode_tiled_2d(&L->map_e0, GEMM_BF16X3, c.ex_w0, 32, c.C, 64, x_box, kDwpChannels, shape.x_row_bytes);
  if (err.empty() && expand) err = encode_tiled_2d(&L->map_e1, GEMM_BF16X3, c.ex_w1, 32, c.C, 64, x_box, kDwpChannels, shape.x_row_bytes);
  if (!err.empty()) return err;
  const uint64_t k_total = static_cast<uint64_t>(p.c_blocks) * kDwpChannels;
  err = encode_tiled_2d(&L->map_b0, GEMM_BF16X3, c.w0, k_total, c.out_channels, k_total * 2, kDwpChannels, p.block_n, 64);
  if (err.empty())
    err = encode_tiled_2d(&L->map_b1, GEMM_BF16X3, c.w1, k_total, c.out_channels, k_total * 2, kDwpChannels, p.block_n, 64);
  if (!err.empty()) return err;
  auto plane = [&](CUtensorMap* map, const void* base, bool bf16) {
    return encode_tiled_4d(map, bf16, base, c.out_channels, c.W, c.H, c.images, bf16 ? 32 : 16, kDwpTileW, th,
                           CU_TENSOR_MAP_SWIZZLE_64B);
  };
  err = plane(&L->map_o0, e.out0, out_bf16);
  if (err.empty() && out_bf16) err = plane(&L->map_o1, e.out1, true);
  if (err.empty() && e.res0 != nullptr) err = plane(&L->map_r0, e.res0, e.res_bf16);
  if (err.empty() && e.res1 != nullptr) err = plane(&L->map_r1, e.res1, e.res_bf16);
  return err;
}

cudaError_t tc_launch_dw_project(const TcDwProjLaunch& L, cudaStream_t stream) {
  static PerDeviceOnce attr_once;
  const cudaError_t attr_err = attr_once.run([] {
    cudaError_t e = cudaFuncSetAttribute(tc_dw_project_kernel<GEMM_BF16X3, 1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tc_dw_project_kernel<GEMM_BF16X3, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tc_dw_project_kernel<GEMM_BF16X3, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
    return e;
  });
  if (attr_err != cudaSuccess) return attr_err;
  KernelLaunchConfig lc(L.grid, kDwpThreads, L.smem_bytes, false, stream);
  cudaError_t e;
  if (!L.expand)
    e = cudaLaunchKernelEx(&lc.cfg, tc_dw_project_kernel<GEMM_BF16X3, 1, false>, L.p, L.map_x, L.map_x1, L.map_e0, L.map_e1, L.map_b0, L.map_b1, L.map_o0, L.map_o1, L.map_r0, L.map_r1);
  else if (L.stride == 1)
    e = cudaLaunchKernelEx(&lc.cfg, tc_dw_project_kernel<GEMM_BF16X3, 1, true>, L.p, L.map_x, L.map_x1, L.map_e0, L.map_e1, L.map_b0, L.map_b1, L.map_o0, L.map_o1, L.map_r0, L.map_r1);
  else
    e = cudaLaunchKernelEx(&lc.cfg, tc_dw_project_kernel<GEMM_BF16X3, 2, true>, L.p, L.map_x, L.map_x1, L.map_e0, L.map_e1, L.map_b0, L.map_b1, L.map_o0, L.map_o1, L.map_r0, L.map_r1);
  return e != cudaSuccess ? e : cudaGetLastError();
}

float tf32_round_host(float x) {
  // round to nearest, ties away from zero, onto 10 explicit mantissa bits
  uint32_t u;
  std::memcpy(&u, &x, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return x;
  u += 0x1000u;
  u &= 0xffffe000u;
  float r;
  std::memcpy(&r, &u, 4);
  return r;
}

void tc_pack_weights_f32(int kind, const float* w, int O, int I, int KH, int KW, int k_elems,
                         std::vector<float>* hi, std::vector<float>* lo) {
  const int c_blocks = (I + k_elems - 1) / k_elems;
  const size_t cpad = static_cast<size_t>(c_blocks) * k_elems;
  const size_t k_total = static_cast<size_t>(KH) * KW * cpad;
  hi->assign(static_cast<size_t>(O) * k_total, 0.0f);
  if (lo != nullptr) lo->assign(kind == GEMM_TF32X3 ? hi->size() : 0, 0.0f);
  for (int o = 0; o < O; ++o)
    for (int i = 0; i < I; ++i)
      for (int kh = 0; kh < KH; ++kh)
        for (int kw = 0; kw < KW; ++kw) {
          const float v = w[((static_cast<size_t>(o) * I + i) * KH + kh) * KW + kw];
          const size_t dst = o * k_total + (static_cast<size_t>(kh) * KW + kw) * cpad + i;
          const float h = tf32_round_host(v);
          (*hi)[dst] = h;
          if (kind == GEMM_TF32X3 && lo != nullptr) (*lo)[dst] = v - h;
        }
}

uint16_t bf16_round_host(float x) {
  // round to nearest even onto 7 explicit mantissa bits; NaN stays NaN
  uint32_t u;
  std::memcpy(&u, &x, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return static_cast<uint16_t>((u >> 16) | ((u & 0xffffu) ? 0x40u : 0u));
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

float bf16_to_float_host(uint16_t h) {
  const uint32_t u = static_cast<uint32_t>(h) << 16;
  float r;
  std::memcpy(&r, &u, 4);
  return r;
}

void tc_pack_weights_bf16x2(const float* w, int O, int I, int KH, int KW, int k_elems,
                            std::vector<uint16_t>* hi, std::vector<uint16_t>* mid) {
  const int c_blocks = (I + k_elems - 1) / k_elems;
  const size_t cpad = static_cast<size_t>(c_blocks) * k_elems;
  const size_t k_total = static_cast<size_t>(KH) * KW * cpad;
  hi->assign(static_cast<size_t>(O) * k_total, 0);
  mid->assign(hi->size(), 0);
  for (int o = 0; o < O; ++o)
    for (int i = 0; i < I; ++i)
      for (int kh = 0; kh < KH; ++kh)
        for (int kw = 0; kw < KW; ++kw) {
          const float v = w[((static_cast<size_t>(o) * I + i) * KH + kh) * KW + kw];
          const size_t dst = o * k_total + (static_cast<size_t>(kh) * KW + kw) * cpad + i;
          const uint16_t h = bf16_round_host(v);
          (*hi)[dst] = h;
          (*mid)[dst] = bf16_round_host(v - bf16_to_float_host(h));
        }
}

void tc_pack_weights_i8(const int8_t* w, int O, int I, int KH, int KW, int k_elems,
                        std::vector<int8_t>* packed) {
  const int c_blocks = (I + k_elems - 1) / k_elems;
  const size_t cpad = static_cast<size_t>(c_blocks) * k_elems;
  const size_t k_total = static_cast<size_t>(KH) * KW * cpad;
  packed->assign(static_cast<size_t>(O) * k_total, 0);
  for (int o = 0; o < O; ++o)
    for (int i = 0; i < I; ++i)
      for (int kh = 0; kh < KH; ++kh)
        for (int kw = 0; kw < KW; ++kw)
          (*packed)[o * k_total + (static_cast<size_t>(kh) * KW + kw) * cpad + i] =
              w[((static_cast<size_t>(o) * I + i) * KH + kh) * KW + kw];
}

// ------------------------------------------------------------------------------ stem kernel
std::string tc_plan_stem(TcStemLaunch* L, const TcStemConv& c, const TcEpilogue& e, int sm_count) {
  load_driver_entry_points();
  if (!g_driver_error.empty()) return g_driver_error;
  TcStemParams& p = L->p;
  const int N = c.out_channels;
  if (c.row_bytes % 128 != 0 || c.row_bytes / 128 > 256) return "padded input rows must be multiples of 128 bytes";
  if (c.OW > kTcBlockM || c.OW < 1) return "an output row must fit one 128-row tile";
  if (N % 16 != 0 || N > 128) return "output channels must be a multiple of 16, at most 128";
  if (c.KH < 1 || c.KH > 16) return "filter height out of range";
  if (e.res0 != nullptr) return "the stem kernel takes no residual";
  const bool i8 = c.kind == GEMM_I8;
  if (c.kind != GEMM_BF16X3 && !i8) return "the stem kernel takes bf16-pair or int8 operands";
  const bool i8_out = e.out_mode == OUT_I8;
  if (e.out_mode != OUT_F32 && !(e.out_mode == OUT_BF16X2 && !i8) && !(i8_out && i8))
    return "output format not handled by the stem kernel";
  const bool bf16_out = e.out_mode == OUT_BF16X2;
  if (bf16_out && N % 32 != 0) return "bf16-pair results need channels in multiples of 32";
  if (i8_out && N % 64 != 0) return "int8 results need channels in multiples of 64";
  if (e.ldo != N || (reinterpret_cast<uintptr_t>(e.out0) & 15) != 0 || (reinterpret_cast<uintptr_t>(e.out1) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(e.outq) & 15) != 0)
    return "the stem kernel writes dense, 16-byte aligned rows";
  const int planes = i8 ? 1 : 2;
  L->kind = c.kind;
  if ((c.OW - 1) * 16 + 64 > c.row_bytes) return "padded rows are shorter than the last window";
  p.tiles = c.images * c.OH;
  p.OH = c.OH;
  p.OW = c.OW;
  p.KH = c.KH;
  p.stride_h = c.stride_h;
  p.pad_t = c.pad_t;
  p.N = N;
  p.M = c.images * c.OH * c.OW;
  p.row_bytes = c.row_bytes;
  // the last filter row's windows of tile rows up to 127 reach 127*16 + 64 bytes into (and past) it
  p.a_plane_bytes = ((c.KH - 1) * c.row_bytes + (kTcBlockM - 1) * 16 + 64 + 1023) / 1024 * 1024;
  p.a_plane_bytes = std::max(p.a_plane_bytes, (c.KH * c.row_bytes + 1023) / 1024 * 1024);
  p.b_slot = (N * 64 + 1023) / 1024 * 1024;
  p.bias = e.bias;
  p.scale = e.scale;
  p.out_scale = e.out_scale;
  p.out_mode = e.out_mode;
  p.act = e.act;
  p.act_a = e.act_a;
  p.act_b = e.act_b;
  p.status = e.status;
  p.wide = !i8_out && (bf16_out || N % 32 == 0) ? 1 : 0;
  const int out_tile = p.wide ? 16384 : 8192;
  const int budget = tc_smem_budget(c.kind);
  const int weights = c.KH * planes * p.b_slot;
  const int stage = planes * p.a_plane_bytes;
  // the epilogue of a 64-channel row takes longer than its 42 MMAs: two epilogue groups when they fit, and
  // staging tiles before a third row stage (a stage holds a whole tile's input: two are a double buffer)
  p.epi_groups = 0;
  for (int groups : {2, 1}) {
    for (int bufs : {4, 3, 2}) {
      if ((budget - weights - groups * bufs * out_tile) / stage >= 2) {
        p.epi_groups = groups;
        p.out_bufs = bufs;
        break;
      }
    }
    if (p.epi_groups != 0) break;
  }
  if (p.epi_groups == 0) return "shared memory cannot hold the weights, two row stages and the staging tiles";
  if (p.tiles < 2 * sm_count) p.epi_groups = 1;
  p.staging_bytes = p.out_bufs * out_tile;
  p.stages = std::min(kStemMaxStages, (budget - weights - p.epi_groups * p.staging_bytes) / stage);
  // four accumulators of 64 columns where they fit, and then a second MMA-issuing warp for alternate tiles
  p.accs = N <= 64 ? 4 : 2;
  p.issuers = p.accs == 4 && env_int("NCNN_B200_STEM_ISSUERS", 2) >= 2 ? 2 : 1;
  L->smem_bytes = weights + p.stages * stage + p.epi_groups * p.staging_bytes + 1024;
  L->smem_bytes = std::max(L->smem_bytes, 120 * 1024);  // one CTA per SM: each allocates tensor memory
  L->grid = std::min(p.tiles, sm_count);
  // input planes: [images][H][row_bytes / 128][64 bf16], KH whole rows per copy, dense in shared memory
  auto rows_map = [&](CUtensorMap* map, const void* base) -> std::string {
    const cuuint64_t line = i8 ? 128 : 64;  // elements per 128-byte line
    const cuuint64_t dims[4] = {line, static_cast<cuuint64_t>(c.row_bytes / 128), static_cast<cuuint64_t>(c.H),
                                static_cast<cuuint64_t>(c.images)};
    const cuuint64_t strides[3] = {128, static_cast<cuuint64_t>(c.row_bytes),
                                   static_cast<cuuint64_t>(c.row_bytes) * c.H};
    const cuuint32_t box[4] = {static_cast<cuuint32_t>(line), static_cast<cuuint32_t>(c.row_bytes / 128),
                               static_cast<cuuint32_t>(c.KH), 1};
    const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
    const CUresult r = g_encode_tiled(map, i8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                                      const_cast<void*>(base), dims, strides, box, elem_strides,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return "cuTensorMapEncodeTiled failed for the stem input rows with code " + std::to_string(static_cast<int>(r));
    return {};
  };
  std::string err = rows_map(&L->map_a0, c.in0);
  if (err.empty() && !i8) err = rows_map(&L->map_a1, c.in1);
  if (!err.empty()) return err;
  const uint64_t window = i8 ? 64 : 32;  // elements of one 64-byte window
  const uint64_t k_total = static_cast<uint64_t>(c.KH) * window;
  err = encode_tiled_2d(&L->map_b0, c.kind, c.w0, k_total, N, k_total * (i8 ? 1 : 2), static_cast<uint32_t>(window), N, 64);
  if (err.empty() && !i8)
    err = encode_tiled_2d(&L->map_b1, c.kind, c.w1, k_total, N, k_total * 2, static_cast<uint32_t>(window), N, 64);
  if (!err.empty()) return err;
  // outputs: [pixels][N], boxes of 64 bytes x OW rows (one output row of the image), 64-byte swizzle
  auto plane = [&](CUtensorMap* map, const void* base) -> std::string {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(p.M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(N) * (i8_out ? 1 : (bf16_out ? 2 : 4))};
    const cuuint32_t box[2] = {i8_out ? 64u : (bf16_out ? 32u : 16u), static_cast<cuuint32_t>(c.OW)};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult r = g_encode_tiled(map, i8_out ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : (bf16_out ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32),
                                      2, const_cast<void*>(base), dims, strides, box, elem_strides,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return "cuTensorMapEncodeTiled failed for a stem output plane with code " + std::to_string(static_cast<int>(r));
    return {};
  };
  err = plane(&L->map_o0, i8_out ? static_cast<const void*>(e.outq) : static_cast<const void*>(e.out0));
  if (err.empty() && bf16_out) err = plane(&L->map_o1, e.out1);
  return err;
}

cudaError_t tc_launch_stem(const TcStemLaunch& L, cudaStream_t stream) {
  static PerDeviceOnce attr_once;
  const cudaError_t attr_err = attr_once.run([] {
    cudaError_t e = cudaFuncSetAttribute(tc_stem_kernel<GEMM_BF16X3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         tc_smem_budget(GEMM_BF16X3) + 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tc_stem_kernel<GEMM_I8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               tc_smem_budget(GEMM_I8) + 1024);
    return e;
  });
  if (attr_err != cudaSuccess) return attr_err;
  KernelLaunchConfig lc(L.grid, kStemThreads, L.smem_bytes, false, stream);
  cudaError_t e;
  if (L.kind == GEMM_I8)
    e = cudaLaunchKernelEx(&lc.cfg, tc_stem_kernel<GEMM_I8>, L.p, L.map_a0, L.map_a1, L.map_b0, L.map_b1, L.map_o0, L.map_o1);
  else
    e = cudaLaunchKernelEx(&lc.cfg, tc_stem_kernel<GEMM_BF16X3>, L.p, L.map_a0, L.map_a1, L.map_b0, L.map_b1, L.map_o0,
                           L.map_o1);
  return e != cudaSuccess ? e : cudaGetLastError();
}

constexpr int kStemPoolMaxSmem = 218 * 1024;  // dynamic shared memory the stem + pooling kernel may ask for

std::string tc_plan_stem_pool(TcStemPoolLaunch* L, const TcStemConv& c, const TcEpilogue& e_in, int pooled_h, int pooled_w, int sm_count) {
  const bool i8 = c.kind == GEMM_I8;
  if (!(c.kind == GEMM_BF16X3 && e_in.out_mode == OUT_BF16X2) && !(i8 && e_in.out_mode == OUT_F32))
    return "the stem + pooling kernel writes bf16 pairs from bf16 pairs, or fp32 from int8";
  const int N = c.out_channels;
  if (N != 32 && N != 64) return "the stem + pooling kernel takes 32 or 64 output channels";
  if (e_in.act != ACT_NONE && e_in.act != ACT_RELU && e_in.act != ACT_CLIP) return "the stem + pooling kernel applies no activation but ReLU and clip";
  if (c.OH != 2 * pooled_h || c.OW != 2 * pooled_w || pooled_h < 1 || pooled_w < 1) return "the pooled extent must be half the convolution's";
  if (e_in.side_count > 1 || (e_in.side_count == 1 && (!i8 || N != 64))) return "one int8 copy of 64 channels at most";
  // the convolution part is planned as for tc_stem_kernel (validation, input and weight maps, operand geometry);
  // the int8 copy belongs to the pooled tensor
  TcEpilogue e = e_in;
  e.side_count = 0;
  TcStemLaunch conv;
  std::string err = tc_plan_stem(&conv, c, e, sm_count);
  if (!err.empty()) return err;
  const int planes = i8 ? 1 : 2;
  TcStemPoolParams& pp = L->pp;
  pp.s = conv.p;
  pp.images = c.images;
  pp.POH = pooled_h;
  pp.POW = pooled_w;
  pp.ring_row_bytes = (c.OW * N * 4 + 1023) / 1024 * 1024;
  pp.stage_tile_bytes = (pooled_w * 64 + 1023) / 1024 * 1024;
  pp.has_side = e_in.side_count;
  pp.side_scale = e_in.side_count ? e_in.side_scale[0] : 0.0f;
  const int weights = c.KH * planes * conv.p.b_slot;
  const int stage = planes * conv.p.a_plane_bytes;
  // staging tiles of 64-byte rows: bf16 pairs 2 planes x N / 32, fp32 N / 16 (+ one for the int8 copy)
  const int tiles = i8 ? N / 16 + pp.has_side : 2 * (N / 32);
  const int fixed = weights + pp.ring_row_bytes + tiles * pp.stage_tile_bytes + 1024;
  pp.row_stages = fixed + 4 * stage <= kStemPoolMaxSmem ? 4 : 2;
  L->smem_bytes = fixed + pp.row_stages * stage;
  if (L->smem_bytes > kStemPoolMaxSmem) return "shared memory cannot hold the weights, two row stages and a result row";
  L->smem_bytes = std::max(L->smem_bytes, 120 * 1024);  // one CTA per SM: each allocates tensor memory
  const long long pooled_rows = static_cast<long long>(c.images) * pooled_h;
  if (pooled_rows * pooled_w > 0x7fffffffll) return "too many pooled pixels for one launch";
  L->grid = static_cast<int>(std::min<long long>(pooled_rows, sm_count));
  L->kind = c.kind;
  L->map_a0 = conv.map_a0;
  L->map_a1 = conv.map_a1;
  L->map_b0 = conv.map_b0;
  L->map_b1 = conv.map_b1;
  const uint64_t pixels = static_cast<uint64_t>(pooled_rows) * pooled_w;
  if (i8) {
    // pooled result: [pooled pixels][N] fp32, boxes of 16 channels x one pooled row; the int8 copy in one box
    err = encode_tiled_2d(&L->map_o0, GEMM_TF32, e.out0, N, pixels, static_cast<uint64_t>(N) * 4, 16, static_cast<uint32_t>(pooled_w), 64);
    if (err.empty() && pp.has_side)
      err = encode_tiled_2d(&L->map_o1, GEMM_I8, e_in.side_q[0], N, pixels, static_cast<uint64_t>(N), 64, static_cast<uint32_t>(pooled_w), 64);
    return err;
  }
  // pooled result: [pooled pixels][N] bf16 per plane, boxes of 32 channels x one pooled row, 64-byte swizzle
  err = encode_tiled_2d(&L->map_o0, GEMM_BF16X3, e.out0, N, pixels, static_cast<uint64_t>(N) * 2, 32, static_cast<uint32_t>(pooled_w), 64);
  if (err.empty())
    err = encode_tiled_2d(&L->map_o1, GEMM_BF16X3, e.out1, N, pixels, static_cast<uint64_t>(N) * 2, 32, static_cast<uint32_t>(pooled_w), 64);
  return err;
}

cudaError_t tc_launch_stem_pool(const TcStemPoolLaunch& L, cudaStream_t stream) {
  static PerDeviceOnce attr_once;
  const cudaError_t attr_err = attr_once.run([] {
    cudaError_t e = cudaFuncSetAttribute(tc_stem_pool_kernel<GEMM_BF16X3>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStemPoolMaxSmem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tc_stem_pool_kernel<GEMM_I8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStemPoolMaxSmem);
    return e;
  });
  if (attr_err != cudaSuccess) return attr_err;
  KernelLaunchConfig lc(L.grid, kStemPoolThreads, L.smem_bytes, false, stream);
  const cudaError_t e =
      L.kind == GEMM_I8 ? cudaLaunchKernelEx(&lc.cfg, tc_stem_pool_kernel<GEMM_I8>, L.pp, L.map_a0, L.map_a1, L.map_b0, L.map_b1, L.map_o0, L.map_o1)
                        : cudaLaunchKernelEx(&lc.cfg, tc_stem_pool_kernel<GEMM_BF16X3>, L.pp, L.map_a0, L.map_a1, L.map_b0, L.map_b1,
                                             L.map_o0, L.map_o1);
  return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace nb
