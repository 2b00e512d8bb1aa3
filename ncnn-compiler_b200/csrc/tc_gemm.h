// Host-side planning for the tensor-core contraction kernel: encodes the TMA
// tensor maps, picks the tile shape and stage count, and launches.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include <cuda.h>
#include <cuda_runtime.h>

#include "tc_conv_halo.cuh"
#include "tc_dw_project.cuh"
#include "tc_gemm.cuh"
#include "tc_gemm2.cuh"
#include "tc_stem.cuh"
#include "tc_stem_pool.cuh"

namespace nb {

struct TcLaunch {
  TcGemmParams p{};
  alignas(64) CUtensorMap map_a0{};
  alignas(64) CUtensorMap map_a1{};
  alignas(64) CUtensorMap map_b0{};
  alignas(64) CUtensorMap map_b1{};
  alignas(64) CUtensorMap map_o0{};  // output planes, boxes of 16 columns x 128 rows
  alignas(64) CUtensorMap map_o1{};
  alignas(64) CUtensorMap map_r0{};  // residual planes
  alignas(64) CUtensorMap map_r1{};
  alignas(64) CUtensorMap map_s0{};  // int8 copies of the result (TcEpilogue::side_q)
  alignas(64) CUtensorMap map_s1{};
  int kind = GEMM_TF32;
  int grid = 0;
  int smem_bytes = 0;
  int cta2 = 0;  // CTAs per worker of tc_gemm2_kernel: 2 = CTA pairs, 1 = single CTAs with split tiles, 0 = tc_gemm_kernel
};

// Activation tensor as TMA sees it for an im2col load, innermost dimension first:
// channels, width, height, images.  For an ordinary NHWC tensor the strides are the
// dense ones; the 7x7 stem uses an overlapping-window view of a channel-padded image.
struct TcIm2colView {
  const void* plane0 = nullptr;
  const void* plane1 = nullptr;  // lo plane (GEMM_TF32X3 only)
  uint64_t C = 0, W = 0, H = 0, N = 0;
  uint64_t stride_w = 0, stride_h = 0, stride_n = 0;  // bytes
  int KH = 1, KW = 1;
  int stride_conv_h = 1, stride_conv_w = 1;
  int pad_t = 0, pad_l = 0;
  int dil_h = 1, dil_w = 1;
  int OH = 0, OW = 0;
};

struct TcEpilogue {
  const float* bias = nullptr;
  const float* scale = nullptr;
  float* out0 = nullptr;
  float* out1 = nullptr;
  int8_t* outq = nullptr;
  const float* res0 = nullptr;
  const float* res1 = nullptr;
  bool res_bf16 = false;  // the residual planes hold bf16 pairs (hi, mid)
  long long ldo = 0;
  int out_mode = OUT_F32;
  int act = ACT_NONE;
  float act_a = 0.0f, act_b = 0.0f;
  float out_scale = 1.0f;
  int* status = nullptr;
  long long* trace = nullptr;
  // int8 copies of an fp32 result, quantised with side_scale[i] (out_mode OUT_F32, channels a multiple of 16)
  int side_count = 0;
  int8_t* side_q[2] = {nullptr, nullptr};
  float side_scale[2] = {0.0f, 0.0f};
  // workspace for tiles split between CTA pairs (tc_gemm2.cuh): partial accumulators and one flag
  // word per CTA, zero before the first launch; without it tiles are never split
  uint32_t* sk_ws = nullptr;
  size_t sk_ws_bytes = 0;
  int* sk_flags = nullptr;
  int sk_flag_count = 0;
};

// bytes of partial-accumulator workspace and flag words that let every layer split tiles
constexpr size_t kTcSplitWorkspaceBytes = 160ull * kTcBlockM * kTc2MaxBlockN * 4;
constexpr int kTcSplitFlagCount = 640;  // two per CTA (one per epilogue group)

// Elements per K block for a kind and a channel count; 0 when the tensor-core
// path cannot address that channel count (rows must be multiples of 16 bytes).
int tc_k_elems(int kind, int channels);
int tc_row_bytes(int kind, int channels);

// Convolution: M = view.N*OH*OW pixels, N = out_channels.  `w0`/`w1` are the packed
// weights [out_channels][KH*KW*c_blocks*k_elems] (see tc_pack_weights).
// Returns an empty string on success, else the reason.
std::string tc_plan_conv(TcLaunch* launch, int kind, const TcIm2colView& view, const void* w0,
                         const void* w1, int out_channels, const TcEpilogue& epilogue,
                         int sm_count);

// Plain GEMM: A is [M][K] row-major with row stride lda elements (planes a0/a1),
// weights packed [N][Kpad].
std::string tc_plan_gemm(TcLaunch* launch, int kind, const void* a0, const void* a1, long long M,
                         int K, long long lda, const void* w0, const void* w1, int N,
                         const TcEpilogue& epilogue, int sm_count);

cudaError_t tc_launch(const TcLaunch& launch, cudaStream_t stream);

// Packs [O][I][KH][KW] (ncnn order) weights into [O][KH*KW][c_blocks*k_elems] with
// zero padding, channel innermost.  For fp32 kinds `hi` receives the values
// rounded to tf32 (GEMM_TF32, GEMM_TF32X3) and `lo` the remainders (GEMM_TF32X3).
void tc_pack_weights_f32(int kind, const float* w, int O, int I, int KH, int KW, int k_elems,
                         std::vector<float>* hi, std::vector<float>* lo);
void tc_pack_weights_i8(const int8_t* w, int O, int I, int KH, int KW, int k_elems,
                        std::vector<int8_t>* packed);

// GEMM_BF16X3: two bf16 planes, hi = bf16(w) and mid = bf16(w - hi), same layout.
void tc_pack_weights_bf16x2(const float* w, int O, int I, int KH, int KW, int k_elems,
                            std::vector<uint16_t>* hi, std::vector<uint16_t>* mid);

float tf32_round_host(float x);
uint16_t bf16_round_host(float x);
float bf16_to_float_host(uint16_t h);

// ---- stride-1 convolution with the input patch resident in shared memory (tc_conv_halo.cuh)
struct TcHaloLaunch {
  TcHaloParams p{};
  alignas(64) CUtensorMap map_a0{};
  alignas(64) CUtensorMap map_a1{};
  alignas(64) CUtensorMap map_b0{};
  alignas(64) CUtensorMap map_b1{};
  alignas(64) CUtensorMap map_o0{};
  alignas(64) CUtensorMap map_o1{};
  alignas(64) CUtensorMap map_r0{};
  alignas(64) CUtensorMap map_r1{};
  int kind = GEMM_TF32;
  int grid = 0;
  int smem_bytes = 0;
  int pair = 0;  // 1: two pixel tiles per cluster of two CTAs (grid counts CTAs)
};

struct TcHaloConv {
  const void* in0 = nullptr;  // NHWC activation planes
  const void* in1 = nullptr;
  int images = 0, H = 0, W = 0, C = 0;
  int KH = 1, KW = 1, pad_t = 0, pad_l = 0, OH = 0, OW = 0;
  const void* w0 = nullptr;  // packed like tc_plan_conv's weights
  const void* w1 = nullptr;
  int out_channels = 0;
};

// True when the patch-resident kernel applies and is expected to win: fp32 kind, stride and
// dilation 1, channels in blocks of 32, output rows of 16 bytes, tiles mostly inside the image.
bool tc_halo_applies(int kind, int C, int KH, int KW, int stride_h, int stride_w, int dil_h, int dil_w, int OH,
                     int OW, int out_channels, int out_mode);
// `pair`: plan the form that runs two pixel tiles on a cluster of two CTAs (tiles up to 256 channels wide)
std::string tc_plan_conv_halo(TcHaloLaunch* launch, int kind, const TcHaloConv& conv, const TcEpilogue& epilogue,
                              int sm_count, bool pair = false);
cudaError_t tc_launch_halo(const TcHaloLaunch& launch, cudaStream_t stream);

// ---- 3x3 depthwise convolution fused into the following 1x1 convolution (tc_dw_project.cuh)
struct TcDwProjLaunch {
  TcDwProjParams p{};
  alignas(64) CUtensorMap map_x{};   // fp32 depthwise input, patches of 18 x 10 pixels x 32 channels (expand fused in: bf16 hi plane of the block's input)
  alignas(64) CUtensorMap map_x1{};  // expand fused in: bf16 mid plane of the block's input
  alignas(64) CUtensorMap map_e0{};  // expand weights, bf16 hi / mid planes
  alignas(64) CUtensorMap map_e1{};
  alignas(64) CUtensorMap map_b0{};  // projection weights, bf16 hi / mid planes
  alignas(64) CUtensorMap map_b1{};
  alignas(64) CUtensorMap map_o0{};
  alignas(64) CUtensorMap map_o1{};
  alignas(64) CUtensorMap map_r0{};
  alignas(64) CUtensorMap map_r1{};
  int grid = 0;
  int smem_bytes = 0;
  int stride = 1;
  bool expand = false;
};

struct TcDwProjConv {
  const void* x = nullptr;   // NHWC input: plain fp32 of the depthwise layer, or (expand fused in) the bf16 hi plane of the expand layer's
  const void* x1 = nullptr;  // expand fused in: the bf16 mid plane
  int images = 0, H = 0, W = 0, C = 0;  // depthwise output extent, depthwise channels
  int Hin = 0, Win = 0;                 // depthwise input extent
  int stride = 1;
  int pad_t = 1, pad_l = 1;
  // expand layer fused in (ex_w0 != nullptr): 1x1 convolution Cin -> C on bf16 pairs, Cin <= 32
  int Cin = 0;
  const void* ex_w0 = nullptr;        // packed [C][32] bf16 hi / mid
  const void* ex_w1 = nullptr;
  const float* ex_bias = nullptr;     // [C] or null
  int ex_act = ACT_NONE;
  float ex_act_a = 0.0f, ex_act_b = 0.0f;
  const float* dw_weights = nullptr;  // [9][C]
  const float* dw_bias = nullptr;
  int dw_act = ACT_NONE;
  float dw_act_a = 0.0f, dw_act_b = 0.0f;
  const void* w0 = nullptr;  // projection weights packed [N][ceil(C/32)*32] bf16 hi / mid
  const void* w1 = nullptr;
  int out_channels = 0;
};

// True when the fused kernel takes the pair of layers: 3x3, stride 1, dilation 1, output extent equal to the
// input's, channels in fours; projection 1x1 stride 1 with bf16-pair operands and a staged epilogue.
bool tc_dw_project_applies(int C, int N, int H, int W, int out_mode, bool has_res, bool res_bf16);
// True when the whole inverted-residual block (1x1 expand Cin -> C with at most 32 input channels, 3x3 depthwise of
// stride 1 or 2 with output OH x OW, 1x1 projection C -> N) fits the fused kernel, whatever formats its output and
// residual get.
bool tc_block_applies(int Cin, int C, int N, int OH, int OW, int stride, bool has_res);
std::string tc_plan_dw_project(TcDwProjLaunch* launch, const TcDwProjConv& conv, const TcEpilogue& epilogue, int sm_count);
cudaError_t tc_launch_dw_project(const TcDwProjLaunch& launch, cudaStream_t stream);

// ---- stem convolution with the input rows resident in shared memory (tc_stem.cuh)
struct TcStemLaunch {
  TcStemParams p{};
  alignas(64) CUtensorMap map_a0{};
  alignas(64) CUtensorMap map_a1{};
  alignas(64) CUtensorMap map_b0{};
  alignas(64) CUtensorMap map_b1{};
  alignas(64) CUtensorMap map_o0{};
  alignas(64) CUtensorMap map_o1{};
  int kind = GEMM_BF16X3;
  int grid = 0;
  int smem_bytes = 0;
};

struct TcStemConv {
  int kind = GEMM_BF16X3;     // GEMM_BF16X3 (4-channel pixels, bf16 hi/mid planes) or GEMM_I8 (8-channel int8 pixels)
  const void* in0 = nullptr;  // [images][H][row_bytes]: padded rows of 8-byte pixels (bf16 hi plane, or int8)
  const void* in1 = nullptr;  // bf16 mid plane
  int images = 0, H = 0;
  int row_bytes = 0;          // bytes of one padded row (a multiple of 128)
  int KH = 1, stride_h = 1, pad_t = 0, OH = 0, OW = 0;
  const void* w0 = nullptr;   // packed [O][KH][32] bf16 hi / mid, or [O][KH][64] int8 (one 64-byte window per filter row)
  const void* w1 = nullptr;
  int out_channels = 0;
};

// ---- stem convolution + 3x3 stride-2 max pooling in one kernel (tc_stem_pool.cuh)
struct TcStemPoolLaunch {
  TcStemPoolParams pp{};
  alignas(64) CUtensorMap map_a0{};
  alignas(64) CUtensorMap map_a1{};
  alignas(64) CUtensorMap map_b0{};
  alignas(64) CUtensorMap map_b1{};
  alignas(64) CUtensorMap map_o0{};  // pooled result: bf16 hi / mid planes, or fp32 and its int8 copy
  alignas(64) CUtensorMap map_o1{};
  int grid = 0;
  int smem_bytes = 0;
  int kind = GEMM_BF16X3;
};
// `epilogue` describes the POOLED tensor (dense rows of out_channels: bf16 pairs behind a bf16-pair stem, fp32 with at
// most one int8 copy behind an int8 stem); pooled extent pooled_h x pooled_w = half the convolution's output extent
// (3x3 windows, stride 2, one pixel of padding above and to the left).
std::string tc_plan_stem_pool(TcStemPoolLaunch* launch, const struct TcStemConv& conv, const TcEpilogue& epilogue, int pooled_h,
                              int pooled_w, int sm_count);
cudaError_t tc_launch_stem_pool(const TcStemPoolLaunch& launch, cudaStream_t stream);

// Applies when output pixels are 16 bytes apart in the padded input row (stride 2 x 4 channels x
// bf16), a row of output fits one 128-row tile, and the rows and resident weights fit shared memory.
std::string tc_plan_stem(TcStemLaunch* launch, const TcStemConv& conv, const TcEpilogue& epilogue, int sm_count);
cudaError_t tc_launch_stem(const TcStemLaunch& launch, cudaStream_t stream);

}  // namespace nb
