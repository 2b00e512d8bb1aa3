// Internals of the graph executor, shared by its translation units: engine_import.cu (ncnn layers -> nodes),
// engine_plan.cu (fusion passes, weight packing, memory plan), engine_emit.cu (nodes -> kernel launches) and
// engine.cu (plans, CUDA graphs, the run paths and the public Engine facade).
#pragma once

#include "engine.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <functional>
#include <limits>
#include <map>
#include <sstream>

#include "ip_rows.cuh"
#include "kernels.cuh"
#include "loader.h"
#include "tc_gemm.h"

namespace nb {

enum NodeKind { N_CONV, N_DW, N_IP, N_GEMM, N_POOL, N_BINARY, N_UNARY, N_RELAYOUT, N_SOFTMAX, N_CONCAT, N_REMAP, N_REDUCE, N_DECONV };
enum Impl { IMPL_NONE, IMPL_TC, IMPL_DIRECT };

struct Tensor {
  std::string name;
  int rank = 0;
  int c = 1, h = 1, w = 1;  // logical dims (rank 1: w; rank 2: h x w; rank 3: c x h x w)
  int d = 1;                // rank 4: c x d x h x w, stored in that order (only data-movement layers take rank 4)
  bool i8 = false;
  int alias = -1;  // Split: shares the storage of another tensor
  bool is_input = false;
  int input_index = -1;
  // storage
  int fmt = FMT_F32;
  int Cp = 1, Wp = 1, w_off = 0;  // padded layout of a stem input
  float input_quant_scale = 0.0f;  // > 0: the input edge quantises to int8
  size_t plane_elems = 0;          // storage elements per image and plane
  size_t plane_bytes = 0;          // per image, rounded to 256
  size_t offset = 0;               // byte offset per image inside the arena
  int first_def = -1, last_use = -1;
  bool dedicated = false;          // never shares arena space (padding must stay zero)

  long long logical() const { return static_cast<long long>(c) * d * h * w; }
  int planes() const { return fmt == FMT_SPLIT || fmt == FMT_BF16X2 ? 2 : 1; }
  int elem_bytes() const { return fmt == FMT_I8 ? 1 : (fmt == FMT_BF16X2 ? 2 : 4); }
};

struct Node {
  NodeKind kind = N_UNARY;
  std::string name, type;
  std::vector<int> in;
  int out = -1;
  // int8 copies of the fp32 result that this node writes as well, each quantised with the input scale of
  // the int8 contraction that reads it (tensor id, scale): the Quantize steps they replace are gone
  std::vector<std::pair<int, float>> side_q;
  // contraction geometry
  int KH = 1, KW = 1, sh = 1, sw = 1, pt = 0, pl = 0, dh = 1, dw = 1, O = 0, OH = 1, OW = 1;
  int term = 0;
  int act = ACT_NONE;
  float act_a = 0.0f, act_b = 0.0f;
  int res = -1;
  int impl = IMPL_NONE;
  bool stem = false;
  bool stem_bf16 = false;  // stem whose window view holds bf16 pairs (64-byte rows)
  bool stem_rows = false;  // stem (bf16 pairs or int8) whose input rows can stay resident in shared memory (tc_stem.cuh)
  // host-side parameters
  std::vector<float> w_f32;   // [O][I][KH][KW] (conv), [O][K] (ip/gemm), [C][KH][KW] (dw)
  std::vector<int8_t> w_i8;
  std::vector<float> bias, deq;  // deq = 1/(s_w*s_in) per output channel
  float s_in = 0.0f, s_out = 0.0f, s_b = 0.0f;
  bool has_bias = false;
  int K = 0;                     // contraction length (ip / gemm)
  float alpha = 1.0f, beta = 1.0f;
  // pooling / element-wise
  PoolParams pool{};
  BinaryParams bin{};
  UnaryParams un{};
  std::vector<float> un_scale, un_offset;
  RelayoutParams relayout{};
  SoftmaxParams softmax{};
  std::vector<ConcatParams> concat;  // one per input
  RemapParams remap{};
  ReduceParams reduce{};
  bool broadcast = false;  // N_BINARY whose operands differ in shape
  // N_CONV (tensor-core path) that writes straight into a channel Concat's result: its output
  // rows are `out_ld` channels long and start `out_ch_off` channels in (0 = dense, its own tensor)
  int out_ld = 0, out_ch_off = 0;
  BroadcastParams bcast{};
  // device-side parameters
  void* d_w0 = nullptr;
  void* d_w1 = nullptr;
  float* d_bias = nullptr;
  float* d_deq = nullptr;
  float* d_scale = nullptr;
  float* d_offset = nullptr;
  int k_elems = 0;
  double flops = 0.0;  // per image
  // N_CONV (1x1, tensor cores) that also computes the 3x3 depthwise layer in front of it (tc_dw_project.cuh):
  // in[0] is then the depthwise layer's input, these are its parameters
  bool dw_fused = false;
  const float* dw_w = nullptr;  // [9][C]
  const float* dw_bias = nullptr;
  int dw_act = ACT_NONE;
  float dw_act_a = 0.0f, dw_act_b = 0.0f;
  int dw_pt = 1, dw_pl = 1;
  int dw_stride = 1;
  int dw_c = 0, dw_hin = 0, dw_win = 0;  // channels and input extent of the depthwise layer
  std::string dw_name;
  // a 3x3 stride-2 max pooling that runs inside the stem kernel in front of it (fuse_stem_pooling)
  bool pool_fused = false;
  int pool_oh = 0, pool_ow = 0;
  std::string pool_name;
  // the 1x1 expand convolution in front of that depthwise layer, merged into the projection node by the same pass
  bool ex_fused = false;
  const void* ex_w0 = nullptr;
  const void* ex_w1 = nullptr;
  const float* ex_bias = nullptr;
  int ex_act = ACT_NONE;
  float ex_act_a = 0.0f, ex_act_b = 0.0f;
  int ex_cin = 0;
  std::string ex_name;
};

struct Step {
  std::string name, kernel;
  std::function<cudaError_t(cudaStream_t)> run;
  double flops = 0.0, bytes = 0.0;
};

constexpr int kMaxChunks = 4;

struct Plan {
  int64_t n = 0;
  uint64_t last_used = 0;  // for the bounded plan cache
  std::vector<Step> steps;
  std::vector<float*> d_in, d_out;  // staging used by host-pointer runs
  cudaGraphExec_t graph = nullptr;
  std::vector<const void*> graph_ptrs;  // the edge pointers the graph was captured with
  // Pipelined host-pointer runs: the batch is uploaded in `chunks` pieces; as soon as a piece
  // has landed, its input edge and the first `head_end` layers run on its images alone
  // (head[c]); the remaining layers and the output edges run once on the whole batch (tail).
  int chunks = 0;
  int head_end = 0;
  std::vector<Step> head[kMaxChunks], tail;
  cudaGraphExec_t head_graph[kMaxChunks] = {};
  cudaGraphExec_t tail_graph = nullptr;
  void release() {
    if (graph != nullptr) cudaGraphExecDestroy(graph);
    graph = nullptr;
    for (cudaGraphExec_t& g : head_graph) {
      if (g != nullptr) cudaGraphExecDestroy(g);
      g = nullptr;
    }
    if (tail_graph != nullptr) cudaGraphExecDestroy(tail_graph);
    tail_graph = nullptr;
    for (float* p : d_in) cudaFree(p);
    for (float* p : d_out) cudaFree(p);
    d_in.clear();
    d_out.clear();
  }
};

constexpr size_t kMaxCachedPlans = 8;  // batch sizes whose plans (graphs, staging buffers) stay alive

// Host-pointer runs that upload at least this much are pipelined.
constexpr size_t kPipelineUploadBytes = 4u << 20;

inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline int grid_for(long long work, int block = 256) {
  const long long g = (work + block - 1) / block;
  return static_cast<int>(std::max<long long>(1, std::min<long long>(g, 148ll * 32)));
}

inline int conv_extent(int in, int k, int s, int d, int p0, int p1) {
  return 1 + (in + p0 + p1 - ((k - 1) * d + 1)) / s;
}

inline void same_pads(int in, int k, int s, int d, bool lower, int* before, int* after) {
  const int extent = d * (k - 1) + 1;
  const int out = 1 + (in - 1) / s;
  const int total = std::max((out - 1) * s + extent - in, 0);
  *before = lower ? total / 2 + total % 2 : total / 2;
  *after = total - *before;
}

inline int host_quantize(float x, float s) {
  volatile float v = x * s;
  volatile float t;
  float r;
  if (v >= 0.0f) {
    t = v + 0.5f;
    r = std::floor(t);
  } else {
    t = v + -0.5f;
    r = std::ceil(t);
  }
  r = std::max(std::min(r, 127.0f), -127.0f);
  return static_cast<int>(r);
}


// Makes the model's device current for the duration of a call and puts the caller's device back:
// a process may hold one handle per GPU and call them in any order from one thread.
struct DeviceGuard {
  int previous = -1;
  bool switched = false;
  explicit DeviceGuard(int device) {
    if (device < 0) return;
    if (cudaGetDevice(&previous) != cudaSuccess) {
      previous = -1;
      cudaGetLastError();
    }
    if (previous != device) switched = cudaSetDevice(device) == cudaSuccess && previous >= 0;
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(previous);
  }
  DeviceGuard(const DeviceGuard&) = delete;
  DeviceGuard& operator=(const DeviceGuard&) = delete;
};

class EngineImpl {
 public:
  ~EngineImpl() {
    DeviceGuard guard(device_);
    for (auto& kv : plans_) kv.second.release();
    for (void* p : device_allocs_) cudaFree(p);
    if (arena_ != nullptr) cudaFree(arena_);
    for (cudaEvent_t e : upload_done_)
      if (e != nullptr) cudaEventDestroy(e);
    if (copy_stream_ != nullptr) cudaStreamDestroy(copy_stream_);
    if (stream_ != nullptr) cudaStreamDestroy(stream_);
  }

  bool build(const std::string& param, const std::string& bin, const EngineOptions& opt,
             std::string* err);
  int run(int64_t n, const float* const* in, float* const* out, bool host, cudaStream_t stream);
  int run_host_pipelined(Plan* plan, const float* const* in, float* const* out);
  bool build_pipeline(Plan* plan);
  bool ensure_staging(Plan* plan);
  bool issue_steps(const std::vector<Step>& steps, cudaStream_t st);
  cudaGraphExec_t capture_steps(const std::vector<Step>& steps);
  int launch(Plan* plan, const std::vector<const float*>& d_in, const std::vector<float*>& d_out, cudaStream_t st);
  int finish_host_run(cudaStream_t st);
  void choose_head_limit();
  void fold_channel_concats();
  void fuse_quantize_steps();
  void fuse_depthwise_projection();
  void fuse_stem_pooling();
  int profile(int64_t n, int repeat, std::vector<LayerTiming>* out);
  Plan* plan_for(int64_t n);

  EngineOptions opt_;
  ModelDef model_;
  std::vector<Tensor> tensors_;
  std::vector<Node> nodes_;
  std::map<std::string, int> by_name_;
  std::vector<int> inputs_, outputs_;
  std::string error_;
  std::map<int64_t, Plan> plans_;
  std::vector<void*> device_allocs_;
  uint8_t* arena_ = nullptr;
  size_t arena_bytes_ = 0;
  size_t arena_per_image_ = 0;
  bool stall_injected_ = false;
  int device_ = -1;  // the CUDA device that owns every allocation, stream and graph of this model
  uint64_t use_counter_ = 0;
  int* d_status_ = nullptr;
  uint32_t* d_split_ws_ = nullptr;
  int* d_split_flags_ = nullptr;
  int sm_count_ = 148;
  cudaStream_t stream_ = nullptr;
  cudaStream_t copy_stream_ = nullptr;  // uploads of the pipelined host-pointer path
  cudaEvent_t upload_done_[kMaxChunks] = {};
  // image window applied by ref(): tensors are laid out for layout_n_ images (0: the n
  // passed in) and pointers start at image img0_
  int64_t layout_n_ = 0, img0_ = 0;
  int head_limit_ = 0;  // layers [0, head_limit_) may run per chunk (their tensors never share arena space)
  bool any_fp32_tc_ = false;

 private:
  int resolve(int t) const {
    while (tensors_[t].alias >= 0) t = tensors_[t].alias;
    return t;
  }
  int new_tensor(const std::string& name) {
    Tensor t;
    t.name = name;
    tensors_.push_back(t);
    by_name_[name] = static_cast<int>(tensors_.size()) - 1;
    return static_cast<int>(tensors_.size()) - 1;
  }
  bool fail(std::string* err, const std::string& msg) {
    *err = msg;
    return false;
  }
  // Every device allocation of the engine.  NCNN_B200_TEST_FAIL_ALLOC=k makes the k-th one of this engine
  // fail as the driver would when memory runs out (the out-of-memory paths are tested without filling a GPU).
  cudaError_t device_alloc(void** p, size_t bytes) {
    const char* env = std::getenv("NCNN_B200_TEST_FAIL_ALLOC");
    if (env != nullptr && std::atol(env) == ++alloc_count_) {
      *p = nullptr;
      return cudaErrorMemoryAllocation;
    }
    return cudaMalloc(p, bytes);
  }
  long alloc_count_ = 0;
  bool upload_failed_ = false;
  template <class T>
  T* upload(const std::vector<T>& v) {
    if (v.empty()) return nullptr;
    void* d = nullptr;
    if (device_alloc(&d, v.size() * sizeof(T)) != cudaSuccess) {
      upload_failed_ = true;  // prepare_weights() reports it: no kernel may ever see the null pointer
      return nullptr;
    }
    cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice);
    device_allocs_.push_back(d);
    return static_cast<T*>(d);
  }

  bool import_layers(std::string* err);
  bool import_conv(const LayerDef& l, bool depthwise, std::string* err);
  bool import_ip(const LayerDef& l, std::string* err);
  bool import_gemm(const LayerDef& l, std::string* err);
  bool import_pool(const LayerDef& l, std::string* err);
  bool decode_activation(const LayerDef& l, int id_type, int id_params, Node* n, std::string* err);
  void fold_batchnorm();
  void fuse();
  bool choose_impl(std::string* err);
  bool prepare_weights(std::string* err);
  void plan_memory();
  ActRef ref(int tensor, int64_t n) const;
  bool emit_node(Plan& plan, const Node& node, int64_t n, std::string* err);
  void restore_padding(int64_t n, cudaStream_t st);
  int64_t last_run_n_ = 0;  // batch size of the previous run (0: none yet)
  void make_edge_steps(int64_t n, const std::vector<const float*>& d_in, const std::vector<float*>& d_out,
                       std::vector<Step>* pre, std::vector<Step>* post);
};


// NCNN_B200_STEM_ROWS=0 at load time keeps the stem on the im2col-window path of tc_gemm_kernel.
inline bool stem_rows_enabled() {
  const char* f = std::getenv("NCNN_B200_STEM_ROWS");
  return f == nullptr || f[0] != '0';
}

// The patch-resident convolution kernel applies to stride-1 filters; measured inside whole
// networks (batch 64, 3x3 filters at 56/28/14 pixels) it ties with the im2col kernel once the
// operands are bf16 pairs, and loses a little where its 16x8 tiles overhang the image, so it
// is opt-in: NCNN_B200_HALO=1 at load time selects it wherever it applies (2: on pairs of CTAs).
inline int halo_level() {
  const char* f = std::getenv("NCNN_B200_HALO");
  return f == nullptr || f[0] == 0 ? 0 : std::atoi(f);
}
inline bool halo_preferred() { return halo_level() >= 1; }

inline int env_int_or(const char* name, int fallback) {
  const char* f = std::getenv(name);
  return f == nullptr || f[0] == 0 ? fallback : std::atoi(f);
}

// NAME=0 in the environment switches an optional pass off
inline bool env_flag_off(const char* name) {
  const char* f = std::getenv(name);
  return f != nullptr && f[0] == '0';
}

}  // namespace nb
