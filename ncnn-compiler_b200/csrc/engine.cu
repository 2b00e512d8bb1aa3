#include "engine.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <functional>
#include <limits>
#include <map>
#include <sstream>

#include "kernels.cuh"
#include "loader.h"
#include "tc_gemm.h"

namespace nb {
namespace {

enum NodeKind { N_CONV, N_DW, N_IP, N_GEMM, N_POOL, N_BINARY, N_UNARY, N_RELAYOUT, N_SOFTMAX, N_CONCAT, N_REMAP, N_REDUCE, N_DECONV };
enum Impl { IMPL_NONE, IMPL_TC, IMPL_DIRECT };

struct Tensor {
  std::string name;
  int rank = 0;
  int c = 1, h = 1, w = 1;  // logical dims (rank 1: w; rank 2: h x w; rank 3: c x h x w)
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

  long long logical() const { return static_cast<long long>(c) * h * w; }
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
  std::string dw_name;
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

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int grid_for(long long work, int block = 256) {
  const long long g = (work + block - 1) / block;
  return static_cast<int>(std::max<long long>(1, std::min<long long>(g, 148ll * 32)));
}

int conv_extent(int in, int k, int s, int d, int p0, int p1) {
  return 1 + (in + p0 + p1 - ((k - 1) * d + 1)) / s;
}

void same_pads(int in, int k, int s, int d, bool lower, int* before, int* after) {
  const int extent = d * (k - 1) + 1;
  const int out = 1 + (in - 1) / s;
  const int total = std::max((out - 1) * s + extent - in, 0);
  *before = lower ? total / 2 + total % 2 : total / 2;
  *after = total - *before;
}

int host_quantize(float x, float s) {
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

}  // namespace

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

// ---------------------------------------------------------------------- import
bool EngineImpl::decode_activation(const LayerDef& l, int id_type, int id_params, Node* n,
                                   std::string* err) {
  // The reference splits a fused activation into its own op and accepts none(0),
  // ReLU(1) and Sigmoid(4) (lib/Importer/ImportConvolution.cpp:69-78,236-246).  This
  // runtime takes 0, 1, 4, leaky ReLU (2, one parameter) and clip (3, two parameters);
  // everything else is rejected.
  const int64_t type = l.params.get_int(id_type, 0);
  const std::vector<float>* ap = l.params.get_float_array(id_params);
  if (type == 0) return true;
  if (type == 1) {
    n->act = ACT_RELU;
    return true;
  }
  if (type == 2 && ap != nullptr && ap->size() == 1) {
    n->act = ACT_LEAKY;
    n->act_a = (*ap)[0];
    return true;
  }
  if (type == 3 && ap != nullptr && ap->size() == 2) {
    n->act = ACT_CLIP;
    n->act_a = (*ap)[0];
    n->act_b = (*ap)[1];
    return true;
  }
  if (type == 4 && n->term == 0) {
    n->act = ACT_SIGMOID;
    return true;
  }
  return fail(err, "layer " + l.name + ": activation_type " + std::to_string(type) +
                       " is outside the supported path");
}

bool EngineImpl::import_conv(const LayerDef& l, bool depthwise, std::string* err) {
  const std::string where = "layer " + l.name + " (" + l.type + "): ";
  if (l.bottoms.size() != 1 || l.tops.size() != 1) return fail(err, where + "expects one input and one output");
  const int in = by_name_.at(l.bottoms[0]);
  const Tensor ti = tensors_[resolve(in)];  // copy: new_tensor() below may reallocate
  if (ti.rank != 3) return fail(err, where + "convolution input must have [C,H,W] layout");
  const ParamDict& p = l.params;
  if (p.get_int(19, 0) != 0) return fail(err, where + "dynamic weights are not supported");
  Node n;
  n.kind = depthwise ? N_DW : N_CONV;
  n.name = l.name;
  n.type = l.type;
  n.O = static_cast<int>(p.get_int(0, 0));
  n.KW = static_cast<int>(p.get_int(1, 0));
  n.KH = static_cast<int>(p.get_int(11, n.KW));
  n.dw = static_cast<int>(p.get_int(2, 1));
  n.dh = static_cast<int>(p.get_int(12, n.dw));
  n.sw = static_cast<int>(p.get_int(3, 1));
  n.sh = static_cast<int>(p.get_int(13, n.sw));
  int pl = static_cast<int>(p.get_int(4, 0));
  int pr = static_cast<int>(p.get_int(15, pl));
  int pt = static_cast<int>(p.get_int(14, pl));
  int pb = static_cast<int>(p.get_int(16, pt));
  n.has_bias = p.get_int(5, 0) == 1;
  n.term = static_cast<int>(p.get_int(8, 0));
  if (n.dw <= 0 || n.dh <= 0 || n.sw <= 0 || n.sh <= 0) return fail(err, where + "stride and dilation must be positive");
  if (p.get_float(18, 0.0f) != 0.0f) return fail(err, where + "non-zero pad_value is not supported");
  if (!decode_activation(l, 9, 10, &n, err)) return false;
  const bool same_u = pl == -233 && pr == -233 && pt == -233 && pb == -233;
  const bool same_l = pl == -234 && pr == -234 && pt == -234 && pb == -234;
  if (same_u || same_l) {
    // NormalizeNCNN.cpp:30-50: SAME padding becomes explicit pads, output = ceil(in/stride)
    same_pads(ti.h, n.KH, n.sh, n.dh, same_l, &pt, &pb);
    same_pads(ti.w, n.KW, n.sw, n.dw, same_l, &pl, &pr);
  } else if (pl < 0 || pr < 0 || pt < 0 || pb < 0) {
    return fail(err, where + "convolution padding has unsupported value");
  }
  if (ti.h + pt + pb < (n.KH - 1) * n.dh + 1) return fail(err, where + "convolution kernel exceeds padded input height");
  if (ti.w + pl + pr < (n.KW - 1) * n.dw + 1) return fail(err, where + "convolution kernel exceeds padded input width");
  n.pt = pt;
  n.pl = pl;
  n.OH = conv_extent(ti.h, n.KH, n.sh, n.dh, pt, pb);
  n.OW = conv_extent(ti.w, n.KW, n.sw, n.dw, pl, pr);
  const size_t expected = 1 + (n.has_bias ? 1 : 0) + (n.term ? 2 : 0) + (n.term > 100 ? 1 : 0);
  if (l.weights.size() != expected) return fail(err, where + "weights are missing (was a .bin supplied?)");
  const WeightTensor& wt = l.weights[0];
  const int I = static_cast<int>(wt.shape[1]);
  if (depthwise) {
    const int group = static_cast<int>(p.get_int(7, 1));
    if (!(group == ti.c && n.O == ti.c && I == 1))
      return fail(err, where + "only pure depthwise (group == channels == num_output) is supported");
  } else if (I != ti.c) {
    return fail(err, where + "convolution input channels do not match weight channels");
  }
  if (n.term == 0 && wt.type == WeightType::kI8) return fail(err, where + "non-quantized convolution weight cannot be i8");
  if (n.term != 0 && wt.type == WeightType::kF16) return fail(err, where + "quantized convolution weight must be f32 or i8");
  if (ti.i8 && n.term == 0) return fail(err, where + "non-quantized convolution input must be f32");
  size_t wi = 1;
  if (n.has_bias) n.bias = l.weights[wi++].as_f32();
  if (n.term != 0) {
    std::vector<float> ws = l.weights[wi++].as_f32();
    n.s_in = l.weights[wi++].as_f32()[0];
    if (n.term > 100) n.s_out = l.weights[wi++].as_f32()[0];
    if (ws.size() == 1 && n.O > 1) ws.assign(n.O, ws[0]);
    for (float s : ws)
      if (!(s >= 0.0f) || !std::isfinite(s)) return fail(err, where + "int8 scales must be finite and non-negative");
    if (!(n.s_in > 0.0f) || (n.term > 100 && !(n.s_out > 0.0f))) return fail(err, where + "int8 activation scales must be positive");
    // dequantizeAccumulator (NCNNToTosa.cpp:577-596): r = 1/(s_w*s_in), 0 where s_w == 0
    n.deq.resize(n.O);
    for (int o = 0; o < n.O; ++o) {
      volatile float combined = ws[o] * n.s_in;
      n.deq[o] = ws[o] == 0.0f ? 0.0f : 1.0f / combined;
    }
    if (wt.type == WeightType::kI8) {
      n.w_i8.assign(wt.as_i8(), wt.as_i8() + wt.count());
    } else {
      // quantizeConstantToI8 (NCNNToTosa.cpp:234-301): per output channel
      const std::vector<float> wf = wt.as_f32();
      const size_t row = wf.size() / n.O;
      n.w_i8.resize(wf.size());
      for (size_t i = 0; i < wf.size(); ++i)
        n.w_i8[i] = static_cast<int8_t>(host_quantize(wf[i], ws[i / row]));
    }
  } else {
    n.w_f32 = wt.as_f32();
  }
  n.in = {in};
  n.out = new_tensor(l.tops[0]);
  Tensor& to = tensors_[n.out];
  to.rank = 3;
  to.c = n.O;
  to.h = n.OH;
  to.w = n.OW;
  to.i8 = n.term > 100;
  if (to.i8 && n.act != ACT_NONE && n.act != ACT_RELU)
    return fail(err, where + "only ReLU can follow an int8 result");
  n.flops = 2.0 * n.OH * n.OW * n.O * (depthwise ? 1 : ti.c) * n.KH * n.KW;
  nodes_.push_back(std::move(n));
  return true;
}

bool EngineImpl::import_ip(const LayerDef& l, std::string* err) {
  const std::string where = "layer " + l.name + " (InnerProduct): ";
  if (l.bottoms.size() != 1 || l.tops.size() != 1) return fail(err, where + "expects one input and one output");
  const int in = by_name_.at(l.bottoms[0]);
  const Tensor ti = tensors_[resolve(in)];  // copy: new_tensor() below may reallocate
  const ParamDict& p = l.params;
  Node n;
  n.kind = N_IP;
  n.name = l.name;
  n.type = l.type;
  n.O = static_cast<int>(p.get_int(0, 0));
  n.has_bias = p.get_int(1, 0) == 1;
  n.term = static_cast<int>(p.get_int(8, 0));
  if (!decode_activation(l, 9, 10, &n, err)) return false;
  const size_t expected = 1 + (n.has_bias ? 1 : 0) + (n.term ? 2 : 0);
  if (l.weights.size() != expected) return fail(err, where + "weights are missing (was a .bin supplied?)");
  const WeightTensor& wt = l.weights[0];
  n.K = static_cast<int>(wt.shape[1]);
  if (ti.i8) return fail(err, where + "quantized InnerProduct input must be f32");
  // NCNNOps.cpp:1247-1312: static form flattens any input with numel == K; the
  // rank-2 form [M,K] -> [M,O] keeps the rows.
  bool rows = false;
  if (ti.rank == 2 && ti.w == n.K && (ti.logical() != n.K || opt_.keep_matrix_rows)) {
    rows = true;
  } else if (ti.logical() != n.K) {
    return fail(err, where + "input element count does not match the weight");
  }
  if (n.term == 0 && wt.type == WeightType::kI8) return fail(err, where + "InnerProduct kernel element type does not match scale term");
  size_t wi = 1;
  if (n.has_bias) n.bias = l.weights[wi++].as_f32();
  if (n.term != 0) {
    std::vector<float> ws = l.weights[wi++].as_f32();
    n.s_in = l.weights[wi++].as_f32()[0];
    if (!(n.s_in > 0.0f)) return fail(err, where + "int8 activation scale must be positive");
    n.deq.resize(n.O);
    for (int o = 0; o < n.O; ++o) {
      volatile float combined = ws[o] * n.s_in;
      n.deq[o] = ws[o] == 0.0f ? 0.0f : 1.0f / combined;
    }
    if (wt.type == WeightType::kI8) {
      n.w_i8.assign(wt.as_i8(), wt.as_i8() + wt.count());
    } else {
      const std::vector<float> wf = wt.as_f32();
      n.w_i8.resize(wf.size());
      for (size_t i = 0; i < wf.size(); ++i)
        n.w_i8[i] = static_cast<int8_t>(host_quantize(wf[i], ws[i / n.K]));
    }
  } else {
    n.w_f32 = wt.as_f32();
  }
  n.in = {in};
  n.out = new_tensor(l.tops[0]);
  Tensor& to = tensors_[n.out];
  if (rows) {
    to.rank = 2;
    to.h = ti.h;
    to.w = n.O;
  } else {
    to.rank = 1;
    to.w = n.O;
  }
  n.flops = 2.0 * (rows ? ti.h : 1) * n.K * n.O;
  nodes_.push_back(std::move(n));
  return true;
}

bool EngineImpl::import_gemm(const LayerDef& l, std::string* err) {
  const std::string where = "layer " + l.name + " (Gemm): ";
  const ParamDict& p = l.params;
  if (l.bottoms.size() != 1 || l.weights.empty())
    return fail(err, where + "only dynamic-A, transposed constant-B Gemm with optional row bias and optional int8 B is supported");
  const int in = by_name_.at(l.bottoms[0]);
  const Tensor ti = tensors_[resolve(in)];  // copy: new_tensor() below may reallocate
  Node n;
  n.kind = N_GEMM;
  n.name = l.name;
  n.type = l.type;
  n.alpha = p.get_float(0, 1.0f);
  n.beta = p.get_float(1, 1.0f);
  n.O = static_cast<int>(p.get_int(8, 0));
  n.K = static_cast<int>(p.get_int(9, 0));
  n.term = static_cast<int>(p.get_int(18, 0));
  if (ti.rank != 2 || ti.w != n.K) return fail(err, where + "A must be a rank-2 [M,K] tensor");
  const WeightTensor& wt = l.weights[0];
  size_t wi = 1;
  if (p.get_int(10, 0) == 4) {
    n.has_bias = true;
    n.bias = l.weights[wi++].as_f32();
    // reference order: y = (A*B^T + beta*C) * alpha; beta*C is one fp32 product
    for (float& b : n.bias) {
      volatile float t = b * n.beta;
      b = t;
    }
  }
  if (n.term != 0) {
    n.s_b = l.weights[wi++].as_f32()[0];
    if (wt.type == WeightType::kI8) {
      n.w_i8.assign(wt.as_i8(), wt.as_i8() + wt.count());
    } else {
      const std::vector<float> wf = wt.as_f32();
      n.w_i8.resize(wf.size());
      for (size_t i = 0; i < wf.size(); ++i) n.w_i8[i] = static_cast<int8_t>(host_quantize(wf[i], n.s_b));
    }
  } else {
    if (wt.type == WeightType::kI8) return fail(err, where + "int8 B requires int8_scale_term");
    n.w_f32 = wt.as_f32();
  }
  n.in = {in};
  n.out = new_tensor(l.tops[0]);
  Tensor& to = tensors_[n.out];
  to.rank = 2;
  to.h = ti.h;
  to.w = n.O;
  n.flops = 2.0 * ti.h * n.K * n.O;
  nodes_.push_back(std::move(n));
  return true;
}

bool EngineImpl::import_pool(const LayerDef& l, std::string* err) {
  const std::string where = "layer " + l.name + " (Pooling): ";
  const int in = by_name_.at(l.bottoms[0]);
  const Tensor ti = tensors_[resolve(in)];  // copy: new_tensor() below may reallocate
  if (ti.rank != 3) return fail(err, where + "pooling input must have [C,H,W] layout");
  const ParamDict& p = l.params;
  const int kind = static_cast<int>(p.get_int(0, 0));
  int kw = static_cast<int>(p.get_int(1, 0)), kh = static_cast<int>(p.get_int(11, kw));
  int sw = static_cast<int>(p.get_int(2, 1)), sh = static_cast<int>(p.get_int(12, sw));
  int pl = static_cast<int>(p.get_int(3, 0)), pr = static_cast<int>(p.get_int(14, pl));
  int pt = static_cast<int>(p.get_int(13, pl)), pb = static_cast<int>(p.get_int(15, pt));
  const int global = static_cast<int>(p.get_int(4, 0));
  const int mode = static_cast<int>(p.get_int(5, 0));
  if (kind != 0 && kind != 1) return fail(err, where + "pooling kind or boolean mode parameter is invalid");
  if (mode < 0 || mode > 3) return fail(err, where + "pooling pad_mode must be in [0, 3]");
  const int64_t adaptive = p.get_int(7, 0);
  if ((global != 0 && global != 1) || (adaptive != 0 && adaptive != 1))
    return fail(err, where + "pooling kind or boolean mode parameter is invalid");
  if (adaptive && !global && ti.i8) return fail(err, where + "dynamic or adaptive signed i8 pooling is not supported");
  if (ti.i8 && kind != 0) return fail(err, where + "signed i8 pooling only supports maximum");
  Node n;
  n.kind = N_POOL;
  n.name = l.name;
  n.type = l.type;
  n.in = {in};
  n.out = new_tensor(l.tops[0]);
  Tensor& to = tensors_[n.out];
  to.i8 = ti.i8;
  PoolParams& pp = n.pool;
  pp.kind = kind;
  pp.H = ti.h;
  pp.W = ti.w;
  pp.C = ti.c;
  if (global) {
    // ImportPooling.cpp:71-77: pads and include_pad are ignored, result shape is [C]
    pp.KH = ti.h;
    pp.KW = ti.w;
    pp.sh = pp.sw = 1;
    pp.pt = pp.pl = 0;
    pp.OH = pp.OW = 1;
    to.rank = 1;
    to.w = ti.c;
  } else if (adaptive) {
    // ImportPooling.cpp:66-69, NCNNOps.cpp:577-586: out_w (8) / out_h (18, default out_w), -233 = the input extent
    const int64_t out_w = p.get_int(8, 0), out_h = p.get_int(18, out_w);
    pp.OH = out_h == -233 ? ti.h : static_cast<int>(out_h);
    pp.OW = out_w == -233 ? ti.w : static_cast<int>(out_w);
    if (pp.OH <= 0 || pp.OW <= 0) return fail(err, where + "adaptive pooling output dimensions must be positive");
    pp.adaptive = 1;
    pp.KH = pp.KW = pp.sh = pp.sw = 1;
    pp.pt = pp.pl = 0;
    to.rank = 3;
    to.c = ti.c;
    to.h = pp.OH;
    to.w = pp.OW;
  } else {
    if (kw <= 0 || kh <= 0 || sw <= 0 || sh <= 0) return fail(err, where + "kernel and stride must be positive");
    if (pl < 0 || pr < 0 || pt < 0 || pb < 0) return fail(err, where + "padding must be non-negative");
    if (p.get_int(6, 0) == 1 && kind == 1 && (pl || pr || pt || pb))
      return fail(err, where + "avgpool_count_include_pad=1 with padding is rejected, as the reference's strict gate does");
    auto extent = [&](int inp, int k, int s, int p0, int p1) {
      // inferRegularDimension (NCNNOps.cpp:488-531)
      if (mode == 2 || mode == 3) return 1 + (inp - 1) / s;
      const int num = inp + p0 + p1;
      if (mode == 0) {
        const int diff = num - k;
        return (diff % s == 0 ? 1 : 2) + diff / s;
      }
      return 1 + (num - k) / s;
    };
    if (mode == 2 || mode == 3) {
      same_pads(ti.h, kh, sh, 1, mode == 3, &pt, &pb);
      same_pads(ti.w, kw, sw, 1, mode == 3, &pl, &pr);
    } else if (ti.h + pt + pb < kh || ti.w + pl + pr < kw) {
      return fail(err, where + "kernel exceeds padded input");
    }
    pp.KH = kh;
    pp.KW = kw;
    pp.sh = sh;
    pp.sw = sw;
    pp.pt = pt;
    pp.pl = pl;
    pp.OH = extent(ti.h, kh, sh, pt, pb);
    pp.OW = extent(ti.w, kw, sw, pl, pr);
    to.rank = 3;
    to.c = ti.c;
    to.h = pp.OH;
    to.w = pp.OW;
  }
  nodes_.push_back(std::move(n));
  return true;
}

bool EngineImpl::import_layers(std::string* err) {
  size_t next_shape = 0;
  for (const LayerDef& l : model_.layers) {
    const std::string where = "layer " + l.name + " (" + l.type + "): ";
    for (const auto& b : l.bottoms)
      if (by_name_.find(b) == by_name_.end()) return fail(err, where + "unknown bottom blob " + b);
    const std::string& t = l.type;
    // every importer below reads bottoms[0] and tops[0]: a line without them is malformed, not a crash
    if (t != "Input" && (l.bottoms.empty() || l.tops.empty()))
      return fail(err, where + "layer needs at least one bottom and one top blob");
    if (t == "Input") {
      // ImportInput.cpp:22-80: w/h/c all given (rank 3) or all omitted plus an override
      const int64_t w = l.params.get_int(0, 0), h = l.params.get_int(1, 0), c = l.params.get_int(2, 0);
      for (const auto& top : l.tops) {
        const int id = new_tensor(top);
        Tensor& x = tensors_[id];
        if (w == 0 && h == 0 && c == 0) {
          if (next_shape >= opt_.input_shapes.size())
            return fail(err, where + "Input dimensions are omitted without an override");
          const auto& s = opt_.input_shapes[next_shape++];
          if (s.empty() || s.size() > 3) return fail(err, where + "input shape override must have rank 1..3");
          for (int64_t d : s)
            if (d <= 0) return fail(err, where + "input shape override must have positive extents");
          x.rank = static_cast<int>(s.size());
          if (x.rank == 3) {
            x.c = static_cast<int>(s[0]);
            x.h = static_cast<int>(s[1]);
            x.w = static_cast<int>(s[2]);
          } else if (x.rank == 2) {
            x.h = static_cast<int>(s[0]);
            x.w = static_cast<int>(s[1]);
          } else {
            x.w = static_cast<int>(s[0]);
          }
        } else {
          if (w <= 0 || h <= 0 || c <= 0 || l.params.get_int(11, 0) != 0)
            return fail(err, where + "Input requires positive w/h/c and unsupported depth must be 0");
          x.rank = 3;
          x.c = static_cast<int>(c);
          x.h = static_cast<int>(h);
          x.w = static_cast<int>(w);
        }
        x.is_input = true;
        x.input_index = static_cast<int>(inputs_.size());
        inputs_.push_back(id);
      }
    } else if (t == "Convolution") {
      if (!import_conv(l, false, err)) return false;
    } else if (t == "ConvolutionDepthWise") {
      if (!import_conv(l, true, err)) return false;
    } else if (t == "InnerProduct") {
      if (!import_ip(l, err)) return false;
    } else if (t == "Gemm") {
      if (!import_gemm(l, err)) return false;
    } else if (t == "Pooling") {
      if (!import_pool(l, err)) return false;
    } else if (t == "Split") {
      const int in = by_name_.at(l.bottoms[0]);
      for (const auto& top : l.tops) {
        const int id = new_tensor(top);
        tensors_[id] = tensors_[resolve(in)];
        tensors_[id].name = top;
        tensors_[id].alias = resolve(in);
        tensors_[id].is_input = false;
      }
    } else if (t == "ReLU" || t == "Clip") {
      const int in = by_name_.at(l.bottoms[0]);
      const Tensor ti = tensors_[resolve(in)];
      Node n;
      n.kind = N_UNARY;
      n.name = l.name;
      n.type = t;
      n.un.op = UN_ACT;
      if (t == "ReLU") {
        const float slope = l.params.get_float(0, 0.0f);
        n.un.inner = 1;
        n.un.channels = 1;
        n.un.act = slope == 0.0f ? ACT_RELU : ACT_LEAKY;
        n.un.act_a = slope;
        if (ti.i8 && slope != 0.0f) return fail(err, where + "leaky ReLU on an int8 tensor is not supported");
      } else {
        // Extension: the reference has no Clip importer (NCNNImporter.cpp:110-160).
        // ncnn semantics: min(max(x, min), max).
        if (ti.i8) return fail(err, where + "Clip on an int8 tensor is not supported");
        n.un.act = ACT_CLIP;
        n.un.act_a = l.params.get_float(0, -std::numeric_limits<float>::max());
        n.un.act_b = l.params.get_float(1, std::numeric_limits<float>::max());
      }
      n.in = {in};
      n.out = new_tensor(l.tops[0]);
      Tensor& to = tensors_[n.out];
      const std::string keep = to.name;
      to = ti;
      to.name = keep;
      to.alias = -1;
      to.is_input = false;
      nodes_.push_back(std::move(n));
    } else if (t == "Sigmoid" || t == "Swish" || t == "TanH" || t == "HardSigmoid" || t == "HardSwish" ||
               t == "Dropout" || t == "GELU" || t == "PReLU") {
      if (l.bottoms.size() != 1 || l.tops.size() != 1) return fail(err, where + "expects one input and one output");
      const int in = by_name_.at(l.bottoms[0]);
      const Tensor ti = tensors_[resolve(in)];
      if (ti.i8) return fail(err, where + "supports one f32 tensor only");
      const bool hard = t == "HardSigmoid" || t == "HardSwish";
      const int max_id = hard ? 1 : (t == "Dropout" || t == "GELU" || t == "PReLU" ? 0 : -1);
      // validate_param_ids (NCNNImporter.cpp:271-282): ids 30 and 31 are always allowed
      for (const auto& entry : l.params.entries())
        if ((entry.first > max_id || entry.first < 0) && entry.first != 30 && entry.first != 31)
          return fail(err, where + "unsupported parameter id " + std::to_string(entry.first));
      Node n;
      n.kind = N_UNARY;
      n.name = l.name;
      n.type = t;
      n.un.op = UN_ACT;
      n.un.inner = 1;
      n.un.channels = 1;
      if (hard) {
        // ImportOps.cpp:120-157: alpha (default 0.2, must be positive), beta (default 0.5)
        n.un.act = t == "HardSwish" ? ACT_HARDSWISH : ACT_HARDSIGMOID;
        n.un.act_a = l.params.get_float(0, 0.2f);
        n.un.act_b = l.params.get_float(1, 0.5f);
        if (!(n.un.act_a > 0.0f)) return fail(err, where + "alpha must be positive");
      } else if (t == "Dropout") {
        // ImportActivation.cpp:617-646, ConvertDropout (NCNNToTosa.cpp:2047-2070): x * scale, identity for 1
        n.un.act = ACT_SCALE;
        n.un.act_a = l.params.get_float(0, 1.0f);
      } else if (t == "GELU") {
        // import_gelu (ImportActivation.cpp:543-564): the erf form only
        if (l.params.get_int(0, 0) != 0) return fail(err, where + "invalid GELU parameters");
        n.un.act = ACT_GELU;
      } else if (t == "PReLU") {
        // import_prelu (ImportActivation.cpp:504-541): one finite scalar slope, lowered as a leaky ReLU
        if (l.params.get_int(0, 0) != 1 || l.weights.size() != 1 || l.weights[0].count() != 1)
          return fail(err, where + "PReLU supports exactly one FP32 scalar slope");
        const float slope = l.weights[0].as_f32()[0];
        if (!std::isfinite(slope)) return fail(err, where + "PReLU slope must be finite");
        n.un.act = ACT_LEAKY;
        n.un.act_a = slope;
      } else {
        n.un.act = t == "Sigmoid" ? ACT_SIGMOID : (t == "Swish" ? ACT_SWISH : ACT_TANH);
      }
      if (n.un.act == ACT_SCALE && n.un.act_a == 1.0f) {
        const int id = new_tensor(l.tops[0]);
        tensors_[id] = tensors_[resolve(in)];
        tensors_[id].name = l.tops[0];
        tensors_[id].alias = resolve(in);
        tensors_[id].is_input = false;
      } else {
        n.in = {in};
        n.out = new_tensor(l.tops[0]);
        Tensor& to = tensors_[n.out];
        const std::string keep = to.name;
        to = ti;
        to.name = keep;
        to.alias = -1;
        to.is_input = false;
        nodes_.push_back(std::move(n));
      }
    } else if (t == "Softmax") {
      // ImportActivation.cpp:648-695: axis (default 0) over the logical [c,h,w] / [h,w] / [w] dims,
      // negative counts from the end; anything but axis 0 needs fixbug0 = 1; rank 1 forces axis 0
      if (l.bottoms.size() != 1 || l.tops.size() != 1) return fail(err, where + "expects one input and one output");
      const int in = by_name_.at(l.bottoms[0]);
      const Tensor ti = tensors_[resolve(in)];
      if (ti.i8) return fail(err, where + "supports one f32 tensor only");
      int64_t axis = l.params.get_int(0, 0);
      const int64_t fixbug = l.params.get_int(1, 0);
      if (fixbug != 0 && fixbug != 1) return fail(err, where + "fixbug0 must be 0 or 1");
      if (fixbug == 0 && axis != 0) return fail(err, where + "legacy Softmax only supports axis 0 unless fixbug0 is 1");
      if (ti.rank == 1) axis = 0;
      if (axis < 0) axis += ti.rank;
      if (axis < 0 || axis >= ti.rank) return fail(err, where + "axis is out of range");
      Node n;
      n.kind = N_SOFTMAX;
      n.name = l.name;
      n.type = t;
      // storage order: rank 3 [h][w][c]; logical axis 0 = c, 1 = h, 2 = w
      SoftmaxParams& sp = n.softmax;
      sp.image_elems = ti.logical();
      if (ti.rank == 3) {
        if (axis == 0) { sp.len = ti.c; sp.inner = 1; }
        else if (axis == 1) { sp.len = ti.h; sp.inner = ti.w * ti.c; }
        else { sp.len = ti.w; sp.inner = ti.c; }
      } else if (ti.rank == 2) {
        if (axis == 0) { sp.len = ti.h; sp.inner = ti.w; }
        else { sp.len = ti.w; sp.inner = 1; }
      } else {
        sp.len = ti.w;
        sp.inner = 1;
      }
      sp.lines = static_cast<int>(ti.logical() / sp.len);
      n.in = {in};
      n.out = new_tensor(l.tops[0]);
      Tensor& to = tensors_[n.out];
      const std::string keep = to.name;
      to = ti;
      to.name = keep;
      to.alias = -1;
      to.is_input = false;
      nodes_.push_back(std::move(n));
    } else if (t == "Concat") {
      // ImportTensor.cpp:48-96: at least two inputs, axis (default 0) over the logical dims
      if (l.bottoms.size() < 2 || l.tops.size() != 1) return fail(err, where + "requires at least two inputs and one output");
      const Tensor t0 = tensors_[resolve(by_name_.at(l.bottoms[0]))];
      int64_t axis = l.params.get_int(0, 0);
      if (axis < 0) axis += t0.rank;
      if (axis < 0 || axis >= t0.rank) return fail(err, where + "axis is out of range");
      Node n;
      n.kind = N_CONCAT;
      n.name = l.name;
      n.type = t;
      auto dims_of = [](const Tensor& x) {
        std::vector<int> d;
        if (x.rank == 3) d = {x.c, x.h, x.w};
        else if (x.rank == 2) d = {x.h, x.w};
        else d = {x.w};
        return d;
      };
      std::vector<int> od = dims_of(t0);
      od[axis] = 0;
      for (const std::string& b : l.bottoms) {
        const int id = by_name_.at(b);
        const Tensor& tb = tensors_[resolve(id)];
        if (tb.rank != t0.rank || tb.i8 != t0.i8) return fail(err, where + "inputs must agree in rank and element type");
        const std::vector<int> d = dims_of(tb);
        for (int k = 0; k < t0.rank; ++k)
          if (k != axis && d[k] != dims_of(t0)[k]) return fail(err, where + "inputs must agree outside the concatenation axis");
        od[axis] += d[axis];
        n.in.push_back(id);
      }
      n.out = new_tensor(l.tops[0]);
      Tensor& to = tensors_[n.out];
      const std::string keep = to.name;
      to = t0;
      to.name = keep;
      to.alias = -1;
      to.is_input = false;
      if (t0.rank == 3) { to.c = od[0]; to.h = od[1]; to.w = od[2]; }
      else if (t0.rank == 2) { to.h = od[0]; to.w = od[1]; }
      else to.w = od[0];
      // storage order: rank 3 [h][w][c] -> concatenation axis as (outer, len, inner)
      int offset = 0;
      for (int id : n.in) {
        const Tensor& tb = tensors_[resolve(id)];
        ConcatParams cp{};
        cp.in_image_elems = tb.logical();
        cp.out_image_elems = to.logical();
        if (t0.rank == 3) {
          if (axis == 0) { cp.outer = tb.h * tb.w; cp.len_in = tb.c; cp.len_out = to.c; cp.inner = 1; }
          else if (axis == 1) { cp.outer = 1; cp.len_in = tb.h; cp.len_out = to.h; cp.inner = tb.w * tb.c; }
          else { cp.outer = tb.h; cp.len_in = tb.w; cp.len_out = to.w; cp.inner = tb.c; }
        } else if (t0.rank == 2) {
          if (axis == 0) { cp.outer = 1; cp.len_in = tb.h; cp.len_out = to.h; cp.inner = tb.w; }
          else { cp.outer = tb.h; cp.len_in = tb.w; cp.len_out = to.w; cp.inner = 1; }
        } else {
          cp.outer = 1; cp.len_in = tb.w; cp.len_out = to.w; cp.inner = 1;
        }
        cp.offset = offset;
        offset += cp.len_in;
        n.concat.push_back(cp);
      }
      nodes_.push_back(std::move(n));
    } else if (t == "Eltwise" || t == "BinaryOp") {
      Node n;
      n.kind = N_BINARY;
      n.name = l.name;
      n.type = t;
      const int a = by_name_.at(l.bottoms[0]);
      const Tensor ta = tensors_[resolve(a)];
      if (t == "Eltwise") {
        // ImportOps.cpp:435-506: two inputs, SUM, optional two coefficients
        const std::vector<float>* coeff = l.params.get_float_array(1);
        if (l.bottoms.size() != 2 || l.params.get_int(0, 1) != 1 || (coeff != nullptr && coeff->size() != 2) ||
            (l.params.has(1) && coeff == nullptr))
          return fail(err, where + "Eltwise supports unweighted or coefficient-weighted SUM of two inputs only");
        n.bin.op = BIN_ADD;
        if (coeff != nullptr) {
          n.bin.scale_a = (*coeff)[0] != 1.0f;
          n.bin.scale_b = (*coeff)[1] != 1.0f;
          n.bin.ca = (*coeff)[0];
          n.bin.cb = (*coeff)[1];
        }
      } else {
        const int64_t op = l.params.get_int(0, 0);
        if (op != 0 && op != 1 && op != 2 && op != 4) return fail(err, where + "BinaryOp supports add, sub, mul and max");
        n.bin.op = static_cast<int>(op);
        n.bin.use_scalar = l.params.get_int(1, 0) == 1;
        n.bin.scalar = l.params.get_float(2, 0.0f);
        if (!n.bin.use_scalar && l.bottoms.size() != 2) return fail(err, where + "BinaryOp needs two inputs or a scalar");
      }
      n.in = {a};
      if (!n.bin.use_scalar) {
        const int b = by_name_.at(l.bottoms[1]);
        const Tensor& tb = tensors_[resolve(b)];
        if (ta.i8 != tb.i8 || (ta.i8 && n.bin.op != BIN_MAX))
          return fail(err, where + "int8 operands support only two-input max");
        if (tb.rank != ta.rank || tb.c != ta.c || tb.h != ta.h || tb.w != ta.w) {
          // computeBinaryResult (NCNNOps.cpp:1219-1244): right-aligned broadcasting of the logical dims
          if (t == "Eltwise" || ta.i8) return fail(err, where + "operands must have the same shape");
          auto dims3 = [](const Tensor& x, int d[3]) {
            d[0] = x.rank == 3 ? x.c : 1;
            d[1] = x.rank >= 2 ? x.h : 1;
            d[2] = x.w;
          };
          int da[3], db[3], dout[3];
          dims3(ta, da);
          dims3(tb, db);
          for (int k = 0; k < 3; ++k) {
            if (da[k] == 1) dout[k] = db[k];
            else if (db[k] == 1 || db[k] == da[k]) dout[k] = da[k];
            else return fail(err, where + "BinaryOp input shapes are not broadcastable");
          }
          n.broadcast = true;
          BroadcastParams& bp = n.bcast;
          bp.rank = std::max(ta.rank, tb.rank);
          bp.C = dout[0];
          bp.H = dout[1];
          bp.W = dout[2];
          auto strides = [](const Tensor& x, const int d[3], int* sc, int* sh, int* sw) {
            // storage: rank 3 [h][w][c], rank 2 [h][w], rank 1 [w]
            const int c_stride = 1, w_stride = x.rank == 3 ? x.c : 1, h_stride = x.rank == 3 ? x.w * x.c : x.w;
            *sc = (x.rank == 3 && d[0] != 1) ? c_stride : 0;
            *sh = (x.rank >= 2 && d[1] != 1) ? h_stride : 0;
            *sw = d[2] != 1 ? w_stride : 0;
          };
          strides(ta, da, &bp.a_sc, &bp.a_sh, &bp.a_sw);
          strides(tb, db, &bp.b_sc, &bp.b_sh, &bp.b_sw);
          bp.a_image = ta.logical();
          bp.b_image = tb.logical();
          bp.o_image = static_cast<long long>(dout[0]) * dout[1] * dout[2];
        }
        n.in.push_back(b);
      } else if (ta.i8) {
        return fail(err, where + "int8 operands support only two-input max");
      }
      n.out = new_tensor(l.tops[0]);
      Tensor& to = tensors_[n.out];
      const std::string keep = to.name;
      to = ta;
      to.name = keep;
      to.alias = -1;
      to.is_input = false;
      if (n.broadcast) {
        to.rank = n.bcast.rank;
        to.c = n.bcast.C;
        to.h = n.bcast.H;
        to.w = n.bcast.W;
        to.Cp = to.rank == 3 ? to.c : 1;
        to.Wp = to.w;
      }
      nodes_.push_back(std::move(n));
    } else if (t == "UnaryOp") {
      // import_unary_op (ImportOps.cpp:407-433): the square operation only
      if (l.bottoms.size() != 1 || l.tops.size() != 1) return fail(err, where + "expects one input and one output");
      const int in = by_name_.at(l.bottoms[0]);
      const Tensor ti = tensors_[resolve(in)];
      if (ti.i8 || l.params.get_int(0, 0) != 4) return fail(err, where + "UnaryOp supports the square operation (op_type=4) on f32 only");
      Node n;
      n.kind = N_UNARY;
      n.name = l.name;
      n.type = t;
      n.un.op = UN_ACT;
      n.un.act = ACT_SQUARE;
      n.in = {in};
      n.out = new_tensor(l.tops[0]);
      Tensor& to = tensors_[n.out];
      const std::string keep = to.name;
      to = ti;
      to.name = keep;
      to.alias = -1;
      to.is_input = false;
      nodes_.push_back(std::move(n));
    } else if (t == "Slice") {
      // import_slice (ImportTensor.cpp:136-193) + inferSliceResults (NCNNOps.cpp:1538-1591)
      if (l.bottoms.size() != 1 || l.tops.size() < 2) return fail(err, where + "requires one input and at least two outputs");
      const int in = by_name_.at(l.bottoms[0]);
      const Tensor ti = tensors_[resolve(in)];
      if (ti.i8) return fail(err, where + "Slice input must be f32");
      const std::vector<int64_t>* sizes = l.params.get_int_array(0);
      if (sizes == nullptr) return fail(err, where + "parameter 0 (slices) must be an integer array");
      if (sizes->size() != l.tops.size()) return fail(err, where + "slice count must match output count");
      int64_t axis = l.params.get_int(1, 0);
      if (axis < 0) axis += ti.rank;
      if (axis < 0 || axis >= ti.rank) return fail(err, where + "Slice axis is outside input rank");
      std::vector<int> dims;
      if (ti.rank == 3) dims = {ti.c, ti.h, ti.w};
      else if (ti.rank == 2) dims = {ti.h, ti.w};
      else dims = {ti.w};
      const int extent = dims[axis];
      int consumed = 0;
      for (size_t k = 0; k < sizes->size(); ++k) {
        int64_t size = (*sizes)[k];
        if (size == -233) size = (extent - consumed) / static_cast<int64_t>(sizes->size() - k);
        if (size <= 0 || size > extent - consumed) return fail(err, where + "Slice sizes must be positive and fit input");
        Node n;
        n.kind = N_CONCAT;
        n.name = l.name + ":" + std::to_string(k);
        n.type = t;
        n.in = {in};
        n.out = new_tensor(l.tops[k]);
        Tensor& to = tensors_[n.out];
        const std::string keep = to.name;
        to = ti;
        to.name = keep;
        to.alias = -1;
        to.is_input = false;
        std::vector<int> od = dims;
        od[axis] = static_cast<int>(size);
        if (ti.rank == 3) { to.c = od[0]; to.h = od[1]; to.w = od[2]; to.Cp = to.c; to.Wp = to.w; }
        else if (ti.rank == 2) { to.h = od[0]; to.w = od[1]; to.Wp = to.w; }
        else { to.w = od[0]; to.Wp = to.w; }
        ConcatParams cp{};
        cp.slice = 1;
        cp.in_image_elems = to.logical();
        cp.out_image_elems = ti.logical();
        if (ti.rank == 3) {
          if (axis == 0) { cp.outer = ti.h * ti.w; cp.len_in = to.c; cp.len_out = ti.c; cp.inner = 1; }
          else if (axis == 1) { cp.outer = 1; cp.len_in = to.h; cp.len_out = ti.h; cp.inner = ti.w * ti.c; }
          else { cp.outer = ti.h; cp.len_in = to.w; cp.len_out = ti.w; cp.inner = ti.c; }
        } else if (ti.rank == 2) {
          if (axis == 0) { cp.outer = 1; cp.len_in = to.h; cp.len_out = ti.h; cp.inner = ti.w; }
          else { cp.outer = ti.h; cp.len_in = to.w; cp.len_out = ti.w; cp.inner = 1; }
        } else {
          cp.outer = 1; cp.len_in = to.w; cp.len_out = ti.w; cp.inner = 1;
        }
        cp.offset = consumed;
        consumed += static_cast<int>(size);
        n.concat.push_back(cp);
        nodes_.push_back(std::move(n));
      }
      if (consumed != extent) return fail(err, where + "Slice sizes must consume the entire axis");
    } else if (t == "Reduction") {
      // import_reduction (ImportTensor.cpp:195-255) + computeReductionResult (NCNNOps.cpp:1593-1640):
      // f32 mean only; explicit axes need fixbug0 = 1
      if (l.bottoms.size() != 1 || l.tops.size() != 1) return fail(err, where + "expects one input and one output");
      const int in = by_name_.at(l.bottoms[0]);
      const Tensor ti = tensors_[resolve(in)];
      const int64_t reduce_all = l.params.get_int(1, 1), keep = l.params.get_int(4, 0);
      const std::vector<int64_t>* axes = l.params.get_int_array(3);
      if (ti.i8 || l.params.get_int(0, 0) != 3 || (reduce_all != 0 && reduce_all != 1) || (keep != 0 && keep != 1) ||
          (l.params.has(3) && axes == nullptr))
        return fail(err, where + "Reduction supports static FP32 mean with integer axes only");
      if (!reduce_all && (axes == nullptr || axes->empty() || l.params.get_int(5, 0) != 1))
        return fail(err, where + "explicit Reduction axes require fixbug0=1");
      if (ti.rank != 3) return fail(err, where + "Reduction of tensors that are not rank 3 is outside the supported path");
      bool red[3] = {reduce_all != 0, reduce_all != 0, reduce_all != 0};
      if (!reduce_all) {
        for (int64_t a : *axes) {
          if (a < 0) a += 3;
          if (a < 0 || a > 2 || red[a]) return fail(err, where + "Reduction axes must be unique and in range");
          red[a] = true;
        }
      }
      std::vector<int> kept;
      const int dims[3] = {ti.c, ti.h, ti.w};
      long long count = 1;
      for (int a = 0; a < 3; ++a) {
        if (red[a]) count *= dims[a];
        if (!red[a]) kept.push_back(dims[a]);
        else if (keep) kept.push_back(1);
      }
      if (kept.empty()) kept.push_back(1);
      // Without keepdims, dropping only h or only w leaves a rank-2 result whose element order the
      // reference takes from a plain reshape of its channel-last buffer; that case stays out.
      if (!keep && kept.size() == 2 && !red[0]) return fail(err, where + "this combination of Reduction axes is outside the supported path");
      Node n;
      n.kind = N_REDUCE;
      n.name = l.name;
      n.type = t;
      n.reduce.C = ti.c;
      n.reduce.H = ti.h;
      n.reduce.W = ti.w;
      n.reduce.red_c = red[0];
      n.reduce.red_h = red[1];
      n.reduce.red_w = red[2];
      n.reduce.factor = static_cast<float>(static_cast<double>(l.params.get_float(2, 1.0f)) / static_cast<double>(count));
      n.in = {in};
      n.out = new_tensor(l.tops[0]);
      Tensor& to = tensors_[n.out];
      const std::string keep_name = to.name;
      to = ti;
      to.name = keep_name;
      to.alias = -1;
      to.is_input = false;
      to.rank = static_cast<int>(kept.size());
      to.w = kept.back();
      to.h = to.rank >= 2 ? kept[to.rank - 2] : 1;
      to.c = to.rank == 3 ? kept[0] : 1;
      to.Cp = to.rank == 3 ? to.c : 1;
      to.Wp = to.w;
      nodes_.push_back(std::move(n));
    } else if (t == "ShuffleChannel" || t == "Padding" || t == "Interp") {
      if (l.bottoms.size() != 1 || l.tops.size() != 1)
        return fail(err, where + (t == "Interp" ? "a dynamic target size is outside the supported path" : "expects one input and one output"));
      const int in = by_name_.at(l.bottoms[0]);
      const Tensor ti = tensors_[resolve(in)];
      if (ti.i8 || ti.rank != 3) return fail(err, where + "requires a rank-3 f32 input");
      Node n;
      n.kind = N_REMAP;
      n.name = l.name;
      n.type = t;
      RemapParams& r = n.remap;
      r.C = ti.c;
      r.H = ti.h;
      r.W = ti.w;
      r.OH = ti.h;
      r.OW = ti.w;
      if (t == "ShuffleChannel") {
        // import_shuffle_channel (ImportTensor.cpp:98-134), ConvertShuffleChannel (NCNNToTosa.cpp:5394-5456)
        const int64_t group = l.params.get_int(0, 1), reverse = l.params.get_int(1, 0);
        if ((reverse != 0 && reverse != 1) || group <= 0) return fail(err, where + "group must be positive and reverse 0 or 1");
        if (ti.c % group != 0) return fail(err, where + "group must divide channel count");
        r.mode = REMAP_SHUFFLE;
        r.group = static_cast<int>(reverse ? ti.c / group : group);
      } else if (t == "Padding") {
        // import_padding (ImportDetection.cpp:31-112): constant spatial padding only
        const int64_t top = l.params.get_int(0, 0), bottom = l.params.get_int(1, 0), left = l.params.get_int(2, 0),
                      right = l.params.get_int(3, 0);
        if (l.params.get_int(4, 0) != 0 || l.params.get_int(6, 0) != 0 || l.params.get_int(7, 0) != 0 ||
            l.params.get_int(8, 0) != 0)
          return fail(err, where + "Padding only supports constant spatial padding without per-channel data");
        if (top < 0 || bottom < 0 || left < 0 || right < 0) return fail(err, where + "padding must be non-negative");
        r.mode = REMAP_PAD;
        r.top = static_cast<int>(top);
        r.left = static_cast<int>(left);
        r.value = l.params.get_float(5, 0.0f);
        r.OH = static_cast<int>(ti.h + top + bottom);
        r.OW = static_cast<int>(ti.w + left + right);
      } else {
        // import_interp (ImportDetection.cpp:114-205)
        const int64_t type = l.params.get_int(0, 0), oh = l.params.get_int(3, 0), ow = l.params.get_int(4, 0),
                      align = l.params.get_int(6, 0);
        const float hs = l.params.get_float(1, 1.0f), ws = l.params.get_float(2, 1.0f);
        if ((type != 1 && type != 2) || (type == 1 && align != 0) || (align != 0 && align != 1) ||
            l.params.get_int(5, 0) != 0 || l.params.has(9) || !std::isfinite(hs) || !std::isfinite(ws) || hs < 1.0f ||
            ws < 1.0f || std::trunc(hs) != hs || std::trunc(ws) != ws || oh < 0 || ow < 0)
          return fail(err, where + "Interp supports nearest or bilinear resize with valid integer scale and alignment only");
        r.mode = type == 1 ? REMAP_NEAREST : REMAP_BILINEAR;
        r.scale_h = static_cast<int>(hs);
        r.scale_w = static_cast<int>(ws);
        r.explicit_h = oh != 0;
        r.explicit_w = ow != 0;
        r.align_corner = static_cast<int>(align);
        r.OH = static_cast<int>(oh != 0 ? oh : ti.h * r.scale_h);
        r.OW = static_cast<int>(ow != 0 ? ow : ti.w * r.scale_w);
        if (type == 2 && (ti.h < 2 || ti.w < 2)) return fail(err, where + "bilinear resize needs at least two rows and columns");
      }
      n.in = {in};
      n.out = new_tensor(l.tops[0]);
      Tensor& to = tensors_[n.out];
      const std::string keep = to.name;
      to = ti;
      to.name = keep;
      to.alias = -1;
      to.is_input = false;
      to.h = r.OH;
      to.w = r.OW;
      to.Wp = to.w;
      nodes_.push_back(std::move(n));
    } else if (t == "BatchNorm") {
      const int in = by_name_.at(l.bottoms[0]);
      const Tensor ti = tensors_[resolve(in)];
      if (l.weights.size() != 4) return fail(err, where + "weights are missing (was a .bin supplied?)");
      const int ch = static_cast<int>(l.params.get_int(0, 0));
      // channel axis: the last storage axis for rank 3, dimension 0 otherwise (NCNNToTosa.cpp:4752-4754)
      if (ti.i8 || (ti.rank == 3 && ti.c != ch) || (ti.rank == 1 && ti.w != ch) || (ti.rank == 2 && ti.h != ch))
        return fail(err, where + "BatchNorm channel count does not match its input");
      const float eps = l.params.get_float(1, 0.0f);
      const std::vector<float> slope = l.weights[0].as_f32(), mean = l.weights[1].as_f32(),
                               var = l.weights[2].as_f32(), bias = l.weights[3].as_f32();
      Node n;
      n.kind = N_UNARY;
      n.name = l.name;
      n.type = t;
      n.un.op = UN_AFFINE;
      n.un.channels = ch;
      n.un.inner = ti.rank == 2 ? ti.w : 1;
      n.un_scale.resize(ch);
      n.un_offset.resize(ch);
      for (int c = 0; c < ch; ++c) {
        // FoldNCNNBatchNorm.cpp:99-124 / ConvertBatchNorm (NCNNToTosa.cpp:4740-4800)
        volatile float ve = var[c] + eps;
        const float inv = ve == 0.0f ? 10000.0f : std::pow(static_cast<float>(ve), -0.5f);
        volatile float scale = slope[c] * inv;
        volatile float sm = scale * mean[c];
        n.un_scale[c] = scale;
        n.un_offset[c] = bias[c] - sm;
      }
      n.in = {in};
      n.out = new_tensor(l.tops[0]);
      Tensor& to = tensors_[n.out];
      const std::string keep = to.name;
      to = ti;
      to.name = keep;
      to.alias = -1;
      to.is_input = false;
      nodes_.push_back(std::move(n));
    } else if (t == "Quantize") {
      const int in = by_name_.at(l.bottoms[0]);
      const Tensor ti = tensors_[resolve(in)];
      if (ti.i8 || l.weights.size() != 1) return fail(err, where + "Quantize needs an f32 input and its scale");
      Node n;
      n.kind = N_UNARY;
      n.name = l.name;
      n.type = t;
      n.un.op = UN_QUANT;
      n.un_scale = l.weights[0].as_f32();
      n.un.nscale = static_cast<int>(n.un_scale.size());
      n.un.channels = ti.rank == 3 ? ti.c : ti.w;
      n.un.inner = 1;
      // ConvertQuantize (NCNNToTosa.cpp:4802-4824): scalar scale or one per channel (dim 0)
      if (n.un.nscale != 1 && (n.un.nscale != n.un.channels || ti.rank == 2))
        return fail(err, where + "Quantize scale count must be 1 or the channel count");
      n.in = {in};
      n.out = new_tensor(l.tops[0]);
      Tensor& to = tensors_[n.out];
      const std::string keep = to.name;
      to = ti;
      to.name = keep;
      to.alias = -1;
      to.is_input = false;
      to.i8 = true;
      nodes_.push_back(std::move(n));
    } else if (t == "Flatten" || t == "Reshape" || t == "Squeeze" || t == "ExpandDims" || t == "Permute") {
      const int in = by_name_.at(l.bottoms[0]);
      const Tensor ti = tensors_[resolve(in)];
      Node n;
      n.kind = N_RELAYOUT;
      n.name = l.name;
      n.type = t;
      n.in = {in};
      n.out = new_tensor(l.tops[0]);
      Tensor& to = tensors_[n.out];
      to.i8 = ti.i8;
      bool transpose = false;
      if (t == "Flatten") {
        to.rank = 1;
        to.w = static_cast<int>(ti.logical());
      } else if (t == "Reshape") {
        // ncnn Reshape: 0=w 1=h 2=c, -233 marks an unused dimension, 0 copies, -1 infers
        int64_t d[3] = {l.params.get_int(0, -233), l.params.get_int(1, -233), l.params.get_int(2, -233)};
        const int src[3] = {ti.w, ti.rank >= 2 ? ti.h : 1, ti.rank == 3 ? ti.c : 1};
        int rank = d[2] != -233 ? 3 : (d[1] != -233 ? 2 : 1);
        long long known = 1;
        int infer = -1;
        for (int i = 0; i < rank; ++i) {
          if (d[i] == 0) d[i] = src[i];
          if (d[i] == -1) {
            infer = i;
          } else {
            known *= d[i];
          }
        }
        if (infer >= 0) d[infer] = ti.logical() / std::max<long long>(known, 1);
        long long total = 1;
        for (int i = 0; i < rank; ++i) total *= d[i];
        if (total != ti.logical()) return fail(err, where + "Reshape does not preserve the element count");
        to.rank = rank;
        to.w = static_cast<int>(d[0]);
        to.h = rank >= 2 ? static_cast<int>(d[1]) : 1;
        to.c = rank == 3 ? static_cast<int>(d[2]) : 1;
      } else if (t == "Squeeze" || t == "ExpandDims") {
        // explicit axes over the logical [c,h,w] order only (import_squeeze / import_expand_dims,
        // ImportTensor.cpp:270-341; computeSqueezeResult / computeExpandDimsResult, NCNNOps.cpp:868-927)
        const std::vector<int64_t>* axes = l.params.get_int_array(3);
        if (axes == nullptr) return fail(err, where + "parameter 3 (axes) must be an integer array");
        if (t == "Squeeze" && (l.params.has(0) || l.params.has(1) || l.params.has(2) || l.params.has(11)))
          return fail(err, where + "Squeeze requires explicit axes only");
        std::vector<int> dims;
        if (ti.rank == 3) dims = {ti.c, ti.h, ti.w};
        if (ti.rank == 2) dims = {ti.h, ti.w};
        if (ti.rank == 1) dims = {ti.w};
        std::vector<int> kept;
        if (t == "Squeeze") {
          std::vector<char> drop(dims.size(), 0);
          for (int64_t a : *axes) {
            if (a < 0) a += static_cast<int64_t>(dims.size());
            if (a < 0 || a >= static_cast<int64_t>(dims.size()) || drop[a] == 2)
              return fail(err, where + "Squeeze axes must be unique and in range");
            drop[a] = 2;
          }
          // a named axis whose extent is not 1 stays
          for (size_t i = 0; i < dims.size(); ++i)
            if (!(drop[i] == 2 && dims[i] == 1)) kept.push_back(dims[i]);
          if (kept.empty()) kept.push_back(1);
        } else {
          const int64_t out_rank = static_cast<int64_t>(dims.size() + axes->size());
          if (out_rank > 3) return fail(err, where + "rank-4 tensors are outside the supported path");
          std::vector<char> fresh(static_cast<size_t>(out_rank), 0);
          for (int64_t a : *axes) {
            if (a < 0) a += out_rank;
            if (a < 0 || a >= out_rank || fresh[a]) return fail(err, where + "ExpandDims axes must be unique and in output rank");
            fresh[a] = 1;
          }
          size_t next = 0;
          for (int64_t i = 0; i < out_rank; ++i) kept.push_back(fresh[i] ? 1 : dims[next++]);
        }
        to.rank = static_cast<int>(kept.size());
        to.w = kept.back();
        to.h = to.rank >= 2 ? kept[to.rank - 2] : 1;
        to.c = to.rank == 3 ? kept[0] : 1;
      } else {  // Permute
        // import_permute (ImportTensor.cpp:343-400): rank 2 order 0/1, rank 3 order 2 ([h,c,w]) or
        // 4 ([w,c,h]); result extent i is the input extent perm[i]
        const int64_t order = l.params.get_int(0, 0);
        if (ti.rank == 2 && (order == 0 || order == 1)) {
          to.rank = 2;
          if (order == 1) {
            to.h = ti.w;
            to.w = ti.h;
            transpose = true;
          } else {
            to.h = ti.h;
            to.w = ti.w;
          }
        } else if (ti.rank == 3 && (order == 2 || order == 4)) {
          const int src[3] = {ti.c, ti.h, ti.w};
          const int perm[3] = {order == 2 ? 1 : 2, 0, order == 2 ? 2 : 1};
          to.rank = 3;
          to.c = src[perm[0]];
          to.h = src[perm[1]];
          to.w = src[perm[2]];
          for (int i = 0; i < 3; ++i) n.relayout.perm[i] = perm[i];
          n.relayout.permute3d = 1;
        } else {
          return fail(err, where + "Permute supports rank-2 order 0/1 and rank-3 order 2/4 only");
        }
      }
      RelayoutParams& r = n.relayout;
      r.count = ti.logical();
      r.src_rank = ti.rank;
      r.sc = ti.c;
      r.sh = ti.h;
      r.sw = ti.w;
      r.dst_rank = to.rank;
      r.dc = to.c;
      r.dh = to.h;
      r.dw = to.w;
      r.transpose2d = transpose ? 1 : 0;
      nodes_.push_back(std::move(n));
    } else if (t == "Deconvolution") {
      // import_deconvolution (ImportDetection.cpp:349-470): static fp32 2x2 kernel, stride 2, no
      // padding, no output padding, activation none or ReLU
      if (l.bottoms.size() != 1 || l.tops.size() != 1) return fail(err, where + "expects one input and one output");
      static const int allowed[] = {0, 1, 2, 3, 4, 5, 6, 9, 10, 11, 12, 13, 14, 15, 16, 18, 19, 20, 21, 28, 30, 31};
      for (const auto& entry : l.params.entries())
        if (std::find(std::begin(allowed), std::end(allowed), entry.first) == std::end(allowed))
          return fail(err, where + "unsupported parameter id " + std::to_string(entry.first));
      const ParamDict& p = l.params;
      const int64_t kw = p.get_int(1, 0), kh = p.get_int(11, kw), dw = p.get_int(2, 1), dh = p.get_int(12, dw);
      const int64_t sw = p.get_int(3, 1), sh = p.get_int(13, sw), pl = p.get_int(4, 0), pr = p.get_int(15, pl);
      const int64_t pt = p.get_int(14, pl), pb = p.get_int(16, pt), opr = p.get_int(18, 0), opb = p.get_int(19, opr);
      const int64_t ow = p.get_int(20, 0), oh = p.get_int(21, ow), act = p.get_int(9, 0), has_bias = p.get_int(5, 0);
      if (p.get_int(28, 0) != 0 || kh != 2 || kw != 2 || sh != 2 || sw != 2 || dh != 1 || dw != 1 || pt != 0 || pb != 0 ||
          pl != 0 || pr != 0 || opb != 0 || opr != 0 || oh != 0 || ow != 0 || (act != 0 && act != 1) ||
          l.weights.size() != static_cast<size_t>(1 + (has_bias ? 1 : 0)))
        return fail(err, where + "only static FP32 2x2 stride-2 Deconvolution is supported");
      const int in = by_name_.at(l.bottoms[0]);
      const Tensor ti = tensors_[resolve(in)];
      const WeightTensor& wt = l.weights[0];
      const int64_t O = p.get_int(0, 0);
      if (ti.i8 || ti.rank != 3 || wt.shape.size() != 4 || wt.shape[0] != O || wt.shape[1] != ti.c || wt.shape[2] != 2 ||
          wt.shape[3] != 2 || static_cast<int64_t>(wt.count()) != p.get_int(6, 0))
        return fail(err, where + "Deconvolution weight shape or weight_data_size is inconsistent");
      if (wt.type == WeightType::kI8) return fail(err, where + "Deconvolution weight must be floating point");
      Node n;
      n.kind = N_DECONV;
      n.name = l.name;
      n.type = t;
      n.O = static_cast<int>(O);
      n.has_bias = has_bias == 1;
      n.act = act == 1 ? ACT_RELU : ACT_NONE;
      if (n.has_bias) n.bias = l.weights[1].as_f32();
      // repack [o][c][a][b] -> [a][b][c][o]
      const std::vector<float> w = wt.as_f32();
      n.w_f32.resize(w.size());
      for (int o = 0; o < n.O; ++o)
        for (int c = 0; c < ti.c; ++c)
          for (int k = 0; k < 4; ++k)
            n.w_f32[(static_cast<size_t>(k) * ti.c + c) * n.O + o] = w[(static_cast<size_t>(o) * ti.c + c) * 4 + k];
      n.flops = 2.0 * 4.0 * ti.h * ti.w * ti.c * n.O;
      n.in = {in};
      n.out = new_tensor(l.tops[0]);
      Tensor& to = tensors_[n.out];
      const std::string keep = to.name;
      to = ti;
      to.name = keep;
      to.alias = -1;
      to.is_input = false;
      to.c = n.O;
      to.h = 2 * ti.h;
      to.w = 2 * ti.w;
      nodes_.push_back(std::move(n));
    } else if (t == "Dequantize" || t == "Requantize") {
      return fail(err, where + "needs an int32 producer, which no importable layer provides; "
                               "use the operator entry points instead");
    } else {
      return fail(err, where + "layer type is outside the supported path");
    }
  }
  for (const auto& name : model_.outputs) outputs_.push_back(by_name_.at(name));
  if (inputs_.empty() || outputs_.empty()) return fail(err, "model has no inputs or no outputs");
  return true;
}

// ---------------------------------------------------------------------- graph passes
void EngineImpl::fold_batchnorm() {
  // FoldNCNNBatchNorm.cpp:55-178: fp32, non-quantised, single-use conv followed by BatchNorm.
  std::vector<int> uses(tensors_.size(), 0);
  for (const Node& n : nodes_)
    for (int t : n.in) ++uses[resolve(t)];
  for (int o : outputs_) ++uses[resolve(o)];
  for (size_t k = 0; k < nodes_.size(); ++k) {
    Node& bn = nodes_[k];
    if (bn.kind != N_UNARY || bn.un.op != UN_AFFINE) continue;
    const int src = resolve(bn.in[0]);
    if (uses[src] != 1) continue;
    for (size_t j = 0; j < k; ++j) {
      Node& cv = nodes_[j];
      if ((cv.kind != N_CONV && cv.kind != N_DW) || resolve(cv.out) != src) continue;
      if (cv.term != 0 || cv.act != ACT_NONE) break;
      const size_t row = cv.w_f32.size() / cv.O;
      for (size_t i = 0; i < cv.w_f32.size(); ++i) {
        volatile float t = cv.w_f32[i] * bn.un_scale[i / row];
        cv.w_f32[i] = t;
      }
      if (cv.has_bias) {
        for (int o = 0; o < cv.O; ++o) {
          volatile float t = cv.bias[o] * bn.un_scale[o];
          cv.bias[o] = t + bn.un_offset[o];
        }
      } else {
        cv.bias = bn.un_offset;
        cv.has_bias = true;
      }
      cv.out = bn.out;
      nodes_.erase(nodes_.begin() + k);
      --k;
      break;
    }
  }
}

void EngineImpl::fuse() {
  auto count_uses = [&]() {
    std::vector<int> uses(tensors_.size(), 0);
    for (const Node& n : nodes_) {
      for (int t : n.in) ++uses[resolve(t)];
      if (n.res >= 0) ++uses[resolve(n.res)];
    }
    for (int o : outputs_) ++uses[resolve(o)];
    return uses;
  };
  auto producer_of = [&](int tensor, size_t before) -> int {
    for (size_t j = 0; j < before && j < nodes_.size(); ++j)
      if (resolve(nodes_[j].out) == tensor) return static_cast<int>(j);
    return -1;
  };
  auto fuse_activations = [&]() {
    for (size_t k = 0; k < nodes_.size(); ++k) {
      Node& u = nodes_[k];
      if (u.kind != N_UNARY || u.un.op != UN_ACT) continue;
      const std::vector<int> uses = count_uses();
      const int src = resolve(u.in[0]);
      if (uses[src] != 1) continue;
      const int pj = producer_of(src, k);
      if (pj < 0) continue;
      Node& p = nodes_[pj];
      const bool contraction = p.kind == N_CONV || p.kind == N_DW || p.kind == N_IP;
      const bool binary = p.kind == N_BINARY;
      if (!(contraction || binary)) continue;
      if (contraction && p.act != ACT_NONE) continue;
      if (binary && p.bin.act != ACT_NONE) continue;
      if (tensors_[src].i8 && u.un.act != ACT_RELU) continue;
      if (p.kind == N_GEMM) continue;
      if (contraction) {
        p.act = u.un.act;
        p.act_a = u.un.act_a;
        p.act_b = u.un.act_b;
      } else {
        p.bin.act = u.un.act;
        p.bin.act_a = u.un.act_a;
        p.bin.act_b = u.un.act_b;
      }
      p.out = u.out;
      nodes_.erase(nodes_.begin() + k);
      --k;
    }
  };
  fuse_activations();
  // residual: Eltwise SUM (no coefficients) of two fp32 tensors, one of which is the
  // single-use result of a contraction without activation that runs after the other
  // operand exists.
  for (size_t k = 0; k < nodes_.size(); ++k) {
    Node& b = nodes_[k];
    if (b.kind != N_BINARY || b.broadcast || b.bin.op != BIN_ADD || b.bin.use_scalar || b.bin.scale_a || b.bin.scale_b) continue;
    if (tensors_[resolve(b.in[0])].i8) continue;
    const std::vector<int> uses = count_uses();
    int best = -1, other = -1;
    for (int side = 0; side < 2; ++side) {
      const int x = resolve(b.in[side]), y = resolve(b.in[1 - side]);
      if (x == y || uses[x] != 1) continue;
      const int pj = producer_of(x, k);
      if (pj < 0) continue;
      const Node& p = nodes_[pj];
      if (!(p.kind == N_CONV || p.kind == N_DW) || p.act != ACT_NONE || p.res >= 0) continue;
      if (tensors_[x].i8) continue;
      const int py = producer_of(y, k);  // -1: graph input, always available
      if (py >= pj) continue;
      if (pj > best) {
        best = pj;
        other = y;
      }
    }
    if (best < 0) continue;
    Node& p = nodes_[best];
    p.res = other;
    p.out = b.out;
    p.act = b.bin.act;
    p.act_a = b.bin.act_a;
    p.act_b = b.bin.act_b;
    nodes_.erase(nodes_.begin() + k);
    --k;
  }
  fuse_activations();
}

// NCNN_B200_STEM_ROWS=0 at load time keeps the stem on the im2col-window path of tc_gemm_kernel.
static bool stem_rows_enabled() {
  const char* f = std::getenv("NCNN_B200_STEM_ROWS");
  return f == nullptr || f[0] != '0';
}

bool EngineImpl::choose_impl(std::string* err) {
  const bool exact = opt_.accuracy_mode == kAccuracyFp32Cuda;
  std::vector<int> uses(tensors_.size(), 0);
  for (const Node& n : nodes_) {
    for (int t : n.in) ++uses[resolve(t)];
    if (n.res >= 0) ++uses[resolve(n.res)];
  }
  for (int o : outputs_) ++uses[resolve(o)];
  for (Node& n : nodes_) {
    if (n.kind == N_CONV) {
      const Tensor& ti = tensors_[resolve(n.in[0])];
      const bool i8 = n.term != 0;
      const int kind = i8 ? GEMM_I8 : GEMM_TF32;
      const int last_w = -n.pl + (n.OW - 1) * n.sw - (ti.w - 1);
      const int last_h = -n.pt + (n.OH - 1) * n.sh - (ti.h - 1);
      const bool geometry_ok = n.sw <= 8 && n.sh <= 8 && n.pl <= 128 && n.pt <= 128 && last_w >= -128 &&
                               last_w <= 127 && last_h >= -128 && last_h <= 127 &&
                               (n.KW - 1) * n.dw < 65536 && (n.KH - 1) * n.dh < 65536;
      n.impl = IMPL_DIRECT;
      if ((!exact || i8) && geometry_ok) {
        if (tc_k_elems(kind, ti.c) > 0) {
          n.impl = IMPL_TC;
        } else {
          // stem: few channels, graph input consumed only here -> overlapping-window view
          const int cp = i8 ? 16 : 4;
          const int window = i8 ? 128 : 32;
          if (ti.is_input && uses[resolve(n.in[0])] == 1 && ti.c <= 4 && n.dw == 1 && n.KW * cp <= window &&
              (n.sw * cp * (i8 ? 1 : 4)) % 16 == 0) {
            n.impl = IMPL_TC;
            n.stem = true;
            // bf16 pairs halve the window to 64-byte rows and the MMA count with it; the pixel
            // stride of the view must stay a multiple of 16 bytes
            n.stem_bf16 = !i8 && opt_.accuracy_mode == kAccuracyFp32Split && (n.sw * cp * 2) % 16 == 0;
            // output pixels 16 bytes apart in the padded row: the windows can overlap in shared memory
            // (bf16 pairs: 4 channels x 2 bytes; int8: 8 channels per pixel instead of 16)
            const bool rows_geometry = stem_rows_enabled() && n.sw == 2 && n.OW <= 128 && n.O % 16 == 0 && n.O <= 128 &&
                                       n.KW <= 8 && n.KH <= 16 && n.dh == 1;
            n.stem_rows = rows_geometry && (n.stem_bf16 || (i8 && (n.term <= 100 || n.O % 64 == 0)));
          }
        }
      }
      if (n.impl == IMPL_TC && !i8) any_fp32_tc_ = true;
    } else if (n.kind == N_IP || n.kind == N_GEMM) {
      const bool i8 = n.term != 0;
      n.impl = IMPL_DIRECT;
      if (n.kind == N_GEMM && i8) continue;  // per-row dynamic scales: dedicated kernel
      const int es = i8 ? 1 : 4;
      if ((!exact || i8) && (static_cast<long long>(n.K) * es) % 16 == 0) n.impl = IMPL_TC;
      if (n.impl == IMPL_TC && !i8) any_fp32_tc_ = true;
    } else if (n.kind == N_DW) {
      n.impl = IMPL_DIRECT;
    }
  }
  (void)err;
  return true;
}

// A channel Concat whose inputs are all single-use results of tensor-core convolutions needs no
// copy: each convolution's epilogue already takes an output row stride, so it writes its
// channels straight into the Concat's tensor (TMA stores clip at the convolution's own width).
// Offsets and the total width must keep every row 16-byte aligned in any format (multiples of 8).
void EngineImpl::fold_channel_concats() {
  for (size_t k = 0; k < nodes_.size(); ++k) {
    Node& cat = nodes_[k];
    if (cat.kind != N_CONCAT || cat.concat.empty() || cat.concat[0].slice) continue;
    const Tensor& to = tensors_[resolve(cat.out)];
    if (to.rank != 3 || to.i8 || to.c % 8 != 0) continue;
    bool channel_axis = true;
    for (const ConcatParams& cp : cat.concat) channel_axis = channel_axis && cp.inner == 1 && cp.len_out == to.c;
    if (!channel_axis) continue;
    std::vector<int> uses(tensors_.size(), 0);
    for (const Node& n : nodes_) {
      for (int t : n.in) ++uses[resolve(t)];
      if (n.res >= 0) ++uses[resolve(n.res)];
    }
    for (int o : outputs_) ++uses[resolve(o)];
    std::vector<int> producers;
    bool ok = true;
    for (size_t i = 0; i < cat.in.size() && ok; ++i) {
      const int src = resolve(cat.in[i]);
      int pj = -1;
      for (size_t j = 0; j < k; ++j)
        if (resolve(nodes_[j].out) == src) pj = static_cast<int>(j);
      ok = pj >= 0 && uses[src] == 1 && cat.concat[i].offset % 8 == 0;
      if (ok) {
        const Node& p = nodes_[pj];
        ok = p.kind == N_CONV && p.impl == IMPL_TC && !p.stem && p.term == 0 && p.out_ld == 0 && p.res < 0 &&
             p.O == cat.concat[i].len_in;
        for (int other : producers) ok = ok && other != pj;
      }
      producers.push_back(pj);
    }
    if (!ok) continue;
    const int target = resolve(cat.out);
    for (size_t i = 0; i < cat.in.size(); ++i) {
      Node& p = nodes_[producers[i]];
      p.out_ld = to.c;
      p.out_ch_off = cat.concat[i].offset;
      tensors_[resolve(p.out)].alias = target;
    }
    nodes_.erase(nodes_.begin() + k);
    --k;
  }
}

static bool halo_preferred();

// A Quantize step in front of an int8 contraction re-reads an fp32 tensor that a tensor-core contraction or
// a pooling layer has just written.  Where that producer can quantise on the way out (plain fp32 result,
// channels in multiples of 16 for the contraction's 16-byte stores, 4 for pooling), the int8 copy becomes a
// second result of the producer and the Quantize step disappears.  The value quantised is the value stored,
// so the bits are those of the separate step.
// Measured on the int8 ResNet-18 at batch 64: folding into the pooling layers pays (they run at full
// occupancy: +3 us on the pooling pass for a 16 us Quantize pass saved); folding into the residual
// convolutions' epilogue does not (+20..29 us on the convolution for 16 us saved: the epilogue warps run one
// per scheduler and are what bounds those layers already), so it is opt-in.
//   NCNN_B200_FUSE_QUANT=0  keep every Quantize step;  =1 (default) fold into pooling layers;
//   =2 fold into tensor-core contractions as well.
void EngineImpl::fuse_quantize_steps() {
  const char* env = std::getenv("NCNN_B200_FUSE_QUANT");
  const int level = env == nullptr || env[0] == 0 ? 1 : std::atoi(env);
  if (level <= 0) return;
  for (size_t k = 0; k < nodes_.size(); ++k) {
    const Node& q = nodes_[k];
    if (q.kind != N_UNARY || q.un.op != UN_QUANT || q.un.nscale != 1 || q.un_scale.empty()) continue;
    const int src = resolve(q.in[0]);
    const Tensor& ts = tensors_[src];
    if (ts.fmt != FMT_F32 || ts.is_input) continue;
    int pj = -1;
    for (size_t j = 0; j < k; ++j)
      if (resolve(nodes_[j].out) == src) pj = static_cast<int>(j);
    if (pj < 0) continue;
    Node& p = nodes_[pj];
    const int channels = ts.rank == 3 ? ts.c : ts.w;
    bool ok = false;
    if (level >= 2 && (p.kind == N_CONV || p.kind == N_IP) && p.impl == IMPL_TC && p.term != 0 && !p.stem && p.out_ld == 0)
      ok = channels % 16 == 0 && p.side_q.size() < 2;
    else if (p.kind == N_POOL)
      ok = channels % 4 == 0 && p.side_q.empty() && ts.Cp == ts.c && ts.Wp == ts.w;
    if (!ok) continue;
    p.side_q.emplace_back(q.out, q.un_scale[0]);
    nodes_.erase(nodes_.begin() + k);
    --k;
  }
}

// A stride-1 3x3 depthwise layer whose only consumer is a 1x1 tensor-core convolution (the second half of
// an inverted-residual block) runs inside that convolution's kernel: its result goes from the CUDA cores
// into the shared-memory operand tile of the MMAs and never to HBM.  The values, their bf16 split and the
// order of the products are those of the two separate layers.  NCNN_B200_FUSE_DW=0 keeps them apart.
void EngineImpl::fuse_depthwise_projection() {
  const char* env = std::getenv("NCNN_B200_FUSE_DW");
  if (env != nullptr && env[0] == '0') return;
  if (opt_.accuracy_mode != kAccuracyFp32Split) return;
  std::vector<int> uses(tensors_.size(), 0);
  for (const Node& n : nodes_) {
    for (int t : n.in) ++uses[resolve(t)];
    if (n.res >= 0) ++uses[resolve(n.res)];
    for (const auto& side : n.side_q) (void)side;
  }
  for (int o : outputs_) ++uses[resolve(o)];
  for (size_t k = 0; k + 1 < nodes_.size(); ++k) {
    const Node& dw = nodes_[k];
    if (dw.kind != N_DW || dw.term != 0 || dw.KH != 3 || dw.KW != 3 || dw.sh != 1 || dw.sw != 1 || dw.dh != 1 ||
        dw.dw != 1 || dw.res >= 0 || !dw.side_q.empty() || dw.d_w0 == nullptr)
      continue;
    const int mid = resolve(dw.out);
    const int src = resolve(dw.in[0]);
    const Tensor& tin = tensors_[src];
    const Tensor& tmid = tensors_[mid];
    if (uses[mid] != 1 || tin.rank != 3 || tin.fmt != FMT_F32 || tin.Cp != tin.c || tin.Wp != tin.w || tin.w_off != 0 ||
        tmid.fmt != FMT_BF16X2 || dw.OH != tin.h || dw.OW != tin.w || dw.pt > 2 || dw.pl > 2)
      continue;
    // the consumer: the next node that reads the depthwise result
    size_t j = k + 1;
    for (; j < nodes_.size(); ++j)
      if (!nodes_[j].in.empty() && resolve(nodes_[j].in[0]) == mid) break;
    if (j >= nodes_.size()) continue;
    Node& pw = nodes_[j];
    if (pw.kind != N_CONV || pw.impl != IMPL_TC || pw.term != 0 || pw.stem || pw.out_ld != 0 || pw.KH != 1 || pw.KW != 1 ||
        pw.sh != 1 || pw.sw != 1 || pw.pt != 0 || pw.pl != 0 || !pw.side_q.empty() || pw.d_w0 == nullptr || pw.d_w1 == nullptr)
      continue;
    const Tensor& tout = tensors_[resolve(pw.out)];
    const int out_mode = tout.fmt == FMT_BF16X2 ? OUT_BF16X2 : (tout.fmt == FMT_F32 ? OUT_F32 : -1);
    if (out_mode < 0) continue;
    const bool has_res = pw.res >= 0;
    const bool res_bf16 = has_res && tensors_[resolve(pw.res)].fmt == FMT_BF16X2;
    if (has_res && !res_bf16 && tensors_[resolve(pw.res)].fmt != FMT_F32) continue;
    if (dw.act != ACT_NONE && dw.act != ACT_RELU && dw.act != ACT_CLIP) continue;  // the fused kernel clamps, nothing else
    if (!tc_dw_project_applies(tin.c, pw.O, tin.h, tin.w, out_mode, has_res, res_bf16)) continue;
    pw.dw_fused = true;
    pw.dw_w = static_cast<const float*>(dw.d_w0);
    pw.dw_bias = dw.d_bias;
    pw.dw_act = dw.act;
    pw.dw_act_a = dw.act_a;
    pw.dw_act_b = dw.act_b;
    pw.dw_pt = dw.pt;
    pw.dw_pl = dw.pl;
    pw.dw_name = dw.name;
    pw.in[0] = dw.in[0];
    pw.flops += dw.flops;
    nodes_.erase(nodes_.begin() + k);
    --k;
  }
}

bool EngineImpl::prepare_weights(std::string* err) {
  const int f32_kind = opt_.accuracy_mode == kAccuracyTf32 ? GEMM_TF32 : GEMM_TF32X3;
  // insert Quantize steps in front of int8 contractions whose input is fp32
  for (size_t k = 0; k < nodes_.size(); ++k) {
    Node& n = nodes_[k];
    if (!((n.kind == N_CONV || n.kind == N_DW || n.kind == N_IP) && n.term != 0)) continue;
    const int src = resolve(n.in[0]);
    if (tensors_[src].i8) continue;
    if (n.stem) {
      tensors_[src].input_quant_scale = n.s_in;  // the input edge quantises directly
      continue;
    }
    Node q;
    q.kind = N_UNARY;
    q.name = n.name + ":quantize";
    q.type = "Quantize";
    q.un.op = UN_QUANT;
    q.un_scale = {n.s_in};
    q.un.nscale = 1;
    q.un.channels = 1;
    q.un.inner = 1;
    q.in = {src};
    q.out = new_tensor(n.name + ":q");
    Tensor& tq = tensors_[q.out];
    const std::string keep = tq.name;
    tq = tensors_[src];
    tq.name = keep;
    tq.alias = -1;
    tq.is_input = false;
    tq.i8 = true;
    n.in[0] = q.out;
    nodes_.insert(nodes_.begin() + k, std::move(q));
    ++k;
  }
  // formats: an fp32 tensor is kept as hi/lo planes (or tf32-rounded in the fast mode) only
  // when a tensor-core contraction reads it as its operand; everything else stays one
  // plain fp32 plane, which halves the traffic of the memory-bound layers around it
  // In the accurate mode such a tensor is a bf16 pair (hi, mid) when every contraction that
  // reads it can take 64-channel K blocks: three bf16 MMAs run at twice the rate of three
  // tf32 MMAs on half the operand bytes, at the same ~1e-5 error.  Otherwise fp32 hi/lo planes.
  std::vector<char> feeds_tc(tensors_.size(), 0), bf16_ok(tensors_.size(), 1);
  for (const Node& n : nodes_) {
    const bool contraction = n.kind == N_CONV || n.kind == N_IP || n.kind == N_GEMM;
    if (!(contraction && n.impl == IMPL_TC && n.term == 0)) continue;
    const int src = resolve(n.in[0]);
    feeds_tc[src] = 1;
    const bool can = n.kind == N_CONV ? (n.stem ? n.stem_bf16 : tensors_[src].c % 8 == 0) : (n.K % 8 == 0);
    if (!can) bf16_ok[src] = 0;
  }
  for (size_t i = 0; i < tensors_.size(); ++i) {
    Tensor& t = tensors_[i];
    t.Cp = t.rank == 3 ? t.c : 1;
    t.Wp = t.w;
    t.w_off = 0;
    if (t.i8) {
      t.fmt = FMT_I8;
    } else if (feeds_tc[resolve(static_cast<int>(i))]) {
      t.fmt = opt_.accuracy_mode == kAccuracyTf32 ? FMT_TF32 : (bf16_ok[resolve(static_cast<int>(i))] ? FMT_BF16X2 : FMT_SPLIT);
    } else {
      t.fmt = FMT_F32;
    }
  }
  fuse_quantize_steps();
  for (Node& n : nodes_) {
    const bool i8 = n.term != 0;
    if (n.has_bias) n.d_bias = upload(n.bias);
    if (!n.deq.empty()) n.d_deq = upload(n.deq);
    if (!n.un_scale.empty()) n.d_scale = upload(n.un_scale);
    if (!n.un_offset.empty()) n.d_offset = upload(n.un_offset);
    n.un.scale = n.d_scale;
    n.un.offset = n.d_offset;
    if (n.kind == N_DECONV) n.d_w0 = upload(n.w_f32);
    if (n.kind == N_CONV) {
      const int src = resolve(n.in[0]);
      Tensor& ti = tensors_[src];
      const int C = ti.c;
      if (n.impl == IMPL_TC) {
        const int kind = i8 ? GEMM_I8 : (ti.fmt == FMT_BF16X2 ? GEMM_BF16X3 : f32_kind);
        if (n.stem) {
          // (row-resident int8 stems: 8 channels per pixel, 64-byte windows of 8 pixels)
          const int cp = i8 ? (n.stem_rows ? 8 : 16) : 4;
          const int window = i8 ? (n.stem_rows ? 64 : 128) : 32;
          n.k_elems = window;
          // storage of the input: rows padded on the left by pad_l, wide enough for the
          // last window, channels padded to cp
          ti.Cp = cp;
          ti.w_off = n.pl;
          ti.Wp = std::max(ti.w + n.pl, ((n.OW - 1) * n.sw * cp + window + cp - 1) / cp);
          if (n.stem_rows) ti.Wp = (ti.Wp + 15) / 16 * 16;  // rows of whole 128-byte lines
          ti.dedicated = true;
          if (i8) {
            ti.i8 = true;
            ti.fmt = FMT_I8;
          }
          // virtual weights [O][I' = window][KH][1], I' index = kw*cp + c
          if (i8) {
            std::vector<int8_t> v(static_cast<size_t>(n.O) * window * n.KH, 0), packed;
            for (int o = 0; o < n.O; ++o)
              for (int c = 0; c < C; ++c)
                for (int kh = 0; kh < n.KH; ++kh)
                  for (int kw = 0; kw < n.KW; ++kw)
                    v[(static_cast<size_t>(o) * window + kw * cp + c) * n.KH + kh] =
                        n.w_i8[((static_cast<size_t>(o) * C + c) * n.KH + kh) * n.KW + kw];
            tc_pack_weights_i8(v.data(), n.O, window, n.KH, 1, window, &packed);
            n.d_w0 = upload(packed);
          } else {
            std::vector<float> v(static_cast<size_t>(n.O) * window * n.KH, 0.0f), hi, lo;
            for (int o = 0; o < n.O; ++o)
              for (int c = 0; c < C; ++c)
                for (int kh = 0; kh < n.KH; ++kh)
                  for (int kw = 0; kw < n.KW; ++kw)
                    v[(static_cast<size_t>(o) * window + kw * cp + c) * n.KH + kh] =
                        n.w_f32[((static_cast<size_t>(o) * C + c) * n.KH + kh) * n.KW + kw];
            if (kind == GEMM_BF16X3) {
              std::vector<uint16_t> bh, bm;
              tc_pack_weights_bf16x2(v.data(), n.O, window, n.KH, 1, window, &bh, &bm);
              n.d_w0 = upload(bh);
              n.d_w1 = upload(bm);
            } else {
              tc_pack_weights_f32(kind, v.data(), n.O, window, n.KH, 1, window, &hi, &lo);
              n.d_w0 = upload(hi);
              if (kind == GEMM_TF32X3) n.d_w1 = upload(lo);
            }
          }
        } else {
          n.k_elems = tc_k_elems(kind, C);
          if (i8) {
            std::vector<int8_t> packed;
            tc_pack_weights_i8(n.w_i8.data(), n.O, C, n.KH, n.KW, n.k_elems, &packed);
            n.d_w0 = upload(packed);
          } else if (kind == GEMM_BF16X3) {
            std::vector<uint16_t> hi, mid;
            tc_pack_weights_bf16x2(n.w_f32.data(), n.O, C, n.KH, n.KW, n.k_elems, &hi, &mid);
            n.d_w0 = upload(hi);
            n.d_w1 = upload(mid);
          } else {
            std::vector<float> hi, lo;
            tc_pack_weights_f32(kind, n.w_f32.data(), n.O, C, n.KH, n.KW, n.k_elems, &hi, &lo);
            n.d_w0 = upload(hi);
            if (kind == GEMM_TF32X3) n.d_w1 = upload(lo);
          }
        }
      } else {
        // direct kernel: [KH*KW][C][O]
        const size_t total = static_cast<size_t>(n.KH) * n.KW * C * n.O;
        if (i8) {
          std::vector<int8_t> v(total);
          for (int o = 0; o < n.O; ++o)
            for (int c = 0; c < C; ++c)
              for (int t = 0; t < n.KH * n.KW; ++t)
                v[(static_cast<size_t>(t) * C + c) * n.O + o] = n.w_i8[(static_cast<size_t>(o) * C + c) * n.KH * n.KW + t];
          n.d_w0 = upload(v);
        } else {
          std::vector<float> v(total);
          for (int o = 0; o < n.O; ++o)
            for (int c = 0; c < C; ++c)
              for (int t = 0; t < n.KH * n.KW; ++t)
                v[(static_cast<size_t>(t) * C + c) * n.O + o] = n.w_f32[(static_cast<size_t>(o) * C + c) * n.KH * n.KW + t];
          n.d_w0 = upload(v);
        }
      }
      if (n.d_w0 == nullptr) return fail(err, "out of device memory while uploading weights of " + n.name);
    } else if (n.kind == N_DW) {
      const int C = n.O, taps = n.KH * n.KW;
      if (i8) {
        std::vector<int8_t> v(static_cast<size_t>(taps) * C);
        for (int c = 0; c < C; ++c)
          for (int t = 0; t < taps; ++t) v[static_cast<size_t>(t) * C + c] = n.w_i8[static_cast<size_t>(c) * taps + t];
        n.d_w0 = upload(v);
      } else {
        std::vector<float> v(static_cast<size_t>(taps) * C);
        for (int c = 0; c < C; ++c)
          for (int t = 0; t < taps; ++t) v[static_cast<size_t>(t) * C + c] = n.w_f32[static_cast<size_t>(c) * taps + t];
        n.d_w0 = upload(v);
      }
    } else if (n.kind == N_IP || n.kind == N_GEMM) {
      const Tensor& ti = tensors_[resolve(n.in[0])];
      // The reference flattens in [C][H][W] order (NCNNToTosa.cpp:5305-5337); activations
      // are stored channel-last, so the weight columns are permuted once here.
      std::vector<int> perm(n.K);
      for (int k = 0; k < n.K; ++k) perm[k] = k;
      if (n.kind == N_IP && ti.rank == 3) {
        for (int c = 0; c < ti.c; ++c)
          for (int h = 0; h < ti.h; ++h)
            for (int w = 0; w < ti.w; ++w) perm[(h * ti.w + w) * ti.c + c] = (c * ti.h + h) * ti.w + w;
      }
      if (n.kind == N_GEMM && i8) {
        n.d_w0 = upload(n.w_i8);  // [N][K] as is
      } else if (n.impl == IMPL_TC) {
        const int kind = i8 ? GEMM_I8 : (ti.fmt == FMT_BF16X2 ? GEMM_BF16X3 : f32_kind);
        n.k_elems = i8 ? 128 : (kind == GEMM_BF16X3 ? 64 : 32);
        if (i8) {
          std::vector<int8_t> v(n.w_i8.size()), packed;
          for (int o = 0; o < n.O; ++o)
            for (int k = 0; k < n.K; ++k) v[static_cast<size_t>(o) * n.K + k] = n.w_i8[static_cast<size_t>(o) * n.K + perm[k]];
          tc_pack_weights_i8(v.data(), n.O, n.K, 1, 1, n.k_elems, &packed);
          n.d_w0 = upload(packed);
        } else if (kind == GEMM_BF16X3) {
          std::vector<float> v(n.w_f32.size());
          std::vector<uint16_t> hi, mid;
          for (int o = 0; o < n.O; ++o)
            for (int k = 0; k < n.K; ++k) v[static_cast<size_t>(o) * n.K + k] = n.w_f32[static_cast<size_t>(o) * n.K + perm[k]];
          tc_pack_weights_bf16x2(v.data(), n.O, n.K, 1, 1, n.k_elems, &hi, &mid);
          n.d_w0 = upload(hi);
          n.d_w1 = upload(mid);
        } else {
          std::vector<float> v(n.w_f32.size()), hi, lo;
          for (int o = 0; o < n.O; ++o)
            for (int k = 0; k < n.K; ++k) v[static_cast<size_t>(o) * n.K + k] = n.w_f32[static_cast<size_t>(o) * n.K + perm[k]];
          tc_pack_weights_f32(kind, v.data(), n.O, n.K, 1, 1, n.k_elems, &hi, &lo);
          n.d_w0 = upload(hi);
          if (kind == GEMM_TF32X3) n.d_w1 = upload(lo);
        }
      } else {
        // direct kernel: [K][N]
        if (i8) {
          std::vector<int8_t> v(n.w_i8.size());
          for (int o = 0; o < n.O; ++o)
            for (int k = 0; k < n.K; ++k) v[static_cast<size_t>(k) * n.O + o] = n.w_i8[static_cast<size_t>(o) * n.K + perm[k]];
          n.d_w0 = upload(v);
        } else {
          std::vector<float> v(n.w_f32.size());
          for (int o = 0; o < n.O; ++o)
            for (int k = 0; k < n.K; ++k) v[static_cast<size_t>(k) * n.O + o] = n.w_f32[static_cast<size_t>(o) * n.K + perm[k]];
          n.d_w0 = upload(v);
        }
      }
      if (n.d_w0 == nullptr) return fail(err, "out of device memory while uploading weights of " + n.name);
    }
  }
  if (upload_failed_) return fail(err, "out of device memory while uploading weights");
  // host copies are no longer needed
  for (Node& n : nodes_) {
    std::vector<float>().swap(n.w_f32);
    std::vector<int8_t>().swap(n.w_i8);
  }
  return true;
}

// How many leading layers may be run per upload chunk: as many as it takes to keep the GPU
// busy for about the time the upload of the inputs needs (estimated per image at 50 GB/s over
// PCIe against 150 TFLOP/s on the tensor cores, 8 TFLOP/s on the CUDA cores and 2 TB/s for
// memory-bound layers).  Which of them a given batch really runs per chunk is decided per plan.
void EngineImpl::choose_head_limit() {
  double upload = 0.0;
  for (int t : inputs_) upload += static_cast<double>(tensors_[resolve(t)].logical()) * 4.0 / 50e9;
  double spent = 0.0;
  head_limit_ = 0;
  for (size_t k = 0; k < nodes_.size(); ++k) {
    const Node& n = nodes_[k];
    double bytes = static_cast<double>(tensors_[resolve(n.out)].logical()) * 4.0;
    for (int t : n.in) bytes += static_cast<double>(tensors_[resolve(t)].logical()) * 4.0;
    const bool contraction = n.kind == N_CONV || n.kind == N_IP || n.kind == N_GEMM;
    const double cost = std::max(bytes / 2e12, contraction ? n.flops / (n.impl == IMPL_TC ? 150e12 : 8e12) : 0.0);
    if (spent + cost > 1.25 * upload) break;
    spent += cost;
    head_limit_ = static_cast<int>(k) + 1;
  }
}

void EngineImpl::plan_memory() {
  // sizes
  for (Tensor& t : tensors_) {
    if (t.alias >= 0) continue;
    t.plane_elems = t.rank == 3 ? static_cast<size_t>(t.h) * t.Wp * t.Cp : static_cast<size_t>(t.logical());
    if (t.dedicated) t.plane_elems += 256;  // the last window may read past the last row
    t.plane_bytes = round_up(t.plane_elems * t.elem_bytes(), 256);
  }
  // liveness over node order; inputs are defined before node 0, outputs live to the end
  const int end = static_cast<int>(nodes_.size());
  for (Tensor& t : tensors_) {
    t.first_def = -1;
    t.last_use = -1;
  }
  for (int k = 0; k < end; ++k) {
    const Node& n = nodes_[k];
    Tensor& o = tensors_[resolve(n.out)];
    if (o.first_def < 0) o.first_def = k;
    o.last_use = std::max(o.last_use, k);
    for (int t : n.in) tensors_[resolve(t)].last_use = std::max(tensors_[resolve(t)].last_use, k);
    if (n.res >= 0) tensors_[resolve(n.res)].last_use = std::max(tensors_[resolve(n.res)].last_use, k);
    for (const auto& side : n.side_q) {
      Tensor& sq = tensors_[resolve(side.first)];
      if (sq.first_def < 0) sq.first_def = k;
      sq.last_use = std::max(sq.last_use, k);
    }
  }
  for (int t : inputs_) {
    tensors_[resolve(t)].first_def = -1;
    tensors_[resolve(t)].last_use = std::max(tensors_[resolve(t)].last_use, 0);
  }
  for (int t : outputs_) tensors_[resolve(t)].last_use = end;
  // Layers [0, head_limit_) may run chunk by chunk (pipelined host path): while one chunk
  // is in them, another chunk's results of the same layers are waiting for the tail, so the
  // tensors they touch must all be live together.
  for (Tensor& t : tensors_) {
    if (t.alias >= 0 || head_limit_ == 0) continue;
    if (t.first_def < head_limit_ && (t.last_use >= 0 || t.is_input)) {
      t.first_def = -1;
      t.last_use = std::max(t.last_use, head_limit_ - 1);
    }
  }
  // greedy first fit, largest first
  struct Placed {
    size_t off, size;
    int a, b;
  };
  std::vector<int> order;
  for (size_t i = 0; i < tensors_.size(); ++i)
    if (tensors_[i].alias < 0 && (tensors_[i].last_use >= 0 || tensors_[i].is_input)) order.push_back(static_cast<int>(i));
  std::sort(order.begin(), order.end(), [&](int x, int y) {
    return tensors_[x].plane_bytes * tensors_[x].planes() > tensors_[y].plane_bytes * tensors_[y].planes();
  });
  std::vector<Placed> placed;
  size_t top = 0;
  for (int id : order) {
    Tensor& t = tensors_[id];
    const size_t size = t.plane_bytes * t.planes();
    const int a = t.dedicated ? -2 : t.first_def, b = t.dedicated ? end + 1 : t.last_use;
    size_t off = 0;
    bool moved = true;
    while (moved) {
      moved = false;
      for (const Placed& p : placed) {
        const bool time_overlap = !(b < p.a || p.b < a);
        const bool space_overlap = off < p.off + p.size && p.off < off + size;
        if (time_overlap && space_overlap) {
          off = p.off + p.size;
          moved = true;
        }
      }
    }
    t.offset = off;
    placed.push_back({off, size, a, b});
    top = std::max(top, off + size);
  }
  arena_per_image_ = top;
}

ActRef EngineImpl::ref(int tensor, int64_t n) const {
  const Tensor& t = tensors_[resolve(tensor)];
  ActRef r;
  r.fmt = t.fmt;
  // layout for `ln` images; pointers start at image img0_ (images are dense inside a plane)
  const size_t ln = static_cast<size_t>(layout_n_ > 0 ? layout_n_ : n);
  const size_t image_elems = t.rank == 3 ? static_cast<size_t>(t.h) * t.Wp * t.Cp : static_cast<size_t>(t.logical());
  uint8_t* base = arena_ + t.offset * ln + static_cast<size_t>(img0_) * image_elems * t.elem_bytes();
  if (t.fmt == FMT_I8) {
    r.q = reinterpret_cast<int8_t*>(base);
  } else {
    r.p0 = reinterpret_cast<float*>(base);
    if (t.planes() == 2) r.p1 = reinterpret_cast<float*>(base + t.plane_bytes * ln);
  }
  return r;
}

// ---------------------------------------------------------------------- build
bool EngineImpl::build(const std::string& param, const std::string& bin, const EngineOptions& opt,
                       std::string* err) {
  opt_ = opt;
  // the requested device is current only inside this call; the caller's choice is put back on return
  DeviceGuard guard(opt.plan_only ? -1 : opt.device);
  if (opt.accuracy_mode < 0 || opt.accuracy_mode > 2) return fail(err, "unknown accuracy mode");
  if (!opt.plan_only) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0)
      return fail(err, "no CUDA device is available: this runtime has no CPU path");
    int dev = 0;
    if (opt.device >= 0) {
      int available = 0;
      if (cudaGetDeviceCount(&available) != cudaSuccess || opt.device >= available)
        return fail(err, "cannot select the requested CUDA device");
      dev = opt.device;
    } else {
      cudaGetDevice(&dev);
    }
    device_ = dev;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return fail(err, "cannot query the CUDA device");
    if (prop.major != 10) return fail(err, std::string("this runtime is built for sm_100a only; device is ") + prop.name);
    sm_count_ = prop.multiProcessorCount;
  }
  if (!load_model(param, bin, &model_, err)) return false;
  if (!model_.weights_loaded) return fail(err, "a .bin file is required");
  if (!import_layers(err)) return false;
  fold_batchnorm();
  fuse();
  if (!choose_impl(err)) return false;
  fold_channel_concats();
  if (opt.plan_only) return true;
  if (!prepare_weights(err)) return false;
  fuse_depthwise_projection();
  choose_head_limit();
  plan_memory();
  if (cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking) != cudaSuccess) return fail(err, "cannot create a stream");
  void* st = nullptr;
  if (device_alloc(&st, 256) != cudaSuccess) return fail(err, "out of device memory");
  cudaMemset(st, 0, 256);
  device_allocs_.push_back(st);
  d_status_ = static_cast<int*>(st);
  // workspace of the contraction kernel that splits tiles between CTA pairs: partial accumulators
  // and one flag word per CTA (zero between launches); all launches of a model run on one stream
  void* ws = nullptr;
  if (device_alloc(&ws, kTcSplitWorkspaceBytes + 4096) != cudaSuccess) return fail(err, "out of device memory");
  cudaMemset(ws, 0, kTcSplitWorkspaceBytes + 4096);
  device_allocs_.push_back(ws);
  d_split_ws_ = static_cast<uint32_t*>(ws);
  d_split_flags_ = reinterpret_cast<int*>(static_cast<uint8_t*>(ws) + kTcSplitWorkspaceBytes);
  return true;
}

static cudaError_t launch_ok() { return cudaGetLastError(); }

// The patch-resident convolution kernel applies to stride-1 filters; measured inside whole
// networks (batch 64, 3x3 filters at 56/28/14 pixels) it ties with the im2col kernel once the
// operands are bf16 pairs, and loses a little where its 16x8 tiles overhang the image, so it
// is opt-in: NCNN_B200_HALO=1 at load time selects it wherever it applies.
static int halo_level() {
  const char* f = std::getenv("NCNN_B200_HALO");
  return f == nullptr || f[0] == 0 ? 0 : std::atoi(f);
}
static bool halo_preferred() { return halo_level() >= 1; }

bool EngineImpl::emit_node(Plan& plan, const Node& node, int64_t n, std::string* err) {
  const Tensor& to = tensors_[resolve(node.out)];
  const ActRef out = ref(node.out, n);
  Step s;
  s.name = node.name;
  s.flops = node.flops * n;
  const int f32_kind = opt_.accuracy_mode == kAccuracyTf32 ? GEMM_TF32 : GEMM_TF32X3;
  auto bytes_of = [&](int t) {
    const Tensor& x = tensors_[resolve(t)];
    return static_cast<double>(x.logical()) * (x.i8 ? 1 : 4) * n;
  };
  s.bytes = bytes_of(node.out);
  for (int t : node.in) s.bytes += bytes_of(t);
  if (node.res >= 0) s.bytes += bytes_of(node.res);

  if (node.kind == N_CONV || node.kind == N_IP || node.kind == N_GEMM || node.kind == N_DW) {
    const Tensor& ti = tensors_[resolve(node.in[0])];
    const ActRef in = ref(node.in[0], n);
    const bool i8 = node.term != 0;
    ConvEpilogue e{};
    e.bias = node.d_bias;
    e.scale = node.d_deq;
    e.out_scale = node.s_out;
    e.act = node.act;
    e.act_a = node.act_a;
    e.act_b = node.act_b;
    e.has_res = node.res >= 0;
    if (e.has_res) e.res = ref(node.res, n);
    if (node.kind == N_GEMM && i8) {
      const int K = node.K, N = node.O;
      const long long M = static_cast<long long>(ti.h) * n;
      const int8_t* wq = static_cast<const int8_t*>(node.d_w0);
      const float s_b = node.s_b, alpha = node.alpha, beta = 1.0f;
      const float* c_bias = node.d_bias;
      const int has_c = node.has_bias, scale_alpha = node.alpha != 1.0f;
      s.kernel = "k_gemm_i8_rowscale";
      s.run = [=](cudaStream_t st) {
        k_gemm_i8_rowscale<<<static_cast<unsigned>(M), 128, K, st>>>(in, out, wq, K, N, s_b, c_bias, alpha, beta, has_c, scale_alpha);
        return launch_ok();
      };
      plan.steps.push_back(std::move(s));
      return true;
    }
    if (node.impl == IMPL_TC) {
      TcEpilogue te;
      te.bias = node.d_bias;
      te.scale = node.d_deq;
      te.out0 = out.p0;
      te.out1 = out.p1;
      te.outq = out.q;
      te.ldo = node.O;
      if (node.out_ld > 0) {
        // a view into a Concat result: longer rows, starting `out_ch_off` channels in
        te.ldo = node.out_ld;
        const size_t skip = static_cast<size_t>(node.out_ch_off) * to.elem_bytes();
        te.out0 = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(out.p0) + skip);
        if (out.p1 != nullptr) te.out1 = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(out.p1) + skip);
      }
      te.act = node.act;
      te.act_a = node.act_a;
      te.act_b = node.act_b;
      // Gemm: (A*B^T + beta*C) * alpha; beta is in the bias already, alpha multiplies in the epilogue
      const bool alpha_fused = node.kind == N_GEMM && node.alpha != 1.0f && node.act == ACT_NONE;
      if (alpha_fused) {
        te.act = ACT_SCALE;
        te.act_a = node.alpha;
      }
      te.out_scale = node.s_out;
      te.status = d_status_;
      te.side_count = static_cast<int>(node.side_q.size());
      for (int i = 0; i < te.side_count; ++i) {
        te.side_q[i] = ref(node.side_q[i].first, n).q;
        te.side_scale[i] = node.side_q[i].second;
      }
      te.sk_ws = d_split_ws_;
      te.sk_ws_bytes = kTcSplitWorkspaceBytes;
      te.sk_flags = d_split_flags_;
      te.sk_flag_count = kTcSplitFlagCount;
      te.out_mode = to.fmt == FMT_I8 ? OUT_I8 : (to.fmt == FMT_SPLIT ? OUT_F32_SPLIT : (to.fmt == FMT_TF32 ? OUT_F32_TF32 : (to.fmt == FMT_BF16X2 ? OUT_BF16X2 : OUT_F32)));
      if (node.res >= 0) {
        const ActRef r = ref(node.res, n);
        te.res0 = r.p0;
        te.res1 = r.p1;
        te.res_bf16 = r.fmt == FMT_BF16X2;
      }
      const int kind = i8 ? GEMM_I8 : (ti.fmt == FMT_BF16X2 ? GEMM_BF16X3 : f32_kind);
      const char* kind_name = kind == GEMM_I8 ? "i8" : (kind == GEMM_TF32 ? "tf32" : (kind == GEMM_BF16X3 ? "bf16x3" : "tf32x3"));
      auto launch = std::make_shared<TcLaunch>();
      std::string perr;
      if (node.dw_fused) {
        TcDwProjConv dc;
        dc.x = in.p0;
        dc.images = static_cast<int>(n);
        dc.H = ti.h;
        dc.W = ti.w;
        dc.C = ti.c;
        dc.pad_t = node.dw_pt;
        dc.pad_l = node.dw_pl;
        dc.dw_weights = node.dw_w;
        dc.dw_bias = node.dw_bias;
        dc.dw_act = node.dw_act;
        dc.dw_act_a = node.dw_act_a;
        dc.dw_act_b = node.dw_act_b;
        dc.w0 = node.d_w0;
        dc.w1 = node.d_w1;
        dc.out_channels = node.O;
        auto dl = std::make_shared<TcDwProjLaunch>();
        const std::string derr = tc_plan_dw_project(dl.get(), dc, te, sm_count_);
        if (!derr.empty()) return fail(err, "layers " + node.dw_name + " + " + node.name + ": " + derr);
        s.name = node.dw_name + "+" + node.name;
        s.kernel = "tc_dw_project_kernel<bf16x3>";
        s.run = [dl](cudaStream_t st) { return tc_launch_dw_project(*dl, st); };
        plan.steps.push_back(std::move(s));
        return true;
      }
      // stride-1 filters with spatial extent: the patch-resident kernel loads each input pixel
      // once per tile instead of once per tap
      if (node.kind == N_CONV && !i8 && !node.stem && node.out_ld == 0 && halo_preferred() &&
          tc_halo_applies(kind, ti.c, node.KH, node.KW, node.sh, node.sw, node.dh, node.dw, node.OH, node.OW, node.O,
                          te.out_mode)) {
        TcHaloConv hc;
        hc.in0 = in.p0;
        hc.in1 = in.p1;
        hc.images = static_cast<int>(n);
        hc.H = ti.h;
        hc.W = ti.w;
        hc.C = ti.c;
        hc.KH = node.KH;
        hc.KW = node.KW;
        hc.pad_t = node.pt;
        hc.pad_l = node.pl;
        hc.OH = node.OH;
        hc.OW = node.OW;
        hc.w0 = node.d_w0;
        hc.w1 = node.d_w1;
        hc.out_channels = node.O;
        auto hl = std::make_shared<TcHaloLaunch>();
        if (tc_plan_conv_halo(hl.get(), kind, hc, te, sm_count_, halo_level() >= 2).empty()) {
          s.kernel = std::string(hl->pair ? "tc_conv_halo_kernel:pairs<" : "tc_conv_halo_kernel<") + kind_name + ">";
          s.run = [hl](cudaStream_t st) { return tc_launch_halo(*hl, st); };
          plan.steps.push_back(std::move(s));
          return true;
        }
      }
      if (node.kind == N_CONV && node.stem && node.stem_rows && node.res < 0 && node.out_ld == 0) {
        TcStemConv sc;
        sc.kind = kind;
        sc.in0 = i8 ? static_cast<const void*>(in.q) : static_cast<const void*>(in.p0);
        sc.in1 = in.p1;
        sc.images = static_cast<int>(n);
        sc.H = ti.h;
        sc.row_bytes = ti.Wp * ti.Cp * (i8 ? 1 : 2);
        sc.KH = node.KH;
        sc.stride_h = node.sh;
        sc.pad_t = node.pt;
        sc.OH = node.OH;
        sc.OW = node.OW;
        sc.w0 = node.d_w0;
        sc.w1 = node.d_w1;
        sc.out_channels = node.O;
        auto sl = std::make_shared<TcStemLaunch>();
        if (tc_plan_stem(sl.get(), sc, te, sm_count_).empty()) {
          s.kernel = std::string("tc_stem_kernel<") + kind_name + ">";
          s.run = [sl](cudaStream_t st) { return tc_launch_stem(*sl, st); };
          plan.steps.push_back(std::move(s));
          return true;
        }
      }
      if (node.kind == N_CONV) {
        TcIm2colView v;
        v.plane0 = i8 ? static_cast<const void*>(in.q) : static_cast<const void*>(in.p0);
        v.plane1 = in.p1;
        const size_t es = static_cast<size_t>(tc_elem_bytes(kind));
        if (node.stem) {
          v.C = node.k_elems;
          v.W = node.OW;
          v.H = ti.h;
          v.N = n;
          v.stride_w = static_cast<uint64_t>(node.sw) * ti.Cp * es;
          v.stride_h = static_cast<uint64_t>(ti.Wp) * ti.Cp * es;
          v.stride_n = v.stride_h * ti.h;
          v.KH = node.KH;
          v.KW = 1;
          v.stride_conv_h = node.sh;
          v.stride_conv_w = 1;
          v.pad_t = node.pt;
          v.pad_l = 0;
          v.dil_h = node.dh;
          v.dil_w = 1;
        } else {
          v.C = ti.c;
          v.W = ti.w;
          v.H = ti.h;
          v.N = n;
          v.stride_w = static_cast<uint64_t>(ti.c) * es;
          v.stride_h = v.stride_w * ti.w;
          v.stride_n = v.stride_h * ti.h;
          v.KH = node.KH;
          v.KW = node.KW;
          v.stride_conv_h = node.sh;
          v.stride_conv_w = node.sw;
          v.pad_t = node.pt;
          v.pad_l = node.pl;
          v.dil_h = node.dh;
          v.dil_w = node.dw;
        }
        v.OH = node.OH;
        v.OW = node.OW;
        perr = tc_plan_conv(launch.get(), kind, v, node.d_w0, node.d_w1, node.O, te, sm_count_);
      } else {
        const long long M = (to.rank == 2 ? static_cast<long long>(ti.h) : 1) * n;
        const void* a0 = i8 ? static_cast<const void*>(in.q) : static_cast<const void*>(in.p0);
        perr = tc_plan_gemm(launch.get(), kind, a0, in.p1, M, node.K, node.K, node.d_w0, node.d_w1, node.O, te, sm_count_);
      }
      if (!perr.empty()) return fail(err, "layer " + node.name + ": " + perr);
      s.kernel = std::string(launch->cta2 == 2 ? (launch->p.streamk ? "tc_gemm2_kernel:pairs+split<" : "tc_gemm2_kernel:pairs<") : (launch->cta2 == 1 ? "tc_gemm2_kernel:split<" : "tc_gemm_kernel<")) + kind_name + ">";
      s.run = [launch](cudaStream_t st) { return tc_launch(*launch, st); };
      plan.steps.push_back(std::move(s));
    } else if (node.kind == N_CONV || node.kind == N_DW) {
      ConvGeom g{};
      g.images = n;
      g.H = ti.h;
      g.W = ti.w;
      g.C = ti.c;
      g.OH = node.OH;
      g.OW = node.OW;
      g.O = node.O;
      g.KH = node.KH;
      g.KW = node.KW;
      g.sh = node.sh;
      g.sw = node.sw;
      g.pt = node.pt;
      g.pl = node.pl;
      g.dh = node.dh;
      g.dw = node.dw;
      const void* w = node.d_w0;
      if (node.kind == N_DW && !i8 && ti.c % 4 == 0 && node.KH == 3 && node.KW == 3 && node.dh == 1 &&
          node.dw == 1 && node.sh == node.sw && (node.sh == 1 || node.sh == 2) && n <= 65535) {
        const dim3 grid(((node.OH + 7) / 8) * ((node.OW + 7) / 8), (ti.c / 4 + 7) / 8, static_cast<unsigned>(n));
        const int stride = node.sh;
        const float* wf = static_cast<const float*>(w);
        s.kernel = "k_depthwise3x3_tile";
        s.run = [=](cudaStream_t st) {
          if (stride == 1) k_depthwise3x3_tile<1><<<grid, 256, 0, st>>>(in, out, wf, g, e);
          else k_depthwise3x3_tile<2><<<grid, 256, 0, st>>>(in, out, wf, g, e);
          return launch_ok();
        };
      } else if (node.kind == N_DW) {
        const bool vec = ti.c % 4 == 0;
        const long long work = n * node.OH * node.OW * (vec ? ti.c / 4 : ti.c);
        const int grid = grid_for(work);
        s.kernel = i8 ? "k_depthwise<i8>" : "k_depthwise<f32>";
        s.run = [=](cudaStream_t st) {
          if (i8) {
            if (vec) k_depthwise<4, true><<<grid, 256, 0, st>>>(in, out, w, g, e);
            else k_depthwise<1, true><<<grid, 256, 0, st>>>(in, out, w, g, e);
          } else {
            if (vec) k_depthwise<4, false><<<grid, 256, 0, st>>>(in, out, w, g, e);
            else k_depthwise<1, false><<<grid, 256, 0, st>>>(in, out, w, g, e);
          }
          return launch_ok();
        };
      } else {
        const int grid = grid_for(n * node.OH * node.OW * node.O);
        s.kernel = i8 ? "k_conv_direct<i8>" : "k_conv_direct<f32>";
        s.run = [=](cudaStream_t st) {
          if (i8) k_conv_direct<true><<<grid, 256, 0, st>>>(in, out, w, g, e);
          else k_conv_direct<false><<<grid, 256, 0, st>>>(in, out, w, g, e);
          return launch_ok();
        };
      }
      plan.steps.push_back(std::move(s));
    } else {
      const long long M = (to.rank == 2 ? static_cast<long long>(ti.h) : 1) * n;
      const int K = node.K, N = node.O;
      const void* w = node.d_w0;
      const int grid = grid_for(M * N);
      s.kernel = i8 ? "k_matmul_direct<i8>" : "k_matmul_direct<f32>";
      s.run = [=](cudaStream_t st) {
        if (i8) k_matmul_direct<true><<<grid, 256, 0, st>>>(in, out, w, M, K, N, e, 0.0f);
        else k_matmul_direct<false><<<grid, 256, 0, st>>>(in, out, w, M, K, N, e, 0.0f);
        return launch_ok();
      };
      plan.steps.push_back(std::move(s));
    }
    if (node.kind == N_GEMM && node.alpha != 1.0f && !(node.impl == IMPL_TC && node.act == ACT_NONE)) {
      Step m;
      m.name = node.name + ":alpha";
      m.kernel = "k_binary";
      BinaryParams bp{};
      bp.op = BIN_MUL;
      bp.use_scalar = 1;
      bp.scalar = node.alpha;
      const long long count = to.logical() * n;
      const int grid = grid_for(count);
      m.run = [=](cudaStream_t st) {
        k_binary<1><<<grid, 256, 0, st>>>(out, out, out, count, bp);
        return launch_ok();
      };
      plan.steps.push_back(std::move(m));
    }
    return true;
  }
  if (node.kind == N_POOL) {
    const ActRef in = ref(node.in[0], n);
    PoolParams p = node.pool;
    p.images = n;
    p.side_q = node.side_q.empty() ? nullptr : ref(node.side_q[0].first, n).q;
    p.side_scale = node.side_q.empty() ? 0.0f : node.side_q[0].second;
    const bool vec = p.C % 4 == 0;
    if (p.kind == 0 && p.KH == 3 && p.KW == 3 && p.sh == 2 && p.sw == 2 && vec && !tensors_[resolve(node.in[0])].i8 &&
        n <= 65535 && p.OH * p.OW >= 64) {
      const dim3 grid(((p.OH + 7) / 8) * ((p.OW + 7) / 8), (p.C / 4 + 7) / 8, static_cast<unsigned>(n));
      s.kernel = "k_maxpool3x3s2_tile";
      s.run = [=](cudaStream_t st) {
        k_maxpool3x3s2_tile<<<grid, 256, 0, st>>>(in, out, p);
        return launch_ok();
      };
      plan.steps.push_back(std::move(s));
      return true;
    }
    const int grid = grid_for(n * p.OH * p.OW * (vec ? p.C / 4 : p.C));
    s.kernel = "k_pool";
    s.run = [=](cudaStream_t st) {
      if (vec) k_pool<4><<<grid, 256, 0, st>>>(in, out, p);
      else k_pool<1><<<grid, 256, 0, st>>>(in, out, p);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_DECONV) {
    const Tensor& ti = tensors_[resolve(node.in[0])];
    const ActRef in = ref(node.in[0], n);
    DeconvParams dp{n, ti.h, ti.w, ti.c, node.O, node.act == ACT_RELU ? 1 : 0};
    const float* w = static_cast<const float*>(node.d_w0);
    const float* bias = node.d_bias;
    const int grid = grid_for(to.logical() * n);
    s.kernel = "k_deconv2x2";
    s.run = [=](cudaStream_t st) {
      k_deconv2x2<<<grid, 256, 0, st>>>(in, out, w, bias, dp);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_REDUCE) {
    const ActRef in = ref(node.in[0], n);
    ReduceParams rp = node.reduce;
    rp.images = n;
    const int grid = grid_for(to.logical() * n);
    s.kernel = "k_reduce_mean";
    s.run = [=](cudaStream_t st) {
      k_reduce_mean<<<grid, 256, 0, st>>>(in, out, rp);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_REMAP) {
    const ActRef in = ref(node.in[0], n);
    RemapParams rp = node.remap;
    rp.images = n;
    const int grid = grid_for(to.logical() * n);
    s.kernel = "k_remap";
    s.run = [=](cudaStream_t st) {
      k_remap<<<grid, 256, 0, st>>>(in, out, rp);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_BINARY && node.broadcast) {
    const ActRef a = ref(node.in[0], n);
    const ActRef b = ref(node.in[1], n);
    BroadcastParams bp = node.bcast;
    bp.images = n;
    bp.op = node.bin;
    const int grid = grid_for(bp.o_image * n);
    s.kernel = "k_binary_broadcast";
    s.run = [=](cudaStream_t st) {
      k_binary_broadcast<<<grid, 256, 0, st>>>(a, b, out, bp);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_BINARY) {
    const ActRef a = ref(node.in[0], n);
    const ActRef b = node.in.size() > 1 ? ref(node.in[1], n) : a;
    const BinaryParams bp = node.bin;
    const long long count = to.logical() * n;
    const bool vec = count % 4 == 0;
    const int grid = grid_for(vec ? count / 4 : count);
    s.kernel = "k_binary";
    s.run = [=](cudaStream_t st) {
      if (vec) k_binary<4><<<grid, 256, 0, st>>>(a, b, out, count, bp);
      else k_binary<1><<<grid, 256, 0, st>>>(a, b, out, count, bp);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_UNARY) {
    const ActRef in = ref(node.in[0], n);
    const UnaryParams up = node.un;
    const long long count = to.logical() * n;
    const bool vec = count % 4 == 0;
    if (up.op == UN_QUANT && up.nscale == 1 && in.fmt == FMT_F32 && out.fmt == FMT_I8 && count % 16 == 0 &&
        !node.un_scale.empty()) {
      const float scale = node.un_scale[0];
      const int grid16 = grid_for(count / 16);
      const float* xp = in.p0;
      int8_t* yp = out.q;
      s.kernel = "k_quantize16";
      s.run = [=](cudaStream_t st) {
        k_quantize16<<<grid16, 256, 0, st>>>(xp, yp, count / 16, scale);
        return launch_ok();
      };
      plan.steps.push_back(std::move(s));
      return true;
    }
    const int grid = grid_for(vec ? count / 4 : count);
    s.kernel = "k_unary";
    s.run = [=](cudaStream_t st) {
      if (vec) k_unary<4><<<grid, 256, 0, st>>>(in, out, count, up);
      else k_unary<1><<<grid, 256, 0, st>>>(in, out, count, up);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_SOFTMAX) {
    const ActRef in = ref(node.in[0], n);
    SoftmaxParams sp = node.softmax;
    sp.images = n;
    const int grid = grid_for(n * sp.lines * 32);
    s.kernel = "k_softmax";
    s.run = [=](cudaStream_t st) {
      k_softmax<<<grid, 256, 0, st>>>(in, out, sp);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_CONCAT) {
    for (size_t k = 0; k < node.in.size(); ++k) {
      Step c = s;
      c.name = node.name + ":" + std::to_string(k);
      c.flops = 0;
      c.bytes = 2.0 * bytes_of(node.in[k]);
      const ActRef in = ref(node.in[k], n);
      ConcatParams cp = node.concat[k];
      cp.images = n;
      const int grid = grid_for(n * cp.in_image_elems);
      c.kernel = "k_concat_copy";
      c.run = [=](cudaStream_t st) {
        k_concat_copy<<<grid, 256, 0, st>>>(in, out, cp);
        return launch_ok();
      };
      plan.steps.push_back(std::move(c));
    }
    return true;
  }
  if (node.kind == N_RELAYOUT) {
    const ActRef in = ref(node.in[0], n);
    RelayoutParams rp = node.relayout;
    rp.images = n;
    const int grid = grid_for(rp.count * n);
    s.kernel = "k_relayout";
    s.run = [=](cudaStream_t st) {
      k_relayout<<<grid, 256, 0, st>>>(in, out, rp);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  return fail(err, "internal: unknown node kind");
}

void EngineImpl::make_edge_steps(int64_t n, const std::vector<const float*>& d_in,
                                 const std::vector<float*>& d_out, std::vector<Step>* pre,
                                 std::vector<Step>* post) {
  for (size_t i = 0; i < inputs_.size(); ++i) {
    const Tensor& t = tensors_[resolve(inputs_[i])];
    const ActRef dst = ref(inputs_[i], n);
    const float* src_ptr = d_in[i];
    Step s;
    s.name = "input:" + t.name;
    s.bytes = static_cast<double>(t.logical()) * n * (4 + t.elem_bytes() * t.planes());
    // one channel, or one pixel: channel-last order is the caller's order, a flat copy does it
    const bool flat_layout = (t.c == 1 || t.h * t.w == 1) && t.Cp == t.c && t.Wp == t.w && t.w_off == 0;
    const bool flat_quant = t.rank == 3 && flat_layout && t.input_quant_scale > 0.0f && dst.fmt == FMT_I8 &&
                            (t.logical() * n) % 16 == 0 && (reinterpret_cast<uintptr_t>(src_ptr) & 15) == 0 &&
                            (reinterpret_cast<uintptr_t>(dst.q) & 15) == 0;
    const bool flat_in = t.rank != 3 || (flat_layout && t.input_quant_scale <= 0.0f);
    if (flat_quant) {
      const long long count16 = t.logical() * n / 16;
      const int grid = grid_for(count16);
      const float scale = t.input_quant_scale;
      int8_t* q = dst.q;
      s.kernel = "k_quantize16";
      s.run = [=](cudaStream_t st) {
        k_quantize16<<<grid, 256, 0, st>>>(src_ptr, q, count16, scale);
        return launch_ok();
      };
    } else if (!flat_in) {
      EdgeParams ep{};
      ep.images = n;
      ep.C = t.c;
      ep.H = t.h;
      ep.W = t.w;
      ep.Cp = t.Cp;
      ep.Wp = t.Wp;
      ep.w_off = t.w_off;
      ep.quant_scale = t.input_quant_scale;
      if (t.c <= 4 && ((t.Cp == 4 && t.fmt != FMT_I8) || (t.Cp == 8 && t.fmt == FMT_I8)) && t.w % 4 == 0 &&
          n <= 65535 &&
          (reinterpret_cast<uintptr_t>(src_ptr) & 15) == 0) {
        const dim3 grid(static_cast<unsigned>(std::min(148 * 8, (t.h * t.w / 4 + 255) / 256)), static_cast<unsigned>(n));
        s.kernel = "k_chw_to_nhwc_small_x4";
        s.run = [=](cudaStream_t st) {
          k_chw_to_nhwc_small_x4<<<grid, 256, 0, st>>>(src_ptr, dst, ep);
          return launch_ok();
        };
      } else if (t.c <= 4 && (t.Cp == 4 || t.Cp == 16 || (t.Cp == 8 && t.fmt == FMT_I8))) {
        const int grid = grid_for(n * t.h * t.w);
        s.kernel = "k_chw_to_nhwc_small";
        s.run = [=](cudaStream_t st) {
          k_chw_to_nhwc_small<<<grid, 256, 0, st>>>(src_ptr, dst, ep);
          return launch_ok();
        };
      } else {
        const dim3 grid((t.h * t.w + 31) / 32, (t.c + 31) / 32, static_cast<unsigned>(n));
        s.kernel = "k_chw_to_nhwc_tiled";
        s.run = [=](cudaStream_t st) {
          k_chw_to_nhwc_tiled<<<grid, dim3(32, 8), 0, st>>>(src_ptr, dst, ep);
          return launch_ok();
        };
      }
    } else {
      ActRef src;
      src.fmt = FMT_F32;
      src.p0 = const_cast<float*>(src_ptr);
      UnaryParams up{};
      up.op = UN_COPY;
      const long long count = t.logical() * n;
      const bool vec = count % 4 == 0 && (reinterpret_cast<uintptr_t>(src_ptr) & 15) == 0;
      const int grid = grid_for(vec ? count / 4 : count);
      s.kernel = "k_unary";
      s.run = [=](cudaStream_t st) {
        if (vec) k_unary<4><<<grid, 256, 0, st>>>(src, dst, count, up);
        else k_unary<1><<<grid, 256, 0, st>>>(src, dst, count, up);
        return launch_ok();
      };
    }
    pre->push_back(std::move(s));
  }
  for (size_t i = 0; i < outputs_.size(); ++i) {
    const Tensor& t = tensors_[resolve(outputs_[i])];
    const ActRef src = ref(outputs_[i], n);
    float* dst_ptr = d_out[i];
    Step s;
    s.name = "output:" + t.name;
    s.bytes = static_cast<double>(t.logical()) * n * (4 + t.elem_bytes() * t.planes());
    const bool flat_out = t.rank != 3 || ((t.c == 1 || t.h * t.w == 1) && t.Cp == t.c && t.Wp == t.w && t.w_off == 0);
    if (!flat_out) {
      const dim3 grid((t.h * t.w + 31) / 32, (t.c + 31) / 32, static_cast<unsigned>(n));
      const int C = t.c, HW = t.h * t.w, Cp = t.Cp;
      s.kernel = "k_nhwc_to_chw_tiled";
      s.run = [=](cudaStream_t st) {
        k_nhwc_to_chw_tiled<<<grid, dim3(32, 8), 0, st>>>(src, dst_ptr, n, C, HW, Cp);
        return launch_ok();
      };
    } else {
      ActRef dst;
      dst.fmt = FMT_F32;
      dst.p0 = dst_ptr;
      UnaryParams up{};
      up.op = UN_COPY;
      const long long count = t.logical() * n;
      const bool vec = count % 4 == 0 && (reinterpret_cast<uintptr_t>(dst_ptr) & 15) == 0;
      const int grid = grid_for(vec ? count / 4 : count);
      s.kernel = "k_unary";
      s.run = [=](cudaStream_t st) {
        if (vec) k_unary<4><<<grid, 256, 0, st>>>(src, dst, count, up);
        else k_unary<1><<<grid, 256, 0, st>>>(src, dst, count, up);
        return launch_ok();
      };
    }
    post->push_back(std::move(s));
  }
}

Plan* EngineImpl::plan_for(int64_t n) {
  if (opt_.plan_only) {
    error_ = "the model was loaded in plan-only mode and cannot run";
    return nullptr;
  }
  auto it = plans_.find(n);
  if (it != plans_.end()) {
    it->second.last_used = ++use_counter_;
    return &it->second;
  }
  // A new batch size lays the shared arena out anew and clears it: nothing of this model may still be
  // running, on any stream (one call in flight per handle is the rule; this makes a violation harmless).
  cudaDeviceSynchronize();
  // bounded cache: a plan owns graphs and staging buffers; the least recently used one goes first
  while (plans_.size() >= kMaxCachedPlans) {
    auto oldest = plans_.begin();
    for (auto p = plans_.begin(); p != plans_.end(); ++p)
      if (p->second.last_used < oldest->second.last_used) oldest = p;
    oldest->second.release();
    plans_.erase(oldest);
  }
  // the arena is shared by all plans; grow it when a larger batch arrives.  Offsets
  // scale with n, so plans of other batch sizes stay valid only for their own n.
  const size_t need = arena_per_image_ * static_cast<size_t>(n) + 4096;
  if (need > arena_bytes_) {
    for (auto& kv : plans_) kv.second.release();
    plans_.clear();
    if (arena_ != nullptr) cudaFree(arena_);
    arena_ = nullptr;
    void* p = nullptr;
    if (device_alloc(&p, need) != cudaSuccess) {
      error_ = "out of device memory for a batch of " + std::to_string(n) + " (" + std::to_string(need >> 20) + " MiB of activations)";
      arena_bytes_ = 0;
      return nullptr;
    }
    arena_ = static_cast<uint8_t*>(p);
    arena_bytes_ = need;
  }
  // padding of stem inputs must read as zero: clear once, nothing writes there later
  cudaMemsetAsync(arena_, 0, arena_bytes_, stream_);
  cudaStreamSynchronize(stream_);
  Plan plan;
  plan.n = n;
  for (const Node& node : nodes_) {
    std::string err;
    if (!emit_node(plan, node, n, &err)) {
      error_ = err;
      return nullptr;
    }
  }
  plan.last_used = ++use_counter_;
  auto res = plans_.emplace(n, std::move(plan));
  return &res.first->second;
}

// Plans of different batch sizes lay the same arena out differently.  The zero padding
// around a stem input is written once per plan, so after a run of another size it has to
// be restored before this plan reads it.
void EngineImpl::restore_padding(int64_t n, cudaStream_t st) {
  if (last_run_n_ == n) return;
  if (last_run_n_ != 0) {
    for (const Tensor& t : tensors_) {
      if (!t.dedicated || t.alias >= 0) continue;
      cudaMemsetAsync(arena_ + t.offset * static_cast<size_t>(n), 0, t.plane_bytes * t.planes() * static_cast<size_t>(n), st);
    }
  }
  last_run_n_ = n;
}

bool EngineImpl::ensure_staging(Plan* plan) {
  if (!plan->d_in.empty() || inputs_.empty()) return true;
  // all or nothing: a plan with part of its staging arrays would pass the test above on the next call
  auto give_up = [&](const char* what) {
    for (float* p : plan->d_in) cudaFree(p);
    for (float* p : plan->d_out) cudaFree(p);
    plan->d_in.clear();
    plan->d_out.clear();
    error_ = std::string("out of device memory for ") + what + " staging";
    return false;
  };
  for (int t : inputs_) {
    void* p = nullptr;
    if (device_alloc(&p, tensors_[resolve(t)].logical() * 4 * plan->n) != cudaSuccess) return give_up("input");
    plan->d_in.push_back(static_cast<float*>(p));
  }
  for (int t : outputs_) {
    void* p = nullptr;
    if (device_alloc(&p, tensors_[resolve(t)].logical() * 4 * plan->n) != cudaSuccess) return give_up("output");
    plan->d_out.push_back(static_cast<float*>(p));
  }
  return true;
}

bool EngineImpl::issue_steps(const std::vector<Step>& steps, cudaStream_t st) {
  for (const Step& step : steps) {
    const cudaError_t e = step.run(st);
    if (e != cudaSuccess) {
      error_ = "launch of " + step.kernel + " for layer " + step.name + " failed: " + cudaGetErrorString(e);
      return false;
    }
  }
  return true;
}

// Captures the steps into an executable graph.  Capture happens on the runtime's own stream
// with nothing in flight, so that queued work does not end up inside the graph.
cudaGraphExec_t EngineImpl::capture_steps(const std::vector<Step>& steps) {
  cudaStreamSynchronize(stream_);
  cudaGraph_t g = nullptr;
  cudaGraphExec_t exec = nullptr;
  cudaError_t e = cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal);
  if (e == cudaSuccess) {
    const bool ok = issue_steps(steps, stream_);
    const cudaError_t ee = cudaStreamEndCapture(stream_, &g);
    e = ok ? ee : cudaErrorUnknown;
  }
  if (e == cudaSuccess) e = cudaGraphInstantiate(&exec, g, 0);
  if (g != nullptr) cudaGraphDestroy(g);
  if (e != cudaSuccess) {
    if (error_.empty()) error_ = std::string("CUDA graph capture failed: ") + cudaGetErrorString(e);
    return nullptr;
  }
  return exec;
}

// Enqueues one pass of `plan` on `st`: input edges, layers, output edges; as a replay of the
// captured graph when graphs are enabled (re-captured when the edge pointers changed).
int EngineImpl::launch(Plan* plan, const std::vector<const float*>& d_in, const std::vector<float*>& d_out,
                       cudaStream_t st) {
  const int64_t n = plan->n;
  restore_padding(n, st);
  std::vector<Step> all, post;
  make_edge_steps(n, d_in, d_out, &all, &post);
  all.insert(all.end(), plan->steps.begin(), plan->steps.end());
  all.insert(all.end(), post.begin(), post.end());
  if (!opt_.use_cuda_graph) return issue_steps(all, st) ? 0 : 6;
  std::vector<const void*> ptrs;
  for (auto p : d_in) ptrs.push_back(p);
  for (auto p : d_out) ptrs.push_back(p);
  if (plan->graph == nullptr || plan->graph_ptrs != ptrs) {
    if (plan->graph != nullptr) {
      cudaGraphExecDestroy(plan->graph);
      plan->graph = nullptr;
    }
    plan->graph = capture_steps(all);
    if (plan->graph == nullptr) return 6;
    plan->graph_ptrs = ptrs;
  }
  const cudaError_t e = cudaGraphLaunch(plan->graph, st);
  if (e != cudaSuccess) {
    error_ = std::string("launch failed: ") + cudaGetErrorString(e);
    return 6;
  }
  return 0;
}

// Reads back the device status word, waits for the stream and maps the outcome to a status.
int EngineImpl::finish_host_run(cudaStream_t st) {
  int status = 0;
  cudaMemcpyAsync(&status, d_status_, 4, cudaMemcpyDeviceToHost, st);
  const cudaError_t e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) {
    error_ = std::string("execution failed: ") + cudaGetErrorString(e);
    return 6;
  }
  if (status != 0) {
    error_ = "a tensor-core pipeline wait timed out (status " + std::to_string(status) + ")";
    cudaMemset(d_status_, 0, 4);
    cudaMemset(d_split_flags_, 0, kTcSplitFlagCount * sizeof(int));  // pieces nobody consumed
    return 7;
  }
  return 0;
}

// Splits the plan into per-chunk heads and a whole-batch tail (see Plan).  A layer joins the
// head only while a chunk still fills the GPU: a tensor-core convolution needs at least two
// 128-pixel tiles per SM in every chunk.
bool EngineImpl::build_pipeline(Plan* plan) {
  if (plan->chunks != 0) return true;
  const int64_t n = plan->n;
  // four chunks measured best on a 64-image ResNet-18 batch (two leave more upload exposed,
  // eight make the per-chunk layers too small)
  const int chunks = n % 4 == 0 ? 4 : 2;
  const int64_t cnt = n / chunks;
  int head_end = 0;
  for (; head_end < head_limit_; ++head_end) {
    const Node& node = nodes_[head_end];
    if ((node.kind == N_CONV && node.impl == IMPL_TC) &&
        cnt * node.OH * node.OW < 2ll * kTcBlockM * sm_count_)
      break;
    if (node.kind == N_IP || node.kind == N_GEMM) break;
  }
  for (int c = 0; c < chunks; ++c) {
    layout_n_ = n;
    img0_ = c * cnt;
    std::vector<const float*> d_in;
    for (size_t i = 0; i < inputs_.size(); ++i)
      d_in.push_back(plan->d_in[i] + static_cast<size_t>(tensors_[resolve(inputs_[i])].logical()) * img0_);
    std::vector<Step> post;
    plan->head[c].clear();
    make_edge_steps(cnt, d_in, plan->d_out, &plan->head[c], &post);
    Plan piece;
    piece.n = cnt;
    bool ok = true;
    for (int k = 0; k < head_end && ok; ++k) {
      std::string err;
      ok = emit_node(piece, nodes_[k], cnt, &err);
      if (!ok) error_ = err;
    }
    layout_n_ = 0;
    img0_ = 0;
    if (!ok) return false;
    plan->head[c].insert(plan->head[c].end(), piece.steps.begin(), piece.steps.end());
  }
  {
    Plan piece;
    piece.n = n;
    for (size_t k = head_end; k < nodes_.size(); ++k) {
      std::string err;
      if (!emit_node(piece, nodes_[k], n, &err)) {
        error_ = err;
        return false;
      }
    }
    std::vector<const float*> d_in(plan->d_in.begin(), plan->d_in.end());
    std::vector<Step> pre, post;
    make_edge_steps(n, d_in, plan->d_out, &pre, &post);
    plan->tail = piece.steps;
    plan->tail.insert(plan->tail.end(), post.begin(), post.end());
  }
  if (opt_.use_cuda_graph) {
    for (int c = 0; c < chunks; ++c) {
      plan->head_graph[c] = capture_steps(plan->head[c]);
      if (plan->head_graph[c] == nullptr) return false;
    }
    plan->tail_graph = capture_steps(plan->tail);
    if (plan->tail_graph == nullptr) return false;
  }
  plan->head_end = head_end;
  plan->chunks = chunks;
  return true;
}

// Host-pointer run with the upload hidden behind the first layers: all chunks go to the copy
// stream at once, the compute stream handles chunk c as soon as its upload has landed, then
// the rest of the network runs on the whole batch.  Results equal the one-piece run bit for
// bit: images are independent and every kernel accumulates in the same order.
int EngineImpl::run_host_pipelined(Plan* plan, const float* const* in, float* const* out) {
  const int64_t n = plan->n;
  if (copy_stream_ == nullptr) {
    bool ok = cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking) == cudaSuccess;
    for (int c = 0; c < kMaxChunks && ok; ++c)
      ok = cudaEventCreateWithFlags(&upload_done_[c], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
      error_ = "cannot create the upload stream";
      return 6;
    }
  }
  if (!ensure_staging(plan) || !build_pipeline(plan)) return 6;
  const int64_t cnt = n / plan->chunks;
  for (int c = 0; c < plan->chunks; ++c) {
    for (size_t i = 0; i < inputs_.size(); ++i) {
      const size_t count = static_cast<size_t>(tensors_[resolve(inputs_[i])].logical()) * cnt;
      cudaMemcpyAsync(plan->d_in[i] + count * c, in[i] + count * c, count * 4, cudaMemcpyHostToDevice, copy_stream_);
    }
    cudaEventRecord(upload_done_[c], copy_stream_);
  }
  restore_padding(n, stream_);
  bool ok = true;
  for (int c = 0; c < plan->chunks && ok; ++c) {
    cudaStreamWaitEvent(stream_, upload_done_[c], 0);
    if (opt_.use_cuda_graph) ok = cudaGraphLaunch(plan->head_graph[c], stream_) == cudaSuccess;
    else ok = issue_steps(plan->head[c], stream_);
  }
  if (ok) {
    if (opt_.use_cuda_graph) ok = cudaGraphLaunch(plan->tail_graph, stream_) == cudaSuccess;
    else ok = issue_steps(plan->tail, stream_);
  }
  if (!ok) {
    if (error_.empty()) error_ = "launch failed in the pipelined host path";
    cudaStreamSynchronize(copy_stream_);
    cudaStreamSynchronize(stream_);
    return 6;
  }
  for (size_t i = 0; i < outputs_.size(); ++i)
    cudaMemcpyAsync(out[i], plan->d_out[i], tensors_[resolve(outputs_[i])].logical() * 4 * n, cudaMemcpyDeviceToHost, stream_);
  return finish_host_run(stream_);
}

int EngineImpl::run(int64_t n, const float* const* in, float* const* out, bool host, cudaStream_t user_stream) {
  if (opt_.plan_only) {
    error_ = "the model was loaded in plan-only mode and cannot run";
    return 6;
  }
  if (n <= 0) {
    error_ = "batch size must be positive";
    return 2;
  }
  Plan* plan = plan_for(n);
  if (plan == nullptr) return 6;
  // Host tests of the time-out path: NCNN_B200_TEST_STALL makes the one-CTA contraction kernel leave one stage
  // unfilled, so its bounded waits run out (nothing faults or hangs; the run returns status 7).
  const bool stall = std::getenv("NCNN_B200_TEST_STALL") != nullptr;
  if (stall != stall_injected_) {
    cudaMemsetAsync(d_status_ + 1, stall ? 1 : 0, sizeof(int), host ? stream_ : user_stream);
    stall_injected_ = stall;
  }
  const char* pipe_env = std::getenv("NCNN_B200_PIPELINE");
  if (host && n % 2 == 0 && !(pipe_env != nullptr && pipe_env[0] == '0')) {
    // worth it when the upload is a visible part of the call: a few MB or more
    size_t upload = 0;
    for (int t : inputs_) upload += static_cast<size_t>(tensors_[resolve(t)].logical()) * 4 * n;
    if (upload >= kPipelineUploadBytes) return run_host_pipelined(plan, in, out);
  }
  cudaStream_t st = host ? stream_ : user_stream;
  std::vector<const float*> d_in(inputs_.size());
  std::vector<float*> d_out(outputs_.size());
  if (host) {
    if (!ensure_staging(plan)) return 6;
    for (size_t i = 0; i < inputs_.size(); ++i) {
      d_in[i] = plan->d_in[i];
      cudaMemcpyAsync(plan->d_in[i], in[i], tensors_[resolve(inputs_[i])].logical() * 4 * n, cudaMemcpyHostToDevice, st);
    }
    for (size_t i = 0; i < outputs_.size(); ++i) d_out[i] = plan->d_out[i];
  } else {
    for (size_t i = 0; i < inputs_.size(); ++i) d_in[i] = in[i];
    for (size_t i = 0; i < outputs_.size(); ++i) d_out[i] = out[i];
  }
  const int rc = launch(plan, d_in, d_out, st);
  if (rc != 0) return rc;
  if (host) {
    for (size_t i = 0; i < outputs_.size(); ++i)
      cudaMemcpyAsync(out[i], plan->d_out[i], tensors_[resolve(outputs_[i])].logical() * 4 * n, cudaMemcpyDeviceToHost, st);
    return finish_host_run(st);
  }
  return 0;
}

int EngineImpl::profile(int64_t n, int repeat, std::vector<LayerTiming>* out) {
  Plan* plan = plan_for(n);
  if (plan == nullptr) return 6;
  restore_padding(n, stream_);
  out->clear();
  // every launch of one run: input edges, layers, output edges
  std::vector<Step> all;
  if (ensure_staging(plan) && !plan->d_in.empty()) {
    std::vector<Step> pre, post;
    std::vector<const float*> d_in(plan->d_in.begin(), plan->d_in.end());
    make_edge_steps(n, d_in, plan->d_out, &pre, &post);
    all = pre;
    all.insert(all.end(), plan->steps.begin(), plan->steps.end());
    all.insert(all.end(), post.begin(), post.end());
  } else {
    all = plan->steps;
  }
  struct Events {
    std::vector<cudaEvent_t> ev;
    explicit Events(size_t n) : ev(n, nullptr) {
      for (auto& e : ev) cudaEventCreate(&e);
    }
    ~Events() {
      for (auto& e : ev)
        if (e != nullptr) cudaEventDestroy(e);
    }
    cudaEvent_t operator[](size_t i) const { return ev[i]; }
  } ev(all.size() + 1);
  std::vector<double> total(all.size(), 0.0);
  for (int r = 0; r < repeat + 1; ++r) {
    cudaEventRecord(ev[0], stream_);
    for (size_t i = 0; i < all.size(); ++i) {
      const cudaError_t e = all[i].run(stream_);
      if (e != cudaSuccess) {
        error_ = std::string("launch failed while profiling: ") + cudaGetErrorString(e);
        return 6;
      }
      cudaEventRecord(ev[i + 1], stream_);
    }
    if (cudaStreamSynchronize(stream_) != cudaSuccess) {
      error_ = "execution failed while profiling";
      return 6;
    }
    if (r == 0) continue;  // warm-up
    for (size_t i = 0; i < all.size(); ++i) {
      float ms = 0.0f;
      cudaEventElapsedTime(&ms, ev[i], ev[i + 1]);
      total[i] += ms;
    }
  }
  for (size_t i = 0; i < all.size(); ++i) {
    LayerTiming t;
    t.name = all[i].name;
    t.kernel = all[i].kernel;
    t.ms = static_cast<float>(total[i] / std::max(repeat, 1));
    t.flops = all[i].flops;
    t.bytes = all[i].bytes;
    out->push_back(t);
  }
  return 0;
}

// ---------------------------------------------------------------------- Engine
Engine::Engine() : impl_(new EngineImpl) {}
Engine::~Engine() = default;  // (~EngineImpl selects the model's device while it frees)

std::unique_ptr<Engine> Engine::create(const std::string& param_path, const std::string& bin_path,
                                       const EngineOptions& options, std::string* error) {
  std::unique_ptr<Engine> e(new Engine);
  if (!e->impl_->build(param_path, bin_path, options, error)) return nullptr;
  return e;
}

int Engine::input_count() const { return static_cast<int>(impl_->inputs_.size()); }
int Engine::output_count() const { return static_cast<int>(impl_->outputs_.size()); }

static TensorShape shape_of(const Tensor& t) {
  TensorShape s;
  s.rank = t.rank;
  if (t.rank == 3) {
    s.dims[0] = t.c;
    s.dims[1] = t.h;
    s.dims[2] = t.w;
  } else if (t.rank == 2) {
    s.dims[0] = t.h;
    s.dims[1] = t.w;
  } else {
    s.dims[0] = t.w;
  }
  return s;
}

TensorShape Engine::input_shape(int i) const { return shape_of(impl_->tensors_[impl_->inputs_[i]]); }
TensorShape Engine::output_shape(int i) const {
  int t = impl_->outputs_[i];
  while (impl_->tensors_[t].alias >= 0) t = impl_->tensors_[t].alias;
  return shape_of(impl_->tensors_[t]);
}
const std::string& Engine::input_name(int i) const { return impl_->tensors_[impl_->inputs_[i]].name; }
const std::string& Engine::output_name(int i) const { return impl_->tensors_[impl_->outputs_[i]].name; }

int Engine::run_host(int64_t n, const float* const* inputs, float* const* outputs) {
  DeviceGuard guard(impl_->device_);
  impl_->error_.clear();
  return impl_->run(n, inputs, outputs, true, nullptr);
}
int Engine::run_device(int64_t n, const float* const* inputs, float* const* outputs, cudaStream_t stream) {
  DeviceGuard guard(impl_->device_);
  impl_->error_.clear();
  return impl_->run(n, inputs, outputs, false, stream);
}
int Engine::profile(int64_t n, int repeat, std::vector<LayerTiming>* out) {
  DeviceGuard guard(impl_->device_);
  return impl_->profile(n, repeat, out);
}
int Engine::check_status() {
  if (impl_->opt_.plan_only) return 0;
  DeviceGuard guard(impl_->device_);
  int status = 0;
  if (cudaDeviceSynchronize() != cudaSuccess ||
      cudaMemcpy(&status, impl_->d_status_, 4, cudaMemcpyDeviceToHost) != cudaSuccess) {
    impl_->error_ = "execution failed";
    return 6;
  }
  if (status != 0) {
    impl_->error_ = "a tensor-core pipeline wait timed out (status " + std::to_string(status) + ")";
    cudaMemset(impl_->d_status_, 0, 4);
    cudaMemset(impl_->d_split_flags_, 0, kTcSplitFlagCount * sizeof(int));
    return 7;
  }
  return 0;
}
int Engine::launches_per_run(int64_t n) {
  DeviceGuard guard(impl_->device_);
  Plan* p = impl_->plan_for(n);
  if (p == nullptr) return -1;
  return static_cast<int>(p->steps.size() + impl_->inputs_.size() + impl_->outputs_.size());
}
const std::string& Engine::last_error() const { return impl_->error_; }

std::string Engine::plan_summary(int64_t n) {
  DeviceGuard guard(impl_->device_);
  Plan* p = impl_->plan_for(n);
  std::ostringstream o;
  if (p == nullptr) return "error: " + impl_->error_;
  o << "batch " << n << ": " << p->steps.size() << " launches, arena "
    << (impl_->arena_per_image_ * n >> 10) << " KiB\n";
  for (const Step& s : p->steps) o << "  " << s.kernel << "  " << s.name << "\n";
  return o.str();
}

}  // namespace nb
