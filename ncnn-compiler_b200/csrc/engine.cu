// Graph executor: model construction, plans per batch size, CUDA graphs, the host- and device-pointer run paths,
// per-layer profiling and the public Engine facade.
#include "engine_impl.h"

namespace nb {


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
  fuse_stem_pooling();
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
  if (t.rank == 4) {
    s.dims[0] = t.c;
    s.dims[1] = t.d;
    s.dims[2] = t.h;
    s.dims[3] = t.w;
  } else if (t.rank == 3) {
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
