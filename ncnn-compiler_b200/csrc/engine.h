// Graph executor of the runtime: turns a loaded ncnn model into a fused sequence
// of CUDA launches and runs it for a batch of images.
//
// The reference evaluates one image per call (every activation is rank-3 [C,H,W],
// lib/Conversion/NCNNToTosa/NCNNToTosa.cpp:48-52); this executor adds a leading image
// dimension to every tensor and guarantees that a batch of n equals n single calls.
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include <cuda_runtime.h>

namespace nb {

// Status of a failed load: the device or the runtime let us down (6), or the model was rejected (8).
inline int load_failure_status(const std::string& err) {
  for (const char* runtime_sign : {"no CUDA device", "sm_100a", "cannot select", "out of device memory", "cannot create a stream"})
    if (err.find(runtime_sign) != std::string::npos) return 6;
  return 8;
}


enum AccuracyMode : int {
  kAccuracyFp32Split = 0,  // tensor cores, operands split into two bf16 (or tf32) terms, 3 MMAs: ~1e-5
  kAccuracyTf32 = 1,       // tensor cores, one tf32 MMA: ~1e-3, reported separately
  kAccuracyFp32Cuda = 2,   // CUDA-core fp32 FMA for every contraction
};

struct EngineOptions {
  int accuracy_mode = kAccuracyFp32Split;
  int device = -1;        // -1: current device
  int use_cuda_graph = 1;
  // 1: parse, validate, fuse and infer shapes only (no CUDA call, nothing uploaded); the
  // model can describe itself and emit its stub but cannot run -- what a compile step needs
  int plan_only = 0;
  // 1: InnerProduct over a rank-2 [M,K] input yields [M,N] even when M is 1 (dynamic-M lowering)
  int keep_matrix_rows = 0;
  // shape overrides for Input layers that carry no dimensions, in Input order,
  // each as ncnn dims [c,h,w] / [h,w] / [w]
  std::vector<std::vector<int64_t>> input_shapes;
};

struct TensorShape {
  int rank = 0;
  int64_t dims[4] = {0, 0, 0, 0};  // logical dims, outermost first ([c,h,w] for rank 3, [c,d,h,w] for rank 4)
  int64_t elements() const {
    int64_t n = 1;
    for (int i = 0; i < rank; ++i) n *= dims[i];
    return n;
  }
};

struct LayerTiming {
  std::string name;
  std::string kernel;
  float ms = 0.0f;
  double flops = 0.0;  // algorithmic, per launch
  double bytes = 0.0;  // algorithmic, per launch
};

class EngineImpl;

class Engine {
 public:
  // Returns null and sets *error when the model cannot be loaded or uses a layer,
  // parameter combination or shape outside the supported path.
  static std::unique_ptr<Engine> create(const std::string& param_path, const std::string& bin_path,
                                        const EngineOptions& options, std::string* error);
  ~Engine();

  int input_count() const;
  int output_count() const;
  TensorShape input_shape(int i) const;
  TensorShape output_shape(int i) const;
  const std::string& input_name(int i) const;
  const std::string& output_name(int i) const;

  // n images; inputs[i] points at n back-to-back images of input i in the caller's
  // layout (contiguous fp32 [C][H][W]); outputs likewise.  Host-pointer variant copies
  // to and from the device inside the call.  Returns 0 on success, non-zero with
  // last_error() set otherwise.
  int run_host(int64_t n, const float* const* inputs, float* const* outputs);
  int run_device(int64_t n, const float* const* inputs, float* const* outputs, cudaStream_t stream);

  // Runs the batch `repeat` times without graph replay, timing every launch with
  // CUDA events; inputs must have been set by a previous run of the same n.
  int profile(int64_t n, int repeat, std::vector<LayerTiming>* out);

  // Synchronises the device and reports a device-side pipeline time-out (7), 0 otherwise.
  int check_status();

  // number of kernel launches one run of batch n issues
  int launches_per_run(int64_t n);

  const std::string& last_error() const;
  std::string plan_summary(int64_t n);

 private:
  Engine();
  std::unique_ptr<EngineImpl> impl_;
};

}  // namespace nb
