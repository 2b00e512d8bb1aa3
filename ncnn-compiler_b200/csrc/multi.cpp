// One model on several GPUs of a box: the batch-sharded form of the runtime behind the C ABI
// (declarations: include/ncnn_b200.h).
//
// Images are independent (the reference's entry point takes one image per call and keeps no state
// between calls, NCNNToTosa.cpp:48-52), so a batch of n images is cut into contiguous shards, one
// per device, and every device runs its shard with its own replica of the weights, its own stream
// and its own captured graph.  Nothing is exchanged between devices: with host buffers each device
// copies its shard's results straight into the caller's output array.  One host thread per device
// drives its replica, so the uploads, kernels and downloads of all devices overlap.
#include "../../include/ncnn_b200.h"

#include <condition_variable>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "engine.h"

namespace nb {
void set_global_error(const std::string& message);  // c_api.cu
}

namespace {

struct Shard {
  int64_t first = 0, count = 0;
};

// contiguous shards of ceil(n / parts) items; the last ones may be short or empty
std::vector<Shard> partition(int64_t n, int parts) {
  std::vector<Shard> out(static_cast<size_t>(parts));
  const int64_t per = (n + parts - 1) / parts;
  int64_t next = 0;
  for (int g = 0; g < parts; ++g) {
    out[g].first = next;
    out[g].count = std::max<int64_t>(0, std::min<int64_t>(per, n - next));
    next += out[g].count;
  }
  return out;
}

struct Job {
  const float* const* inputs = nullptr;
  float* const* outputs = nullptr;
  Shard shard;
};

struct Replica {
  std::unique_ptr<nb::Engine> engine;
  std::thread thread;
  std::mutex mutex;
  std::condition_variable wake;
  bool has_job = false, done = false, quit = false;
  Job job;
  int status = 0;
  std::vector<size_t> in_elems, out_elems;  // elements per image of every argument

  void loop() {
    std::unique_lock<std::mutex> lock(mutex);
    while (true) {
      wake.wait(lock, [&] { return has_job || quit; });
      if (quit) return;
      const Job j = job;
      lock.unlock();
      int st = 0;
      if (j.shard.count > 0) {
        std::vector<const float*> in(in_elems.size());
        std::vector<float*> out(out_elems.size());
        for (size_t i = 0; i < in.size(); ++i) in[i] = j.inputs[i] + static_cast<size_t>(j.shard.first) * in_elems[i];
        for (size_t i = 0; i < out.size(); ++i) out[i] = j.outputs[i] + static_cast<size_t>(j.shard.first) * out_elems[i];
        st = engine->run_host(j.shard.count, in.data(), out.data());
      }
      lock.lock();
      status = st;
      has_job = false;
      done = true;
      wake.notify_all();
    }
  }
};

}  // namespace

struct ncnn_b200_multi {
  std::vector<std::unique_ptr<Replica>> replicas;
  std::string error;
  ~ncnn_b200_multi() {
    for (auto& r : replicas) {
      {
        std::lock_guard<std::mutex> lock(r->mutex);
        r->quit = true;
      }
      r->wake.notify_all();
      if (r->thread.joinable()) r->thread.join();
    }
  }
};

extern "C" {

int ncnn_b200_multi_partition(int64_t n, int32_t parts, int64_t* first, int64_t* count) {
  if (first == nullptr || count == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  if (n < 0 || parts <= 0) return NCNN_B200_STATUS_INVALID_SHAPE;
  const std::vector<Shard> s = partition(n, parts);
  for (int g = 0; g < parts; ++g) {
    first[g] = s[g].first;
    count[g] = s[g].count;
  }
  return NCNN_B200_STATUS_SUCCESS;
}

int ncnn_b200_multi_load(const char* param_path, const char* bin_path, const ncnn_b200_options* options,
                         const int32_t* devices, int32_t device_count, ncnn_b200_multi** out) try {
  if (out == nullptr || param_path == nullptr || devices == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  *out = nullptr;
  if (device_count <= 0 || device_count > 64) {
    nb::set_global_error("multi_load: device_count must be between 1 and 64");
    return NCNN_B200_STATUS_INVALID_SHAPE;
  }
  std::unique_ptr<ncnn_b200_multi> m(new ncnn_b200_multi);
  for (int g = 0; g < device_count; ++g) {
    nb::EngineOptions opt;
    if (options != nullptr) {
      opt.accuracy_mode = options->accuracy_mode;
      opt.use_cuda_graph = options->use_cuda_graph;
      const int64_t* p = options->input_shapes;
      for (int i = 0; i < options->input_shape_count && p != nullptr; ++i) {
        const int64_t rank = *p++;
        if (rank < 1 || rank > 3) {
          nb::set_global_error("input shape override must have rank 1..3");
          return NCNN_B200_STATUS_LOAD;
        }
        opt.input_shapes.emplace_back(p, p + rank);
        p += rank;
      }
    }
    opt.device = devices[g];
    std::string err;
    std::unique_ptr<Replica> r(new Replica);
    r->engine = nb::Engine::create(param_path, bin_path != nullptr ? bin_path : "", opt, &err);
    if (!r->engine) {
      nb::set_global_error("device " + std::to_string(devices[g]) + ": " + err);
      return nb::load_failure_status(err);
    }
    for (int i = 0; i < r->engine->input_count(); ++i)
      r->in_elems.push_back(static_cast<size_t>(r->engine->input_shape(i).elements()));
    for (int i = 0; i < r->engine->output_count(); ++i)
      r->out_elems.push_back(static_cast<size_t>(r->engine->output_shape(i).elements()));
    m->replicas.push_back(std::move(r));
  }
  for (auto& r : m->replicas) r->thread = std::thread([p = r.get()] { p->loop(); });
  *out = m.release();
  return NCNN_B200_STATUS_SUCCESS;
} catch (const std::exception& e) {
  nb::set_global_error(std::string("internal error: ") + e.what());
  return NCNN_B200_STATUS_RUNTIME;
} catch (...) {
  nb::set_global_error("internal error");
  return NCNN_B200_STATUS_RUNTIME;
}

void ncnn_b200_multi_free(ncnn_b200_multi* model) { delete model; }

const char* ncnn_b200_multi_last_error(const ncnn_b200_multi* model) {
  return model == nullptr ? ncnn_b200_last_error(nullptr) : model->error.c_str();
}

int32_t ncnn_b200_multi_device_count(const ncnn_b200_multi* model) {
  return model == nullptr ? -1 : static_cast<int32_t>(model->replicas.size());
}

int ncnn_b200_multi_run_batch(ncnn_b200_multi* m, int64_t n, const float* const* inputs, float* const* outputs) try {
  if (m == nullptr || inputs == nullptr || outputs == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  const Replica& first = *m->replicas.front();
  for (size_t i = 0; i < first.in_elems.size(); ++i)
    if (inputs[i] == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  for (size_t i = 0; i < first.out_elems.size(); ++i)
    if (outputs[i] == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  if (n <= 0) {
    m->error = "batch size must be positive";
    return NCNN_B200_STATUS_INVALID_SHAPE;
  }
  const std::vector<Shard> shards = partition(n, static_cast<int>(m->replicas.size()));
  for (size_t g = 0; g < m->replicas.size(); ++g) {
    Replica& r = *m->replicas[g];
    {
      std::lock_guard<std::mutex> lock(r.mutex);
      r.job = Job{inputs, outputs, shards[g]};
      r.has_job = true;
      r.done = false;
    }
    r.wake.notify_all();
  }
  int status = 0;
  for (size_t g = 0; g < m->replicas.size(); ++g) {
    Replica& r = *m->replicas[g];
    std::unique_lock<std::mutex> lock(r.mutex);
    r.wake.wait(lock, [&] { return r.done; });
    if (r.status != 0 && status == 0) {
      status = r.status;
      m->error = "device shard " + std::to_string(g) + ": " + r.engine->last_error();
    }
  }
  return status;
} catch (const std::exception& e) {
  nb::set_global_error(std::string("internal error: ") + e.what());
  return NCNN_B200_STATUS_RUNTIME;
} catch (...) {
  nb::set_global_error("internal error");
  return NCNN_B200_STATUS_RUNTIME;
}

}  // extern "C"
