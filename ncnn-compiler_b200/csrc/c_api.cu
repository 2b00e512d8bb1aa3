// extern "C" boundary of the runtime (declarations and reference citations: include/ncnn_b200.h).
#include "../../include/ncnn_b200.h"

#include <cctype>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "engine.h"
#include "kernels.cuh"
#include "loader.h"

struct ncnn_b200_model {
  std::unique_ptr<nb::Engine> engine;
  std::string error;
  std::vector<std::string> names;
};

namespace {

thread_local std::string g_load_error;

int copy_out(const std::string& text, char* buffer, size_t capacity) {
  if (buffer != nullptr && capacity > 0) {
    const size_t n = std::min(text.size(), capacity - 1);
    std::memcpy(buffer, text.data(), n);
    buffer[n] = '\0';
  }
  return static_cast<int>(text.size());
}

// (a rank-4 tensor does not fit the three-extent accessors: they answer -1 for it)
int shape_out(const nb::TensorShape& s, int64_t* dims, int capacity) {
  if (s.rank > capacity) return -1;
  for (int i = 0; i < capacity; ++i) dims[i] = i < s.rank ? s.dims[i] : 0;
  return s.rank;
}

std::string upper(std::string s) {
  for (char& c : s) c = static_cast<char>(std::toupper(static_cast<unsigned char>(c)));
  return s;
}

int grid_for(long long work) {
  const long long g = (work + 255) / 256;
  return static_cast<int>(std::max<long long>(1, std::min<long long>(g, 148ll * 32)));
}

}  // namespace

namespace nb {
// lets other translation units of the library report through ncnn_b200_last_error(NULL)
void set_global_error(const std::string& message) { g_load_error = message; }

// a path as the inside of a C string literal
std::string c_string_escape(const char* text) {
  std::string out;
  for (const char* c = text; *c != 0; ++c) {
    if (*c == '\\' || *c == '"') out.push_back('\\');
    if (*c == '\n') {
      out += "\\n";
      continue;
    }
    out.push_back(*c);
  }
  return out;
}

}  // namespace nb

extern "C" {

int ncnn_b200_load(const char* param_path, const char* bin_path, const ncnn_b200_options* options,
                   ncnn_b200_model** out) try {
  if (out == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  *out = nullptr;
  if (param_path == nullptr) {
    g_load_error = "param path is NULL";
    return NCNN_B200_STATUS_NULL_POINTER;
  }
  nb::EngineOptions opt;
  if (options != nullptr) {
    if (options->struct_size != sizeof(ncnn_b200_options)) {
      g_load_error = "ncnn_b200_options.struct_size does not match this library";
      return NCNN_B200_STATUS_LOAD;
    }
    opt.accuracy_mode = options->accuracy_mode;
    opt.device = options->device;
    opt.use_cuda_graph = options->use_cuda_graph;
    opt.plan_only = options->plan_only;
    opt.keep_matrix_rows = options->keep_matrix_rows;
    const int64_t* p = options->input_shapes;
    for (int i = 0; i < options->input_shape_count && p != nullptr; ++i) {
      const int64_t rank = *p++;
      if (rank < 1 || rank > 3) {
        g_load_error = "input shape override must have rank 1..3";
        return NCNN_B200_STATUS_LOAD;
      }
      opt.input_shapes.emplace_back(p, p + rank);
      p += rank;
    }
  }
  std::string err;
  std::unique_ptr<nb::Engine> engine =
      nb::Engine::create(param_path, bin_path != nullptr ? bin_path : "", opt, &err);
  if (!engine) {
    g_load_error = err;
    return nb::load_failure_status(err);
  }
  auto* m = new ncnn_b200_model;
  m->engine = std::move(engine);
  *out = m;
  return NCNN_B200_STATUS_SUCCESS;
} catch (const std::exception& e) {
  nb::set_global_error(std::string("internal error: ") + e.what());
  return NCNN_B200_STATUS_LOAD;
} catch (...) {
  nb::set_global_error("internal error");
  return NCNN_B200_STATUS_LOAD;
}

void ncnn_b200_free(ncnn_b200_model* model) { delete model; }

const char* ncnn_b200_last_error(const ncnn_b200_model* model) {
  if (model == nullptr) return g_load_error.c_str();
  return model->error.c_str();
}

int ncnn_b200_input_count(const ncnn_b200_model* m) { return m ? m->engine->input_count() : -1; }
int ncnn_b200_output_count(const ncnn_b200_model* m) { return m ? m->engine->output_count() : -1; }

int ncnn_b200_input_shape(const ncnn_b200_model* m, int i, int64_t dims[3]) {
  if (m == nullptr || dims == nullptr || i < 0 || i >= m->engine->input_count()) return -1;
  return shape_out(m->engine->input_shape(i), dims, 3);
}

int ncnn_b200_output_shape(const ncnn_b200_model* m, int i, int64_t dims[3]) {
  if (m == nullptr || dims == nullptr || i < 0 || i >= m->engine->output_count()) return -1;
  return shape_out(m->engine->output_shape(i), dims, 3);
}

int ncnn_b200_input_shape4(const ncnn_b200_model* m, int i, int64_t dims[4]) {
  if (m == nullptr || dims == nullptr || i < 0 || i >= m->engine->input_count()) return -1;
  return shape_out(m->engine->input_shape(i), dims, 4);
}

int ncnn_b200_output_shape4(const ncnn_b200_model* m, int i, int64_t dims[4]) {
  if (m == nullptr || dims == nullptr || i < 0 || i >= m->engine->output_count()) return -1;
  return shape_out(m->engine->output_shape(i), dims, 4);
}

const char* ncnn_b200_input_name(const ncnn_b200_model* m, int i) {
  if (m == nullptr || i < 0 || i >= m->engine->input_count()) return nullptr;
  return m->engine->input_name(i).c_str();
}

const char* ncnn_b200_output_name(const ncnn_b200_model* m, int i) {
  if (m == nullptr || i < 0 || i >= m->engine->output_count()) return nullptr;
  return m->engine->output_name(i).c_str();
}

static int check_pointers(ncnn_b200_model* m, const float* const* inputs, float* const* outputs) {
  if (m == nullptr || inputs == nullptr || outputs == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  for (int i = 0; i < m->engine->input_count(); ++i)
    if (inputs[i] == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  for (int i = 0; i < m->engine->output_count(); ++i)
    if (outputs[i] == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  return NCNN_B200_STATUS_SUCCESS;
}

int ncnn_b200_run_batch(ncnn_b200_model* m, int64_t n, const float* const* inputs,
                        float* const* outputs) try {
  const int st = check_pointers(m, inputs, outputs);
  if (st != 0) return st;
  if (n <= 0) {
    m->error = "batch size must be positive";
    return NCNN_B200_STATUS_INVALID_SHAPE;
  }
  const int r = m->engine->run_host(n, inputs, outputs);
  if (r != 0) m->error = m->engine->last_error();
  return r;
} catch (const std::exception& e) {
  nb::set_global_error(std::string("internal error: ") + e.what());
  return NCNN_B200_STATUS_RUNTIME;
} catch (...) {
  nb::set_global_error("internal error");
  return NCNN_B200_STATUS_RUNTIME;
}

int ncnn_b200_run(ncnn_b200_model* m, const float* const* inputs, float* const* outputs) {
  return ncnn_b200_run_batch(m, 1, inputs, outputs);
}

int ncnn_b200_run_batch_device(ncnn_b200_model* m, int64_t n, const float* const* inputs,
                               float* const* outputs, void* stream) try {
  const int st = check_pointers(m, inputs, outputs);
  if (st != 0) return st;
  if (n <= 0) {
    m->error = "batch size must be positive";
    return NCNN_B200_STATUS_INVALID_SHAPE;
  }
  const int r = m->engine->run_device(n, inputs, outputs, static_cast<cudaStream_t>(stream));
  if (r != 0) m->error = m->engine->last_error();
  return r;
} catch (const std::exception& e) {
  nb::set_global_error(std::string("internal error: ") + e.what());
  return NCNN_B200_STATUS_RUNTIME;
} catch (...) {
  nb::set_global_error("internal error");
  return NCNN_B200_STATUS_RUNTIME;
}

int ncnn_b200_check_status(ncnn_b200_model* m) try {
  if (m == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  const int r = m->engine->check_status();
  if (r != 0) m->error = m->engine->last_error();
  return r;
} catch (const std::exception& e) {
  nb::set_global_error(std::string("internal error: ") + e.what());
  return NCNN_B200_STATUS_RUNTIME;
} catch (...) {
  nb::set_global_error("internal error");
  return NCNN_B200_STATUS_RUNTIME;
}

int ncnn_b200_launch_count(ncnn_b200_model* m, int64_t n) try {
  if (m == nullptr) return -1;
  return m->engine->launches_per_run(n);
} catch (const std::exception& e) {
  nb::set_global_error(std::string("internal error: ") + e.what());
  return -1;
} catch (...) {
  nb::set_global_error("internal error");
  return -1;
}

int64_t ncnn_b200_profile(ncnn_b200_model* m, int64_t n, int repeat, char* buffer, size_t capacity) try {
  if (m == nullptr) return -NCNN_B200_STATUS_NULL_POINTER;
  std::vector<nb::LayerTiming> t;
  const int r = m->engine->profile(n, repeat, &t);
  if (r != 0) {
    m->error = m->engine->last_error();
    return -r;
  }
  std::ostringstream o;
  for (const auto& x : t)
    o << x.kernel << "\t" << x.name << "\t" << x.ms << "\t" << x.flops << "\t" << x.bytes << "\n";
  return copy_out(o.str(), buffer, capacity);
} catch (const std::exception& e) {
  nb::set_global_error(std::string("internal error: ") + e.what());
  return -1;
} catch (...) {
  nb::set_global_error("internal error");
  return -1;
}

int64_t ncnn_b200_describe(const char* param_path, const char* bin_path, char* buffer,
                           size_t capacity) try {
  if (param_path == nullptr) return -NCNN_B200_STATUS_NULL_POINTER;
  nb::ModelDef model;
  std::string err;
  std::string text;
  if (!nb::load_model(param_path, bin_path != nullptr ? bin_path : "", &model, &err)) {
    text = "ERROR: " + err + "\n";
  } else {
    text = nb::describe_model(model);
  }
  return copy_out(text, buffer, capacity);
} catch (const std::exception& e) {
  nb::set_global_error(std::string("internal error: ") + e.what());
  return -1;
} catch (...) {
  nb::set_global_error("internal error");
  return -1;
}

int ncnn_b200_emit_stub(const ncnn_b200_model* m, const char* name, const char* param_path,
                        const char* bin_path, const char* directory) try {
  if (m == nullptr || name == nullptr || param_path == nullptr || bin_path == nullptr ||
      directory == nullptr)
    return NCNN_B200_STATUS_NULL_POINTER;
  const std::string fn = name;
  const std::string macro = upper(fn);
  const std::string guard = "NCNN_" + macro + "_H";
  const nb::Engine& e = *m->engine;
  std::ostringstream h;
  h << "#ifndef " << guard << "\n#define " << guard << "\n\n#include <stdint.h>\n\n"
    << "#define NCNN_DYNAMIC_DIM INT64_C(-1)\n"
    << "#define NCNN_MAX_RANK 4\n"
    << "#define NCNN_STATUS_SUCCESS 0\n"
    << "#define NCNN_STATUS_NULL_POINTER 1\n"
    << "#define NCNN_STATUS_INVALID_SHAPE 2\n"
    << "#define NCNN_STATUS_CONSTRAINT_VIOLATION 3\n"
    << "#define NCNN_STATUS_SHAPE_ARITHMETIC_OVERFLOW 4\n"
    << "#define NCNN_STATUS_OUTPUT_CAPACITY_INSUFFICIENT 5\n\n"
    << "typedef uint16_t ncnn_float16_t;\n"
    << "typedef uint16_t ncnn_bfloat16_t;\n\n"
    << "#define " << macro << "_INPUT_COUNT " << e.input_count() << "\n"
    << "#define " << macro << "_OUTPUT_COUNT " << e.output_count() << "\n\n";
  std::ostringstream json_in, json_out;
  auto argument = [&](const std::string& arg, const nb::TensorShape& s, bool is_output,
                      std::ostringstream& json) {
    const std::string prefix = macro + "_" + upper(arg) + "_";
    h << "#define " << prefix << "RANK " << s.rank << "\n";
    for (int d = 0; d < s.rank; ++d)
      h << "#define " << prefix << "DIM" << d << " INT64_C(" << s.dims[d] << ")\n";
    h << "#define " << prefix << "DYNAMIC_DIM_MASK UINT32_C(0x0)\n";
    h << "#define " << prefix << "ELEMENTS UINT64_C(" << s.elements() << ")\n";
    if (is_output) h << "#define " << prefix << "SHAPE_DEPENDS_ON_DATA 0\n";
    h << "\n";
    json << "    {\"name\": \"" << arg << "\", \"shape\": [";
    for (int d = 0; d < s.rank; ++d) json << (d ? ", " : "") << s.dims[d];
    json << "], \"element_type\": \"f32\", \"dynamic_dim_mask\": 0}";
  };
  for (int i = 0; i < e.input_count(); ++i) {
    if (i) json_in << ",\n";
    argument("input" + std::to_string(i + 1), e.input_shape(i), false, json_in);
  }
  for (int i = 0; i < e.output_count(); ++i) {
    if (i) json_out << ",\n";
    argument("output" + std::to_string(i + 1), e.output_shape(i), true, json_out);
  }
  std::ostringstream proto;
  proto << "int " << fn << "(";
  for (int i = 0; i < e.input_count(); ++i) proto << (i ? ", " : "") << "const float *input" << i + 1;
  for (int i = 0; i < e.output_count(); ++i) proto << ", float *output" << i + 1;
  proto << ")";
  h << "\n#ifdef __cplusplus\nextern \"C\" {\n#endif\n\n" << proto.str() << ";\n"
    << "\n#ifdef __cplusplus\n}\n#endif\n\n#endif  // " << guard << "\n";

  std::ostringstream c;
  c << "/* Generated stub: exports the model entry point and forwards to libncnn_b200. */\n"
    << "#include <stddef.h>\n#include \"" << fn << ".h\"\n#include \"ncnn_b200.h\"\n\n"
    << "static ncnn_b200_model *g_model;\nstatic volatile int g_lock;\n\n"
    << "__attribute__((visibility(\"default\"))) " << proto.str() << " {\n";
  c << "  const float *inputs[" << e.input_count() << "] = {";
  for (int i = 0; i < e.input_count(); ++i) c << (i ? ", " : "") << "input" << i + 1;
  c << "};\n  float *outputs[" << e.output_count() << "] = {";
  for (int i = 0; i < e.output_count(); ++i) c << (i ? ", " : "") << "output" << i + 1;
  c << "};\n";
  c << "  for (size_t i = 0; i < sizeof(inputs) / sizeof(inputs[0]); ++i)\n"
    << "    if (inputs[i] == NULL) return NCNN_STATUS_NULL_POINTER;\n"
    << "  for (size_t i = 0; i < sizeof(outputs) / sizeof(outputs[0]); ++i)\n"
    << "    if (outputs[i] == NULL) return NCNN_STATUS_NULL_POINTER;\n"
    << "  while (__atomic_exchange_n(&g_lock, 1, __ATOMIC_ACQUIRE)) {\n  }\n"
    << "  int status = 0;\n"
    << "  if (g_model == NULL) status = ncnn_b200_load(\"" << nb::c_string_escape(param_path) << "\", \"" << nb::c_string_escape(bin_path)
    << "\", NULL, &g_model);\n"
    << "  if (status == 0) status = ncnn_b200_run(g_model, inputs, outputs);\n"
    << "  __atomic_store_n(&g_lock, 0, __ATOMIC_RELEASE);\n"
    << "  return status;\n}\n";

  std::ostringstream j;
  j << "{\n  \"function\": \"" << fn << "\",\n  \"target\": {\"triple\": \"nvptx64-nvidia-cuda\", "
    << "\"cpu\": \"sm_100a\", \"march\": \"\", \"tune\": \"\", \"features\": [], "
    << "\"execution_profile\": \"b200-runtime\"},\n  \"inputs\": [\n"
    << json_in.str() << "\n  ],\n  \"outputs\": [\n" << json_out.str() << "\n  ]\n}\n";

  const std::string dir = directory;
  const std::pair<std::string, std::string> files[] = {
      {dir + "/" + fn + ".h", h.str()}, {dir + "/" + fn + ".c", c.str()}, {dir + "/" + fn + ".json", j.str()}};
  for (const auto& f : files) {
    std::ofstream out(f.first, std::ios::binary);
    if (!out) return NCNN_B200_STATUS_RUNTIME;
    out << f.second;
  }
  return NCNN_B200_STATUS_SUCCESS;
} catch (const std::exception& e) {
  nb::set_global_error(std::string("internal error: ") + e.what());
  return NCNN_B200_STATUS_RUNTIME;
} catch (...) {
  nb::set_global_error("internal error");
  return NCNN_B200_STATUS_RUNTIME;
}

int ncnn_b200_op_quantize(const float* x, int8_t* y, int64_t count, int64_t inner, int32_t channels,
                          const float* scale, int32_t scale_count, void* stream) {
  if (x == nullptr || y == nullptr || scale == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  if (count < 0 || inner <= 0 || channels <= 0 || (scale_count != 1 && scale_count != channels))
    return NCNN_B200_STATUS_INVALID_SHAPE;
  if (count == 0) return NCNN_B200_STATUS_SUCCESS;
  nb::QuantOpParams p{};
  p.count = count;
  p.inner = inner;
  p.channels = channels;
  p.scale_in = scale;
  p.nscale_in = scale_count;
  nb::k_op_quantize<<<grid_for(count), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, p);
  return cudaGetLastError() == cudaSuccess ? NCNN_B200_STATUS_SUCCESS : NCNN_B200_STATUS_RUNTIME;
}

int ncnn_b200_op_dequantize(const int32_t* x, float* y, int64_t count, int64_t inner,
                            int32_t channels, const float* scale, int32_t scale_count,
                            const float* bias, int32_t bias_count, void* stream) {
  if (x == nullptr || y == nullptr || scale == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  if (count < 0 || inner <= 0 || channels <= 0 || (scale_count != 1 && scale_count != channels) ||
      (bias != nullptr && bias_count != 1 && bias_count != channels))
    return NCNN_B200_STATUS_INVALID_SHAPE;
  if (count == 0) return NCNN_B200_STATUS_SUCCESS;
  nb::QuantOpParams p{};
  p.count = count;
  p.inner = inner;
  p.channels = channels;
  p.scale_in = scale;
  p.nscale_in = scale_count;
  p.bias = bias;
  p.nbias = bias_count;
  nb::k_op_dequantize<<<grid_for(count), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, p);
  return cudaGetLastError() == cudaSuccess ? NCNN_B200_STATUS_SUCCESS : NCNN_B200_STATUS_RUNTIME;
}

int ncnn_b200_op_requantize(const int32_t* x, int8_t* y, int64_t count, int64_t inner,
                            int32_t channels, const float* scale_in, int32_t scale_in_count,
                            const float* scale_out, int32_t scale_out_count, const float* bias,
                            int32_t bias_count, int32_t relu, void* stream) {
  if (x == nullptr || y == nullptr || scale_in == nullptr || scale_out == nullptr)
    return NCNN_B200_STATUS_NULL_POINTER;
  if (count < 0 || inner <= 0 || channels <= 0 ||
      (scale_in_count != 1 && scale_in_count != channels) ||
      (scale_out_count != 1 && scale_out_count != channels) ||
      (bias != nullptr && bias_count != 1 && bias_count != channels))
    return NCNN_B200_STATUS_INVALID_SHAPE;
  if (count == 0) return NCNN_B200_STATUS_SUCCESS;
  nb::QuantOpParams p{};
  p.count = count;
  p.inner = inner;
  p.channels = channels;
  p.scale_in = scale_in;
  p.nscale_in = scale_in_count;
  p.scale_out = scale_out;
  p.nscale_out = scale_out_count;
  p.bias = bias;
  p.nbias = bias_count;
  p.relu = relu;
  nb::k_op_requantize<<<grid_for(count), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, p);
  return cudaGetLastError() == cudaSuccess ? NCNN_B200_STATUS_SUCCESS : NCNN_B200_STATUS_RUNTIME;
}

}  // extern "C"
