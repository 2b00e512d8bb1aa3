// Fixed-rank dynamic input shapes on top of the static engine.
//
// The reference compiles `--input-shape=3x?x?` models into one body with symbolic extents and a
// wrapper that validates the caller's shape arrays before it runs (GenerateCAPI.cpp:1092-1520;
// command line: docs/ncnn-compile-command-line.md sections 2.5-2.6).  This runtime plans a network
// for concrete extents (tile shapes, tensor maps and the arena depend on them), so a dynamic model
// here is a table of specialisations keyed by the dynamic extents: the first call with a new shape
// plans it, later calls replay it.  Validation order and status codes are the wrapper's:
// NULL pointer 1, extent <= 0 or static extent mismatch 2, minimum/multiple violated 3, element or
// byte count overflow 4, non-positive output extent 2, output capacity too small 5.
#include "../../include/ncnn_b200.h"

#include <algorithm>
#include <cctype>
#include <climits>
#include <cstring>
#include <fstream>
#include <list>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <sstream>
#include <string>
#include <utility>
#include <vector>

#include "loader.h"

namespace nb {
void set_global_error(const std::string& message);
std::string c_string_escape(const char* text);  // c_api.cu
}

namespace {

struct DimLimit {
  bool present = false;
  int64_t minimum = 1, multiple_of = 1;
};

struct DynInput {
  bool templated = false;        // dimensions come from the load-time template, not the .param
  std::vector<int64_t> dims;     // outermost first, -1 where the caller supplies the extent
  std::vector<DimLimit> limits;  // one per dimension
  uint32_t mask = 0;
};

struct DynOutput {
  int rank = 0;
  int64_t dims[3] = {0, 0, 0};  // -1 where the extent follows the inputs
  uint32_t mask = 0;
};

constexpr size_t kMaxPlans = 64;   // shape-only specialisations kept for shape inference
constexpr size_t kMaxEngines = 8;  // runnable specialisations (each owns an arena and graphs)

std::string upper(std::string s) {
  for (char& c : s) c = static_cast<char>(std::toupper(static_cast<unsigned char>(c)));
  return s;
}

}  // namespace

struct ncnn_b200_dynamic_model {
  std::string param, bin;
  ncnn_b200_options options{};
  std::vector<DynInput> inputs;
  std::vector<DynOutput> outputs;
  std::map<std::vector<int64_t>, ncnn_b200_model*> plans;
  std::list<std::pair<std::vector<int64_t>, ncnn_b200_model*>> engines;  // most recent first
  std::mutex lock;
  std::string error;

  ~ncnn_b200_dynamic_model() {
    for (auto& p : plans) ncnn_b200_free(p.second);
    for (auto& e : engines) ncnn_b200_free(e.second);
  }

  // Loads the static engine for one choice of the dynamic extents (`key`: the templated inputs'
  // extents, input after input).
  int specialise(const std::vector<int64_t>& key, bool plan_only, ncnn_b200_model** out) {
    std::vector<int64_t> flat;
    size_t next = 0;
    int count = 0;
    for (const DynInput& in : inputs) {
      if (!in.templated) continue;
      flat.push_back(static_cast<int64_t>(in.dims.size()));
      for (size_t d = 0; d < in.dims.size(); ++d) flat.push_back(key[next++]);
      ++count;
    }
    ncnn_b200_options opt = options;
    opt.input_shape_count = count;
    opt.input_shapes = flat.empty() ? nullptr : flat.data();
    opt.plan_only = plan_only ? 1 : 0;
    opt.keep_matrix_rows = 1;
    const int status = ncnn_b200_load(param.c_str(), bin.c_str(), &opt, out);
    if (status != NCNN_B200_STATUS_SUCCESS) error = ncnn_b200_last_error(nullptr);
    return status;
  }

  ncnn_b200_model* plan_for(const std::vector<int64_t>& key) {
    auto it = plans.find(key);
    if (it != plans.end()) return it->second;
    ncnn_b200_model* m = nullptr;
    if (specialise(key, true, &m) != NCNN_B200_STATUS_SUCCESS) return nullptr;
    if (plans.size() >= kMaxPlans) {
      ncnn_b200_free(plans.begin()->second);
      plans.erase(plans.begin());
    }
    plans.emplace(key, m);
    return m;
  }

  int engine_for(const std::vector<int64_t>& key, ncnn_b200_model** out) {
    for (auto it = engines.begin(); it != engines.end(); ++it) {
      if (it->first == key) {
        engines.splice(engines.begin(), engines, it);
        *out = engines.front().second;
        return NCNN_B200_STATUS_SUCCESS;
      }
    }
    ncnn_b200_model* m = nullptr;
    const int status = specialise(key, false, &m);
    if (status != NCNN_B200_STATUS_SUCCESS) return status;
    if (engines.size() >= kMaxEngines) {
      ncnn_b200_free(engines.back().second);
      engines.pop_back();
    }
    engines.emplace_front(key, m);
    *out = m;
    return NCNN_B200_STATUS_SUCCESS;
  }

  // The wrapper's checks on the input shape arrays, in its order.
  int validate(const int64_t* const* shapes, std::vector<int64_t>* key) {
    if (shapes == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
    for (size_t i = 0; i < inputs.size(); ++i)
      if (inputs[i].mask != 0 && shapes[i] == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
    bool invalid = false, violated = false, overflow = false;
    for (size_t i = 0; i < inputs.size(); ++i) {
      const DynInput& in = inputs[i];
      if (!in.templated) continue;
      uint64_t elements = 1;
      for (size_t d = 0; d < in.dims.size(); ++d) {
        const int64_t extent = in.mask != 0 ? shapes[i][d] : in.dims[d];
        if (in.dims[d] < 0 ? extent <= 0 : extent != in.dims[d]) invalid = true;
        if (in.limits[d].present && (extent < in.limits[d].minimum || extent % in.limits[d].multiple_of != 0))
          violated = true;
        // the engine addresses extents as int; the wrapper multiplies in 64 bits unsigned
        if (extent > INT_MAX || __builtin_mul_overflow(elements, static_cast<uint64_t>(extent), &elements))
          overflow = true;
        key->push_back(extent);
      }
      uint64_t bytes = 0;
      if (__builtin_mul_overflow(elements, static_cast<uint64_t>(sizeof(float)), &bytes)) overflow = true;
    }
    if (invalid) return NCNN_B200_STATUS_INVALID_SHAPE;
    if (violated) return NCNN_B200_STATUS_CONSTRAINT_VIOLATION;
    if (overflow) return NCNN_B200_STATUS_SHAPE_OVERFLOW;
    return NCNN_B200_STATUS_SUCCESS;
  }
};

namespace {

int fail_load(const std::string& message, int status = NCNN_B200_STATUS_LOAD) {
  nb::set_global_error(message);
  return status;
}

int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

}  // namespace

extern "C" {

int ncnn_b200_dynamic_load(const char* param_path, const char* bin_path, const ncnn_b200_options* options,
                           const ncnn_b200_dim_constraint* constraints, int32_t constraint_count,
                           ncnn_b200_dynamic_model** out) try {
  if (out == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  *out = nullptr;
  if (param_path == nullptr || options == nullptr || (constraint_count > 0 && constraints == nullptr))
    return fail_load("param path, options or constraints are NULL", NCNN_B200_STATUS_NULL_POINTER);
  if (options->struct_size != sizeof(ncnn_b200_options))
    return fail_load("ncnn_b200_options.struct_size does not match this library");
  nb::ModelDef def;
  std::string err;
  if (!nb::load_model(param_path, "", &def, &err)) return fail_load(err);
  auto model = std::make_unique<ncnn_b200_dynamic_model>();
  model->param = param_path;
  model->bin = bin_path != nullptr ? bin_path : "";
  model->options = *options;
  model->options.input_shapes = nullptr;
  model->options.input_shape_count = 0;

  // templates go to the Input layers that carry no dimensions, in layer order
  const int64_t* p = options->input_shapes;
  int used = 0;
  for (const nb::LayerDef& l : def.layers) {
    if (l.type != "Input") continue;
    const int64_t w = l.params.get_int(0, 0), h = l.params.get_int(1, 0), c = l.params.get_int(2, 0);
    for (size_t t = 0; t < l.tops.size(); ++t) {
      DynInput in;
      if (w == 0 && h == 0 && c == 0) {
        if (used >= options->input_shape_count || p == nullptr)
          return fail_load("Input dimensions are omitted without an override");
        const int64_t rank = *p++;
        if (rank < 1 || rank > 3) return fail_load("input shape override must have rank 1..3");
        in.templated = true;
        in.dims.assign(p, p + rank);
        p += rank;
        ++used;
        for (size_t d = 0; d < in.dims.size(); ++d) {
          if (in.dims[d] == 0 || in.dims[d] < -1) return fail_load("input shape extents are positive or -1 (dynamic)");
          if (in.dims[d] < 0) in.mask |= 1u << d;
        }
      } else {
        in.dims = {c, h, w};
      }
      in.limits.resize(in.dims.size());
      model->inputs.push_back(std::move(in));
    }
  }
  if (used != options->input_shape_count)
    return fail_load("the number of input shape overrides must equal the number of Inputs without dimensions");

  // constraints name an input (Input order) and one of its dynamic dimensions, once
  for (int32_t k = 0; k < constraint_count; ++k) {
    const ncnn_b200_dim_constraint& c = constraints[k];
    if (c.input < 0 || static_cast<size_t>(c.input) >= model->inputs.size())
      return fail_load("input dimension constraint names an input that does not exist");
    DynInput& in = model->inputs[c.input];
    if (c.dim < 0 || static_cast<size_t>(c.dim) >= in.dims.size() || in.dims[c.dim] >= 0)
      return fail_load("input dimension constraint must name a dynamic dimension");
    if (in.limits[c.dim].present) return fail_load("input dimension constraint is repeated");
    if (c.minimum <= 0 || c.multiple_of <= 0) return fail_load("constraint minimum and multiple must be positive");
    in.limits[c.dim] = {true, c.minimum, c.multiple_of};
  }

  // Which output extents follow the inputs: plan the network at a base shape, then with each
  // dynamic extent doubled in turn, and compare the result shapes.  (The reference derives a
  // symbolic program per output extent; here the concrete plan is the shape function.)
  std::vector<int64_t> base;
  ncnn_b200_model* base_plan = nullptr;
  for (int64_t start : {32, 64, 128, 256, 512}) {
    base.clear();
    for (const DynInput& in : model->inputs) {
      if (!in.templated) continue;
      for (size_t d = 0; d < in.dims.size(); ++d)
        base.push_back(in.dims[d] >= 0 ? in.dims[d]
                                       : round_up(std::max<int64_t>(start, in.limits[d].minimum), in.limits[d].multiple_of));
    }
    base_plan = model->plan_for(base);
    if (base_plan != nullptr) break;
  }
  if (base_plan == nullptr) return fail_load("no specialisation could be planned: " + model->error);
  const int n_out = ncnn_b200_output_count(base_plan);
  model->outputs.resize(static_cast<size_t>(n_out));
  for (int o = 0; o < n_out; ++o) {
    DynOutput& out_shape = model->outputs[o];
    out_shape.rank = ncnn_b200_output_shape(base_plan, o, out_shape.dims);
    if (out_shape.rank < 0) return fail_load("rank-4 outputs are outside the dynamic-shape path");
  }
  size_t slot = 0;
  for (const DynInput& in : model->inputs) {
    if (!in.templated) continue;
    for (size_t d = 0; d < in.dims.size(); ++d, ++slot) {
      if (in.dims[d] >= 0) continue;
      std::vector<int64_t> varied = base;
      varied[slot] *= 2;
      ncnn_b200_model* plan = model->plan_for(varied);
      if (plan == nullptr) return fail_load("the network cannot be planned when a dynamic extent doubles: " + model->error);
      for (int o = 0; o < n_out; ++o) {
        int64_t dims[3];
        const int rank = ncnn_b200_output_shape(plan, o, dims);
        if (rank != model->outputs[o].rank) return fail_load("an output changes rank with the input shape");
        for (int k = 0; k < rank; ++k)
          if (dims[k] != model->outputs[o].dims[k]) model->outputs[o].mask |= 1u << k;
      }
    }
  }
  for (DynOutput& o : model->outputs)
    for (int k = 0; k < o.rank; ++k)
      if (o.mask & (1u << k)) o.dims[k] = -1;
  *out = model.release();
  return NCNN_B200_STATUS_SUCCESS;
} catch (const std::exception& e) {
  nb::set_global_error(std::string("internal error: ") + e.what());
  return NCNN_B200_STATUS_LOAD;
} catch (...) {
  nb::set_global_error("internal error");
  return NCNN_B200_STATUS_LOAD;
}

void ncnn_b200_dynamic_free(ncnn_b200_dynamic_model* model) { delete model; }

const char* ncnn_b200_dynamic_last_error(const ncnn_b200_dynamic_model* model) {
  return model == nullptr ? ncnn_b200_last_error(nullptr) : model->error.c_str();
}

int ncnn_b200_dynamic_input_count(const ncnn_b200_dynamic_model* m) { return m == nullptr ? -1 : static_cast<int>(m->inputs.size()); }
int ncnn_b200_dynamic_output_count(const ncnn_b200_dynamic_model* m) { return m == nullptr ? -1 : static_cast<int>(m->outputs.size()); }

int ncnn_b200_dynamic_input_shape(const ncnn_b200_dynamic_model* m, int i, int64_t dims[3]) {
  if (m == nullptr || dims == nullptr || i < 0 || static_cast<size_t>(i) >= m->inputs.size()) return -1;
  const DynInput& in = m->inputs[i];
  for (size_t d = 0; d < 3; ++d) dims[d] = d < in.dims.size() ? in.dims[d] : 0;
  return static_cast<int>(in.dims.size());
}

int ncnn_b200_dynamic_output_shape(const ncnn_b200_dynamic_model* m, int i, int64_t dims[3]) {
  if (m == nullptr || dims == nullptr || i < 0 || static_cast<size_t>(i) >= m->outputs.size()) return -1;
  for (int d = 0; d < 3; ++d) dims[d] = m->outputs[i].dims[d];
  return m->outputs[i].rank;
}

int ncnn_b200_dynamic_infer_output_shapes(ncnn_b200_dynamic_model* m, const int64_t* const* input_shapes,
                                          int64_t* const* output_shapes) try {
  if (m == nullptr || output_shapes == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  std::lock_guard<std::mutex> guard(m->lock);
  std::vector<int64_t> key;
  const int status = m->validate(input_shapes, &key);
  if (status != NCNN_B200_STATUS_SUCCESS) return status;
  ncnn_b200_model* plan = m->plan_for(key);
  if (plan == nullptr) return NCNN_B200_STATUS_INVALID_SHAPE;  // an extent of the result is not positive
  for (size_t o = 0; o < m->outputs.size(); ++o) {
    if (output_shapes[o] == nullptr) continue;
    int64_t dims[3];
    const int rank = ncnn_b200_output_shape(plan, static_cast<int>(o), dims);
    for (int k = 0; k < rank; ++k) output_shapes[o][k] = dims[k];
  }
  return NCNN_B200_STATUS_SUCCESS;
} catch (const std::exception& e) {
  nb::set_global_error(std::string("internal error: ") + e.what());
  return NCNN_B200_STATUS_RUNTIME;
} catch (...) {
  nb::set_global_error("internal error");
  return NCNN_B200_STATUS_RUNTIME;
}

int ncnn_b200_dynamic_run(ncnn_b200_dynamic_model* m, const float* const* inputs, const int64_t* const* input_shapes,
                          float* const* outputs, const uint64_t* output_capacities) try {
  if (m == nullptr || inputs == nullptr || outputs == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  for (size_t i = 0; i < m->inputs.size(); ++i)
    if (inputs[i] == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  bool dynamic_output = false;
  for (size_t o = 0; o < m->outputs.size(); ++o) {
    if (outputs[o] == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
    dynamic_output = dynamic_output || m->outputs[o].mask != 0;
  }
  if (dynamic_output && output_capacities == nullptr) return NCNN_B200_STATUS_NULL_POINTER;
  std::lock_guard<std::mutex> guard(m->lock);
  std::vector<int64_t> key;
  int status = m->validate(input_shapes, &key);
  if (status != NCNN_B200_STATUS_SUCCESS) return status;
  ncnn_b200_model* plan = m->plan_for(key);
  if (plan == nullptr) return NCNN_B200_STATUS_INVALID_SHAPE;
  for (size_t o = 0; o < m->outputs.size(); ++o) {
    if (m->outputs[o].mask == 0) continue;
    int64_t dims[3];
    const int rank = ncnn_b200_output_shape(plan, static_cast<int>(o), dims);
    uint64_t required = 1;
    for (int k = 0; k < rank; ++k) required *= static_cast<uint64_t>(dims[k]);
    if (output_capacities[o] < required) return NCNN_B200_STATUS_OUTPUT_CAPACITY;
  }
  ncnn_b200_model* engine = nullptr;
  status = m->engine_for(key, &engine);
  if (status != NCNN_B200_STATUS_SUCCESS) return status;
  status = ncnn_b200_run(engine, inputs, outputs);
  if (status != NCNN_B200_STATUS_SUCCESS) m->error = ncnn_b200_last_error(engine);
  return status;
} catch (const std::exception& e) {
  nb::set_global_error(std::string("internal error: ") + e.what());
  return NCNN_B200_STATUS_RUNTIME;
} catch (...) {
  nb::set_global_error("internal error");
  return NCNN_B200_STATUS_RUNTIME;
}

int ncnn_b200_dynamic_emit_stub(const ncnn_b200_dynamic_model* m, const char* name, const char* param_path,
                                const char* bin_path, const char* directory) try {
  if (m == nullptr || name == nullptr || param_path == nullptr || bin_path == nullptr || directory == nullptr)
    return NCNN_B200_STATUS_NULL_POINTER;
  const std::string fn = name, macro = upper(fn), guard = "NCNN_" + macro + "_H";
  const size_t n_in = m->inputs.size(), n_out = m->outputs.size();
  std::ostringstream h, json_in, json_out;
  h << "#ifndef " << guard << "\n#define " << guard << "\n\n#include <stdint.h>\n\n"
    << "#define NCNN_DYNAMIC_DIM INT64_C(-1)\n#define NCNN_MAX_RANK 4\n"
    << "#define NCNN_STATUS_SUCCESS 0\n#define NCNN_STATUS_NULL_POINTER 1\n#define NCNN_STATUS_INVALID_SHAPE 2\n"
    << "#define NCNN_STATUS_CONSTRAINT_VIOLATION 3\n#define NCNN_STATUS_SHAPE_ARITHMETIC_OVERFLOW 4\n"
    << "#define NCNN_STATUS_OUTPUT_CAPACITY_INSUFFICIENT 5\n\n"
    << "typedef uint16_t ncnn_float16_t;\ntypedef uint16_t ncnn_bfloat16_t;\n\n"
    << "#define " << macro << "_INPUT_COUNT " << n_in << "\n#define " << macro << "_OUTPUT_COUNT " << n_out << "\n\n";
  // per-argument macros in the layout of the reference's header (tools/ncnn-compile.cpp:1042-1104)
  auto argument = [&](const std::string& arg, size_t rank, const int64_t* dims, uint32_t mask,
                      const std::vector<DimLimit>* limits, bool is_output, std::ostringstream& json) {
    const std::string prefix = macro + "_" + upper(arg) + "_";
    h << "#define " << prefix << "RANK " << rank << "\n";
    uint64_t elements = 1;
    for (size_t d = 0; d < rank; ++d) {
      h << "#define " << prefix << "DIM" << d << " ";
      if (dims[d] < 0) h << "NCNN_DYNAMIC_DIM\n";
      else h << "INT64_C(" << dims[d] << ")\n";
      if (dims[d] > 0) elements *= static_cast<uint64_t>(dims[d]);
    }
    h << "#define " << prefix << "DYNAMIC_DIM_MASK UINT32_C(0x" << std::hex << mask << std::dec << ")\n";
    if (limits != nullptr)
      for (size_t d = 0; d < rank; ++d)
        if ((*limits)[d].present)
          h << "#define " << prefix << "DIM" << d << "_MINIMUM INT64_C(" << (*limits)[d].minimum << ")\n"
            << "#define " << prefix << "DIM" << d << "_MULTIPLE_OF INT64_C(" << (*limits)[d].multiple_of << ")\n";
    if (mask == 0) h << "#define " << prefix << "ELEMENTS UINT64_C(" << elements << ")\n";
    if (is_output) h << "#define " << prefix << "SHAPE_DEPENDS_ON_DATA 0\n";
    h << "\n";
    json << "    {\"name\": \"" << arg << "\", \"shape\": [";
    for (size_t d = 0; d < rank; ++d) json << (d ? ", " : "") << dims[d];
    json << "], \"element_type\": \"f32\", \"dynamic_dim_mask\": " << mask << "}";
  };
  for (size_t i = 0; i < n_in; ++i) {
    if (i) json_in << ",\n";
    argument("input" + std::to_string(i + 1), m->inputs[i].dims.size(), m->inputs[i].dims.data(), m->inputs[i].mask,
             &m->inputs[i].limits, false, json_in);
  }
  for (size_t o = 0; o < n_out; ++o) {
    if (o) json_out << ",\n";
    argument("output" + std::to_string(o + 1), static_cast<size_t>(m->outputs[o].rank), m->outputs[o].dims,
             m->outputs[o].mask, nullptr, true, json_out);
  }
  // prototypes: data pointers, a shape array after every dynamic input, capacities of the dynamic
  // outputs last (tools/ncnn-compile.cpp:1108-1215)
  bool dynamic_output = false;
  std::ostringstream run, infer;
  run << "int " << fn << "(";
  infer << "int " << fn << "_infer_output_shapes(";
  bool first_infer = true;
  for (size_t i = 0; i < n_in; ++i) {
    run << (i ? ", " : "") << "const float *input" << i + 1;
    if (m->inputs[i].mask != 0) {
      run << ", const int64_t input" << i + 1 << "_shape[" << m->inputs[i].dims.size() << "]";
      infer << (first_infer ? "" : ", ") << "const int64_t input" << i + 1 << "_shape[" << m->inputs[i].dims.size() << "]";
      first_infer = false;
    }
  }
  for (size_t o = 0; o < n_out; ++o) run << ", float *output" << o + 1;
  for (size_t o = 0; o < n_out; ++o) {
    if (m->outputs[o].mask == 0) continue;
    dynamic_output = true;
    run << ", uint64_t output" << o + 1 << "_capacity";
    infer << (first_infer ? "" : ", ") << "int64_t output" << o + 1 << "_shape[" << m->outputs[o].rank << "]";
    first_infer = false;
  }
  run << ")";
  infer << ")";
  h << "\n#ifdef __cplusplus\nextern \"C\" {\n#endif\n\n" << run.str() << ";\n";
  if (dynamic_output) h << "\n" << infer.str() << ";\n";
  h << "\n#ifdef __cplusplus\n}\n#endif\n\n#endif  // " << guard << "\n";

  std::ostringstream c;
  c << "/* Generated stub: exports the model entry points and forwards to libncnn_b200. */\n"
    << "#include <stddef.h>\n#include <string.h>\n#include \"" << fn << ".h\"\n#include \"ncnn_b200.h\"\n\n"
    << "static ncnn_b200_dynamic_model *g_model;\nstatic volatile int g_lock;\n\n"
    << "static int ensure_model(void) {\n  if (g_model != NULL) return 0;\n"
    << "  static const int64_t shapes[] = {";
  int templated = 0;
  bool first = true;
  for (const DynInput& in : m->inputs) {
    if (!in.templated) continue;
    ++templated;
    c << (first ? "" : ", ") << in.dims.size();
    first = false;
    for (int64_t d : in.dims) c << ", " << d;
  }
  c << (first ? "0" : "") << "};\n";
  int n_limits = 0;
  std::ostringstream limits;
  for (size_t i = 0; i < n_in; ++i)
    for (size_t d = 0; d < m->inputs[i].limits.size(); ++d)
      if (m->inputs[i].limits[d].present) {
        limits << (n_limits ? ", " : "") << "{" << i << ", " << d << ", " << m->inputs[i].limits[d].minimum << ", "
               << m->inputs[i].limits[d].multiple_of << "}";
        ++n_limits;
      }
  c << "  static const ncnn_b200_dim_constraint limits[] = {" << (n_limits ? limits.str() : "{0, 0, 0, 0}") << "};\n"
    << "  ncnn_b200_options options;\n  memset(&options, 0, sizeof(options));\n"
    << "  options.struct_size = sizeof(options);\n  options.device = -1;\n  options.use_cuda_graph = 1;\n"
    << "  options.accuracy_mode = " << m->options.accuracy_mode << ";\n"
    << "  options.input_shape_count = " << templated << ";\n  options.input_shapes = shapes;\n"
    << "  return ncnn_b200_dynamic_load(\"" << nb::c_string_escape(param_path) << "\", \"" << nb::c_string_escape(bin_path) << "\", &options, limits, "
    << n_limits << ", &g_model);\n}\n\n";
  auto shape_table = [&]() {
    c << "  const int64_t *shapes[" << n_in << "] = {";
    for (size_t i = 0; i < n_in; ++i) {
      c << (i ? ", " : "");
      if (m->inputs[i].mask != 0) c << "input" << i + 1 << "_shape";
      else c << "NULL";
    }
    c << "};\n";
  };
  auto locked_call = [&](const std::string& call) {
    c << "  while (__atomic_exchange_n(&g_lock, 1, __ATOMIC_ACQUIRE)) {\n  }\n"
      << "  int status = ensure_model();\n  if (status == 0) status = " << call << ";\n"
      << "  __atomic_store_n(&g_lock, 0, __ATOMIC_RELEASE);\n  return status;\n}\n";
  };
  c << "__attribute__((visibility(\"default\"))) " << run.str() << " {\n";
  c << "  const float *inputs[" << n_in << "] = {";
  for (size_t i = 0; i < n_in; ++i) c << (i ? ", " : "") << "input" << i + 1;
  c << "};\n  float *outputs[" << n_out << "] = {";
  for (size_t o = 0; o < n_out; ++o) c << (o ? ", " : "") << "output" << o + 1;
  c << "};\n";
  shape_table();
  c << "  const uint64_t capacities[" << n_out << "] = {";
  for (size_t o = 0; o < n_out; ++o) {
    c << (o ? ", " : "");
    if (m->outputs[o].mask != 0) c << "output" << o + 1 << "_capacity";
    else c << "0";
  }
  c << "};\n"
    << "  for (size_t i = 0; i < " << n_in << "; ++i)\n    if (inputs[i] == NULL) return NCNN_STATUS_NULL_POINTER;\n"
    << "  for (size_t i = 0; i < " << n_out << "; ++i)\n    if (outputs[i] == NULL) return NCNN_STATUS_NULL_POINTER;\n";
  for (size_t i = 0; i < n_in; ++i)
    if (m->inputs[i].mask != 0) c << "  if (input" << i + 1 << "_shape == NULL) return NCNN_STATUS_NULL_POINTER;\n";
  locked_call("ncnn_b200_dynamic_run(g_model, inputs, shapes, outputs, capacities)");
  if (dynamic_output) {
    c << "\n__attribute__((visibility(\"default\"))) " << infer.str() << " {\n";
    shape_table();
    c << "  int64_t *results[" << n_out << "] = {";
    for (size_t o = 0; o < n_out; ++o) {
      c << (o ? ", " : "");
      if (m->outputs[o].mask != 0) c << "output" << o + 1 << "_shape";
      else c << "NULL";
    }
    c << "};\n";
    for (size_t i = 0; i < n_in; ++i)
      if (m->inputs[i].mask != 0) c << "  if (input" << i + 1 << "_shape == NULL) return NCNN_STATUS_NULL_POINTER;\n";
    for (size_t o = 0; o < n_out; ++o)
      if (m->outputs[o].mask != 0) c << "  if (output" << o + 1 << "_shape == NULL) return NCNN_STATUS_NULL_POINTER;\n";
    locked_call("ncnn_b200_dynamic_infer_output_shapes(g_model, shapes, results)");
  }

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

}  // extern "C"
