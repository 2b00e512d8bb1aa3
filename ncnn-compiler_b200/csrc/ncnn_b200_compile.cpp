// ncnn-b200-compile: the `--target=sm_100a` counterpart of the reference's ncnn-compile.
//
// The reference driver (tools/ncnn-compile.cpp) turns model.param/.bin into
// lib<model>.so + <model>.h by running four CPU lowering pipelines, clang and a link
// (:1824-2066).  For the sm_100a target none of that is needed: the graph is validated
// and shape-inferred by the runtime library (no GPU required), which also writes
// <model>.h in the reference's header layout, <model>.json and a stub <model>.c; this
// tool compiles the stub into lib<model>.so and keeps the reference's export rule: the
// library exports the entry symbol and nothing else (tools/ncnn-compile.cpp:2129-2136).
// Flag names follow the reference (tools/ncnn-compile.cpp:40-198); CPU code-generation
// flags are accepted and ignored.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <set>
#include <string>
#include <vector>

#include <sys/stat.h>

#include "../../include/ncnn_b200.h"

namespace {

// Same rule as the reference's c_identifier (tools/ncnn-compile.cpp:292): every run of
// bytes that cannot appear in a C identifier becomes one '_'; names that start with a
// digit or '_', C23 keywords and `main` get the prefix ncnn_.
std::string c_identifier(const std::string& name) {
  std::string out;
  bool replaced = false;
  for (unsigned char ch : name) {
    const bool ok = (ch >= 'a' && ch <= 'z') || (ch >= 'A' && ch <= 'Z') || (ch >= '0' && ch <= '9') || ch == '_';
    if (ok) {
      out += static_cast<char>(ch);
      replaced = false;
    } else if (!replaced) {
      out += '_';
      replaced = true;
    }
  }
  static const std::set<std::string> reserved = {
      "alignas", "alignof", "auto", "bool", "break", "case", "char", "const", "constexpr", "continue",
      "default", "do", "double", "else", "enum", "extern", "false", "float", "for", "goto", "if", "inline",
      "int", "long", "main", "nullptr", "register", "restrict", "return", "short", "signed", "sizeof", "static",
      "static_assert", "struct", "switch", "thread_local", "true", "typedef", "typeof", "typeof_unqual", "union",
      "unsigned", "void", "volatile", "while", "_Alignas", "_Alignof", "_Atomic", "_BitInt", "_Bool", "_Complex",
      "_Decimal128", "_Decimal32", "_Decimal64", "_Generic", "_Imaginary", "_Noreturn", "_Static_assert",
      "_Thread_local"};
  if (out.empty() || (out[0] >= '0' && out[0] <= '9') || out[0] == '_' || reserved.count(out)) out = "ncnn_" + out;
  return out;
}

std::string stem_of(const std::string& path) {
  const size_t slash = path.find_last_of('/');
  std::string file = slash == std::string::npos ? path : path.substr(slash + 1);
  const size_t dot = file.rfind(".param");
  if (dot != std::string::npos && dot + 6 == file.size()) file.erase(dot);
  const size_t ncnn = file.rfind(".ncnn");
  if (ncnn != std::string::npos && ncnn + 5 == file.size()) file.erase(ncnn);
  return file;
}

std::string dir_of(const char* argv0) {
  std::string p = argv0;
  const size_t slash = p.find_last_of('/');
  return slash == std::string::npos ? "." : p.substr(0, slash);
}

bool value_of(const std::string& arg, const char* flag, std::string* out) {
  const std::string prefix = std::string(flag) + "=";
  if (arg.rfind(prefix, 0) == 0) {
    *out = arg.substr(prefix.size());
    return true;
  }
  return false;
}

int fail(const std::string& message) {
  std::fprintf(stderr, "ncnn-b200-compile: error: %s\n", message.c_str());
  return 1;
}

}  // namespace

int main(int argc, char** argv) {
  std::string param, bin, name, out_dir, target = "sm_100a", value;
  std::vector<std::vector<int64_t>> shapes;
  std::vector<ncnn_b200_dim_constraint> constraints;
  bool verbose = false, name_only = false, dynamic = false;
  int accuracy = NCNN_B200_FP32_SPLIT;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    if (value_of(a, "--param", &param) || value_of(a, "--bin", &bin) || value_of(a, "--model-name", &name) ||
        value_of(a, "--output-dir", &out_dir) || value_of(a, "--target", &target)) {
      continue;
    } else if (a == "-o" && i + 1 < argc) {
      out_dir = argv[++i];
    } else if (value_of(a, "--input-shape", &value)) {
      std::vector<int64_t> dims;
      size_t pos = 0;
      while (pos <= value.size()) {
        const size_t x = value.find_first_of("xX", pos);
        const std::string tok = value.substr(pos, x == std::string::npos ? std::string::npos : x - pos);
        if (tok.empty() || tok == "*") return fail("--input-shape takes CxHxW with positive extents or ? (dynamic rank is not supported by the sm_100a target)");
        const int64_t extent = tok == "?" ? -1 : std::atoll(tok.c_str());
        if (extent == 0 || extent < -1) return fail("--input-shape extents are positive integers or ?");
        if (extent < 0) dynamic = true;
        dims.push_back(extent);
        if (x == std::string::npos) break;
        pos = x + 1;
      }
      shapes.push_back(dims);
    } else if (value_of(a, "--input-dim-constraint", &value)) {
      // INPUT:DIM:min=N,multiple=N (docs/ncnn-compile-command-line.md 2.6)
      ncnn_b200_dim_constraint c{};
      long long input = 0, dim = 0, minimum = 0, multiple = 0;
      if (std::sscanf(value.c_str(), "%lld:%lld:min=%lld,multiple=%lld", &input, &dim, &minimum, &multiple) != 4)
        return fail("--input-dim-constraint takes INPUT:DIM:min=N,multiple=N");
      c.input = static_cast<int32_t>(input);
      c.dim = static_cast<int32_t>(dim);
      c.minimum = minimum;
      c.multiple_of = multiple;
      constraints.push_back(c);
    } else if (value_of(a, "--accuracy-mode", &value)) {
      if (value == "fp32" || value == "fp32-split") accuracy = NCNN_B200_FP32_SPLIT;
      else if (value == "tf32") accuracy = NCNN_B200_TF32;
      else if (value == "fp32-cuda") accuracy = NCNN_B200_FP32_CUDA;
      else return fail("--accuracy-mode must be fp32, tf32 or fp32-cuda");
    } else if (a == "-v") {
      verbose = true;
    } else if (a == "--print-model-name") {
      name_only = true;
    } else if (a.rfind("--threads", 0) == 0 || a.rfind("--vector-width", 0) == 0 || a.rfind("--march", 0) == 0 ||
               a.rfind("--mcpu", 0) == 0 || a.rfind("--mtune", 0) == 0 || a.rfind("--precision", 0) == 0 ||
               a.rfind("-O", 0) == 0 || a.rfind("--target-feature", 0) == 0) {
      continue;  // CPU code-generation flags of the reference: accepted, meaningless here
    } else if (a.rfind("-", 0) != 0 && param.empty()) {
      param = a;
    } else {
      return fail("unknown argument: " + a);
    }
  }
  if (param.empty()) return fail("usage: ncnn-b200-compile model.param [--bin=model.bin] [--model-name=N] [--output-dir=D] [--input-shape=CxHxW]");
  if (target != "sm_100a") return fail("this tool emits the sm_100a target only");
  if (bin.empty()) {
    bin = param;
    const size_t dot = bin.rfind(".param");
    if (dot == std::string::npos) return fail("cannot derive the .bin path from " + param);
    bin.replace(dot, 6, ".bin");
  }
  const std::string fn = c_identifier(name.empty() ? stem_of(param) : name);
  if (name_only) {
    std::printf("%s\n", fn.c_str());
    return 0;
  }
  if (out_dir.empty()) out_dir = fn;
  mkdir(out_dir.c_str(), 0755);

  std::vector<int64_t> flat;
  for (const auto& s : shapes) {
    flat.push_back(static_cast<int64_t>(s.size()));
    flat.insert(flat.end(), s.begin(), s.end());
  }
  ncnn_b200_options opt;
  std::memset(&opt, 0, sizeof(opt));
  opt.struct_size = sizeof(opt);
  opt.accuracy_mode = accuracy;
  opt.device = -1;
  opt.use_cuda_graph = 1;
  opt.input_shape_count = static_cast<int32_t>(shapes.size());
  opt.input_shapes = flat.empty() ? nullptr : flat.data();
  opt.plan_only = 1;
  char real_param[4096], real_bin[4096];
  if (realpath(param.c_str(), real_param) == nullptr || realpath(bin.c_str(), real_bin) == nullptr)
    return fail("cannot resolve the model paths");
  bool infer_entry = false;
  if (dynamic) {
    // fixed-rank dynamic extents: the stub carries the shape templates and constraints
    ncnn_b200_dynamic_model* model = nullptr;
    if (ncnn_b200_dynamic_load(param.c_str(), bin.c_str(), &opt, constraints.data(),
                               static_cast<int32_t>(constraints.size()), &model) != 0)
      return fail(ncnn_b200_last_error(nullptr));
    for (int o = 0; o < ncnn_b200_dynamic_output_count(model); ++o) {
      int64_t dims[3];
      const int rank = ncnn_b200_dynamic_output_shape(model, o, dims);
      for (int d = 0; d < rank; ++d) infer_entry = infer_entry || dims[d] < 0;
    }
    if (ncnn_b200_dynamic_emit_stub(model, fn.c_str(), real_param, real_bin, out_dir.c_str()) != 0)
      return fail("cannot write into " + out_dir);
    ncnn_b200_dynamic_free(model);
  } else {
    if (!constraints.empty()) return fail("--input-dim-constraint must name a dynamic (?) dimension");
    ncnn_b200_model* model = nullptr;
    if (ncnn_b200_load(param.c_str(), bin.c_str(), &opt, &model) != 0) return fail(ncnn_b200_last_error(nullptr));
    if (ncnn_b200_emit_stub(model, fn.c_str(), real_param, real_bin, out_dir.c_str()) != 0)
      return fail("cannot write into " + out_dir);
    ncnn_b200_free(model);
  }

  const std::string lib_dir = dir_of(argv[0]);
  char real_lib[4096];
  if (realpath(lib_dir.c_str(), real_lib) == nullptr) return fail("cannot resolve the runtime directory");
  const std::string include_dir = std::string(real_lib) + "/../include";
  const std::string so = out_dir + "/lib" + fn + ".so";
  const std::string cmd = "gcc -O2 -shared -fPIC -fvisibility=hidden -I" + out_dir + " -I" + include_dir + " " + out_dir + "/" +
                          fn + ".c -o " + so + " -L" + real_lib + " -lncnn_b200 -Wl,-rpath," + real_lib +
                          " -Wl,-z,defs";
  if (verbose) std::fprintf(stderr, "%s\n", cmd.c_str());
  if (std::system(cmd.c_str()) != 0) return fail("the host compiler failed on the stub");

  // export audit, as the reference does after its link: the entry symbol and nothing else
  const std::string nm = "nm -D --defined-only " + so + " | awk '$2 == \"T\" {print $3}'";
  FILE* pipe = popen(nm.c_str(), "r");
  if (pipe == nullptr) return fail("cannot run nm for the export audit");
  std::vector<std::string> exported;
  char line[512];
  while (std::fgets(line, sizeof(line), pipe) != nullptr) {
    std::string sym = line;
    while (!sym.empty() && (sym.back() == '\n' || sym.back() == ' ')) sym.pop_back();
    if (!sym.empty()) exported.push_back(sym);
  }
  pclose(pipe);
  std::vector<std::string> expected = {fn};
  if (infer_entry) expected.push_back(fn + "_infer_output_shapes");
  std::sort(exported.begin(), exported.end());
  std::sort(expected.begin(), expected.end());
  if (exported != expected) {
    std::remove(so.c_str());
    return fail("export audit failed: the library must export exactly '" + fn + "'" +
                (infer_entry ? " and its shape inference entry" : ""));
  }
  if (verbose) std::fprintf(stderr, "wrote %s/{lib%s.so,%s.h,%s.json,%s.c}\n", out_dir.c_str(), fn.c_str(), fn.c_str(), fn.c_str(), fn.c_str());
  return 0;
}
