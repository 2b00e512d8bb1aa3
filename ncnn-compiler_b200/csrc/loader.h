// ncnn .param / .bin loader of the runtime.
//
// Mirrors the behaviour of the reference's front end, lib/Graph/graph.cpp
// (Graph::load :2129-2333, load_weight :1260-1327, per-layer weight loaders
// :1381-2023) and lib/Graph/parser.cpp (lexically typed values :138-198, array
// ids :91-108): same grammar, same consumption order of the .bin, same
// rejection of files that are truncated or carry trailing bytes.
#pragma once

#include <cstdint>
#include <string>
#include <utility>
#include <vector>

namespace nb {

struct ParamValue {
  enum Kind { kInt, kFloat, kIntArray, kFloatArray, kString };
  Kind kind = kInt;
  int64_t i = 0;
  float f = 0.0f;
  std::vector<int64_t> ia;
  std::vector<float> fa;
  std::string s;
};

class ParamDict {
 public:
  void set(int id, ParamValue v);
  const ParamValue* find(int id) const;
  bool has(int id) const { return find(id) != nullptr; }
  // Typed getters fall back to the default when the id is missing or holds
  // another kind, like the reference's ParamDict (graph.cpp:121-160).
  int64_t get_int(int id, int64_t dflt = 0) const;
  float get_float(int id, float dflt = 0.0f) const;
  const std::vector<float>* get_float_array(int id) const;
  const std::vector<int64_t>* get_int_array(int id) const;
  const std::vector<std::pair<int, ParamValue>>& entries() const { return entries_; }

 private:
  std::vector<std::pair<int, ParamValue>> entries_;
};

enum class WeightType { kF32, kF16, kI8 };

struct WeightTensor {
  std::vector<int64_t> shape;
  WeightType type = WeightType::kF32;
  std::vector<uint8_t> bytes;  // as stored in the .bin
  size_t count() const;
  // fp32 view (fp16 storage is widened, int8 is converted value by value)
  std::vector<float> as_f32() const;
  const int8_t* as_i8() const { return reinterpret_cast<const int8_t*>(bytes.data()); }
};

struct LayerDef {
  std::string type, name;
  std::vector<std::string> bottoms, tops;
  ParamDict params;
  std::vector<WeightTensor> weights;
};

struct ModelDef {
  std::vector<LayerDef> layers;
  std::vector<std::string> blobs;    // in creation order
  std::vector<std::string> inputs;   // tops of Input layers, layer order
  std::vector<std::string> outputs;  // blobs nobody consumes, creation order
  bool weights_loaded = false;
};

// Parses the tail of a layer line ("0=64 1=3 -23310=2,0.0,6.0 ...").
bool parse_layer_params(const std::string& tail, ParamDict* out, std::string* error);

// Loads param (and bin when bin_path is non-empty).  Returns false and sets *error.
bool load_model(const std::string& param_path, const std::string& bin_path, ModelDef* model,
                std::string* error);

// Text description in the layout of the reference's Graph::dump()
// (graph.cpp:2335-2446) followed by one FNV-1a hash per weight tensor, so a
// test can compare loaders byte for byte.
std::string describe_model(const ModelDef& model);

}  // namespace nb
