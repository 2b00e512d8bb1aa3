#include "loader.h"

#include <algorithm>
#include <cctype>
#include <cerrno>
#include <charconv>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>

namespace nb {

// ------------------------------------------------------------------ ParamDict
void ParamDict::set(int id, ParamValue v) {
  for (auto& e : entries_) {
    if (e.first == id) {
      e.second = std::move(v);
      return;
    }
  }
  entries_.emplace_back(id, std::move(v));
}

const ParamValue* ParamDict::find(int id) const {
  for (const auto& e : entries_)
    if (e.first == id) return &e.second;
  return nullptr;
}

int64_t ParamDict::get_int(int id, int64_t dflt) const {
  const ParamValue* v = find(id);
  return (v != nullptr && v->kind == ParamValue::kInt) ? v->i : dflt;
}

float ParamDict::get_float(int id, float dflt) const {
  const ParamValue* v = find(id);
  return (v != nullptr && v->kind == ParamValue::kFloat) ? v->f : dflt;
}

const std::vector<float>* ParamDict::get_float_array(int id) const {
  const ParamValue* v = find(id);
  return (v != nullptr && v->kind == ParamValue::kFloatArray) ? &v->fa : nullptr;
}

const std::vector<int64_t>* ParamDict::get_int_array(int id) const {
  const ParamValue* v = find(id);
  return (v != nullptr && v->kind == ParamValue::kIntArray) ? &v->ia : nullptr;
}

// ------------------------------------------------------------------ value parsing
namespace {

std::string lower(std::string s) {
  for (char& c : s) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
  return s;
}

bool is_nonfinite_token(std::string t) {
  if (!t.empty() && (t[0] == '-' || t[0] == '+')) t.erase(0, 1);
  t = lower(t);
  return t == "nan" || t == "inf" || t == "infinity";
}

bool is_float_token(const std::string& t) {
  return is_nonfinite_token(t) || t.find_first_of(".eE") != std::string::npos;
}

bool is_string_token(const std::string& t) {
  return !t.empty() && (std::isalpha(static_cast<unsigned char>(t[0])) || t[0] == '"');
}

bool parse_i64(const std::string& t, const char* what, int64_t* out, std::string* err) {
  if (t.empty()) {
    *err = std::string("empty ") + what;
    return false;
  }
  const char* b = t.data();
  const char* e = b + t.size();
  auto r = std::from_chars(b, e, *out);
  if (r.ec == std::errc::result_out_of_range) {
    *err = std::string(what) + " out of range: " + t;
    return false;
  }
  if (r.ec != std::errc() || r.ptr != e) {
    *err = std::string("bad ") + what + ": " + t;
    return false;
  }
  return true;
}

bool parse_f32(const std::string& t, const char* what, float* out, std::string* err) {
  if (t.empty()) {
    *err = std::string("empty ") + what;
    return false;
  }
  const char* b = t.data();
  const char* e = b + t.size();
  auto r = std::from_chars(b, e, *out);
  if (r.ec == std::errc::result_out_of_range) {
    *err = std::string(what) + " out of range: " + t;
    return false;
  }
  if (r.ec != std::errc() || r.ptr != e) {
    *err = std::string("bad ") + what + ": " + t;
    return false;
  }
  if (!std::isfinite(*out)) {
    *err = std::string("non-finite ") + what + ": " + t;
    return false;
  }
  return true;
}

bool split_commas(const std::string& text, std::vector<std::string>* out, std::string* err) {
  size_t begin = 0;
  while (true) {
    const size_t comma = text.find(',', begin);
    const size_t end = comma == std::string::npos ? text.size() : comma;
    if (end == begin) {
      *err = "array contains an empty element";
      return false;
    }
    out->push_back(text.substr(begin, end - begin));
    if (comma == std::string::npos) break;
    begin = comma + 1;
  }
  return true;
}

bool parse_array(const std::vector<std::string>& elems, size_t first, ParamValue* v,
                 std::string* err) {
  bool as_float = false;
  for (size_t i = first; i < elems.size(); ++i) as_float = as_float || is_float_token(elems[i]);
  if (as_float) {
    v->kind = ParamValue::kFloatArray;
    for (size_t i = first; i < elems.size(); ++i) {
      float f;
      if (!parse_f32(elems[i], "float array element", &f, err)) return false;
      v->fa.push_back(f);
    }
  } else {
    v->kind = ParamValue::kIntArray;
    for (size_t i = first; i < elems.size(); ++i) {
      int64_t x;
      if (!parse_i64(elems[i], "integer array element", &x, err)) return false;
      v->ia.push_back(x);
    }
  }
  return true;
}

bool parse_value(const std::string& tok, bool explicit_array, ParamValue* v, std::string* err) {
  if (tok.empty()) {
    *err = "empty param value";
    return false;
  }
  if (!explicit_array && tok[0] == '"') {
    if (tok.size() < 2 || tok.back() != '"') {
      *err = "unterminated quoted string param value";
      return false;
    }
    v->kind = ParamValue::kString;
    v->s = tok.substr(1, tok.size() - 2);
    return true;
  }
  std::vector<std::string> elems;
  if (!split_commas(tok, &elems, err)) return false;
  if (explicit_array) {
    int64_t n;
    if (!parse_i64(elems[0], "array length", &n, err)) return false;
    if (n < 0) {
      *err = "array length must be non-negative";
      return false;
    }
    if (static_cast<size_t>(n) != elems.size() - 1) {
      *err = "array length mismatch: declared " + std::to_string(n) + ", got " +
             std::to_string(elems.size() - 1);
      return false;
    }
    return parse_array(elems, 1, v, err);
  }
  if (elems.size() > 1) return parse_array(elems, 0, v, err);
  if (is_nonfinite_token(tok)) {
    v->kind = ParamValue::kFloat;
    return parse_f32(tok, "float param value", &v->f, err);
  }
  if (is_string_token(tok)) {
    v->kind = ParamValue::kString;
    v->s = tok;
    return true;
  }
  if (is_float_token(tok)) {
    v->kind = ParamValue::kFloat;
    return parse_f32(tok, "float param value", &v->f, err);
  }
  v->kind = ParamValue::kInt;
  return parse_i64(tok, "integer param value", &v->i, err);
}

std::vector<std::string> split_ws(const std::string& text) {
  std::vector<std::string> out;
  size_t pos = 0;
  while (pos < text.size()) {
    while (pos < text.size() && std::isspace(static_cast<unsigned char>(text[pos]))) ++pos;
    if (pos >= text.size()) break;
    size_t end = pos;
    while (end < text.size() && !std::isspace(static_cast<unsigned char>(text[end]))) ++end;
    out.push_back(text.substr(pos, end - pos));
    pos = end;
  }
  return out;
}

}  // namespace

bool parse_layer_params(const std::string& tail, ParamDict* out, std::string* error) {
  constexpr int64_t kArrayBase = 23300;
  constexpr int kMaxId = 31;
  size_t pos = 0;
  while (pos < tail.size()) {
    while (pos < tail.size() && std::isspace(static_cast<unsigned char>(tail[pos]))) ++pos;
    if (pos >= tail.size()) break;
    size_t end = pos;
    bool quoted = false;
    while (end < tail.size()) {
      const char c = tail[end];
      if (c == '"') {
        quoted = !quoted;
      } else if (!quoted && std::isspace(static_cast<unsigned char>(c))) {
        break;
      }
      ++end;
    }
    if (quoted) {
      *error = "unterminated quoted param value";
      return false;
    }
    const std::string assignment = tail.substr(pos, end - pos);
    const size_t eq = assignment.find('=');
    if (eq == std::string::npos) {
      *error = "missing '=' in param: " + assignment;
      return false;
    }
    if (assignment.find('=', eq + 1) != std::string::npos) {
      *error = "multiple '=' in param: " + assignment;
      return false;
    }
    int64_t raw;
    if (!parse_i64(assignment.substr(0, eq), "param id", &raw, error)) return false;
    bool explicit_array = false;
    int id;
    if (raw >= 0 && raw <= kMaxId) {
      id = static_cast<int>(raw);
    } else if (raw >= -kArrayBase - kMaxId && raw <= -kArrayBase) {
      explicit_array = true;
      id = static_cast<int>(-raw - kArrayBase);
    } else {
      *error = "param id out of range: " + assignment.substr(0, eq);
      return false;
    }
    ParamValue v;
    std::string verr;
    if (!parse_value(assignment.substr(eq + 1), explicit_array, &v, &verr)) {
      *error = "param " + std::to_string(id) + ": " + verr;
      return false;
    }
    out->set(id, std::move(v));
    pos = end;
  }
  return true;
}

// ------------------------------------------------------------------ weights
size_t WeightTensor::count() const {
  size_t n = 1;
  for (int64_t d : shape) n *= static_cast<size_t>(d);
  return n;
}

namespace {

float half_to_float(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do {
        ++e;
        man <<= 1;
      } while ((man & 0x400u) == 0);
      bits = sign | ((112 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

}  // namespace

std::vector<float> WeightTensor::as_f32() const {
  const size_t n = count();
  std::vector<float> out(n);
  if (type == WeightType::kF32) {
    std::memcpy(out.data(), bytes.data(), n * 4);
  } else if (type == WeightType::kF16) {
    const uint16_t* h = reinterpret_cast<const uint16_t*>(bytes.data());
    for (size_t i = 0; i < n; ++i) out[i] = half_to_float(h[i]);
  } else {
    const int8_t* q = as_i8();
    for (size_t i = 0; i < n; ++i) out[i] = static_cast<float>(q[i]);
  }
  return out;
}

namespace {

constexpr uint32_t kFlagF16 = 0x01306B47u;
constexpr uint32_t kFlagI8 = 0x000D4B38u;
constexpr uint32_t kFlagF32 = 0x0002C056u;

class BinCursor {
 public:
  explicit BinCursor(const std::vector<uint8_t>& d) : d_(d) {}
  size_t pos() const { return pos_; }
  size_t size() const { return d_.size(); }
  size_t remaining() const { return d_.size() - pos_; }
  std::string eof(size_t want) const {
    return "unexpected EOF at offset " + std::to_string(pos_) + ": requested " +
           std::to_string(want) + " bytes, " + std::to_string(remaining()) + " remain";
  }

  // typed == 0: a 4-byte storage flag precedes the payload; typed == 1: raw fp32.
  bool read(int64_t count, int typed, std::vector<int64_t> shape, WeightTensor* out,
            std::string* err) {
    if (count <= 0) {
      *err = "weight element count must be positive";
      return false;
    }
    size_t width = 4;
    bool align = false;
    out->type = WeightType::kF32;
    if (typed == 0) {
      if (remaining() < 4) {
        *err = "weight flag: " + eof(4);
        return false;
      }
      uint32_t flag;
      std::memcpy(&flag, d_.data() + pos_, 4);
      const size_t flag_offset = pos_;
      pos_ += 4;
      if (flag == kFlagF16) {
        out->type = WeightType::kF16;
        width = 2;
        align = true;
      } else if (flag == kFlagI8) {
        out->type = WeightType::kI8;
        width = 1;
        align = true;
      } else if (flag != kFlagF32 && flag != 0) {
        char buf[96];
        std::snprintf(buf, sizeof(buf),
                      "quantized lookup-table weight flag 0x%08x at offset %zu is unsupported", flag,
                      flag_offset);
        *err = buf;
        return false;
      }
    }
    const size_t bytes = static_cast<size_t>(count) * width;
    if (remaining() < bytes) {
      *err = "weight data: " + eof(bytes);
      return false;
    }
    out->bytes.assign(d_.begin() + pos_, d_.begin() + pos_ + bytes);
    pos_ += bytes;
    if (align) {
      const size_t pad = (4 - pos_ % 4) % 4;
      if (remaining() < pad) {
        *err = "weight alignment: " + eof(pad);
        return false;
      }
      pos_ += pad;
    }
    out->shape = std::move(shape);
    return true;
  }

 private:
  const std::vector<uint8_t>& d_;
  size_t pos_ = 0;
};

bool int_param(const ParamDict& p, int id, int64_t dflt, const char* name, int64_t* out,
               std::string* err) {
  const ParamValue* v = p.find(id);
  if (v == nullptr) {
    *out = dflt;
    return true;
  }
  if (v->kind != ParamValue::kInt) {
    *err = "parameter " + std::to_string(id) + " (" + name + ") must be integer";
    return false;
  }
  *out = v->i;
  return true;
}

bool push(LayerDef& l, BinCursor& c, int64_t n, int typed, std::vector<int64_t> shape,
          const char* what, std::string* err) {
  WeightTensor w;
  std::string e;
  if (!c.read(n, typed, std::move(shape), &w, &e)) {
    *err = std::string(what) + ": " + e;
    return false;
  }
  l.weights.push_back(std::move(w));
  return true;
}

bool load_conv_like(LayerDef& l, BinCursor& c, bool depthwise, std::string* err) {
  const char* tag = depthwise ? "depthwise" : "conv";
  int64_t dyn, nout, kw, kh, bias, wsize, term, group = 1;
  if (!int_param(l.params, 19, 0, "dynamic_weight", &dyn, err)) return false;
  if (dyn != 0 && dyn != 1) {
    *err = "convolution dynamic_weight must be 0 or 1";
    return false;
  }
  if (dyn == 1) return true;
  if (!int_param(l.params, 0, 0, "num_output", &nout, err) ||
      !int_param(l.params, 1, 0, "kernel_w", &kw, err))
    return false;
  if (!int_param(l.params, 11, kw, "kernel_h", &kh, err) ||
      !int_param(l.params, 5, 0, "bias_term", &bias, err) ||
      !int_param(l.params, 6, 0, "weight_data_size", &wsize, err) ||
      !int_param(l.params, 8, 0, "int8_scale_term", &term, err))
    return false;
  if (depthwise && !int_param(l.params, 7, 1, "group", &group, err)) return false;
  if (nout <= 0) {
    *err = "convolution num_output must be positive";
    return false;
  }
  if (wsize <= 0) {
    *err = "convolution weight count must be positive";
    return false;
  }
  if (kw <= 0 || kh <= 0) {
    *err = "convolution kernel dimensions must be positive";
    return false;
  }
  if (bias != 0 && bias != 1) {
    *err = "convolution bias_term must be 0 or 1";
    return false;
  }
  if (term != 0 && term != 1 && term != 2 && term != 101 && term != 102) {
    *err = "convolution int8_scale_term must be 0, 1, 2, 101, or 102";
    return false;
  }
  if (depthwise && (group <= 0 || nout % group != 0)) {
    *err = "convolution depthwise group must be positive and divide num_output";
    return false;
  }
  const int64_t ok = nout * kh * kw;
  if (wsize % ok != 0) {
    *err = std::string(depthwise ? "depthwise" : "convolution") +
           " weight count is not divisible by output/kernel size";
    return false;
  }
  const int64_t nin = wsize / ok;
  if (!push(l, c, wsize, 0, {nout, nin, kh, kw}, depthwise ? "depthwise weight" : "conv weight",
            err))
    return false;
  if (bias == 1 && !push(l, c, nout, 1, {nout}, depthwise ? "depthwise bias" : "conv bias", err))
    return false;
  if (term != 0) {
    const int64_t nscale = depthwise ? ((term == 1 || term == 101) ? group : 1) : nout;
    if (!push(l, c, nscale, 1, {nscale},
              depthwise ? "depthwise weight int8 scales" : "conv weight int8 scales", err))
      return false;
    if (!push(l, c, 1, 1, {1},
              depthwise ? "depthwise bottom int8 scale" : "conv bottom int8 scale", err))
      return false;
  }
  if (term > 100 &&
      !push(l, c, 1, 1, {1}, depthwise ? "depthwise top int8 scale" : "conv top int8 scale", err))
    return false;
  (void)tag;
  return true;
}

bool load_inner_product(LayerDef& l, BinCursor& c, std::string* err) {
  int64_t nout, bias, wsize, term;
  if (!int_param(l.params, 0, 0, "num_output", &nout, err) ||
      !int_param(l.params, 1, 0, "bias_term", &bias, err) ||
      !int_param(l.params, 2, 0, "weight_data_size", &wsize, err) ||
      !int_param(l.params, 8, 0, "int8_scale_term", &term, err)) {
    *err = "invalid inner product parameter type";
    return false;
  }
  if (nout <= 0) {
    *err = "inner product num_output must be positive";
    return false;
  }
  if (wsize <= 0 || wsize % nout != 0) {
    *err = "inner product weight count must be positive and divisible by num_output";
    return false;
  }
  if (bias != 0 && bias != 1) {
    *err = "inner product bias_term must be 0 or 1";
    return false;
  }
  if (term != 0 && term != 1 && term != 2) {
    *err = "inner product int8_scale_term must be 0, 1, or 2";
    return false;
  }
  if (!push(l, c, wsize, 0, {nout, wsize / nout}, "inner product weight", err)) return false;
  if (bias == 1 && !push(l, c, nout, 1, {nout}, "inner product bias", err)) return false;
  if (term != 0) {
    if (!push(l, c, nout, 1, {nout}, "inner product weight int8 scales", err)) return false;
    if (!push(l, c, 1, 1, {1}, "inner product bottom int8 scale", err)) return false;
  }
  return true;
}

bool load_gemm(LayerDef& l, BinCursor& c, std::string* err) {
  int64_t v[19];
  static const int ids[] = {2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 18};
  static const char* names[] = {"transA", "transB", "constantA", "constantB", "constantC",
                                "constantM", "constantN", "constantK", "broadcast_type_C",
                                "output_N1M", "output_elempack", "output_elemtype",
                                "output_transpose", "int8_scale_term"};
  for (size_t i = 0; i < sizeof(ids) / sizeof(ids[0]); ++i) {
    if (!int_param(l.params, ids[i], 0, names[i], &v[ids[i]], err)) {
      *err = "invalid Gemm parameter type";
      return false;
    }
  }
  for (int id : {0, 1}) {
    const ParamValue* pv = l.params.find(id);
    if (pv != nullptr && pv->kind != ParamValue::kFloat) {
      *err = "invalid Gemm parameter type";
      return false;
    }
  }
  const bool ta = v[2], tb = v[3], ca = v[4], cb = v[5], cc = v[6];
  const int64_t n = v[8], k = v[9], bc = v[10], term = v[18];
  for (int id : {2, 3, 4, 5, 6}) {
    if (v[id] != 0 && v[id] != 1) {
      *err = "Gemm boolean parameter must be 0 or 1";
      return false;
    }
  }
  if (cb && (n <= 0 || k <= 0)) {
    *err = "Gemm constantN and constantK must be positive for constant B";
    return false;
  }
  if (cc && (bc < -1 || bc > 4)) {
    *err = "Gemm C broadcast type must be -1 through 4";
    return false;
  }
  const bool dynamic = !ca && !cb && !cc;
  if (dynamic && !ta && !tb && v[11] == 0 && v[12] == 0 && v[13] == 0 && v[14] == 0 && term == 0)
    return true;
  if (ca || !cb || !cc || ta || !tb || (bc != -1 && bc != 4) || v[11] != 0 || v[12] != 0 ||
      v[13] != 0 || v[14] != 0 || (term != 0 && term != 1 && term != 2)) {
    *err =
        "only dynamic-A, transposed constant-B Gemm with optional row bias and optional int8 B "
        "is supported";
    return false;
  }
  if (!push(l, c, n * k, 0, {n, k}, "Gemm B", err)) return false;
  if (bc == 4) {
    if (!push(l, c, n, 0, {n}, "Gemm C", err)) return false;
    WeightTensor& bias = l.weights.back();
    if (bias.type == WeightType::kF16) {  // promoted like the reference does (graph.cpp:1907-1911)
      std::vector<float> f = bias.as_f32();
      bias.type = WeightType::kF32;
      bias.bytes.resize(f.size() * 4);
      std::memcpy(bias.bytes.data(), f.data(), bias.bytes.size());
    }
  }
  if (term != 0 && !push(l, c, 1, 1, {1}, "Gemm B int8 scale", err)) return false;
  return true;
}

bool load_counts(LayerDef& l, BinCursor& c, std::initializer_list<std::pair<int, int64_t>> id_dflt,
                 const char* const* names, bool last_optional, std::string* err) {
  size_t i = 0;
  for (auto [id, dflt] : id_dflt) {
    int64_t n;
    if (!int_param(l.params, id, dflt, names[i], &n, err)) return false;
    const bool optional = last_optional && i + 1 == id_dflt.size();
    if (n < 0 || (n == 0 && !optional)) {
      *err = std::string(l.type) + " " + names[i] + " count must be positive";
      return false;
    }
    if (n > 0 && !push(l, c, n, 1, {n}, (l.type + " " + names[i]).c_str(), err)) return false;
    ++i;
  }
  return true;
}

bool load_layer_weights(LayerDef& l, BinCursor& c, std::string* err) {
  const std::string& t = l.type;
  if (t == "Convolution") return load_conv_like(l, c, false, err);
  if (t == "ConvolutionDepthWise") return load_conv_like(l, c, true, err);
  if (t == "InnerProduct") return load_inner_product(l, c, err);
  if (t == "Gemm") return load_gemm(l, c, err);
  if (t == "BatchNorm") {
    int64_t ch;
    if (!int_param(l.params, 0, 0, "channels", &ch, err)) return false;
    if (ch <= 0) {
      *err = "BatchNorm channels must be positive";
      return false;
    }
    for (const char* name : {"BatchNorm slope", "BatchNorm mean", "BatchNorm variance",
                             "BatchNorm bias"})
      if (!push(l, c, ch, 1, {ch}, name, err)) return false;
    return true;
  }
  if (t == "Quantize") {
    static const char* n[] = {"scale"};
    return load_counts(l, c, {{0, 1}}, n, false, err);
  }
  if (t == "Dequantize") {
    static const char* n[] = {"scale", "bias"};
    return load_counts(l, c, {{0, 1}, {1, 0}}, n, true, err);
  }
  if (t == "Requantize") {
    static const char* n[] = {"input scale", "output scale", "bias"};
    return load_counts(l, c, {{0, 1}, {1, 1}, {2, 0}}, n, true, err);
  }
  if (t == "Deconvolution") {  // load_deconvolution_weights, graph.cpp:1573-1636
    int64_t dyn, nout, kw, kh, bias, wsize;
    if (!int_param(l.params, 28, 0, "dynamic_weight", &dyn, err)) return false;
    if (dyn != 0 && dyn != 1) {
      *err = "deconvolution dynamic_weight must be 0 or 1";
      return false;
    }
    if (dyn == 1) return true;
    if (!int_param(l.params, 0, 0, "num_output", &nout, err) || !int_param(l.params, 1, 0, "kernel_w", &kw, err) ||
        !int_param(l.params, 11, kw, "kernel_h", &kh, err) || !int_param(l.params, 5, 0, "bias_term", &bias, err) ||
        !int_param(l.params, 6, 0, "weight_data_size", &wsize, err))
      return false;
    if (nout <= 0 || kw <= 0 || kh <= 0 || wsize <= 0) {
      *err = "deconvolution channels, kernel, stride, dilation, and weight count must be positive";
      return false;
    }
    if (bias != 0 && bias != 1) {
      *err = "deconvolution bias_term must be 0 or 1";
      return false;
    }
    const int64_t per_input = nout * kh * kw;
    if (wsize % per_input != 0) {
      *err = "deconvolution weight count is not divisible by output/kernel size";
      return false;
    }
    if (!push(l, c, wsize, 0, {nout, wsize / per_input, kh, kw}, "deconvolution weight", err)) return false;
    return bias == 0 || push(l, c, nout, 1, {nout}, "deconvolution bias", err);
  }
  if (t == "PReLU") {  // load_prelu_weights, graph.cpp:1697-1709
    int64_t count;
    if (!int_param(l.params, 0, 0, "num_slope", &count, err)) return false;
    if (count <= 0) {
      *err = "PReLU num_slope must be positive";
      return false;
    }
    return push(l, c, count, 1, {count}, "PReLU slope", err);
  }
  // Layer types that carry weights in ncnn but lie outside this runtime's path:
  // their payload cannot be skipped reliably, so the file is rejected.
  for (const char* w : {"MemoryData", "LayerNorm", "Embed",
                        "MultiHeadAttention", "Scale", "DeconvolutionDepthWise", "InstanceNorm",
                        "GroupNorm", "RNN", "LSTM", "GRU"}) {
    if (t == w) {
      *err = "layer type " + t + " carries weights and is not supported by this runtime";
      return false;
    }
  }
  return true;
}

}  // namespace

bool load_model(const std::string& param_path, const std::string& bin_path, ModelDef* model,
                std::string* error) {
  std::ifstream file(param_path);
  if (!file) {
    *error = "cannot open param file: " + param_path;
    return false;
  }
  std::vector<std::string> lines;
  std::string line;
  while (std::getline(file, line)) {
    const size_t first = line.find_first_not_of(" \t\r\n");
    const size_t last = line.find_last_not_of(" \t\r\n");
    if (first != std::string::npos) lines.push_back(line.substr(first, last - first + 1));
  }
  if (lines.empty()) {
    *error = "empty param file";
    return false;
  }
  size_t idx = 0;
  const auto first_line = split_ws(lines[0]);
  if (first_line.size() == 1) {
    int64_t magic;
    if (!parse_i64(first_line[0], "param magic", &magic, error)) return false;
    if (magic != 7767517) {
      *error = "param magic mismatch (expected 7767517)";
      return false;
    }
    idx = 1;
  } else if (first_line.size() != 2) {
    *error = "bad param magic/header line";
    return false;
  }
  if (idx >= lines.size()) {
    *error = "missing layer/blob count header";
    return false;
  }
  const auto header = split_ws(lines[idx]);
  if (header.size() != 2) {
    *error = "bad layer/blob count header";
    return false;
  }
  int64_t layer_count, blob_count;
  if (!parse_i64(header[0], "layer count", &layer_count, error)) return false;
  if (!parse_i64(header[1], "blob count", &blob_count, error)) return false;
  if (layer_count < 0) {
    *error = "layer count must be non-negative";
    return false;
  }
  if (blob_count < 0) {
    *error = "blob count must be non-negative";
    return false;
  }
  if (layer_count > 0x7fffffff || blob_count > 0x7fffffff) {
    *error = "layer count does not fit int";
    return false;
  }
  ++idx;
  if (static_cast<size_t>(layer_count) > lines.size() - idx) {
    *error = "param truncated before all layers read";
    return false;
  }

  std::vector<uint8_t> bin;
  const bool have_bin = !bin_path.empty();
  if (have_bin) {
    std::ifstream bf(bin_path, std::ios::binary);
    if (!bf) {
      *error = "cannot open bin file: " + bin_path;
      return false;
    }
    bin.assign(std::istreambuf_iterator<char>(bf), std::istreambuf_iterator<char>());
  }

  ModelDef m;
  std::vector<int> producer, consumer;  // per blob
  auto find_blob = [&](const std::string& name) -> int {
    for (size_t i = 0; i < m.blobs.size(); ++i)
      if (m.blobs[i] == name) return static_cast<int>(i);
    return -1;
  };
  for (int64_t li = 0; li < layer_count; ++li) {
    const auto tok = split_ws(lines[idx++]);
    if (tok.size() < 4) {
      *error = "layer line too short";
      return false;
    }
    LayerDef layer;
    layer.type = tok[0];
    layer.name = tok[1];
    int64_t nb, nt;
    if (!parse_i64(tok[2], "bottom count", &nb, error)) return false;
    if (!parse_i64(tok[3], "top count", &nt, error)) return false;
    if (nb < 0) {
      *error = "bottom count must be non-negative";
      return false;
    }
    if (nt < 0) {
      *error = "top count must be non-negative";
      return false;
    }
    size_t off = 4;
    if (static_cast<size_t>(nb) > tok.size() - off) {
      *error = "layer line missing bottom blob names";
      return false;
    }
    for (int64_t i = 0; i < nb; ++i) layer.bottoms.push_back(tok[off++]);
    if (static_cast<size_t>(nt) > tok.size() - off) {
      *error = "layer line missing top blob names";
      return false;
    }
    for (int64_t i = 0; i < nt; ++i) layer.tops.push_back(tok[off++]);
    std::string tail;
    for (size_t i = off; i < tok.size(); ++i) {
      if (i > off) tail += ' ';
      tail += tok[i];
    }
    if (!tail.empty()) {
      std::string perr;
      if (!parse_layer_params(tail, &layer.params, &perr)) {
        *error = "layer " + std::to_string(li) + " (" + layer.type + "): " + perr;
        return false;
      }
    }
    for (const auto& name : layer.bottoms) {
      const int b = find_blob(name);
      if (b < 0 || producer[b] == -1) {
        *error = "layer " + std::to_string(li) + " has unresolved bottom blob: " + name;
        return false;
      }
      if (consumer[b] == -1) consumer[b] = static_cast<int>(li);
    }
    for (const auto& name : layer.tops) {
      int b = find_blob(name);
      if (b < 0) {
        if (m.blobs.size() >= static_cast<size_t>(blob_count)) {
          *error = "model creates more blobs than declared";
          return false;
        }
        b = static_cast<int>(m.blobs.size());
        m.blobs.push_back(name);
        producer.push_back(-1);
        consumer.push_back(-1);
      }
      if (producer[b] != -1) {
        *error = "blob has multiple producers: " + name;
        return false;
      }
      producer[b] = static_cast<int>(li);
    }
    m.layers.push_back(std::move(layer));
  }
  if (idx != lines.size()) {
    *error = "param contains trailing layer lines";
    return false;
  }
  if (have_bin) {
    BinCursor cursor(bin);
    for (size_t li = 0; li < m.layers.size(); ++li) {
      std::string werr;
      if (!load_layer_weights(m.layers[li], cursor, &werr)) {
        *error = "layer " + std::to_string(li) + " (" + m.layers[li].type + ", " +
                 m.layers[li].name + "): " + werr;
        return false;
      }
    }
    if (cursor.remaining() != 0) {
      *error = "bin size mismatch: consumed " + std::to_string(cursor.pos()) + " bytes of " +
               std::to_string(cursor.size()) + " (difference " +
               std::to_string(cursor.remaining()) + ")";
      return false;
    }
    m.weights_loaded = true;
  }
  for (const auto& l : m.layers)
    if (l.type == "Input")
      for (const auto& t : l.tops) m.inputs.push_back(t);
  for (size_t b = 0; b < m.blobs.size(); ++b)
    if (consumer[b] == -1) m.outputs.push_back(m.blobs[b]);
  *model = std::move(m);
  return true;
}

std::string describe_model(const ModelDef& m) {
  std::ostringstream o;
  o << "ncnn_graph: " << m.layers.size() << " layers, " << m.blobs.size() << " blobs\n";
  o << "inputs: " << m.inputs.size() << "\n";
  for (const auto& n : m.inputs) o << "  - " << n << "\n";
  o << "outputs: " << m.outputs.size() << "\n";
  for (const auto& n : m.outputs) o << "  - " << n << "\n";
  o << "layers:\n";
  for (size_t i = 0; i < m.layers.size(); ++i) {
    const LayerDef& l = m.layers[i];
    char head[160];
    std::snprintf(head, sizeof(head), "  [%3zu] %-14s %-22s in=[", i, l.type.c_str(),
                  l.name.c_str());
    o << head;
    for (size_t k = 0; k < l.bottoms.size(); ++k) o << (k ? "," : "") << l.bottoms[k];
    o << "] out=[";
    for (size_t k = 0; k < l.tops.size(); ++k) o << (k ? "," : "") << l.tops[k];
    o << "]";
    if (!l.params.entries().empty()) {
      o << " {";
      bool first = true;
      for (const auto& [id, v] : l.params.entries()) {
        if (!first) o << " ";
        first = false;
        o << id << "=";
        switch (v.kind) {
          case ParamValue::kInt: o << v.i; break;
          case ParamValue::kFloat: o << v.f; break;
          case ParamValue::kString: o << "\"" << v.s << "\""; break;
          case ParamValue::kIntArray:
            o << "[";
            for (size_t k = 0; k < v.ia.size(); ++k) o << (k ? "," : "") << v.ia[k];
            o << "]";
            break;
          case ParamValue::kFloatArray:
            o << "[";
            for (size_t k = 0; k < v.fa.size(); ++k) o << (k ? "," : "") << v.fa[k];
            o << "]";
            break;
        }
      }
      o << "}";
    }
    if (!l.weights.empty()) {
      o << " w=[";
      for (size_t k = 0; k < l.weights.size(); ++k) {
        const WeightTensor& w = l.weights[k];
        o << (k ? "," : "") << "[";
        for (size_t d = 0; d < w.shape.size(); ++d) o << (d ? "," : "") << w.shape[d];
        o << ":" << (w.type == WeightType::kF32 ? "f32" : (w.type == WeightType::kF16 ? "f16" : "i8"))
          << ":" << w.bytes.size() << "B]";
      }
      o << "]";
    }
    o << "\n";
  }
  o << "weights:\n";
  for (size_t i = 0; i < m.layers.size(); ++i) {
    for (size_t k = 0; k < m.layers[i].weights.size(); ++k) {
      uint64_t h = 1469598103934665603ull;
      for (uint8_t b : m.layers[i].weights[k].bytes) {
        h ^= b;
        h *= 1099511628211ull;
      }
      char buf[64];
      std::snprintf(buf, sizeof(buf), "  [%3zu].%zu %016llx\n", i, k,
                    static_cast<unsigned long long>(h));
      o << buf;
    }
  }
  return o.str();
}

}  // namespace nb
