// ncnn layers -> nodes of the executor: one importer per layer type, with the checks of the reference's importers.
#include "engine_impl.h"

namespace nb {

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
    // rank-4 tensors [c,d,h,w] exist between data-movement layers only (Reshape, Permute order 3, Slice, Concat,
    // Flatten, Split and the elementwise activations): a detection head reshapes into them and back
    static const char* const rank4_layers[] = {"Reshape", "Flatten", "Permute", "Slice", "Concat", "Split", "Sigmoid", "ReLU",
                                               "Clip", "TanH", "Swish", "HardSigmoid", "HardSwish", "Dropout"};
    for (const auto& b : l.bottoms)
      if (tensors_[resolve(by_name_.at(b))].rank == 4 &&
          std::find_if(std::begin(rank4_layers), std::end(rank4_layers), [&](const char* name) { return t == name; }) ==
              std::end(rank4_layers))
        return fail(err, where + "rank-4 input is outside the supported path");
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
        if (x.rank == 4) d = {x.c, x.d, x.h, x.w};
        else if (x.rank == 3) d = {x.c, x.h, x.w};
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
      if (t0.rank == 4) { to.c = od[0]; to.d = od[1]; to.h = od[2]; to.w = od[3]; }
      else if (t0.rank == 3) { to.c = od[0]; to.h = od[1]; to.w = od[2]; }
      else if (t0.rank == 2) { to.h = od[0]; to.w = od[1]; }
      else to.w = od[0];
      // storage order: rank 3 [h][w][c] -> concatenation axis as (outer, len, inner)
      int offset = 0;
      for (int id : n.in) {
        const Tensor& tb = tensors_[resolve(id)];
        ConcatParams cp{};
        cp.in_image_elems = tb.logical();
        cp.out_image_elems = to.logical();
        if (t0.rank == 4) {
          // stored in logical order: what lies before the axis is the outer extent, what lies behind it the inner
          const std::vector<int> d = dims_of(tb);
          cp.outer = 1;
          cp.inner = 1;
          for (int k = 0; k < axis; ++k) cp.outer *= d[k];
          for (int k = static_cast<int>(axis) + 1; k < 4; ++k) cp.inner *= d[k];
          cp.len_in = d[axis];
          cp.len_out = od[axis];
        } else if (t0.rank == 3) {
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
      if (ti.rank == 4) dims = {ti.c, ti.d, ti.h, ti.w};
      else if (ti.rank == 3) dims = {ti.c, ti.h, ti.w};
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
        if (ti.rank == 4) { to.c = od[0]; to.d = od[1]; to.h = od[2]; to.w = od[3]; to.Wp = to.w; }
        else if (ti.rank == 3) { to.c = od[0]; to.h = od[1]; to.w = od[2]; to.Cp = to.c; to.Wp = to.w; }
        else if (ti.rank == 2) { to.h = od[0]; to.w = od[1]; to.Wp = to.w; }
        else { to.w = od[0]; to.Wp = to.w; }
        ConcatParams cp{};
        cp.slice = 1;
        cp.in_image_elems = to.logical();
        cp.out_image_elems = ti.logical();
        if (ti.rank == 4) {
          cp.outer = 1;
          cp.inner = 1;
          for (int k = 0; k < axis; ++k) cp.outer *= dims[k];
          for (int k = static_cast<int>(axis) + 1; k < 4; ++k) cp.inner *= dims[k];
          cp.len_in = od[axis];
          cp.len_out = dims[axis];
        } else if (ti.rank == 3) {
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
        // import_reshape (ImportOps.cpp:166-300): 0=w 1=h 11=d 2=c; the result's dims are the given ones in the
        // order [c,d,h,w] (-233 marks an absent one), 0 copies an input extent (w: last, h: last but one, d:
        // second of a rank-4 input, c: first of a rank >= 3 input), a single -1 is inferred
        const int64_t raw[4] = {l.params.get_int(2, -233), l.params.get_int(11, -233), l.params.get_int(1, -233),
                                l.params.get_int(0, -233)};
        std::vector<int64_t> dims;
        int infer = -1;
        for (int i = 0; i < 4; ++i) {
          int64_t v = raw[i];
          if (v == -233) continue;
          if (v == 0) {
            if (i == 3) v = ti.w;
            else if (i == 2) {
              if (ti.rank < 2) return fail(err, where + "reshape cannot copy missing height dimension");
              v = ti.h;
            } else if (i == 1) {
              if (ti.rank != 4) return fail(err, where + "reshape cannot copy missing depth dimension");
              v = ti.d;
            } else {
              if (ti.rank < 3) return fail(err, where + "reshape cannot copy missing channel dimension");
              v = ti.c;
            }
          }
          if (v == -1) {
            if (infer >= 0) return fail(err, where + "reshape allows at most one -1 dimension");
            infer = static_cast<int>(dims.size());
          } else if (v <= 0) {
            return fail(err, where + "reshape dimensions must be positive, 0, -1 or -233");
          }
          dims.push_back(v);
        }
        if (dims.empty()) return fail(err, where + "reshape needs at least one dimension");
        long long known = 1;
        for (size_t i = 0; i < dims.size(); ++i)
          if (static_cast<int>(i) != infer) known *= dims[i];
        if (infer >= 0) dims[infer] = ti.logical() / std::max<long long>(known, 1);
        long long total = 1;
        for (int64_t v : dims) total *= v;
        if (total != ti.logical()) return fail(err, where + "Reshape does not preserve the element count");
        const int rank = static_cast<int>(dims.size());
        to.rank = rank;
        to.w = static_cast<int>(dims[rank - 1]);
        to.h = rank >= 2 ? static_cast<int>(dims[rank - 2]) : 1;
        to.d = rank == 4 ? static_cast<int>(dims[1]) : 1;
        to.c = rank >= 3 ? static_cast<int>(dims[0]) : 1;
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
        } else if (ti.rank == 4 && order == 3) {
          // ncnn order_type 3 of a rank-4 tensor: result [c,h,w,d] (permutation {0,2,3,1} of [c,d,h,w])
          to.rank = 4;
          to.c = ti.c;
          to.d = ti.h;
          to.h = ti.w;
          to.w = ti.d;
          n.relayout.permute4d = 1;
          n.relayout.s4d = ti.d;
          n.relayout.s4h = ti.h;
          n.relayout.s4w = ti.w;
        } else {
          return fail(err, where + "Permute supports rank-2 order 0/1, rank-3 order 2/4, and rank-4 order 3 only");
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

}  // namespace nb
