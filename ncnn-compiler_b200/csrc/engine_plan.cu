// Graph passes of the executor (BatchNorm folding, activation / residual / quantize / depthwise fusion), the choice of
// implementation per node, weight packing and upload, and the memory plan of the activation arena.
#include "engine_impl.h"

namespace nb {


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
  // Two Quantize steps that are left reading the same fp32 tensor (a block input that feeds the first convolution
  // and the downsample convolution, each with its own scale) become one pass with two int8 results.
  for (size_t a = 0; a < nodes_.size(); ++a) {
    Node& q1 = nodes_[a];
    if (q1.kind != N_UNARY || q1.un.op != UN_QUANT || q1.un.nscale != 1 || q1.un_scale.size() != 1 || !q1.side_q.empty()) continue;
    const int src = resolve(q1.in[0]);
    // (only where the 16-wide kernel runs at every batch size: it is the one with the second result)
    if (tensors_[src].fmt != FMT_F32 || tensors_[src].logical() % 16 != 0) continue;
    for (size_t b = a + 1; b < nodes_.size(); ++b) {
      const Node& q2 = nodes_[b];
      if (q2.kind != N_UNARY || q2.un.op != UN_QUANT || q2.un.nscale != 1 || q2.un_scale.size() != 1 || !q2.side_q.empty() ||
          resolve(q2.in[0]) != src)
        continue;
      q1.side_q.emplace_back(q2.out, q2.un_scale[0]);
      nodes_.erase(nodes_.begin() + b);
      break;
    }
  }
}

// A stride-1 3x3 depthwise layer whose only consumer is a 1x1 tensor-core convolution (the second half of
// an inverted-residual block) runs inside that convolution's kernel: its result goes from the CUDA cores
// into the shared-memory operand tile of the MMAs and never to HBM.  The values, their bf16 split and the
// order of the products are those of the two separate layers.  NCNN_B200_FUSE_DW=0 keeps them apart.
// Where the depthwise input itself comes from a 1x1 convolution with at most 32 input channels and no other
// consumer (the "expand" layer of the block; its bf16 weights are already packed as 64-byte rows of 32 input
// channels, which is what the fused kernel multiplies a patch by), that layer joins too, for depthwise strides
// 1 and 2: the whole block is one kernel and the expanded tensor never exists in HBM.  NCNN_B200_FUSE_EXPAND=0
// leaves the expand layers alone.
void EngineImpl::fuse_depthwise_projection() {
  const char* env = std::getenv("NCNN_B200_FUSE_DW");
  const bool enabled = !(env != nullptr && env[0] == '0') && opt_.accuracy_mode == kAccuracyFp32Split;
  std::vector<int> uses(tensors_.size(), 0);
  for (const Node& n : nodes_) {
    for (int t : n.in) ++uses[resolve(t)];
    if (n.res >= 0) ++uses[resolve(n.res)];
  }
  for (int o : outputs_) ++uses[resolve(o)];
  for (size_t k = 0; enabled && k + 1 < nodes_.size(); ++k) {
    const Node& dw = nodes_[k];
    if (dw.kind != N_DW || dw.term != 0 || dw.KH != 3 || dw.KW != 3 || dw.sh != dw.sw || dw.dh != 1 ||
        dw.dw != 1 || dw.res >= 0 || !dw.side_q.empty() || dw.d_w0 == nullptr)
      continue;
    const int mid = resolve(dw.out);
    const int src = resolve(dw.in[0]);
    const Tensor& tin = tensors_[src];
    const Tensor& tmid = tensors_[mid];
    // the producer of the depthwise input, when it qualifies as the block's expand layer
    int je = -1;
    for (size_t j = 0; j < k && !env_flag_off("NCNN_B200_FUSE_EXPAND"); ++j) {
      const Node& ex = nodes_[j];
      if (resolve(ex.out) != src) continue;
      const bool clamp = ex.act == ACT_NONE || ex.act == ACT_RELU || ex.act == ACT_CLIP;
      if (ex.kind == N_CONV && ex.impl == IMPL_TC && ex.term == 0 && !ex.stem && ex.out_ld == 0 && ex.KH == 1 && ex.KW == 1 &&
          ex.sh == 1 && ex.sw == 1 && ex.pt == 0 && ex.pl == 0 && ex.res < 0 && ex.side_q.empty() && clamp && uses[src] == 1 &&
          ex.k_elems == 32 && ex.d_w0 != nullptr && ex.d_w1 != nullptr)
        je = static_cast<int>(j);
    }
    // Measured on MobileNetV2 at batch 256: with the expand layer inside, stride-2 blocks are 10-16 % faster than
    // their three layers (the expanded tensor is four times the block's output), stride-1 blocks 35 % slower than
    // expand + fused pair (per block of 32 channels the kernel then runs 12 more MMAs and a TMEM read-back on top of
    // the depthwise arithmetic).  So stride-1 blocks join only with NCNN_B200_FUSE_EXPAND=2.
    if (je >= 0 && dw.sh == 1 && env_int_or("NCNN_B200_FUSE_EXPAND", 1) < 2) je = -1;
    if (je < 0 && dw.sh != 1) continue;
    if (dw.sh != 1 && dw.sh != 2) continue;
    if (uses[mid] != 1 || tin.rank != 3 || tin.fmt != FMT_F32 || tin.Cp != tin.c || tin.Wp != tin.w || tin.w_off != 0 ||
        tmid.fmt != FMT_BF16X2 || dw.pt > 2 || dw.pl > 2)
      continue;
    if (dw.sh == 1 && (dw.OH != tin.h || dw.OW != tin.w)) continue;
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
    if (je >= 0) {
      const Node& ex = nodes_[je];
      const Tensor& tx = tensors_[resolve(ex.in[0])];
      if (tx.rank != 3 || tx.fmt != FMT_BF16X2 || tx.Cp != tx.c || tx.Wp != tx.w || tx.w_off != 0 ||
          !tc_block_applies(tx.c, ex.O, pw.O, dw.OH, dw.OW, dw.sh, has_res))
        je = -1;  // (the depthwise layer and the projection may still pair up)
    }
    if (je < 0 && (dw.sh != 1 || !tc_dw_project_applies(tin.c, pw.O, tin.h, tin.w, out_mode, has_res, res_bf16))) continue;
    pw.dw_fused = true;
    pw.dw_w = static_cast<const float*>(dw.d_w0);
    pw.dw_bias = dw.d_bias;
    pw.dw_act = dw.act;
    pw.dw_act_a = dw.act_a;
    pw.dw_act_b = dw.act_b;
    pw.dw_pt = dw.pt;
    pw.dw_pl = dw.pl;
    pw.dw_stride = dw.sh;
    pw.dw_c = tin.c;
    pw.dw_hin = tin.h;
    pw.dw_win = tin.w;
    pw.dw_name = dw.name;
    pw.in[0] = dw.in[0];
    pw.flops += dw.flops;
    if (je >= 0) {
      Node& ex = nodes_[je];
      pw.ex_fused = true;
      pw.ex_w0 = ex.d_w0;
      pw.ex_w1 = ex.d_w1;
      pw.ex_bias = ex.d_bias;
      pw.ex_act = ex.act;
      pw.ex_act_a = ex.act_a;
      pw.ex_act_b = ex.act_b;
      pw.ex_cin = tensors_[resolve(ex.in[0])].c;
      pw.ex_name = ex.name;
      pw.in[0] = ex.in[0];
      pw.flops += ex.flops;
    }
    nodes_.erase(nodes_.begin() + k);
    if (je >= 0) nodes_.erase(nodes_.begin() + je);  // (je < k: the index is still valid)
    k -= je >= 0 ? 2 : 1;
  }
}

// The 3x3 stride-2 max pooling behind a stem that runs on the row-resident kernel moves into that kernel: the
// stem's result (the largest tensor of the network) is pooled out of shared memory and never written to HBM.
// Same values, same maxima, same bf16 split as the two launches.  NCNN_B200_STEM_POOL=0 keeps them apart.
void EngineImpl::fuse_stem_pooling() {
  if (env_flag_off("NCNN_B200_STEM_POOL")) return;
  std::vector<int> uses(tensors_.size(), 0);
  for (const Node& n : nodes_) {
    for (int t : n.in) ++uses[resolve(t)];
    if (n.res >= 0) ++uses[resolve(n.res)];
  }
  for (int o : outputs_) ++uses[resolve(o)];
  for (size_t k = 0; k + 1 < nodes_.size(); ++k) {
    Node& st = nodes_[k];
    if (st.kind != N_CONV || !st.stem || !st.stem_rows || st.impl != IMPL_TC || st.res >= 0 || st.out_ld != 0 || !st.side_q.empty() ||
        (st.O != 32 && st.O != 64) || st.OW > 128 || st.OH % 2 != 0 || st.OW % 2 != 0)
      continue;
    if (st.act != ACT_NONE && st.act != ACT_RELU && st.act != ACT_CLIP) continue;  // the kernel clamps, nothing else
    // bf16 pairs in, bf16 pairs out (fp32 accuracy mode); or int8 in, fp32 out with at most one int8 copy of 64 channels
    const bool i8 = st.term != 0;
    const int mid = resolve(st.out);
    const int want_in = i8 ? FMT_I8 : FMT_BF16X2, want_out = i8 ? FMT_F32 : FMT_BF16X2;
    if (!i8 && opt_.accuracy_mode != kAccuracyFp32Split) continue;
    if (uses[mid] != 1 || tensors_[mid].fmt != FMT_F32 || tensors_[resolve(st.in[0])].fmt != want_in) continue;
    const Node& pl = nodes_[k + 1];
    if (pl.kind != N_POOL || resolve(pl.in[0]) != mid) continue;
    if (!pl.side_q.empty() && (!i8 || pl.side_q.size() > 1 || st.O != 64)) continue;
    const PoolParams& pp = pl.pool;
    if (pp.kind != 0 || pp.adaptive || pp.KH != 3 || pp.KW != 3 || pp.sh != 2 || pp.sw != 2 || pp.pt != 1 || pp.pl != 1 ||
        pp.OH * 2 != st.OH || pp.OW * 2 != st.OW || tensors_[resolve(pl.out)].fmt != want_out)
      continue;
    st.pool_fused = true;
    st.pool_oh = pp.OH;
    st.pool_ow = pp.OW;
    st.pool_name = pl.name;
    st.out = pl.out;
    st.side_q = pl.side_q;
    st.flops += pl.flops;
    nodes_.erase(nodes_.begin() + k + 1);
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

}  // namespace nb
