// Nodes -> kernel launches: every node of a plan becomes one Step (a closure that enqueues its kernel), and the
// edges between the caller's CHW arrays and the channel-last arena.
#include "engine_impl.h"

namespace nb {

static cudaError_t launch_ok() { return cudaGetLastError(); }


bool EngineImpl::emit_node(Plan& plan, const Node& node, int64_t n, std::string* err) {
  const Tensor& to = tensors_[resolve(node.out)];
  const ActRef out = ref(node.out, n);
  Step s;
  s.name = node.name;
  s.flops = node.flops * n;
  const int f32_kind = opt_.accuracy_mode == kAccuracyTf32 ? GEMM_TF32 : GEMM_TF32X3;
  auto bytes_of = [&](int t) {
    const Tensor& x = tensors_[resolve(t)];
    return static_cast<double>(x.logical()) * (x.i8 ? 1 : 4) * n;
  };
  s.bytes = bytes_of(node.out);
  for (int t : node.in) s.bytes += bytes_of(t);
  if (node.res >= 0) s.bytes += bytes_of(node.res);

  if (node.kind == N_CONV || node.kind == N_IP || node.kind == N_GEMM || node.kind == N_DW) {
    const Tensor& ti = tensors_[resolve(node.in[0])];
    const ActRef in = ref(node.in[0], n);
    const bool i8 = node.term != 0;
    ConvEpilogue e{};
    e.bias = node.d_bias;
    e.scale = node.d_deq;
    e.out_scale = node.s_out;
    e.act = node.act;
    e.act_a = node.act_a;
    e.act_b = node.act_b;
    e.has_res = node.res >= 0;
    if (e.has_res) e.res = ref(node.res, n);
    if (node.kind == N_GEMM && i8) {
      const int K = node.K, N = node.O;
      const long long M = static_cast<long long>(ti.h) * n;
      const int8_t* wq = static_cast<const int8_t*>(node.d_w0);
      const float s_b = node.s_b, alpha = node.alpha, beta = 1.0f;
      const float* c_bias = node.d_bias;
      const int has_c = node.has_bias, scale_alpha = node.alpha != 1.0f;
      s.kernel = "k_gemm_i8_rowscale";
      s.run = [=](cudaStream_t st) {
        k_gemm_i8_rowscale<<<static_cast<unsigned>(M), 128, K, st>>>(in, out, wq, K, N, s_b, c_bias, alpha, beta, has_c, scale_alpha);
        return launch_ok();
      };
      plan.steps.push_back(std::move(s));
      return true;
    }
    if (node.impl == IMPL_TC) {
      TcEpilogue te;
      te.bias = node.d_bias;
      te.scale = node.d_deq;
      te.out0 = out.p0;
      te.out1 = out.p1;
      te.outq = out.q;
      te.ldo = node.O;
      if (node.out_ld > 0) {
        // a view into a Concat result: longer rows, starting `out_ch_off` channels in
        te.ldo = node.out_ld;
        const size_t skip = static_cast<size_t>(node.out_ch_off) * to.elem_bytes();
        te.out0 = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(out.p0) + skip);
        if (out.p1 != nullptr) te.out1 = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(out.p1) + skip);
      }
      te.act = node.act;
      te.act_a = node.act_a;
      te.act_b = node.act_b;
      // Gemm: (A*B^T + beta*C) * alpha; beta is in the bias already, alpha multiplies in the epilogue
      const bool alpha_fused = node.kind == N_GEMM && node.alpha != 1.0f && node.act == ACT_NONE;
      if (alpha_fused) {
        te.act = ACT_SCALE;
        te.act_a = node.alpha;
      }
      te.out_scale = node.s_out;
      te.status = d_status_;
      te.side_count = static_cast<int>(node.side_q.size());
      for (int i = 0; i < te.side_count; ++i) {
        te.side_q[i] = ref(node.side_q[i].first, n).q;
        te.side_scale[i] = node.side_q[i].second;
      }
      te.sk_ws = d_split_ws_;
      te.sk_ws_bytes = kTcSplitWorkspaceBytes;
      te.sk_flags = d_split_flags_;
      te.sk_flag_count = kTcSplitFlagCount;
      te.out_mode = to.fmt == FMT_I8 ? OUT_I8 : (to.fmt == FMT_SPLIT ? OUT_F32_SPLIT : (to.fmt == FMT_TF32 ? OUT_F32_TF32 : (to.fmt == FMT_BF16X2 ? OUT_BF16X2 : OUT_F32)));
      if (node.res >= 0) {
        const ActRef r = ref(node.res, n);
        te.res0 = r.p0;
        te.res1 = r.p1;
        te.res_bf16 = r.fmt == FMT_BF16X2;
      }
      const int kind = i8 ? GEMM_I8 : (ti.fmt == FMT_BF16X2 ? GEMM_BF16X3 : f32_kind);
      const char* kind_name = kind == GEMM_I8 ? "i8" : (kind == GEMM_TF32 ? "tf32" : (kind == GEMM_BF16X3 ? "bf16x3" : "tf32x3"));
      auto launch = std::make_shared<TcLaunch>();
      std::string perr;
      if (node.dw_fused) {
        TcDwProjConv dc;
        dc.x = in.p0;
        dc.images = static_cast<int>(n);
        dc.H = node.OH;
        dc.W = node.OW;
        dc.Hin = node.dw_hin;
        dc.Win = node.dw_win;
        dc.C = node.dw_c;
        dc.stride = node.dw_stride;
        if (node.ex_fused) {
          dc.Cin = node.ex_cin;
          dc.x1 = in.p1;
          dc.ex_w0 = node.ex_w0;
          dc.ex_w1 = node.ex_w1;
          dc.ex_bias = node.ex_bias;
          dc.ex_act = node.ex_act;
          dc.ex_act_a = node.ex_act_a;
          dc.ex_act_b = node.ex_act_b;
        }
        dc.pad_t = node.dw_pt;
        dc.pad_l = node.dw_pl;
        dc.dw_weights = node.dw_w;
        dc.dw_bias = node.dw_bias;
        dc.dw_act = node.dw_act;
        dc.dw_act_a = node.dw_act_a;
        dc.dw_act_b = node.dw_act_b;
        dc.w0 = node.d_w0;
        dc.w1 = node.d_w1;
        dc.out_channels = node.O;
        auto dl = std::make_shared<TcDwProjLaunch>();
        const std::string derr = tc_plan_dw_project(dl.get(), dc, te, sm_count_);
        if (!derr.empty()) return fail(err, "layers " + node.dw_name + " + " + node.name + ": " + derr);
        s.name = (node.ex_fused ? node.ex_name + "+" : std::string()) + node.dw_name + "+" + node.name;
        s.kernel = node.ex_fused ? (node.dw_stride == 2 ? "tc_dw_project_kernel:expand+stride2<bf16x3>" : "tc_dw_project_kernel:expand<bf16x3>")
                                 : "tc_dw_project_kernel<bf16x3>";
        s.run = [dl](cudaStream_t st) { return tc_launch_dw_project(*dl, st); };
        plan.steps.push_back(std::move(s));
        return true;
      }
      // stride-1 filters with spatial extent: the patch-resident kernel loads each input pixel
      // once per tile instead of once per tap
      if (node.kind == N_CONV && !i8 && !node.stem && node.out_ld == 0 && halo_preferred() &&
          tc_halo_applies(kind, ti.c, node.KH, node.KW, node.sh, node.sw, node.dh, node.dw, node.OH, node.OW, node.O,
                          te.out_mode)) {
        TcHaloConv hc;
        hc.in0 = in.p0;
        hc.in1 = in.p1;
        hc.images = static_cast<int>(n);
        hc.H = ti.h;
        hc.W = ti.w;
        hc.C = ti.c;
        hc.KH = node.KH;
        hc.KW = node.KW;
        hc.pad_t = node.pt;
        hc.pad_l = node.pl;
        hc.OH = node.OH;
        hc.OW = node.OW;
        hc.w0 = node.d_w0;
        hc.w1 = node.d_w1;
        hc.out_channels = node.O;
        auto hl = std::make_shared<TcHaloLaunch>();
        if (tc_plan_conv_halo(hl.get(), kind, hc, te, sm_count_, halo_level() >= 2).empty()) {
          s.kernel = std::string(hl->pair ? "tc_conv_halo_kernel:pairs<" : "tc_conv_halo_kernel<") + kind_name + ">";
          s.run = [hl](cudaStream_t st) { return tc_launch_halo(*hl, st); };
          plan.steps.push_back(std::move(s));
          return true;
        }
      }
      if (node.kind == N_CONV && node.stem && node.stem_rows && node.res < 0 && node.out_ld == 0) {
        TcStemConv sc;
        sc.kind = kind;
        sc.in0 = i8 ? static_cast<const void*>(in.q) : static_cast<const void*>(in.p0);
        sc.in1 = in.p1;
        sc.images = static_cast<int>(n);
        sc.H = ti.h;
        sc.row_bytes = ti.Wp * ti.Cp * (i8 ? 1 : 2);
        sc.KH = node.KH;
        sc.stride_h = node.sh;
        sc.pad_t = node.pt;
        sc.OH = node.OH;
        sc.OW = node.OW;
        sc.w0 = node.d_w0;
        sc.w1 = node.d_w1;
        sc.out_channels = node.O;
        if (node.pool_fused) {
          auto pl = std::make_shared<TcStemPoolLaunch>();
          const std::string perr2 = tc_plan_stem_pool(pl.get(), sc, te, node.pool_oh, node.pool_ow, sm_count_);
          if (!perr2.empty()) return fail(err, "layers " + node.name + " + " + node.pool_name + ": " + perr2);
          s.name = node.name + "+" + node.pool_name;
          s.kernel = std::string("tc_stem_pool_kernel<") + kind_name + ">";
          s.run = [pl](cudaStream_t st) { return tc_launch_stem_pool(*pl, st); };
          plan.steps.push_back(std::move(s));
          return true;
        }
        auto sl = std::make_shared<TcStemLaunch>();
        if (tc_plan_stem(sl.get(), sc, te, sm_count_).empty()) {
          s.kernel = std::string("tc_stem_kernel<") + kind_name + ">";
          s.run = [sl](cudaStream_t st) { return tc_launch_stem(*sl, st); };
          plan.steps.push_back(std::move(s));
          return true;
        }
      }
      if (node.kind == N_CONV) {
        TcIm2colView v;
        v.plane0 = i8 ? static_cast<const void*>(in.q) : static_cast<const void*>(in.p0);
        v.plane1 = in.p1;
        const size_t es = static_cast<size_t>(tc_elem_bytes(kind));
        if (node.stem) {
          v.C = node.k_elems;
          v.W = node.OW;
          v.H = ti.h;
          v.N = n;
          v.stride_w = static_cast<uint64_t>(node.sw) * ti.Cp * es;
          v.stride_h = static_cast<uint64_t>(ti.Wp) * ti.Cp * es;
          v.stride_n = v.stride_h * ti.h;
          v.KH = node.KH;
          v.KW = 1;
          v.stride_conv_h = node.sh;
          v.stride_conv_w = 1;
          v.pad_t = node.pt;
          v.pad_l = 0;
          v.dil_h = node.dh;
          v.dil_w = 1;
        } else {
          v.C = ti.c;
          v.W = ti.w;
          v.H = ti.h;
          v.N = n;
          v.stride_w = static_cast<uint64_t>(ti.c) * es;
          v.stride_h = v.stride_w * ti.w;
          v.stride_n = v.stride_h * ti.h;
          v.KH = node.KH;
          v.KW = node.KW;
          v.stride_conv_h = node.sh;
          v.stride_conv_w = node.sw;
          v.pad_t = node.pt;
          v.pad_l = node.pl;
          v.dil_h = node.dh;
          v.dil_w = node.dw;
        }
        v.OH = node.OH;
        v.OW = node.OW;
        perr = tc_plan_conv(launch.get(), kind, v, node.d_w0, node.d_w1, node.O, te, sm_count_);
      } else {
        const long long M = (to.rank == 2 ? static_cast<long long>(ti.h) : 1) * n;
        const void* a0 = i8 ? static_cast<const void*>(in.q) : static_cast<const void*>(in.p0);
        // a handful of rows: one pass over the weights on the CUDA cores instead of mostly empty 128-row tiles
        if ((kind == GEMM_BF16X3 || kind == GEMM_I8) && !env_flag_off("NCNN_B200_IP_ROWS") &&
            ip_rows_applies(M, node.K, node.O, i8, te.out_mode, te.res0 != nullptr, te.side_count > 0)) {
          IpRowsParams ip{};
          ip.M = static_cast<int>(M);
          ip.K = node.K;
          ip.N = node.O;
          ip.lda = node.K;
          ip.ldw = (node.K + node.k_elems - 1) / node.k_elems * node.k_elems;
          ip.a0 = a0;
          ip.a1 = in.p1;
          ip.w0 = node.d_w0;
          ip.w1 = node.d_w1;
          ip.bias = te.bias;
          ip.scale = te.scale;
          ip.out_scale = te.out_scale;
          ip.act = te.act;
          ip.act_a = te.act_a;
          ip.act_b = te.act_b;
          ip.out_mode = te.out_mode;
          ip.out0 = te.out0;
          ip.out1 = te.out1;
          ip.outq = te.outq;
          ip.ldo = te.ldo;
          const int smem = static_cast<int>(ip_rows_smem_bytes(ip.M, ip.K, i8));
          const cudaError_t ae = i8 ? cudaFuncSetAttribute(k_ip_rows<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024)
                                    : cudaFuncSetAttribute(k_ip_rows<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
          if (ae != cudaSuccess) return fail(err, "layer " + node.name + ": " + cudaGetErrorString(ae));
          const int tasks = (ip.N + kIpRowsCols - 1) / kIpRowsCols;
          const int grid = std::max(1, std::min(sm_count_, tasks));
          s.kernel = i8 ? "k_ip_rows<i8>" : "k_ip_rows<bf16x2>";
          s.run = [=](cudaStream_t st) {
            if (i8) k_ip_rows<true><<<grid, kIpRowsThreads, smem, st>>>(ip);
            else k_ip_rows<false><<<grid, kIpRowsThreads, smem, st>>>(ip);
            return launch_ok();
          };
          plan.steps.push_back(std::move(s));
          return true;
        }
        perr = tc_plan_gemm(launch.get(), kind, a0, in.p1, M, node.K, node.K, node.d_w0, node.d_w1, node.O, te, sm_count_);
      }
      if (!perr.empty()) return fail(err, "layer " + node.name + ": " + perr);
      s.kernel = std::string(launch->cta2 == 2 ? (launch->p.streamk ? "tc_gemm2_kernel:pairs+split<" : "tc_gemm2_kernel:pairs<") : (launch->cta2 == 1 ? "tc_gemm2_kernel:split<" : "tc_gemm_kernel<")) + kind_name + ">";
      s.run = [launch](cudaStream_t st) { return tc_launch(*launch, st); };
      plan.steps.push_back(std::move(s));
    } else if (node.kind == N_CONV || node.kind == N_DW) {
      ConvGeom g{};
      g.images = n;
      g.H = ti.h;
      g.W = ti.w;
      g.C = ti.c;
      g.OH = node.OH;
      g.OW = node.OW;
      g.O = node.O;
      g.KH = node.KH;
      g.KW = node.KW;
      g.sh = node.sh;
      g.sw = node.sw;
      g.pt = node.pt;
      g.pl = node.pl;
      g.dh = node.dh;
      g.dw = node.dw;
      const void* w = node.d_w0;
      if (node.kind == N_DW && !i8 && ti.c % 4 == 0 && node.KH == 3 && node.KW == 3 && node.dh == 1 &&
          node.dw == 1 && node.sh == node.sw && (node.sh == 1 || node.sh == 2) && n <= 65535) {
        const dim3 grid(((node.OH + 7) / 8) * ((node.OW + 7) / 8), (ti.c / 4 + 7) / 8, static_cast<unsigned>(n));
        const int stride = node.sh;
        const float* wf = static_cast<const float*>(w);
        s.kernel = "k_depthwise3x3_tile";
        s.run = [=](cudaStream_t st) {
          if (stride == 1) k_depthwise3x3_tile<1><<<grid, 256, 0, st>>>(in, out, wf, g, e);
          else k_depthwise3x3_tile<2><<<grid, 256, 0, st>>>(in, out, wf, g, e);
          return launch_ok();
        };
      } else if (node.kind == N_DW) {
        const bool vec = ti.c % 4 == 0;
        const long long work = n * node.OH * node.OW * (vec ? ti.c / 4 : ti.c);
        const int grid = grid_for(work);
        s.kernel = i8 ? "k_depthwise<i8>" : "k_depthwise<f32>";
        s.run = [=](cudaStream_t st) {
          if (i8) {
            if (vec) k_depthwise<4, true><<<grid, 256, 0, st>>>(in, out, w, g, e);
            else k_depthwise<1, true><<<grid, 256, 0, st>>>(in, out, w, g, e);
          } else {
            if (vec) k_depthwise<4, false><<<grid, 256, 0, st>>>(in, out, w, g, e);
            else k_depthwise<1, false><<<grid, 256, 0, st>>>(in, out, w, g, e);
          }
          return launch_ok();
        };
      } else {
        const int grid = grid_for(n * node.OH * node.OW * node.O);
        s.kernel = i8 ? "k_conv_direct<i8>" : "k_conv_direct<f32>";
        s.run = [=](cudaStream_t st) {
          if (i8) k_conv_direct<true><<<grid, 256, 0, st>>>(in, out, w, g, e);
          else k_conv_direct<false><<<grid, 256, 0, st>>>(in, out, w, g, e);
          return launch_ok();
        };
      }
      plan.steps.push_back(std::move(s));
    } else {
      const long long M = (to.rank == 2 ? static_cast<long long>(ti.h) : 1) * n;
      const int K = node.K, N = node.O;
      const void* w = node.d_w0;
      const int grid = grid_for(M * N);
      s.kernel = i8 ? "k_matmul_direct<i8>" : "k_matmul_direct<f32>";
      s.run = [=](cudaStream_t st) {
        if (i8) k_matmul_direct<true><<<grid, 256, 0, st>>>(in, out, w, M, K, N, e, 0.0f);
        else k_matmul_direct<false><<<grid, 256, 0, st>>>(in, out, w, M, K, N, e, 0.0f);
        return launch_ok();
      };
      plan.steps.push_back(std::move(s));
    }
    if (node.kind == N_GEMM && node.alpha != 1.0f && !(node.impl == IMPL_TC && node.act == ACT_NONE)) {
      Step m;
      m.name = node.name + ":alpha";
      m.kernel = "k_binary";
      BinaryParams bp{};
      bp.op = BIN_MUL;
      bp.use_scalar = 1;
      bp.scalar = node.alpha;
      const long long count = to.logical() * n;
      const int grid = grid_for(count);
      m.run = [=](cudaStream_t st) {
        k_binary<1><<<grid, 256, 0, st>>>(out, out, out, count, bp);
        return launch_ok();
      };
      plan.steps.push_back(std::move(m));
    }
    return true;
  }
  if (node.kind == N_POOL) {
    const ActRef in = ref(node.in[0], n);
    PoolParams p = node.pool;
    p.images = n;
    p.side_q = node.side_q.empty() ? nullptr : ref(node.side_q[0].first, n).q;
    p.side_scale = node.side_q.empty() ? 0.0f : node.side_q[0].second;
    const bool vec = p.C % 4 == 0;
    if (p.kind == 0 && p.KH == 3 && p.KW == 3 && p.sh == 2 && p.sw == 2 && vec && !tensors_[resolve(node.in[0])].i8 &&
        n <= 65535 && p.OH * p.OW >= 64) {
      const dim3 grid(((p.OH + 7) / 8) * ((p.OW + 7) / 8), (p.C / 4 + 7) / 8, static_cast<unsigned>(n));
      s.kernel = "k_maxpool3x3s2_tile";
      s.run = [=](cudaStream_t st) {
        k_maxpool3x3s2_tile<<<grid, 256, 0, st>>>(in, out, p);
        return launch_ok();
      };
      plan.steps.push_back(std::move(s));
      return true;
    }
    // one window over the whole image (global pooling, or a window at least as large as an unpadded image)
    const bool whole = !p.adaptive && p.OH == 1 && p.OW == 1 && p.pt == 0 && p.pl == 0 && p.KH >= p.H && p.KW >= p.W;
    if (whole && vec && n <= 65535) {
      const dim3 grid((p.C / 4 + 127) / 128, static_cast<unsigned>(n));
      s.kernel = "k_global_pool4";
      s.run = [=](cudaStream_t st) {
        k_global_pool4<<<grid, 128, 0, st>>>(in, out, p);
        return launch_ok();
      };
      plan.steps.push_back(std::move(s));
      return true;
    }
    const int grid = grid_for(n * p.OH * p.OW * (vec ? p.C / 4 : p.C));
    s.kernel = "k_pool";
    s.run = [=](cudaStream_t st) {
      if (vec) k_pool<4><<<grid, 256, 0, st>>>(in, out, p);
      else k_pool<1><<<grid, 256, 0, st>>>(in, out, p);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_DECONV) {
    const Tensor& ti = tensors_[resolve(node.in[0])];
    const ActRef in = ref(node.in[0], n);
    DeconvParams dp{n, ti.h, ti.w, ti.c, node.O, node.act == ACT_RELU ? 1 : 0};
    const float* w = static_cast<const float*>(node.d_w0);
    const float* bias = node.d_bias;
    const int grid = grid_for(to.logical() * n);
    s.kernel = "k_deconv2x2";
    s.run = [=](cudaStream_t st) {
      k_deconv2x2<<<grid, 256, 0, st>>>(in, out, w, bias, dp);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_REDUCE) {
    const ActRef in = ref(node.in[0], n);
    ReduceParams rp = node.reduce;
    rp.images = n;
    const int grid = grid_for(to.logical() * n);
    s.kernel = "k_reduce_mean";
    s.run = [=](cudaStream_t st) {
      k_reduce_mean<<<grid, 256, 0, st>>>(in, out, rp);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_REMAP) {
    const ActRef in = ref(node.in[0], n);
    RemapParams rp = node.remap;
    rp.images = n;
    const int grid = grid_for(to.logical() * n);
    s.kernel = "k_remap";
    s.run = [=](cudaStream_t st) {
      k_remap<<<grid, 256, 0, st>>>(in, out, rp);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_BINARY && node.broadcast) {
    const ActRef a = ref(node.in[0], n);
    const ActRef b = ref(node.in[1], n);
    BroadcastParams bp = node.bcast;
    bp.images = n;
    bp.op = node.bin;
    const int grid = grid_for(bp.o_image * n);
    s.kernel = "k_binary_broadcast";
    s.run = [=](cudaStream_t st) {
      k_binary_broadcast<<<grid, 256, 0, st>>>(a, b, out, bp);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_BINARY) {
    const ActRef a = ref(node.in[0], n);
    const ActRef b = node.in.size() > 1 ? ref(node.in[1], n) : a;
    const BinaryParams bp = node.bin;
    const long long count = to.logical() * n;
    const bool vec = count % 4 == 0;
    const int grid = grid_for(vec ? count / 4 : count);
    s.kernel = "k_binary";
    s.run = [=](cudaStream_t st) {
      if (vec) k_binary<4><<<grid, 256, 0, st>>>(a, b, out, count, bp);
      else k_binary<1><<<grid, 256, 0, st>>>(a, b, out, count, bp);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_UNARY) {
    const ActRef in = ref(node.in[0], n);
    const UnaryParams up = node.un;
    const long long count = to.logical() * n;
    const bool vec = count % 4 == 0;
    if (up.op == UN_QUANT && up.nscale == 1 && in.fmt == FMT_F32 && out.fmt == FMT_I8 && count % 16 == 0 &&
        !node.un_scale.empty()) {
      const float scale = node.un_scale[0];
      const int grid16 = grid_for(count / 16);
      const float* xp = in.p0;
      int8_t* yp = out.q;
      int8_t* y2 = node.side_q.empty() ? nullptr : ref(node.side_q[0].first, n).q;
      const float scale2 = node.side_q.empty() ? 0.0f : node.side_q[0].second;
      s.kernel = node.side_q.empty() ? "k_quantize16" : "k_quantize16:two results";
      s.run = [=](cudaStream_t st) {
        k_quantize16<<<grid16, 256, 0, st>>>(xp, yp, count / 16, scale, y2, scale2);
        return launch_ok();
      };
      plan.steps.push_back(std::move(s));
      return true;
    }
    const int grid = grid_for(vec ? count / 4 : count);
    s.kernel = "k_unary";
    s.run = [=](cudaStream_t st) {
      if (vec) k_unary<4><<<grid, 256, 0, st>>>(in, out, count, up);
      else k_unary<1><<<grid, 256, 0, st>>>(in, out, count, up);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_SOFTMAX) {
    const ActRef in = ref(node.in[0], n);
    SoftmaxParams sp = node.softmax;
    sp.images = n;
    const int grid = grid_for(n * sp.lines * 32);
    s.kernel = "k_softmax";
    s.run = [=](cudaStream_t st) {
      k_softmax<<<grid, 256, 0, st>>>(in, out, sp);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  if (node.kind == N_CONCAT) {
    for (size_t k = 0; k < node.in.size(); ++k) {
      Step c = s;
      c.name = node.name + ":" + std::to_string(k);
      c.flops = 0;
      c.bytes = 2.0 * bytes_of(node.in[k]);
      const ActRef in = ref(node.in[k], n);
      ConcatParams cp = node.concat[k];
      cp.images = n;
      const int grid = grid_for(n * cp.in_image_elems);
      c.kernel = "k_concat_copy";
      c.run = [=](cudaStream_t st) {
        k_concat_copy<<<grid, 256, 0, st>>>(in, out, cp);
        return launch_ok();
      };
      plan.steps.push_back(std::move(c));
    }
    return true;
  }
  if (node.kind == N_RELAYOUT) {
    const ActRef in = ref(node.in[0], n);
    RelayoutParams rp = node.relayout;
    rp.images = n;
    const int grid = grid_for(rp.count * n);
    s.kernel = "k_relayout";
    s.run = [=](cudaStream_t st) {
      k_relayout<<<grid, 256, 0, st>>>(in, out, rp);
      return launch_ok();
    };
    plan.steps.push_back(std::move(s));
    return true;
  }
  return fail(err, "internal: unknown node kind");
}

void EngineImpl::make_edge_steps(int64_t n, const std::vector<const float*>& d_in,
                                 const std::vector<float*>& d_out, std::vector<Step>* pre,
                                 std::vector<Step>* post) {
  for (size_t i = 0; i < inputs_.size(); ++i) {
    const Tensor& t = tensors_[resolve(inputs_[i])];
    const ActRef dst = ref(inputs_[i], n);
    const float* src_ptr = d_in[i];
    Step s;
    s.name = "input:" + t.name;
    s.bytes = static_cast<double>(t.logical()) * n * (4 + t.elem_bytes() * t.planes());
    // one channel, or one pixel: channel-last order is the caller's order, a flat copy does it
    const bool flat_layout = (t.c == 1 || t.h * t.w == 1) && t.Cp == t.c && t.Wp == t.w && t.w_off == 0;
    const bool flat_quant = t.rank == 3 && flat_layout && t.input_quant_scale > 0.0f && dst.fmt == FMT_I8 &&
                            (t.logical() * n) % 16 == 0 && (reinterpret_cast<uintptr_t>(src_ptr) & 15) == 0 &&
                            (reinterpret_cast<uintptr_t>(dst.q) & 15) == 0;
    const bool flat_in = t.rank != 3 || (flat_layout && t.input_quant_scale <= 0.0f);
    if (flat_quant) {
      const long long count16 = t.logical() * n / 16;
      const int grid = grid_for(count16);
      const float scale = t.input_quant_scale;
      int8_t* q = dst.q;
      s.kernel = "k_quantize16";
      s.run = [=](cudaStream_t st) {
        k_quantize16<<<grid, 256, 0, st>>>(src_ptr, q, count16, scale, nullptr, 0.0f);
        return launch_ok();
      };
    } else if (!flat_in) {
      EdgeParams ep{};
      ep.images = n;
      ep.C = t.c;
      ep.H = t.h;
      ep.W = t.w;
      ep.Cp = t.Cp;
      ep.Wp = t.Wp;
      ep.w_off = t.w_off;
      ep.quant_scale = t.input_quant_scale;
      if (t.c <= 4 && ((t.Cp == 4 && t.fmt != FMT_I8) || (t.Cp == 8 && t.fmt == FMT_I8)) && t.w % 4 == 0 &&
          n <= 65535 &&
          (reinterpret_cast<uintptr_t>(src_ptr) & 15) == 0) {
        const dim3 grid(static_cast<unsigned>(std::min(148 * 8, (t.h * t.w / 4 + 255) / 256)), static_cast<unsigned>(n));
        s.kernel = "k_chw_to_nhwc_small_x4";
        s.run = [=](cudaStream_t st) {
          k_chw_to_nhwc_small_x4<<<grid, 256, 0, st>>>(src_ptr, dst, ep);
          return launch_ok();
        };
      } else if (t.c <= 4 && (t.Cp == 4 || t.Cp == 16 || (t.Cp == 8 && t.fmt == FMT_I8))) {
        const int grid = grid_for(n * t.h * t.w);
        s.kernel = "k_chw_to_nhwc_small";
        s.run = [=](cudaStream_t st) {
          k_chw_to_nhwc_small<<<grid, 256, 0, st>>>(src_ptr, dst, ep);
          return launch_ok();
        };
      } else {
        const dim3 grid((t.h * t.w + 31) / 32, (t.c + 31) / 32, static_cast<unsigned>(n));
        s.kernel = "k_chw_to_nhwc_tiled";
        s.run = [=](cudaStream_t st) {
          k_chw_to_nhwc_tiled<<<grid, dim3(32, 8), 0, st>>>(src_ptr, dst, ep);
          return launch_ok();
        };
      }
    } else {
      ActRef src;
      src.fmt = FMT_F32;
      src.p0 = const_cast<float*>(src_ptr);
      UnaryParams up{};
      up.op = UN_COPY;
      const long long count = t.logical() * n;
      const bool vec = count % 4 == 0 && (reinterpret_cast<uintptr_t>(src_ptr) & 15) == 0;
      const int grid = grid_for(vec ? count / 4 : count);
      s.kernel = "k_unary";
      s.run = [=](cudaStream_t st) {
        if (vec) k_unary<4><<<grid, 256, 0, st>>>(src, dst, count, up);
        else k_unary<1><<<grid, 256, 0, st>>>(src, dst, count, up);
        return launch_ok();
      };
    }
    pre->push_back(std::move(s));
  }
  for (size_t i = 0; i < outputs_.size(); ++i) {
    const Tensor& t = tensors_[resolve(outputs_[i])];
    const ActRef src = ref(outputs_[i], n);
    float* dst_ptr = d_out[i];
    Step s;
    s.name = "output:" + t.name;
    s.bytes = static_cast<double>(t.logical()) * n * (4 + t.elem_bytes() * t.planes());
    const bool flat_out = t.rank != 3 || ((t.c == 1 || t.h * t.w == 1) && t.Cp == t.c && t.Wp == t.w && t.w_off == 0);
    if (!flat_out) {
      const dim3 grid((t.h * t.w + 31) / 32, (t.c + 31) / 32, static_cast<unsigned>(n));
      const int C = t.c, HW = t.h * t.w, Cp = t.Cp;
      s.kernel = "k_nhwc_to_chw_tiled";
      s.run = [=](cudaStream_t st) {
        k_nhwc_to_chw_tiled<<<grid, dim3(32, 8), 0, st>>>(src, dst_ptr, n, C, HW, Cp);
        return launch_ok();
      };
    } else {
      ActRef dst;
      dst.fmt = FMT_F32;
      dst.p0 = dst_ptr;
      UnaryParams up{};
      up.op = UN_COPY;
      const long long count = t.logical() * n;
      const bool vec = count % 4 == 0 && (reinterpret_cast<uintptr_t>(dst_ptr) & 15) == 0;
      const int grid = grid_for(vec ? count / 4 : count);
      s.kernel = "k_unary";
      s.run = [=](cudaStream_t st) {
        if (vec) k_unary<4><<<grid, 256, 0, st>>>(src, dst, count, up);
        else k_unary<1><<<grid, 256, 0, st>>>(src, dst, count, up);
        return launch_ok();
      };
    }
    post->push_back(std::move(s));
  }
}

}  // namespace nb
