"""Known answers for the CPU oracle, derived independently of oracle/ncnn_ops.c.

The reference keeps no stored golden outputs for these operators (its tests call
upstream ncnn at run time), so each case here restates the arithmetic of the cited
lowering with plain Python loops over the fixture's literal weights, or states the
expected integers by hand.  Inputs are the reference's own fixtures under
tests/golden/fixtures (bins produced by running the reference's generators).
"""
import struct

import numpy as np
import pytest

from conftest import fixture

F32 = np.float32


def rha(v):
    """Round half away from zero as the reference evaluates it in fp32
    (lib/Conversion/NCNNToTosa/NCNNToTosa.cpp:356-385), clamped to [-127, 127]."""
    v = F32(v)
    r = np.floor(F32(v + F32(0.5))) if v >= 0 else np.ceil(F32(v + F32(-0.5)))
    return int(max(min(r, 127.0), -127.0))


def test_quantize_rounding_known_answers(oracle):
    x = np.array([0.49999997, -0.49999997, 0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 126.5, -126.5, 127.49, -127.49,
                  200.0, -200.0, 0.0, 0.4999999, 1e9, -1e9], F32)
    # 0.49999997f + 0.5f is exactly representable only after rounding to 1.0f -> floor gives 1;
    # roundf()/rintf() would give 0.  0.4999999f + 0.5f = 0.9999999f -> 0.
    want = [1, -1, 1, -1, 2, -2, 3, -3, 127, -127, 127, -127, 127, -127, 0, 0, 127, -127]
    got = oracle.quantize(x, np.array([1.0], F32))
    assert got.tolist() == want
    assert [rha(v) for v in x] == want
    # per-channel scales along an axis
    y = oracle.quantize(np.array([[1.0, 1.0], [1.0, 1.0]], F32), np.array([2.0, 3.0], F32), axis=1)
    assert y.tolist() == [[2, 3], [2, 3]]


def test_quantize_c_and_numpy_paths_agree(oracle):
    import ctypes
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(4096) * 40).astype(F32)
    x[:8] = [0.49999997, -0.49999997, 0.5, -0.5, 126.5, 127.5, -127.5, 0.0]
    s = np.array([1.0], F32)
    y = np.empty(x.size, np.int8)
    oracle._ops().orc_quantize(x.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), ctypes.c_size_t(x.size),
                               ctypes.c_size_t(1), s.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                               ctypes.c_size_t(1), y.ctypes.data_as(ctypes.POINTER(ctypes.c_int8)))
    assert np.array_equal(y, oracle.quantize(x, s))


def naive_conv(x, w, bias, stride, pad, dil=1, pad_after=None):
    """x [C,H,W], w [O,C,KH,KW]: bias + sum, zero padding, cross-correlation
    (NCNNToTosa.cpp:1485-1498), accumulated in float64."""
    C, H, W = x.shape
    O, _, KH, KW = w.shape
    after = pad if pad_after is None else pad_after
    OH = (H + pad + after - ((KH - 1) * dil + 1)) // stride + 1
    OW = (W + pad + after - ((KW - 1) * dil + 1)) // stride + 1
    y = np.zeros((O, OH, OW))
    for o in range(O):
        for oh in range(OH):
            for ow in range(OW):
                acc = float(bias[o]) if bias is not None else 0.0
                for c in range(C):
                    for kh in range(KH):
                        for kw in range(KW):
                            ih, iw = oh * stride - pad + kh * dil, ow * stride - pad + kw * dil
                            if 0 <= ih < H and 0 <= iw < W:
                                acc += float(x[c, ih, iw]) * float(w[o, c, kh, kw])
                y[o, oh, ow] = acc
    return y


def read_f32(path, offset, count):
    with open(path, "rb") as f:
        data = f.read()
    return np.array(struct.unpack_from(f"<{count}f", data, offset), F32)


def test_convolution_fixture_known_answer(oracle):
    param, bin_ = fixture("convolution")  # 1x4x4 input, 2 outputs, 3x3, pad 1, bias
    w = read_f32(bin_, 4, 18).reshape(2, 1, 3, 3)
    b = read_f32(bin_, 4 + 72, 2)
    assert b.tolist() == [0.125, -0.25] and w[0, 0, 0].tolist() == [0.25, -0.5, 0.75]
    x = (np.arange(16, dtype=F32).reshape(1, 4, 4) - 7.5) / 4
    want = naive_conv(x, w, b, 1, 1)
    got = oracle.Model(param, bin_).run([x])[0]
    assert got.shape == (2, 4, 4)
    assert np.allclose(got, want, rtol=1e-6, atol=1e-6)
    # one value entirely by hand: output channel 0 at (0,0) sees x[0:2,0:2] under w[1:,1:]
    hand = 0.125 + (-1.875) * 0.5 + (-1.625) * 0.125 + (-0.875) * (-0.25) + (-0.625) * 1.0
    assert abs(float(got[0, 0, 0]) - hand) < 1e-6


@pytest.mark.parametrize("name,stride,pad,dil", [("convolution_dilated", 1, 1, 2), ("convolution_no_bias", 1, 1, 1)])
def test_more_convolution_fixtures(oracle, name, stride, pad, dil):
    param, bin_ = fixture(name)
    layers = oracle.load_graph(param, bin_)
    conv = layers[1]
    C = layers[0].geti(2)
    O, k = conv.geti(0), conv.geti(1)
    w = conv.weights[0].reshape(O, C, k, k)
    b = conv.weights[1] if conv.geti(5) else None
    x = np.random.default_rng(7).standard_normal((C, layers[0].geti(1), layers[0].geti(0))).astype(F32)
    want = naive_conv(x, w, b, conv.geti(3, 1), conv.geti(4, 0), conv.geti(2, 1), conv.geti(15, conv.geti(4, 0)))
    got = oracle.Model(param, bin_).run([x])[0]
    assert np.allclose(got, want, rtol=1e-5, atol=1e-6)


def test_pooling_shapes_and_values(oracle):
    x = np.arange(2 * 5 * 5, dtype=F32).reshape(2, 5, 5)
    # pooling.param: max 3x3 stride 2, pad_mode 1 (valid): 5 -> 2
    got = oracle.Model(*fixture("pooling")).run([x])[0]
    assert got.shape == (2, 2, 2)
    assert got[0].tolist() == [[12, 14], [22, 24]]
    # pooling_tail.param: 4x4, k3 s2, pad_mode 0 ("full"): (4-3)%2 != 0 -> one tail window: 2x2
    x4 = np.arange(2 * 4 * 4, dtype=F32).reshape(2, 4, 4)
    got = oracle.Model(*fixture("pooling_tail")).run([x4])[0]
    assert got.shape == (2, 2, 2)
    assert got[0].tolist() == [[10, 11], [14, 15]]  # the tail windows only see the last column/row
    # pooling_average.param: avg 3x3 s2 pad 1, valid mode, exclude-pad divisor
    got = oracle.Model(*fixture("pooling_average")).run([x])[0]
    assert got.shape == (2, 3, 3)  # (5 + 2 - 3) / 2 + 1
    assert got[0, 0, 0] == F32((0 + 1 + 5 + 6) / 4)  # corner window: 4 in-bounds elements
    assert got[0, 1, 1] == F32(sum([6, 7, 8, 11, 12, 13, 16, 17, 18]) / 9)
    # global average -> rank 1
    got = oracle.Model(*fixture("pooling_global_average")).run([x])[0]
    assert got.shape == (2,) and got.tolist() == [12.0, 37.0]
    # SAME upper on 4x5 (h=4,w=5), k3 s2: out = ceil(in/2)
    xs = np.arange(2 * 4 * 5, dtype=F32).reshape(2, 4, 5)
    got = oracle.Model(*fixture("pooling_same_upper")).run([xs])[0]
    assert got.shape == (2, 2, 3)


def test_eltwise_weighted_and_binary(oracle):
    a = np.array([[[1, 2], [3, 4]], [[5, 6], [7, 8]]], F32)
    b = np.array([[[0.5, 1], [1.5, 2]], [[2.5, 3], [3.5, 4]]], F32)
    got = oracle.Model(*fixture("eltwise_weighted")).run([a, b])[0]
    assert np.array_equal(got, (a * F32(2.0)) + (b * F32(-1.5)))  # coefficients first, then the sum
    a43 = np.arange(24, dtype=F32).reshape(2, 3, 4)
    got = oracle.Model(*fixture("binary_add")).run([a43, a43 * 2])[0]
    assert np.array_equal(got, a43 * 3)


def test_int8_convolution_term1_by_hand(oracle):
    """convolution_int8_term1: 1x1 conv 2->3 channels, int8 weights ((7i+3)%15)-7, bias 0.125(i-1),
    weight scales 5+1.5i, input scale 8 (generate_int8_bins.py:19-29)."""
    param, bin_ = fixture("convolution_int8_term1")
    wq = [((i * 7 + 3) % 15) - 7 for i in range(6)]
    bias = [0.125 * (i - 1) for i in range(3)]
    ws = [5.0 + 1.5 * i for i in range(3)]
    x = np.random.default_rng(0xC001).uniform(-1.5, 1.5, (2, 3, 4)).astype(F32)
    got = oracle.Model(param, bin_).run([x])[0]
    for o in range(3):
        r = F32(1.0) / F32(F32(ws[o]) * F32(8.0))
        for h in range(3):
            for w in range(4):
                acc = sum(rha(F32(x[c, h, w]) * F32(8.0)) * wq[o * 2 + c] for c in range(2))
                y = F32(F32(F32(acc) * r) + F32(bias[o]))
                assert got[o, h, w] == y


def test_int8_chain_requantizes_between_layers(oracle):
    """int8_complete_chain: conv(101) -> depthwise(101) -> conv(1); every stage by hand."""
    param, bin_ = fixture("int8_complete_chain")
    x = np.random.default_rng(0x8C11).uniform(-1.5, 1.5, (2, 3, 4)).astype(F32)
    got = oracle.Model(param, bin_).run([x])[0]
    w1 = [((i * 7 + 3) % 15) - 7 for i in range(6)]
    b1 = [0.125 * (i - 1) for i in range(3)]
    s1 = [5.0 + 1.5 * i for i in range(3)]
    wd = [((i * 5 + 1) % 11) - 5 for i in range(3)]
    bd = [0.1 * (i - 1) for i in range(3)]
    sd = [4.0 + i for i in range(3)]
    w3 = [((i * 7 + 3) % 15) - 7 for i in range(6)]
    b3 = [0.125 * (i - 1) for i in range(2)]
    s3 = [5.0 + 1.5 * i for i in range(2)]
    for h in range(3):
        for w in range(4):
            q0 = [rha(F32(x[c, h, w]) * F32(8.0)) for c in range(2)]
            q1 = []
            for o in range(3):
                acc = sum(q0[c] * w1[o * 2 + c] for c in range(2))
                y = F32(F32(F32(acc) * (F32(1.0) / F32(F32(s1[o]) * F32(8.0)))) + F32(b1[o]))
                q1.append(rha(y * F32(6.0)))
            q2 = []
            for c in range(3):
                y = F32(F32(F32(q1[c] * wd[c]) * (F32(1.0) / F32(F32(sd[c]) * F32(7.0)))) + F32(bd[c]))
                q2.append(rha(y * F32(5.0)))
            for o in range(2):
                acc = sum(q2[c] * w3[o * 3 + c] for c in range(3))
                y = F32(F32(F32(acc) * (F32(1.0) / F32(F32(s3[o]) * F32(8.0)))) + F32(b3[o]))
                assert got[o, h, w] == y


def test_gemm_applies_beta_to_bias_then_alpha_to_the_sum(oracle):
    """gemm.param: y = (A*B^T + beta*C)*alpha with alpha .5, beta -1.25 (NCNNToTosa.cpp:5079-5096)."""
    param, bin_ = fixture("gemm")
    B = np.array([0.5, -0.25, 1.0, 0.75, -0.5, 0.125, 0.25, -1.0], F32).reshape(4, 2)
    C = np.array([0.2, -0.4, 0.6, -0.8], F32)
    x = np.arange(6, dtype=F32).reshape(2, 1, 3)  # [c=2,h=1,w=3] -> squeeze [2,3] -> permute [3,2]
    A = x.reshape(2, 3).T
    want = (A.astype(np.float64) @ B.T.astype(np.float64) + (-1.25) * C) * 0.5
    got = oracle.Model(param, bin_).run([x])[0]
    assert got.shape == (3, 4)
    assert np.allclose(got, want, rtol=1e-6, atol=1e-6)


def test_gemm_int8_uses_row_scales_and_true_division(oracle):
    param, bin_ = fixture("gemm_int8_term2")
    Bq = np.array([3, -2, 1, 4, -4, 2, 5, -1], np.int64).reshape(4, 2)
    C = np.array([0.25, -0.5, 0.125, 0.75], F32)
    x = np.array([[[0.5, -1.25, 0.0]], [[1.5, 0.25, 0.0]]], F32)  # third row of A is all zero
    A = x.reshape(2, 3).T
    got = oracle.Model(param, bin_).run([x])[0]
    for m in range(3):
        absmax = F32(max(abs(A[m, 0]), abs(A[m, 1])))
        s = F32(1.0) if absmax == 0 else F32(F32(127.0) / absmax)
        aq = [rha(F32(A[m, k]) * s) for k in range(2)]
        for n in range(4):
            acc = sum(aq[k] * int(Bq[n, k]) for k in range(2))
            y = F32(F32(acc) / F32(s * F32(6.0)))
            y = F32(F32(y + F32(C[n] * F32(-1.25))) * F32(0.5))
            assert got[m, n] == y


def test_batchnorm_fold_matches_the_reference_formula(oracle, tmp_path):
    """Conv -> BatchNorm folds to w*scale, b*scale + (bias - scale*mean), scale = slope*pow(var+eps,-0.5)
    and 10000 when var+eps == 0 (FoldNCNNBatchNorm.cpp:99-160)."""
    rng = np.random.default_rng(3)
    w = rng.standard_normal((3, 2, 1, 1)).astype(F32)
    b = rng.standard_normal(3).astype(F32)
    slope, mean = np.array([1.5, -0.5, 2.0], F32), np.array([0.1, -0.2, 0.3], F32)
    var, beta = np.array([0.0, 0.25, 4.0], F32), np.array([0.5, 0.0, -1.0], F32)
    p = tmp_path / "bn.param"
    p.write_text("7767517\n3 3\nInput in 0 1 data 0=3 1=3 2=2\n"
                 "Convolution conv 1 1 data c 0=3 1=1 5=1 6=6\nBatchNorm bn 1 1 c out 0=3 1=0.0\n")
    (tmp_path / "bn.bin").write_bytes(struct.pack("<I", 0) + w.tobytes() + b.tobytes() + slope.tobytes() +
                                      mean.tobytes() + var.tobytes() + beta.tobytes())
    m = oracle.Model(str(p), str(tmp_path / "bn.bin"))
    assert [l.type for l in m.layers] == ["Input", "Convolution"]  # folded away
    x = rng.standard_normal((2, 3, 3)).astype(F32)
    got = m.run([x])[0]
    scale = np.array([1.5 * 10000.0, -0.5 * 0.25 ** -0.5, 2.0 * 4.0 ** -0.5])
    want = naive_conv(x, w, b, 1, 0) * scale[:, None, None] + (beta - scale * mean)[:, None, None]
    assert np.allclose(got, want, rtol=1e-5, atol=1e-4)


def test_oracle_is_deterministic_and_thread_count_independent(oracle, pkg, tmp_path):
    import os
    param, bin_ = pkg.zoo.resnet18(str(tmp_path / "r18"), size=64)
    x = np.random.default_rng(5).uniform(-1, 1, (3, 64, 64)).astype(F32)
    a = oracle.Model(param, bin_).run([x])[0]
    b = oracle.Model(param, bin_).run([x])[0]
    assert np.array_equal(a, b)
    assert a.shape == (1000,) and np.isfinite(a).all()


# ------------------------------------------------------------------ activations, softmax, concat
def _run_fixture(oracle, name, *inputs):
    param, bin_ = fixture(name)
    return oracle.Model(param, bin_).run(list(inputs))[0]


def test_sigmoid_and_hard_activations_by_hand(oracle):
    import math
    x = np.array([-100.0, -3.0, -1.0, 0.0, 0.5, 2.9, 3.0, 100.0], F32)
    full = np.zeros((2, 2, 5), F32)
    full.reshape(-1)[:8] = x
    got = _run_fixture(oracle, "sigmoid", full).reshape(-1)[:8]
    # clamp to +-88.376..., then 1/(1+exp(-x)) (NCNNToTosa.cpp:3008-3015)
    want = [1.0 / (1.0 + math.exp(-min(max(float(v), -88.3762626647949), 88.3762626647949))) for v in x]
    assert np.allclose(got, want, rtol=2e-7, atol=1e-38)
    assert got[3] == F32(0.5) and got[0] > 0 and got[7] == F32(1.0)
    # hard_sigmoid / hard_swish fixtures: alpha 0.166667, beta 0.5 -> gate = clamp(x/6 + 0.5, 0, 1)
    full = np.zeros((3, 4, 5), F32)
    full.reshape(-1)[:8] = x
    gate = np.clip((x * F32(0.166667)).astype(F32) + F32(0.5), 0, 1).astype(F32)
    assert np.array_equal(_run_fixture(oracle, "hard_sigmoid", full).reshape(-1)[:8], gate)
    assert np.array_equal(_run_fixture(oracle, "hard_swish", full).reshape(-1)[:8], (x * gate).astype(F32))
    # dropout fixture: scale 0.375 is a plain multiplication
    assert np.array_equal(_run_fixture(oracle, "dropout", full).reshape(-1)[:8], (x * F32(0.375)).astype(F32))


@pytest.mark.parametrize("name,axis", [("softmax", 0), ("softmax_channel", 0), ("softmax_height", 1), ("softmax_width", 2),
                                       ("softmax_negative_channel", 0), ("softmax_negative_height", 1),
                                       ("softmax_negative_width", 2)])
def test_softmax_axes(oracle, name, axis):
    """Axis numbers are over the logical [c, h, w] dims (negative from the end); every line sums
    to one and equals the textbook formula computed in float64."""
    x = np.random.default_rng(11).standard_normal((3, 4, 5)).astype(F32)
    got = _run_fixture(oracle, name, x)
    e = np.exp(x.astype(np.float64) - x.max(axis=axis, keepdims=True))
    want = e / e.sum(axis=axis, keepdims=True)
    assert got.shape == x.shape
    assert np.allclose(got, want, rtol=3e-6, atol=1e-9)
    assert np.allclose(got.sum(axis=axis), 1.0, atol=1e-6)


@pytest.mark.parametrize("name,axis,shapes", [("concat", 0, [(1, 3, 4), (2, 3, 4)]), ("concat_height", 1, [(2, 3, 4), (2, 2, 4)]),
                                              ("concat_width", 2, [(2, 3, 4), (2, 3, 2)]),
                                              ("concat_negative_channel", 0, [(1, 3, 4), (2, 3, 4)]),
                                              ("concat_negative_height", 1, [(2, 3, 4), (2, 2, 4)]),
                                              ("concat_negative_width", 2, [(2, 3, 4), (2, 3, 2)])])
def test_concat_axes(oracle, name, axis, shapes):
    rng = np.random.default_rng(12)
    ins = [rng.standard_normal(s).astype(F32) for s in shapes]
    got = _run_fixture(oracle, name, *ins)
    assert np.array_equal(got, np.concatenate(ins, axis=axis))


def test_split_three_concat_chain(oracle):
    x = np.random.default_rng(13).standard_normal((3, 4, 5)).astype(F32)
    got = _run_fixture(oracle, "split_three", x)
    assert np.array_equal(got, np.concatenate([x, x, x], axis=0))


# ------------------------------------------------------------------ rank-4 tensors between data-movement layers
def test_rank4_reshape_permute_slice_concat(oracle):
    """The reference's three rank-4 fixtures (PermuteRankFourOrderThree, SliceRankFourWidthAxis, ConcatRankFourWidthAxis,
    test/Numerical/operators/supported_ops_test.cpp:1035-1078): Reshape with 11=d gives [c,d,h,w]; Permute order 3
    gives [c,h,w,d]; Slice and Concat count their axis over [c,d,h,w].  Data movement only: exact."""
    rng = np.random.default_rng(44)
    x = rng.standard_normal((3, 2, 4)).astype(F32)
    got = _run_fixture(oracle, "permute_rank4", x)
    assert got.shape == (2, 2, 2, 3) and np.array_equal(got, x.reshape(2, 3, 2, 2).transpose(0, 2, 3, 1))
    x = rng.standard_normal((4, 1, 6)).astype(F32)
    param, bin_ = fixture("slice_rank4")
    left, right = oracle.Model(param, bin_).run([x], want=["left", "right"])
    m = x.reshape(4, 1, 1, 6)
    assert left.shape == (4, 1, 1, 2) and right.shape == (4, 1, 1, 4)
    assert np.array_equal(left, m[..., :2]) and np.array_equal(right, m[..., 2:])
    a, b = rng.standard_normal((2, 2, 3)).astype(F32), rng.standard_normal((1, 2, 2)).astype(F32)
    got = _run_fixture(oracle, "concat_rank4", a, b)
    assert got.shape == (1, 2, 2, 4)
    assert np.array_equal(got, np.concatenate([a.reshape(1, 2, 2, 3), b.reshape(1, 2, 2, 1)], axis=3))


def test_detection_head_through_rank4(oracle, pkg, tmp_path):
    """Convolution -> rank-4 Reshape -> Permute -> Sigmoid -> Slice -> Reshape -> Concat equals the same steps in numpy."""
    param, bin_ = pkg.zoo.detection_head(str(tmp_path / "head"), h=6, w=5, cin=16, anchors=3, values=7)
    x = np.random.default_rng(45).uniform(-1, 1, (16, 6, 5)).astype(F32)
    m = oracle.Model(param, bin_)
    raw = m.run([x], want=["raw"])[0]
    got = m.run([x])[0]
    cells = raw.reshape(3, 7, 6, 5).transpose(0, 2, 3, 1)
    prob = m.run([x], want=["prob"])[0]
    assert prob.shape == (3, 6, 5, 7)
    assert np.allclose(prob, 1.0 / (1.0 + np.exp(-cells.astype(np.float64))), rtol=1e-6, atol=1e-7)
    assert got.shape == (90, 7) and np.array_equal(got, prob.reshape(90, 7))


# ------------------------------------------------------------------ broadcast, slice, shuffle, padding, interp
def test_binary_broadcast_square_slice_shuffle(oracle):
    rng = np.random.default_rng(14)
    a, s = rng.standard_normal((2, 3, 4)).astype(F32), rng.standard_normal((2, 1, 1)).astype(F32)
    assert np.array_equal(_run_fixture(oracle, "binary_mul_channel", a, s), a * s)
    assert np.array_equal(_run_fixture(oracle, "binary_mul_reverse_broadcast", s, a), s * a)
    x = rng.standard_normal((4, 2, 3)).astype(F32)
    assert np.array_equal(_run_fixture(oracle, "unary_square", x), x * x)
    # slice fixture (array notation: count first): 5 channels as 2 and the rest along axis 0
    x = rng.standard_normal((5, 3, 4)).astype(F32)
    param, bin_ = fixture("slice")
    m = oracle.Model(param, bin_)
    outs = m.run([x], want=["left", "right"])
    assert np.array_equal(outs[0], x[:2]) and np.array_equal(outs[1], x[2:])
    # shuffle: 6 channels, group 2: output channel j = a*2 + b takes input channel b*3 + a
    x = rng.standard_normal((6, 3, 4)).astype(F32)
    want = x.reshape(2, 3, 3, 4).transpose(1, 0, 2, 3).reshape(6, 3, 4)
    assert np.array_equal(_run_fixture(oracle, "shuffle_channel", x), want)
    want = x.reshape(3, 2, 3, 4).transpose(1, 0, 2, 3).reshape(6, 3, 4)  # reverse: 6/2 = 3 groups
    assert np.array_equal(_run_fixture(oracle, "shuffle_channel_reverse", x), want)


def test_padding_and_interp_by_hand(oracle):
    x = np.arange(12, dtype=F32).reshape(2, 2, 3)
    got = _run_fixture(oracle, "padding_four_sides", x)  # top 1, bottom 2, left 3, right 4, value -7.25
    assert got.shape == (2, 5, 10)
    assert np.array_equal(got[:, 1:3, 3:6], x) and got[0, 0, 0] == F32(-7.25) and got[1, 4, 9] == F32(-7.25)
    assert np.array_equal(_run_fixture(oracle, "padding_identity", np.ones((2, 3, 4), F32)), np.ones((2, 3, 4), F32))
    got = _run_fixture(oracle, "interp", x)  # nearest, scale 2: out[y, x] = in[y // 2, x // 2]
    assert np.array_equal(got, x.repeat(2, axis=1).repeat(2, axis=2))
    got = _run_fixture(oracle, "interp_asymmetric", x)  # explicit 6 x 12 from 2 x 3: (o * in) // out
    assert got.shape == (2, 6, 12)
    assert np.array_equal(got, x[:, (np.arange(6) * 2) // 6][:, :, (np.arange(12) * 3) // 12])


def test_bilinear_interp_matches_textbook(oracle, tmp_path):
    for align in (0, 1):
        p = tmp_path / f"bil{align}.param"
        p.write_text("7767517\n2 2\nInput input 0 1 data 0=5 1=4 2=2\n"
                     f"Interp up 1 1 data output 0=2 1=2.0 2=3.0 6={align}\n")
        (tmp_path / f"bil{align}.bin").write_bytes(b"")
        x = np.random.default_rng(15).standard_normal((2, 4, 5)).astype(F32)
        got = oracle.Model(str(p), str(tmp_path / f"bil{align}.bin")).run([x])[0]
        assert got.shape == (2, 8, 15)
        want = np.zeros((2, 8, 15))
        for oy in range(8):
            for ox in range(15):
                sy = oy * 3 / 7 if align else (oy + 0.5) * 4 / 8 - 0.5
                sx = ox * 4 / 14 if align else (ox + 0.5) * 5 / 15 - 0.5
                sy, sx = min(max(sy, 0), 3), min(max(sx, 0), 4)
                y0, x0 = min(int(np.floor(sy)), 2), min(int(np.floor(sx)), 3)
                fy, fx = sy - y0, sx - x0
                v = x[:, y0:y0 + 2, x0:x0 + 2].astype(np.float64)
                want[:, oy, ox] = (v[:, 0, 0] * (1 - fx) + v[:, 0, 1] * fx) * (1 - fy) + (v[:, 1, 0] * (1 - fx) + v[:, 1, 1] * fx) * fy
        assert np.allclose(got, want, rtol=1e-5, atol=2e-6)


def test_reduction_mean_fixtures(oracle):
    x = np.random.default_rng(16).standard_normal((4, 3, 4)).astype(F32)
    got = _run_fixture(oracle, "reduction_mean", x)  # axes (1, 2) without keepdims -> [c]
    assert got.shape == (4,) and np.allclose(got, x.mean(axis=(1, 2)), rtol=1e-6, atol=1e-7)
    got = _run_fixture(oracle, "reduction_mean_keepdims_coeff", x)  # keepdims, coeff 0.5
    assert got.shape == (4, 1, 1) and np.allclose(got[:, 0, 0], 0.5 * x.mean(axis=(1, 2)), rtol=1e-6, atol=1e-7)


def test_squeeze_expand_dims_permute_by_hand(oracle, tmp_path):
    """Explicit axes only; a named axis that is not 1 stays (computeSqueezeResult, NCNNOps.cpp:868-901);
    ExpandDims axes index the result rank (:903-927); rank-3 Permute orders 2 and 4."""
    x = np.arange(12, dtype=F32).reshape(3, 1, 4)
    assert np.array_equal(_run_fixture(oracle, "squeeze", x), x.reshape(3, 4))
    assert np.array_equal(_run_fixture(oracle, "expand_dims", x), x.reshape(3, 1, 4))  # squeeze axis 1, expand at -2
    assert np.array_equal(_run_fixture(oracle, "permute", x), x.reshape(3, 4).T)

    def run(text, x):
        p = tmp_path / "m.param"
        p.write_text(text)
        (tmp_path / "m.bin").write_bytes(b"")
        return oracle.Model(str(p), str(tmp_path / "m.bin")).run([x])[0]

    head = "7767517\n2 2\nInput input 0 1 data 0=4 1=1 2=3\n"
    assert run(head + "Squeeze s 1 1 data output -23303=2,0,1\n", x).shape == (3, 4)   # axis 0 has extent 3: kept
    assert run(head + "Squeeze s 1 1 data output -23303=1,-2\n", x).shape == (3, 4)
    with pytest.raises(ValueError):
        run(head + "Squeeze s 1 1 data output 0=1\n", x)                                 # flags instead of axes
    y = np.arange(24, dtype=F32).reshape(2, 3, 4)
    head = "7767517\n2 2\nInput input 0 1 data 0=4 1=3 2=2\n"
    assert np.array_equal(run(head + "Permute p 1 1 data output 0=2\n", y), y.transpose(1, 0, 2))
    assert np.array_equal(run(head + "Permute p 1 1 data output 0=4\n", y), y.transpose(2, 0, 1))


def test_gelu_and_prelu_by_hand(oracle, tmp_path):
    """GELU erf form (x * erfc(-x/sqrt 2)) * 0.5 against the closed form in double; PReLU = leaky ReLU with the
    stored slope; both reject what the reference's importers reject."""
    import math
    x = np.array([-10, -8, -6, -5, -4, -3, -2, -1, 0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 0.5], F32).reshape(2, 2, 5)
    got = _run_fixture(oracle, "gelu", x).reshape(-1)
    want = [0.5 * float(v) * (1.0 + math.erf(float(v) / math.sqrt(2.0))) for v in x.reshape(-1)]
    assert np.max(np.abs(got - np.array(want))) <= 1e-6
    (tmp_path / "m.bin").write_bytes(np.float32(-0.5).tobytes())
    p = tmp_path / "m.param"
    p.write_text("7767517\n2 2\nInput input 0 1 data 0=5 1=2 2=2\nPReLU prelu 1 1 data output 0=1\n")
    got = oracle.Model(str(p), str(tmp_path / "m.bin")).run([x])[0]
    assert np.array_equal(got, np.where(x >= 0, x, x * F32(-0.5)))
    p.write_text("7767517\n2 2\nInput input 0 1 data 0=5 1=2 2=2\nGELU gelu 1 1 data output 0=1\n")
    with pytest.raises(ValueError):
        oracle.Model(str(p), str(tmp_path / "m.bin")).run([x])


def test_deconvolution_by_hand(oracle):
    """2x2 stride-2 transposed convolution with the reference's literal weights (generate_bins.py:62-78) and its
    test input (supported_ops_test.cpp:569-599): out[2h+a, 2w+b, o] = bias[o] + sum_c x[c,h,w] * W[o,c,a,b], ReLU."""
    x = np.array([(i + 1) * (0.25 if i % 2 == 0 else -0.20) for i in range(12)], F32).reshape(2, 2, 3)  # [c,h,w]
    got = _run_fixture(oracle, "deconvolution", x)
    w = np.array([0.10, 0.20, 0.30, 0.40, -0.50, -0.60, -0.70, -0.80, -0.15, 0.25, -0.35, 0.45, 0.55, -0.65, 0.75, -0.85],
                 np.float64).reshape(2, 2, 2, 2)
    bias = np.array([-0.05, 0.10])
    want = np.zeros((2, 4, 6))
    for o in range(2):
        for h in range(2):
            for ww in range(3):
                for a in range(2):
                    for b in range(2):
                        want[o, 2 * h + a, 2 * ww + b] = bias[o] + sum(float(x[c, h, ww]) * w[o, c, a, b] for c in range(2))
    want = np.maximum(want, 0)
    assert got.shape == (2, 4, 6) and np.max(np.abs(got - want)) <= 1e-6
    assert np.all(got >= 0) and np.any(got == 0) and np.any(got > 0)   # what the reference's test also asserts
    assert _run_fixture(oracle, "deconvolution_tiny_head", np.ones((16, 2, 2), F32)).shape == (1, 4, 4)


def test_adaptive_pooling_by_hand(oracle, tmp_path):
    """Adaptive windows [floor(o*in/out), ceil((o+1)*in/out)) (NCNNToTosa.cpp:1706-1745): 5 -> 3 gives [0,2) [1,4) [3,5)."""
    x = np.arange(2 * 5 * 4, dtype=F32).reshape(2, 5, 4)
    p = tmp_path / "a.param"
    (tmp_path / "a.bin").write_bytes(b"")

    def run(params):
        p.write_text(f"7767517\n2 2\nInput input 0 1 data 0=4 1=5 2=2\nPooling pool 1 1 data output {params}\n")
        return oracle.Model(str(p), str(tmp_path / "a.bin")).run([x])[0]

    got = run("0=1 7=1 8=2 18=3")
    rows = [(0, 2), (1, 4), (3, 5)]
    want = np.stack([np.stack([x[:, a:b, c:d].mean(axis=(1, 2)) for c, d in [(0, 2), (2, 4)]], -1) for a, b in rows], 1)
    assert got.shape == (2, 3, 2) and np.allclose(got, want, rtol=0, atol=1e-6)
    got = run("0=0 7=1 8=-233 18=1")   # width kept, height pooled to one row
    assert got.shape == (2, 1, 4) and np.array_equal(got, x.max(axis=1, keepdims=True))
    with pytest.raises(ValueError):
        run("0=0 7=1 8=0 18=0")
