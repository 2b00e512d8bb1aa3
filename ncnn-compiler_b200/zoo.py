"""Synthetic ncnn models for the benchmark configurations.

Writes ordinary ncnn ``.param`` text and ``.bin`` weight files (the format read by
the reference's lib/Graph/graph.cpp:2129-2333 and by this runtime's loader) for
the topologies the benchmark names: one 3x3 convolution layer, a ResNet-18
topology (fp32 and int8-quantised), a MobileNetV2 topology, and single
InnerProduct layers.  Weights are drawn from seeded NumPy generators; no
third-party model file is reproduced.
"""
from __future__ import annotations

import os
import struct

import numpy as np

INT8_TAG = 0x000D4B38


class _Writer:
    def __init__(self):
        self.lines = []
        self.blobs = 0
        self.bin = bytearray()

    def layer(self, type_, name, bottoms, tops, params=""):
        self.blobs += len(tops)
        parts = [f"{type_:<24}", f"{name:<24}", str(len(bottoms)), str(len(tops)), *bottoms, *tops]
        if params:
            parts.append(params)
        self.lines.append(" ".join(parts))

    def f32(self, a, tagged=False):
        if tagged:
            self.bin += struct.pack("<I", 0)
        self.bin += np.ascontiguousarray(a, np.float32).tobytes()

    def i8(self, a):
        payload = np.ascontiguousarray(a, np.int8).tobytes()
        self.bin += struct.pack("<I", INT8_TAG) + payload + bytes((-len(payload)) % 4)

    def save(self, prefix):
        os.makedirs(os.path.dirname(os.path.abspath(prefix)), exist_ok=True)
        with open(prefix + ".param", "w") as f:
            f.write("7767517\n")
            f.write(f"{len(self.lines)} {self.blobs}\n")
            f.write("\n".join(self.lines) + "\n")
        with open(prefix + ".bin", "wb") as f:
            f.write(bytes(self.bin))
        return prefix + ".param", prefix + ".bin"


def quantize_rha(x, scale):
    """ncnn round-half-away-from-zero evaluated in fp32, clamped to [-127, 127]."""
    v = (np.asarray(x, np.float32) * np.float32(scale)).astype(np.float32)
    r = np.where(v >= 0, np.floor((v + np.float32(0.5)).astype(np.float32)),
                 np.ceil((v + np.float32(-0.5)).astype(np.float32)))
    return np.clip(r, -127, 127).astype(np.int8)


class _Net:
    """Small helper that emits conv-style layers in fp32 or int8-quantised form."""

    def __init__(self, seed, int8=False):
        self.w = _Writer()
        self.rng = np.random.default_rng(seed)
        self.int8 = int8
        self.pending_scale = None  # s_out promised by the previous term-101 layer

    def _he(self, shape, fan_in):
        return (self.rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)

    def _quant_tail(self, w2d, term):
        """Appends per-output weight scales, the input scale and (term > 100) the
        output scale; returns the int8 weights."""
        absmax = np.abs(w2d).max(axis=1)
        ws = np.where(absmax > 0, np.float32(127.0) / absmax, np.float32(1.0)).astype(np.float32)
        wq = np.stack([quantize_rha(w2d[o], ws[o]) for o in range(w2d.shape[0])])
        return wq, ws

    def conv(self, name, bottom, top, cin, cout, k, stride, pad, act=0, bias=None, term=0,
             weights=None, zero_bias=True):
        w = weights if weights is not None else self._he((cout, cin, k, k), cin * k * k)
        b = bias if bias is not None else (np.zeros(cout, np.float32) if zero_bias else
                                           (self.rng.standard_normal(cout) * 0.01).astype(np.float32))
        p = f"0={cout} 1={k} 3={stride} 4={pad} 5=1 6={w.size}"
        if act:
            p += f" 9={act}"
        if self.int8:
            p += f" 8={term}"
            wq, ws = self._quant_tail(w.reshape(cout, -1), term)
            s_in = self.pending_scale if self.pending_scale is not None else np.float32(self.rng.uniform(8, 64))
            self.w.layer("Convolution", name, [bottom], [top], p)
            self.w.i8(wq)
            self.w.f32(b)
            self.w.f32(ws)
            self.w.f32([s_in])
            if term > 100:
                s_out = np.float32(self.rng.uniform(8, 64))
                self.w.f32([s_out])
                self.pending_scale = s_out
            else:
                self.pending_scale = None
        else:
            self.w.layer("Convolution", name, [bottom], [top], p)
            self.w.f32(w, tagged=True)
            self.w.f32(b)

    def depthwise(self, name, bottom, top, ch, k, stride, pad):
        w = self._he((ch, 1, k, k), k * k)
        self.w.layer("ConvolutionDepthWise", name, [bottom], [top],
                     f"0={ch} 1={k} 3={stride} 4={pad} 5=1 6={w.size} 7={ch}")
        self.w.f32(w, tagged=True)
        self.w.f32(np.zeros(ch, np.float32))

    def inner_product(self, name, bottom, top, k, n, act=0, std=0.01, bias_std=0.0):
        w = (self.rng.standard_normal((n, k)) * std).astype(np.float32)
        b = (self.rng.standard_normal(n) * bias_std).astype(np.float32) if bias_std else np.zeros(n, np.float32)
        p = f"0={n} 1=1 2={w.size}"
        if act:
            p += f" 9={act}"
        if self.int8:
            p += " 8=1"
            wq, ws = self._quant_tail(w, 1)
            s_in = np.float32(self.rng.uniform(8, 64))
            self.w.layer("InnerProduct", name, [bottom], [top], p)
            self.w.i8(wq)
            self.w.f32(b)
            self.w.f32(ws)
            self.w.f32([s_in])
        else:
            self.w.layer("InnerProduct", name, [bottom], [top], p)
            self.w.f32(w, tagged=True)
            self.w.f32(b)


def single_conv(prefix, seed=100, h=56, w=56, cin=64, cout=64, k=3, stride=1, pad=1, relu=True):
    """Config 0: Input -> Convolution(3x3, bias, fused ReLU).  Weights N(0, 0.05^2), bias N(0, 0.01^2)."""
    net = _Net(seed)
    net.w.layer("Input", "input", [], ["data"], f"0={w} 1={h} 2={cin}")
    wt = (net.rng.standard_normal((cout, cin, k, k)) * 0.05).astype(np.float32)
    b = (net.rng.standard_normal(cout) * 0.01).astype(np.float32)
    net.conv("conv", "data", "output", cin, cout, k, stride, pad, act=1 if relu else 0, bias=b, weights=wt)
    return net.w.save(prefix)


def residual_block(prefix, seed=600, h=16, w=16, c=64, cout=96, k=3):
    """Input -> [k x k conv + ReLU -> k x k conv] + identity -> ReLU -> 1x1 conv to `cout` channels.
    With c a multiple of 64 every tensor-core operand is a bf16 pair: the first convolution writes
    one, the second adds a bf16-pair residual and writes one, the last writes plain fp32."""
    net = _Net(seed)
    wr = net.w
    wr.layer("Input", "input", [], ["data"], f"0={w} 1={h} 2={c}")
    wr.layer("Split", "split", ["data"], ["a", "b"])
    net.conv("conv1", "a", "c1", c, c, k, 1, k // 2, act=1, zero_bias=False)
    net.conv("conv2", "c1", "c2", c, c, k, 1, k // 2, act=0, zero_bias=False)
    wr.layer("Eltwise", "add", ["c2", "b"], ["sum"], "0=1")
    wr.layer("ReLU", "relu", ["sum"], ["act"], "0=0.0")
    net.conv("conv3", "act", "output", c, cout, 1, 1, 0, act=0, zero_bias=False)
    return wr.save(prefix)


def fire_classifier(prefix, seed=700, size=32, classes=10, act="ReLU"):
    """SqueezeNet-style stand-in for the operators next to the hot path: stem convolution, two
    fire modules (1x1 squeeze, 1x1 and 3x3 expand joined by a channel Concat), Dropout, a 1x1
    classifier convolution, global average pooling and Softmax.  `act` names the activation
    layer placed after every convolution (ReLU, Swish, HardSwish, Sigmoid, TanH)."""
    net = _Net(seed)
    wr = net.w

    def activation(name, bottom, top):
        extra = "0=0.166667 1=0.5" if act in ("HardSwish", "HardSigmoid") else ("0=0.0" if act == "ReLU" else "")
        wr.layer(act, name, [bottom], [top], extra)

    wr.layer("Input", "input", [], ["data"], f"0={size} 1={size} 2=3")
    net.conv("conv1", "data", "c1", 3, 64, 3, 2, 1, zero_bias=False)
    activation("act1", "c1", "a1")
    cur, cin = "a1", 64
    for k, (sq, ex) in enumerate([(16, 64), (32, 128)]):
        tag = f"fire{k + 1}"
        net.conv(f"{tag}_squeeze", cur, f"{tag}_s", cin, sq, 1, 1, 0, zero_bias=False)
        activation(f"{tag}_sa", f"{tag}_s", f"{tag}_sq")
        wr.layer("Split", f"{tag}_split", [f"{tag}_sq"], [f"{tag}_l", f"{tag}_r"])
        net.conv(f"{tag}_e1", f"{tag}_l", f"{tag}_e1c", sq, ex, 1, 1, 0, zero_bias=False)
        activation(f"{tag}_e1a", f"{tag}_e1c", f"{tag}_e1o")
        net.conv(f"{tag}_e3", f"{tag}_r", f"{tag}_e3c", sq, ex, 3, 1, 1, zero_bias=False)
        activation(f"{tag}_e3a", f"{tag}_e3c", f"{tag}_e3o")
        wr.layer("Concat", f"{tag}_cat", [f"{tag}_e1o", f"{tag}_e3o"], [f"{tag}_out"], "0=0")
        cur, cin = f"{tag}_out", 2 * ex
    wr.layer("Dropout", "drop", [cur], ["dropped"], "0=0.5")
    net.conv("classifier", "dropped", "logits", cin, classes, 1, 1, 0, zero_bias=False)
    wr.layer("Pooling", "gap", ["logits"], ["pooled"], "0=1 4=1")
    wr.layer("Softmax", "prob", ["pooled"], ["output"], "0=0 1=1")
    return wr.save(prefix)


def resnet18(prefix, seed=200, int8=False, size=224, classes=1000):
    """Configs 1 and 3: ResNet-18 topology, BatchNorm folded (zero bias), He-normal weights."""
    net = _Net(seed if not int8 else seed + 200, int8=int8)
    w = net.w
    w.layer("Input", "input", [], ["data"], f"0={size} 1={size} 2=3")
    net.conv("conv1", "data", "conv1", 3, 64, 7, 2, 3, act=1, term=1)
    w.layer("Pooling", "pool1", ["conv1"], ["pool1"], "0=0 1=3 2=2 3=1 5=1")
    cur, cin = "pool1", 64
    for stage, cout in enumerate([64, 128, 256, 512]):
        for block in range(2):
            stride = 2 if (stage > 0 and block == 0) else 1
            tag = f"l{stage + 1}b{block}"
            w.layer("Split", f"{tag}_split", [cur], [f"{tag}_a", f"{tag}_b"])
            net.conv(f"{tag}_conv1", f"{tag}_a", f"{tag}_c1", cin, cout, 3, stride, 1, act=1, term=101)
            net.conv(f"{tag}_conv2", f"{tag}_c1", f"{tag}_c2", cout, cout, 3, 1, 1, act=0, term=1)
            shortcut = f"{tag}_b"
            if stride != 1 or cin != cout:
                net.conv(f"{tag}_down", f"{tag}_b", f"{tag}_sc", cin, cout, 1, stride, 0, act=0, term=1)
                shortcut = f"{tag}_sc"
            w.layer("Eltwise", f"{tag}_add", [f"{tag}_c2", shortcut], [f"{tag}_sum"], "0=1")
            w.layer("ReLU", f"{tag}_relu", [f"{tag}_sum"], [f"{tag}_out"], "0=0.0")
            cur, cin = f"{tag}_out", cout
    w.layer("Pooling", "gap", [cur], ["gap"], "0=1 4=1")
    net.inner_product("fc", "gap", "output", 512, classes, std=0.01)
    return w.save(prefix)


def mobilenet_v2(prefix, seed=300, size=224, classes=1000):
    """Config 2: MobileNetV2 topology; ReLU6 written as Clip 0..6 layers."""
    net = _Net(seed)
    w = net.w
    w.layer("Input", "input", [], ["data"], f"0={size} 1={size} 2=3")

    def relu6(name, bottom, top):
        w.layer("Clip", name, [bottom], [top], "0=0.0 1=6.0")

    net.conv("stem", "data", "stem", 3, 32, 3, 2, 1)
    relu6("stem_relu6", "stem", "stem_a")
    cur, cin = "stem_a", 32
    cfg = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2),
           (6, 320, 1, 1)]
    idx = 0
    for t, c, n, s in cfg:
        for i in range(n):
            stride = s if i == 0 else 1
            tag = f"b{idx}"
            idx += 1
            residual = stride == 1 and cin == c
            src = cur
            if residual:
                w.layer("Split", f"{tag}_split", [cur], [f"{tag}_x", f"{tag}_id"])
                src = f"{tag}_x"
            hidden = cin * t
            if t != 1:
                net.conv(f"{tag}_expand", src, f"{tag}_e", cin, hidden, 1, 1, 0)
                relu6(f"{tag}_expand_relu6", f"{tag}_e", f"{tag}_ea")
                src = f"{tag}_ea"
            net.depthwise(f"{tag}_dw", src, f"{tag}_d", hidden, 3, stride, 1)
            relu6(f"{tag}_dw_relu6", f"{tag}_d", f"{tag}_da")
            net.conv(f"{tag}_project", f"{tag}_da", f"{tag}_p", hidden, c, 1, 1, 0)
            cur = f"{tag}_p"
            if residual:
                w.layer("Eltwise", f"{tag}_add", [f"{tag}_p", f"{tag}_id"], [f"{tag}_o"], "0=1")
                cur = f"{tag}_o"
            cin = c
    net.conv("last", cur, "last", cin, 1280, 1, 1, 0)
    relu6("last_relu6", "last", "last_a")
    w.layer("Pooling", "gap", ["last_a"], ["gap"], "0=1 4=1")
    net.inner_product("fc", "gap", "output", 1280, classes, std=float(np.sqrt(2.0 / 1280)))
    return w.save(prefix)


def inverted_residual(prefix, h, w, cin, hidden, cout, stride=1, seed=310, expand_bias=True):
    """One MobileNetV2 block on its own: 1x1 expand + ReLU6, 3x3 depthwise (stride 1 or 2) + ReLU6, 1x1 projection,
    and the residual add when stride and channel counts allow it."""
    net = _Net(seed)
    wr = net.w
    wr.layer("Input", "input", [], ["data"], f"0={w} 1={h} 2={cin}")
    residual = stride == 1 and cin == cout
    src = "data"
    if residual:
        wr.layer("Split", "split", ["data"], ["x", "id"])
        src = "x"
    net.conv("expand", src, "e", cin, hidden, 1, 1, 0, zero_bias=not expand_bias)
    wr.layer("Clip", "expand_relu6", ["e"], ["ea"], "0=0.0 1=6.0")
    net.depthwise("dw", "ea", "d", hidden, 3, stride, 1)
    wr.layer("Clip", "dw_relu6", ["d"], ["da"], "0=0.0 1=6.0")
    net.conv("project", "da", "p" if residual else "output", hidden, cout, 1, 1, 0, zero_bias=False)
    if residual:
        wr.layer("Eltwise", "add", ["p", "id"], ["output"], "0=1")
    return wr.save(prefix)


def detection_head(prefix, seed=900, h=8, w=8, cin=32, anchors=3, values=7):
    """A YOLOv5-style head: 1x1 convolution to anchors * values channels, Reshape to the rank-4 tensor
    [anchors, values, h, w], Permute (order 3) to [anchors, h, w, values], Sigmoid, Slice of the value axis into
    (box, rest), Reshape of both to matrices [anchors * h * w, n] and Concat back along the width."""
    net = _Net(seed)
    wr = net.w
    wr.layer("Input", "input", [], ["data"], f"0={w} 1={h} 2={cin}")
    net.conv("head", "data", "raw", cin, anchors * values, 1, 1, 0, act=0, zero_bias=False)
    wr.layer("Reshape", "to_rank4", ["raw"], ["grid"], f"0={w} 1={h} 11={values} 2={anchors}")
    wr.layer("Permute", "values_last", ["grid"], ["cells"], "0=3")
    wr.layer("Sigmoid", "sigmoid", ["cells"], ["prob"], "")
    wr.layer("Slice", "split_values", ["prob"], ["box", "rest"], f"-23300=2,4,-233 1=3")
    wr.layer("Reshape", "box_rows", ["box"], ["box_m"], "0=4 1=-1")
    wr.layer("Reshape", "rest_rows", ["rest"], ["rest_m"], f"0={values - 4} 1=-1")
    wr.layer("Concat", "join", ["box_m", "rest_m"], ["output"], "0=1")
    return wr.save(prefix)


def inner_product(prefix, k, n, seed=500, int8=False, relu=True):
    """Config 4: Input [1,1,K] -> InnerProduct(K -> N, bias, fused ReLU); run with batch M."""
    net = _Net(seed + (7 if int8 else 0), int8=int8)
    net.w.layer("Input", "input", [], ["data"], f"0={k} 1=1 2=1")
    net.inner_product("ip", "data", "output", k, n, act=1 if relu else 0, std=0.02, bias_std=0.01)
    return net.w.save(prefix)


def dynamic_convnet(prefix, seed=800, cin=3, classes=0):
    """A network whose Input carries no dimensions (compile with `--input-shape=3x?x?`): 3x3 stride-2
    stem, two 3x3 convolutions around a residual add, then either a 1x1 convolution to 8 channels
    (classes=0: the result follows the input size, [8, H/2, W/2]) or global average pooling and an
    InnerProduct (classes>0: a fixed [classes] result)."""
    net = _Net(seed)
    wr = net.w
    wr.layer("Input", "input", [], ["data"], "0=0 1=0 2=0")
    net.conv("stem", "data", "s", cin, 32, 3, 2, 1, act=1, zero_bias=False)
    wr.layer("Split", "split", ["s"], ["a", "b"])
    net.conv("conv1", "a", "c1", 32, 32, 3, 1, 1, act=1, zero_bias=False)
    net.conv("conv2", "c1", "c2", 32, 32, 3, 1, 1, act=0, zero_bias=False)
    wr.layer("Eltwise", "add", ["c2", "b"], ["sum"], "0=1")
    wr.layer("ReLU", "relu", ["sum"], ["act"], "0=0.0")
    if classes:
        wr.layer("Pooling", "gap", ["act"], ["pooled"], "0=1 4=1")
        net.inner_product("fc", "pooled", "output", 32, classes, std=0.1, bias_std=0.01)
    else:
        net.conv("head", "act", "output", 32, 8, 1, 1, 0, act=0, zero_bias=False)
    return wr.save(prefix)


def gemm(prefix, m, k, n, alpha=0.5, beta=-1.25, seed=510):
    """Gemm in the one form the reference lowers (dynamic A [M,K], constant transposed B [N,K], constant
    row bias C [N]): y = (A * B^T + beta * C) * alpha.  Run with any batch; each image is one [M,K] matrix."""
    net = _Net(seed)
    wr = net.w
    wr.layer("Input", "input", [], ["data"], f"0={k} 1=1 2={m}")
    wr.layer("Squeeze", "squeeze", ["data"], ["matrix"], "-23303=1,1")
    wr.layer("Gemm", "gemm", ["matrix"], ["output"], f"0={alpha!r} 1={beta!r} 3=1 5=1 6=1 8={n} 9={k} 10=4")
    wr.f32((net.rng.standard_normal((n, k)) * 0.02).astype(np.float32), tagged=True)
    wr.f32((net.rng.standard_normal(n) * 0.01).astype(np.float32), tagged=True)
    return wr.save(prefix)


def conv_batchnorm(prefix, kind="conv", c=64, cout=64, h=14, w=14, eps=1e-5, zero_var_channels=(), bias=True,
                   int8=False, seed=900):
    """Input -> Convolution | ConvolutionDepthWise (3x3, no activation) -> BatchNorm -> ReLU.  The reference folds
    the BatchNorm into an fp32 convolution and leaves it alone after a quantised one.  Channels listed in
    `zero_var_channels` get variance 0 (with eps = 0 they take the reference's 10000 branch)."""
    net = _Net(seed, int8=int8)
    wr = net.w
    wr.layer("Input", "input", [], ["data"], f"0={w} 1={h} 2={c}")
    if kind == "depthwise":
        cout = c
        net.depthwise("dw", "data", "x", c, 3, 1, 1)
    else:
        wt = net._he((cout, c, 3, 3), c * 9)
        if bias:
            net.conv("conv", "data", "x", c, cout, 3, 1, 1, act=0, zero_bias=False, term=1 if int8 else 0, weights=wt)
        else:
            wr.layer("Convolution", "conv", ["data"], ["x"], f"0={cout} 1=3 3=1 4=1 5=0 6={wt.size}")
            wr.f32(wt, tagged=True)
    rng = net.rng
    slope = rng.uniform(0.5, 1.5, cout).astype(np.float32)
    mean = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    var = rng.uniform(0.5, 2.0, cout).astype(np.float32)
    for ch in zero_var_channels:
        var[ch] = 0.0
    beta = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    wr.layer("BatchNorm", "bn", ["x"], ["y"], f"0={cout} 1={float(eps)!r}")
    for a in (slope, mean, var, beta):
        wr.f32(a)
    wr.layer("ReLU", "relu", ["y"], ["output"], "0=0.0")
    return wr.save(prefix)
