"""TEST INFRASTRUCTURE ONLY -- CPU oracle for the hot path of hqu-little-boy/ncnn-compiler.

This module restates, operation for operation, what the reference's lowering
(lib/Conversion/NCNNToTosa/NCNNToTosa.cpp) makes of an ncnn ``.param``/``.bin``
graph for the operators on the hot path: Convolution, ConvolutionDepthWise,
InnerProduct, Gemm, Pooling, Eltwise/BinaryOp, ReLU (and the Clip extension),
Quantize/Dequantize/Requantize and BatchNorm folding.  Only tests, the smoke
check and the bench's cpu_baseline/reference legs may import it; the product
never does.

Parity status: "parity unpinned" for values -- the reference stores no golden
outputs (its numerical tests call upstream ncnn at test time,
test/Numerical/support/numerical_test_support.cpp:542-699) and its LLVM/MLIR 21
toolchain cannot run here.  What pins this file: (1) the loader is checked
against the reference's own lib/Graph code compiled as oracle/_ref, (2) every
function cites the lowering it follows, (3) hand-derived known answers for the
reference's fixtures live in tests/golden.

Heavy loops run in oracle/ncnn_ops.c (plain C, no fast-math); element-wise
steps run in numpy float32, which performs the same single IEEE operations the
reference's arith ops do (no FMA contraction).
"""
from __future__ import annotations

import ctypes
import os
import struct
import subprocess
from dataclasses import dataclass, field

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libncnn_oracle.so")
_FAST_LIB_PATH = os.path.join(_HERE, "libncnn_oracle_fast.so")
_lib = None

F32 = np.float32


def build(force: bool = False, fast: bool = False) -> str:
    """Compiles ncnn_ops.c (gcc, no fast-math, no contraction, OpenMP).  The checker is the -O2 build
    libncnn_oracle.so; `fast` builds libncnn_oracle_fast.so with -O3 -march=native for the timed CPU arm of
    the benchmark (same source, same fp32 semantics: contraction and fast-math stay off)."""
    src = os.path.join(_HERE, "ncnn_ops.c")
    out = _FAST_LIB_PATH if fast else _LIB_PATH
    if force or not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(src):
        opt = ["-O3", "-march=native"] if fast else ["-O2"]
        subprocess.check_call(
            ["gcc", *opt, "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC",
             "-o", out, src, "-lm"])
    return out


def use_fast_library() -> str:
    """Switches this process to the -O3 -march=native build (benchmark arm only; tests keep the checker).
    The library is compiled on the machine that runs it, since -march=native binds it to that CPU."""
    global _lib
    path = build(fast=True, force=not _built_here(_FAST_LIB_PATH))
    _lib = ctypes.CDLL(path)
    return path


def _built_here(path: str) -> bool:
    """True when `path` was compiled by this host (a marker file holds the host's CPU model)."""
    marker = path + ".host"
    try:
        with open("/proc/cpuinfo") as f:
            model = next((l.split(":", 1)[1].strip() for l in f if l.startswith("model name")), "unknown")
    except OSError:
        model = "unknown"
    try:
        with open(marker) as f:
            same = f.read() == model
    except OSError:
        same = False
    if not same:
        with open(marker, "w") as f:
            f.write(model)
    return same and os.path.exists(path)


def _ops():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


_libm = None


def _powf(x: float, y: float) -> float:
    """powf of the C library (single precision in, single precision out)."""
    global _libm
    if _libm is None:
        import ctypes.util
        _libm = ctypes.CDLL(ctypes.util.find_library("m") or "libm.so.6")
        _libm.powf.restype = ctypes.c_float
        _libm.powf.argtypes = [ctypes.c_float, ctypes.c_float]
    return float(_libm.powf(x, y))


def _p(a, t):
    return a.ctypes.data_as(ctypes.POINTER(t))


# --------------------------------------------------------------------------- .param / .bin
# Grammar: lib/Graph/parser.cpp:33-44,138-198 (lexical typing), :91-108 (array ids),
# lib/Graph/graph.cpp:2129-2333 (file structure).

def _is_float_token(tok: str) -> bool:
    t = tok.lstrip("+-").lower()
    return t in ("nan", "inf", "infinity") or any(ch in tok for ch in ".eE")


def parse_param_value(tok: str, explicit_array: bool):
    if not explicit_array and tok.startswith('"'):
        return tok[1:-1]
    parts = tok.split(",")
    if explicit_array:
        n = int(parts[0])
        if n != len(parts) - 1:
            raise ValueError("array length mismatch")
        parts = parts[1:]
        if any(_is_float_token(p) for p in parts):
            return [float(np.float32(p)) for p in parts]
        return [int(p) for p in parts]
    if len(parts) > 1:
        if any(_is_float_token(p) for p in parts):
            return [float(np.float32(p)) for p in parts]
        return [int(p) for p in parts]
    if tok[0].isalpha() and not _is_float_token(tok):
        return tok
    if _is_float_token(tok):
        return float(np.float32(tok))
    return int(tok)


def parse_layer_params(tokens):
    params = {}
    for tok in tokens:
        key, _, val = tok.partition("=")
        pid = int(key)
        explicit = False
        if pid <= -23300:
            pid = -pid - 23300
            explicit = True
        params[pid] = parse_param_value(val, explicit)
    return params


@dataclass
class Layer:
    type: str
    name: str
    bottoms: list
    tops: list
    params: dict
    weights: list = field(default_factory=list)

    def geti(self, pid, default=0):
        v = self.params.get(pid, default)
        return int(v)

    def getf(self, pid, default=0.0):
        return float(self.params.get(pid, default))


class _Bin:
    def __init__(self, data: bytes):
        self.data = data
        self.pos = 0

    def read(self, count: int, typed: int):
        """load_weight (lib/Graph/graph.cpp:1260-1327): typed 0 reads a 4-byte storage
        flag first; fp16/int8 payloads are padded to 4 bytes."""
        if typed == 0:
            (flag,) = struct.unpack_from("<I", self.data, self.pos)
            self.pos += 4
            if flag == 0x01306B47:
                a = np.frombuffer(self.data, np.float16, count, self.pos).astype(F32)
                self.pos += 2 * count
                self.pos += (-self.pos) % 4
                return a
            if flag == 0x000D4B38:
                a = np.frombuffer(self.data, np.int8, count, self.pos).copy()
                self.pos += count
                self.pos += (-self.pos) % 4
                return a
            if flag not in (0, 0x0002C056):
                raise ValueError(f"unsupported weight flag 0x{flag:08x}")
        a = np.frombuffer(self.data, F32, count, self.pos).copy()
        self.pos += 4 * count
        return a


def _load_weights(layer: Layer, b: _Bin):
    t = layer.type
    if t in ("Convolution", "ConvolutionDepthWise"):
        # graph.cpp:1381-1478 / :1480-1571
        nout, wsize, term = layer.geti(0), layer.geti(6), layer.geti(8)
        layer.weights.append(b.read(wsize, 0))
        if layer.geti(5):
            layer.weights.append(b.read(nout, 1))
        if term:
            if t == "Convolution":
                nscale = nout
            else:
                nscale = layer.geti(7, 1) if term in (1, 101) else 1
            layer.weights.append(b.read(nscale, 1))
            layer.weights.append(b.read(1, 1))
        if term > 100:
            layer.weights.append(b.read(1, 1))
    elif t == "InnerProduct":
        nout, wsize, term = layer.geti(0), layer.geti(2), layer.geti(8)
        layer.weights.append(b.read(wsize, 0))
        if layer.geti(1):
            layer.weights.append(b.read(nout, 1))
        if term:
            layer.weights.append(b.read(nout, 1))
            layer.weights.append(b.read(1, 1))
    elif t == "BatchNorm":
        for _ in range(4):
            layer.weights.append(b.read(layer.geti(0), 1))
    elif t == "Gemm":
        # graph.cpp:1858-1926: constant B [N,K] (transB=1), optional row bias C, int8 scale
        if layer.geti(5) and layer.geti(6):
            n, k = layer.geti(8), layer.geti(9)
            layer.weights.append(b.read(n * k, 0))
            if layer.geti(10, 0) == 4:
                layer.weights.append(b.read(n, 0))
            if layer.geti(18):
                layer.weights.append(b.read(1, 1))
    elif t == "Deconvolution":
        # load_deconvolution_weights (graph.cpp:1573-1636): [O, I, kh, kw] then the bias
        nout, wsize = layer.geti(0), layer.geti(6)
        layer.weights.append(b.read(wsize, 0))
        if layer.geti(5):
            layer.weights.append(b.read(nout, 1))
    elif t == "PReLU":
        # load_prelu_weights (graph.cpp:1697-1709)
        if layer.geti(0, 0) <= 0:
            raise ValueError("PReLU num_slope must be positive")
        layer.weights.append(b.read(layer.geti(0), 1))
    elif t == "Quantize":
        layer.weights.append(b.read(layer.geti(0, 1), 1))
    elif t == "Dequantize":
        layer.weights.append(b.read(layer.geti(0, 1), 1))
        if layer.geti(1):
            layer.weights.append(b.read(layer.geti(1), 1))
    elif t == "Requantize":
        layer.weights.append(b.read(layer.geti(0, 1), 1))
        layer.weights.append(b.read(layer.geti(1, 1), 1))
        if layer.geti(2):
            layer.weights.append(b.read(layer.geti(2), 1))


def load_graph(param_path: str, bin_path: str | None):
    with open(param_path) as f:
        lines = [ln for ln in f.read().splitlines()]
    while lines and not lines[-1].strip():
        lines.pop()
    idx = 0
    first = lines[0].split()
    if len(first) == 1:
        if int(first[0]) != 7767517:
            raise ValueError("param magic mismatch (expected 7767517)")
        idx = 1
    nlayers, nblobs = (int(t) for t in lines[idx].split())
    idx += 1
    layers = []
    for i in range(nlayers):
        tok = lines[idx + i].split()
        nb, nt = int(tok[2]), int(tok[3])
        layers.append(Layer(tok[0], tok[1], tok[4:4 + nb], tok[4 + nb:4 + nb + nt],
                            parse_layer_params(tok[4 + nb + nt:])))
    if bin_path:
        with open(bin_path, "rb") as f:
            b = _Bin(f.read())
        for layer in layers:
            _load_weights(layer, b)
        if b.pos != len(b.data):
            raise ValueError(f"bin size mismatch: consumed {b.pos} bytes of {len(b.data)}")
    return layers


# --------------------------------------------------------------------------- arithmetic

def quantize(x: np.ndarray, scale: np.ndarray, axis: int | None = None) -> np.ndarray:
    """quantizeSignedI8 (NCNNToTosa.cpp:322-389).  `axis` is the dimension the scale
    vector runs along (None: scalar scale)."""
    x = np.asarray(x, F32)
    scale = np.asarray(scale, F32).reshape(-1)
    if scale.size == 1 or axis is None:
        s = scale[0]
    else:
        shape = [1] * x.ndim
        shape[axis] = scale.size
        s = scale.reshape(shape)
    v = (x * s).astype(F32)
    pos = np.floor((v + F32(0.5)).astype(F32))
    neg = np.ceil((v + F32(-0.5)).astype(F32))
    r = np.where(v >= 0, pos, neg).astype(F32)
    r = np.maximum(np.minimum(r, F32(127.0)), F32(-127.0))
    return r.astype(np.int8)


def dequant_factor(weight_scale: np.ndarray, input_scale: np.ndarray) -> np.ndarray:
    """dequantizeAccumulator (NCNNToTosa.cpp:577-596): 1/(s_w*s_in), 0 where s_w == 0."""
    ws = np.asarray(weight_scale, F32).reshape(-1)
    combined = (ws * F32(np.asarray(input_scale, F32).reshape(-1)[0])).astype(F32)
    with np.errstate(divide="ignore"):
        r = (F32(1.0) / combined).astype(F32)
    return np.where(ws == 0, F32(0), r).astype(F32)


def conv_out_extent(inp, k, s, d, p0, p1):
    """computeConvResult (lib/Dialect/NCNN/IR/NCNNOps.cpp:181-207)."""
    if p0 in (-233, -234):
        return 1 + (inp - 1) // s
    return 1 + (inp + p0 + p1 - ((k - 1) * d + 1)) // s


def same_padding(inp, k, s, d, lower):
    """computeSamePadding (lib/Transforms/NormalizeNCNN/NormalizeNCNN.cpp:30-50)."""
    extent = d * (k - 1) + 1
    out = 1 + (inp - 1) // s
    total = max((out - 1) * s + extent - inp, 0)
    before = total // 2 + total % 2 if lower else total // 2
    return before, total - before


def pool_out_extent(inp, k, s, p0, p1, mode):
    """inferRegularDimension (NCNNOps.cpp:488-531)."""
    if mode in (2, 3):
        return 1 + (inp - 1) // s
    num = inp + p0 + p1
    if mode == 0:
        diff = num - k
        return (1 if diff % s == 0 else 2) + diff // s
    return 1 + (num - k) // s


def _conv_geometry(layer: Layer, H, W):
    kw = layer.geti(1); kh = layer.geti(11, kw)
    dw = layer.geti(2, 1); dh = layer.geti(12, dw)
    sw = layer.geti(3, 1); sh = layer.geti(13, sw)
    pl = layer.geti(4, 0); pr = layer.geti(15, pl); pt = layer.geti(14, pl); pb = layer.geti(16, pt)
    OH = conv_out_extent(H, kh, sh, dh, pt, pb)
    OW = conv_out_extent(W, kw, sw, dw, pl, pr)
    if pl in (-233, -234):
        lower = pl == -234
        pt, pb = same_padding(H, kh, sh, dh, lower)
        pl, pr = same_padding(W, kw, sw, dw, lower)
    return kh, kw, sh, sw, dh, dw, pt, pl, OH, OW


def _act(y, act_type, act_params=None):
    """Fused activation is split into its own op (ImportConvolution.cpp:236-246):
    1 -> relu clamp(x,0,inf) (ConvertRelu, NCNNToTosa.cpp:1532-1578); 3 -> clip
    (extension, not in the reference)."""
    if act_type == 0:
        return y
    if act_type == 1:
        if y.dtype == np.int8:
            return np.maximum(y, np.int8(0))
        return np.maximum(y, F32(0))
    if act_type == 2:
        slope = F32(act_params[0])
        return np.where(y >= 0, y, (y * slope).astype(F32)).astype(F32)
    if act_type == 3:
        return np.minimum(np.maximum(y, F32(act_params[0])), F32(act_params[1]))
    if act_type == 4:
        return op_sigmoid(y)
    raise ValueError(f"unsupported activation {act_type}")


def op_convolution(layer: Layer, x: np.ndarray) -> np.ndarray:
    """x: [H,W,C] f32 or int8.  ConvertConvolution (NCNNToTosa.cpp:1136-1528)."""
    L = _ops()
    H, W, C = x.shape
    O, term = layer.geti(0), layer.geti(8)
    kh, kw, sh, sw, dh, dw, pt, pl, OH, OW = _conv_geometry(layer, H, W)
    wts = layer.weights
    w = wts[0]
    bias = wts[1] if layer.geti(5) else None
    act = layer.geti(9)
    actp = layer.params.get(10)
    if term == 0:
        y = np.empty((OH, OW, O), F32)
        x = np.ascontiguousarray(x, F32)
        L.orc_conv2d_f32(_p(x, ctypes.c_float), H, W, C, _p(np.ascontiguousarray(w, F32), ctypes.c_float),
                         _p(bias, ctypes.c_float) if bias is not None else None, O, kh, kw, sh, sw,
                         pt, pl, dh, dw, OH, OW, _p(y, ctypes.c_float))
        return _act(y, act, actp)
    off = 1 + (1 if bias is not None else 0)
    ws, s_in = wts[off], wts[off + 1]
    xq = x if x.dtype == np.int8 else quantize(x, s_in)
    if w.dtype == np.int8:
        wq = w
    else:
        wq = quantize(w.reshape(O, -1), ws, 0 if ws.size > 1 else None).reshape(-1)
    acc = np.empty((OH, OW, O), np.int32)
    L.orc_conv2d_i8(_p(np.ascontiguousarray(xq), ctypes.c_int8), H, W, C,
                    _p(np.ascontiguousarray(wq), ctypes.c_int8), O, kh, kw, sh, sw, pt, pl, dh, dw,
                    OH, OW, _p(acc, ctypes.c_int32))
    y = (acc.astype(F32) * dequant_factor(ws, s_in)).astype(F32)
    if bias is not None:
        y = (y + bias.astype(F32)).astype(F32)
    if term > 100:
        y = quantize(y, wts[off + 2])
    return _act(y, act, actp)


def op_depthwise(layer: Layer, x: np.ndarray) -> np.ndarray:
    """ConvertDepthwiseConvolution (NCNNToTosa.cpp:3074-3503); group == channels."""
    L = _ops()
    H, W, C = x.shape
    O, term, group = layer.geti(0), layer.geti(8), layer.geti(7, 1)
    if not (group == C == O):
        raise ValueError("only pure depthwise (group == channels == num_output) is supported")
    kh, kw, sh, sw, dh, dw, pt, pl, OH, OW = _conv_geometry(layer, H, W)
    wts = layer.weights
    w = wts[0]
    bias = wts[1] if layer.geti(5) else None
    act = layer.geti(9)
    actp = layer.params.get(10)
    if term == 0:
        y = np.empty((OH, OW, C), F32)
        x = np.ascontiguousarray(x, F32)
        L.orc_depthwise_f32(_p(x, ctypes.c_float), H, W, C, _p(np.ascontiguousarray(w, F32), ctypes.c_float),
                            _p(bias, ctypes.c_float) if bias is not None else None, kh, kw, sh, sw,
                            pt, pl, dh, dw, OH, OW, _p(y, ctypes.c_float))
        return _act(y, act, actp)
    off = 1 + (1 if bias is not None else 0)
    ws, s_in = wts[off], wts[off + 1]
    xq = x if x.dtype == np.int8 else quantize(x, s_in)
    wq = w if w.dtype == np.int8 else quantize(w.reshape(C, -1), ws, 0 if ws.size > 1 else None).reshape(-1)
    acc = np.empty((OH, OW, C), np.int32)
    L.orc_depthwise_i8(_p(np.ascontiguousarray(xq), ctypes.c_int8), H, W, C,
                       _p(np.ascontiguousarray(wq), ctypes.c_int8), kh, kw, sh, sw, pt, pl, dh, dw,
                       OH, OW, _p(acc, ctypes.c_int32))
    y = (acc.astype(F32) * dequant_factor(ws, s_in)).astype(F32)
    if bias is not None:
        y = (y + bias.astype(F32)).astype(F32)
    if term > 100:
        y = quantize(y, wts[off + 2])
    return _act(y, act, actp)


def _matmul_f32(a, b):
    L = _ops()
    M, K = a.shape
    N = b.shape[0]
    y = np.empty((M, N), F32)
    L.orc_matmul_f32(_p(np.ascontiguousarray(a, F32), ctypes.c_float),
                     _p(np.ascontiguousarray(b, F32), ctypes.c_float), M, K, N, _p(y, ctypes.c_float))
    return y


def _matmul_i8(a, b):
    L = _ops()
    M, K = a.shape
    N = b.shape[0]
    y = np.empty((M, N), np.int32)
    L.orc_matmul_i8(_p(np.ascontiguousarray(a), ctypes.c_int8), _p(np.ascontiguousarray(b), ctypes.c_int8),
                    M, K, N, _p(y, ctypes.c_int32))
    return y


def op_inner_product(layer: Layer, x_chw_flat: np.ndarray) -> np.ndarray:
    """x_chw_flat: [M,K] rows flattened in CHW order (NCNNToTosa.cpp:5305-5337).
    y = x*W^T, then + bias (:5371-5381); int8: per-tensor input scale, per-output
    weight scale, y = float(acc)*r (+bias) (:5312-5319,5366-5370)."""
    O, term = layer.geti(0), layer.geti(8)
    wts = layer.weights
    K = wts[0].size // O
    w = wts[0].reshape(O, K)
    bias = wts[1] if layer.geti(1) else None
    if term == 0:
        y = _matmul_f32(x_chw_flat.reshape(-1, K), w)
    else:
        off = 1 + (1 if bias is not None else 0)
        ws, s_in = wts[off], wts[off + 1]
        xq = quantize(x_chw_flat.reshape(-1, K), s_in)
        wq = w if w.dtype == np.int8 else quantize(w, ws, 0)
        y = (_matmul_i8(xq, wq).astype(F32) * dequant_factor(ws, s_in)).astype(F32)
    if bias is not None:
        y = (y + bias.astype(F32)).astype(F32)
    return _act(y, layer.geti(9), layer.params.get(10))


def op_gemm(layer: Layer, a: np.ndarray) -> np.ndarray:
    """ConvertGemm (NCNNToTosa.cpp:4990-5109): y = (A*B^T + beta*C) * alpha; int8:
    per-row scale 127/absmax (1 if row is all zero), y = float(acc) / (s_row * s_B)."""
    alpha, beta = F32(layer.getf(0, 1.0)), F32(layer.getf(1, 1.0))
    n, k = layer.geti(8), layer.geti(9)
    wts = layer.weights
    b = wts[0].reshape(n, k)
    c = wts[1] if layer.geti(10, 0) == 4 else None
    a = np.asarray(a, F32).reshape(-1, k)
    if layer.geti(18) == 0:
        y = _matmul_f32(a, b)
    else:
        s_b = wts[-1]
        absmax = np.zeros(a.shape[0], F32)
        for col in range(a.shape[1]):  # running max, same order as the reduction
            absmax = np.maximum(np.abs(a[:, col]), absmax)
        with np.errstate(divide="ignore"):
            s_row = np.where(absmax == 0, F32(1), (F32(127.0) / absmax).astype(F32)).astype(F32)
        aq = quantize(a, s_row, 0)
        bq = b if b.dtype == np.int8 else quantize(b, s_b)
        acc = _matmul_i8(aq, bq).astype(F32)
        combined = (s_row * F32(s_b.reshape(-1)[0])).astype(F32)
        y = (acc / combined[:, None]).astype(F32)
    if c is not None:
        y = (y + (c.astype(F32) * beta).astype(F32)).astype(F32)
    if alpha != F32(1.0):
        y = (y * alpha).astype(F32)
    return y


def _adaptive_pooling(layer: Layer, x: np.ndarray, kind: int) -> np.ndarray:
    """Adaptive mode (ImportPooling.cpp:66-69; ConvertPooling NCNNToTosa.cpp:1706-1745,1768-1870): out_w = param 8,
    out_h = param 18 (default out_w), -233 keeps the input extent; window of output o on an axis is
    [floor(o*in/out), ceil((o+1)*in/out)); max, or the row-major sequential sum divided by rows*columns."""
    if x.dtype == np.int8:
        raise ValueError("dynamic or adaptive signed i8 pooling is not supported")
    H, W, C = x.shape
    out_w = layer.geti(8, 0)
    out_h = layer.geti(18, out_w)
    OH = H if out_h == -233 else out_h
    OW = W if out_w == -233 else out_w
    if OH <= 0 or OW <= 0:
        raise ValueError("adaptive pooling output dimensions must be positive")
    y = np.empty((OH, OW, C), F32)
    for oh in range(OH):
        hb, he = (oh * H) // OH, ((oh + 1) * H + OH - 1) // OH
        for ow in range(OW):
            wb, we = (ow * W) // OW, ((ow + 1) * W + OW - 1) // OW
            acc = np.full(C, -np.inf if kind == 0 else 0.0, F32)
            for r in range(hb, he):
                for c in range(wb, we):
                    acc = np.maximum(acc, x[r, c]) if kind == 0 else (acc + x[r, c]).astype(F32)
            y[oh, ow] = acc if kind == 0 else (acc / F32((he - hb) * (we - wb))).astype(F32)
    return y


def op_pooling(layer: Layer, x: np.ndarray) -> np.ndarray:
    """ConvertPooling static branch (NCNNToTosa.cpp:1879-1994)."""
    L = _ops()
    H, W, C = x.shape
    kind = layer.geti(0)
    kw = layer.geti(1); kh = layer.geti(11, kw)
    sw = layer.geti(2, 1); sh = layer.geti(12, sw)
    pl = layer.geti(3, 0); pr = layer.geti(14, pl); pt = layer.geti(13, pl); pb = layer.geti(15, pt)
    mode = layer.geti(5, 0)
    if layer.geti(4):  # global: kernel = H x W, result shape [C] (ImportPooling.cpp:71-77)
        kh, kw, sh, sw, pt, pl, OH, OW = H, W, 1, 1, 0, 0, 1, 1
    elif layer.geti(7):
        return _adaptive_pooling(layer, x, kind)
    else:
        if layer.geti(6) and (pt or pb or pl or pr):
            raise ValueError("avgpool_count_include_pad=1 is rejected by the reference's strict gate")
        if mode in (2, 3):
            pt, pb = same_padding(H, kh, sh, 1, mode == 3)
            pl, pr = same_padding(W, kw, sw, 1, mode == 3)
        OH = pool_out_extent(H, kh, sh, pt, pb, mode)
        OW = pool_out_extent(W, kw, sw, pl, pr, mode)
    if x.dtype == np.int8:
        if kind != 0:
            raise ValueError("signed i8 pooling only supports maximum")
        y = np.empty((OH, OW, C), np.int8)
        L.orc_pool_max_i8(_p(np.ascontiguousarray(x), ctypes.c_int8), H, W, C, kh, kw, sh, sw, pt, pl,
                          OH, OW, _p(y, ctypes.c_int8))
    else:
        y = np.empty((OH, OW, C), F32)
        L.orc_pool_f32(_p(np.ascontiguousarray(x, F32), ctypes.c_float), H, W, C, kind, kh, kw, sh, sw,
                       pt, pl, OH, OW, _p(y, ctypes.c_float))
    if layer.geti(4):
        return y.reshape(C)
    return y


def op_eltwise(layer: Layer, a, b):
    """import_eltwise (ImportOps.cpp:435-506): SUM only; a coefficient != 1 first
    multiplies its input, then a + b."""
    if layer.geti(0, 1) != 1:
        raise ValueError("Eltwise supports SUM only")
    coeffs = layer.params.get(1)
    if coeffs:
        if F32(coeffs[0]) != F32(1.0):
            a = (a * F32(coeffs[0])).astype(F32)
        if F32(coeffs[1]) != F32(1.0):
            b = (b * F32(coeffs[1])).astype(F32)
    return (a + b).astype(F32)


def op_binary(layer: Layer, ins):
    """ConvertBinary (NCNNToTosa.cpp:5111-5223): 0 add, 1 sub, 2 mul, 4 max."""
    op = layer.geti(0, 0)
    a = ins[0]
    b = F32(layer.getf(2, 0.0)) if layer.geti(1, 0) else ins[1]
    if not layer.geti(1, 0) and a.shape != b.shape:
        # computeBinaryResult (NCNNOps.cpp:1219-1244): right-aligned broadcasting over the logical
        # [c,h,w] dims; this oracle keeps rank-3 arrays as HWC, so go through CHW views
        def chw(x):
            return x.transpose(2, 0, 1) if x.ndim == 3 else x
        a, b = np.broadcast_arrays(chw(a), chw(b))
        back = (lambda y: np.ascontiguousarray(y.transpose(1, 2, 0))) if a.ndim == 3 else (lambda y: y)
        a, b = back(a), back(b)
    if op == 0:
        return (a + b).astype(F32)
    if op == 1:
        return (a - b).astype(F32)
    if op == 2:
        return (a * b).astype(F32)
    if op == 4:
        return np.maximum(a, b)
    raise ValueError(f"BinaryOp {op} is outside the hot path")


def op_relu(layer: Layer, x):
    slope = layer.getf(0, 0.0)
    return _act(x, 1 if slope == 0.0 else 2, [slope])


def op_clip(layer: Layer, x):
    """Extension: the reference has no Clip importer; ncnn's Clip is min(max(x,lo),hi)."""
    return _act(x, 3, [layer.getf(0, -np.finfo(F32).max), layer.getf(1, np.finfo(F32).max)])


def op_sigmoid(x):
    """ConvertSigmoid (NCNNToTosa.cpp:2991-3021): clamp to +-88.3762626647949, then
    tosa.sigmoid = 1 / (1 + exp(-x)), all in f32."""
    c = np.minimum(np.maximum(x.astype(F32), F32(-88.3762626647949)), F32(88.3762626647949))
    return (F32(1) / (F32(1) + np.exp(-c, dtype=F32))).astype(F32)


def op_gelu(layer: Layer, x):
    """ConvertGELU (NCNNToTosa.cpp:4670-4738), erf form only (import_gelu, ImportActivation.cpp:543-564):
    (x * erfc(x * -0.7071067811865476)) * 0.5, every step rounded to f32."""
    from scipy.special import erfc
    if layer.geti(0, 0) != 0:
        raise ValueError("invalid GELU parameters")
    x = x.astype(F32)
    tail = erfc((x * F32(-0.7071067811865476)).astype(F32)).astype(F32)
    return ((x * tail).astype(F32) * F32(0.5)).astype(F32)


def op_deconvolution(layer: Layer, x):
    """The one Deconvolution the reference imports (import_deconvolution, ImportDetection.cpp:349-470): static
    fp32 2x2 kernel, stride 2, no padding; ConvertDeconvolution (NCNNToTosa.cpp:2737-2990) computes
    out[2h+a, 2w+b, o] = bias[o] + sum_c in[h, w, c] * W[o, c, a, b] (no kernel flip), then ReLU for type 1."""
    kw = layer.geti(1, 0)
    geom = [layer.geti(11, kw), kw, layer.geti(13, layer.geti(3, 1)), layer.geti(3, 1), layer.geti(12, layer.geti(2, 1)),
            layer.geti(2, 1)]
    pl = layer.geti(4, 0)
    pads = [pl, layer.geti(15, pl), layer.geti(14, pl), layer.geti(16, layer.geti(14, pl)), layer.geti(18, 0),
            layer.geti(19, layer.geti(18, 0)), layer.geti(20, 0), layer.geti(21, layer.geti(20, 0))]
    act = layer.geti(9, 0)
    if layer.geti(28, 0) or geom != [2, 2, 2, 2, 1, 1] or any(pads) or act not in (0, 1):
        raise ValueError("only static FP32 2x2 stride-2 Deconvolution is supported")
    H, W, C = x.shape
    O = layer.geti(0)
    w = layer.weights[0].astype(F32).reshape(O, C, 2, 2)
    bias = layer.weights[1].astype(F32) if layer.geti(5) else np.zeros(O, F32)
    out = np.empty((2 * H, 2 * W, O), F32)
    xs = x.astype(F32)
    for a in range(2):
        for bb in range(2):
            acc = np.broadcast_to(bias, (H, W, O)).astype(F32)
            for c in range(C):  # reduction over input channels in index order, one rounding per step
                acc = (acc + (xs[:, :, c, None] * w[None, None, :, c, a, bb]).astype(F32)).astype(F32)
            out[a::2, bb::2, :] = acc
    return np.maximum(out, F32(0)) if act == 1 else out


def op_prelu(layer: Layer, x):
    """import_prelu (ImportActivation.cpp:504-541): exactly one finite f32 slope, lowered as ncnn.relu
    with that slope: x >= 0 ? x : x * slope."""
    if layer.geti(0, 0) != 1 or len(layer.weights) != 1 or layer.weights[0].size != 1:
        raise ValueError("PReLU supports exactly one FP32 scalar slope")
    slope = F32(layer.weights[0].reshape(-1)[0])
    if not np.isfinite(slope):
        raise ValueError("PReLU slope must be finite")
    x = x.astype(F32)
    return np.where(x >= 0, x, (x * slope).astype(F32)).astype(F32)


def op_swish(x):
    """ConvertSwish (NCNNToTosa.cpp:3702-3720): x * sigmoid(x), no clamp."""
    x = x.astype(F32)
    with np.errstate(over="ignore"):
        return (x * (F32(1) / (F32(1) + np.exp(-x, dtype=F32)))).astype(F32)


def op_hard_activation(layer: Layer, x, swish):
    """ConvertHardActivation (NCNNToTosa.cpp:3023-3072): gate = clamp(x*alpha + beta, 0, 1)
    (separate multiply and add); HardSwish multiplies x by the gate.  Defaults alpha 0.2,
    beta 0.5; alpha must be positive (ImportOps.cpp:120-157)."""
    alpha, beta = F32(layer.getf(0, 0.2)), F32(layer.getf(1, 0.5))
    if not alpha > 0:
        raise ValueError("alpha must be positive")
    x = x.astype(F32)
    gate = np.minimum(np.maximum(((x * alpha).astype(F32) + beta).astype(F32), F32(0)), F32(1))
    return (x * gate).astype(F32) if swish else gate


def op_dropout(layer: Layer, x):
    """ConvertDropout (NCNNToTosa.cpp:2047-2070): identity for scale 1, else x * scale."""
    scale = F32(layer.getf(0, 1.0))
    return x if scale == 1 else (x.astype(F32) * scale).astype(F32)


def _storage_axis(rank, axis):
    """Logical ncnn axis ([c,d,h,w] / [c,h,w] / [h,w] / [w], negative from the end) -> axis of the
    array as this oracle stores it (rank 3 is HWC, like the reference's NHWC; convertAxis; rank 4 is kept in
    its logical order [c,d,h,w])."""
    if axis < 0:
        axis += rank
    if not 0 <= axis < rank:
        raise ValueError("axis is out of range")
    return {0: 2, 1: 0, 2: 1}[axis] if rank == 3 else axis


def op_softmax(layer: Layer, x):
    """import_softmax (ImportActivation.cpp:648-695) + ConvertSoftmax (NCNNToTosa.cpp:2072-2112):
    m = reduce_max, e = exp(x - m), s = reduce_sum(e), out = e * reciprocal(s)."""
    axis, fixbug = layer.geti(0, 0), layer.geti(1, 0)
    if fixbug not in (0, 1):
        raise ValueError("fixbug0 must be 0 or 1")
    if fixbug == 0 and axis != 0:
        raise ValueError("legacy Softmax only supports axis 0 unless fixbug0 is 1")
    if x.ndim == 1:
        axis = 0
    ax = _storage_axis(x.ndim, axis)
    x = x.astype(F32)
    e = np.exp((x - x.max(axis=ax, keepdims=True)).astype(F32), dtype=F32)
    s = e.sum(axis=ax, keepdims=True, dtype=F32)
    return (e * (F32(1) / s).astype(F32)).astype(F32)


def op_concat(layer: Layer, ins):
    """import_concat (ImportTensor.cpp:48-96) + ConvertConcat (NCNNToTosa.cpp:2012-2045)."""
    if len(ins) < 2:
        raise ValueError("Concat requires at least two inputs")
    return np.ascontiguousarray(np.concatenate(ins, axis=_storage_axis(ins[0].ndim, layer.geti(0, 0))))


def op_slice(layer: Layer, x):
    """import_slice (ImportTensor.cpp:136-193) + inferSliceResults (NCNNOps.cpp:1538-1591): sizes along
    one logical axis, -233 = an equal share of what is left; the sizes must consume the axis."""
    sizes = list(layer.params[0])
    if len(sizes) < 2:
        raise ValueError("Slice requires at least two slices")
    ax = _storage_axis(x.ndim, layer.geti(1, 0))
    extent, consumed, outs = x.shape[ax], 0, []
    for k, size in enumerate(sizes):
        if size == -233:
            size = (extent - consumed) // (len(sizes) - k)
        if size <= 0 or size > extent - consumed:
            raise ValueError("Slice sizes must be positive and fit input")
        outs.append(np.ascontiguousarray(np.take(x, range(consumed, consumed + size), axis=ax)))
        consumed += size
    if consumed != extent:
        raise ValueError("Slice sizes must consume the entire axis")
    return outs


def op_shuffle_channel(layer: Layer, x):
    """ConvertShuffleChannel (NCNNToTosa.cpp:5394-5456): channels [group][C/group] -> [C/group][group];
    reverse uses C/group groups."""
    group, reverse = layer.geti(0, 1), layer.geti(1, 0)
    C = x.shape[2]
    if group <= 0 or C % group:
        raise ValueError("group must divide channel count")
    g = C // group if reverse else group
    H, W = x.shape[:2]
    return np.ascontiguousarray(x.reshape(H, W, g, C // g).transpose(0, 1, 3, 2).reshape(H, W, C))


def op_padding(layer: Layer, x):
    """import_padding (ImportDetection.cpp:31-112) + ConvertPadding (NCNNToTosa.cpp:2231-2248):
    constant spatial padding of a rank-3 tensor."""
    if layer.geti(4, 0) != 0 or layer.geti(6, 0) or layer.geti(7, 0) or layer.geti(8, 0):
        raise ValueError("Padding only supports constant spatial padding without per-channel data")
    t, b, l, r = (layer.geti(k, 0) for k in range(4))
    v = layer.params.get(5, 0.0)
    value = F32(0.0) if isinstance(v, int) else F32(v)
    return np.pad(x, ((t, b), (l, r), (0, 0)), constant_values=value).astype(F32)


def _bilinear_coordinate(index, n_in, n_out, align):
    """Source coordinate exactly as ConvertInterp spells it in f32 (NCNNToTosa.cpp:2371-2434)."""
    idx, fin, fout = index.astype(F32), F32(n_in), F32(n_out)
    in_max = F32(fin - F32(1))
    if align:
        src = ((idx * in_max).astype(F32) / F32(fout - F32(1))).astype(F32)
    else:
        src = ((((idx + F32(0.5)).astype(F32) * fin).astype(F32) / fout).astype(F32) - F32(0.5)).astype(F32)
    src = np.minimum(np.maximum(src, F32(0)), in_max)
    base = np.minimum(np.floor(src).astype(np.int64), n_in - 2)
    return base, (src - base.astype(F32)).astype(F32)


def op_interp(layer: Layer, x):
    """import_interp (ImportDetection.cpp:114-205) + ConvertInterp (NCNNToTosa.cpp:2252-2572): nearest
    = floor(out / scale), or (out * in) / out_size with an explicit size; bilinear in f32 step by step."""
    kind, align = layer.geti(0, 0), layer.geti(6, 0)
    hs, ws = layer.getf(1, 1.0), layer.getf(2, 1.0)
    oh, ow = layer.geti(3, 0), layer.geti(4, 0)
    if kind not in (1, 2) or (kind == 1 and align) or hs < 1 or ws < 1 or hs != int(hs) or ws != int(ws) or layer.geti(5, 0):
        raise ValueError("Interp supports nearest or bilinear resize with valid integer scale and alignment only")
    H, W, _ = x.shape
    OH, OW = (oh or H * int(hs)), (ow or W * int(ws))
    ys, xs = np.arange(OH), np.arange(OW)
    if kind == 1:
        iy = (ys * H) // OH if oh else ys // int(hs)
        ix = (xs * W) // OW if ow else xs // int(ws)
        return np.ascontiguousarray(x[iy][:, ix])
    y0, fy = _bilinear_coordinate(ys, H, OH, align)
    x0, fx = _bilinear_coordinate(xs, W, OW, align)
    fx, fy = fx[None, :, None], fy[:, None, None]
    gx, gy = (F32(1) - fx).astype(F32), (F32(1) - fy).astype(F32)
    v00, v01 = x[y0][:, x0], x[y0][:, x0 + 1]
    v10, v11 = x[y0 + 1][:, x0], x[y0 + 1][:, x0 + 1]
    top = ((v00 * gx).astype(F32) + (v01 * fx).astype(F32)).astype(F32)
    bottom = ((v10 * gx).astype(F32) + (v11 * fx).astype(F32)).astype(F32)
    return ((top * gy).astype(F32) + (bottom * fy).astype(F32)).astype(F32)


def op_reduction(layer: Layer, x):
    """import_reduction (ImportTensor.cpp:195-255) + ConvertReduction (NCNNToTosa.cpp:5546-5682): f32
    mean = reduce_sum axis by axis in storage order (h, w, c), times float(coeff / count)."""
    reduce_all, keep = layer.geti(1, 1), layer.geti(4, 0)
    axes = list(layer.params.get(3, []))
    if layer.geti(0, 0) != 3:
        raise ValueError("Reduction supports static FP32 mean with integer axes only")
    if not reduce_all and (not axes or layer.geti(5, 0) != 1):
        raise ValueError("explicit Reduction axes require fixbug0=1")
    if x.ndim != 3:
        raise ValueError("Reduction of tensors that are not rank 3 is outside the supported path")
    logical = sorted({a + 3 if a < 0 else a for a in axes}) if not reduce_all else [0, 1, 2]
    if not reduce_all and len(logical) != len(axes):
        raise ValueError("Reduction axes must be unique and in range")
    y = x.astype(F32)
    count = 1
    for sa in sorted(_storage_axis(3, a) for a in logical):
        count *= y.shape[sa]
        acc = np.zeros(np.delete(y.shape, sa), F32)
        for k in range(y.shape[sa]):  # sequential accumulation, like the lowered loop
            acc = (acc + np.take(y, k, axis=sa)).astype(F32)
        y = np.expand_dims(acc, sa)
    y = (y * F32(float(F32(layer.getf(2, 1.0))) / count)).astype(F32)
    kept = [d for a, d in enumerate((x.shape[2], x.shape[0], x.shape[1])) if a not in logical]  # logical c, h, w
    if keep:
        return y
    if len(kept) == 2 and 0 in logical:
        return y.reshape(kept)  # [h, w]
    if len(kept) == 2:
        raise ValueError("this combination of Reduction axes is outside the supported path")
    return y.reshape(kept if kept else [1])


def op_dequantize(acc_i32, scale, bias=None):
    """dequantizeNcnn (NCNNToTosa.cpp:411-460): float(v)*s[c] (+bias[c]); c = last axis."""
    y = (acc_i32.astype(F32) * np.asarray(scale, F32)).astype(F32)
    if bias is not None:
        y = (y + np.asarray(bias, F32)).astype(F32)
    return y


def op_requantize(acc_i32, scale_in, scale_out, bias=None, relu=False):
    """ConvertRequantize (NCNNToTosa.cpp:4846-4888)."""
    t = op_dequantize(acc_i32, scale_in, bias)
    if relu:
        t = np.maximum(t, F32(0))
    so = np.asarray(scale_out, F32).reshape(-1)
    return quantize(t, so, t.ndim - 1 if so.size > 1 else None)


def batchnorm_scale_offset(slope, mean, var, bias, eps):
    """FoldNCNNBatchNorm.cpp:99-124 / ConvertBatchNorm (NCNNToTosa.cpp:4740-4800)."""
    ve = (var.astype(F32) + F32(eps)).astype(F32)
    # std::pow(float, float) in the fold and math.powf behind tosa.pow: the C library's powf, not NumPy's
    inv = np.array([_powf(float(v), -0.5) if v != 0 else 10000.0 for v in ve], F32)
    inv = np.where(ve == 0, F32(10000.0), inv).astype(F32)
    scale = (slope.astype(F32) * inv).astype(F32)
    offset = (bias.astype(F32) - (scale * mean.astype(F32)).astype(F32)).astype(F32)
    return scale, offset


# --------------------------------------------------------------------------- graph walk

class Model:
    """Loads a .param/.bin pair and evaluates it one image at a time, as the
    reference's entry point does (no batch dimension: NCNNToTosa.cpp:48-52)."""

    def __init__(self, param_path, bin_path, input_shapes=None):
        self.layers = load_graph(param_path, bin_path)
        self.input_shapes = input_shapes or []
        consumed = set()
        self.inputs, produced = [], []
        for l in self.layers:
            consumed.update(l.bottoms)
            produced.extend(l.tops)
            if l.type == "Input":
                self.inputs.extend(l.tops)
        self.outputs = [b for b in produced if b not in consumed]
        self._fold_batchnorm()

    def _fold_batchnorm(self):
        """A BatchNorm whose only producer is a single-use, non-quantised fp32
        Convolution/ConvolutionDepthWise is folded into it (FoldNCNNBatchNorm.cpp:55-178)."""
        uses = {}
        for l in self.layers:
            for b in l.bottoms:
                uses[b] = uses.get(b, 0) + 1
        producer = {t: l for l in self.layers for t in l.tops}
        keep = []
        for l in self.layers:
            if l.type == "BatchNorm":
                p = producer.get(l.bottoms[0])
                if (p is not None and p.type in ("Convolution", "ConvolutionDepthWise")
                        and p.geti(8) == 0 and uses.get(l.bottoms[0], 0) == 1 and p.geti(9) == 0
                        and p.weights[0].dtype == F32):
                    scale, offset = batchnorm_scale_offset(*l.weights, l.getf(1, 0.0))
                    O = p.geti(0)
                    p.weights[0] = (p.weights[0].reshape(O, -1) * scale[:, None]).astype(F32).reshape(-1)
                    if p.geti(5):
                        p.weights[1] = ((p.weights[1] * scale).astype(F32) + offset).astype(F32)
                    else:
                        p.weights.insert(1, offset)
                        p.params[5] = 1
                    p.tops = list(l.tops)
                    for t in l.tops:
                        producer[t] = p
                    continue
            keep.append(l)
        self.layers = keep

    def run(self, inputs, want=None):
        """inputs: CHW float32 arrays in Input-layer order.  Returns CHW outputs."""
        env = {}
        it = iter(inputs)
        for l in self.layers:
            t = l.type
            if t == "Input":
                for top in l.tops:
                    a = np.asarray(next(it), F32)
                    env[top] = np.ascontiguousarray(a.transpose(1, 2, 0)) if a.ndim == 3 else a
                continue
            ins = [env[b] for b in l.bottoms]
            if t == "Convolution":
                out = op_convolution(l, ins[0])
            elif t == "ConvolutionDepthWise":
                out = op_depthwise(l, ins[0])
            elif t == "InnerProduct":
                x = ins[0]
                if x.ndim == 3:
                    x = x.transpose(2, 0, 1).reshape(1, -1)  # back to CHW, then flatten
                elif x.ndim == 1:
                    x = x.reshape(1, -1)
                y = op_inner_product(l, np.ascontiguousarray(x))
                out = y.reshape(-1) if ins[0].ndim != 2 else y
            elif t == "Gemm":
                out = op_gemm(l, ins[0])
            elif t == "Pooling":
                out = op_pooling(l, ins[0])
            elif t == "Eltwise":
                out = op_eltwise(l, ins[0], ins[1])
            elif t == "BinaryOp":
                out = op_binary(l, ins)
            elif t == "ReLU":
                out = op_relu(l, ins[0])
            elif t == "Clip":
                out = op_clip(l, ins[0])
            elif t == "Sigmoid":
                out = op_sigmoid(ins[0])
            elif t == "Swish":
                out = op_swish(ins[0])
            elif t == "Deconvolution":
                out = op_deconvolution(l, ins[0])
            elif t == "GELU":
                out = op_gelu(l, ins[0])
            elif t == "PReLU":
                out = op_prelu(l, ins[0])
            elif t == "TanH":
                out = np.tanh(ins[0].astype(F32), dtype=F32)  # ConvertTanH (NCNNToTosa.cpp:3722-3736)
            elif t in ("HardSigmoid", "HardSwish"):
                out = op_hard_activation(l, ins[0], t == "HardSwish")
            elif t == "Dropout":
                out = op_dropout(l, ins[0])
            elif t == "Softmax":
                out = op_softmax(l, ins[0])
            elif t == "Concat":
                out = op_concat(l, ins)
            elif t == "UnaryOp":
                if l.geti(0, 0) != 4:  # ConvertUnary (NCNNToTosa.cpp:5225-5252): square only
                    raise ValueError("UnaryOp supports the square operation (op_type=4) only")
                out = (ins[0].astype(F32) * ins[0].astype(F32)).astype(F32)
            elif t == "Slice":
                for top, piece in zip(l.tops, op_slice(l, ins[0])):
                    env[top] = piece
                continue
            elif t == "ShuffleChannel":
                out = op_shuffle_channel(l, ins[0])
            elif t == "Padding":
                out = op_padding(l, ins[0])
            elif t == "Interp":
                out = op_interp(l, ins[0])
            elif t == "Reduction":
                out = op_reduction(l, ins[0])
            elif t == "BatchNorm":
                scale, offset = batchnorm_scale_offset(*l.weights, l.getf(1, 0.0))
                if ins[0].ndim == 2:  # channel axis is dimension 0 unless the tensor is rank 3
                    scale, offset = scale[:, None], offset[:, None]
                out = ((ins[0] * scale).astype(F32) + offset).astype(F32)
            elif t == "Quantize":
                s = l.weights[0]
                out = quantize(ins[0], s, ins[0].ndim - 1 if s.size > 1 else None)
            elif t == "Split":
                for top in l.tops:
                    env[top] = ins[0]
                continue
            elif t == "Flatten":
                x = ins[0]
                out = x.transpose(2, 0, 1).reshape(-1) if x.ndim == 3 else np.ascontiguousarray(x).reshape(-1)
            elif t == "Reshape":
                # import_reshape (ImportOps.cpp:166-300): 0=w 1=h 11=d 2=c; the result's dims are the given ones
                # in the order [c,d,h,w] (-233 = absent), 0 copies an input extent (w: last, h: last but one,
                # d: second of a rank-4 input, c: first of a rank >= 3 input), a single -1 is inferred
                x = ins[0]
                chw = np.ascontiguousarray(x.transpose(2, 0, 1)) if x.ndim == 3 else np.ascontiguousarray(x)
                raw = [l.geti(2, -233), l.geti(11, -233), l.geti(1, -233), l.geti(0, -233)]
                dims = []
                for i, v in enumerate(raw):
                    if v == -233:
                        continue
                    if v == 0:
                        if i == 3:
                            v = chw.shape[-1]
                        elif i == 2:
                            if chw.ndim < 2:
                                raise ValueError("reshape cannot copy missing height dimension")
                            v = chw.shape[-2]
                        elif i == 1:
                            if chw.ndim != 4:
                                raise ValueError("reshape cannot copy missing depth dimension")
                            v = chw.shape[1]
                        else:
                            if chw.ndim < 3:
                                raise ValueError("reshape cannot copy missing channel dimension")
                            v = chw.shape[0]
                    dims.append(v)
                if dims.count(-1) > 1:
                    raise ValueError("reshape allows at most one -1 dimension")
                flat = chw.reshape(dims)  # numpy infers a single -1
                out = np.ascontiguousarray(flat.transpose(1, 2, 0)) if flat.ndim == 3 else flat
            elif t in ("Squeeze", "ExpandDims"):
                # explicit axes over the logical [c,h,w] order (computeSqueezeResult /
                # computeExpandDimsResult, NCNNOps.cpp:868-927); a named axis that is not 1 stays
                x = ins[0]
                chw = x.transpose(2, 0, 1) if x.ndim == 3 else x
                axes = l.params.get(3)
                if not isinstance(axes, (list, tuple, np.ndarray)):
                    raise ValueError(f"{t}: parameter 3 (axes) must be an integer array")
                axes = [int(a) for a in axes]
                if t == "Squeeze":
                    axes = [a + chw.ndim if a < 0 else a for a in axes]
                    keep = [d for i, d in enumerate(chw.shape) if not (i in axes and d == 1)] or [1]
                else:
                    rank = chw.ndim + len(axes)
                    if rank > 3:
                        raise ValueError("rank-4 tensors are outside the hot path")
                    axes = [a + rank if a < 0 else a for a in axes]
                    it = iter(chw.shape)
                    keep = [1 if i in axes else next(it) for i in range(rank)]
                flat = np.ascontiguousarray(chw).reshape(keep)
                out = np.ascontiguousarray(flat.transpose(1, 2, 0)) if flat.ndim == 3 else flat
            elif t == "Permute":
                # import_permute (ImportTensor.cpp:343-400): rank 2 order 0/1; rank 3 order 2 -> [h,c,w],
                # order 4 -> [w,c,h] (result extent i = input extent perm[i])
                x = ins[0]
                order = l.geti(0, 0)
                if x.ndim == 2 and order in (0, 1):
                    out = np.ascontiguousarray(x.T) if order == 1 else x
                elif x.ndim == 3 and order in (2, 4):
                    chw = x.transpose(2, 0, 1)
                    res = chw.transpose((1, 0, 2) if order == 2 else (2, 0, 1))
                    out = np.ascontiguousarray(res.transpose(1, 2, 0))
                elif x.ndim == 4 and order == 3:
                    # rank 4 keeps its logical order [c,d,h,w]; order_type 3 gives [c,h,w,d] (permutation {0,2,3,1})
                    out = np.ascontiguousarray(x.transpose(0, 2, 3, 1))
                else:
                    raise ValueError("Permute supports rank-2 order 0/1, rank-3 order 2/4, and rank-4 order 3 only")
            else:
                raise ValueError(f"layer type {t} is outside the hot path")
            env[l.tops[0]] = out
        outs = []
        for name in (want or self.outputs):
            a = env[name]
            if a.dtype != F32:
                a = a.astype(F32)
            outs.append(np.ascontiguousarray(a.transpose(2, 0, 1)) if a.ndim == 3 else a)
        return outs
