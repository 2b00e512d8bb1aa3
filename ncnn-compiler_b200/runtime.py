"""ctypes binding of libncnn_b200.so (include/ncnn_b200.h)."""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, byref, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

import numpy as np

FP32_SPLIT, TF32, FP32_CUDA = 0, 1, 2

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class NcnnB200Error(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"ncnn_b200 status {status}: {message}")
        self.status = status
        self.message = message


class _Options(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_uint32), ("accuracy_mode", c_int32), ("device", c_int32),
                ("use_cuda_graph", c_int32), ("input_shape_count", c_int32),
                ("input_shapes", POINTER(c_int64)), ("plan_only", c_int32), ("keep_matrix_rows", c_int32)]


class _DimConstraint(ctypes.Structure):
    _fields_ = [("input", c_int32), ("dim", c_int32), ("minimum", c_int64), ("multiple_of", c_int64)]


def lib_path() -> str:
    return os.path.join(_HERE, "libncnn_b200.so")


def load_library():
    """Loads the CUDA library; there is no fallback when it is missing."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not os.path.exists(path):
        raise NcnnB200Error(6, f"{path} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                               "(the runtime has no CPU path)")
    L = ctypes.CDLL(path)
    pp_in, pp_out = POINTER(c_void_p), POINTER(c_void_p)
    L.ncnn_b200_load.argtypes = [c_char_p, c_char_p, POINTER(_Options), POINTER(c_void_p)]
    L.ncnn_b200_free.argtypes = [c_void_p]
    L.ncnn_b200_free.restype = None
    L.ncnn_b200_last_error.argtypes = [c_void_p]
    L.ncnn_b200_last_error.restype = c_char_p
    for f in ("ncnn_b200_input_count", "ncnn_b200_output_count", "ncnn_b200_check_status"):
        getattr(L, f).argtypes = [c_void_p]
    for f in ("ncnn_b200_input_shape", "ncnn_b200_output_shape", "ncnn_b200_input_shape4", "ncnn_b200_output_shape4"):
        getattr(L, f).argtypes = [c_void_p, c_int, POINTER(c_int64)]
    for f in ("ncnn_b200_input_name", "ncnn_b200_output_name"):
        getattr(L, f).argtypes = [c_void_p, c_int]
        getattr(L, f).restype = c_char_p
    L.ncnn_b200_run.argtypes = [c_void_p, pp_in, pp_out]
    L.ncnn_b200_run_batch.argtypes = [c_void_p, c_int64, pp_in, pp_out]
    L.ncnn_b200_run_batch_device.argtypes = [c_void_p, c_int64, pp_in, pp_out, c_void_p]
    L.ncnn_b200_launch_count.argtypes = [c_void_p, c_int64]
    L.ncnn_b200_profile.argtypes = [c_void_p, c_int64, c_int, c_char_p, c_size_t]
    L.ncnn_b200_profile.restype = c_int64
    L.ncnn_b200_describe.argtypes = [c_char_p, c_char_p, c_char_p, c_size_t]
    L.ncnn_b200_describe.restype = c_int64
    L.ncnn_b200_emit_stub.argtypes = [c_void_p, c_char_p, c_char_p, c_char_p, c_char_p]
    L.ncnn_b200_op_quantize.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_void_p, c_int32, c_void_p]
    L.ncnn_b200_op_dequantize.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_void_p, c_int32,
                                          c_void_p, c_int32, c_void_p]
    L.ncnn_b200_op_requantize.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_void_p, c_int32,
                                          c_void_p, c_int32, c_void_p, c_int32, c_int32, c_void_p]
    L.ncnn_b200_inner_product_int8_noalloc.argtypes = [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                                       c_int64, c_int32, c_int32, c_int32, c_void_p]
    L.ncnn_b200_multi_load.argtypes = [c_char_p, c_char_p, POINTER(_Options), POINTER(c_int32), c_int32, POINTER(c_void_p)]
    L.ncnn_b200_multi_free.argtypes = [c_void_p]
    L.ncnn_b200_multi_free.restype = None
    L.ncnn_b200_multi_last_error.argtypes = [c_void_p]
    L.ncnn_b200_multi_last_error.restype = c_char_p
    L.ncnn_b200_multi_device_count.argtypes = [c_void_p]
    L.ncnn_b200_multi_run_batch.argtypes = [c_void_p, c_int64, pp_in, pp_out]
    L.ncnn_b200_multi_partition.argtypes = [c_int64, c_int32, POINTER(c_int64), POINTER(c_int64)]
    L.ncnn_b200_dynamic_load.argtypes = [c_char_p, c_char_p, POINTER(_Options), POINTER(_DimConstraint), c_int32,
                                         POINTER(c_void_p)]
    L.ncnn_b200_dynamic_free.argtypes = [c_void_p]
    L.ncnn_b200_dynamic_free.restype = None
    L.ncnn_b200_dynamic_last_error.argtypes = [c_void_p]
    L.ncnn_b200_dynamic_last_error.restype = c_char_p
    for f in ("ncnn_b200_dynamic_input_count", "ncnn_b200_dynamic_output_count"):
        getattr(L, f).argtypes = [c_void_p]
    for f in ("ncnn_b200_dynamic_input_shape", "ncnn_b200_dynamic_output_shape"):
        getattr(L, f).argtypes = [c_void_p, c_int, POINTER(c_int64)]
    L.ncnn_b200_dynamic_infer_output_shapes.argtypes = [c_void_p, pp_in, pp_out]
    L.ncnn_b200_dynamic_run.argtypes = [c_void_p, pp_in, pp_in, pp_out, POINTER(ctypes.c_uint64)]
    L.ncnn_b200_dynamic_emit_stub.argtypes = [c_void_p, c_char_p, c_char_p, c_char_p, c_char_p]
    _LIB = L
    return L


def describe(param_path: str, bin_path: str | None = None) -> str:
    """Loader dump (no GPU needed), same layout as the reference's Graph::dump()."""
    L = load_library()
    b = bin_path.encode() if bin_path else None
    need = L.ncnn_b200_describe(param_path.encode(), b, None, 0)
    buf = ctypes.create_string_buffer(int(need) + 1)
    L.ncnn_b200_describe(param_path.encode(), b, buf, len(buf))
    return buf.value.decode()


def _ptr_array(values):
    arr = (c_void_p * len(values))()
    for i, v in enumerate(values):
        arr[i] = v
    return arr


class Model:
    """A loaded model.  `run` takes and returns numpy arrays shaped [n, *dims] (or
    [*dims] for a single image), like n calls of the reference's entry point."""

    def __init__(self, param_path, bin_path, accuracy_mode=FP32_SPLIT, device=-1, use_cuda_graph=True,
                 input_shapes=None, plan_only=False):
        self._L = load_library()
        self._h = c_void_p()
        flat = []
        for s in input_shapes or []:
            flat.append(len(s))
            flat.extend(int(d) for d in s)
        arr = (c_int64 * max(len(flat), 1))(*flat)
        opt = _Options(ctypes.sizeof(_Options), accuracy_mode, device, 1 if use_cuda_graph else 0,
                       len(input_shapes or []), ctypes.cast(arr, POINTER(c_int64)), 1 if plan_only else 0, 0)
        st = self._L.ncnn_b200_load(param_path.encode(), bin_path.encode() if bin_path else None, byref(opt),
                                    byref(self._h))
        if st != 0:
            raise NcnnB200Error(st, self._L.ncnn_b200_last_error(None).decode())
        self.input_shapes = [self._shape(self._L.ncnn_b200_input_shape4, i, 4)
                             for i in range(self._L.ncnn_b200_input_count(self._h))]
        self.output_shapes = [self._shape(self._L.ncnn_b200_output_shape4, i, 4)
                              for i in range(self._L.ncnn_b200_output_count(self._h))]
        self.input_names = [self._L.ncnn_b200_input_name(self._h, i).decode() for i in range(len(self.input_shapes))]
        self.output_names = [self._L.ncnn_b200_output_name(self._h, i).decode()
                             for i in range(len(self.output_shapes))]

    def _shape(self, fn, i, capacity=3):
        dims = (c_int64 * capacity)()
        rank = fn(self._h, i, dims)
        return tuple(int(dims[k]) for k in range(rank))

    def close(self):
        if self._h:
            self._L.ncnn_b200_free(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st):
        if st != 0:
            raise NcnnB200Error(st, self._L.ncnn_b200_last_error(self._h).decode())

    def run(self, *inputs):
        """Host arrays in, host arrays out (copies to and from the device inside the call)."""
        ins = [np.ascontiguousarray(x, np.float32) for x in inputs]
        single = ins[0].ndim == len(self.input_shapes[0])
        n = 1 if single else ins[0].shape[0]
        for x, s in zip(ins, self.input_shapes):
            if tuple(x.shape[-len(s):]) != s or x.size != n * int(np.prod(s)):
                raise ValueError(f"input shape {x.shape} does not match {s} (batch {n})")
        outs = [np.empty((n, *s), np.float32) for s in self.output_shapes]
        self._check(self._L.ncnn_b200_run_batch(self._h, n, _ptr_array([x.ctypes.data for x in ins]),
                                                 _ptr_array([y.ctypes.data for y in outs])))
        if single:
            outs = [y[0] for y in outs]
        return outs

    def run_raw(self, n, in_ptrs, out_ptrs):
        """Host pointers (ints); returns the status code without raising."""
        return self._L.ncnn_b200_run_batch(self._h, n, _ptr_array(in_ptrs), _ptr_array(out_ptrs))

    def run_device(self, n, in_ptrs, out_ptrs, stream=0):
        """Device pointers (ints) on a CUDA stream handle; asynchronous."""
        self._check(self._L.ncnn_b200_run_batch_device(self._h, n, _ptr_array(in_ptrs), _ptr_array(out_ptrs),
                                                        c_void_p(stream)))

    def check_status(self):
        self._check(self._L.ncnn_b200_check_status(self._h))

    def launch_count(self, n):
        return int(self._L.ncnn_b200_launch_count(self._h, n))

    def profile(self, n, repeat=5):
        need = self._L.ncnn_b200_profile(self._h, n, repeat, None, 0)
        if need < 0:
            self._check(int(-need))
        buf = ctypes.create_string_buffer(int(need) + 4096)
        self._L.ncnn_b200_profile(self._h, n, repeat, buf, len(buf))
        rows = []
        for line in buf.value.decode().splitlines():
            k, name, ms, fl, by = line.split("\t")
            rows.append({"kernel": k, "layer": name, "ms": float(ms), "flops": float(fl), "bytes": float(by)})
        return rows

    def emit_stub(self, name, param_path, bin_path, directory):
        self._check(self._L.ncnn_b200_emit_stub(self._h, name.encode(), param_path.encode(), bin_path.encode(),
                                                 directory.encode()))


class DynamicModel:
    """A model with fixed-rank dynamic input extents: the counterpart of the reference's
    `--input-shape=3x?x?` libraries.  `input_shapes` holds one [c,h,w] template per Input without
    dimensions, None (or -1) where the extent is dynamic; `constraints` are tuples
    (input, dim, minimum, multiple_of).  Loading and shape inference need no GPU."""

    def __init__(self, param_path, bin_path, input_shapes, constraints=(), accuracy_mode=FP32_SPLIT, device=-1,
                 use_cuda_graph=True):
        self._L = load_library()
        self._h = c_void_p()
        flat = []
        for s in input_shapes:
            flat.append(len(s))
            flat.extend(-1 if d is None else int(d) for d in s)
        arr = (c_int64 * max(len(flat), 1))(*flat)
        opt = _Options(ctypes.sizeof(_Options), accuracy_mode, device, 1 if use_cuda_graph else 0,
                       len(input_shapes), ctypes.cast(arr, POINTER(c_int64)), 0, 0)
        lim = (_DimConstraint * max(len(constraints), 1))()
        for k, c in enumerate(constraints):
            lim[k] = _DimConstraint(*[int(v) for v in c])
        st = self._L.ncnn_b200_dynamic_load(param_path.encode(), bin_path.encode() if bin_path else None, byref(opt),
                                            lim, len(constraints), byref(self._h))
        if st != 0:
            raise NcnnB200Error(st, self._L.ncnn_b200_last_error(None).decode())
        self.input_shapes = [self._shape(self._L.ncnn_b200_dynamic_input_shape, i)
                             for i in range(self._L.ncnn_b200_dynamic_input_count(self._h))]
        self.output_shapes = [self._shape(self._L.ncnn_b200_dynamic_output_shape, i)
                              for i in range(self._L.ncnn_b200_dynamic_output_count(self._h))]

    def _shape(self, fn, i):
        dims = (c_int64 * 3)()
        rank = fn(self._h, i, dims)
        return tuple(int(dims[k]) for k in range(rank))

    def close(self):
        if self._h:
            self._L.ncnn_b200_dynamic_free(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _shape_table(self, shapes):
        keep = [(c_int64 * 3)(*[int(d) for d in s]) if s is not None else None for s in shapes]
        return keep, _ptr_array([ctypes.addressof(a) if a is not None else None for a in keep])

    def infer_status(self, shapes):
        """(status, output shapes) of `<model>_infer_output_shapes` for per-input [c,h,w] lists."""
        keep, table = self._shape_table(shapes)
        outs = [(c_int64 * 3)() for _ in self.output_shapes]
        st = self._L.ncnn_b200_dynamic_infer_output_shapes(self._h, table,
                                                           _ptr_array([ctypes.addressof(o) for o in outs]))
        return st, [tuple(int(o[k]) for k in range(len(s))) for o, s in zip(outs, self.output_shapes)]

    def infer(self, shapes):
        st, out = self.infer_status(shapes)
        if st != 0:
            raise NcnnB200Error(st, self._L.ncnn_b200_dynamic_last_error(self._h).decode())
        return out

    def run_status(self, inputs, shapes, outputs, capacities):
        """Status of the reference-shaped call: host arrays, per-input shapes, per-output capacities."""
        keep, table = self._shape_table(shapes)
        caps = (ctypes.c_uint64 * max(len(capacities), 1))(*[int(c) for c in capacities])
        return self._L.ncnn_b200_dynamic_run(self._h, _ptr_array([x.ctypes.data for x in inputs]), table,
                                             _ptr_array([y.ctypes.data for y in outputs]), caps)

    def run(self, *inputs):
        """One image per input, shaped like its template with concrete extents."""
        ins = [np.ascontiguousarray(x, np.float32) for x in inputs]
        shapes = [list(x.shape) for x in ins]
        out_shapes = self.infer(shapes)
        outs = [np.empty(s, np.float32) for s in out_shapes]
        st = self.run_status(ins, shapes, outs, [y.size for y in outs])
        if st != 0:
            raise NcnnB200Error(st, self._L.ncnn_b200_dynamic_last_error(self._h).decode())
        return outs

    def emit_stub(self, name, param_path, bin_path, directory):
        st = self._L.ncnn_b200_dynamic_emit_stub(self._h, name.encode(), param_path.encode(), bin_path.encode(),
                                                 directory.encode())
        if st != 0:
            raise NcnnB200Error(st, "cannot write the stub")


def _op_status(st):
    if st != 0:
        raise NcnnB200Error(st, "operator entry point rejected its arguments" if st in (1, 2) else "CUDA error")


def op_quantize(x_ptr, y_ptr, count, inner, channels, scale_ptr, scale_count, stream=0):
    _op_status(load_library().ncnn_b200_op_quantize(x_ptr, y_ptr, count, inner, channels, scale_ptr, scale_count,
                                                    c_void_p(stream)))


def op_dequantize(x_ptr, y_ptr, count, inner, channels, scale_ptr, scale_count, bias_ptr=None, bias_count=0,
                  stream=0):
    _op_status(load_library().ncnn_b200_op_dequantize(x_ptr, y_ptr, count, inner, channels, scale_ptr, scale_count,
                                                      bias_ptr, bias_count, c_void_p(stream)))


def op_requantize(x_ptr, y_ptr, count, inner, channels, scale_in_ptr, scale_in_count, scale_out_ptr,
                  scale_out_count, bias_ptr=None, bias_count=0, relu=False, stream=0):
    _op_status(load_library().ncnn_b200_op_requantize(x_ptr, y_ptr, count, inner, channels, scale_in_ptr,
                                                      scale_in_count, scale_out_ptr, scale_out_count, bias_ptr,
                                                      bias_count, 1 if relu else 0, c_void_p(stream)))


def inner_product_int8_noalloc(x_ptr, weight_ptr, weight_scales_ptr, input_scale, bias_ptr, y_ptr, m, k, n,
                               relu=False, stream=0):
    """int8 InnerProduct on device arrays for hosts that may not allocate on the GPU: the
    scratch lives in an 8 MiB array inside the library (m*k <= 8 388 608).  Returns the raw
    status; the message of a refusal is ncnn_b200_last_error(NULL)."""
    L = load_library()
    st = L.ncnn_b200_inner_product_int8_noalloc(x_ptr, weight_ptr, weight_scales_ptr, c_float(input_scale), bias_ptr,
                                                y_ptr, m, k, n, 1 if relu else 0, c_void_p(stream))
    return st, L.ncnn_b200_last_error(None).decode()


def multi_partition(n, parts):
    """[(first, count)] of the contiguous shards ncnn_b200_multi_run_batch gives each device."""
    L = load_library()
    first = (c_int64 * parts)()
    count = (c_int64 * parts)()
    st = L.ncnn_b200_multi_partition(n, parts, first, count)
    if st != 0:
        raise NcnnB200Error(st, "invalid partition request")
    return [(int(first[g]), int(count[g])) for g in range(parts)]


class MultiModel:
    """One model replicated on several GPUs of a box; `run` shards the batch across them
    (ncnn_b200_multi_*).  Host arrays in, host arrays out."""

    def __init__(self, param_path, bin_path, devices, accuracy_mode=FP32_SPLIT, use_cuda_graph=True):
        self._L = load_library()
        self._h = c_void_p()
        opt = _Options(ctypes.sizeof(_Options), accuracy_mode, -1, 1 if use_cuda_graph else 0, 0, None, 0, 0)
        devs = (c_int32 * len(devices))(*devices)
        st = self._L.ncnn_b200_multi_load(param_path.encode(), bin_path.encode() if bin_path else None, byref(opt), devs,
                                          len(devices), byref(self._h))
        if st != 0:
            raise NcnnB200Error(st, self._L.ncnn_b200_last_error(None).decode())
        single = Model(param_path, bin_path, plan_only=True)
        self.input_shapes, self.output_shapes = single.input_shapes, single.output_shapes
        single.close()

    def close(self):
        if self._h:
            self._L.ncnn_b200_multi_free(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def run_raw(self, n, in_ptrs, out_ptrs):
        return self._L.ncnn_b200_multi_run_batch(self._h, n, _ptr_array(in_ptrs), _ptr_array(out_ptrs))

    def run(self, *inputs):
        xs = [np.ascontiguousarray(x, np.float32) for x in inputs]
        n = xs[0].shape[0]
        outs = [np.empty((n, *s), np.float32) for s in self.output_shapes]
        st = self.run_raw(n, [x.ctypes.data for x in xs], [y.ctypes.data for y in outs])
        if st != 0:
            raise NcnnB200Error(st, self._L.ncnn_b200_multi_last_error(self._h).decode())
        return outs
