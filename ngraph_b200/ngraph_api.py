"""Python (ctypes) view of nGraph's client API, through ``libng_capi.so``.

It lets the tests and the benchmark do what any nGraph client does - build a ``Function`` out of
ops, ``Backend.create("B200")``, ``compile``, ``create_tensor``, ``write``, ``call``, ``read`` -
without a pybind build of nGraph.  Names follow nGraph (``op::v0::Quantize`` -> ``quantize`` ...).
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
CAPI_PATH = os.path.join(HERE, "libng_capi.so")
PLUGIN_PATH = os.path.join(HERE, "libb200_backend.so")

ET = {np.dtype(np.uint8): 0, np.dtype(np.int8): 1, np.dtype(np.int32): 2, np.dtype(np.float32): 3, np.dtype(np.int64): 4}
NP = {v: k for k, v in ET.items()}
_lib = None
_loaded_backends = set()


class NgraphError(RuntimeError):
    pass


def capi():
    global _lib
    if _lib is None:
        if not os.path.exists(CAPI_PATH):
            raise ImportError("%s is missing: run `python -m ngraph_b200.build` where nGraph's headers and "
                              "libngraph.so are available" % CAPI_PATH)
        lib = ctypes.CDLL(CAPI_PATH, mode=ctypes.RTLD_GLOBAL)
        vp, ci, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
        p64, pvp = ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_void_p)
        sigs = {
            "ngc_last_error": (ctypes.c_char_p, []),
            "ngc_load_backend": (ci, [ctypes.c_char_p, ctypes.c_char_p]),
            "ngc_backend_create": (vp, [ctypes.c_char_p]), "ngc_backend_free": (None, [vp]),
            "ngc_registered_backends": (ci, [ctypes.c_char_p, ci]),
            "ngc_value_free": (None, [vp]),
            "ngc_parameter": (vp, [ci, p64, ci]), "ngc_constant": (vp, [ci, p64, ci, vp]),
            "ngc_quantize": (vp, [vp, vp, vp, ci, p64, ci, ci]), "ngc_dequantize": (vp, [vp, vp, vp, ci, p64, ci]),
            "ngc_quantized_dot": (vp, [vp] * 8 + [ci]), "ngc_quantized_dot_bias": (vp, [vp, vp, vp, vp, ci, ci]),
            "ngc_quantized_conv": (vp, [vp, vp, p64] + [vp] * 6 + [ci]),
            "ngc_quantized_conv_bias": (vp, [vp, vp, vp, p64, vp, ci]),
            "ngc_quantized_conv_bias_add": (vp, [vp, vp, vp, vp, p64, vp, vp, ci, ci]),
            "ngc_quantized_conv_relu": (vp, [vp, vp, p64, vp]),
            "ngc_convolution": (vp, [vp, vp, p64]),
            "ngc_max_pool": (vp, [vp, p64, p64, p64, p64]), "ngc_avg_pool": (vp, [vp, p64, p64]),
            "ngc_max_pool_ex": (vp, [vp, p64, p64, p64, p64, ci]), "ngc_avg_pool_ex": (vp, [vp, p64, p64, p64, p64, ci, ci]),
            "ngc_convert": (vp, [vp, ci]), "ngc_reshape": (vp, [vp, p64, ci, p64, ci]), "ngc_relu": (vp, [vp]), "ngc_tanh": (vp, [vp]),
            "ngc_add": (vp, [vp, vp]), "ngc_multiply": (vp, [vp, vp]), "ngc_dot": (vp, [vp, vp, i64]),
            "ngc_broadcast": (vp, [vp, p64, ci, p64, ci]),
            "ngc_value_shape": (ci, [vp, p64, ci, ctypes.POINTER(ci)]),
            "ngc_function": (vp, [pvp, ci, pvp, ci]), "ngc_function_free": (None, [vp]),
            "ngc_function_op_count": (ci, [vp]),
            "ngc_bert_encoder": (vp, [ci] * 7 + [ctypes.c_uint64, ci]),
            "ngc_function_op_names": (ci, [vp, ci, ctypes.c_char_p, ci]),
            "ngc_concat": (vp, [pvp, ci, i64]),
            "ngc_sum": (vp, [vp, p64, ci]), "ngc_softmax": (vp, [vp, p64, ci]),
            "ngc_layer_norm": (vp, [vp, vp, vp, i64, ctypes.c_double]), "ngc_gelu": (vp, [vp]),
            "ngc_batch_mat_mul": (vp, [vp, vp]),
            "ngc_quantized_concat": (vp, [pvp, pvp, pvp, ci, i64]),
            "ngc_function_after_b200_passes": (vp, [vp, ci]),
            "ngc_function_split_batch": (vp, [vp, i64, ctypes.c_char_p, p64]),
            "ngc_compile": (vp, [vp, vp, ci]), "ngc_executable_free": (None, [vp]),
            "ngc_executable_save": (ci, [vp, ctypes.c_char_p]), "ngc_backend_load": (vp, [vp, ctypes.c_char_p]),
            "ngc_function_roundtrip": (vp, [vp, p64]),
            "ngc_tensor_create": (vp, [vp, ci, p64, ci]), "ngc_tensor_wrap": (vp, [vp, ci, p64, ci, vp]),
            "ngc_tensor_free": (None, [vp]),
            "ngc_tensor_write": (ci, [vp, vp, i64]), "ngc_tensor_read": (ci, [vp, vp, i64]),
            "ngc_call": (ci, [vp, pvp, ci, pvp, ci, ci]),
            "ngc_executable_create_tensors": (ci, [vp, ci, ci, ci, pvp]),
            "ngc_performance_data": (ci, [vp, ctypes.c_char_p, ci, p64, p64, ci]),
        }
        for name, (res, args) in sigs.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def _err(what):
    raise NgraphError("%s: %s" % (what, capi().ngc_last_error().decode()))


def _i64(v):
    return (ctypes.c_int64 * max(len(v), 1))(*[int(x) for x in v])


def load_backend_library(path, register_symbol):
    """dlopen a backend plugin and run its ngraph_register_*_backend function."""
    key = (path, register_symbol)
    if key in _loaded_backends:
        return
    if capi().ngc_load_backend(path.encode(), register_symbol.encode()) != 0:
        _err("loading backend library " + path)
    _loaded_backends.add(key)


def load_b200():
    if not os.path.exists(PLUGIN_PATH):
        raise ImportError("%s is missing: the B200 plugin has not been built" % PLUGIN_PATH)
    load_backend_library(PLUGIN_PATH, "ngraph_register_b200_backend")


class Value:
    """An ``Output<Node>``."""

    def __init__(self, handle, what):
        if not handle:
            _err(what)
        self.h = handle

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.ngc_value_free(self.h)

    def _info(self):
        shape, et = (ctypes.c_int64 * 8)(), ctypes.c_int()
        r = capi().ngc_value_shape(self.h, shape, 8, ctypes.byref(et))
        if r < 0:
            _err("value shape")
        return tuple(shape[:r]), NP[et.value]

    @property
    def shape(self):
        return self._info()[0]

    @property
    def dtype(self):
        return self._info()[1]


def parameter(dtype, shape):
    return Value(capi().ngc_parameter(ET[np.dtype(dtype)], _i64(shape), len(shape)), "Parameter")


def constant(array, dtype=None):
    a = np.require(np.asarray(array, dtype=dtype), requirements="C")  # keeps 0-d arrays 0-d (Shape{})
    return Value(capi().ngc_constant(ET[a.dtype], _i64(a.shape), a.ndim, a.ctypes.data_as(ctypes.c_void_p)), "Constant")


def _val(x, dtype=None):
    return x if isinstance(x, Value) else constant(x, dtype)


def quantize(x, scale, zero_point, dtype, axes=(), round_mode=4):
    axes = sorted(axes)
    s, z = _val(scale, np.float32), _val(zero_point, dtype)  # kept alive across the call
    return Value(capi().ngc_quantize(x.h, s.h, z.h, ET[np.dtype(dtype)], _i64(axes), len(axes), round_mode), "Quantize")


def dequantize(x, scale, zero_point, axes=()):
    axes = sorted(axes)
    s, z = _val(scale, np.float32), _val(zero_point, x.dtype)
    return Value(capi().ngc_dequantize(x.h, s.h, z.h, ET[np.dtype(np.float32)], _i64(axes), len(axes)), "Dequantize")


def quantized_dot(a, b, sa, za, sb, zb, so, zo, out_dtype):
    f = np.float32
    c = [_val(np.array(sa, f)), _val(np.array(za, a.dtype)), _val(np.array(sb, f)), _val(np.array(zb, b.dtype)),
         _val(np.array(so, f)), _val(np.array(zo, out_dtype))]
    return Value(capi().ngc_quantized_dot(a.h, b.h, c[0].h, c[1].h, c[2].h, c[3].h, c[4].h, c[5].h, ET[np.dtype(out_dtype)]),
                 "QuantizedDot")


def quantized_dot_bias(x, w, bias, scale, requantize=True, relu=False):
    w, bias, scale = _val(w), _val(bias), _val(scale, np.float32)
    return Value(capi().ngc_quantized_dot_bias(x.h, w.h, bias.h, scale.h, int(requantize), int(relu)), "QuantizedDotBias")


def _geom(stride, dilation, below, above, data_dilation=(1, 1)):
    above = below if above is None else above
    return _i64(list(stride) + list(dilation) + list(below) + list(above) + list(data_dilation))


def quantized_convolution(data, filt, sd, zd, sf, zf, so, zo, out_dtype, stride=(1, 1), dilation=(1, 1), pad_below=(0, 0),
                          pad_above=None, data_dilation=(1, 1)):
    f = np.float32
    filt = _val(filt)
    c = [_val(np.array(sd, f)), _val(np.array(zd, data.dtype)), _val(np.array(sf, f)), _val(np.array(zf, filt.dtype)),
         _val(np.array(so, f)), _val(np.array(zo, out_dtype))]
    return Value(capi().ngc_quantized_conv(data.h, filt.h, _geom(stride, dilation, pad_below, pad_above, data_dilation), c[0].h, c[1].h, c[2].h,
                                           c[3].h, c[4].h, c[5].h, ET[np.dtype(out_dtype)]), "QuantizedConvolution")


def quantized_conv_bias(data, filt, bias, scale, relu=False, stride=(1, 1), dilation=(1, 1), pad_below=(0, 0), pad_above=None, data_dilation=(1, 1)):
    filt, bias, scale = _val(filt), _val(bias), _val(scale, np.float32)
    return Value(capi().ngc_quantized_conv_bias(data.h, filt.h, bias.h, _geom(stride, dilation, pad_below, pad_above, data_dilation), scale.h,
                                                int(relu)), "QuantizedConvolutionBias")


def quantized_conv_bias_add(data, filt, bias, sum_in, scale, sum_scale, relu=True, signed=False, stride=(1, 1), dilation=(1, 1),
                            pad_below=(0, 0), pad_above=None, data_dilation=(1, 1)):
    filt, bias, scale, sum_scale = _val(filt), _val(bias), _val(scale, np.float32), _val(sum_scale, np.float32)
    return Value(capi().ngc_quantized_conv_bias_add(data.h, filt.h, bias.h, sum_in.h, _geom(stride, dilation, pad_below, pad_above, data_dilation),
                                                    scale.h, sum_scale.h, int(relu), int(signed)),
                 "QuantizedConvolutionBias(Signed)Add")


def quantized_conv_relu(data, filt, scale, stride=(1, 1), dilation=(1, 1), pad_below=(0, 0), pad_above=None, data_dilation=(1, 1)):
    filt, scale = _val(filt), _val(scale, np.float32)
    return Value(capi().ngc_quantized_conv_relu(data.h, filt.h, _geom(stride, dilation, pad_below, pad_above, data_dilation), scale.h),
                 "QuantizedConvolutionRelu")


def convolution(data, filt, stride=(1, 1), dilation=(1, 1), pad_below=(0, 0), pad_above=None, data_dilation=(1, 1)):
    filt = _val(filt)
    return Value(capi().ngc_convolution(data.h, filt.h, _geom(stride, dilation, pad_below, pad_above, data_dilation)), "Convolution")


def max_pool(x, window, stride, pad_below=(0, 0), pad_above=None, ceil_mode=False):
    pad_above = pad_below if pad_above is None else pad_above
    return Value(capi().ngc_max_pool_ex(x.h, _i64(window), _i64(stride), _i64(pad_below), _i64(pad_above), int(ceil_mode)), "MaxPool")


def avg_pool(x, window, stride=(1, 1), pad_below=(0, 0), pad_above=None, include_padding=False, ceil_mode=False):
    pad_above = pad_below if pad_above is None else pad_above
    return Value(capi().ngc_avg_pool_ex(x.h, _i64(window), _i64(stride), _i64(pad_below), _i64(pad_above), int(include_padding),
                                        int(ceil_mode)), "AvgPool")


def concat(values, axis):
    arr = (ctypes.c_void_p * len(values))(*[v.h for v in values])
    return Value(capi().ngc_concat(arr, len(values), axis), "Concat")


def quantized_concat(values, mins, maxs, axis):
    """builder::QuantizedConcatBuilder: mins / maxs are f32 [1] values, one pair per operand"""
    arr = lambda vs: (ctypes.c_void_p * len(vs))(*[v.h for v in vs])
    return Value(capi().ngc_quantized_concat(arr(values), arr(mins), arr(maxs), len(values), axis), "QuantizedConcat")


def reduce_sum(x, axes):
    axes = sorted(axes)
    return Value(capi().ngc_sum(x.h, _i64(axes), len(axes)), "Sum")


def softmax(x, axes):
    axes = sorted(axes)
    return Value(capi().ngc_softmax(x.h, _i64(axes), len(axes)), "Softmax")


def layer_norm(x, scale, bias, begin_norm_axis=1, epsilon=1e-5):
    scale, bias = _val(scale, np.float32), _val(bias, np.float32)  # kept alive across the call
    return Value(capi().ngc_layer_norm(x.h, scale.h, bias.h, begin_norm_axis, epsilon), "LayerNorm")


def gelu(x):
    return Value(capi().ngc_gelu(x.h), "Gelu")


def batch_mat_mul(a, b):
    return Value(capi().ngc_batch_mat_mul(a.h, b.h), "BatchMatMul")


def convert(x, dtype):
    return Value(capi().ngc_convert(x.h, ET[np.dtype(dtype)]), "Convert")


def reshape(x, order, shape):
    return Value(capi().ngc_reshape(x.h, _i64(order), len(order), _i64(shape), len(shape)), "Reshape")


def tanh(x):
    return Value(capi().ngc_tanh(x.h), "Tanh")


def relu(x):
    return Value(capi().ngc_relu(x.h), "Relu")


def add(a, b):
    return Value(capi().ngc_add(a.h, b.h), "Add")


def multiply(a, b):
    return Value(capi().ngc_multiply(a.h, b.h), "Multiply")


def dot(a, b, reduction_axes=1):
    return Value(capi().ngc_dot(a.h, b.h, reduction_axes), "Dot")


def broadcast(x, shape, axes):
    axes = sorted(axes)
    return Value(capi().ngc_broadcast(x.h, _i64(shape), len(shape), _i64(axes), len(axes)), "Broadcast")


class Function:
    def __init__(self, results, params):
        self.results, self.params = list(results), list(params)
        r = (ctypes.c_void_p * len(self.results))(*[v.h for v in self.results])
        p = (ctypes.c_void_p * max(len(self.params), 1))(*[v.h for v in self.params])
        self.h = capi().ngc_function(r, len(self.results), p, len(self.params))
        if not self.h:
            _err("Function")

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.ngc_function_free(self.h)


class _Spec:
    """dtype and shape of a Parameter / Result of a Function that was built on the C++ side"""

    def __init__(self, dtype, shape):
        self.dtype, self.shape = np.dtype(dtype), tuple(shape)


class BuiltFunction(Function):
    def __init__(self, handle, params, results, what):
        if not handle:
            _err(what)
        self.h, self.params, self.results = handle, params, results


def bert_encoder(layers, hidden, heads, ffn, seq, batch, vocab, seed=1, decomposed=False):
    """int8 BERT-base-shaped encoder (ngraph_b200/harness/bert_int8.cpp): Function(ids i32 [B*S], segments i32 [B*S])
    -> f32 [B*S, hidden].  decomposed=True replaces QuantizedDotBias by ops the INTERPRETER backend implements."""
    h = capi().ngc_bert_encoder(layers, hidden, heads, ffn, seq, batch, vocab, seed, int(decomposed))
    m = batch * seq
    return BuiltFunction(h, [_Spec(np.int32, (m,)), _Spec(np.int32, (m,))], [_Spec(np.float32, (m, hidden))], "bert_encoder")


def after_b200_passes(function, decompose_all=False):
    """a copy of `function` after the graph passes the B200 plugin runs in compile() (quantisation fusion included); needs no
    device.  decompose_all=True also decomposes the fused ops the device would run as one kernel (LayerNorm, Gelu)."""
    h = capi().ngc_function_after_b200_passes(function.h, int(decompose_all))
    if not h:
        _err("after_b200_passes")
    return BuiltFunction(h, list(function.params), list(function.results), "after_b200_passes")


def split_batch(function, rows):
    """The Function the multi-device backend option ("B200:all") gives each device: `function` (after the plugin's passes) for
    `rows` of its batch.  Returns (split Function, [is Parameter i split], [is Result j split]); raises NgraphError with the
    reason when the graph cannot be proven independent along the batch.  Needs no device."""
    n = len(function.params) + len(function.results)
    flags = ctypes.create_string_buffer(n)
    shapes = (ctypes.c_int64 * (9 * n))()
    h = capi().ngc_function_split_batch(function.h, rows, flags, shapes)
    if not h:
        _err("split_batch")
    specs = []
    for i, old in enumerate(list(function.params) + list(function.results)):
        rank = shapes[9 * i]
        specs.append(_Spec(old.dtype, tuple(shapes[9 * i + 1 + k] for k in range(rank))))
    np_, f = len(function.params), [bool(b) for b in flags.raw]
    return BuiltFunction(h, specs[:np_], specs[np_:], "split_batch"), f[:np_], f[np_:]


def function_roundtrip(function):
    """(a copy of `function` written and read back through the plugin's binary Function form, bytes written)"""
    n = ctypes.c_int64(0)
    h = capi().ngc_function_roundtrip(function.h, ctypes.byref(n))
    if not h:
        _err("function_roundtrip")
    return BuiltFunction(h, list(function.params), list(function.results), "function_roundtrip"), n.value


def function_op_names(function, lowered=True):
    """op type names in topological order, optionally after the passes a backend runs before lowering"""
    buf = ctypes.create_string_buffer(1 << 22)
    n = capi().ngc_function_op_names(function.h, int(lowered), buf, len(buf))
    if n < 0:
        _err("function_op_names")
    return buf.value.decode().split()


class Tensor:
    def __init__(self, backend, dtype, shape, device_pointer=None):
        self.dtype, self.shape, self.backend = np.dtype(dtype), tuple(int(s) for s in shape), backend
        if device_pointer is None:
            self.h = capi().ngc_tensor_create(backend.h, ET[self.dtype], _i64(self.shape), len(self.shape))
        else:
            self.h = capi().ngc_tensor_wrap(backend.h, ET[self.dtype], _i64(self.shape), len(self.shape),
                                            ctypes.c_void_p(device_pointer))
        if not self.h:
            _err("create_tensor")

    @classmethod
    def from_handle(cls, backend, dtype, shape, handle):
        t = cls.__new__(cls)
        t.dtype, t.shape, t.backend, t.h = np.dtype(dtype), tuple(int(s) for s in shape), backend, handle
        return t

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.ngc_tensor_free(self.h)

    @property
    def nbytes(self):
        return int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize

    def write(self, array):
        a = np.ascontiguousarray(array, dtype=self.dtype)
        assert a.nbytes == self.nbytes, (a.shape, self.shape)
        if capi().ngc_tensor_write(self.h, a.ctypes.data_as(ctypes.c_void_p), a.nbytes) != 0:
            _err("Tensor::write")

    def write_ptr(self, host_pointer, nbytes):
        if capi().ngc_tensor_write(self.h, ctypes.c_void_p(host_pointer), nbytes) != 0:
            _err("Tensor::write")

    def read(self):
        out = np.empty(self.shape, dtype=self.dtype)
        if capi().ngc_tensor_read(self.h, out.ctypes.data_as(ctypes.c_void_p), out.nbytes) != 0:
            _err("Tensor::read")
        return out

    def read_ptr(self, host_pointer, nbytes):
        if capi().ngc_tensor_read(self.h, ctypes.c_void_p(host_pointer), nbytes) != 0:
            _err("Tensor::read")


class Executable:
    def __init__(self, backend, function, perf=False, handle=None):
        self.backend, self.function = backend, function
        self.h = handle if handle is not None else capi().ngc_compile(backend.h, function.h, int(perf))
        if not self.h:
            _err("Backend::compile")

    def save(self, path):
        """Executable::save into the file `path`"""
        if capi().ngc_executable_save(self.h, str(path).encode()) != 0:
            _err("Executable::save")

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.ngc_executable_free(self.h)

    def call(self, outputs, inputs, validate=True):
        o = (ctypes.c_void_p * max(len(outputs), 1))(*[t.h for t in outputs])
        i = (ctypes.c_void_p * max(len(inputs), 1))(*[t.h for t in inputs])
        if capi().ngc_call(self.h, o, len(outputs), i, len(inputs), int(validate)) != 0:
            _err("Executable::call")

    def _pipeline_tensors(self, is_input, index, depth):
        spec = (self.function.params if is_input else self.function.results)[index]
        handles = (ctypes.c_void_p * depth)()
        if capi().ngc_executable_create_tensors(self.h, int(is_input), index, depth, handles) != 0:
            _err("Executable::create_%s_tensor" % ("input" if is_input else "output"))
        return [Tensor.from_handle(self.backend, spec.dtype, spec.shape, h) for h in handles]

    def create_input_tensors(self, index, depth):
        """Executable::create_input_tensor(index, pipeline_depth): `depth` tensors for one Parameter"""
        return self._pipeline_tensors(True, index, depth)

    def create_output_tensors(self, index, depth):
        return self._pipeline_tensors(False, index, depth)

    def run(self, *arrays):
        """create tensors, write the inputs, call_with_validate, read every result."""
        ins = []
        for v, a in zip(self.function.params, arrays):
            t = Tensor(self.backend, v.dtype, v.shape)
            t.write(a)
            ins.append(t)
        outs = [Tensor(self.backend, v.dtype, v.shape) for v in self.function.results]
        self.call(outs, ins)
        return [t.read() for t in outs]

    def performance_data(self):
        cap = 1 << 14  # nodes; a 12-layer encoder has a few thousand
        names = ctypes.create_string_buffer(cap * 96)
        us, calls = (ctypes.c_int64 * cap)(), (ctypes.c_int64 * cap)()
        n = capi().ngc_performance_data(self.h, names, len(names), us, calls, cap)
        if n < 0:
            _err("get_performance_data")
        return [(nm, us[i], calls[i]) for i, nm in enumerate(names.value.decode().split("\n")[:n])]


class Backend:
    def __init__(self, name):
        self.name = name
        self.h = capi().ngc_backend_create(name.encode())
        if not self.h:
            _err("Backend::create(%r)" % name)

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.ngc_backend_free(self.h)

    def compile(self, function, perf=False):
        return Executable(self, function, perf)

    def create_tensor(self, dtype, shape, device_pointer=None):
        return Tensor(self, dtype, shape, device_pointer)

    def load(self, path, like):
        """Backend::load of a file written by Executable.save; `like` (a Function or Executable with the same parameters and
        results) only tells this Python wrapper the tensor types and shapes"""
        h = capi().ngc_backend_load(self.h, str(path).encode())
        if not h:
            _err("Backend::load")
        return Executable(self, like.function if isinstance(like, Executable) else like, handle=h)


def registered_backends():
    buf = ctypes.create_string_buffer(1024)
    capi().ngc_registered_backends(buf, len(buf))
    return buf.value.decode().split()
