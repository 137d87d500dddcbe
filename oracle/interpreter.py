"""The reference itself as a checker: nGraph's INTERPRETER backend (built by ``make -C oracle ref``
into oracle/_ref/lib) plus the decomposed graphs that define the fused ops on it.  Test
infrastructure only.

INTERPRETER does not implement the fused experimental ops (QuantizedConvolutionBias..., QuantizedDotBias:
src/ngraph/runtime/interpreter/int_executable.hpp:1560-1653 treats them as QuantizedDot), so their
oracle is the decomposition into ops it does implement, evaluated by nGraph's own reference kernels:
  acc = QuantizedConvolution(data, filters, scales 1, zero points 0 -> i32)   (or Dot on i32 Converts)
  v   = Convert_f32(acc + Broadcast(bias)) * Broadcast(scale) [+ sum_scale * Convert_f32(sum)] [Relu]
  out = Quantize(v, scale 1, zero point 0, ROUND_NEAREST_TOWARD_EVEN)  [Convert to u8 for SignedAdd]
"""
import os

import numpy as np

from ngraph_b200 import ngraph_api as ng

_LIB = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "lib", "libinterpreter_backend.so")


def available():
    return os.path.exists(_LIB) and os.path.exists(ng.CAPI_PATH)


def backend():
    ng.load_backend_library(_LIB, "ngraph_register_interpreter_backend")
    return ng.Backend("INTERPRETER")


def _tail(acc, bias, scale, chan_axis, out_dtype, relu, sum_in=None, sum_scale=None):
    shape = acc.shape
    others = [i for i in range(len(shape)) if i != chan_axis]
    v = acc
    if bias is not None:
        v = ng.add(v, ng.broadcast(bias, shape, others))
    v = ng.convert(v, np.float32)
    if int(np.prod(scale.shape)) == 1:
        sc = ng.broadcast(ng.reshape(scale, list(range(len(scale.shape))), ()), shape, range(len(shape)))
    else:
        sc = ng.broadcast(scale, shape, others)
    v = ng.multiply(v, sc)
    if sum_in is not None:
        ss = ng.broadcast(ng.reshape(sum_scale, list(range(len(sum_scale.shape))), ()), shape, range(len(shape)))
        v = ng.add(v, ng.multiply(ss, ng.convert(sum_in, np.float32)))
    if relu:
        v = ng.relu(v)
    if np.dtype(out_dtype) == np.float32:
        return v
    return ng.quantize(v, np.float32(1.0), np.zeros((), out_dtype), out_dtype, (), 4)


def decomposed_conv(data, filt, bias, scale, out_dtype, relu, stride=(1, 1), dilation=(1, 1), pad_below=(0, 0), pad_above=None,
                    sum_in=None, sum_scale=None, signed=False, data_dilation=(1, 1)):
    """Oracle graph of QuantizedConvolutionBias / Relu / BiasAdd / BiasSignedAdd (bias may be None)."""
    if np.dtype(data.dtype) == np.uint8:
        acc = ng.quantized_convolution(data, filt, 1.0, 0, 1.0, 0, 1.0, 0, np.int32, stride, dilation, pad_below, pad_above, data_dilation)
    else:
        # i8 activations: INTERPRETER's QuantizedConvolution takes u8 data only, its plain Convolution on
        # i32 (reference::convolution<int32_t>, same loop nest) gives the same exact accumulators
        acc = ng.convolution(ng.convert(data, np.int32), ng.convert(filt, np.int32), stride, dilation, pad_below, pad_above, data_dilation)
    y = _tail(acc, bias, scale, 1, np.int8 if signed else out_dtype, relu, sum_in, sum_scale)
    return ng.convert(y, np.uint8) if signed and np.dtype(out_dtype) == np.uint8 else y


def decomposed_dot_bias(x, w, bias, scale, out_dtype, relu):
    """Oracle graph of QuantizedDotBias: data [M,K], weights [N,K]."""
    m, k = x.shape
    n = w.shape[0]
    x32 = ng.convert(x, np.int32)
    w32 = ng.reshape(ng.convert(w, np.int32), (1, 0), (k, n))
    return _tail(ng.dot(x32, w32, 1), bias, scale, 1, out_dtype, relu)
