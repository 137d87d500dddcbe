"""numpy-facing wrappers over the C oracle (``ngraph_oracle.c``).  Test infrastructure only.

Every function mirrors one entry of ``libngraph_oracle.so`` and takes/returns numpy arrays in
nGraph's public layouts (NCHW data, KCRS filters, [M,K]x[K,N] for QuantizedDot, [N,K] weights
for QuantizedDotBias).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

U8, I8, I32, F32 = 0, 1, 2, 3
_DT = {np.dtype(np.uint8): U8, np.dtype(np.int8): I8, np.dtype(np.int32): I32, np.dtype(np.float32): F32}
_NP = {U8: np.uint8, I8: np.int8, I32: np.int32, F32: np.float32}


def build():
    """Compile the C restatement with gcc (a second or two)."""
    subprocess.check_call(["make", "-s", "-C", _HERE], stdout=subprocess.DEVNULL)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libngraph_oracle.so")
        src = os.path.join(_HERE, "ngraph_oracle.c")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
            build()
        _LIB = ctypes.CDLL(path)
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _i64(v):
    arr = (ctypes.c_int64 * max(len(v), 1))(*v)
    return arr


def _c(a, dtype=None):
    a = np.ascontiguousarray(a) if dtype is None else np.ascontiguousarray(a, dtype=dtype)
    return a


class ConvShape(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in ("N", "C", "H", "W", "K", "R", "S", "stride_h", "stride_w", "pad_h",
                                              "pad_w", "pad_h_above", "pad_w_above", "dil_h", "dil_w")]


def conv_shape(data_shape, filt_shape, stride=(1, 1), pad_below=(0, 0), pad_above=None, dilation=(1, 1)):
    pad_above = pad_below if pad_above is None else pad_above
    n, c, h, w = data_shape
    k, c2, r, s = filt_shape
    assert c == c2
    return ConvShape(n, c, h, w, k, r, s, stride[0], stride[1], pad_below[0], pad_below[1], pad_above[0],
                     pad_above[1], dilation[0], dilation[1])


def conv_out_hw(cs):
    p, q = ctypes.c_int64(), ctypes.c_int64()
    lib().ora_conv_out_shape(ctypes.byref(cs), ctypes.byref(p), ctypes.byref(q))
    return p.value, q.value


def quantize(x, scale, zero_point, axes=(), round_mode=4):
    x = _c(x, np.float32)
    scale = _c(scale, np.float32)
    zero_point = _c(zero_point)
    qt = _DT[zero_point.dtype]
    out = np.empty(x.shape, dtype=zero_point.dtype)
    lib().ora_quantize(_p(x), _p(scale), _p(zero_point), _p(out), qt, _i64(x.shape), x.ndim, _i64(list(axes)),
                       len(axes), int(round_mode))
    return out


def dequantize(x, scale, zero_point, axes=()):
    x = _c(x)
    scale = _c(scale, np.float32)
    zero_point = _c(zero_point, x.dtype)
    out = np.empty(x.shape, dtype=np.float32)
    lib().ora_dequantize(_p(x), _p(scale), _p(zero_point), _p(out), _DT[x.dtype], _i64(x.shape), x.ndim,
                         _i64(list(axes)), len(axes))
    return out


def qdot_core(a, b, sa, za, sb, zb, so, zo, out_dtype):
    a, b = _c(a), _c(b)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    out = np.empty((m, n), dtype=out_dtype)
    lib().ora_qdot_core(_p(a), _DT[a.dtype], _p(b), _DT[b.dtype], _p(out), _DT[out.dtype], ctypes.c_int64(m),
                        ctypes.c_int64(k), ctypes.c_int64(n), ctypes.c_float(sa), ctypes.c_int32(za),
                        ctypes.c_float(sb), ctypes.c_int32(zb), ctypes.c_float(so), ctypes.c_int32(zo))
    return out


def qgemm_fused(a, w, bias, scale, out_dtype, relu=False, sum_in=None, sum_scale=0.0):
    a, w = _c(a), _c(w, np.int8)
    m, k = a.shape
    n, k2 = w.shape
    assert k == k2
    bias = None if bias is None else _c(bias, np.int32)
    scale = _c(np.atleast_1d(scale), np.float32)
    sum_in = None if sum_in is None else _c(sum_in)
    out = np.empty((m, n), dtype=out_dtype)
    lib().ora_qgemm_fused(_p(a), _DT[a.dtype], _p(w), _p(bias), _p(scale), ctypes.c_int64(scale.size), _p(sum_in),
                          0 if sum_in is None else _DT[sum_in.dtype], ctypes.c_float(sum_scale), int(relu), _p(out),
                          _DT[out.dtype], ctypes.c_int64(m), ctypes.c_int64(n), ctypes.c_int64(k))
    return out


def qgemm_core(a, w, scale, out_zp, out_dtype):
    a, w = _c(a), _c(w, np.int8)
    m, k = a.shape
    n, _ = w.shape
    out = np.empty((m, n), dtype=out_dtype)
    lib().ora_qgemm_core(_p(a), _DT[a.dtype], _p(w), ctypes.c_float(scale), ctypes.c_int32(out_zp), _p(out),
                         _DT[out.dtype], ctypes.c_int64(m), ctypes.c_int64(n), ctypes.c_int64(k))
    return out


def qconv_core(data, filt, cs, sd, zd, sf, zf, so, zo, out_dtype):
    data, filt = _c(data), _c(filt)
    p, q = conv_out_hw(cs)
    out = np.empty((cs.N, cs.K, p, q), dtype=out_dtype)
    lib().ora_qconv_core(_p(data), _DT[data.dtype], _p(filt), _DT[filt.dtype], _p(out), _DT[out.dtype],
                         ctypes.byref(cs), ctypes.c_float(sd), ctypes.c_int32(zd), ctypes.c_float(sf),
                         ctypes.c_int32(zf), ctypes.c_float(so), ctypes.c_int32(zo))
    return out


def qconv_fused(data, filt, bias, scale, cs, out_dtype, relu=False, sum_in=None, sum_scale=0.0):
    data, filt = _c(data), _c(filt, np.int8)
    bias = None if bias is None else _c(bias, np.int32)
    scale = _c(np.atleast_1d(scale), np.float32)
    sum_in = None if sum_in is None else _c(sum_in)
    p, q = conv_out_hw(cs)
    out = np.empty((cs.N, cs.K, p, q), dtype=out_dtype)
    lib().ora_qconv_fused(_p(data), _DT[data.dtype], _p(filt), _p(bias), _p(scale), ctypes.c_int64(scale.size),
                          _p(sum_in), 0 if sum_in is None else _DT[sum_in.dtype], ctypes.c_float(sum_scale),
                          int(relu), _p(out), _DT[out.dtype], ctypes.byref(cs))
    return out


def maxpool_u8(x, window, stride, pad_below, pad_above):
    x = _c(x, np.uint8)
    n, c, h, w = x.shape
    p = (h + pad_below[0] + pad_above[0] - window[0]) // stride[0] + 1
    q = (w + pad_below[1] + pad_above[1] - window[1]) // stride[1] + 1
    out = np.empty((n, c, p, q), dtype=np.uint8)
    args = [n, c, h, w, window[0], window[1], stride[0], stride[1], pad_below[0], pad_below[1], pad_above[0],
            pad_above[1]]
    lib().ora_maxpool_u8(_p(x), _p(out), *[ctypes.c_int64(v) for v in args])
    return out


def global_avgpool_q(x, s_in, s_out):
    """Dequantize -> AvgPool(f32, whole H x W window) -> Quantize(RNE), the u8 pooling head.

    AvgPool follows runtime::reference::avg_pool (src/ngraph/runtime/reference/avg_pool.hpp:
    sequential float sum in H,W order, then one division by the element count)."""
    x = _c(x, np.uint8)
    n, c, h, w = x.shape
    f = dequantize(x, np.float32(s_in), np.uint8(0)).reshape(n * c, h * w)
    acc = np.zeros(n * c, dtype=np.float32)
    for i in range(h * w):
        acc = (acc + f[:, i]).astype(np.float32)
    avg = (acc / np.float32(h * w)).astype(np.float32)
    return quantize(avg.reshape(n, c, 1, 1), np.float32(s_out), np.uint8(0))
