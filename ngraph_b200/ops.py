"""torch-tensor-facing wrappers over the C ABI (device pointers + the current CUDA stream).

torch supplies device memory and streams; every computation below is one call into
``libb200_kernels.so``.  Names and argument meaning follow the nGraph ops they run
(``op::v0::Quantize``, ``Dequantize``, ``QuantizedDotBias``, ``QuantizedConvolutionBias`` ...).
"""
import ctypes

import torch

from . import lib
from .lib import F32, I8, I32, LIB, U8, ConvParams, Epilogue, check

_DT = {torch.uint8: U8, torch.int8: I8, torch.int32: I32, torch.float32: F32}
_TORCH = {U8: torch.uint8, I8: torch.int8, I32: torch.int32, F32: torch.float32}


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _i64(v):
    return (ctypes.c_int64 * max(len(v), 1))(*[int(x) for x in v])


def _dev(t, dtype=None):
    assert t.is_cuda, "b200 ops take CUDA tensors"
    if dtype is not None:
        assert t.dtype == dtype, (t.dtype, dtype)
    return t.contiguous()


def quantize(x, scale, zero_point, axes=(), round_mode=4, out=None):
    """op::v0::Quantize(x, scale, zero_point, type=zero_point.dtype, axes, round_mode)."""
    x, scale, zero_point = _dev(x, torch.float32), _dev(scale, torch.float32), _dev(zero_point)
    out = torch.empty(x.shape, dtype=zero_point.dtype, device=x.device) if out is None else out
    axes = sorted(int(a) for a in axes)
    check(LIB.b200_quantize(_ptr(x), _ptr(scale), _ptr(zero_point), _ptr(out), _DT[zero_point.dtype], _i64(x.shape),
                            x.dim(), _i64(axes), len(axes), int(round_mode), _stream()), "b200_quantize")
    return out


def dequantize(x, scale, zero_point, axes=(), out=None):
    """op::v0::Dequantize(x, scale, zero_point, f32, axes)."""
    x, scale, zero_point = _dev(x), _dev(scale, torch.float32), _dev(zero_point)
    assert zero_point.dtype == x.dtype
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device) if out is None else out
    axes = sorted(int(a) for a in axes)
    check(LIB.b200_dequantize(_ptr(x), _ptr(scale), _ptr(zero_point), _ptr(out), _DT[x.dtype], _i64(x.shape), x.dim(),
                              _i64(axes), len(axes), _stream()), "b200_dequantize")
    return out


WEIGHTS_U8 = 0x100


def _operands(data, weights):
    """data type code, plus the flag for unsigned weights"""
    return _DT[data.dtype] | (WEIGHTS_U8 if weights.dtype == torch.uint8 else 0)


def _epilogue(n_out, scale, out_dtype, bias=None, relu=False, sum_in=None, sum_scale=None, core=False, out_zp=0):
    scale = _dev(scale, torch.float32)
    keep = [scale]
    e = Epilogue()
    e.scale = scale.data_ptr()
    e.scale_count = scale.numel()
    if bias is not None:
        bias = _dev(bias, torch.int32)
        keep.append(bias)
        e.bias = bias.data_ptr()
    if sum_in is not None:
        sum_in = _dev(sum_in)
        sum_scale = _dev(sum_scale, torch.float32)
        keep += [sum_in, sum_scale]
        e.sum_in = sum_in.data_ptr()
        e.sum_type = _DT[sum_in.dtype]
        e.sum_scale = sum_scale.data_ptr()
    e.relu = int(bool(relu))
    e.round_half_away = int(bool(core))
    e.out_zero_point = int(out_zp)
    e.out_type = _DT[out_dtype]
    return e, keep


def pack_weights(w, bk):
    """Host int8 [N,K] matrix (numpy or CPU tensor) -> device tensor holding the packed image for k-blocks of bk bytes."""
    import numpy as np
    w = np.ascontiguousarray(w.cpu().numpy() if isinstance(w, torch.Tensor) else w).view(np.int8)
    n, k = w.shape
    packed = np.empty(LIB.b200_packed_weights_bytes(n, k, bk), np.int8)
    check(LIB.b200_pack_weights_host(w.ctypes.data, packed.ctypes.data, n, k, bk), "b200_pack_weights_host")
    return torch.from_numpy(packed).cuda()


def qgemm(a, w, scale, out_dtype, bias=None, relu=False, sum_in=None, sum_scale=None, core=False, out_zp=0, out=None,
          packed=False):
    """out[M,N] = epilogue(a[M,K] @ w[N,K]^T): QuantizedDotBias (fused contract) or, with core=True,
    QuantizedDot's requantisation on a pre-transposed B.  packed=True sends the weights through the packed image."""
    a, w = _dev(a), _dev(w)
    assert w.dtype in (torch.int8, torch.uint8)
    m, k = a.shape
    n, k2 = w.shape
    assert k == k2
    e, keep = _epilogue(n, scale, out_dtype, bias, relu, sum_in, sum_scale, core, out_zp)
    out = torch.empty((m, n), dtype=out_dtype, device=a.device) if out is None else out
    if packed:
        pw = pack_weights(w, 128)
        check(LIB.b200_qgemm_packed(_ptr(a), _operands(a, w), _ptr(pw), _ptr(out), m, n, k, ctypes.byref(e), _stream()),
              "b200_qgemm_packed")
        torch.cuda.current_stream().synchronize()  # pw is released on return
        return out
    check(LIB.b200_qgemm(_ptr(a), _operands(a, w), _ptr(w), _ptr(out), m, n, k, ctypes.byref(e), _stream()), "b200_qgemm")
    return out


def conv_params(data_shape_nhwc, filt_shape_krsc, stride=(1, 1), pad_below=(0, 0), pad_above=None, dilation=(1, 1)):
    pad_above = pad_below if pad_above is None else pad_above
    n, h, w, c = data_shape_nhwc
    k, r, s, c2 = filt_shape_krsc
    assert c == c2
    return ConvParams(n, h, w, c, k, r, s, stride[0], stride[1], pad_below[0], pad_below[1], pad_above[0], pad_above[1],
                      dilation[0], dilation[1])


def conv_out_hw(cp):
    p, q = ctypes.c_int64(), ctypes.c_int64()
    check(LIB.b200_qconv_out_shape(ctypes.byref(cp), ctypes.byref(p), ctypes.byref(q)), "b200_qconv_out_shape")
    return p.value, q.value


def qconv(data, filters, scale, out_dtype, cp, bias=None, relu=False, sum_in=None, sum_scale=None, core=False, out_zp=0,
          out=None, packed=False):
    """Channels-last int8 convolution with the fused epilogue: data [N,H,W,C], filters [K,R,S,C] -> [N,P,Q,K]."""
    data, filters = _dev(data), _dev(filters)
    assert filters.dtype in (torch.int8, torch.uint8)
    e, keep = _epilogue(cp.K, scale, out_dtype, bias, relu, sum_in, sum_scale, core, out_zp)
    p, q = conv_out_hw(cp)
    out = torch.empty((cp.N, p, q, cp.K), dtype=out_dtype, device=data.device) if out is None else out
    if packed:
        pw = filters if packed == "prepacked" else pack_weights(filters.reshape(cp.K, -1), LIB.b200_qconv_weight_block(cp.C))
        check(LIB.b200_qconv_packed(_ptr(data), _operands(data, filters), _ptr(pw), _ptr(out), ctypes.byref(cp), ctypes.byref(e),
                                    _stream()), "b200_qconv_packed")
        if packed != "prepacked":
            torch.cuda.current_stream().synchronize()  # pw is released on return
        return out
    check(LIB.b200_qconv(_ptr(data), _operands(data, filters), _ptr(filters), _ptr(out), ctypes.byref(cp), ctypes.byref(e),
                         _stream()), "b200_qconv")
    return out


def stem_geometry(h, w, r, s, pad_below, pad_above):
    vals = [ctypes.c_int64() for _ in range(5)]
    check(LIB.b200_stem_geometry(h, w, r, s, pad_below[0], pad_below[1], pad_above[0], pad_above[1],
                                 *[ctypes.byref(v) for v in vals]), "b200_stem_geometry")
    return tuple(v.value for v in vals)  # P, Q, Hc, Wc, Rc


def qconv_stem(data_nchw, filters_kcrs, scale, out_dtype, pad_below, pad_above=None, bias=None, relu=False):
    """Stride-2 convolution over <= 4 channels: NCHW one-byte data, host KCRS int8 filters (numpy) -> [N,P,Q,K]."""
    import numpy as np
    pad_above = pad_below if pad_above is None else pad_above
    data = _dev(data_nchw)
    n, c, h, w = data.shape
    f = np.ascontiguousarray(filters_kcrs, dtype=np.int8)
    k, c2, r, s = f.shape
    assert c == c2
    p, q, hc, wc, rc = stem_geometry(h, w, r, s, pad_below, pad_above)
    packed = np.empty((k, rc * 64), np.int8)
    check(LIB.b200_stem_pack_filter_host(f.ctypes.data, packed.ctypes.data, k, c, r, s, pad_below[0], pad_below[1]),
          "b200_stem_pack_filter_host")
    packed_d = torch.from_numpy(packed).to(data.device)
    cells = torch.empty(LIB.b200_stem_cells_bytes(n, h, w, r, s, pad_below[0], pad_below[1], pad_above[0], pad_above[1]),
                        dtype=torch.uint8, device=data.device)
    check(LIB.b200_stem_pack_input(_ptr(data), _ptr(cells), n, c, h, w, r, s, pad_below[0], pad_below[1], pad_above[0],
                                   pad_above[1], _stream()), "b200_stem_pack_input")
    e, keep = _epilogue(k, scale, out_dtype, bias, relu)
    out = torch.empty((n, p, q, k), dtype=out_dtype, device=data.device)
    check(LIB.b200_qconv_stem(_ptr(cells), _DT[data.dtype], _ptr(packed_d), _ptr(out), n, h, w, k, r, s, pad_below[0],
                              pad_below[1], pad_above[0], pad_above[1], ctypes.byref(e), _stream()), "b200_qconv_stem")
    return out


def nchw_to_nhwc(x, c_pad=None):
    x = _dev(x)
    assert x.element_size() == 1
    n, c, h, w = x.shape
    c_pad = c if c_pad is None else c_pad
    out = torch.empty((n, h, w, c_pad), dtype=x.dtype, device=x.device)
    check(LIB.b200_nchw_to_nhwc_u8(_ptr(x), _ptr(out), n, c, h, w, c_pad, _stream()), "b200_nchw_to_nhwc_u8")
    return out


def nhwc_to_nchw(x, c=None):
    x = _dev(x)
    assert x.element_size() == 1
    n, h, w, c_pad = x.shape
    c = c_pad if c is None else c
    out = torch.empty((n, c, h, w), dtype=x.dtype, device=x.device)
    check(LIB.b200_nhwc_to_nchw_u8(_ptr(x), _ptr(out), n, c, h, w, c_pad, _stream()), "b200_nhwc_to_nchw_u8")
    return out


def transpose_u8(x):
    x = _dev(x)
    assert x.element_size() == 1 and x.dim() == 2
    r, c = x.shape
    out = torch.empty((c, r), dtype=x.dtype, device=x.device)
    check(LIB.b200_transpose_u8(_ptr(x), _ptr(out), r, c, _stream()), "b200_transpose_u8")
    return out


def maxpool_nhwc(x, window, stride, pad_below=(0, 0), pad_above=None):
    x = _dev(x, torch.uint8)
    pad_above = pad_below if pad_above is None else pad_above
    n, h, w, c = x.shape
    p = (h + pad_below[0] + pad_above[0] - window[0]) // stride[0] + 1
    q = (w + pad_below[1] + pad_above[1] - window[1]) // stride[1] + 1
    out = torch.empty((n, p, q, c), dtype=torch.uint8, device=x.device)
    check(LIB.b200_maxpool_nhwc_u8(_ptr(x), _ptr(out), n, h, w, c, window[0], window[1], stride[0], stride[1],
                                   pad_below[0], pad_below[1], pad_above[0], pad_above[1], _stream()),
          "b200_maxpool_nhwc_u8")
    return out


def global_avgpool_q(x, scale_in, scale_out):
    x = _dev(x, torch.uint8)
    n, h, w, c = x.shape
    out = torch.empty((n, c), dtype=torch.uint8, device=x.device)
    check(LIB.b200_global_avgpool_q_nhwc_u8(_ptr(x), _ptr(out), _ptr(_dev(scale_in, torch.float32)),
                                            _ptr(_dev(scale_out, torch.float32)), n, h, w, c, _stream()),
          "b200_global_avgpool_q_nhwc_u8")
    return out
