"""ctypes binding of the C ABI declared in include/b200_kernels.h.

There is no fallback of any kind: if ``libb200_kernels.so`` has not been built, importing this
module raises; if a call returns a non-zero status, ``check`` raises ``B200Error``.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("B200_KERNELS_LIB", os.path.join(HERE, "libb200_kernels.so"))

U8, I8, I32, F32 = 0, 1, 2, 3


class B200Error(RuntimeError):
    def __init__(self, status, text):
        super().__init__(text)
        self.status = status


class Epilogue(ctypes.Structure):
    _fields_ = [("bias", ctypes.c_void_p), ("scale", ctypes.c_void_p), ("scale_count", ctypes.c_int64),
                ("sum_in", ctypes.c_void_p), ("sum_type", ctypes.c_int), ("sum_scale", ctypes.c_void_p),
                ("relu", ctypes.c_int), ("round_half_away", ctypes.c_int), ("out_zero_point", ctypes.c_int32),
                ("out_type", ctypes.c_int)]


class ConvParams(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in ("N", "H", "W", "C", "K", "R", "S", "stride_h", "stride_w", "pad_h",
                                              "pad_w", "pad_h_above", "pad_w_above", "dilation_h", "dilation_w")]


class PoolParams(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in ("N", "C", "H", "W", "P", "Q", "win_h", "win_w", "stride_h", "stride_w", "pad_h", "pad_w",
                                              "pad_h_above", "pad_w_above")] + [("include_padding", ctypes.c_int32)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError("%s is missing: run `python -m ngraph_b200.build` (needs nvcc); "
                          "there is no CPU or PyTorch fallback" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    vp, i64, ci = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    p64 = ctypes.POINTER(ctypes.c_int64)
    sigs = {
        "b200_status_string": (ctypes.c_char_p, [ci]),
        "b200_last_cuda_error": (ctypes.c_char_p, []),
        "b200_launch_count": (ctypes.c_uint64, []),
        "b200_reset_launch_count": (None, []),
        "b200_device_status": (ci, [ctypes.POINTER(ci)]),
        "b200_set_fast_division": (ci, [ci]),
        "b200_quantize": (ci, [vp, vp, vp, vp, ci, p64, ci, p64, ci, ci, vp]),
        "b200_dequantize": (ci, [vp, vp, vp, vp, ci, p64, ci, p64, ci, vp]),
        "b200_qgemm": (ci, [vp, ci, vp, vp, i64, i64, i64, ctypes.POINTER(Epilogue), vp]),
        "b200_qconv": (ci, [vp, ci, vp, vp, ctypes.POINTER(ConvParams), ctypes.POINTER(Epilogue), vp]),
        "b200_qconv_out_shape": (ci, [ctypes.POINTER(ConvParams), p64, p64]),
        "b200_nchw_to_nhwc_u8": (ci, [vp, vp, i64, i64, i64, i64, i64, vp]),
        "b200_nhwc_to_nchw_u8": (ci, [vp, vp, i64, i64, i64, i64, i64, vp]),
        "b200_transpose_u8": (ci, [vp, vp, i64, i64, vp]),
        "b200_nhwc_to_nchw_b32": (ci, [vp, vp, i64, i64, i64, vp]),
        "b200_maxpool_nhwc_u8": (ci, [vp, vp] + [i64] * 12 + [vp]),
        "b200_maxpool_nhwc_i8": (ci, [vp, vp] + [i64] * 12 + [vp]),
        "b200_global_avgpool_q_nhwc_u8": (ci, [vp, vp, vp, vp, i64, i64, i64, i64, vp]),
        "b200_im2col_c4_u8": (ci, [vp, vp] + [i64] * 11 + [vp]),
        "b200_requant_scale": (ci, [vp, vp, vp, vp, vp]),
        "b200_f32_binary": (ci, [ci, vp, vp, vp, i64, vp]),
        "b200_f32_binary_periodic": (ci, [ci, vp, vp, vp, i64, i64, ci, vp]),
        "b200_f32_unary": (ci, [ci, vp, vp, i64, vp]),
        "b200_broadcast_b32": (ci, [vp, vp, p64, ci, p64, ci, vp]),
        "b200_permute_b32": (ci, [vp, vp, p64, ci, p64, vp]),
        "b200_reduce_f32": (ci, [ci, vp, vp, p64, ci, p64, ci, vp]),
        "b200_strided_sums": (ci, [vp, ci, vp] + [i64] * 6 + [vp]),
        "b200_window_sums": (ci, [vp, vp, vp, vp]),
        "b200_requant_zero_points": (ci, [vp, vp, vp, vp, ctypes.POINTER(Epilogue), vp, vp]),
        "b200_copy_rows": (ci, [vp, vp, i64, i64, i64, vp]),
        "b200_layer_norm_rows_f32": (ci, [vp, vp, vp, vp, i64, i64, ctypes.c_float, vp]),
        "b200_softmax_rows_scaled_f32": (ci, [vp, vp, vp, i64, i64, vp]),
        "b200_layer_norm_rows_sum_f32": (ci, [vp, vp, vp, vp, vp, i64, i64, ctypes.c_float, vp]),
        "b200_gelu_f32": (ci, [vp, vp, i64, vp]),
        "b200_softmax_rows_f32": (ci, [vp, vp, i64, i64, vp]),
        "b200_bmm_f32": (ci, [vp, vp, vp, i64, i64, i64, i64, vp]),
        "b200_gather_rows_b32": (ci, [vp, i64, i64, vp, ci, i64, vp, vp]),
        "b200_packed_weights_bytes": (i64, [i64] * 3),
        "b200_pack_weights_host": (ci, [vp, vp] + [i64] * 3),
        "b200_qconv_weight_block": (i64, [i64]),
        "b200_qgemm_packed": (ci, [vp, ci, vp, vp, i64, i64, i64, ctypes.POINTER(Epilogue), vp]),
        "b200_qconv_packed": (ci, [vp, ci, vp, vp, ctypes.POINTER(ConvParams), ctypes.POINTER(Epilogue), vp]),
        "b200_stem_geometry": (ci, [i64] * 8 + [p64] * 5),
        "b200_stem_cells_bytes": (i64, [i64] * 9),
        "b200_stem_pack_filter_host": (ci, [vp, vp] + [i64] * 6),
        "b200_stem_pack_input": (ci, [vp, vp] + [i64] * 10 + [vp]),
        "b200_stem_pack_input_f32": (ci, [vp, vp, vp, ci, ci, vp] + [i64] * 10 + [vp]),
        "b200_qconv_stem": (ci, [vp, ci, vp, vp] + [i64] * 10 + [ctypes.POINTER(Epilogue), vp]),
        "b200_selftest_bounded_wait": (ci, [i64, vp]),
        "b200_dilate_crop_nhwc_u8": (ci, [vp, vp] + [i64] * 10 + [vp]),
        "b200_avgpool_f32_nchw": (ci, [vp, vp, ctypes.POINTER(PoolParams), vp]),
        "b200_avgpool_nhwc_bytes": (ci, [vp, vp, ci, ctypes.POINTER(PoolParams), vp]),
        "b200_avgpool_q_nhwc": (ci, [vp, ci, vp, ci, vp, vp, ctypes.POINTER(PoolParams), vp]),
        "b200_qconv_stem_static_capacity": (i64, []),
        "b200_qconv_stem_static": (ci, [vp, ci, vp, vp] + [i64] * 11 + [ctypes.POINTER(Epilogue), vp]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


LIB = _load()


def check(status, what=""):
    if status != 0:
        text = LIB.b200_status_string(status).decode()
        if status > 0:
            text += ": " + LIB.b200_last_cuda_error().decode()
        raise B200Error(status, "%s failed: %s" % (what or "b200 call", text))


def device_status():
    """Raises if a kernel reported a bounded-wait timeout; synchronises with the device."""
    code = ctypes.c_int(0)
    st = LIB.b200_device_status(ctypes.byref(code))
    if st != 0:
        raise B200Error(st, "device status word = %d (%s)" % (code.value, LIB.b200_status_string(st).decode()))


def launch_count():
    return int(LIB.b200_launch_count())
