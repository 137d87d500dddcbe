"""b200_qconv_stem_static through the C ABI: the stem convolution whose scratch cell grid is a fixed device array.
Compared with the caller-allocated path (b200_stem_pack_input + b200_qconv_stem) on two calls in a row with
different inputs, and refused beyond the array's capacity.  Collected last on purpose: it must pass after every
other test has used the device as well as alone."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, ops, data, filt, scale, bias, pad, relu=True):
    from ngraph_b200.lib import LIB, check
    n, c, h, w = data.shape
    k, _, r, s = filt.shape
    p, q, hc, wc, rc = ops.stem_geometry(h, w, r, s, pad, pad)
    packed = np.empty((k, rc * 64), np.int8)
    check(LIB.b200_stem_pack_filter_host(filt.ctypes.data, packed.ctypes.data, k, c, r, s, pad[0], pad[1]), "pack filter")
    packed_d = torch.from_numpy(packed).cuda()
    out = torch.empty((n, p, q, k), dtype=torch.uint8, device="cuda")
    e, keep = ops._epilogue(k, scale, torch.uint8, bias, relu)
    status = LIB.b200_qconv_stem_static(data.data_ptr(), lib.U8 if data.dtype == torch.uint8 else lib.I8,
                                        packed_d.data_ptr(), out.data_ptr(), n, c, h, w, k, r, s, pad[0], pad[1], pad[0], pad[1],
                                        ctypes.byref(e), torch.cuda.current_stream().cuda_stream)
    torch.cuda.current_stream().synchronize()
    return status, out


def test_static_scratch_stem_matches_allocated_path_twice():
    from ngraph_b200 import lib, ops
    rng = np.random.default_rng(2024)
    filt = rng.integers(-127, 128, (64, 3, 7, 7)).astype(np.int8)
    bias = torch.from_numpy(rng.integers(-2000, 2000, 64).astype(np.int32)).cuda()
    scale = torch.from_numpy((rng.uniform(0.5, 1.5, 64) * 255.0 / (147 * 127 * 40)).astype(np.float32)).cuda()
    # two calls in a row, different inputs and sizes: the second must not see anything of the first
    for shape in ((3, 3, 64, 48), (2, 3, 40, 72)):
        data = torch.from_numpy(rng.integers(0, 256, shape).astype(np.uint8)).cuda()
        status, got = _call_static(lib, ops, data, filt, scale, bias, (3, 3))
        assert status == 0, lib.LIB.b200_status_string(status)
        want = ops.qconv_stem(data, filt, scale, torch.uint8, (3, 3), bias=bias, relu=True)
        assert torch.equal(got, want)
    lib.device_status()


def test_static_scratch_capacity_is_enforced():
    from ngraph_b200 import lib, ops
    cap = lib.LIB.b200_qconv_stem_static_capacity()
    assert cap == 16 << 20
    p, q, hc, wc, rc = ops.stem_geometry(224, 224, 7, 7, (3, 3), (3, 3))
    too_many = (cap - 2112) // (hc * wc * 16) + 1
    # refused before any launch: the pointers are never touched
    e, keep = ops._epilogue(64, torch.ones(1, device="cuda"), torch.uint8)
    status = lib.LIB.b200_qconv_stem_static(None, lib.U8, None, None, too_many, 3, 224, 224, 64, 7, 7, 3, 3, 3, 3,
                                            ctypes.byref(e), None)
    assert status == -3  # B200_ERR_TOO_LARGE
    assert b"size limit" in lib.LIB.b200_status_string(status).lower()
