"""b200_qconv_stem_static through the C ABI: the stem convolution whose scratch cell grid is a fixed device array inside the
library, for callers that must not enter an allocator (a serving loop with a fixed memory budget, a region where
cudaMalloc would synchronise the device).  Checked on two calls in a row with different inputs against the caller-allocated
path (b200_stem_pack_input + b200_qconv_stem) and against the CPU oracle, for leaving the device's free memory untouched,
at the largest batch the array holds, and for refusing anything beyond it before a kernel is queued.
Collected last on purpose: it must pass after every other test has used the device as well as alone."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _prepare(ops, data, filt, scale, bias, pad, relu=True):
    """everything a call needs, allocated BEFORE the call: packed filters, the output and the epilogue record"""
    from ngraph_b200.lib import LIB, check
    n, c, h, w = data.shape
    k, _, r, s = filt.shape
    p, q, hc, wc, rc = ops.stem_geometry(h, w, r, s, pad, pad)
    packed = np.empty((k, rc * 64), np.int8)
    check(LIB.b200_stem_pack_filter_host(filt.ctypes.data, packed.ctypes.data, k, c, r, s, pad[0], pad[1]), "pack filter")
    packed_d = torch.from_numpy(packed).cuda()
    out = torch.empty((n, p, q, k), dtype=torch.uint8, device="cuda")
    e, keep = ops._epilogue(k, scale, torch.uint8, bias, relu)
    return packed_d, out, e, keep


def _call_static(lib, data, packed_d, out, e, filt_shape, pad):
    n, c, h, w = data.shape
    k, _, r, s = filt_shape
    status = lib.LIB.b200_qconv_stem_static(data.data_ptr(), lib.U8 if data.dtype == torch.uint8 else lib.I8,
                                            packed_d.data_ptr(), out.data_ptr(), n, c, h, w, k, r, s, pad[0], pad[1], pad[0], pad[1],
                                            ctypes.byref(e), torch.cuda.current_stream().cuda_stream)
    torch.cuda.current_stream().synchronize()
    return status


def _oracle(data, filt, bias, scale, pad):
    from oracle import ref
    cs = ref.conv_shape(data.shape, filt.shape, (2, 2), pad, pad)
    return ref.qconv_fused(data, filt, bias, scale, cs, np.uint8, relu=True).transpose(0, 2, 3, 1)  # NCHW -> [N,P,Q,K]


def _weights(rng):
    filt = rng.integers(-127, 128, (64, 3, 7, 7)).astype(np.int8)
    bias = rng.integers(-2000, 2000, 64).astype(np.int32)
    scale = (rng.uniform(0.5, 1.5, 64) * 255.0 / (147 * 127 * 40)).astype(np.float32)
    return filt, bias, scale


def test_static_scratch_stem_matches_allocated_path_and_oracle_twice():
    from ngraph_b200 import lib, ops
    rng = np.random.default_rng(2024)
    filt, bias, scale = _weights(rng)
    bias_d, scale_d = torch.from_numpy(bias).cuda(), torch.from_numpy(scale).cuda()
    # two calls in a row, different inputs and sizes: the second must not see anything of the first
    for shape in ((3, 3, 64, 48), (2, 3, 40, 72)):
        host = rng.integers(0, 256, shape).astype(np.uint8)
        data = torch.from_numpy(host).cuda()
        packed_d, got, e, keep = _prepare(ops, data, filt, scale_d, bias_d, (3, 3))
        status = _call_static(lib, data, packed_d, got, e, filt.shape, (3, 3))
        assert status == 0, lib.LIB.b200_status_string(status)
        want = ops.qconv_stem(data, filt, scale_d, torch.uint8, (3, 3), bias=bias_d, relu=True)
        assert torch.equal(got, want)
        np.testing.assert_array_equal(got.cpu().numpy(), _oracle(host, filt, bias, scale, (3, 3)))
    lib.device_status()


def test_static_scratch_call_leaves_free_device_memory_unchanged():
    """The property the entry point exists for: between "everything prepared" and "result ready" the device's free memory
    does not move (cudaMemGetInfo through torch), i.e. no allocation was made on the caller's behalf."""
    from ngraph_b200 import lib, ops
    rng = np.random.default_rng(7)
    filt, bias, scale = _weights(rng)
    bias_d, scale_d = torch.from_numpy(bias).cuda(), torch.from_numpy(scale).cuda()
    data = torch.from_numpy(rng.integers(0, 256, (4, 3, 96, 96)).astype(np.uint8)).cuda()
    packed_d, out, e, keep = _prepare(ops, data, filt, scale_d, bias_d, (3, 3))
    assert _call_static(lib, data, packed_d, out, e, filt.shape, (3, 3)) == 0  # first call on the device: symbol set-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    for _ in range(3):
        assert _call_static(lib, data, packed_d, out, e, filt.shape, (3, 3)) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before and torch.cuda.memory_reserved() == reserved_before


def test_static_scratch_at_the_largest_batch_it_holds():
    """224x224 images, as many as the 16 MiB array takes: the last cells of the grid sit right below the slack the kernel may
    read past them.  First and last image against the oracle, all of them against the allocated path."""
    from ngraph_b200 import lib, ops
    cap = lib.LIB.b200_qconv_stem_static_capacity()
    p, q, hc, wc, rc = ops.stem_geometry(224, 224, 7, 7, (3, 3), (3, 3))
    n = (cap - 2112) // (hc * wc * 16)
    rng = np.random.default_rng(5)
    filt, bias, scale = _weights(rng)
    bias_d, scale_d = torch.from_numpy(bias).cuda(), torch.from_numpy(scale).cuda()
    host = rng.integers(0, 256, (n, 3, 224, 224)).astype(np.uint8)
    data = torch.from_numpy(host).cuda()
    packed_d, got, e, keep = _prepare(ops, data, filt, scale_d, bias_d, (3, 3))
    status = _call_static(lib, data, packed_d, got, e, filt.shape, (3, 3))
    assert status == 0, lib.LIB.b200_status_string(status)
    assert torch.equal(got, ops.qconv_stem(data, filt, scale_d, torch.uint8, (3, 3), bias=bias_d, relu=True))
    ends = np.ascontiguousarray(host[[0, n - 1]])
    np.testing.assert_array_equal(got[[0, n - 1]].cpu().numpy(), _oracle(ends, filt, bias, scale, (3, 3)))
    lib.device_status()


def test_static_scratch_capacity_and_arguments_are_checked_before_any_launch():
    from ngraph_b200 import lib, ops
    cap = lib.LIB.b200_qconv_stem_static_capacity()
    assert cap == 16 << 20
    p, q, hc, wc, rc = ops.stem_geometry(224, 224, 7, 7, (3, 3), (3, 3))
    too_many = (cap - 2112) // (hc * wc * 16) + 1
    # refused before any launch: the pointers are never touched
    e, keep = ops._epilogue(64, torch.ones(1, device="cuda"), torch.uint8)
    before = lib.launch_count()
    status = lib.LIB.b200_qconv_stem_static(None, lib.U8, None, None, too_many, 3, 224, 224, 64, 7, 7, 3, 3, 3, 3,
                                            ctypes.byref(e), None)
    assert status == -3  # B200_ERR_TOO_LARGE
    assert b"size limit" in lib.LIB.b200_status_string(status).lower()
    # bad arguments of the convolution itself are found before the pack kernel is queued into the shared array
    x = torch.zeros((1, 3, 32, 32), dtype=torch.uint8, device="cuda")
    for args in ((x.data_ptr(), 3, None, None, 1, 3, 32, 32, 64),          # data type that is neither u8 nor i8
                 (x.data_ptr(), lib.U8, None, None, 1, 3, 32, 32, 0),       # no output channels
                 (x.data_ptr(), lib.U8, None, None, 1, 5, 32, 32, 64),      # more channels than a cell holds
                 (x.data_ptr(), lib.U8, None, None, 1, 3, 32, 32, 64)):     # null filters / output
        assert lib.LIB.b200_qconv_stem_static(*args, 7, 7, 3, 3, 3, 3, ctypes.byref(e), None) == -1
    assert lib.launch_count() == before
