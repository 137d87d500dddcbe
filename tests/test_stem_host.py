"""Host side of the stride-2 small-channel (stem) convolution: the cell-grid geometry and the filter
packing of the C ABI, checked on the CPU by carrying out the cell-grid convolution in numpy and
comparing its int32 sums with the oracle's convolution (no GPU code runs here)."""
import ctypes

import numpy as np
import pytest

from oracle import ref

CASES = [
    (2, 3, 32, 32, 8, 7, 7, (3, 3), (3, 3)),
    (1, 1, 17, 23, 4, 3, 3, (1, 1), (1, 1)),
    (2, 4, 20, 18, 5, 5, 7, (2, 3), (1, 2)),
    (1, 2, 16, 16, 3, 8, 8, (0, 0), (0, 0)),
    (1, 3, 9, 9, 2, 7, 7, (2, 2), (3, 3)),
    (1, 3, 12, 10, 2, 1, 1, (0, 0), (0, 0)),
]


@pytest.fixture(scope="module")
def klib():
    from ngraph_b200 import lib
    return lib.LIB


def cells_of(data, hc, wc, pad_h, pad_w):
    """numpy statement of the cell grid b200_stem_pack_input writes: [N, Hc, Wc, (dy, dx, 4 channels)]."""
    n, c, h, w = data.shape
    eh, ew = pad_h + (pad_h & 1), pad_w + (pad_w & 1)
    big = np.zeros((n, 4, 2 * hc, 2 * wc), data.dtype)
    hh, ww = min(h, 2 * hc - eh), min(w, 2 * wc - ew)
    big[:, :c, eh:eh + hh, ew:ew + ww] = data[:, :, :hh, :ww]
    return big.reshape(n, 4, hc, 2, wc, 2).transpose(0, 2, 4, 3, 5, 1).reshape(n, hc, wc, 16)


@pytest.mark.parametrize("case", CASES, ids=lambda c: "x".join(str(v) for v in c[:7]))
def test_cell_grid_convolution_matches_oracle(klib, case):
    n, c, h, w, k, r, s, pb, pa = case
    rng = np.random.default_rng(7)
    data = rng.integers(0, 256, (n, c, h, w)).astype(np.uint8)
    filt = rng.integers(-127, 128, (k, c, r, s)).astype(np.int8)
    vals = [ctypes.c_int64() for _ in range(5)]
    assert klib.b200_stem_geometry(h, w, r, s, pb[0], pb[1], pa[0], pa[1], *[ctypes.byref(v) for v in vals]) == 0
    p, q, hc, wc, rc = (v.value for v in vals)
    packed = np.empty((k, rc, 64), np.int8)
    assert klib.b200_stem_pack_filter_host(filt.ctypes.data, packed.ctypes.data, k, c, r, s, pb[0], pb[1]) == 0
    cells = cells_of(data, hc, wc, pb[0], pb[1]).astype(np.int32)
    flat = cells.reshape(n, hc, wc * 16)
    acc = np.zeros((n, p, q, k), np.int64)
    for rr in range(rc):
        for qq in range(q):
            window = flat[:, rr:rr + p, qq * 16:qq * 16 + 64]  # 4 neighbouring cells
            acc[:, :, qq, :] += window @ packed[:, rr, :].astype(np.int32).T
    cs = ref.conv_shape(data.shape, filt.shape, (2, 2), pb, pa)
    exp = ref.qconv_fused(data, filt, None, np.float32(1.0), cs, np.int32)
    np.testing.assert_array_equal(acc.transpose(0, 3, 1, 2), exp)


def test_geometry_rejects_wide_filters(klib):
    vals = [ctypes.c_int64() for _ in range(5)]
    assert klib.b200_stem_geometry(32, 32, 9, 9, 0, 0, 0, 0, *[ctypes.byref(v) for v in vals]) != 0
