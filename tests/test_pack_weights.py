"""The packed weight image of the C ABI (host function, no GPU): every source byte lands at the offset the
kernel's shared-memory layout expects, padding is zero."""
import numpy as np
import pytest


@pytest.fixture(scope="module")
def klib():
    from ngraph_b200 import lib
    return lib.LIB


@pytest.mark.parametrize("n,k,bk", [(64, 128, 128), (100, 200, 128), (1, 16, 64), (130, 576, 64), (256, 1152, 128)])
def test_pack_weights_layout(klib, n, k, bk):
    rng = np.random.default_rng(n + k)
    w = rng.integers(-127, 128, (n, k)).astype(np.int8)
    size = klib.b200_packed_weights_bytes(n, k, bk)
    nb, kbs = (n + 63) // 64, (k + bk - 1) // bk
    assert size == nb * 64 * kbs * bk
    packed = np.full(size, 77, np.int8)
    assert klib.b200_pack_weights_host(w.ctypes.data, packed.ctypes.data, n, k, bk) == 0
    img = packed.reshape(kbs, nb, 64, bk // 16, 16)
    # undo the 16-byte piece swizzle: piece p of row r is stored at p ^ f(r)
    r = np.arange(64)
    flip = (r & 7) if bk == 128 else ((r >> 1) & 3)
    plain = np.empty_like(img)
    for piece in range(bk // 16):
        plain[:, :, r, piece, :] = img[:, :, r, piece ^ flip, :]
    full = plain.reshape(kbs, nb * 64, bk).transpose(1, 0, 2).reshape(nb * 64, kbs * bk)
    np.testing.assert_array_equal(full[:n, :k], w)
    assert not full[n:].any() and not full[:, k:].any()


def test_pack_weights_rejects_bad_block(klib):
    assert klib.b200_packed_weights_bytes(64, 64, 32) == 0
    w = np.zeros((4, 16), np.int8)
    assert klib.b200_pack_weights_host(w.ctypes.data, w.ctypes.data, 4, 16, 32) != 0
