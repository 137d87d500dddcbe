"""The give-up path of the kernels' bounded waits, on a device and without faulting, trapping or hanging it: a one-warp
self-test kernel (b200_selftest_bounded_wait) waits, through the same ptx::mbar_wait the contraction kernel's roles use, on
an mbarrier that nothing arrives at, with a limit of about a millisecond.  It must return by itself, leave code 9001 in the
device status word, b200_device_status must report it exactly once, the plugin's Tensor::read must turn it into an
exception exactly once, and the next kernels must run as if nothing had happened."""
import ctypes
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _stream():
    return torch.cuda.current_stream().cuda_stream


def test_wait_runs_out_status_is_latched_once_and_the_context_stays_usable():
    from ngraph_b200 import lib, ops
    lib.device_status()  # clean to begin with
    t0 = time.time()
    assert lib.LIB.b200_selftest_bounded_wait(1_000_000, _stream()) == 0
    torch.cuda.synchronize()  # returns: the wait gave up by itself
    assert time.time() - t0 < 5.0
    code = ctypes.c_int(0)
    assert lib.LIB.b200_device_status(ctypes.byref(code)) == -4  # B200_ERR_DEVICE_STATUS
    assert code.value == 9001
    assert lib.LIB.b200_device_status(ctypes.byref(code)) == 0 and code.value == 0  # reported once, then clear
    with pytest.raises(RuntimeError):
        assert lib.LIB.b200_selftest_bounded_wait(1_000_000, _stream()) == 0
        lib.device_status()  # the Python wrapper raises on a latched status
    # the same context runs a contraction right afterwards, bit-exact
    from oracle import ref
    rng = np.random.default_rng(3)
    a = rng.integers(0, 256, (130, 256)).astype(np.uint8)
    w = rng.integers(-127, 128, (80, 256)).astype(np.int8)
    s = np.array([3e-4], np.float32)
    got = ops.qgemm(torch.from_numpy(a).cuda(), torch.from_numpy(w).cuda(), torch.from_numpy(s).cuda(), torch.uint8, relu=True)
    np.testing.assert_array_equal(got.cpu().numpy(), ref.qgemm_fused(a, w, None, s, np.uint8, relu=True))
    lib.device_status()


def test_bad_limits_are_refused_on_the_host():
    from ngraph_b200 import lib
    before = lib.launch_count()
    assert lib.LIB.b200_selftest_bounded_wait(0, None) == -1
    assert lib.LIB.b200_selftest_bounded_wait(10_000_000_000, None) == -1  # seconds-long waits are not offered
    assert lib.launch_count() == before


def test_plugin_tensor_read_throws_once_after_a_wait_ran_out():
    ng = pytest.importorskip("ngraph_b200.ngraph_api")
    from oracle import interpreter
    if not interpreter.available():
        pytest.skip("nGraph host library not built here")
    from ngraph_b200 import lib
    ng.load_b200()
    be = ng.Backend("B200")
    p = ng.parameter(np.float32, (4, 64))
    exe = be.compile(ng.Function([ng.relu(p)], [p]))
    x = np.linspace(-1, 1, 256, dtype=np.float32).reshape(4, 64)
    tin, tout = ng.Tensor(be, np.float32, x.shape), ng.Tensor(be, np.float32, x.shape)
    tin.write(x)
    exe.call([tout], [tin])
    assert lib.LIB.b200_selftest_bounded_wait(500_000, None) == 0
    with pytest.raises(ng.NgraphError, match="bounded wait"):
        tout.read()
    np.testing.assert_array_equal(tout.read(), np.maximum(x, 0))  # cleared by the first report; the data are intact
    exe.call([tout], [tin])
    np.testing.assert_array_equal(tout.read(), np.maximum(x, 0))
