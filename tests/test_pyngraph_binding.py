"""The reference's own Python binding (pyngraph, built from the reference's sources by oracle/Makefile.pyngraph) driving the
B200 plugin: what a user of `ngraph.runtime(backend_name=...)` gets when the name is "B200".

* through the compiled binding alone (`_pyngraph`, travels with the repository's built files): Backend.create by name,
  compile, create_tensor, write, call_with_validate, read;
* through the reference's pure-Python API on top of it (`import ngraph`, only where the reference checkout is present).

Nothing of the plugin is special-cased for Python: BackendManager finds lib<name>_backend.so beside libngraph.so (a link
into ngraph_b200/) exactly as it finds the INTERPRETER."""
import ctypes
import glob
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINDING_DIR = os.path.join(ROOT, "oracle", "_ref", "python")
from ngraph_b200.build import ngraph_checkout  # noqa: E402

REFERENCE_PY = os.path.join(ngraph_checkout() or "", "python", "src")

pytestmark = pytest.mark.skipif(not glob.glob(os.path.join(BINDING_DIR, "_pyngraph*.so")),
                                reason="the reference's Python binding has not been built (oracle/Makefile.pyngraph)")


@pytest.fixture(scope="module")
def p():
    sys.path.insert(0, BINDING_DIR)
    try:
        import _pyngraph
    finally:
        sys.path.remove(BINDING_DIR)
    return _pyngraph


def relu_plus(p):
    """f(a, b) = relu(a) * b + a, built with the binding's NodeFactory like ngraph/ops.py does"""
    a, b = p.op.Parameter(p.Type.f32, p.Shape([4, 6])), p.op.Parameter(p.Type.f32, p.Shape([4, 6]))
    nf = p.NodeFactory("opset3")
    y = nf.create("Add", [nf.create("Multiply", [nf.create("Relu", [a], {}), b], {}), a], {})
    return p.Function([y], [a, b], "relu_plus")


def run(p, backend, fn, *arrays):
    exe = backend.compile(fn)
    ins = []
    for x in arrays:
        t = backend.create_tensor(p.Type.f32, p.Shape(list(x.shape)))
        t.write(p.util.numpy_to_c(np.ascontiguousarray(x)), x.nbytes)
        ins.append(t)
    out_t = backend.create_tensor(p.Type.f32, p.Shape(list(arrays[0].shape)))
    exe.call_with_validate([out_t], ins)
    out = np.empty(arrays[0].shape, np.float32)
    out_t.read(p.util.numpy_to_c(out), out.nbytes)
    return out


def inputs():
    rng = np.random.default_rng(0)
    return rng.standard_normal((4, 6)).astype(np.float32), rng.standard_normal((4, 6)).astype(np.float32)


def test_binding_runs_the_interpreter(p):
    a, b = inputs()
    got = run(p, p.runtime.Backend.create("INTERPRETER"), relu_plus(p), a, b)
    np.testing.assert_array_equal(got, np.maximum(a, 0) * b + a)


def test_backend_create_by_name_reaches_the_plugin(p):
    """without a device the plugin's own constructor refuses: the name was resolved, the library loaded and registered"""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    if not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "lib", "libb200_backend.so")):
        pytest.skip("the plugin is not linked beside libngraph.so")
    with pytest.raises(RuntimeError) as e:
        p.runtime.Backend.create("B200")
    assert str(e.value).startswith("B200 backend:"), str(e.value)
    with pytest.raises(RuntimeError) as e:
        p.runtime.Backend.create("NOSUCHBACKEND")
    assert "Unable to find backend 'NOSUCHBACKEND'" in str(e.value)


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE_PY, "ngraph")), reason="the reference checkout is not on this machine")
def test_reference_python_api_finds_the_plugin():
    """`import ngraph` (the reference's package, unmodified) in a fresh interpreter"""
    script = r'''
import sys, warnings
warnings.simplefilter("ignore")
sys.path[:0] = [%r, %r]
import numpy as np
import ngraph as ng
a = ng.parameter([2, 3], name="a", dtype=np.float32)
rt = ng.runtime(backend_name="INTERPRETER")
print("INTERPRETER", rt.computation(ng.relu(a), a)(np.array([[1, -2, 3], [-4, 5, -6]], np.float32))[0].tolist())
try:
    rt = ng.runtime(backend_name="B200")
    print("B200 created")
except RuntimeError as e:
    print("B200 refused:", e)
''' % (BINDING_DIR, REFERENCE_PY)
    out = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=300, cwd="/tmp")
    if "No module named 'pkg_resources'" in out.stderr:
        pytest.skip("the reference's package imports pkg_resources, which this Python no longer ships")
    assert out.returncode == 0, out.stderr[-2000:]
    assert "INTERPRETER [[1.0, 0.0, 3.0], [0.0, 5.0, 0.0]]" in out.stdout
    assert "B200 created" in out.stdout or "B200 refused: B200 backend:" in out.stdout, out.stdout


@pytest.mark.gpu
def test_binding_runs_the_plugin_on_the_device(p):
    if not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "lib", "libb200_backend.so")):
        # no link beside libngraph.so on this machine: register the plugin the static way first
        lib = ctypes.CDLL(os.path.join(ROOT, "ngraph_b200", "libb200_backend.so"), mode=ctypes.RTLD_GLOBAL)
        lib.ngraph_register_b200_backend()
    a, b = inputs()
    fn = relu_plus(p)
    got = run(p, p.runtime.Backend.create("B200"), fn, a, b)
    want = run(p, p.runtime.Backend.create("INTERPRETER"), fn, a, b)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
