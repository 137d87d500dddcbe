"""B200 (sm_100a) quantized-inference backend for nGraph.

The product is native: ``libb200_kernels.so`` (CUDA kernels behind the C ABI of
``include/b200_kernels.h``) and ``libb200_backend.so`` (the nGraph ``runtime::Backend`` plugin).
This Python package only builds them (``ngraph_b200.build``) and binds the C ABI with ctypes
(``ngraph_b200.lib``, ``ngraph_b200.ops``) for the tests and the benchmark; torch is used for
device memory and streams only.  ``ngraph_b200.lib`` raises on import when the native library
is missing or stale: there is no fallback.
"""
