"""CPU oracle for the quantized-inference path (test infrastructure only).

``oracle.ref`` exposes numpy-facing wrappers over ``libngraph_oracle.so`` (the C
restatement in ``ngraph_oracle.c``).  Only tests, the smoke test and the bench's
CPU-baseline leg import this package; the product (``ngraph_b200``) never does.
"""
