"""ngraph_b200/backend/unit_test.manifest: the skip list for nGraph's backend-parametrised gtest suite.  It must leave
enabled exactly the reference tests whose vectors tests/golden/reference_tests.json carries (the ones the GPU tests
reproduce) and skip every other test of test/backend/*.in.cpp."""
import glob
import json
import os
import re

import pytest

from ngraph_b200.build import ngraph_checkout

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MANIFEST = os.path.join(ROOT, "ngraph_b200", "backend", "unit_test.manifest")


def skipped_names():
    return [l.strip() for l in open(MANIFEST) if l.strip() and not l.startswith("#")]


def test_manifest_keeps_the_reproduced_tests_enabled():
    skipped = skipped_names()
    assert len(skipped) == len(set(skipped)) > 1000
    verified = {c["name"] for c in json.load(open(os.path.join(ROOT, "tests", "golden", "reference_tests.json")))}
    assert not verified & set(skipped)
    assert {"quantize", "dequantize_axes", "quantized_convolution", "quantized_dot_u8u8"} <= verified


REFERENCE_TESTS = os.path.join(ngraph_checkout() or "", "test", "backend")


@pytest.mark.skipif(not os.path.isdir(REFERENCE_TESTS), reason="the reference checkout is not on this machine")
def test_manifest_covers_the_whole_backend_suite():
    every = set()
    for path in glob.glob(os.path.join(REFERENCE_TESTS, "*.in.cpp")):
        every |= set(re.findall(r"NGRAPH_TEST\(\$\{BACKEND_NAME\},\s*(\w+)\)", open(path).read()))
    verified = {c["name"] for c in json.load(open(os.path.join(ROOT, "tests", "golden", "reference_tests.json")))}
    assert set(skipped_names()) == every - verified
