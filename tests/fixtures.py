"""Loading of the committed golden fixtures (tests/golden/*.json)."""
import json
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NP = {"u8": np.uint8, "i8": np.int8, "i32": np.int32, "f32": np.float32, "i64": np.int64}


def blob(b):
    """{"dtype","shape","data"} -> ndarray; f32 data are stored as uint32 bit patterns."""
    if b["dtype"] == "f32":
        a = np.array(b["data"], dtype=np.uint32).view(np.float32)
    else:
        a = np.array(b["data"], dtype=NP[b["dtype"]])
    return a.reshape(b["shape"])


def typed(v, shape=None):
    """{"dtype","data"} of the reference-test fixtures (values, not bit patterns)."""
    a = np.array(v["data"], dtype=NP[v["dtype"]])
    return a if shape is None else a.reshape(shape)


def f32_from_bits(bits):
    return np.array([bits], dtype=np.uint32).view(np.float32)[0]


_cache = {}


def interpreter_cases(op=None):
    if "interp" not in _cache:
        with open(os.path.join(GOLDEN, "interpreter_cases.json")) as f:
            _cache["interp"] = json.load(f)
    return [c for c in _cache["interp"] if op is None or c["op"] == op or (isinstance(op, tuple) and c["op"] in op)]


def reference_tests(op=None):
    if "ref" not in _cache:
        with open(os.path.join(GOLDEN, "reference_tests.json")) as f:
            _cache["ref"] = json.load(f)
    return [c for c in _cache["ref"] if op is None or c["op"] == op or (isinstance(op, tuple) and c["op"] in op)]
