"""Writes unit_test.manifest for the B200 backend: the names of nGraph's backend-parametrised tests
(test/backend/*.in.cpp, NGRAPH_TEST(${BACKEND_NAME}, name)) that are to be SKIPPED when that suite is configured for
"B200" (test/CMakeLists.txt:486-515 picks the file up from the backend's directory; test/util/test_control.cpp reads one
name per line, '#' starts a comment).

Enabled (= not listed) are exactly the tests whose inputs and expected outputs this repository carries as fixtures
(tests/golden/reference_tests.json) and reproduces on the device in its own GPU tests; every other test is listed,
because it either uses ops outside the quantized-inference path or has not been run against this backend.

    python ngraph_b200/backend/make_manifest.py [--ref /path/to/ngraph]
"""
import argparse
import glob
import json
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def main():
    ap = argparse.ArgumentParser()
    from ngraph_b200.build import ngraph_checkout
    ap.add_argument("--ref", default=ngraph_checkout(), help="root of the nGraph checkout (default: $NGRAPH_REF or the reference build recipe's)")
    a = ap.parse_args()
    verified = {c["name"] for c in json.load(open(os.path.join(ROOT, "tests", "golden", "reference_tests.json")))}
    per_file = {}
    for path in sorted(glob.glob(os.path.join(a.ref, "test", "backend", "*.in.cpp"))):
        names = re.findall(r"NGRAPH_TEST\(\$\{BACKEND_NAME\},\s*(\w+)\)", open(path).read())
        per_file[os.path.basename(path)] = names
    enabled = sorted(n for names in per_file.values() for n in names if n in verified)
    with open(os.path.join(HERE, "unit_test.manifest"), "w") as f:
        f.write("# B200 backend: tests of nGraph's backend suite to skip (written by make_manifest.py).\n")
        f.write("# Not listed, i.e. enabled: the %d tests this repository reproduces on the device from its fixtures:\n" % len(enabled))
        for i in range(0, len(enabled), 4):
            f.write("#   " + ", ".join(enabled[i:i + 4]) + "\n")
        for fname, names in per_file.items():
            skip = [n for n in names if n not in verified]
            if not skip:
                continue
            f.write("\n# %s\n" % fname)
            f.write("\n".join(skip) + "\n")
    print("enabled %d, skipped %d" % (len(enabled), sum(len(v) for v in per_file.values()) - len(enabled)))


if __name__ == "__main__":
    main()
