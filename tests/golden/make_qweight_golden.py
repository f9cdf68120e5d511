"""Extracts the literal known-answer vector of the reference's QWeight layout test into a fixture.

Source: test/QWeightTestData.cs:13-173 of GilesBathgate/ManagedLlama2 (128 packed weight words,
8 zero nibbles and their packed word, 8 scales given as fp32 bit patterns, 1024 expected
dequantised values given as fp32 bit patterns), consumed by Test_QWeight_FromData,
test/QWeightTests.cs:29-48. Only the numbers are taken; run it where the reference checkout is
available:

    python tests/golden/make_qweight_golden.py /path/to/ManagedLlama2 > tests/golden/qweight_fromdata.json
"""
import json
import re
import os
import sys


def parse(path):
    text = open(path, encoding="utf-8-sig").read()

    def array(name):
        m = re.search(r"\b" + name + r"\s*=\s*new\s+uint\[(\d+)\]\s*\{(.*?)\};", text, re.S)
        n = int(m.group(1))
        vals = [int(t.rstrip("u"), 0) for t in re.findall(r"0x[0-9a-fA-F]+|\d+u?", m.group(2))]
        assert len(vals) == n, (name, len(vals), n)
        return vals

    zero = int(re.search(r"\bzero\s*=\s*(\d+)\s*;", text).group(1))
    return {
        "source": "test/QWeightTestData.cs:13-173",
        "zero_packed": zero,
        "zeros": array("zeros"),
        "scales_f32_bits": array("scales"),
        "weights": array("weights"),
        "checks_f32_bits": array("checks"),
    }


if __name__ == "__main__":
    # the reference checkout: first argument, else ML2_REFERENCE_ROOT, else a `reference` directory beside this repository
    here = os.path.dirname(os.path.abspath(__file__))
    root = sys.argv[1] if len(sys.argv) > 1 else (os.environ.get("ML2_REFERENCE_ROOT") or
                                                  os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(here))), "reference"))
    json.dump(parse(root + "/test/QWeightTestData.cs"), sys.stdout, separators=(",", ":"))
    sys.stdout.write("\n")
