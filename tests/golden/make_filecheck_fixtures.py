"""Extracts the FileCheck expectations that the reference's C++ EDSL tests embed as comments
(plaidml/edsl/tests/edsl_test.cc: `// CHECK...` lines after each program is built) into
tests/golden/edsl_filecheck.json, one list of [directive, pattern] per test name.

    python tests/golden/make_filecheck_fixtures.py <path to a plaidml checkout>

Only the tests named in WANTED are taken (those with expectations worth replaying)."""

import json
import os
import re
import sys

WANTED = [
    "SimpleTensor", "ConstAdd", "Dot", "DotF16", "DoubleDot", "EltwiseAdd", "EltwiseMod", "Relu", "MnistMlp",
    "Convolution", "MnistCnn", "RepeatElements", "GlobalMin", "CumSum", "ComplexConv2d", "Reciprocal",
    "DefractLong", "Select", "ConvI8", "UniqueNames", "dup_out", "HigherPrecisionConstants", "LarsMomentum4d",
    "ReshapeFold", "ReshapeScalar", "ReshapeIntoScalar", "ReshapeFromScalar", "Shape", "Trace",
    "Layer", "LayerOperandOrder", "LayerEmbeddedConst", "LayerUnusedOperand", "LayerMultipleReturnValues", "LayerMulti",
    "LayerException",
    "Prng", "ArgSort1d", "ArgSort1dInt", "ArgSort1dDup", "ArgSort2dAxis0", "ArgSort2dAxis1", "ArgSort3dAxis0Asc",
    "ArgSort3dAxis2Desc", "ArgSort3dAxisNeg2Asc",
]


def main() -> None:
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    src = os.path.join(sys.argv[1], "plaidml", "edsl", "tests", "edsl_test.cc")
    out = {}
    name = None
    for line in open(src):
        m = re.match(r"\s*// (CHECK(?:-[A-Z]+)?): ?(.*)$", line.rstrip("\n"))
        if not m:
            continue
        directive, pattern = m.group(1), m.group(2).strip()
        if directive == "CHECK-LABEL":
            name = pattern.split("CppEdsl.")[-1].strip()
            continue
        if directive == "CHECK" and pattern.startswith("module @") and name in out:
            name = pattern[len("module @"):].split()[0]      # a test without a label of its own: keyed by its module name
        if name in WANTED:
            out.setdefault(name, []).append([directive, pattern])
    missing = [n for n in WANTED if n not in out]
    if missing:
        sys.exit(f"no CHECK lines found for {missing}")
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "edsl_filecheck.json")
    with open(dst, "w") as f:
        json.dump(out, f, indent=1)
        f.write("\n")
    print(f"{dst}: {sum(len(v) for v in out.values())} directives of {len(out)} tests")


if __name__ == "__main__":
    main()
