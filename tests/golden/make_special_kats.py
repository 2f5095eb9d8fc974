"""Extracts the known-answer vectors of the reference's tests for gather / scatter / argsort / prng
(plaidml/edsl/tests/edsl_test.cc) into ``reference_special_kats.json`` next to this script.

    python tests/golden/make_special_kats.py /path/to/plaidml

The test sources are read AS TEXT.  Per test the file records the placeholders (name, element type, shape) and
every ``std::vector`` initialiser of the test body; ``tests/test_oracle_special.py`` knows which operation each
test builds (written there with the line it restates) and which vectors are its inputs and expected output.
"""

import json
import re
import sys
from pathlib import Path

from make_reference_kats import cpp_vectors

TESTS = (
    ["Prng", "Gather", "GatherND", "GatherNDWithBatchDims"]
    + ["InterpolatedGather" + s for s in ("Nearest", "Linear", "LinearOutOfBoundsReturnZero", "Cubic",
                                          "CubicOutOfBoundsReturnZero", "CubicDouble", "CubicHalf", "MultiDIndices")]
    + ["Scatter" + s for s in ("1D", "3D", "Dup1D", "Dup3D", "1DUpdateSlice", "3DUpdateSlice", "NDUpdateSlice",
                               "NDUpdateSlice2", "NDUpdateSlice3", "Elt")]
    + ["ArgSort" + s for s in ("1d", "1dInt", "1dDup", "2dAxis0", "2dAxis1", "3dAxis0Asc", "3dAxis2Desc", "3dAxisNeg2Asc")]
)


def main(ref_root: str) -> None:
    src = "plaidml/edsl/tests/edsl_test.cc"
    text = (Path(ref_root) / src).read_text()
    out = {}
    for name in TESTS:
        head = "TEST_F(CppEdsl, " + name + ")"
        start = text.index(head)
        body = text[start:text.index("\nTEST_F", start + 1)]
        holders = {m.group(1): {"dtype": m.group(2), "shape": [int(t) for t in m.group(3).split(",") if t.strip()]}
                   for m in re.finditer(r"auto (\w+) = Placeholder\(DType::(\w+), \{([^}]*)\}\)", body)}
        out[name] = {"source": f"{src}:{text[:start].count(chr(10)) + 1}", "placeholders": holders,
                     "vectors": {k: v["values"] for k, v in cpp_vectors(text, head).items()}}
    dst = Path(__file__).resolve().parent / "reference_special_kats.json"
    dst.write_text(json.dumps(out) + "\n")
    print(f"wrote {len(out)} tests to {dst}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_special_kats.py <checkout of plaidml/plaidml>")
    main(sys.argv[1])
