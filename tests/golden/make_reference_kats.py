"""Extracts the known-answer vectors the reference's own tests hold for the contraction path.

Reads the reference's test sources AS TEXT (nothing of the reference is executed; it cannot be
built here) and writes ``reference_kats.json`` next to this script.  Run where the reference
checkout is mounted:  ``python tests/golden/make_reference_kats.py /path/to/plaidml``.
Each entry records the file and the test it came from; ``tests/test_golden_kats.py`` rebuilds
the same programs through this library's EDSL and checks the outputs.
"""

import ast
import json
import re
import sys
from pathlib import Path


def cpp_vectors(text: str, test_name: str) -> dict:
    """All `std::vector<T> name{...}` / `= {...}` initialisers inside one TEST_F body."""
    start = text.index(test_name)
    body = text[start:text.index("\nTEST_F", start + 1) if "\nTEST_F" in text[start + 1:] else len(text)]
    out = {}
    for m in re.finditer(r"std::vector<(\w+)>\s+(\w+)\s*(?:=\s*)?\{([^}]*)\}", body, flags=re.S):
        nums = [t.strip().rstrip("f") for t in re.sub(r"//.*", "", m.group(3)).replace("\n", " ").split(",") if t.strip()]
        out[m.group(2)] = {"ctype": m.group(1), "values": [float(n) if ("." in n or "e" in n.lower()) else int(n) for n in nums]}
    return out


def py_arrays(text: str, test_name: str):
    """The literal lists of the first `checkProgram(program, [inputs], [outputs])` call of a test."""
    start = text.index("def " + test_name + "(")
    body = text[start:]
    call = body.index("self.checkProgram(")
    i = body.index("(", call)
    depth, j = 0, i
    while True:
        if body[j] == "(":
            depth += 1
        elif body[j] == ")":
            depth -= 1
            if depth == 0:
                break
        j += 1
    args = body[i + 1:j]
    args = re.sub(r"np\.array\(", "(", args)
    parsed = ast.literal_eval("(" + args.split(",", 1)[1] + ")")  # drop `program`
    return parsed[0], parsed[1]


def main(ref_root: str) -> None:
    ref = Path(ref_root)
    kats = []
    gemm = (ref / "plaidml/edsl/examples/gemm.cc").read_text()
    for name, dtype in [("GEMM_INT64", "INT64"), ("GEMM_UINT64", "UINT64"), ("GEMM_INT32", "INT32"),
                        ("GEMM_INT8", "INT8"), ("GEMM_FLOAT32", "FLOAT32")]:
        v = cpp_vectors(gemm, "TEST_F(ExampleCppEdsl, " + name + ")")
        kats.append({"name": name, "source": "plaidml/edsl/examples/gemm.cc", "program": "gemm_plus_c", "dtype": dtype,
                     "shape": [3, 3], "inputs": [v["data_A"]["values"], v["data_B"]["values"], v["data_C"]["values"]],
                     "outputs": [v["data_O"]["values"]], "check": "exact"})
    cc = (ref / "plaidml/edsl/tests/edsl_test.cc").read_text()
    v = cpp_vectors(cc, "TEST_F(CppEdsl, Max)")
    kats.append({"name": "Max", "source": "plaidml/edsl/tests/edsl_test.cc", "program": "row_max", "dtype": "FLOAT32",
                 "shape": [3, 3], "inputs": [v["input"]["values"]], "outputs": [v["expected"]["values"]], "check": "exact"})
    v = cpp_vectors(cc, "TEST_F(CppEdsl, SimpleAdd)")
    kats.append({"name": "SimpleAdd", "source": "plaidml/edsl/tests/edsl_test.cc", "program": "add", "dtype": "FLOAT32",
                 "shape": [3, 3], "inputs": [v["A_input"]["values"], v["B_input"]["values"]],
                 "outputs": [v["C_output"]["values"]], "check": "exact"})
    v = cpp_vectors(cc, "TEST_F(CppEdsl, HigherPrecisionConstants)")
    kats.append({"name": "HigherPrecisionConstants", "source": "plaidml/edsl/tests/edsl_test.cc",
                 "program": "higher_precision_constants", "dtype": "FLOAT32", "shape": [3, 3],
                 "inputs": [v["A_input"]["values"]], "outputs": [v["C_output"]["values"]], "check": "exact"})
    py = (ref / "plaidml/edsl/tests/edsl_test.py").read_text()
    for name in ["test_defract", "test_defract_short", "test_defract_long", "test_broadcast_cmp", "test_eltwise",
                 "test_higher_precision_constants"]:
        ins, outs = py_arrays(py, name)
        kats.append({"name": name, "source": "plaidml/edsl/tests/edsl_test.py", "program": name[5:],
                     "inputs": [list(map(lambda a: a, ins))][0], "outputs": outs, "check": "exact"})
    out_path = Path(__file__).resolve().parent / "reference_kats.json"
    out_path.write_text(json.dumps(kats, indent=1))
    print(f"wrote {len(kats)} known-answer tests to {out_path}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_reference_kats.py <checkout of plaidml/plaidml>")
    main(sys.argv[1])
