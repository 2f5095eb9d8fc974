"""Extracts the known-answer vectors the reference's own tests hold for the contraction path.

Reads the reference's test sources AS TEXT (nothing of the reference is executed; it cannot be
built here) and writes ``reference_kats.json`` next to this script.  Run where the reference
checkout is mounted:  ``python tests/golden/make_reference_kats.py /path/to/plaidml``.
Each entry records the file and the test it came from; ``tests/test_oracle_golden.py`` pins the CPU
checker to them and ``tests/test_gpu_edsl.py`` rebuilds the same programs through this library's EDSL and
checks the outputs on the GPU.

A second file, ``reference_xsmm_kats.json``, holds the two printed results of the reference's x86
microkernel test (``pmlc/target/x86/tests/xsmm_call.mlir``): an 8 x 8 dot product and a 1x1 convolution
1x6x5x7 (*) 1x1x7x11, the only convolution numbers the reference's tests contain.  Their inputs are not
literals there but two fill functions, restated below; all values are small integers, so every correct
implementation reproduces the printed matrices exactly in any float type.
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


def mlir_check_rows(text: str, start_marker: str, end_marker: str) -> list:
    """The numbers of the `// CHECK: [a, b, ...]` lines between two markers, one list per line."""
    body = text[text.index(start_marker):]
    body = body[:body.index(end_marker)]
    rows = []
    for line in body.splitlines():
        m = re.search(r"//\s*CHECK:\s*\[+([^\]]*)\]", line)
        if m:
            rows.append([int(t) for t in m.group(1).replace(" ", "").split(",") if t])
    return rows


def fill_2d(rows: int, cols: int, alt: bool) -> list:
    """xsmm_call.mlir:98-116 (@fill_2d): v = x + y + (alt ? x * cols + y : 0) - 5."""
    return [[x + y + ((x * cols + y) if alt else 0) - 5 for y in range(cols)] for x in range(rows)]


def fill_4d(shape, alt: bool) -> list:
    """xsmm_call.mlir:118-142 (@fill_4d): v = x + y + z + w + (alt ? x * Y + y * W + z * W + w : 0) - 5 (the linear
    term is written exactly like that in the test, with W twice)."""
    X, Y, Z, W = shape
    return [[[[x + y + z + w + ((x * Y + y * W + z * W + w) if alt else 0) - 5 for w in range(W)] for z in range(Z)]
             for y in range(Y)] for x in range(X)]


def xsmm_kats(ref: Path) -> list:
    src = "pmlc/target/x86/tests/xsmm_call.mlir"
    text = (ref / src).read_text()
    dot = mlir_check_rows(text, "func @test_dot(", "func @dot(")
    conv = mlir_check_rows(text, "func @test_conv2(", "func @conv2(")
    assert len(dot) == 8 and all(len(r) == 8 for r in dot)
    assert len(conv) == 30 and all(len(r) == 11 for r in conv)
    return [
        {"name": "xsmm_dot_8x8", "source": src + ":144-172", "what": "C[i,j] += A[i,k] * B[k,j], f32",
         "inputs": [fill_2d(8, 8, False), fill_2d(8, 8, True)], "outputs": [dot], "check": "exact"},
        {"name": "xsmm_conv_1x1", "source": src + ":213-262", "what": "O[0,x,y,co] += I[0,x,y,ci] * K[0,0,ci,co], f32",
         "inputs": [fill_4d((1, 6, 5, 7), False), fill_4d((1, 1, 7, 11), True)],
         "outputs": [[conv[5 * x:5 * x + 5] for x in range(6)]], "check": "exact"},
    ]


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
    xs = xsmm_kats(ref)
    xs_path = Path(__file__).resolve().parent / "reference_xsmm_kats.json"
    xs_path.write_text(json.dumps(xs))
    print(f"wrote {len(xs)} microkernel known-answer tests to {xs_path}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_reference_kats.py <checkout of plaidml/plaidml>")
    main(sys.argv[1])
