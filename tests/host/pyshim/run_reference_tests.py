"""Runs test modules of the reference's Python package (assembled as byte code next to this file's stand-ins) with
unittest and prints one line per test.

    python run_reference_tests.py [--build-only] module [module ...]

--build-only: no device is used -- `plaidml.exec.run` and `Executable.run` compile the program for the target and
return zero-filled outputs, and value comparisons of the test fixture are skipped; the tests then check that every
program builds, prints and compiles through the reference's own Python API.
"""

import sys
import unittest

import numpy as np


def build_only_patches():
    import plaidml
    import plaidml.exec

    def run(program, inputs, device=''):
        program.compile()
        return [np.zeros(shape.sizes, dtype=shape.dtype.into_numpy()) for shape in program.outputs]

    def compile_only(self, program, device=''):
        program.compile()

    plaidml.exec.run = run
    plaidml.exec.Executable.__init__ = compile_only
    plaidml.exec.Executable.run = lambda self, inputs, outputs: None
    unittest.TestCase.assertEqual = lambda self, first, second, msg=None: None
    unittest.TestCase.assertTrue = lambda self, expr, msg=None: None


class Lines(unittest.TextTestResult):
    def addSuccess(self, test):
        super().addSuccess(test)
        print("[  OK ]", test.id(), flush=True)

    def addFailure(self, test, err):
        super().addFailure(test, err)
        print("[ FAIL]", test.id(), flush=True)

    def addError(self, test, err):
        super().addError(test, err)
        print("[ FAIL]", test.id(), flush=True)

    def addSkip(self, test, reason):
        super().addSkip(test, reason)
        print("[ SKIP]", test.id(), reason, flush=True)


def main(argv):
    build_only = "--build-only" in argv
    modules = [a for a in argv[1:] if not a.startswith("--")]
    if build_only:
        build_only_patches()
    suite = unittest.TestSuite()
    for name in modules:
        suite.addTests(unittest.defaultTestLoader.loadTestsFromName(name))
    result = unittest.TextTestRunner(resultclass=Lines, verbosity=0, stream=sys.stderr).run(suite)
    print(f"{result.testsRun} tests, {len(result.failures) + len(result.errors)} failures" + (" (build only)" if build_only else ""))
    return 0 if result.wasSuccessful() else 1


if __name__ == "__main__":
    sys.exit(main(sys.argv))
