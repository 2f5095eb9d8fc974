"""Stand-in for the module the reference's build generates with cffi (`plaidml._ffi`, CMakeLists.txt: NAME _ffi MODULE
plaidml._ffi): the declarations of the C ABI, here taken from this repository's include/plaidml_ffi.h.  The header's
path comes from PLAIDML_FFI_HEADER (set by the test that assembles the package)."""

import os
import re

import cffi

ffi = cffi.FFI()


def _declarations() -> str:
    text = open(os.environ["PLAIDML_FFI_HEADER"]).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    keep = []
    for line in text.splitlines():
        s = line.strip()
        if s.startswith("#") or s == 'extern "C" {' or s == "}":
            continue
        keep.append(line)
    return "\n".join(keep)


ffi.cdef(_declarations())
