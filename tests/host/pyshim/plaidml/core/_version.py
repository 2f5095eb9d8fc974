"""Stand-in for the file the reference's build generates from plaidml/core/_version.in.py.  The build stamps the
package and the library with one version string; here the package's copy is read from the library it will bind."""

import ctypes
import os


class _Error(ctypes.Structure):
    _fields_ = [("code", ctypes.c_size_t), ("msg", ctypes.c_void_p)]


def _library_version() -> str:
    lib = ctypes.CDLL(os.environ["PLAIDML_LIB_PATH"])
    lib.plaidml_version.restype = ctypes.c_char_p
    lib.plaidml_version.argtypes = [ctypes.POINTER(_Error)]
    err = _Error()
    return lib.plaidml_version(ctypes.byref(err)).decode()


PLAIDML_VERSION = _library_version()
