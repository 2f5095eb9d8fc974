"""cffi (ABI mode) loader for ``libplaidml.so``.

Same role as the reference's ``plaidml/ffi.py:18-107``: locate the shared library (next to the
package, or ``$PLAIDML_LIB_PATH``), ``cdef`` the C ABI, and turn ``plaidml_error`` results into
Python exceptions.  The declarations come straight from ``include/plaidml_ffi.h`` with the
preprocessor lines removed, so the Python side can never drift from the header.
"""

from __future__ import annotations

import os
import re
import threading
from pathlib import Path

import cffi

_PKG = Path(__file__).resolve().parent
_HEADER = _PKG.parent / "include" / "plaidml_ffi.h"

ffi = cffi.FFI()


def _cdef_source() -> str:
    text = _HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    lines = []
    for line in text.splitlines():
        s = line.strip()
        if s.startswith("#") or s == 'extern "C" {' or s == "}":
            continue
        lines.append(line)
    return "\n".join(lines)


ffi.cdef(_cdef_source())


def _library_path() -> Path:
    override = os.environ.get("PLAIDML_LIB_PATH")
    return Path(override) if override else _PKG / "libplaidml.so"


def _load():
    path = _library_path()
    if not path.exists():
        raise ImportError(
            f"{path} not found. Build it with `python -m plaidml_b200.build`; the cuda target has no "
            "pure-Python or CPU fallback.")
    return ffi.dlopen(str(path))


lib = _load()

_tls = threading.local()


class Error(Exception):
    """An error reported through ``plaidml_error``."""


def _error_slot():
    err = getattr(_tls, "err", None)
    if err is None:
        err = ffi.new("plaidml_error*")
        _tls.err = err
    return err


def decode_str(ptr) -> str:
    """Copies and frees a ``plaidml_string*``."""
    if ptr == ffi.NULL:
        return ""
    try:
        return ffi.string(lib.plaidml_string_ptr(ptr)).decode()
    finally:
        lib.plaidml_string_free(ptr)


def ffi_call(func, *args):
    """Calls ``func(err, *args)`` and raises :class:`Error` if it reports one."""
    err = _error_slot()
    ret = func(err, *args)
    if err.code:
        raise Error(decode_str(err.msg))
    return ret


class ForeignObject:
    """Owns one C handle; ``__ffi_del__`` names its release function."""

    __ffi_del__ = None
    __ffi_repr__ = None

    def __init__(self, ffi_obj):
        self._ffi_obj = ffi_obj

    def __del__(self):
        obj = getattr(self, "_ffi_obj", None)
        if obj is not None and obj != ffi.NULL and self.__ffi_del__ is not None:
            try:
                self.__ffi_del__(_error_slot(), obj)
            except Exception:  # interpreter shutdown
                pass
            self._ffi_obj = None

    def as_ptr(self):
        return self._ffi_obj if self._ffi_obj is not None else ffi.NULL

    def take_ptr(self):
        obj, self._ffi_obj = self._ffi_obj, None
        return obj

    def __repr__(self):
        if self.__ffi_repr__ is None or self._ffi_obj is None:
            return super().__repr__()
        return decode_str(self.__ffi_repr__(_error_slot(), self.as_ptr()))


def get_strings(func) -> list[str]:
    """Decodes a ``plaidml_strings*`` result (the list does not own its elements)."""
    raw = ffi_call(func)
    try:
        return [decode_str(raw.elts[i]) for i in range(raw.size)]
    finally:
        ffi_call(lib.plaidml_strings_free, raw)
