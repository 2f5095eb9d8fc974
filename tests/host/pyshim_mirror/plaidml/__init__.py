"""`plaidml` as an alias of this repository's own Python package, so that code written against the reference's Python
API -- its test modules -- runs on `plaidml_b200.{core,edsl,exec,op}` unmodified: the same names one level up."""

import sys
import types

import plaidml_b200
from plaidml_b200 import core, edsl, op
from plaidml_b200 import exec as _exec
from plaidml_b200.core import Buffer, DType, Program, TensorShape, list_targets
from plaidml_b200.ffi import Error

exec = _exec

settings = types.ModuleType("plaidml.settings")
settings.set = core.settings_set
settings.get = core.settings_get

for _name, _module in (("settings", settings), ("edsl", edsl), ("exec", _exec), ("op", op), ("core", core)):
    sys.modules["plaidml." + _name] = _module
