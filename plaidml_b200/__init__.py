"""plaidml_b200: a B200-native execution backend for PlaidML's Tile contraction path.

``libplaidml.so`` (built by ``python -m plaidml_b200.build``) exports the reference's C ABI
with a ``cuda`` target and ``cuda.N`` devices; this package is its Python face:

* ``plaidml_b200.edsl``  -- ``Tensor``, ``TensorDim``, ``TensorIndex``, ``Contraction`` ...
* ``plaidml_b200.op``    -- the operation library (convolution, pool, dot, relu, mean, ...)
* ``plaidml_b200.exec``  -- ``Executable``, ``list_devices``
* ``plaidml_b200.kernels`` -- the kernel-level C ABI (dispatch / invoke on raw device pointers)

Importing the sub-modules loads the shared library; there is no fallback if it is missing.
"""

__version__ = "0.1.0"


def __getattr__(name):
    # Lazy so that `import plaidml_b200.build` works before the library exists.
    if name in ("DType", "TensorShape", "Buffer", "Program", "list_targets", "settings_get", "settings_set"):
        from . import core
        return getattr(core, name)
    if name == "Error":
        from .ffi import Error
        return Error
    raise AttributeError(name)


def init():
    from .ffi import ffi_call, lib
    ffi_call(lib.plaidml_init)
    ffi_call(lib.plaidml_edsl_init)
    ffi_call(lib.plaidml_exec_init)
