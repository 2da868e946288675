"""camel_b200: B200 (sm_100a) kernels behind the operator surface of Camel's `tensor` module.

`camel_b200.tensor` mirrors the reference operators (add, matmul, sum, ...); `camel_b200._lib`
is the raw ctypes binding of the C ABI declared in include/camel_tensor_b200.h;
`camel_b200.build` compiles the library.  The library is loaded on first use of anything but
`build`, so that `python -m camel_b200.build` works before it exists.
"""
import importlib

_LAZY = {
    "tensor": ("camel_b200.tensor", None),
    "_lib": ("camel_b200._lib", None),
    "lib": ("camel_b200._lib", "lib"),
    "CamelTensorError": ("camel_b200._lib", "CamelTensorError"),
    "Tensor": ("camel_b200.tensor", "Tensor"),
    "from_numpy": ("camel_b200.tensor", "from_numpy"),
    "wrap_device": ("camel_b200.tensor", "wrap_device"),
}


def __getattr__(name):
    if name in _LAZY:
        mod, attr = _LAZY[name]
        m = importlib.import_module(mod)
        return m if attr is None else getattr(m, attr)
    raise AttributeError(f"module 'camel_b200' has no attribute {name!r}")
