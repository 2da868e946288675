"""Host-side mirror of the reference `tensor` module's operator surface.

Each function has the name, argument meaning and error text of the operator it mirrors in
OpenCML/Camel's modules/tensor/operators.cpp (URI `tensor:<name>`), unpacks its arguments the
way the reference operator body does, and calls the C ABI of libcamel_tensor_b200.so.  All
arithmetic happens on the GPU; nothing here computes.

Tensors are device-resident (`Tensor.ptr` is a device pointer); `from_numpy` / `numpy()` are
the explicit host<->device transfers of a graph boundary.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence, Union

import numpy as np

from . import _lib as L
from ._lib import CamelTensorError, check, lib

Number = Union[int, float, bool]

_NP = {L.F32: np.float32, L.I64: np.int64, L.BOOL: np.uint8}
_SIZE = {L.F32: 4, L.I64: 8, L.BOOL: 1}


def _invalid(msg: str) -> CamelTensorError:
    return CamelTensorError(L.ERR_INVALID, msg)


def _normalize_np(a: np.ndarray) -> tuple[np.ndarray, int]:
    """normalizeTensorDType, modules/tensor/runtime.cpp:553-566."""
    if a.dtype in (np.float32, np.float64):
        return np.ascontiguousarray(a, dtype=np.float32), L.F32
    if a.dtype in (np.int32, np.int64):
        return np.ascontiguousarray(a, dtype=np.int64), L.I64
    if a.dtype in (np.bool_, np.uint8):
        return np.ascontiguousarray(a.astype(np.uint8) != 0, dtype=np.uint8), L.BOOL
    raise _invalid("Unsupported Tensor dtype")


class Tensor:
    """Device-resident counterpart of TensorObject (modules/tensor/runtime.h:55-109)."""

    __slots__ = ("dtype", "shape", "ptr", "_owns", "_keep", "_packed")

    def __init__(self, dtype: int, shape: Sequence[int], ptr: int | None = None, keep=None):
        self._packed = None  # {precision: handle} once the tensor has served as the weights of dense()
        self.dtype = dtype
        self.shape = tuple(int(d) for d in shape)
        for d in self.shape:
            if d < 0:
                raise _invalid("Tensor shape cannot contain negative dimensions")
        self._keep = keep
        if ptr is None:
            p = C.c_void_p()
            check(lib.ct_alloc(C.byref(p), self.nbytes))
            self.ptr = p.value
            self._owns = True
        else:
            self.ptr = ptr
            self._owns = False

    def __dlpack__(self, stream=None, **_unused):
        """DLPack export of the device buffer itself (no copy); see camel_b200.dlpack."""
        from . import dlpack
        return dlpack.to_dlpack(self)

    def __dlpack_device__(self):
        from . import dlpack
        return (dlpack.kDLCUDA, dlpack.current_device())

    def invalidate(self) -> None:
        """Drops what was derived from the contents (packed weights).  Tensors are immutable
        values, as in the reference; code that overwrites a buffer through the raw C ABI calls this."""
        packed, self._packed = getattr(self, "_packed", None), None
        for handle in (packed or {}).values():
            try:
                lib.ct_weights_free(handle)
            except Exception:
                pass

    def __del__(self):
        self.invalidate()
        if getattr(self, "_owns", False) and self.ptr:
            try:
                lib.ct_free(self.ptr)
            except Exception:
                pass
            self.ptr = None

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    @property
    def rank(self) -> int:
        return len(self.shape)

    @property
    def nbytes(self) -> int:
        return self.numel * _SIZE[self.dtype]

    def numpy(self) -> np.ndarray:
        out = np.empty(self.shape, dtype=_NP[self.dtype])
        check(lib.ct_d2h(out.ctypes.data, self.ptr, self.nbytes))
        return out

    def __repr__(self):
        return f"Tensor(dtype={['f32', 'i64', 'bool'][self.dtype]}, shape={self.shape})"


def from_numpy(a: np.ndarray) -> Tensor:
    arr, dt = _normalize_np(np.asarray(a))
    t = Tensor(dt, arr.shape)
    check(lib.ct_h2d(t.ptr, arr.ctypes.data, t.nbytes))
    return t


def wrap_device(ptr: int, dtype: int, shape: Sequence[int], keep=None) -> Tensor:
    """View over device memory owned by someone else (e.g. a torch tensor's data_ptr())."""
    return Tensor(dtype, shape, ptr=ptr, keep=keep)


# ---- helpers ------------------------------------------------------------------------------


def _scalar_dtype(v: Number) -> int:
    """Tensor dtype a Camel scalar type normalises to (tensorDTypeFromValueType)."""
    if isinstance(v, (bool, np.bool_)):
        return L.BOOL
    if isinstance(v, (int, np.integer)):
        return L.I64
    if isinstance(v, (float, np.floating)):
        return L.F32
    raise _invalid("Unsupported scalar type for Tensor operation")


def _is_tensor(x) -> bool:
    return isinstance(x, Tensor)


def _binary(op: int, lhs, rhs) -> Tensor:
    lt, rt = _is_tensor(lhs), _is_tensor(rhs)
    if lt and rt:
        if lhs.shape != rhs.shape:
            raise _invalid("Tensor binary operation requires matching shapes")
        out = Tensor(lib.ct_result_dtype(op, lhs.dtype, rhs.dtype), lhs.shape)
        check(lib.ct_binary(op, lhs.dtype, lhs.ptr, rhs.dtype, rhs.ptr, lhs.numel, out.ptr))
        return out
    if lt:
        sdt = _scalar_dtype(rhs)
        out = Tensor(lib.ct_result_dtype(op, lhs.dtype, sdt), lhs.shape)
        check(lib.ct_binary_scalar(op, lhs.dtype, lhs.ptr, float(rhs), sdt, 0, lhs.numel, out.ptr))
        return out
    if rt:
        sdt = _scalar_dtype(lhs)
        out = Tensor(lib.ct_result_dtype(op, sdt, rhs.dtype), rhs.shape)
        check(lib.ct_binary_scalar(op, rhs.dtype, rhs.ptr, float(lhs), sdt, 1, rhs.numel, out.ptr))
        return out
    raise _invalid("Expected Tensor argument")


def _compare(op: int, lhs, rhs) -> Tensor:
    lt, rt = _is_tensor(lhs), _is_tensor(rhs)
    if lt and rt:
        if lhs.shape != rhs.shape:
            raise _invalid("Tensor comparison requires matching shapes")
        out = Tensor(L.BOOL, lhs.shape)
        check(lib.ct_compare(op, lhs.dtype, lhs.ptr, rhs.dtype, rhs.ptr, lhs.numel, out.ptr))
        return out
    if lt:
        _scalar_dtype(rhs)
        out = Tensor(L.BOOL, lhs.shape)
        check(lib.ct_compare_scalar(op, lhs.dtype, lhs.ptr, float(rhs), 0, lhs.numel, out.ptr))
        return out
    if rt:
        _scalar_dtype(lhs)
        out = Tensor(L.BOOL, rhs.shape)
        check(lib.ct_compare_scalar(op, rhs.dtype, rhs.ptr, float(lhs), 1, rhs.numel, out.ptr))
        return out
    raise _invalid("Expected Tensor argument")


# ---- tensor:add .. tensor:pow (operators.cpp:585-738) ---------------------------------------


def add(lhs, rhs) -> Tensor:
    return _binary(L.ADD, lhs, rhs)


def subtract(lhs, rhs) -> Tensor:
    return _binary(L.SUB, lhs, rhs)


def multiply(lhs, rhs) -> Tensor:
    return _binary(L.MUL, lhs, rhs)


def divide(lhs, rhs) -> Tensor:
    return _binary(L.DIV, lhs, rhs)


def pow(base, exponent) -> Tensor:  # noqa: A001 - the reference's operator name
    if not _is_tensor(base):
        raise _invalid("Expected Tensor argument")
    return _binary(L.POW, base, exponent)


# ---- tensor:lt .. tensor:eq (operators.cpp:791-956) -----------------------------------------


def lt(lhs, rhs) -> Tensor:
    return _compare(L.LT, lhs, rhs)


def le(lhs, rhs) -> Tensor:
    return _compare(L.LE, lhs, rhs)


def gt(lhs, rhs) -> Tensor:
    return _compare(L.GT, lhs, rhs)


def ge(lhs, rhs) -> Tensor:
    return _compare(L.GE, lhs, rhs)


def eq(lhs, rhs) -> Tensor:
    return _compare(L.EQ, lhs, rhs)


# ---- tensor:matmul (operators.cpp:740-769) --------------------------------------------------


def matmul(lhs: Tensor, rhs: Tensor) -> Tensor:
    if not (_is_tensor(lhs) and _is_tensor(rhs)):
        raise _invalid("Expected Tensor argument")
    if lhs.rank != 2 or rhs.rank != 2:
        raise _invalid("matmul currently only supports rank-2 tensors")
    if lhs.shape[1] != rhs.shape[0]:
        raise _invalid("matmul dimension mismatch")
    m, k = lhs.shape
    n = rhs.shape[1]
    out = Tensor(lib.ct_result_dtype(L.ADD, lhs.dtype, rhs.dtype), (m, n))
    check(lib.ct_matmul(lhs.dtype, lhs.ptr, rhs.dtype, rhs.ptr, m, k, n, out.ptr))
    return out


def matmul_tn(lhs: Tensor, rhs: Tensor) -> Tensor:
    """transpose(lhs) @ rhs without the transposed copy (the gradient of test/run/nn/mnist.cml:39);
    float tensors, same bytes as matmul(transpose(lhs), rhs)."""
    if not (_is_tensor(lhs) and _is_tensor(rhs)):
        raise _invalid("Expected Tensor argument")
    if lhs.rank != 2 or rhs.rank != 2:
        raise _invalid("matmul currently only supports rank-2 tensors")
    if lhs.shape[0] != rhs.shape[0]:
        raise _invalid("matmul dimension mismatch")
    _require_float(lhs, "matmul_tn")
    _require_float(rhs, "matmul_tn")
    k, m = lhs.shape
    n = rhs.shape[1]
    out = Tensor(L.F32, (m, n))
    check(lib.ct_matmul_tn(lhs.ptr, rhs.ptr, m, k, n, out.ptr))
    return out


def scaled_sub(w: Tensor, g: Tensor, lr: float) -> Tensor:
    """w - lr * g in one pass (the update of test/run/nn/mnist.cml:40), same bytes as
    subtract(w, multiply(g, lr))."""
    if not (_is_tensor(w) and _is_tensor(g)):
        raise _invalid("Expected Tensor argument")
    if w.shape != g.shape:
        raise _invalid("Tensor binary operation requires matching shapes")
    _require_float(w, "scaled_sub")
    _require_float(g, "scaled_sub")
    out = Tensor(L.F32, w.shape)
    check(lib.ct_scaled_sub(w.ptr, g.ptr, float(lr), w.numel, out.ptr))
    return out


# ---- constructors (operators.cpp:958-1053; runtime.cpp:614-690) -----------------------------


def _shape_arg(shape) -> tuple[int, ...]:
    shp = tuple(int(d) for d in shape)
    for d in shp:
        if d < 0:
            raise _invalid("Shape cannot contain negative values")
    return shp


def zeros(shape) -> Tensor:
    t = Tensor(L.F32, _shape_arg(shape))
    check(lib.ct_fill(L.F32, 0.0, t.numel, t.ptr))
    return t


empty = zeros  # tensorEmpty also zero-initialises (runtime.cpp:614-617)


def ones(shape) -> Tensor:
    return full(shape, 1.0)  # always Float32 (operators.cpp:991-1001)


def full(shape, value: Number) -> Tensor:
    # the tensor's dtype follows the value's type (operators.cpp:1003-1014): int -> Int64, ...
    dt = _scalar_dtype(value)
    t = Tensor(dt, _shape_arg(shape))
    check(lib.ct_fill(dt, float(value), t.numel, t.ptr))
    return t


def range(start: int, stop: int | None = None, step: int = 1) -> Tensor:  # noqa: A001
    if stop is None:
        start, stop = 0, start
    if step == 0:
        raise _invalid("range step cannot be zero")
    if step > 0:
        count = _builtins.max(0, -((start - stop) // step))
    else:
        count = _builtins.max(0, -((stop - start) // (-step)))
    t = Tensor(L.I64, (count,))
    check(lib.ct_arange(start, step, count, t.ptr))
    return t


def eye(n: int) -> Tensor:
    if n < 0:
        raise _invalid("eye size cannot be negative")
    t = Tensor(L.F32, (n, n))
    check(lib.ct_eye(n, t.ptr))
    return t


def shape(t: Tensor) -> list[int]:
    return list(t.shape)


# ---- reductions (operators.cpp:1055-1120) ---------------------------------------------------


def sum(t: Tensor, axis: int | None = None):  # noqa: A001
    if axis is None:
        r = C.c_double()
        check(lib.ct_sum(t.dtype, t.ptr, t.numel, C.byref(r)))
        return r.value
    return _axis(lib.ct_sum_axis, "sum", t, axis, L.F32)


def max(t: Tensor, axis: int) -> Tensor:  # noqa: A001
    return _axis(lib.ct_max_axis, "max", t, axis, L.F32)


def argmax(t: Tensor, axis: int) -> Tensor:
    return _axis(lib.ct_argmax_axis, "argmax", t, axis, L.I64)


def _axis(fn, name: str, t: Tensor, axis: int, odt: int) -> Tensor:
    if t.rank != 2:
        raise _invalid(f"{name}(axis) currently only supports rank-2 tensors")
    a = axis + 2 if axis < 0 else axis
    if a not in (0, 1):
        raise _invalid(f"{name}(axis): axis must be 0 or 1 for rank-2 tensors")
    rows, cols = t.shape
    out = Tensor(odt, (cols,) if a == 0 else (rows,))
    check(fn(t.dtype, t.ptr, rows, cols, a, out.ptr))
    return out


# ---- exp / log / transpose / concat / reshape / idx -----------------------------------------


def _require_float(t: Tensor, name: str) -> None:
    if t.dtype != L.F32:
        raise _invalid(f"{name} requires floating-point tensor")


def exp(t: Tensor) -> Tensor:
    _require_float(t, "exp")
    out = Tensor(L.F32, t.shape)
    check(lib.ct_exp(t.ptr, t.numel, out.ptr))
    return out


def log(t: Tensor) -> Tensor:
    _require_float(t, "log")
    out = Tensor(L.F32, t.shape)
    check(lib.ct_log(t.ptr, t.numel, out.ptr))
    return out


def transpose(t: Tensor) -> Tensor:
    if t.rank != 2:
        raise _invalid("transpose currently only supports rank-2 tensors")
    out = Tensor(t.dtype, (t.shape[1], t.shape[0]))
    check(lib.ct_transpose(t.dtype, t.ptr, t.shape[0], t.shape[1], out.ptr))
    return out


def concat(a: Tensor, b: Tensor, axis: int) -> Tensor:
    if a.rank != b.rank:
        raise _invalid("concat requires tensors with the same rank")
    if axis < 0 or axis >= a.rank:
        raise _invalid("concat axis out of range")
    if a.dtype != b.dtype:
        raise _invalid("concat currently requires matching dtypes")
    for i in builtins_range(a.rank):
        if i != axis and a.shape[i] != b.shape[i]:
            raise _invalid("concat requires equal non-axis dimensions")
    shp = list(a.shape)
    shp[axis] += b.shape[axis]
    outer = int(np.prod(a.shape[:axis], dtype=np.int64)) if axis > 0 else 1
    inner = int(np.prod(a.shape[axis + 1:], dtype=np.int64)) if axis + 1 < a.rank else 1
    out = Tensor(a.dtype, shp)
    check(lib.ct_concat(a.dtype, a.ptr, b.ptr, outer, a.shape[axis], b.shape[axis], inner, out.ptr))
    return out


def reshape(t: Tensor, new_shape) -> Tensor:
    shp = _shape_arg(new_shape)
    n = 1
    for d in shp:
        n *= d
    if n != t.numel:
        raise _invalid("reshape changes tensor element count")
    # The reference copies (runtime.cpp:692-702).  Tensors are immutable values, so a second shape
    # over the same device buffer is the same value without the pass over HBM; `keep` holds the
    # owner alive.
    return Tensor(t.dtype, shp, ptr=t.ptr, keep=t)


def idx(t: Tensor, i: int) -> float:
    if t.rank != 1:
        raise _invalid("Single-index tensor access requires rank-1 tensor")
    if i < 0 or i >= t.shape[0]:
        raise _invalid("Tensor index out of bounds")
    return _fetch(t, i)


def idx2d(t: Tensor, i: int, j: int) -> float:
    if t.rank != 2:
        raise _invalid("Two-index tensor access requires rank-2 tensor")
    if i < 0 or i >= t.shape[0] or j < 0 or j >= t.shape[1]:
        raise _invalid("Tensor index out of bounds")
    return _fetch(t, i * t.shape[1] + j)


def _fetch(t: Tensor, flat: int) -> float:
    buf = np.empty(1, dtype=_NP[t.dtype])
    check(lib.ct_d2h(buf.ctypes.data, t.ptr + flat * _SIZE[t.dtype], _SIZE[t.dtype]))
    return float(buf[0] != 0) if t.dtype == L.BOOL else float(buf[0])


# ---- operators the reference composes from the above; fused here ----------------------------


def relu(t: Tensor) -> Tensor:
    """multiply(t, gt(t, 0)) in one kernel (idiom: test/run/nn/svm.cml:31)."""
    _require_float(t, "relu")
    out = Tensor(L.F32, t.shape)
    check(lib.ct_relu(t.ptr, t.numel, out.ptr))
    return out


def softmax(t: Tensor) -> Tensor:
    """The `softmax` function of test/run/nn/mnist.cml:13-25 as one operator."""
    _require_float(t, "softmax")
    if t.rank != 2:
        raise _invalid("softmax currently only supports rank-2 tensors")
    out = Tensor(L.F32, t.shape)
    check(lib.ct_softmax_rows(t.ptr, t.shape[0], t.shape[1], out.ptr))
    return out


_ACT = {None: L.ACT_NONE, "none": L.ACT_NONE, "relu": L.ACT_RELU, "softmax": L.ACT_SOFTMAX}


def dense(x: Tensor, w: Tensor, b: Tensor | None = None, activation: str | None = None,
          with_argmax: bool = False):
    """dense<w,b>(x): concat(x, ones, 1) @ concat(w, b, 0) (test/run/nn/lr.cml:19-21), fused."""
    if x.rank != 2 or w.rank != 2:
        raise _invalid("matmul currently only supports rank-2 tensors")
    if x.shape[1] != w.shape[0]:
        raise _invalid("matmul dimension mismatch")
    _require_float(x, "dense")
    _require_float(w, "dense")
    m, k = x.shape
    n = w.shape[1]
    if b is not None and (b.numel != n or b.dtype != L.F32):
        raise _invalid("dense: bias must be a float tensor with one value per output column")
    if activation not in _ACT:
        raise _invalid("dense: unknown activation")
    out = Tensor(L.F32, (m, n))
    am = Tensor(L.I64, (m,)) if with_argmax else None
    check(lib.ct_dense_packed(x.ptr, w.ptr, _packed_weights(w, m, k, n), b.ptr if b is not None else None,
                              m, k, n, _ACT[activation], out.ptr, am.ptr if am is not None else None))
    return (out, am) if with_argmax else out


_weight_cache = True
_recording = 0


def set_weight_cache(on: bool) -> None:
    """dense() keeps the tensor-core layout of a weight tensor with the tensor (built at its first
    use with at least 128 rows of input) unless this is switched off."""
    global _weight_cache
    _weight_cache = bool(on)


def _packed_weights(w: Tensor, m: int, k: int, n: int):
    """Handle of w's packed form under the current precision, or None where the call does not use
    one: narrow outputs read w itself, small problems take other kernels, and nothing is packed
    while calls are being recorded (the handle would belong to the recording)."""
    if not _weight_cache or n <= 32 or m < 128 or k == 0:
        return None
    prec = int(lib.ct_get_precision())
    if w._packed is not None and prec in w._packed:
        return w._packed[prec]
    if _recording:
        return None
    handle = C.c_void_p()
    check(lib.ct_weights_pack(w.ptr, k, n, C.byref(handle)))
    if w._packed is None:
        w._packed = {}
    w._packed[prec] = handle
    return handle


def conv2d(x: Tensor, w: Tensor, b: Tensor | None = None, stride: int = 1, pad: int = 0,
           activation: str | None = None, pool: int = 0) -> Tensor:
    """conv2d, + bias, activation; with pool=2 also the 2x2 max-pool of the result (the values of
    maxpool2d(conv2d(...), 2), without writing the full-resolution activation where the layer has
    at most 64 filters)."""
    if pool not in (0, 2):
        raise _invalid("conv2d: pool must be 0 or 2")
    if x.rank != 4 or w.rank != 4:
        raise _invalid("conv2d requires rank-4 input [n,c,h,w] and weights [k,c,kh,kw]")
    if x.shape[1] != w.shape[1]:
        raise _invalid("conv2d channel mismatch")
    _require_float(x, "conv2d")
    _require_float(w, "conv2d")
    n, c, h, wd = x.shape
    ko, _, kh, kw = w.shape
    if b is not None and (b.numel != ko or b.dtype != L.F32):
        raise _invalid("conv2d: bias must be a float tensor with one value per output channel")
    if activation not in (None, "none", "relu"):
        raise _invalid("conv2d: activation must be none or relu")
    if h + 2 * pad < kh or wd + 2 * pad < kw or stride <= 0:
        raise _invalid("conv2d: kernel larger than padded input")
    ho, wo = (h + 2 * pad - kh) // stride + 1, (wd + 2 * pad - kw) // stride + 1
    if pool == 2:
        out = Tensor(L.F32, (n, ko, ho // 2, wo // 2))
        check(lib.ct_conv2d_maxpool2(x.ptr, w.ptr, b.ptr if b is not None else None, n, c, h, wd, ko, kh, kw,
                                     stride, pad, _ACT[activation], out.ptr))
        return out
    out = Tensor(L.F32, (n, ko, ho, wo))
    check(lib.ct_conv2d(x.ptr, w.ptr, b.ptr if b is not None else None, n, c, h, wd, ko, kh, kw,
                        stride, pad, _ACT[activation], out.ptr))
    return out


def maxpool2d(x: Tensor, window: int = 2) -> Tensor:
    if x.rank != 4:
        raise _invalid("maxpool2d requires a rank-4 input [n,c,h,w]")
    _require_float(x, "maxpool2d")
    n, c, h, w = x.shape
    out = Tensor(L.F32, (n, c, h // window, w // window))
    check(lib.ct_maxpool2d(x.ptr, n, c, h, w, window, out.ptr))
    return out


def flatten(x: Tensor) -> Tensor:
    """reshape(x, [n, rest])."""
    if x.rank < 1:
        raise _invalid("flatten requires rank >= 1")
    rest = x.numel // x.shape[0] if x.shape[0] else 0
    return reshape(x, (x.shape[0], rest))


class Graph:
    """Records the operator calls made inside `with Graph() as g:` and replays them with
    `g.launch()` (one CUDA-graph launch).  Tensors created inside the block and still referenced
    afterwards (e.g. kept in `g.keep`) hold the results of the latest replay.  Run the same calls
    once before recording, and do not let tensors created earlier die inside the block."""

    def __init__(self):
        self.handle = C.c_void_p()
        self.keep = None

    def __enter__(self):
        global _recording
        check(lib.ct_graph_begin())
        _recording += 1
        return self

    def __exit__(self, exc_type, exc, tb):
        global _recording
        _recording -= 1
        status = lib.ct_graph_end(C.byref(self.handle))
        if exc_type is None:
            check(status)
        return False

    def launch(self) -> None:
        check(lib.ct_graph_launch(self.handle))

    def __del__(self):
        if getattr(self, "handle", None) is not None and self.handle.value:
            try:
                lib.ct_graph_destroy(self.handle)
            except Exception:
                pass
            self.handle = C.c_void_p()


def sync() -> None:
    check(lib.ct_sync())


def check_async() -> None:
    """Raises if a kernel of an earlier asynchronous call reported an error."""
    check(lib.ct_check())


import builtins as _builtins  # noqa: E402

builtins_range = _builtins.range
