"""TEST INFRASTRUCTURE, not product code.

numpy front ends of the two CPU checkers:

* ``port``  - this repo's C restatement (oracle/camel_tensor_oracle.c -> libcamel_tensor_oracle.so)
* ``ref``   - the reference's own compiled tensor module (oracle/_ref/libcamel_tensor_ref.so,
              built by oracle/Makefile from the reference checkout), driven through its real
              ``operator_t`` entry points.

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import this
package.  Nothing under ``camel_b200/`` does.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
PORT_LIB = HERE / "libcamel_tensor_oracle.so"
REF_LIB = HERE / "_ref" / "libcamel_tensor_ref.so"

F32, I64, BOOL = 0, 1, 2
ADD, SUB, MUL, DIV, POW = range(5)
LT, LE, GT, GE, EQ = range(5)
_NP = {F32: np.float32, I64: np.int64, BOOL: np.uint8}
ERRORS = {1: "Division by zero", 2: "log: input must be positive", 3: "unsupported dtype"}


class OracleError(RuntimeError):
    pass


def reference_checkout() -> str | None:
    """Where the reference's sources are: $CAMEL_REF, else the sibling folder `reference` next to
    the repository; None if neither holds the tensor module."""
    import os

    for cand in (os.environ.get("CAMEL_REF"), str(HERE.parent.parent / "reference")):
        if cand and (Path(cand) / "modules" / "tensor" / "runtime.cpp").exists():
            return cand
    return None


def build(ref: bool = True) -> None:
    """Compiles the checkers (make); the reference one only where its sources are present."""
    subprocess.run(["make", "-s", "-C", str(HERE), "oracle"], check=True)
    src = reference_checkout() if ref else None
    if src:
        subprocess.run(["make", "-s", "-j8", "-C", str(HERE), "all", f"REF={src}"], check=True)


def norm(a) -> tuple[np.ndarray, int]:
    a = np.asarray(a)
    if a.dtype in (np.float32, np.float64):
        return np.ascontiguousarray(a, dtype=np.float32), F32
    if a.dtype in (np.int32, np.int64):
        return np.ascontiguousarray(a, dtype=np.int64), I64
    if a.dtype in (np.bool_, np.uint8):
        return np.ascontiguousarray(a != 0, dtype=np.uint8), BOOL
    raise OracleError(f"unsupported dtype {a.dtype}")


def scalar_dtype(v) -> int:
    if isinstance(v, (bool, np.bool_)):
        return BOOL
    if isinstance(v, (int, np.integer)):
        return I64
    return F32


# ---- the C restatement ------------------------------------------------------------------


class Port:
    def __init__(self):
        if not PORT_LIB.exists():
            build(ref=False)
        self.lib = C.CDLL(str(PORT_LIB))
        self.lib.cto_sum.restype = C.c_double
        self.lib.cto_arange.restype = C.c_int64

    @staticmethod
    def _p(a: np.ndarray):
        return C.c_void_p(a.ctypes.data)

    def _rc(self, rc: int):
        if rc:
            raise OracleError(ERRORS.get(rc, f"oracle error {rc}"))

    def result_dtype(self, op, l, r):
        return self.lib.cto_result_dtype(op, l, r)

    def binary(self, op, lhs, rhs):
        lt, rt = isinstance(lhs, np.ndarray), isinstance(rhs, np.ndarray)
        if lt and rt:
            a, adt = norm(lhs)
            b, bdt = norm(rhs)
            out = np.empty(a.shape, _NP[self.result_dtype(op, adt, bdt)])
            self._rc(self.lib.cto_binary(op, adt, self._p(a), bdt, self._p(b), C.c_uint64(a.size), self._p(out)))
            return out
        t, tdt = norm(lhs if lt else rhs)
        s = rhs if lt else lhs
        sdt = scalar_dtype(s)
        odt = self.result_dtype(op, tdt, sdt) if lt else self.result_dtype(op, sdt, tdt)
        out = np.empty(t.shape, _NP[odt])
        self._rc(self.lib.cto_binary_scalar(op, tdt, self._p(t), C.c_double(float(s)), sdt, 0 if lt else 1,
                                            C.c_uint64(t.size), self._p(out)))
        return out

    def compare(self, op, lhs, rhs):
        lt, rt = isinstance(lhs, np.ndarray), isinstance(rhs, np.ndarray)
        if lt and rt:
            a, adt = norm(lhs)
            b, bdt = norm(rhs)
            out = np.empty(a.shape, np.uint8)
            self.lib.cto_compare(op, adt, self._p(a), bdt, self._p(b), C.c_uint64(a.size), self._p(out))
            return out
        t, tdt = norm(lhs if lt else rhs)
        s = rhs if lt else lhs
        out = np.empty(t.shape, np.uint8)
        self.lib.cto_compare_scalar(op, tdt, self._p(t), C.c_double(float(s)), 0 if lt else 1,
                                    C.c_uint64(t.size), self._p(out))
        return out

    def sum(self, t):
        a, dt = norm(t)
        return self.lib.cto_sum(dt, self._p(a), C.c_uint64(a.size))

    def _axis(self, fn, t, axis, odt):
        a, dt = norm(t)
        rows, cols = a.shape
        ax = axis + 2 if axis < 0 else axis
        out = np.empty((cols,) if ax == 0 else (rows,), odt)
        fn(dt, self._p(a), C.c_int64(rows), C.c_int64(cols), ax, self._p(out))
        return out

    def sum_axis(self, t, axis):
        return self._axis(self.lib.cto_sum_axis, t, axis, np.float32)

    def max_axis(self, t, axis):
        return self._axis(self.lib.cto_max_axis, t, axis, np.float32)

    def argmax_axis(self, t, axis):
        return self._axis(self.lib.cto_argmax_axis, t, axis, np.int64)

    def exp(self, t):
        a, _ = norm(t)
        out = np.empty_like(a)
        self.lib.cto_exp(self._p(a), C.c_uint64(a.size), self._p(out))
        return out

    def log(self, t):
        a, _ = norm(t)
        out = np.empty_like(a)
        self._rc(self.lib.cto_log(self._p(a), C.c_uint64(a.size), self._p(out)))
        return out

    def relu(self, t):
        a, _ = norm(t)
        out = np.empty_like(a)
        self.lib.cto_relu(self._p(a), C.c_uint64(a.size), self._p(out))
        return out

    def transpose(self, t):
        a, dt = norm(t)
        out = np.empty((a.shape[1], a.shape[0]), a.dtype)
        self.lib.cto_transpose(dt, self._p(a), C.c_int64(a.shape[0]), C.c_int64(a.shape[1]), self._p(out))
        return out

    def concat(self, x, y, axis):
        a, dt = norm(x)
        b, _ = norm(y)
        shp = list(a.shape)
        shp[axis] += b.shape[axis]
        outer = int(np.prod(a.shape[:axis], dtype=np.int64))
        inner = int(np.prod(a.shape[axis + 1:], dtype=np.int64))
        out = np.empty(shp, a.dtype)
        self.lib.cto_concat(dt, self._p(a), self._p(b), C.c_uint64(outer), C.c_uint64(a.shape[axis]),
                            C.c_uint64(b.shape[axis]), C.c_uint64(inner), self._p(out))
        return out

    def matmul(self, x, y):
        a, adt = norm(x)
        b, bdt = norm(y)
        m, k = a.shape
        n = b.shape[1]
        out = np.empty((m, n), _NP[self.result_dtype(ADD, adt, bdt)])
        self.lib.cto_matmul(adt, self._p(a), bdt, self._p(b), C.c_int64(m), C.c_int64(k), C.c_int64(n), self._p(out))
        return out

    def softmax_rows(self, t):
        a, _ = norm(t)
        out = np.empty_like(a)
        self._rc(self.lib.cto_softmax_rows(self._p(a), C.c_int64(a.shape[0]), C.c_int64(a.shape[1]), self._p(out)))
        return out

    def dense(self, x, w, b=None, act=0):
        a, _ = norm(x)
        ww, _ = norm(w)
        bb = norm(b)[0] if b is not None else None
        m, k = a.shape
        n = ww.shape[1]
        out = np.empty((m, n), np.float32)
        self.lib.cto_dense(self._p(a), self._p(ww), self._p(bb) if bb is not None else None,
                           C.c_int64(m), C.c_int64(k), C.c_int64(n), act, self._p(out))
        return out

    def conv2d(self, x, w, b=None, stride=1, pad=0, act=0):
        a, _ = norm(x)
        ww, _ = norm(w)
        bb = norm(b)[0] if b is not None else None
        n, c, h, wd = a.shape
        ko, _, kh, kw = ww.shape
        ho, wo = (h + 2 * pad - kh) // stride + 1, (wd + 2 * pad - kw) // stride + 1
        out = np.empty((n, ko, ho, wo), np.float32)
        i64 = C.c_int64
        self.lib.cto_conv2d(self._p(a), self._p(ww), self._p(bb) if bb is not None else None, i64(n), i64(c),
                            i64(h), i64(wd), i64(ko), i64(kh), i64(kw), i64(stride), i64(pad), act, self._p(out))
        return out

    def maxpool2d(self, x, win=2):
        a, _ = norm(x)
        n, c, h, wd = a.shape
        out = np.empty((n, c, h // win, wd // win), np.float32)
        i64 = C.c_int64
        self.lib.cto_maxpool2d(self._p(a), i64(n), i64(c), i64(h), i64(wd), i64(win), self._p(out))
        return out

    def full(self, dt, value, shape):
        out = np.empty(shape, _NP[dt])
        self.lib.cto_full(dt, C.c_double(float(value)), C.c_uint64(out.size), self._p(out))
        return out

    def eye(self, n):
        out = np.empty((n, n), np.float32)
        self.lib.cto_eye(C.c_int64(n), self._p(out))
        return out

    def arange(self, start, stop, step):
        i64 = C.c_int64
        cnt = self.lib.cto_arange(i64(start), i64(stop), i64(step), None)
        out = np.empty((cnt,), np.int64)
        self.lib.cto_arange(i64(start), i64(stop), i64(step), self._p(out))
        return out


# ---- the compiled reference -------------------------------------------------------------


class _Arg(C.Structure):
    _fields_ = [("kind", C.c_int32), ("dtype", C.c_int32), ("rank", C.c_int32), ("pad", C.c_int32),
                ("shape", C.POINTER(C.c_int64)), ("data", C.c_void_p), ("f64", C.c_double), ("i64", C.c_int64)]


class _Out(C.Structure):
    _fields_ = [("kind", C.c_int32), ("dtype", C.c_int32), ("rank", C.c_int32), ("pad", C.c_int32),
                ("shape", C.c_int64 * 8), ("numel", C.c_uint64), ("data", C.c_void_p), ("f64", C.c_double),
                ("seconds", C.c_double)]


class IntArray:
    """Marks a Python list as a Camel int[] argument (e.g. a shape)."""

    def __init__(self, items):
        self.items = [int(i) for i in items]


class NestedArray:
    """Marks a (nested) list as a Camel array literal, e.g. [[1.0, 2.0], [3.0, 4.0]]; `leaf` names
    the element type of the innermost arrays: "f32", "i64", "bool", "f64" or "i32"."""

    LEAF = {"f32": 0, "i64": 1, "bool": 2, "f64": 3, "i32": 4}

    def __init__(self, items, leaf="f64"):
        self.values = np.ascontiguousarray(np.asarray(items, dtype=np.float64))
        if self.values.ndim < 1:
            raise OracleError("an array literal has at least one level")
        self.leaf = self.LEAF[leaf]


class Float32(float):
    """Marks a scalar as Camel float32 (plain Python floats are float64)."""


class With:
    """Marks an argument as a `with` parameter (`op<w, b>(x)`): the plugin's added operators
    take their weights that way; the reference's own operators have none."""

    def __init__(self, value):
        self.value = value


class Reference:
    """Calls `tensor:<op>` of the compiled reference.  Arguments: numpy arrays (tensors),
    Python int (Int64) / float (Float64) / bool scalars, Float32(...), IntArray([...])."""

    def __init__(self, lib_path=None):
        """lib_path: another library with the same driver entry points (the plugin's own test
        harness, camel_b200/host/_build/libcamel_tensor_host_test.so); default: the reference."""
        path = Path(lib_path) if lib_path else REF_LIB
        if not path.exists():
            raise OracleError(f"{path} not built (run `make -C oracle ref` where the reference checkout is)")
        self.lib = C.CDLL(str(path))
        self.last_seconds = 0.0

    @staticmethod
    def available() -> bool:
        return REF_LIB.exists()

    def ops(self) -> list[str]:
        buf = C.create_string_buffer(1 << 14)
        self.lib.camel_ref_list_ops(buf, 1 << 14)
        return sorted(buf.value.decode().split())

    def groups(self) -> list[tuple[str, str, str]]:
        buf = C.create_string_buffer(1 << 16)
        self.lib.camel_ref_list_groups(buf, 1 << 16)
        return [tuple(line.split("\t")) for line in buf.value.decode().splitlines() if line]

    def call(self, op: str, *args):
        keep, cargs = _marshal(args)
        out, err = _Out(), C.create_string_buffer(512)
        rc = self.lib.camel_ref_call(op.encode(), len(args), cargs, C.byref(out), err, 512)
        if rc:
            raise OracleError(err.value.decode())
        self.last_seconds = out.seconds
        return _unmarshal(out)

    def session(self, lazy: bool | None = None) -> "Session":
        """A chain of operator calls whose values stay inside the library (the plugin's harness
        only; the reference is driven call by call, which is the same thing for host tensors)."""
        return Session(self.lib, lazy)


class Handle:
    """A value an earlier call of a Session returned."""

    def __init__(self, index: int):
        self.index = index


def _marshal(args):
    keep, cargs = [], (_Arg * max(1, len(args)))()
    for i, a in enumerate(args):
        x = cargs[i]
        in_with = isinstance(a, With)
        if in_with:
            a = a.value
        if isinstance(a, Handle):
            x.kind, x.i64 = 7, a.index
        elif isinstance(a, np.ndarray):
            arr, dt = norm(a)
            shp = (C.c_int64 * max(1, arr.ndim))(*arr.shape)
            keep += [arr, shp]
            x.kind, x.dtype, x.rank, x.shape, x.data = 0, dt, arr.ndim, shp, arr.ctypes.data
        elif isinstance(a, NestedArray):
            shp = (C.c_int64 * a.values.ndim)(*a.values.shape)
            keep += [a.values, shp]
            x.kind, x.dtype, x.rank, x.shape, x.data = 8, a.leaf, a.values.ndim, shp, a.values.ctypes.data
        elif isinstance(a, IntArray):
            shp = (C.c_int64 * max(1, len(a.items)))(*a.items)
            keep.append(shp)
            x.kind, x.rank, x.shape = 6, len(a.items), shp
        elif isinstance(a, (bool, np.bool_)):
            x.kind, x.i64 = 5, int(a)
        elif isinstance(a, (int, np.integer)):
            x.kind, x.i64 = 1, int(a)
        elif isinstance(a, Float32):
            x.kind, x.f64 = 3, float(a)
        elif isinstance(a, (float, np.floating)):
            x.kind, x.f64 = 2, float(a)
        else:
            raise OracleError(f"unsupported argument {type(a)}")
        if in_with:
            x.kind |= 0x100
    return keep, cargs


def _unmarshal(out: "_Out"):
    if out.kind == 1:
        return out.f64
    if out.kind == 2:
        return [out.shape[i] for i in range(out.rank)]
    if out.kind == 3:
        return None
    shp = tuple(out.shape[i] for i in range(out.rank))
    n = int(out.numel)
    dt = _NP[out.dtype]
    if n == 0:
        return np.zeros(shp, dt)
    buf = (C.c_char * (n * np.dtype(dt).itemsize)).from_address(out.data)
    return np.frombuffer(buf, dtype=dt).reshape(shp).copy()


class Session:
    """Drives camel_host_session_* of the plugin's harness: `put` uploads a tensor, `call` runs an
    operator on handles and plain arguments and returns the handle of its value, `fetch` reads a
    value back, `finish` has a value computed and waits, returning the library's launch count.
    Starting a session releases everything earlier calls created."""

    def __init__(self, lib, lazy: bool | None = None):
        self.lib = lib
        lib.camel_host_session_finish.restype = C.c_int64
        lib.camel_host_session_finish.argtypes = [C.c_int64, C.c_char_p, C.c_int]
        lib.camel_host_session_fetch.argtypes = [C.c_int64, C.POINTER(_Out), C.c_char_p, C.c_int]
        lib.camel_host_session_pending.argtypes = [C.c_int64]
        lib.camel_host_session_begin(-1 if lazy is None else int(lazy))

    def put(self, value) -> Handle:
        keep, cargs = _marshal((value,))
        h, err = C.c_int64(-1), C.create_string_buffer(512)
        if self.lib.camel_host_session_put(cargs, C.byref(h), err, 512):
            raise OracleError(err.value.decode())
        return Handle(h.value)

    def call(self, op: str, *args) -> Handle:
        keep, cargs = _marshal(args)
        h, err = C.c_int64(-1), C.create_string_buffer(512)
        if self.lib.camel_host_session_call(op.encode(), len(args), cargs, C.byref(h), err, 512):
            raise OracleError(err.value.decode())
        return Handle(h.value)

    def fetch(self, handle: Handle):
        out, err = _Out(), C.create_string_buffer(512)
        if self.lib.camel_host_session_fetch(handle.index, C.byref(out), err, 512):
            raise OracleError(err.value.decode())
        return _unmarshal(out)

    def finish(self, handle: Handle | None = None) -> int:
        err = C.create_string_buffer(512)
        n = self.lib.camel_host_session_finish(-1 if handle is None else handle.index, err, 512)
        if n < 0:
            raise OracleError(err.value.decode())
        return n

    def pending(self, handle: Handle) -> bool:
        return self.lib.camel_host_session_pending(handle.index) == 1


_port = None
_ref = None


def port() -> Port:
    global _port
    if _port is None:
        _port = Port()
    return _port


def ref() -> Reference:
    global _ref
    if _ref is None:
        _ref = Reference()
    return _ref
