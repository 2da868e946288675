"""Zero-copy exchange of device tensors through DLPack.

The reference's Python bridge copies tensors through host memory (`tensorToDLPackCopy` /
`tensorFromDLPackCopy`, modules/tensor/runtime.cpp:1079-1124; its `dlpack.h:7-9` defines only the
CPU device).  With device-resident storage the natural form is the CUDA device type: the consumer
(torch, cupy, jax) gets the tensor's own device pointer, no copy.

    t  = camel_b200.tensor.from_numpy(a)
    tt = torch.from_dlpack(t)                 # Tensor has __dlpack__ / __dlpack_device__
    u  = camel_b200.dlpack.from_dlpack(tt)    # and back: a Tensor that keeps `tt` alive

Only what the tensor module stores is exchanged: dense row-major float32 / int64 / bool(uint8).
"""
from __future__ import annotations

import ctypes as C

from . import _lib as L
from . import tensor as T

kDLCPU, kDLCUDA, kDLCUDAHost = 1, 2, 3
kDLInt, kDLUInt, kDLFloat, kDLBool = 0, 1, 2, 6


class DLDevice(C.Structure):
    _fields_ = [("device_type", C.c_int32), ("device_id", C.c_int32)]


class DLDataType(C.Structure):
    _fields_ = [("code", C.c_uint8), ("bits", C.c_uint8), ("lanes", C.c_uint16)]


class DLTensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("device", DLDevice), ("ndim", C.c_int32), ("dtype", DLDataType),
                ("shape", C.POINTER(C.c_int64)), ("strides", C.POINTER(C.c_int64)), ("byte_offset", C.c_uint64)]


class DLManagedTensor(C.Structure):
    pass


_DELETER = C.CFUNCTYPE(None, C.POINTER(DLManagedTensor))
DLManagedTensor._fields_ = [("dl_tensor", DLTensor), ("manager_ctx", C.c_void_p), ("deleter", _DELETER)]

_PyCapsule_New = C.pythonapi.PyCapsule_New
_PyCapsule_New.restype = C.py_object
_PyCapsule_New.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p]
_PyCapsule_GetPointer = C.pythonapi.PyCapsule_GetPointer
_PyCapsule_GetPointer.restype = C.c_void_p
_PyCapsule_GetPointer.argtypes = [C.py_object, C.c_char_p]
_PyCapsule_SetName = C.pythonapi.PyCapsule_SetName
_PyCapsule_SetName.restype = C.c_int
_PyCapsule_SetName.argtypes = [C.py_object, C.c_char_p]
_PyCapsule_IsValid = C.pythonapi.PyCapsule_IsValid
_PyCapsule_IsValid.restype = C.c_int
_PyCapsule_IsValid.argtypes = [C.py_object, C.c_char_p]

_TO_DL = {L.F32: (kDLFloat, 32), L.I64: (kDLInt, 64), L.BOOL: (kDLBool, 8)}
_FROM_DL = {(kDLFloat, 32): L.F32, (kDLInt, 64): L.I64, (kDLBool, 8): L.BOOL, (kDLUInt, 8): L.BOOL}

# exported tensors stay alive here until the consumer calls the deleter
_exported: dict[int, tuple] = {}


@_DELETER
def _release(managed_ptr):
    _exported.pop(C.addressof(managed_ptr.contents), None)


def current_device() -> int:
    """Index of the device the library is bound to (the device of every Tensor of this process)."""
    dev = C.c_int(-1)
    L.check(L.lib.ct_get_device(C.byref(dev)))
    return int(dev.value)


def to_dlpack(t: "T.Tensor"):
    """A "dltensor" capsule over the tensor's device buffer.  The tensor is kept alive until the
    consumer releases the capsule; work enqueued on the library's stream is finished first, so the
    consumer may read on any stream."""
    T.sync()
    code, bits = _TO_DL[t.dtype]
    shape = (C.c_int64 * max(t.rank, 1))(*t.shape)
    managed = DLManagedTensor()
    managed.dl_tensor.data = t.ptr
    managed.dl_tensor.device = DLDevice(kDLCUDA, current_device())
    managed.dl_tensor.ndim = t.rank
    managed.dl_tensor.dtype = DLDataType(code, bits, 1)
    managed.dl_tensor.shape = C.cast(shape, C.POINTER(C.c_int64))
    managed.dl_tensor.strides = None  # dense row-major
    managed.dl_tensor.byte_offset = 0
    managed.manager_ctx = None
    managed.deleter = _release
    _exported[C.addressof(managed)] = (managed, shape, t)
    return _PyCapsule_New(C.addressof(managed), b"dltensor", None)


def from_dlpack(obj) -> "T.Tensor":
    """A Tensor over the device buffer of `obj` (anything with __dlpack__, or a capsule).  No copy:
    the producer's memory is used as is and released when the Tensor goes away.  The producer must
    be on this process's device, dense row-major, float32 / int64 / bool / uint8."""
    capsule = obj.__dlpack__() if hasattr(obj, "__dlpack__") else obj
    if not _PyCapsule_IsValid(capsule, b"dltensor"):
        raise ValueError("from_dlpack: not an unconsumed dltensor capsule")
    managed = C.cast(_PyCapsule_GetPointer(capsule, b"dltensor"), C.POINTER(DLManagedTensor))
    dl = managed.contents.dl_tensor
    if dl.device.device_type != kDLCUDA or dl.device.device_id != current_device():
        raise ValueError("from_dlpack: the tensor is not on this process's CUDA device")
    key = (int(dl.dtype.code), int(dl.dtype.bits))
    if key not in _FROM_DL or dl.dtype.lanes != 1:
        raise ValueError("from_dlpack: only float32, int64, bool and uint8 tensors are supported")
    shape = tuple(int(dl.shape[i]) for i in range(dl.ndim))
    if dl.strides:
        expect = 1
        for i in range(dl.ndim - 1, -1, -1):
            if shape[i] != 1 and int(dl.strides[i]) != expect:
                raise ValueError("from_dlpack: only dense row-major tensors are supported")
            expect *= shape[i]
    _PyCapsule_SetName(capsule, b"used_dltensor")  # the capsule is consumed: its deleter is ours to call
    return T.Tensor(_FROM_DL[key], shape, ptr=int(dl.data or 0) + int(dl.byte_offset), keep=_Owner(managed))


class _Owner:
    """Calls the producer's deleter when the importing Tensor is collected."""

    def __init__(self, managed):
        self.managed = managed

    def __del__(self):
        m, self.managed = self.managed, None
        if m is not None and m.contents.deleter:
            m.contents.deleter(m)
