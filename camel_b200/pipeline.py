"""Streaming a recorded forward pass over batches that live in host memory.

The reference's tensors are host memory, so a `.cml` program hands the module host buffers and
reads host buffers back (modules/tensor/runtime.cpp:256-279 builds every tensor on the host).
With device-resident storage each batch crosses PCIe twice.  `HostPipeline` hides that behind the
kernels: three streams (copy in, compute, copy out), `depth` staging slots, one recorded graph per
slot, events between the stages.  The copy of batch i+1 runs while the kernels of batch i run and
the results of batch i-1 are read back, so the steady-state time per batch is the slowest of the
three stages instead of their sum.

Host buffers must be page-locked (`pinned_array`, or any allocation registered with CUDA) and
must stay alive until `run` returns.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Sequence

import numpy as np

from . import tensor as T
from ._lib import check, lib


def _handle(create) -> C.c_void_p:
    h = C.c_void_p()
    check(create(C.byref(h)))
    return h


class PinnedBuffer:
    """Page-locked host memory viewed as a numpy array."""

    def __init__(self, shape: Sequence[int], dtype):
        self.shape = tuple(int(d) for d in shape)
        self.dtype = np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize
        self._ptr = C.c_void_p()
        check(lib.ct_host_alloc(C.byref(self._ptr), max(self.nbytes, 1)))
        raw = (C.c_uint8 * max(self.nbytes, 1)).from_address(self._ptr.value)
        self.array = np.frombuffer(raw, dtype=self.dtype, count=self.nbytes // self.dtype.itemsize).reshape(self.shape)

    @property
    def ptr(self) -> int:
        return self._ptr.value

    def __del__(self):
        p = getattr(self, "_ptr", None)
        if p is not None and p.value:
            self.array = None
            try:
                lib.ct_host_free(p)
            except Exception:
                pass
            self._ptr = C.c_void_p()


def pinned_array(shape: Sequence[int], dtype=np.float32) -> PinnedBuffer:
    return PinnedBuffer(shape, dtype)


class HostPipeline:
    """`forward(x)` takes the staged input tensor and returns a tensor or a tuple of tensors.  It is
    run twice eagerly per slot (so that every workspace exists) and then recorded once per slot."""

    def __init__(self, forward: Callable, in_dtype: int, in_shape: Sequence[int], depth: int = 2,
                 home_stream=None, pre_compute: Callable | None = None):
        if depth < 1:
            raise ValueError("depth must be at least 1")
        self.depth = depth
        self.home = home_stream
        self.pre_compute = pre_compute
        self.s_in = _handle(lib.ct_stream_create)
        self.s_compute = _handle(lib.ct_stream_create)
        self.s_out = _handle(lib.ct_stream_create)
        self.start = _handle(lib.ct_event_create)
        self.slots = []
        for _ in range(depth):
            x = T.Tensor(in_dtype, in_shape)
            check(lib.ct_fill(in_dtype, 0.0, x.numel, x.ptr))
            for _ in range(2):
                warm = forward(x)
            T.check_async()
            del warm
            with T.Graph() as g:
                outs = forward(x)
                g.keep = outs
            outs = outs if isinstance(outs, tuple) else (outs,)
            self.slots.append({
                "x": x, "graph": g, "outs": outs,
                "ready": _handle(lib.ct_event_create),
                "computed": _handle(lib.ct_event_create),
                "drained": _handle(lib.ct_event_create),
            })
        self.in_bytes = self.slots[0]["x"].nbytes
        self.out_bytes = [o.nbytes for o in self.slots[0]["outs"]]

    def run(self, inputs: Sequence[int], outputs: Sequence[Sequence[int]]) -> float:
        """inputs[i]: host address of batch i; outputs[i]: host addresses, one per result of
        `forward`.  Returns the device time in ms from the first copy's start to the last
        read-back's end; the host has the results when this returns."""
        n = len(inputs)
        if n == 0:
            return 0.0
        if len(outputs) != n:
            raise ValueError("one output tuple per input batch")
        check(lib.ct_sync())
        try:
            check(lib.ct_set_stream(self.s_in))
            check(lib.ct_event_record(self.start))
            for i in range(n):
                slot = self.slots[i % self.depth]
                check(lib.ct_set_stream(self.s_in))
                if i >= self.depth:
                    check(lib.ct_stream_wait_event(slot["computed"]))  # the slot's previous batch has been consumed
                check(lib.ct_h2d_async(slot["x"].ptr, inputs[i], self.in_bytes))
                check(lib.ct_event_record(slot["ready"]))
                check(lib.ct_set_stream(self.s_compute))
                check(lib.ct_stream_wait_event(slot["ready"]))
                if i >= self.depth:
                    check(lib.ct_stream_wait_event(slot["drained"]))  # its previous results have been read back
                if self.pre_compute is not None:
                    self.pre_compute()
                slot["graph"].launch()
                check(lib.ct_event_record(slot["computed"]))
                check(lib.ct_set_stream(self.s_out))
                check(lib.ct_stream_wait_event(slot["computed"]))
                for dst, out, nbytes in zip(outputs[i], slot["outs"], self.out_bytes):
                    check(lib.ct_d2h_async(dst, out.ptr, nbytes))
                check(lib.ct_event_record(slot["drained"]))
            last = self.slots[(n - 1) % self.depth]["drained"]
            check(lib.ct_event_sync(last))
            for s in (self.s_in, self.s_compute):
                check(lib.ct_set_stream(s))
                check(lib.ct_sync())
            ms = C.c_float()
            check(lib.ct_event_elapsed_ms(self.start, last, C.byref(ms)))
        finally:
            check(lib.ct_set_stream(self.home))
        T.check_async()
        return float(ms.value)

    def close(self) -> None:
        for slot in getattr(self, "slots", []):
            for name in ("ready", "computed", "drained"):
                lib.ct_event_destroy(slot[name])
            slot["graph"] = None
            slot["outs"] = None
            slot["x"] = None
        self.slots = []
        if getattr(self, "start", None) is not None:
            lib.ct_event_destroy(self.start)
            self.start = None
        lib.ct_set_stream(self.home)
        for name in ("s_in", "s_compute", "s_out"):
            s = getattr(self, name, None)
            if s is not None:
                lib.ct_stream_destroy(s)
                setattr(self, name, None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
