"""The C++ host side of the plugin (camel_b200/host): `tensor.cmo` and its operator tables.

CPU: the built plugin exports the two entry points Camel's loader looks up
(src/core/module/dynamic.cpp:83-126), its registration table equals the reference's, entry by
entry, and operators refuse to run without a GPU.
GPU: every parity case of tests/cases.py through the plugin's real operator bodies
(`operator_t(with, norm, ctx)` over an ArgsView, as the graph executors call them), compared with
the CPU oracle under the same bars as the C-ABI tests.

The libraries are built by camel_b200/host/Makefile where the reference headers are; the built
files travel with the repository snapshot.
"""
import subprocess
from pathlib import Path

import numpy as np
import pytest

import oracle
from cases import CASES, PortBackend, RefBackend
from oracle import IntArray, With

ROOT = Path(__file__).resolve().parents[1]
BUILD = ROOT / "camel_b200" / "host" / "_build"
CMO = BUILD / "tensor.cmo"
HARNESS = BUILD / "libcamel_tensor_host_test.so"

needs_build = pytest.mark.skipif(not HARNESS.exists(), reason="camel_b200/host/_build not built (needs the reference headers)")


@pytest.fixture(scope="module")
def plugin():
    return oracle.Reference(HARNESS)


@needs_build
def test_cmo_exports_loader_entry_points():
    syms = subprocess.run(["nm", "-D", "--defined-only", str(CMO)], capture_output=True, text=True).stdout
    assert " T camel_module_abi_version" in syms
    assert " T camel_module_create" in syms


@needs_build
def test_registration_table_equals_reference(plugin):
    """Group, URI and signature string of all 37 reference entries, in order; the plugin's own
    operators come after them."""
    ref = [tuple(l.split("\t")) for l in (ROOT / "tests/golden/operator_table.tsv").read_text().splitlines()]
    mine = plugin.groups()
    assert mine[: len(ref)] == ref
    extra = {u for _, u, _ in mine[len(ref):]}
    assert extra == {"tensor:relu", "tensor:softmax", "tensor:dense", "tensor:dense_relu", "tensor:dense_softmax",
                     "tensor:conv2d", "tensor:conv2d_relu", "tensor:maxpool2d", "tensor:flatten",
                     "tensor:matmul_tn", "tensor:scaled_sub", "tensor:conv2d_relu_maxpool2"}
    ops = set(plugin.ops())
    assert {u.split(":")[1] for _, u, _ in mine} == ops
    if oracle.Reference.available():
        assert set(oracle.ref().ops()) <= ops


@needs_build
def test_no_gpu_no_result(plugin):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(oracle.OracleError, match="no CUDA device"):
        plugin.call("add", np.ones(4, np.float32), np.ones(4, np.float32))


class PluginBackend(RefBackend):
    """The reference's operator names on the plugin's tables; relu / softmax / dense are the
    plugin's fused operators instead of the compositions."""

    name = "plugin"

    def __init__(self, plugin):
        self.r = plugin

    def relu(self, a):
        return self.r.call("relu", a)

    def softmax(self, a):
        return self.r.call("softmax", a)

    def dense(self, x, w, b, act):
        if b is None:
            y = self.r.call("matmul", x, w)
            return self.r.call("relu", y) if act == "relu" else y
        return self.r.call("dense_relu" if act == "relu" else "dense", With(w), With(np.asarray(b, np.float32)), x)

    def conv2d(self, x, w, b, stride, pad, act):
        bias = np.zeros(w.shape[0], np.float32) if b is None else np.asarray(b, np.float32)  # `conv2d<w, b, stride, pad>`
        return self.r.call("conv2d_relu" if act == "relu" else "conv2d", With(w), With(bias), With(stride), With(pad), x)

    def maxpool2d(self, x, win):
        return self.r.call("maxpool2d", x, win)


@needs_build
@pytest.mark.gpu
@pytest.mark.parametrize("name,fn", CASES, ids=[c[0] for c in CASES])
def test_plugin_operators_match_oracle(name, fn, plugin, golden):
    from test_gpu_parity import compare_outputs

    got = fn(PluginBackend(plugin))
    ref = fn(PortBackend())
    assert len(got) == len(ref)
    for i, (g, r) in enumerate(zip(got, ref)):
        compare_outputs(name, g, r, f"{name}[{i}] vs oracle")
        compare_outputs(name, g, golden[f"{name}/{i}"], f"{name}[{i}] vs golden")


@needs_build
@pytest.mark.gpu
def test_plugin_errors_shapes_and_new_operators(plugin):
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    with pytest.raises(oracle.OracleError, match="Division by zero"):
        plugin.call("divide", a, np.zeros((3, 4), np.float32))
    with pytest.raises(oracle.OracleError, match="log: input must be positive"):
        plugin.call("log", a)
    with pytest.raises(oracle.OracleError, match="matching shapes"):
        plugin.call("add", a, a.T.copy())
    with pytest.raises(oracle.OracleError, match="matmul dimension mismatch"):
        plugin.call("matmul", a, a)
    assert plugin.call("shape", a) == [3, 4]
    assert plugin.call("idx2d", a, 2, 1) == 9.0
    assert plugin.call("sum", a) == 66.0
    assert plugin.call("full", IntArray([2, 2]), 3).dtype == np.int64  # dtype follows the value's type
    assert plugin.call("range", 5).tolist() == [0, 1, 2, 3, 4]

    rng = np.random.default_rng(21)
    p = oracle.port()
    x = rng.standard_normal((2, 16, 12, 12)).astype(np.float32)
    w = (rng.standard_normal((32, 16, 3, 3)) * 0.1).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, 32).astype(np.float32)
    got = plugin.call("conv2d_relu", With(w), With(b), With(1), With(1), x)
    ref = p.conv2d(x, w, b, 1, 1, 1)
    assert got.shape == ref.shape
    assert np.max(np.abs(got - ref)) / np.max(np.abs(ref)) <= 1e-5
    pooled = plugin.call("maxpool2d", got, 2)
    assert pooled.tobytes() == p.maxpool2d(got, 2).tobytes()
    fused = plugin.call("conv2d_relu_maxpool2", With(w), With(b), With(1), With(1), x)
    assert fused.tobytes() == pooled.tobytes()
    flat = plugin.call("flatten", pooled)
    assert flat.shape == (2, 32 * 6 * 6)
    logits_w = rng.uniform(-0.05, 0.05, (flat.shape[1], 10)).astype(np.float32)
    probs = plugin.call("dense_softmax", With(logits_w), With(np.zeros(10, np.float32)), flat)
    ref_probs = p.softmax_rows(p.dense(flat, logits_w, np.zeros(10, np.float32), 0))
    assert np.max(np.abs(probs - ref_probs)) <= 1e-5

    # the two fused forms of the training loop equal the operator chains they replace
    xs = rng.uniform(0, 1, (300, 200)).astype(np.float32)
    gs = rng.uniform(-1, 1, (300, 64)).astype(np.float32)
    grad = plugin.call("matmul_tn", xs, gs)
    assert grad.tobytes() == plugin.call("matmul", plugin.call("transpose", xs), gs).tobytes()
    w0 = rng.uniform(-1, 1, (200, 64)).astype(np.float32)
    upd = plugin.call("scaled_sub", w0, grad, 0.01 / 300)
    assert upd.tobytes() == plugin.call("subtract", w0, plugin.call("multiply", grad, 0.01 / 300)).tobytes()
    with pytest.raises(oracle.OracleError, match="matching shapes"):
        plugin.call("scaled_sub", w0, xs, 0.1)


@needs_build
@pytest.mark.gpu
def test_plugin_dlpack_device_export_and_import():
    """tensorToDLPackDevice hands out the tensor's own device buffer (kDLCUDA); import copies on
    the device; the reference's host-copy pair still works; the data survives both round trips."""
    import ctypes as C

    lib = C.CDLL(str(HARNESS))
    lib.camel_host_dlpack_roundtrip.restype = C.c_int
    lib.camel_host_dlpack_roundtrip.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_char_p, C.c_int]
    a = np.random.default_rng(7).uniform(-1, 1, (37, 19)).astype(np.float32)
    out = np.zeros_like(a)
    err = C.create_string_buffer(512)
    rc = lib.camel_host_dlpack_roundtrip(a.ctypes.data, 37, 19, out.ctypes.data, err, 512)
    assert rc == 0, (rc, err.value.decode())
    assert out.tobytes() == a.tobytes()
