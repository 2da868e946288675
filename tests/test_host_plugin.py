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
    # the optional lifetime hooks a scheduler finds with dlsym
    for hook in ("camel_tensor_scope_begin", "camel_tensor_scope_end", "camel_tensor_release",
                 "camel_tensor_live_device_bytes"):
        assert f" T {hook}" in syms


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


def _boundary_golden():
    import json

    return json.loads((ROOT / "tests" / "golden" / "boundary.json").read_text())


@needs_build
@pytest.mark.gpu
def test_plugin_graph_boundary_matches_reference(plugin):
    """Array literals in (tensorFromArray, `==` with an array operand, concat of arrays), host
    reads out (idx, idx2d, shape) and the printed form of `show`: the plugin returns and prints
    what the compiled reference did (tests/golden/boundary.json), byte for byte."""
    from cases import boundary_cases, run_boundary_case

    golden = _boundary_golden()
    for name, op, build in boundary_cases():
        got = run_boundary_case(plugin, op, build)
        assert got == golden[name], f"{name}: {got} != {golden[name]}"


@needs_build
@pytest.mark.gpu
def test_plugin_host_reads_copy_once(plugin):
    """idx / idx2d / show / == read a device tensor on the host: the first read of a tensor copies it
    device-to-host once, later reads of the same tensor reuse the mirror; operators between
    device tensors copy nothing."""
    import ctypes as C

    from cases import capture_stdout

    lib = plugin.lib
    lib.camel_host_read_copies.restype = C.c_uint64
    s = plugin.session()
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    v = np.array([0.5, 1.5, -2.5], np.float32)
    ha, hv = s.put(a), s.put(v)
    before = lib.camel_host_read_copies()
    hb = s.call("add", ha, ha)
    hc = s.call("multiply", hb, 0.5)
    s.finish(hc)
    assert lib.camel_host_read_copies() == before            # device to device: no host copy
    assert s.fetch(s.call("idx", hv, 2)) == -2.5
    assert lib.camel_host_read_copies() == before + 1        # the first host read of v
    assert s.fetch(s.call("idx", hv, 0)) == 0.5
    assert lib.camel_host_read_copies() == before + 1        # the mirror is reused
    assert s.fetch(s.call("idx2d", hc, 2, 3)) == 11.0
    assert lib.camel_host_read_copies() == before + 2        # hc evaluated and read once
    _, text = capture_stdout(lambda: s.call("show", hc))
    assert text.startswith("tensor([[") and lib.camel_host_read_copies() == before + 2
    with pytest.raises(oracle.OracleError, match="out of bounds"):
        s.call("idx", hv, 3)
    with pytest.raises(oracle.OracleError, match="rank-1"):
        s.call("idx", ha, 0)


def _sgd_loop(lib, x, y, w, lr, steps, scopes):
    import ctypes as C

    n, d = x.shape
    classes = y.shape[1]
    w = w.copy()
    live = (C.c_uint64 * steps)()
    secs = C.c_double()
    err = C.create_string_buffer(512)
    lib.camel_host_sgd_loop.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_double,
                                        C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_double), C.c_char_p, C.c_int]
    rc = lib.camel_host_sgd_loop(x.ctypes.data, y.ctypes.data, w.ctypes.data, n, d, classes, lr, steps, int(scopes),
                                 C.cast(live, C.c_void_p), C.byref(secs), err, 512)
    assert rc == 0, err.value.decode()
    return w, np.array(list(live), dtype=np.uint64), secs.value


@needs_build
@pytest.mark.gpu
def test_plugin_training_loop_holds_device_memory_flat(plugin):
    """The loop of test/run/nn/mnist.cml:27-41 at MNIST size (60000 x 785 x 10), 2000 steps through
    the operator bodies, each step inside a scope whose only surviving value is the new W (the replaced
    W is released at its last use): the
    module's device bytes are the same after every step (X, y, W and nothing else), and the weights
    equal the same steps computed in float64.  Without scopes the same loop grows every step, which
    is what the reference's collector (no finalisers, no root set: include/camel/core/mm/gen.h:224-227)
    leaves a module with."""
    rng = np.random.default_rng(71)
    n, d, classes = 60000, 785, 10
    x = rng.uniform(0, 1, (n, d)).astype(np.float32)
    x[:, -1] = 1.0
    labels = rng.integers(0, classes, n)
    y = np.eye(classes, dtype=np.float32)[labels]
    w0 = np.zeros((d, classes), np.float32)
    w, live, secs = _sgd_loop(plugin.lib, x, y, w0, 0.1, 2000, True)
    resident = x.nbytes + y.nbytes + w0.nbytes
    print(f"2000 steps in {secs:.2f} s ({secs / 2000 * 1e6:.0f} us per step); device bytes {int(live[0])} .. {int(live[-1])}")
    assert len(set(live.tolist())) == 1, "device memory must not change from step to step"
    assert resident <= int(live[0]) <= resident + 4096
    # the first 20 steps against float64 (the operators round to float32 at every step)
    w20, _, _ = _sgd_loop(plugin.lib, x, y, w0, 0.1, 20, True)
    ref = w0.astype(np.float64)
    xd, yd = x.astype(np.float64), y.astype(np.float64)
    for _ in range(20):
        logits = xd @ ref
        e = np.exp(logits - logits.max(axis=1, keepdims=True))
        ref = ref - 0.1 / n * (xd.T @ (e / e.sum(axis=1, keepdims=True) - yd))
    assert np.max(np.abs(w20 - ref)) <= 1e-5 * max(1.0, float(np.max(np.abs(ref))))
    # no scopes: every step leaves its values behind
    _, grow, _ = _sgd_loop(plugin.lib, x[:6000], y[:6000], w0, 0.1, 30, False)
    assert np.all(np.diff(grow.astype(np.int64)) > 0)
    # eager evaluation inside scopes is flat as well, and gives the same weights as the deferred run
    plugin.session(lazy=False)
    w_eager, live_eager, _ = _sgd_loop(plugin.lib, x[:6000], y[:6000], w0, 0.1, 30, True)
    plugin.session(lazy=True)
    w_lazy, _, _ = _sgd_loop(plugin.lib, x[:6000], y[:6000], w0, 0.1, 30, True)
    assert len(set(live_eager.tolist())) == 1
    assert np.max(np.abs(w_eager - w_lazy)) <= 1e-6  # fused softmax: within 4 ulp of the operator chain


@needs_build
@pytest.mark.gpu
def test_plugin_scope_semantics(plugin):
    """A kept value survives its scope together with what it still needs; everything else is
    released; a released tensor raises when used."""
    import ctypes as C

    lib = plugin.lib
    lib.camel_host_live_device_bytes.restype = C.c_uint64
    lib.camel_host_scope_begin.restype = C.c_uint64
    lib.camel_host_scope_end.argtypes = [C.c_uint64, C.c_int, C.POINTER(C.c_int64), C.c_char_p, C.c_int]
    err = C.create_string_buffer(512)
    s = plugin.session(lazy=True)
    a = np.random.default_rng(5).uniform(-1, 1, (256, 128)).astype(np.float32)
    ha = s.put(a)
    s.finish(ha)
    base = lib.camel_host_live_device_bytes()
    assert base == a.nbytes
    tok = lib.camel_host_scope_begin()
    hb = s.call("add", ha, ha)              # computed at once
    hm = s.call("gt", hb, 0.0)              # deferred: needs hb
    hc = s.call("multiply", hb, 3.0)        # deferred, dropped with the scope
    assert s.pending(hm) and s.pending(hc)
    keep = (C.c_int64 * 1)(hm.index)
    assert lib.camel_host_scope_end(tok, 1, keep, err, 512) == 0, err.value.decode()
    # hb is still held (the kept mask has not run); hc never ran and owns nothing
    assert lib.camel_host_live_device_bytes() == base + a.nbytes
    mask = s.fetch(hm)
    assert np.array_equal(mask, (a + a > 0).astype(np.uint8))
    # the mask has run: hb is free of it and gone; the mask's own buffer remains
    assert lib.camel_host_live_device_bytes() == base + a.size
    for dead in (hb, hc):
        with pytest.raises(oracle.OracleError, match="after the scope"):
            s.fetch(dead)
    with pytest.raises(oracle.OracleError, match="after the scope"):
        s.fetch(s.call("add", hb, ha))
    assert np.array_equal(s.fetch(s.call("add", ha, ha)), a + a)  # values outside the scope are untouched


@needs_build
@pytest.mark.gpu
def test_plugin_reports_kernel_timeout_at_the_host_read(plugin):
    """A contraction whose bounded wait ran out (the device word written from the host, nothing
    waits on the GPU) surfaces as the operator's RuntimeFault when its result is read on the host,
    not as silent garbage; afterwards the plugin works again."""
    from camel_b200._lib import check, lib

    rng = np.random.default_rng(9)
    a = rng.uniform(-1, 1, (512, 512)).astype(np.float32)
    s = plugin.session(lazy=True)
    ha = s.put(a)
    check(lib.ct_inject_status(2, 8))
    hp = s.call("matmul", ha, ha)
    with pytest.raises(oracle.OracleError, match="bounded wait"):
        s.fetch(hp)
    s = plugin.session(lazy=True)
    ha = s.put(a)
    got = s.fetch(s.call("matmul", ha, ha))
    ref = (a.astype(np.float64) @ a.astype(np.float64)).astype(np.float32)
    assert np.max(np.abs(got - ref)) / np.max(np.abs(ref)) <= 1e-5


@needs_build
def test_signature_file_lists_the_registration_table(plugin):
    """camel_b200/stdlib/signatures/tensor.cml (doc-only signatures in the style of the reference's
    stdlib/signatures/globals.cml:8-10) names every (group, URI) pair the module registers, in
    order, with the registered parameter lists, and nothing else."""
    import re

    text = (ROOT / "camel_b200" / "stdlib" / "signatures" / "tensor.cml").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    found = re.findall(r"(?:with <([^>]*)>\s*)?inner func (\w+)\(([^)]*)\): ([^{]+?) \{\s*return '([^']+)'\s*\}", text)
    listed = [(name, uri) for _, name, _, _, uri in found]
    table = plugin.groups()
    assert listed == [(g, u) for g, u, _ in table]
    assert len(listed) == 49
    for (with_params, name, params, ret, uri), (_, _, sig) in zip(found, table):
        want = (f"<{with_params}>" if with_params else "") + f"({params}) => {ret}"
        assert want == sig or sig == "(Tensor, Tensor) => Tensor", (name, want, sig)
    assert {u for _, u in listed} == {"tensor:" + o for o in plugin.ops()}
