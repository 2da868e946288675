"""CPU: the C restatement (oracle/camel_tensor_oracle.c) against the reference.

Two pins: the committed golden vectors (produced by the compiled reference, see
tests/golden/make_golden.py), and - where oracle/_ref has been built - the compiled reference
itself, live.  Everything is compared bit for bit, NaN payloads included.
"""
import numpy as np
import pytest

import oracle
from cases import CASES, PortBackend, RefBackend
from oracle import IntArray


def same_bits(a, b) -> bool:
    a, b = np.asarray(a), np.asarray(b)
    return a.dtype == b.dtype and a.shape == b.shape and a.tobytes() == b.tobytes()


@pytest.fixture(scope="module")
def port_be():
    oracle.build(ref=False)
    return PortBackend()


@pytest.mark.parametrize("name,fn", CASES, ids=[c[0] for c in CASES])
def test_port_matches_golden(name, fn, port_be, golden):
    outs = fn(port_be)
    keys = [k for k in golden.files if k.startswith(name + "/")]
    assert len(keys) == len(outs), "golden fixture is stale: rerun tests/golden/make_golden.py"
    for i, v in enumerate(outs):
        assert same_bits(v, golden[f"{name}/{i}"]), f"{name} output {i} differs from the reference"


@pytest.mark.skipif(not oracle.Reference.available(), reason="oracle/_ref not built here")
@pytest.mark.parametrize("name,fn", CASES, ids=[c[0] for c in CASES])
def test_port_matches_compiled_reference(name, fn, port_be):
    ref_outs = fn(RefBackend())
    for i, (a, b) in enumerate(zip(fn(port_be), ref_outs)):
        assert same_bits(a, b), f"{name} output {i}"


@pytest.mark.skipif(not oracle.Reference.available(), reason="oracle/_ref not built here")
def test_reference_errors_match_port():
    r, p = oracle.ref(), oracle.port()
    a = np.ones((3, 4), np.float32)
    z = np.zeros((3, 4), np.float32)
    for thrower in (lambda: r.call("divide", a, z), lambda: p.binary(oracle.DIV, a, z)):
        with pytest.raises(oracle.OracleError, match="Division by zero"):
            thrower()
    for thrower in (lambda: r.call("divide", a, 0), lambda: p.binary(oracle.DIV, a, 0)):
        with pytest.raises(oracle.OracleError, match="Division by zero"):
            thrower()
    for thrower in (lambda: r.call("log", z), lambda: p.log(z)):
        with pytest.raises(oracle.OracleError, match="log: input must be positive"):
            thrower()
    with pytest.raises(oracle.OracleError, match="matching shapes"):
        r.call("add", a, np.ones((4, 3), np.float32))
    with pytest.raises(oracle.OracleError, match="matmul dimension mismatch"):
        r.call("matmul", a, a)
    with pytest.raises(oracle.OracleError, match="axis must be 0 or 1"):
        r.call("sum_axis", a, 2)


@pytest.mark.skipif(not oracle.Reference.available(), reason="oracle/_ref not built here")
def test_reference_operator_table():
    """The 31 URIs of getTensorOpsMap() (modules/tensor/operators.cpp:160-194)."""
    ops = oracle.ref().ops()
    assert len(ops) == 31
    for name in ("matmul", "add", "sum", "sum_axis", "argmax_axis", "exp", "log", "concat", "reshape"):
        assert name in ops
    groups = oracle.ref().groups()
    uris = {u for _, u, _ in groups}
    assert uris == {"tensor:" + o for o in ops}


@pytest.mark.skipif(not oracle.Reference.available(), reason="oracle/_ref not built here")
def test_maxpool_by_reference_operators_only(port_be):
    """2x2 max-pool written with nothing but reference operators - reshape (runtime.cpp:692-702),
    transpose (704-720) and max over an axis (924-963) - with no gather outside the reference: the
    columns of a window first, then its rows.  On NaN-free data that nesting picks the same element
    as the window scan (among equal values the earlier one), so the bytes must equal the restatement's.
    """
    r = oracle.ref()
    rng = np.random.default_rng(3200)
    for n, c, h, w in ((2, 3, 8, 12), (1, 64, 28, 28), (3, 1, 2, 2)):
        x = rng.standard_normal((n, c, h, w)).astype(np.float32)
        x[0, 0, 0, 0:2] = (0.0, -0.0)
        x[0, 0, 1, 0:2] = (-0.0, 0.0)
        ho, wo = h // 2, w // 2
        cols = r.call("reshape", x, IntArray([n * c * ho * 2 * wo, 2]))                # [(nc, oy, dy, ox), dx]
        m_dx = r.call("max_axis", cols, 1)                                            # [(nc, oy, dy, ox)]
        rows = r.call("reshape", m_dx, IntArray([n * c * ho, 2 * wo]))                 # [(nc, oy), (dy, ox)]
        rows_t = r.call("reshape", r.call("transpose", rows), IntArray([2, wo * n * c * ho]))  # [dy, (ox, nc, oy)]
        m = r.call("reshape", r.call("max_axis", rows_t, 0), IntArray([wo, n * c * ho]))
        out = r.call("reshape", r.call("transpose", m), IntArray([n, c, ho, wo]))
        assert same_bits(out, port_be.maxpool2d(x, 2))


@pytest.mark.skipif(not oracle.Reference.available(), reason="oracle/_ref not built here")
def test_conv2d_by_taps_on_the_reference(port_be):
    """A second composition, coarser than the one of RefBackend: one reference matmul per filter
    tap on the shifted, zero-padded input slice, the partial products added with the reference's
    add (operators.cpp:740-769, runtime.cpp:775-793).  Each tap's product and each add round to
    float32, so this agrees with the single float64 sum to a few roundings, not to the bit."""
    r = oracle.ref()
    rng = np.random.default_rng(3300)
    n, c, h, w, ko, k, pad = 2, 32, 14, 14, 16, 3, 1
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (rng.standard_normal((ko, c, k, k)) * np.sqrt(2.0 / (c * k * k))).astype(np.float32)
    xp = np.zeros((n, c, h + 2 * pad, w + 2 * pad), np.float32)
    xp[:, :, pad:pad + h, pad:pad + w] = x
    ref = port_be.conv2d(x, wt, None, 1, pad, "none")
    for img in range(n):
        acc = None
        for dy in range(k):
            for dx in range(k):
                sl = np.ascontiguousarray(xp[img, :, dy:dy + h, dx:dx + w]).reshape(c, h * w)
                part = r.call("matmul", np.ascontiguousarray(wt[:, :, dy, dx]), sl)
                acc = part if acc is None else r.call("add", acc, part)
        err = np.max(np.abs(acc.reshape(ko, h, w) - ref[img])) / np.max(np.abs(ref[img]))
        assert err <= 2e-6
