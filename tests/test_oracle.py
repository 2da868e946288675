"""CPU: the C restatement (oracle/camel_tensor_oracle.c) against the reference.

Two pins: the committed golden vectors (produced by the compiled reference, see
tests/golden/make_golden.py), and - where oracle/_ref has been built - the compiled reference
itself, live.  Everything is compared bit for bit, NaN payloads included.
"""
import numpy as np
import pytest

import oracle
from cases import CASES, PortBackend, RefBackend


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
