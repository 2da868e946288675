"""The plugin's deferred expressions: operator chains exactly as the reference's programs write
them (test/run/nn/svm.cml:31, test/run/nn/mnist.cml:13-25 and 33-41) are run through the plugin's
operator table inside one session, so tensors pass from operator to operator on the device.  The
results must equal the same chains run operator by operator on the CPU restatement, the idioms must
collapse to the fused entry points (launch counts, intermediates never computed), and with
deferral switched off the very same calls must give the plain operator-by-operator results."""
from pathlib import Path

import numpy as np
import pytest

import oracle
from oracle import IntArray

HARNESS = Path(__file__).resolve().parents[1] / "camel_b200" / "host" / "_build" / "libcamel_tensor_host_test.so"
needs_build = pytest.mark.skipif(not HARNESS.exists(), reason="plugin harness not built")
pytestmark = [pytest.mark.gpu, needs_build]


@pytest.fixture(scope="module")
def plugin():
    return oracle.Reference(lib_path=HARNESS)


def canonical_nan(a):
    out = a.copy()
    if out.dtype.kind == "f":
        out[np.isnan(out)] = np.nan
    return out


# ---- the programs, written once against a tiny operator interface ---------------------------


class SessionOps:
    """Operator calls on the plugin (values are handles)."""

    def __init__(self, session):
        self.s = session

    def tensor(self, a):
        return self.s.put(np.ascontiguousarray(a))

    def __getattr__(self, op):
        return lambda *args: self.s.call(op, *args)

    def ones(self, shape):
        return self.s.call("ones", IntArray(shape))

    def reshape(self, t, shape):
        return self.s.call("reshape", t, IntArray(shape))


class PortOps:
    """The same operators on the CPU restatement (values are numpy arrays)."""

    def __init__(self):
        self.p = oracle.port()

    def tensor(self, a):
        return np.ascontiguousarray(a)

    def matmul(self, a, b):
        return self.p.matmul(a, b)

    def subtract(self, a, b):
        return self.p.binary(oracle.SUB, a, b)

    def multiply(self, a, b):
        return self.p.binary(oracle.MUL, a, b)

    def divide(self, a, b):
        return self.p.binary(oracle.DIV, a, b)

    def gt(self, a, b):
        return self.p.compare(oracle.GT, a, b)

    def max_axis(self, a, axis):
        return self.p.max_axis(a, axis)

    def sum_axis(self, a, axis):
        return self.p.sum_axis(a, axis)

    def exp(self, a):
        return self.p.exp(a)

    def transpose(self, a):
        return self.p.transpose(a)

    def ones(self, shape):
        return np.ones(shape, np.float32)

    def reshape(self, t, shape):
        return t.reshape(shape).copy()


def softmax_program(o, logits, n, k):
    """func softmax of test/run/nn/mnist.cml:13-25, operator for operator."""
    row_max = o.max_axis(logits, 1)
    row_max_2d = o.reshape(row_max, [n, 1])
    row_max_broadcast = o.matmul(row_max_2d, o.ones([1, k]))
    stable = o.subtract(logits, row_max_broadcast)
    exp_logits = o.exp(stable)
    row_sums = o.sum_axis(exp_logits, 1)
    row_sums_2d = o.reshape(row_sums, [n, 1])
    row_sums_broadcast = o.matmul(row_sums_2d, o.ones([1, k]))
    return o.divide(exp_logits, row_sums_broadcast), exp_logits


def update_program(o, X, y_onehot, W, lr, m, k):
    """sync func update of test/run/nn/mnist.cml:33-41."""
    logits = o.matmul(X, W)
    probs, _ = softmax_program(o, logits, m, k)
    grad = o.matmul(o.transpose(X), o.subtract(probs, y_onehot))
    return o.subtract(W, o.multiply(lr * (1.0 / float(m)), grad)), probs, logits


# ---- tests -----------------------------------------------------------------------------------


@pytest.mark.parametrize("lazy", [True, False], ids=["deferred", "eager"])
def test_relu_idiom(plugin, lazy):
    ref = PortOps()
    cases = [(n, t, mf) for n in (100_000, 100_003) for t, mf in ((0.0, False), (0.0, True), (0.5, False))]
    for n, threshold, mask_first in cases:
        fused = threshold == 0.0
        h = np.random.default_rng(n).standard_normal(n).astype(np.float32)
        h[:8] = [0.0, -0.0, np.nan, np.inf, -np.inf, 1e-45, -1e-45, 3.0]
        s = plugin.session(lazy)
        o = SessionOps(s)
        ht = o.tensor(h)
        before = s.finish()
        mask = o.gt(ht, threshold)
        prod = o.multiply(mask, ht) if mask_first else o.multiply(ht, mask)
        launches = s.finish(prod) - before
        # the comparison never ran where multiply recognised the idiom, and ran inside it otherwise
        assert s.pending(mask) == (lazy and fused)
        if n % 4 == 0:  # otherwise every pass has a second launch for the ragged tail
            assert launches == (1 if lazy and fused else 2)
        ref_mask = ref.gt(h, threshold)
        ref_prod = ref.multiply(ref_mask, h) if mask_first else ref.multiply(h, ref_mask)
        assert canonical_nan(s.fetch(prod)).tobytes() == canonical_nan(ref_prod).tobytes()
        assert s.fetch(mask).tobytes() == ref_mask.tobytes()  # read after the product: evaluated on demand
        assert not s.pending(mask)


@pytest.mark.parametrize("shape", [(4096, 10), (257, 1000), (64, 5000), (3, 1)])
def test_softmax_idiom_is_one_kernel(plugin, shape):
    n, k = shape
    rng = np.random.default_rng(n * 7 + k)
    logits = (rng.standard_normal(shape) * 4).astype(np.float32)
    ref_probs, ref_exp = softmax_program(PortOps(), logits, n, k)

    s = plugin.session(True)
    o = SessionOps(s)
    lt = o.tensor(logits)
    before = s.finish()
    probs, exp_logits = softmax_program(o, lt, n, k)
    launches = s.finish(probs) - before
    assert launches == 1, launches
    assert s.pending(exp_logits)  # none of the nine intermediate tensors was computed
    got = s.fetch(probs)
    from test_gpu_parity import ulp_distance

    assert ulp_distance(got, ref_probs).max() <= 4
    # an intermediate that is read after all still has the value the chain gives it
    assert ulp_distance(s.fetch(exp_logits), ref_exp).max() <= 1

    s = plugin.session(False)
    o = SessionOps(s)
    before = s.finish()
    probs, exp_logits = softmax_program(o, o.tensor(logits), n, k)
    assert s.finish(probs) - before >= 8  # eleven operators; copies are not kernels
    assert ulp_distance(s.fetch(probs), ref_probs).max() <= 4


def test_softmax_idiom_needs_the_exact_pattern(plugin):
    """A chain that differs from the idiom in one place (the maximum of another tensor) is not
    softmax and is computed operator by operator."""
    rng = np.random.default_rng(5)
    a = rng.standard_normal((300, 12)).astype(np.float32)
    b = rng.standard_normal((300, 12)).astype(np.float32)
    ref = PortOps()

    def program(o, x, y):
        mx = o.matmul(o.reshape(o.max_axis(y, 1), [300, 1]), o.ones([1, 12]))
        e = o.exp(o.subtract(x, mx))
        sums = o.matmul(o.reshape(o.sum_axis(e, 1), [300, 1]), o.ones([1, 12]))
        return o.divide(e, sums)

    s = plugin.session(True)
    o = SessionOps(s)
    out = program(o, o.tensor(a), o.tensor(b))
    from test_gpu_parity import ulp_distance

    assert ulp_distance(s.fetch(out), program(ref, a, b)).max() <= 2


@pytest.mark.parametrize("lazy", [True, False], ids=["deferred", "eager"])
def test_mnist_update_step(plugin, lazy):
    """One SGD step of the softmax classifier, mnist.cml:33-41, on 2048 samples of 785 features."""
    m, d, k, lr = 2048, 785, 10, 0.5
    rng = np.random.default_rng(11)
    X = rng.uniform(0, 1, (m, d)).astype(np.float32)
    X[:, -1] = 1.0
    W = (rng.standard_normal((d, k)) * 0.05).astype(np.float32)
    y = np.zeros((m, k), np.float32)
    y[np.arange(m), rng.integers(0, k, m)] = 1.0
    ref_W, ref_probs, ref_logits = update_program(PortOps(), X, y, W, lr, m, k)

    s = plugin.session(lazy)
    o = SessionOps(s)
    Xt, yt, Wt = o.tensor(X), o.tensor(y), o.tensor(W)
    before = s.finish()
    new_W, probs, logits = update_program(o, Xt, yt, Wt, lr, m, k)
    launches = s.finish(new_W) - before
    got_W, got_probs = s.fetch(new_W), s.fetch(probs)
    assert np.max(np.abs(got_probs - ref_probs)) <= 1e-5
    assert np.max(np.abs(got_W - ref_W)) <= 1e-5 * max(1.0, np.max(np.abs(ref_W)))
    if lazy:
        # 17 operators: classifier with softmax, probs - y, the transposed product, the update
        assert s.pending(logits), "the logits are never written: softmax is fused into the classifier"
        assert launches <= 8, launches
    else:
        assert not s.pending(logits)
        assert launches >= 13, launches  # seventeen operators; copies are not kernels
    assert np.max(np.abs(s.fetch(logits) - ref_logits)) <= 1e-5 * np.max(np.abs(ref_logits))


def test_relu_on_a_matmul_runs_in_the_gemm_epilogue(plugin):
    rng = np.random.default_rng(17)
    x = rng.uniform(-1, 1, (512, 300)).astype(np.float32)
    w = rng.uniform(-1, 1, (300, 256)).astype(np.float32)
    ref = PortOps()
    ref_h = ref.matmul(x, w)
    ref_mask = ref.gt(ref_h, 0.0)
    ref_a = ref.multiply(ref_h, ref_mask)

    s = plugin.session(True)
    o = SessionOps(s)
    h = o.matmul(o.tensor(x), o.tensor(w))
    mask = o.gt(h, 0.0)
    a = o.multiply(h, mask)
    got = s.fetch(a)
    assert s.pending(h) and s.pending(mask)
    scale = np.max(np.abs(ref_h))
    assert np.max(np.abs(got - ref_a)) <= 1e-5 * scale
    # the mask, read afterwards, agrees with the product that was returned, element for element,
    # and with the reference's wherever the pre-activation is not within rounding of zero
    got_mask = s.fetch(mask)
    assert np.array_equal(got_mask != 0, got > 0)
    decided = np.abs(ref_h) > 1e-5 * scale
    assert np.array_equal(got_mask[decided], ref_mask[decided])
    assert s.pending(h)  # still never written
    assert np.max(np.abs(s.fetch(h) - ref_h)) <= 1e-5 * scale


def test_errors_are_raised_by_the_operator_that_owns_them(plugin):
    """Deferred operators have no data-dependent errors; shape errors come at the call."""
    s = plugin.session(True)
    o = SessionOps(s)
    a = o.tensor(np.ones((3, 4), np.float32))
    with pytest.raises(oracle.OracleError, match="matmul dimension mismatch"):
        o.matmul(a, a)
    with pytest.raises(oracle.OracleError, match="matching shapes"):
        o.subtract(a, o.transpose(a))
    zero = o.subtract(a, a)  # deferred
    with pytest.raises(oracle.OracleError, match="Division by zero"):
        o.divide(a, zero)
    with pytest.raises(oracle.OracleError, match="log: input must be positive"):
        o.log(zero)


def test_idioms_from_many_threads(plugin):
    """Operators are called from up to 32 scheduler threads at once
    (src/passes/sched/taskflow/taskflow.h:79-80).  24 threads share one input and one deferred mask
    and race for its evaluation, its buffer and its host mirror; every thread must get the results
    of the single-threaded chains."""
    import ctypes as C

    lib = plugin.lib
    fn = lib.camel_host_threads_idioms
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_char_p, C.c_int]
    rows, cols, threads = 1536, 40, 24
    h = (np.random.default_rng(8).standard_normal((rows, cols)) * 3).astype(np.float32)
    ref = PortOps()
    ref_mask = ref.gt(h, 0.0)
    ref_prod = ref.multiply(h, ref_mask)
    ref_probs, _ = softmax_program(ref, h, rows, cols)
    from test_gpu_parity import ulp_distance

    for _ in range(3):
        prod = np.empty((threads, rows, cols), np.float32)
        probs = np.empty((threads, rows, cols), np.float32)
        mask = np.empty((rows, cols), np.uint8)
        err = C.create_string_buffer(512)
        rc = fn(h.ctypes.data, rows, cols, threads, prod.ctypes.data, probs.ctypes.data, mask.ctypes.data, err, 512)
        assert rc == 0, (rc, err.value.decode())
        assert mask.tobytes() == ref_mask.tobytes()
        for t in range(threads):
            assert prod[t].tobytes() == ref_prod.tobytes(), t
            assert ulp_distance(probs[t], ref_probs).max() <= 4, t


def lr_update_program(o, X, y, w, lr, m):
    """sync func update of test/run/nn/lr.cml:23-32 (linear regression, one output column)."""
    pred = o.matmul(X, w)
    errors = o.subtract(pred, y)
    dw = o.matmul(o.transpose(X), errors)
    dw = o.multiply(2.0 / float(m), dw)
    return o.subtract(w, o.multiply(lr, dw))


@pytest.mark.parametrize("lazy", [True, False], ids=["deferred", "eager"])
def test_linear_regression_update_step(plugin, lazy):
    """predict + update of lr.cml: the bias column by concat(X, ones, 1), then two chained scalings
    in front of the subtraction (only the outer one folds into the update)."""
    m, d, lr = 3000, 64, 0.001
    rng = np.random.default_rng(13)
    X0 = rng.uniform(-1, 1, (m, d)).astype(np.float32)
    y = rng.uniform(-1, 1, (m, 1)).astype(np.float32)
    w = rng.uniform(-1, 1, (d + 1, 1)).astype(np.float32)
    p = oracle.port()
    Xb_ref = p.concat(X0, np.ones((m, 1), np.float32), 1)
    ref = lr_update_program(PortOps(), Xb_ref, y, w, lr, m)

    s = plugin.session(lazy)
    o = SessionOps(s)
    Xb = s.call("concat", o.tensor(X0), o.ones([m, 1]), 1)
    before = s.finish(Xb)
    new_w = lr_update_program(o, Xb, o.tensor(y), o.tensor(w), lr, m)
    launches = s.finish(new_w) - before
    got = s.fetch(new_w)
    assert got.shape == (d + 1, 1)
    assert np.max(np.abs(got - ref)) <= 1e-5 * max(1.0, float(np.max(np.abs(ref))))
    assert np.array_equal(s.fetch(Xb), Xb_ref)
    if lazy:
        # product, difference, transposed product (two kernels), scaling and update (65 values: each a
        # vector launch and one for the ragged tail); no transposed copy of X
        assert launches <= 8, launches


def svm_program(o, X, y_adjusted, weights, bias):
    """The forward half of svm_epoch, test/run/nn/svm.cml:26-40: the hinge loss and the masked
    factor of its gradient.  The mask `hinge_loss > 0` is used twice: once in the relu idiom (never
    computed for it), once times another tensor (computed there)."""
    predictions = o.add(o.matmul(X, weights), bias)
    margins = o.multiply(o.multiply(y_adjusted, predictions), 1.0)
    hinge_loss = o.subtract(1.0, margins)
    hinge_loss_positive = o.multiply(hinge_loss, o.gt(hinge_loss, 0))
    masked = o.multiply(o.multiply(y_adjusted, -1.0), o.gt(hinge_loss, 0))
    return hinge_loss_positive, masked


class _PortOpsWithAdd(PortOps):
    def add(self, a, b):
        return self.p.binary(oracle.ADD, a, b)


@pytest.mark.parametrize("lazy", [True, False], ids=["deferred", "eager"])
def test_svm_hinge_chain(plugin, lazy):
    m, d = 5000, 20
    rng = np.random.default_rng(19)
    X = rng.standard_normal((m, d)).astype(np.float32)
    y = np.where(rng.uniform(size=(m, 1)) < 0.5, -1.0, 1.0).astype(np.float32)
    w = (rng.standard_normal((d, 1)) * 0.3).astype(np.float32)
    ref_pos, ref_masked = svm_program(_PortOpsWithAdd(), X, y, w, 0.25)
    s = plugin.session(lazy)
    o = SessionOps(s)
    pos, masked = svm_program(o, o.tensor(X), o.tensor(y), o.tensor(w), 0.25)
    got_pos, got_masked = s.fetch(pos), s.fetch(masked)
    # one output column: the product is float64-accumulated, so everything downstream is exact
    assert canonical_nan(got_pos).tobytes() == canonical_nan(ref_pos).tobytes()
    assert canonical_nan(got_masked).tobytes() == canonical_nan(ref_masked).tobytes()
