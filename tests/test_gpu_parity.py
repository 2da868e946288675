"""GPU: the CUDA library (through its C ABI) against the CPU oracle and the golden vectors.

Bars
 - integer / bool / index outputs, and float32 outputs of + - * / relu, comparisons, movement,
   constructors, max: bit-exact.
 - float32 outputs that pass through exp / log / pow (device libm vs host libm, both rounded
   from float64): at most 1 ulp, and the share of bit-identical values is reported.
 - tensor-core contractions (3xTF32): max |gpu - ref| / max |ref| <= 1e-5, the tolerance the
   path is specified with; also the component-wise error against sum_k |a||b| is bounded.
"""
import numpy as np
import pytest

import oracle
from cases import BIN, CASES, CMP, TOLERANCE_CASES, PortBackend

pytestmark = pytest.mark.gpu

ULP_CASES = ("binary_f32_n", "unary_exp_log", "softmax_rows", "binary_mixed_dtypes")
GEMM_TOL = 1e-5


@pytest.fixture(scope="module")
def T():
    from camel_b200 import tensor

    return tensor


class CudaBackend:
    name = "cuda"

    def __init__(self, T):
        self.T = T

    def _t(self, a):
        return self.T.from_numpy(np.asarray(a)) if isinstance(a, np.ndarray) else a

    def _n(self, t):
        out = t.numpy()
        self.T.check_async()
        return out

    def binary(self, op, a, b):
        return self._n(getattr(self.T, op)(self._t(a), self._t(b)))

    def compare(self, op, a, b):
        return self._n(getattr(self.T, op)(self._t(a), self._t(b)))

    def sum(self, a):
        return self.T.sum(self._t(a))

    def sum_axis(self, a, ax):
        return self._n(self.T.sum(self._t(a), ax))

    def max_axis(self, a, ax):
        return self._n(self.T.max(self._t(a), ax))

    def argmax_axis(self, a, ax):
        return self._n(self.T.argmax(self._t(a), ax))

    def exp(self, a):
        return self._n(self.T.exp(self._t(a)))

    def log(self, a):
        return self._n(self.T.log(self._t(a)))

    def transpose(self, a):
        return self._n(self.T.transpose(self._t(a)))

    def concat(self, a, b, ax):
        return self._n(self.T.concat(self._t(a), self._t(b), ax))

    def reshape(self, a, shape):
        return self._n(self.T.reshape(self._t(a), shape))

    def matmul(self, a, b):
        return self._n(self.T.matmul(self._t(a), self._t(b)))

    def relu(self, a):
        return self._n(self.T.relu(self._t(a)))

    def softmax(self, a):
        return self._n(self.T.softmax(self._t(a)))

    def dense(self, x, w, b, act):
        return self._n(self.T.dense(self._t(x), self._t(w), self._t(b) if b is not None else None, act))

    def conv2d(self, x, w, b, stride, pad, act):
        return self._n(self.T.conv2d(self._t(x), self._t(w), self._t(b) if b is not None else None, stride, pad,
                                     None if act == "none" else act))

    def maxpool2d(self, x, win):
        return self._n(self.T.maxpool2d(self._t(x), win))

    def ones(self, shape):
        return self._n(self.T.ones(shape))

    def zeros(self, shape):
        return self._n(self.T.zeros(shape))

    def full(self, shape, v):
        return self._n(self.T.full(shape, v))

    def eye(self, n):
        return self._n(self.T.eye(n))

    def range(self, start, stop, step):
        return self._n(self.T.range(start, stop, step))


def ulp_distance(a, b):
    """Distance in float32 ulps; NaN==NaN, equal infinities are 0."""
    ai = a.view(np.int32).astype(np.int64)
    bi = b.view(np.int32).astype(np.int64)
    ai = np.where(ai < 0, np.int64(-(2**31)) - ai, ai)
    bi = np.where(bi < 0, np.int64(-(2**31)) - bi, bi)
    d = np.abs(ai - bi)
    both_nan = np.isnan(a) & np.isnan(b)
    return np.where(both_nan, 0, d)


def assert_close_gemm(got, ref):
    assert got.shape == ref.shape and got.dtype == ref.dtype
    if ref.size == 0:
        return
    scale = float(np.max(np.abs(ref))) or 1.0
    err = float(np.max(np.abs(got.astype(np.float64) - ref.astype(np.float64)))) / scale
    assert err <= GEMM_TOL, f"max|d|/max|ref| = {err:.3e} > {GEMM_TOL}"


def canonical_nan(a):
    """NaN payload and sign are not part of the result: x86 SSE produces the 'indefinite' NaN
    0xFFC00000 (and propagates input payloads), the GPU produces 0x7FFFFFFF.  Where one side has
    a NaN the other must have one too; which NaN is not compared."""
    if a.dtype.kind != "f":
        return a
    out = a.copy()
    out[np.isnan(out)] = np.nan
    return out


def compare_outputs(name, got, ref, label):
    got, ref = np.asarray(got), np.asarray(ref)
    assert got.shape == ref.shape, f"{label}: shape {got.shape} vs {ref.shape}"
    assert got.dtype == ref.dtype, f"{label}: dtype {got.dtype} vs {ref.dtype}"
    got, ref = canonical_nan(got), canonical_nan(ref)
    if got.tobytes() == ref.tobytes():
        return 1.0
    if name in TOLERANCE_CASES:
        assert_close_gemm(got, ref)
        return float(np.mean(got == ref))
    if ref.dtype == np.float64:  # full sums: float64 scalars, summation order differs
        assert abs(float(got) - float(ref)) <= 1e-12 * max(1.0, abs(float(ref))) + 1e-9, label
        return 0.0
    if ref.dtype == np.float32 and name.startswith(ULP_CASES):
        d = ulp_distance(got, ref)
        # exp, log, pow: within 1 ulp.  softmax divides an exp (<= 1 ulp) by a rounded sum of them and
        # rounds again: up to 4 ulp (4.8e-7 relative; the path is specified to 1e-5)
        bar = 4 if name.startswith("softmax_rows") else 1
        assert d.max() <= bar, f"{label}: {int(d.max())} ulp apart at {np.unravel_index(d.argmax(), d.shape)}"
        return float(np.mean(d == 0))
    raise AssertionError(f"{label}: not bit-exact")


@pytest.mark.parametrize("name,fn", CASES, ids=[c[0] for c in CASES])
def test_cuda_matches_oracle_and_golden(name, fn, T, golden):
    oracle.build(ref=False)
    got = fn(CudaBackend(T))
    ref = fn(PortBackend())
    assert len(got) == len(ref)
    for i, (g, r) in enumerate(zip(got, ref)):
        compare_outputs(name, g, r, f"{name}[{i}] vs oracle")
        compare_outputs(name, g, golden[f"{name}/{i}"], f"{name}[{i}] vs golden")


def test_error_behaviour(T):
    """Same exceptions, same text, as the reference (modules/tensor/runtime.cpp:122-124, 1039-1041)."""
    import camel_b200

    a = T.from_numpy(np.ones((3, 4), np.float32))
    z = T.from_numpy(np.zeros((3, 4), np.float32))
    zi = T.from_numpy(np.zeros((3, 4), np.int64))
    for bad in (lambda: T.divide(a, z), lambda: T.divide(a, 0), lambda: T.divide(a, zi), lambda: T.divide(1.0, z)):
        with pytest.raises(camel_b200.CamelTensorError, match="Division by zero") as e:
            bad()
        assert e.value.status == camel_b200._lib.ERR_DIV_ZERO
    with pytest.raises(camel_b200.CamelTensorError, match="log: input must be positive"):
        T.log(z)
    with pytest.raises(camel_b200.CamelTensorError, match="matching shapes"):
        T.add(a, T.from_numpy(np.ones((4, 3), np.float32)))
    with pytest.raises(camel_b200.CamelTensorError, match="matmul dimension mismatch"):
        T.matmul(a, a)
    with pytest.raises(camel_b200.CamelTensorError, match="axis must be 0 or 1"):
        T.sum(a, 2)
    # the context is still healthy after the reported errors
    assert T.sum(T.add(a, a)) == 24.0


def _rel_err(got, ref):
    return float(np.max(np.abs(got.astype(np.float64) - ref.astype(np.float64)))) / float(np.max(np.abs(ref)))


def _ref_matmul_f64(a, b):
    return (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)


def test_dense_split_k(T):
    """Few output tiles, long reduction: the k range is sliced across CTAs and the partial sums
    are added (with bias and relu) by a second kernel."""
    rng = np.random.default_rng(12)
    x = rng.uniform(0, 1, (300, 3000)).astype(np.float32)
    w = rng.uniform(-0.05, 0.05, (3000, 100)).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, 100).astype(np.float32)
    ref = np.maximum((x.astype(np.float64) @ w.astype(np.float64) + b).astype(np.float32), 0)
    got = T.dense(T.from_numpy(x), T.from_numpy(w), T.from_numpy(b), "relu").numpy()
    T.check_async()
    assert _rel_err(got, ref) <= GEMM_TOL


@pytest.mark.parametrize("m,k,n,act", [(300, 1000, 10, "softmax"), (257, 36, 7, "relu"), (1024, 1024, 10, "softmax"),
                                       (4096, 128, 10, "softmax"), (512, 2048, 16, None), (260, 40, 1, None),
                                       (512, 1100, 3, "softmax"),
                                       # k not a multiple of four: rows at any 4-byte address (784 features + bias column)
                                       (4096, 785, 10, "softmax"), (300, 33, 10, None), (1000, 1023, 16, "relu"),
                                       (257, 509, 5, "softmax"), (256, 34, 2, None)])
def test_dense_few_columns_row_tiled(T, m, k, n, act):
    """Classifier-layer shapes (n <= 16, many rows): float64 accumulation, so logits agree with
    float64-matmul-rounded-once to the last bit except where the summation order shows (<= 1 ulp),
    rows past a multiple of 32 and slices past k are masked, argmax is exact."""
    rng = np.random.default_rng(m * 7 + k + n)
    x = rng.uniform(0, 1, (m, k)).astype(np.float32)
    w = rng.uniform(-0.1, 0.1, (k, n)).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, n).astype(np.float32)
    logits = (x.astype(np.float64) @ w.astype(np.float64) + b).astype(np.float32)
    if act == "softmax":
        got, arg = T.dense(T.from_numpy(x), T.from_numpy(w), T.from_numpy(b), "softmax", with_argmax=True)
        got, arg = got.numpy(), arg.numpy()
        T.check_async()
        e = np.exp((logits - logits.max(axis=1, keepdims=True)).astype(np.float64))
        ref = (e / e.sum(axis=1, keepdims=True)).astype(np.float32)
        assert np.max(np.abs(got - ref)) <= 1e-6
        srt = np.sort(logits, axis=1)
        decided = (srt[:, -1] - srt[:, -2] > 1e-6) if n > 1 else np.ones(m, bool)
        assert np.array_equal(arg[decided], np.argmax(logits, axis=1)[decided])
    else:
        got = T.dense(T.from_numpy(x), T.from_numpy(w), T.from_numpy(b), act).numpy()
        T.check_async()
        ref = np.maximum(logits, 0) if act == "relu" else logits
        ulp = np.spacing(np.maximum(np.abs(ref), np.float32(1e-3)))
        assert np.all(np.abs(got - ref) <= ulp)


@pytest.mark.parametrize("m,k,n", [(512, 512, 512), (384, 1000, 640), (1024, 784, 1024), (2048, 4096, 512),
                                   (256, 4096, 128), (130, 9000, 257),
                                   (3000, 600, 2500), (4096, 1024, 4096), (2500, 40, 3001)])  # tiles > SMs, k <= 1024
def test_gemm_3xtf32_large(T, m, k, n):
    """Sizes past what the scalar oracle finishes quickly: numpy float64 matmul rounded once is
    the same function (the oracle agrees with it to the last bit on the sizes of tests/cases.py
    up to the summation order, which float64 makes immaterial at 1e-5)."""
    rng = np.random.default_rng(m + k + n)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    got = T.matmul(T.from_numpy(a), T.from_numpy(b)).numpy()
    T.check_async()
    ref = _ref_matmul_f64(a, b)
    err = _rel_err(got, ref)
    comp = float(np.max(np.abs(got.astype(np.float64) - ref) / (np.abs(a).astype(np.float64) @ np.abs(b))))
    print(f"gemm {m}x{k}x{n}: max|d|/max|ref|={err:.3e} componentwise={comp:.3e}")
    assert err <= GEMM_TOL
    assert comp <= 1e-5


def test_gemm_cfg1_against_oracle(T):
    """BASELINE config 1: 512^3, U(-1,1), seed 0 - against the scalar oracle itself."""
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (512, 512)).astype(np.float32)
    b = rng.uniform(-1, 1, (512, 512)).astype(np.float32)
    ref = oracle.port().matmul(a, b)
    got = T.matmul(T.from_numpy(a), T.from_numpy(b)).numpy()
    T.check_async()
    assert _rel_err(got, ref) <= GEMM_TOL


def test_gemm_linearity_property(T):
    """Size-independent property at a larger size: (A1 + A2) B == A1 B + A2 B within tolerance."""
    rng = np.random.default_rng(5)
    m = k = n = 2048
    a1 = T.from_numpy(rng.uniform(-1, 1, (m, k)).astype(np.float32))
    a2 = T.from_numpy(rng.uniform(-1, 1, (m, k)).astype(np.float32))
    b = T.from_numpy(rng.uniform(-1, 1, (k, n)).astype(np.float32))
    lhs = T.matmul(T.add(a1, a2), b).numpy()
    rhs = T.add(T.matmul(a1, b), T.matmul(a2, b)).numpy()
    T.check_async()
    assert _rel_err(lhs, rhs) <= 3 * GEMM_TOL


def test_gemm_bf16_mode(T):
    import camel_b200
    from camel_b200 import _lib

    rng = np.random.default_rng(6)
    a = rng.uniform(-1, 1, (512, 768)).astype(np.float32)
    b = rng.uniform(-1, 1, (768, 384)).astype(np.float32)
    _lib.check(camel_b200.lib.ct_set_precision(_lib.PREC_BF16))
    try:
        got = T.matmul(T.from_numpy(a), T.from_numpy(b)).numpy()
        T.check_async()
    finally:
        _lib.check(camel_b200.lib.ct_set_precision(_lib.PREC_3XTF32))
    assert _rel_err(got, _ref_matmul_f64(a, b)) <= 1e-2


def test_mlp_forward_cfg2_slice(T):
    """BASELINE config 2 on a 512-sample slice: probabilities within tolerance, argmax equal
    wherever the oracle's top-2 logit gap exceeds the contraction tolerance."""
    rng = np.random.default_rng(1)

    def kaiming(fan_in, fan_out):
        lim = np.sqrt(6.0 / fan_in)
        return rng.uniform(-lim, lim, (fan_in, fan_out)).astype(np.float32)

    w1, w2, w3 = kaiming(784, 1024), kaiming(1024, 1024), kaiming(1024, 10)
    b1, b2, b3 = (np.zeros(n, np.float32) for n in (1024, 1024, 10))
    x = np.random.default_rng(2).uniform(0, 1, (512, 784)).astype(np.float32)
    p = oracle.port()
    h1 = p.dense(x, w1, b1, 1)
    h2 = p.dense(h1, w2, b2, 1)
    logits = p.dense(h2, w3, b3, 0)
    probs_ref = p.softmax_rows(logits)
    arg_ref = p.argmax_axis(logits, 1)

    tx = T.from_numpy(x)
    g1 = T.dense(tx, T.from_numpy(w1), T.from_numpy(b1), "relu")
    g2 = T.dense(g1, T.from_numpy(w2), T.from_numpy(b2), "relu")
    probs, arg = T.dense(g2, T.from_numpy(w3), T.from_numpy(b3), "softmax", with_argmax=True)
    probs, arg = probs.numpy(), arg.numpy()
    T.check_async()
    assert np.max(np.abs(probs - probs_ref)) <= 1e-5
    srt = np.sort(logits, axis=1)
    gap = srt[:, -1] - srt[:, -2]
    decided = gap > 1e-4 * np.max(np.abs(logits))
    assert decided.mean() > 0.95
    assert np.array_equal(arg[decided], arg_ref[decided])
    assert arg.dtype == np.int64


@pytest.mark.parametrize("n,c,h,w,ko,kk,stride,pad,act", [
    (2, 3, 9, 11, 5, 3, 1, 1, "relu"),      # few input channels: register-patch kernel
    (1, 8, 6, 6, 4, 3, 1, 1, None),         # tiny: one thread per output
    (1, 1, 28, 28, 32, 3, 1, 1, "relu"),    # first CNN layer: c*kh*kw = 9
    (3, 32, 28, 28, 64, 3, 1, 1, "relu"),   # second CNN layer
    (2, 64, 56, 56, 128, 3, 1, 1, "relu"),  # BASELINE config 3 geometry, small batch
    (2, 16, 20, 20, 48, 5, 2, 2, None),     # stride 2, 5x5: patch-matrix path
    (3, 48, 30, 30, 200, 3, 1, 0, "relu"),  # no padding (wo < w), channels and filters off the tile sizes
    (2, 32, 28, 28, 64, 1, 1, 0, None),     # 1x1 filter
    (2, 20, 13, 16, 130, 3, 1, 1, "relu"),  # odd height, last row tile partial, c < 32
    (1, 64, 7, 40, 16, 5, 1, 2, None),      # 5x5, pad 2
    (12, 32, 56, 56, 128, 3, 1, 1, "relu"), # 168 tiles > SMs, k = 288: one CTA per SM walks the tiles
    (40, 32, 28, 28, 64, 3, 1, 1, "relu"),  # the same with half-used row tiles and a ragged last pixel tile
    (10, 24, 36, 60, 130, 3, 1, 1, None),   # streamed, two row tiles (the second nearly empty), c < 32
])
def test_conv2d(T, n, c, h, w, ko, kk, stride, pad, act):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (rng.standard_normal((ko, c, kk, kk)) * np.sqrt(2.0 / (c * kk * kk))).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, ko).astype(np.float32)
    ref = oracle.port().conv2d(x, wt, b, stride, pad, 1 if act == "relu" else 0)
    got = T.conv2d(T.from_numpy(x), T.from_numpy(wt), T.from_numpy(b), stride, pad, act).numpy()
    T.check_async()
    assert got.shape == ref.shape
    assert _rel_err(got, ref) <= GEMM_TOL


def test_cnn_forward_cfg4_slice(T):
    """BASELINE config 4 on 48 images: conv-relu, conv-relu, maxpool, flatten, dense-relu,
    dense-softmax; probabilities within tolerance and argmax equal where the oracle's top-2 gap
    is above the contraction tolerance."""
    rng = np.random.default_rng(4)

    def kaiming(shape, fan_in):
        lim = np.sqrt(6.0 / fan_in)
        return rng.uniform(-lim, lim, shape).astype(np.float32)

    w1, w2 = kaiming((32, 1, 3, 3), 9), kaiming((64, 32, 3, 3), 288)
    w3, w4 = kaiming((12544, 128), 12544), kaiming((128, 10), 128)
    b1, b2, b3, b4 = (rng.uniform(-0.05, 0.05, n).astype(np.float32) for n in (32, 64, 128, 10))
    x = rng.uniform(0, 1, (48, 1, 28, 28)).astype(np.float32)
    p = oracle.port()
    h = p.conv2d(x, w1, b1, 1, 1, 1)
    h = p.conv2d(h, w2, b2, 1, 1, 1)
    h = p.maxpool2d(h, 2).reshape(48, -1)
    h = p.dense(h, w3, b3, 1)
    logits = p.dense(h, w4, b4, 0)
    probs_ref, arg_ref = p.softmax_rows(logits), p.argmax_axis(logits, 1)

    g = T.conv2d(T.from_numpy(x), T.from_numpy(w1), T.from_numpy(b1), 1, 1, "relu")
    g = T.conv2d(g, T.from_numpy(w2), T.from_numpy(b2), 1, 1, "relu")
    g = T.flatten(T.maxpool2d(g, 2))
    assert g.shape == (48, 12544)
    g = T.dense(g, T.from_numpy(w3), T.from_numpy(b3), "relu")
    probs, arg = T.dense(g, T.from_numpy(w4), T.from_numpy(b4), "softmax", with_argmax=True)
    probs, arg = probs.numpy(), arg.numpy()
    T.check_async()
    assert np.max(np.abs(probs - probs_ref)) <= 1e-5
    srt = np.sort(logits, axis=1)
    decided = (srt[:, -1] - srt[:, -2]) > 1e-4 * np.max(np.abs(logits))
    assert np.array_equal(arg[decided], arg_ref[decided])


def test_softmax_wide_rows(T):
    """Row widths that take the 128-bit block kernels, incl. a NaN first element and -inf."""
    rng = np.random.default_rng(31)
    for shape in ((3, 516), (5, 2048), (2, 4100), (3, 8192), (2, 8196)):
        x = rng.uniform(-8, 8, shape).astype(np.float32)
        x[0, 5] = -np.inf
        if shape[0] > 2:
            x[2, 0] = np.nan
        ref = oracle.port().softmax_rows(x)
        got = T.softmax(T.from_numpy(x)).numpy()
        compare_outputs("softmax_rows", got, ref, f"softmax {shape}")


def test_maxpool2d(T):
    rng = np.random.default_rng(4)
    for shape, win in (((3, 5, 28, 28), 2), ((2, 3, 9, 12), 3), ((1, 1, 7, 7), 2), ((2, 3, 10, 30), 2),
                       ((4, 2, 6, 8), 2)):
        x = rng.standard_normal(shape).astype(np.float32)
        x[0, 0, 0, 0] = np.nan  # a NaN that opens a window stays; one that does not never wins
        x[-1, -1, 1, 3] = np.nan
        ref = oracle.port().maxpool2d(x, win)
        got = T.maxpool2d(T.from_numpy(x), win).numpy()
        assert got.tobytes() == ref.tobytes()


def test_elementwise_large_roundtrip_properties(T):
    """Properties that hold at any size, run at 2^26 elements: (a + b) - b == a wherever the sum is
    exact enough, relu(x) + relu(-x) == |x|, sum of a 0/1 mask equals its popcount."""
    n = 1 << 26
    rng = np.random.default_rng(6)
    x = rng.uniform(-1, 1, n).astype(np.float32)
    tx = T.from_numpy(x)
    pos = T.relu(tx)
    neg = T.relu(T.multiply(tx, -1.0))
    both = T.add(pos, neg).numpy()
    assert np.array_equal(both, np.abs(x))
    mask = T.gt(tx, 0.0)
    assert T.sum(mask) == float(np.count_nonzero(x > 0))
    s = T.sum(tx)
    assert abs(s - float(np.sum(x.astype(np.float64)))) <= 1e-9 * n


def test_graph_replay_matches_eager(T):
    """A recorded dense -> relu -> dense -> softmax chain replays with new input contents and
    gives the same bytes as the call-by-call run."""
    rng = np.random.default_rng(8)
    w1 = T.from_numpy(rng.uniform(-0.2, 0.2, (96, 160)).astype(np.float32))
    b1 = T.from_numpy(rng.uniform(-0.1, 0.1, 160).astype(np.float32))
    w2 = T.from_numpy(rng.uniform(-0.2, 0.2, (160, 10)).astype(np.float32))
    x_np = [rng.uniform(0, 1, (300, 96)).astype(np.float32) for _ in range(3)]
    x = T.from_numpy(x_np[0])

    def forward(inp):
        h = T.dense(inp, w1, b1, "relu")
        return T.dense(h, w2, None, "softmax", with_argmax=True)

    warm = forward(x)
    T.check_async()
    with T.Graph() as g:
        g.keep = forward(x)
    for a in x_np:
        from camel_b200._lib import check, lib
        check(lib.ct_h2d(x.ptr, a.ctypes.data, a.nbytes))
        g.launch()
        probs_g, arg_g = g.keep[0].numpy(), g.keep[1].numpy()
        probs_e, arg_e = forward(T.from_numpy(a))
        assert probs_g.tobytes() == probs_e.numpy().tobytes()
        assert arg_g.tobytes() == arg_e.numpy().tobytes()
    T.check_async()
    del warm


def test_exp_log_float32_paths_against_float64_rounded_once(T):
    """exp and log run in float32 arithmetic with compensation: against float(f(double(x))), the
    reference's definition, never more than 1 ulp, nearly always identical, across the whole range
    (results that overflow, underflow or are subnormal, subnormal arguments, inf, NaN)."""
    rng = np.random.default_rng(33)
    x = np.concatenate([
        rng.uniform(-87, 87, 2_000_000), rng.uniform(-1, 1, 1_000_000), rng.normal(0, 3, 1_000_000),
        rng.uniform(-110, -86, 100_000), rng.uniform(86, 90, 100_000),
        [0.0, -0.0, np.inf, -np.inf, np.nan, 88.72283, 88.72284, -103.97, -104.0, -87.33655, 1e-30, -1e-30],
    ]).astype(np.float32)
    with np.errstate(over="ignore", under="ignore"):
        ref = np.exp(x.astype(np.float64)).astype(np.float32)
    got = T.exp(T.from_numpy(x)).numpy()
    T.check_async()
    d = ulp_distance(canonical_nan(got), canonical_nan(ref))
    print(f"exp: max {int(d.max())} ulp, identical {np.mean(d == 0):.4f}")
    assert d.max() <= 1 and np.mean(d == 0) > 0.97
    assert np.isnan(got[np.isnan(x)]).all() and got[x == np.inf][0] == np.inf and got[x == -np.inf][0] == 0.0

    y = np.concatenate([
        rng.uniform(0.5, 2, 1_000_000), np.exp(rng.uniform(-87, 88, 2_000_000)), rng.uniform(0.99, 1.01, 500_000),
        rng.uniform(0, 1, 500_000), rng.uniform(1e-45, 1.2e-38, 100_000),
        [1.0, np.inf, np.nan, 1.4e-45, 3.4028235e38, 1.1754944e-38, 0.70710677, 0.7071068, 1.4142135, 1.4142137],
    ]).astype(np.float32)
    y = y[~(y <= 0)]
    ref = np.log(y.astype(np.float64)).astype(np.float32)
    got = T.log(T.from_numpy(y)).numpy()
    T.check_async()
    d = ulp_distance(canonical_nan(got), canonical_nan(ref))
    print(f"log: max {int(d.max())} ulp, identical {np.mean(d == 0):.4f}")
    assert d.max() <= 1 and np.mean(d == 0) > 0.97
    assert got[y == 1.0][0] == 0.0 and got[np.isinf(y)][0] == np.inf and np.isnan(got[np.isnan(y)]).all()


@pytest.mark.parametrize("n,c,h,w,ko,kk,pad", [
    (3, 32, 28, 28, 64, 3, 1),    # second CNN layer: fused in the convolution's epilogue
    (40, 32, 28, 28, 64, 3, 1),   # more tiles than SMs
    (2, 16, 12, 40, 24, 3, 1),    # wo = 40: two output rows per tile, 24 filters
    (2, 32, 10, 10, 64, 3, 0),    # no padding: 8 x 8 output
    (2, 32, 14, 14, 128, 3, 1),   # 128 filters: not a shape of the fused kernel (conv, then pool)
    (2, 8, 9, 9, 16, 3, 1),       # odd output size, few channels: conv, then pool
])
def test_conv2d_with_fused_maxpool(T, n, c, h, w, ko, kk, pad):
    """conv2d(..., relu, pool=2) gives the bytes of maxpool2d(conv2d(..., relu), 2), whichever
    kernels serve the shape, including a NaN in the input (it must spread exactly as unfused)."""
    rng = np.random.default_rng(n * 100 + c + h + ko)
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    x[0, 0, 1, 1] = np.nan
    wt = (rng.standard_normal((ko, c, kk, kk)) * np.sqrt(2.0 / (c * kk * kk))).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, ko).astype(np.float32)
    tx, tw, tb = T.from_numpy(x), T.from_numpy(wt), T.from_numpy(b)
    fused = T.conv2d(tx, tw, tb, 1, pad, "relu", pool=2).numpy()
    chain = T.maxpool2d(T.conv2d(tx, tw, tb, 1, pad, "relu"), 2).numpy()
    T.check_async()
    assert fused.shape == chain.shape
    assert canonical_nan(fused).tobytes() == canonical_nan(chain).tobytes()


@pytest.mark.parametrize("n,c,h,w,ko,kk,pad,pool", [
    (3, 32, 28, 28, 64, 3, 1, 0),    # second CNN layer
    (3, 32, 28, 28, 64, 3, 1, 2),    # ... with the pool in the epilogue
    (2, 20, 16, 24, 48, 3, 1, 0),    # fewer than 32 channels: the box reads zeros past the last one
    (2, 32, 12, 20, 64, 5, 2, 0),    # 5 x 5 filter, padding 2
    (2, 32, 10, 12, 64, 3, 0, 0),    # no padding
])
def test_conv2d_reads_its_input_directly_or_from_planes(T, n, c, h, w, ko, kk, pad, pool):
    """The few-channel convolution kernel reads an aligned NCHW input as it is and splits it into
    tf32 parts itself; an input at an address its tensor map cannot take goes through the NHWC-plane
    pre-pass.  Same input at both kinds of address: same bytes out, special values included."""
    import torch

    rng = np.random.default_rng(n + c + h + w + ko + pool)
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    x[0, 0, 1, 1] = np.inf
    x[0, 1, 2, 3] = np.float32(3.4e38)          # rounds up to infinity as tf32: has to be truncated
    x[1, 0, 0, 0] = np.float32(1e-41)           # subnormal
    x[1, 2, 3, 1] = np.nan
    wt = (rng.standard_normal((ko, c, kk, kk)) * np.sqrt(2.0 / (c * kk * kk))).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, ko).astype(np.float32)
    tw, tb = T.from_numpy(wt), T.from_numpy(b)
    outs = []
    for shift in (0, 1):                         # 1: the tensor starts 4 bytes past a 16-byte boundary
        buf = torch.empty(x.size + 4, dtype=torch.float32, device="cuda")
        view = buf[shift:shift + x.size]
        view.copy_(torch.from_numpy(x.reshape(-1)))
        assert view.data_ptr() % 16 == 4 * shift
        tx = T.wrap_device(view.data_ptr(), 0, x.shape, keep=buf)
        outs.append(T.conv2d(tx, tw, tb, 1, pad, "relu", pool=pool).numpy())
    T.check_async()
    assert canonical_nan(outs[0]).tobytes() == canonical_nan(outs[1]).tobytes()


def test_entry_points_from_many_threads(T):
    """The reference's Taskflow scheduler calls operators from up to 32 threads at once.  Entry
    points that enqueue several kernels over a shared workspace must not interleave: eight threads
    run different dense / softmax / sum calls concurrently and get the single-threaded bytes."""
    import threading

    rng = np.random.default_rng(77)
    jobs = []
    for i in range(8):
        m, k, n = 200 + 37 * i, 96 + 32 * i, 64 + 48 * i
        x = T.from_numpy(rng.uniform(0, 1, (m, k)).astype(np.float32))
        w = T.from_numpy(rng.uniform(-0.2, 0.2, (k, n)).astype(np.float32))
        b = T.from_numpy(rng.uniform(-0.1, 0.1, n).astype(np.float32))
        jobs.append((x, w, b))

    def work(job):
        x, w, b = job
        h = T.dense(x, w, b, "relu")
        return T.softmax(h).numpy(), T.sum(h)

    expected = [work(j) for j in jobs]
    T.check_async()
    results, errors = [None] * len(jobs), []

    def runner(idx):
        try:
            for _ in range(20):
                results[idx] = work(jobs[idx])
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=runner, args=(i,)) for i in range(len(jobs))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    T.check_async()
    assert not errors, errors
    for (p_exp, s_exp), (p_got, s_got) in zip(expected, results):
        assert p_got.tobytes() == p_exp.tobytes() and s_got == s_exp


def test_training_step_fused_forms(T):
    """transpose(X) @ G and W - lr * g as single calls give the bytes of the operator chains of
    test/run/nn/mnist.cml:39-40 (tensor-core, few-column and tiny shapes; odd lengths)."""
    rng = np.random.default_rng(55)
    for k, m, n in ((512, 784, 64), (300, 200, 10), (37, 5, 3), (1000, 130, 257)):
        a = T.from_numpy(rng.uniform(-1, 1, (k, m)).astype(np.float32))
        b = T.from_numpy(rng.uniform(-1, 1, (k, n)).astype(np.float32))
        got = T.matmul_tn(a, b).numpy()
        ref = T.matmul(T.transpose(a), b).numpy()
        T.check_async()
        assert got.shape == (m, n) and got.tobytes() == ref.tobytes()
    for count in (100003, 4096, 5):
        w = rng.uniform(-1, 1, count).astype(np.float32)
        g = rng.uniform(-3, 3, count).astype(np.float32)
        lr = 0.01 / 512
        got = T.scaled_sub(T.from_numpy(w), T.from_numpy(g), lr).numpy()
        chain = T.subtract(T.from_numpy(w), T.multiply(T.from_numpy(g), lr)).numpy()
        T.check_async()
        host = w - (g.astype(np.float64) * lr).astype(np.float32)
        assert got.tobytes() == chain.tobytes() == host.tobytes()


@pytest.mark.parametrize("k,m,n", [
    (2048, 785, 10), (60000, 785, 10), (5000, 33, 1), (31, 1000, 2), (4097, 129, 9), (700, 12544, 10),
    (1500, 300, 16), (999, 257, 17), (640, 64, 24), (333, 100, 25), (20000, 40, 32), (1, 7, 3),
])
def test_matmul_tn_few_columns(T, k, m, n):
    """transpose(X) @ G with n <= 32 (the gradient of a classifier, mnist.cml:39) reads X in place:
    float64 products and sums as in the reference, so the float32 result is the correctly rounded
    one except where the summation order moves a float64 sum across a rounding boundary."""
    rng = np.random.default_rng(k + m + n)
    a = rng.uniform(-1, 1, (k, m)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    got = T.matmul_tn(T.from_numpy(a), T.from_numpy(b)).numpy()
    T.check_async()
    ref = (a.T.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
    assert got.shape == (m, n)
    d = ulp_distance(got, ref)
    assert d.max() <= 1 and np.mean(d == 0) >= 0.999, (int(d.max()), float(np.mean(d == 0)))
    if k * m * n <= 3_000_000:  # the restatement itself, k ascending (operators.cpp:757-766)
        port = oracle.port().matmul(np.ascontiguousarray(a.T), b)
        assert np.mean(got == port) >= 0.999 and ulp_distance(got, port).max() <= 1


def test_matmul_with_one_inner_element_is_exact(T):
    """k == 1: one product per output, rounded once - bit-exact, also for wide outputs, where
    larger k goes to the split-precision tensor-core kernel.  The reference's programs broadcast
    a column with it (`v @ ones([1, k])`, mnist.cml:18)."""
    rng = np.random.default_rng(3)
    for m, n in ((64, 5000), (4096, 1000), (300, 33), (7, 130), (1000, 8)):
        v = (rng.standard_normal((m, 1)) * 100).astype(np.float32)
        v[0, 0] = -0.0
        w = rng.standard_normal((1, n)).astype(np.float32)
        ones = np.ones((1, n), np.float32)
        assert T.matmul(T.from_numpy(v), T.from_numpy(ones)).numpy().tobytes() == (np.repeat(v, n, 1) + 0.0).tobytes()
        got = T.matmul(T.from_numpy(v), T.from_numpy(w)).numpy()
        ref = (0.0 + v.astype(np.float64) * w.astype(np.float64)).astype(np.float32)
        assert got.tobytes() == ref.tobytes()
    T.check_async()


def test_dlpack_zero_copy_with_torch(T):
    """Device tensors cross to torch and back through DLPack without a copy (same device pointer)."""
    import torch

    from camel_b200 import dlpack

    rng = np.random.default_rng(44)
    a = rng.uniform(-1, 1, (37, 19)).astype(np.float32)
    t = T.from_numpy(a)
    tt = torch.from_dlpack(t)
    assert tt.is_cuda and tt.data_ptr() == t.ptr and tuple(tt.shape) == (37, 19)
    assert np.array_equal(tt.cpu().numpy(), a)
    tt.mul_(2.0)  # the same memory: visible on our side
    torch.cuda.synchronize()
    assert np.array_equal(t.numpy(), a * 2)
    del tt

    src = torch.arange(12, dtype=torch.int64, device="cuda").reshape(3, 4)
    u = dlpack.from_dlpack(src)
    assert u.ptr == src.data_ptr() and u.shape == (3, 4)
    got = T.add(u, u).numpy()
    T.check_async()
    assert np.array_equal(got, 2 * np.arange(12).reshape(3, 4))
    with pytest.raises(ValueError, match="dense row-major"):
        dlpack.from_dlpack(src.t())
    with pytest.raises(ValueError, match="float32, int64"):
        dlpack.from_dlpack(torch.zeros(4, dtype=torch.float16, device="cuda"))
    mask = dlpack.from_dlpack(torch.tensor([True, False, True], device="cuda"))
    assert mask.dtype == 2 and mask.numpy().astype(np.uint8).tolist() == [1, 0, 1]


def test_dense_packed_weights(T):
    """The tensor-core layout of a weight tensor is built once and kept with the tensor: same bytes
    as the per-call pre-pass, in both precisions; a handle from another matrix is refused."""
    import ctypes as C

    import camel_b200
    from camel_b200._lib import check, lib

    rng = np.random.default_rng(21)
    x = T.from_numpy(rng.uniform(0, 1, (300, 200)).astype(np.float32))
    w_np = rng.uniform(-0.1, 0.1, (200, 150)).astype(np.float32)
    b = T.from_numpy(rng.uniform(-0.1, 0.1, 150).astype(np.float32))
    for prec in (camel_b200._lib.PREC_3XTF32, camel_b200._lib.PREC_BF16):
        check(lib.ct_set_precision(prec))
        try:
            T.set_weight_cache(False)
            plain = T.dense(x, T.from_numpy(w_np), b, "relu").numpy()
            T.set_weight_cache(True)
            w = T.from_numpy(w_np)
            first = T.dense(x, w, b, "relu").numpy()
            assert w._packed is not None and prec in w._packed
            second = T.dense(x, w, b, "relu").numpy()
            T.check_async()
            assert plain.tobytes() == first.tobytes() == second.tobytes()
            if prec == camel_b200._lib.PREC_3XTF32:
                w3x = w
        finally:
            check(lib.ct_set_precision(camel_b200._lib.PREC_3XTF32))
            T.set_weight_cache(True)
    other = T.from_numpy(w_np)
    out = T.Tensor(0, (300, 150))
    with pytest.raises(camel_b200.CamelTensorError, match="packed weights"):
        check(lib.ct_dense_packed(x.ptr, other.ptr, w3x._packed[camel_b200._lib.PREC_3XTF32], None, 300, 200, 150, 0,
                                  out.ptr, None))
    h = C.c_void_p()
    with pytest.raises(camel_b200.CamelTensorError):
        check(lib.ct_weights_pack(None, 4, 4, C.byref(h)))


def test_packed_rows_panels_on_two_streams(T):
    """A left operand split once (ct_rows_pack) and multiplied in row panels of uneven size,
    alternating between two streams, gives the bytes of the one-call product; the handle is reused
    for new contents without allocating; ranges outside the matrix and foreign handles are refused."""
    import ctypes as C

    import camel_b200
    from camel_b200._lib import check, lib

    rng = np.random.default_rng(77)
    m, k, n = 1100, 600, 2000  # enough tiles that the one-call product does not slice k (other summation order)
    w = T.from_numpy(rng.uniform(-1, 1, (k, n)).astype(np.float32))
    wp = C.c_void_p()
    check(lib.ct_weights_pack(w.ptr, k, n, C.byref(wp)))
    ap = C.c_void_p()
    streams = [C.c_void_p(), C.c_void_p()]
    for sh in streams:
        check(lib.ct_stream_create(C.byref(sh)))
    ev = C.c_void_p()
    check(lib.ct_event_create(C.byref(ev)))
    try:
        first_handle = None
        for seed in (1, 2):
            a_np = np.random.default_rng(seed).uniform(-1, 1, (m, k)).astype(np.float32)
            a = T.from_numpy(a_np)
            whole = T.matmul(a, w).numpy()
            check(lib.ct_rows_pack(a.ptr, m, k, C.byref(ap)))
            first_handle = first_handle or ap.value
            assert ap.value == first_handle  # refilled, not re-allocated
            check(lib.ct_event_record(ev))
            out = T.Tensor.empty((m, n)) if hasattr(T.Tensor, "empty") else T.from_numpy(np.zeros((m, n), np.float32))
            plan = [(0, 512), (512, 256), (768, 128), (896, 204)]
            for j, (off, rows) in enumerate(plan):
                check(lib.ct_set_stream(streams[j % 2]))
                check(lib.ct_stream_wait_event(ev))
                check(lib.ct_matmul_packed_rows(ap, off, rows, wp, out.ptr + off * n * 4))
            for sh in streams:  # the default stream waits for both lanes
                check(lib.ct_set_stream(sh))
                check(lib.ct_event_record(ev))
                check(lib.ct_set_stream(None))
                check(lib.ct_stream_wait_event(ev))
            got = out.numpy()
            T.check_async()
            assert got.tobytes() == whole.tobytes()
        with pytest.raises(camel_b200.CamelTensorError, match="row range"):
            check(lib.ct_matmul_packed_rows(ap, 1000, 200, wp, out.ptr))
        with pytest.raises(camel_b200.CamelTensorError, match="packed operand"):
            check(lib.ct_matmul_packed_rows(wp, 0, 10, wp, out.ptr))
        small = T.from_numpy(np.zeros((4, 4), np.float32))
        with pytest.raises(camel_b200.CamelTensorError, match="another shape"):
            check(lib.ct_rows_pack(small.ptr, 4, 4, C.byref(ap)))
    finally:
        check(lib.ct_set_stream(None))
        T.sync()
        check(lib.ct_rows_free(ap))
        check(lib.ct_weights_free(wp))
        check(lib.ct_event_destroy(ev))
        for sh in streams:
            check(lib.ct_stream_destroy(sh))


def test_host_pipeline_streams_batches(T):
    """Seven host batches through a depth-2 pipeline (copy in, recorded forward, copy out on three
    streams): every batch's results equal the call-by-call run on the same bytes, in order."""
    from camel_b200 import pipeline
    from camel_b200._lib import F32

    rng = np.random.default_rng(9)
    w1 = T.from_numpy(rng.uniform(-0.2, 0.2, (96, 160)).astype(np.float32))
    b1 = T.from_numpy(rng.uniform(-0.1, 0.1, 160).astype(np.float32))
    w2 = T.from_numpy(rng.uniform(-0.2, 0.2, (160, 10)).astype(np.float32))

    def forward(inp):
        h = T.dense(inp, w1, b1, "relu")
        return T.dense(h, w2, None, "softmax", with_argmax=True)

    pipe = pipeline.HostPipeline(forward, F32, (300, 96), depth=2)
    ins = [pipeline.pinned_array((300, 96), np.float32) for _ in range(7)]
    for buf in ins:
        buf.array[...] = rng.uniform(0, 1, (300, 96)).astype(np.float32)
    outs = [(pipeline.pinned_array((300, 10), np.float32), pipeline.pinned_array((300,), np.int64)) for _ in range(7)]
    ms = pipe.run([b.ptr for b in ins], [(p.ptr, a.ptr) for p, a in outs])
    assert ms > 0.0
    for buf, (p, a) in zip(ins, outs):
        probs_e, arg_e = forward(T.from_numpy(buf.array.copy()))
        assert p.array.tobytes() == probs_e.numpy().tobytes()
        assert a.array.tobytes() == arg_e.numpy().tobytes()
    T.check_async()
    pipe.close()


def test_full_size_gemm_checksum_16384(T):
    """BASELINE configs[4] at full size (16384^3, U(-1,1), seed 5): the scalar oracle would need days,
    so the product is checked through a property that holds at any size, (A B) 1 = A (B 1), plus 64
    entries recomputed in float64 on the host."""
    import torch

    n = 16384
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    a = torch.rand((n, n), generator=g, device="cuda", dtype=torch.float32) * 2 - 1
    b = torch.rand((n, n), generator=g, device="cuda", dtype=torch.float32) * 2 - 1
    ta, tb = T.wrap_device(a.data_ptr(), 0, (n, n), keep=a), T.wrap_device(b.data_ptr(), 0, (n, n), keep=b)
    c = T.matmul(ta, tb)
    T.check_async()
    ct = torch.from_dlpack(c)
    ones = torch.ones((n, 1), device="cuda", dtype=torch.float64)
    lhs = ct.double() @ ones
    rhs = a.double() @ (b.double() @ ones)
    scale = float((a.double().abs() @ (b.double().abs() @ ones)).max())
    assert float((lhs - rhs).abs().max()) / scale <= 1e-6
    rng = np.random.default_rng(0)
    rows, cols = rng.integers(0, n, 64), rng.integers(0, n, 64)
    for i, j in zip(rows.tolist(), cols.tolist()):
        ref = float((a[i].double() * b[:, j].double()).sum())
        bound = float((a[i].double().abs() * b[:, j].double().abs()).sum())
        assert abs(float(ct[i, j]) - ref) <= 1e-5 * bound


def test_full_size_mlp_rows_are_independent(T):
    """BASELINE configs[1] at full size (batch 4096): rows 0..255 and the last 256 rows agree with
    the same rows run as their own small batches (a row's tile neighbours do not enter its sum;
    the small batch takes other tile shapes and a k-sliced schedule, so sums differ in order, not
    in value beyond the contraction tolerance), and the first rows equal the oracle."""
    rng = np.random.default_rng(1)

    def kaiming(fan_in, fan_out):
        lim = np.sqrt(6.0 / fan_in)
        return rng.uniform(-lim, lim, (fan_in, fan_out)).astype(np.float32)

    w = [kaiming(784, 1024), kaiming(1024, 1024), kaiming(1024, 10)]
    b = [np.zeros(1024, np.float32), np.zeros(1024, np.float32), np.zeros(10, np.float32)]
    x = np.random.default_rng(2).uniform(0, 1, (4096, 784)).astype(np.float32)
    tw, tb = [T.from_numpy(v) for v in w], [T.from_numpy(v) for v in b]

    def forward(inp):
        h = T.dense(inp, tw[0], tb[0], "relu")
        h = T.dense(h, tw[1], tb[1], "relu")
        probs, arg = T.dense(h, tw[2], tb[2], "softmax", with_argmax=True)
        return probs.numpy(), arg.numpy()

    probs, arg = forward(T.from_numpy(x))
    T.check_async()
    assert probs.shape == (4096, 10) and arg.shape == (4096,)
    assert np.all(np.abs(probs.sum(axis=1) - 1.0) <= 1e-5)
    assert np.array_equal(arg, probs.argmax(axis=1)) or np.mean(arg == probs.argmax(axis=1)) > 0.999
    for sl in (slice(0, 256), slice(4096 - 256, 4096)):
        p_small, a_small = forward(T.from_numpy(x[sl]))
        assert np.max(np.abs(p_small - probs[sl])) <= 2e-6
        top2 = np.sort(probs[sl], axis=1)[:, -2:]
        decided = top2[:, 1] - top2[:, 0] > 1e-5
        assert np.array_equal(a_small[decided], arg[sl][decided])
    p = oracle.port()
    h = p.dense(x[:64], w[0], b[0], 1)
    h = p.dense(h, w[1], b[1], 1)
    ref = p.softmax_rows(p.dense(h, w[2], b[2], 0))
    assert np.max(np.abs(probs[:64] - ref)) <= 1e-5


def test_full_size_conv_linearity(T):
    """BASELINE configs[2] geometry at full batch (256 x 64 x 56 x 56 -> 128): conv is linear in its
    input, conv(x1 + x2) = conv(x1) + conv(x2) without bias, within the contraction tolerance, and a
    2-image slice equals the oracle."""
    import torch

    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    x1 = torch.randn((256, 64, 56, 56), generator=g, device="cuda", dtype=torch.float32)
    x2 = torch.randn((256, 64, 56, 56), generator=g, device="cuda", dtype=torch.float32)
    wt = (torch.randn((128, 64, 3, 3), generator=g, device="cuda", dtype=torch.float32) * (2.0 / 576) ** 0.5)
    wrap = lambda t: T.wrap_device(t.data_ptr(), 0, tuple(t.shape), keep=t)  # noqa: E731
    tw = wrap(wt)
    xs = x1 + x2
    ys = torch.from_dlpack(T.conv2d(wrap(xs), tw, None, 1, 1, None))
    y1 = torch.from_dlpack(T.conv2d(wrap(x1), tw, None, 1, 1, None))
    y2 = torch.from_dlpack(T.conv2d(wrap(x2), tw, None, 1, 1, None))
    T.check_async()
    err = float((ys - (y1 + y2)).abs().max()) / float(ys.abs().max())
    assert err <= 3e-5
    ref = oracle.port().conv2d(x1[:2].cpu().numpy(), wt.cpu().numpy(), np.zeros(128, np.float32), 1, 1, 0)
    got = y1[:2].cpu().numpy()
    assert np.max(np.abs(got - ref)) / np.max(np.abs(ref)) <= 1e-5


def test_gemm_bf16_mode_long_k(T):
    """bf16-in / float32-accumulate at a long reduction (k = 16384, the k of BASELINE configs[4]),
    against float64: the stated tolerance of that mode, 1e-2 of the largest entry, and the
    component-wise error against sum |a||b| (bf16 rounding of both operands: 2^-8 each)."""
    import camel_b200
    from camel_b200 import _lib

    rng = np.random.default_rng(61)
    m, k, n = 1024, 16384, 1024
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    _lib.check(camel_b200.lib.ct_set_precision(_lib.PREC_BF16))
    try:
        got = T.matmul(T.from_numpy(a), T.from_numpy(b)).numpy()
        T.check_async()
    finally:
        _lib.check(camel_b200.lib.ct_set_precision(_lib.PREC_3XTF32))
    ref = a.astype(np.float64) @ b.astype(np.float64)
    err = float(np.max(np.abs(got - ref)) / np.max(np.abs(ref)))
    comp = float(np.max(np.abs(got - ref) / (np.abs(a).astype(np.float64) @ np.abs(b))))
    print(f"bf16 {m}x{k}x{n}: max|d|/max|ref|={err:.3e} componentwise={comp:.3e}")
    assert err <= 1e-2
    assert comp <= 2.0 ** -7


def test_kernel_timeout_is_reported_once_and_sticks_until_checked(T):
    """The error path of a bounded in-kernel wait, exercised from the host: the timeout word is
    written as a kernel would write it (ct_inject_status; nothing on the GPU waits).  While it is
    set, contraction kernels return at once without writing; calls enqueued after it do not erase
    it; ct_check reports it exactly once with the block that gave up; afterwards products are
    correct again."""
    import time

    import camel_b200
    from camel_b200._lib import ERR_TIMEOUT, check, lib

    rng = np.random.default_rng(62)
    a_np = rng.uniform(-1, 1, (512, 512)).astype(np.float32)
    b_np = rng.uniform(-1, 1, (512, 512)).astype(np.float32)
    a, b = T.from_numpy(a_np), T.from_numpy(b_np)
    good = T.matmul(a, b).numpy()
    T.check_async()

    out = T.Tensor(0, (512, 512))
    check(lib.ct_fill(0, 7.0, 512 * 512, out.ptr))
    check(lib.ct_inject_status(2, 42))  # as if block 41 of an earlier launch had given up
    t0 = time.perf_counter()
    check(lib.ct_matmul(0, a.ptr, 0, b.ptr, 512, 512, 512, out.ptr))   # enqueued after the failure
    check(lib.ct_matmul(0, a.ptr, 0, b.ptr, 512, 512, 512, out.ptr))   # a second one does not clear it
    elementwise = T.add(a, b).numpy()                                  # other operators are unaffected
    assert time.perf_counter() - t0 < 1.0, "the launches must return at once, not wait out a budget"
    assert np.array_equal(out.numpy(), np.full((512, 512), 7.0, np.float32))
    assert np.array_equal(elementwise, a_np + b_np)
    assert lib.ct_check() == ERR_TIMEOUT
    assert "block 41" in lib.ct_last_error().decode()
    assert lib.ct_check() == 0  # reported once, then clear
    with pytest.raises(camel_b200.CamelTensorError):
        check(lib.ct_inject_status(99, 1))
    check(lib.ct_matmul(0, a.ptr, 0, b.ptr, 512, 512, 512, out.ptr))
    assert out.numpy().tobytes() == good.tobytes()
    T.check_async()
    # the host-buffer form reports it by itself
    check(lib.ct_inject_status(2, 3))
    host_out = np.zeros((512, 512), np.float32)
    rc = lib.ct_matmul_host(a_np.ctypes.data, b_np.ctypes.data, 512, 512, 512, host_out.ctypes.data)
    assert rc == ERR_TIMEOUT and "block 2" in lib.ct_last_error().decode()
    assert lib.ct_check() == 0


def test_tensor_pipe_peak_measurement(T):
    """ct_measure_mma_peak: back-to-back kind::tf32 MMAs on resident operands.  The rate has to lie
    above what the GEMM kernel already reaches (3 x 200 TFLOP/s, a power-capped device included) and the nominal 1.2 PFLOP/s."""
    import ctypes as C

    from camel_b200._lib import PREC_3XTF32, PREC_BF16, check, lib

    tf, ms = C.c_double(), C.c_double()
    check(lib.ct_measure_mma_peak(PREC_3XTF32, 800, 1, C.byref(tf), C.byref(ms)))
    print(f"tf32 MMA burst: {tf.value:.1f} TFLOP/s in {ms.value * 1e3:.1f} us")
    assert 600.0 <= tf.value <= 1250.0   # nominal 1.1-1.2 PFLOP/s dense; the launch's set-up is inside
    check(lib.ct_measure_mma_peak(PREC_BF16, 800, 1, C.byref(tf), C.byref(ms)))
    print(f"bf16 MMA burst: {tf.value:.1f} TFLOP/s in {ms.value * 1e3:.1f} us")
    assert 1200.0 <= tf.value <= 2500.0  # nominal 2.25 PFLOP/s dense
    # the same pipe in SM cycles (stamps inside the kernel): a 128 x 256 x 8 tf32 MMA needs 128 cycles at
    # the nominal 8192 flop per cycle and SM; and the clock those cycles were counted at
    cpm, mhz = C.c_double(), C.c_double()
    check(lib.ct_measure_mma_clocks(PREC_3XTF32, 128, 256, C.byref(cpm), C.byref(mhz)))
    print(f"tf32 128x256x8: {cpm.value:.1f} SM cycles per MMA at {mhz.value:.0f} MHz")
    assert 120.0 <= cpm.value <= 200.0
    assert 700.0 <= mhz.value <= 2100.0


def test_packed_bands_one_launch_with_completion_counters(T):
    """All row bands of a product in one launch (ct_matmul_packed_bands): the bytes of the band-by-band
    calls, bands written to separate places, every band's counter ends at its tile count, and a second
    stream that waits for a band's count (ct_stream_wait_value) sees the finished band."""
    import ctypes as C

    import camel_b200
    from camel_b200._lib import check, lib

    rng = np.random.default_rng(81)
    m, k, n = 1152, 640, 2304   # 9 row tiles x 9 column tiles of 256
    a = T.from_numpy(rng.uniform(-1, 1, (m, k)).astype(np.float32))
    w = T.from_numpy(rng.uniform(-1, 1, (k, n)).astype(np.float32))
    wp, ap = C.c_void_p(), C.c_void_p()
    check(lib.ct_weights_pack(w.ptr, k, n, C.byref(wp)))
    check(lib.ct_rows_pack(a.ptr, m, k, C.byref(ap)))
    side = C.c_void_p()
    check(lib.ct_stream_create(C.byref(side)))
    ev = C.c_void_p()
    check(lib.ct_event_create(C.byref(ev)))
    try:
        whole = T.Tensor(0, (m, n))
        check(lib.ct_matmul_packed_rows(ap, 0, m, wp, whole.ptr))
        want = whole.numpy()
        bands = [512, 256, 384]                      # all but the last a multiple of 128 rows
        # the bands land in reverse order in a larger buffer, with a gap between them
        out = T.Tensor(0, (m + 64, n))
        check(lib.ct_fill(0, -7.0, (m + 64) * n, out.ptr))
        starts = [m + 64 - 512, m + 64 - 512 - 32 - 256, 0]
        rows_arr = (C.c_int64 * 3)(*bands)
        outs_arr = (C.c_void_p * 3)(*[out.ptr + s0 * n * 4 for s0 in starts])
        import torch

        # the counters must come from cudaMalloc (torch's allocator): a stream wait does not accept
        # memory of the stream-ordered pool that ct_alloc draws from
        done_t = torch.zeros(8, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()

        class _Done:
            ptr = done_t.data_ptr()

            @staticmethod
            def numpy():
                return done_t.cpu().numpy()

        done = _Done()
        tiles = (C.c_uint32 * 3)()
        check(lib.ct_event_record(ev))               # the counters are clear from here on
        check(lib.ct_matmul_packed_bands(ap, wp, 3, rows_arr, outs_arr, done.ptr, tiles))
        assert list(tiles) == [4 * 9, 2 * 9, 3 * 9]
        # a second stream takes a copy of band 1 as soon as its count is reached
        copy = T.Tensor(0, (256, n))
        check(lib.ct_set_stream(side))
        check(lib.ct_stream_wait_event(ev))
        check(lib.ct_stream_wait_value(done.ptr + 4, tiles[1]))
        check(lib.ct_d2d(copy.ptr, out.ptr + starts[1] * n * 4, 256 * n * 4))
        check(lib.ct_sync())
        check(lib.ct_set_stream(None))
        got = out.numpy()
        T.check_async()
        counts = done.numpy().view(np.uint32)[:3]
        assert counts.tolist() == list(tiles)
        row = 0
        for rows, s0 in zip(bands, starts):
            assert got[s0:s0 + rows].tobytes() == want[row:row + rows].tobytes()
            row += rows
        assert copy.numpy().tobytes() == want[512:768].tobytes()
        assert np.all(got[starts[1] + 256:starts[0]] == -7.0)  # the gap between the bands is untouched
        with pytest.raises(camel_b200.CamelTensorError, match="multiple of 128"):
            bad = (C.c_int64 * 2)(100, m - 100)
            check(lib.ct_matmul_packed_bands(ap, wp, 2, bad, outs_arr, done.ptr, tiles))
        with pytest.raises(camel_b200.CamelTensorError, match="rows"):
            short = (C.c_int64 * 2)(512, 256)
            check(lib.ct_matmul_packed_bands(ap, wp, 2, short, outs_arr, done.ptr, tiles))
    finally:
        check(lib.ct_set_stream(None))
        T.sync()
        check(lib.ct_rows_free(ap))
        check(lib.ct_weights_free(wp))
        check(lib.ct_event_destroy(ev))
        check(lib.ct_stream_destroy(side))


@pytest.mark.parametrize("nbytes", [(32 << 20) - 4, 32 << 20, (33 << 20) + 12, (100 << 20) + 4])
def test_large_copies_from_ordinary_host_memory(T, nbytes):
    """ct_h2d from pageable memory: sources of 32 MiB and more are staged through the library's ring of
    page-locked buffers by several host threads (one below the limit takes the plain path; one longer
    than the 16 MiB ring makes slots come round again).  Every byte has to arrive, twice in a row."""
    from camel_b200._lib import check, lib

    n = nbytes // 4
    rng = np.random.default_rng(nbytes)
    t = T.Tensor(0, (n,))
    for _ in range(2):
        src = rng.random(n, dtype=np.float32)
        check(lib.ct_h2d(t.ptr, src.ctypes.data, n * 4))
        back = t.numpy()
        assert back.tobytes() == src.tobytes()
