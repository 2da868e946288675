"""Seeded parity cases shared by the CPU and GPU tests and by the golden-vector generator.

A case is (name, fn) where fn(be) runs a few operator calls on backend `be` and returns a list
of numpy arrays / floats.  Backends expose one small API (see `PortBackend`) over
 - the compiled reference (oracle.ref, via its operator_t entry points),
 - the C restatement (oracle.port),
 - the CUDA library (camel_b200.tensor), defined in tests/test_gpu_parity.py.
Inputs come from numpy's PCG64 with a fixed seed per case, so every backend sees the same bytes.
"""
from __future__ import annotations

import numpy as np

import oracle
from oracle import IntArray

BIN = ["add", "subtract", "multiply", "divide", "pow"]
CMP = ["lt", "le", "gt", "ge", "eq"]


class PortBackend:
    name = "port"

    def __init__(self):
        self.p = oracle.port()

    def binary(self, op, a, b):
        return self.p.binary(BIN.index(op), a, b)

    def compare(self, op, a, b):
        return self.p.compare(CMP.index(op), a, b)

    def sum(self, a):
        return self.p.sum(a)

    def sum_axis(self, a, ax):
        return self.p.sum_axis(a, ax)

    def max_axis(self, a, ax):
        return self.p.max_axis(a, ax)

    def argmax_axis(self, a, ax):
        return self.p.argmax_axis(a, ax)

    def exp(self, a):
        return self.p.exp(a)

    def log(self, a):
        return self.p.log(a)

    def transpose(self, a):
        return self.p.transpose(a)

    def concat(self, a, b, ax):
        return self.p.concat(a, b, ax)

    def reshape(self, a, shape):
        return np.ascontiguousarray(oracle.norm(a)[0].reshape(shape))

    def matmul(self, a, b):
        return self.p.matmul(a, b)

    def relu(self, a):
        return self.p.relu(a)

    def softmax(self, a):
        return self.p.softmax_rows(a)

    def dense(self, x, w, b, act):
        return self.p.dense(x, w, b, {"none": 0, "relu": 1}[act])

    def conv2d(self, x, w, b, stride, pad, act):
        return self.p.conv2d(x, w, b, stride, pad, {"none": 0, "relu": 1}[act])

    def maxpool2d(self, x, win):
        return self.p.maxpool2d(x, win)

    def ones(self, shape):
        return self.p.full(oracle.F32, 1.0, tuple(shape))

    def zeros(self, shape):
        return self.p.full(oracle.F32, 0.0, tuple(shape))

    def full(self, shape, v):
        return self.p.full(oracle.scalar_dtype(v), v, tuple(shape))  # dtype follows the value's type

    def eye(self, n):
        return self.p.eye(n)

    def range(self, start, stop, step):
        return self.p.arange(start, stop, step)


def conv_patches(x, kh, kw, stride, pad):
    """Pure data movement (no arithmetic): the zero-padded input windows of one convolution as a
    matrix per image, [n][c*kh*kw][ho*wo], rows in (c, kh, kw) ascending order."""
    n, c, h, w = x.shape
    ho, wo = (h + 2 * pad - kh) // stride + 1, (w + 2 * pad - kw) // stride + 1
    xp = np.zeros((n, c, h + 2 * pad, w + 2 * pad), np.float32)
    xp[:, :, pad:pad + h, pad:pad + w] = x
    out = np.empty((n, c, kh, kw, ho, wo), np.float32)
    for r in range(kh):
        for s in range(kw):
            out[:, :, r, s] = xp[:, :, r:r + stride * (ho - 1) + 1:stride, s:s + stride * (wo - 1) + 1:stride]
    return out.reshape(n, c * kh * kw, ho * wo), ho, wo


def pool_windows(x, win):
    """Pure data movement: the win x win windows of a max-pool as [win*win][n*c*ho*wo], rows in the
    window's scan order (rows, then columns)."""
    n, c, h, w = x.shape
    ho, wo = h // win, w // win
    v = x[:, :, :ho * win, :wo * win].reshape(n, c, ho, win, wo, win)
    return np.ascontiguousarray(v.transpose(3, 5, 0, 1, 2, 4)).reshape(win * win, n * c * ho * wo), ho, wo


class RefBackend:
    """The reference's own operators; relu / softmax / dense by the compositions that define
    them (test/run/nn/svm.cml:31, mnist.cml:13-25, lr.cml:19-21); conv2d and maxpool2d by
    compositions in which every arithmetic step is a reference operator:

    conv2d   the input windows gathered into a patch matrix (movement only, numpy), then the dense
             idiom of lr.cml:19-21 per image - concat(W, bias column) @ concat(patches, ones row) -
             i.e. ONE reference matmul (operators.cpp:757-766: float64 sum over (c, kh, kw) ascending,
             the bias the last term, one rounding), relu as `y * (y > 0)`.  A padded tap enters
             the sum as w * 0.0, which leaves a float64 sum of finite terms unchanged.
    maxpool  the window elements gathered as the rows of a [win*win][outputs] matrix (movement
             only), then the reference's max(axis 0) (runtime.cpp:924-963: the first row seeds, a
             later row replaces on strict '>').
    """

    name = "ref"

    def __init__(self):
        self.r = oracle.ref()

    def binary(self, op, a, b):
        return self.r.call(op, a, b)

    def compare(self, op, a, b):
        return self.r.call(op, a, b)

    def sum(self, a):
        return self.r.call("sum", a)

    def sum_axis(self, a, ax):
        return self.r.call("sum_axis", a, ax)

    def max_axis(self, a, ax):
        return self.r.call("max_axis", a, ax)

    def argmax_axis(self, a, ax):
        return self.r.call("argmax_axis", a, ax)

    def exp(self, a):
        return self.r.call("exp", a)

    def log(self, a):
        return self.r.call("log", a)

    def transpose(self, a):
        return self.r.call("transpose", a)

    def concat(self, a, b, ax):
        return self.r.call("concat", a, b, ax)

    def reshape(self, a, shape):
        return self.r.call("reshape", a, IntArray(shape))

    def matmul(self, a, b):
        return self.r.call("matmul", a, b)

    def relu(self, a):
        return self.r.call("multiply", a, self.r.call("gt", a, 0))

    def softmax(self, x):
        r = self.r
        n, k = x.shape
        row_max = r.call("reshape", r.call("max_axis", x, 1), IntArray([n, 1]))
        stable = r.call("subtract", x, r.call("matmul", row_max, r.call("ones", IntArray([1, k]))))
        e = r.call("exp", stable)
        row_sum = r.call("reshape", r.call("sum_axis", e, 1), IntArray([n, 1]))
        return r.call("divide", e, r.call("matmul", row_sum, r.call("ones", IntArray([1, k]))))

    def dense(self, x, w, b, act):
        r = self.r
        if b is not None:
            xb = r.call("concat", x, r.call("ones", IntArray([x.shape[0], 1])), 1)
            wb = r.call("concat", w, np.asarray(b, np.float32).reshape(1, -1), 0)
            y = r.call("matmul", xb, wb)
        else:
            y = r.call("matmul", x, w)
        return self.relu(y) if act == "relu" else y

    def conv2d(self, x, w, b, stride, pad, act):
        r = self.r
        x, w = np.asarray(x, np.float32), np.asarray(w, np.float32)
        ko, c, kh, kw = w.shape
        patches, ho, wo = conv_patches(x, kh, kw, stride, pad)
        wm = w.reshape(ko, c * kh * kw)
        if b is not None:
            wm = r.call("concat", wm, np.asarray(b, np.float32).reshape(-1, 1), 1)
        if x.shape[0] == 0 or ho * wo == 0:
            return np.zeros((x.shape[0], ko, ho, wo), np.float32)
        outs = []
        for img in patches:
            pm = img
            if b is not None:
                pm = r.call("concat", img, r.call("ones", IntArray([1, img.shape[1]])), 0)
            y = r.call("matmul", wm, pm)
            outs.append(self.relu(y) if act == "relu" else y)
        return np.stack(outs).reshape(x.shape[0], ko, ho, wo)

    def maxpool2d(self, x, win):
        x = np.asarray(x, np.float32)
        rows, ho, wo = pool_windows(x, win)
        if rows.size == 0:
            return np.zeros((x.shape[0], x.shape[1], ho, wo), np.float32)
        return self.r.call("max_axis", rows, 0).reshape(x.shape[0], x.shape[1], ho, wo)

    def ones(self, shape):
        return self.r.call("ones", IntArray(shape))

    def zeros(self, shape):
        return self.r.call("zeros", IntArray(shape))

    def full(self, shape, v):
        return self.r.call("full", IntArray(shape), v)

    def eye(self, n):
        return self.r.call("eye", int(n))

    def range(self, start, stop, step):
        return self.r.call("range", int(start), int(stop), int(step))


def _f(rng, shape, lo=-1.0, hi=1.0):
    return rng.uniform(lo, hi, shape).astype(np.float32)


def _special(rng, shape):
    """Floats with signed zeros, infinities, NaN, denormals and huge/tiny magnitudes mixed in."""
    a = _f(rng, shape, -4, 4)
    flat = a.reshape(-1)
    specials = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-45, -1e-45, 3e38, -3e38, 1e-38, 1.0, -1.0],
                        dtype=np.float32)
    idx = rng.choice(flat.size, size=min(flat.size, 4 * specials.size), replace=False)
    flat[idx] = np.resize(specials, idx.size)
    return a


def build_cases():
    cases = []

    def case(name):
        def deco(fn):
            cases.append((name, fn))
            return fn
        return deco

    # -- elementwise, float32, ragged sizes (vector body + scalar tail, and an empty tensor)
    for n in (0, 1, 3, 4, 1023, 4099):
        @case(f"binary_f32_n{n}")
        def _(be, n=n):
            rng = np.random.default_rng(100 + n)
            a, b = _f(rng, (n,)), _f(rng, (n,))
            b_nz = np.where(b == 0, np.float32(0.5), b)
            outs = [be.binary("add", a, b), be.binary("subtract", a, b), be.binary("multiply", a, b),
                    be.binary("divide", a, b_nz), be.binary("pow", np.abs(a), b)]
            outs += [be.binary("add", a, 0.25), be.binary("subtract", 2, a), be.binary("multiply", a, True),
                     be.binary("divide", a, 3), be.binary("divide", 1.5, b_nz), be.binary("pow", np.abs(a), 2.0),
                     be.binary("multiply", a, 0.1)]
            return outs

    @case("binary_f32_special_values")
    def _(be):
        rng = np.random.default_rng(7)
        a, b = _special(rng, (33, 17)), _special(rng, (33, 17))
        b_nz = np.where(b == 0, np.float32(2.0), b)
        return [be.binary("add", a, b), be.binary("subtract", a, b), be.binary("multiply", a, b),
                be.binary("divide", a, b_nz), be.relu(a), be.compare("gt", a, 0), be.compare("eq", a, b),
                be.compare("le", a, b), be.binary("multiply", a, 0.0)]

    @case("binary_mixed_dtypes")
    def _(be):
        rng = np.random.default_rng(8)
        f = _f(rng, (19, 23), -3, 3)
        i = rng.integers(-7, 8, (19, 23))
        j = rng.integers(1, 5, (19, 23))
        bo = rng.integers(0, 2, (19, 23)).astype(np.uint8)
        outs = []
        for op in ("add", "subtract", "multiply"):
            outs += [be.binary(op, i, j), be.binary(op, i, bo), be.binary(op, bo, bo), be.binary(op, f, i),
                     be.binary(op, bo, f), be.binary(op, i, 3), be.binary(op, i, 0.5), be.binary(op, 2, bo),
                     be.binary(op, bo, True)]
        outs += [be.binary("divide", i, j), be.binary("divide", bo, j), be.binary("pow", j, 2),
                 be.binary("pow", j, bo), be.binary("divide", 7, j)]
        return outs

    @case("compare_all")
    def _(be):
        rng = np.random.default_rng(9)
        a, b = _f(rng, (41, 13)), _f(rng, (41, 13))
        b[::3] = a[::3]
        i = rng.integers(-3, 4, (41, 13))
        outs = []
        for op in CMP:
            outs += [be.compare(op, a, b), be.compare(op, a, 0.0), be.compare(op, 0.25, a),
                     be.compare(op, i, 1), be.compare(op, i, a), be.compare(op, 2, i)]
        return outs

    @case("unary_exp_log")
    def _(be):
        rng = np.random.default_rng(10)
        a = _f(rng, (5, 257), -20, 20)
        wide = np.array([-800, -104, -88.5, -87.3, 0.0, -0.0, 1e-30, 88.7, 89.0, 200, np.inf, -np.inf, np.nan],
                        dtype=np.float32)
        pos = np.abs(_f(rng, (1031,), -9, 9)) + np.float32(1e-30)
        tiny = np.array([1e-45, 1e-38, 1.0, 3e38, np.inf], dtype=np.float32)
        return [be.exp(a), be.exp(wide), be.log(pos), be.log(tiny), be.relu(a)]

    @case("sum_full")
    def _(be):
        rng = np.random.default_rng(11)
        outs = []
        for n in (0, 1, 5, 4096, 100003):
            outs.append(np.float64(be.sum(_f(rng, (n,)))))
        outs.append(np.float64(be.sum(rng.integers(-100, 100, (777,)))))
        outs.append(np.float64(be.sum(rng.integers(0, 2, (13, 11)).astype(np.uint8))))
        return outs

    for shape in ((1, 1), (7, 10), (64, 33), (3, 2500), (300, 5)):
        @case(f"axis_reduce_{shape[0]}x{shape[1]}")
        def _(be, shape=shape):
            rng = np.random.default_rng(12 + shape[0] * 31 + shape[1])
            a = _f(rng, shape)
            ties = np.round(a * 2) / 2  # many repeated maxima: first one must win
            i = rng.integers(-4, 5, shape)
            bo = rng.integers(0, 2, shape).astype(np.uint8)
            outs = []
            for ax in (0, 1, -1, -2):
                outs += [be.sum_axis(a, ax), be.max_axis(a, ax), be.argmax_axis(a, ax), be.argmax_axis(ties, ax),
                         be.sum_axis(i, ax), be.max_axis(i, ax), be.argmax_axis(i, ax), be.argmax_axis(bo, ax)]
            return outs

    @case("axis_reduce_nan")
    def _(be):
        rng = np.random.default_rng(13)
        a = _f(rng, (9, 70))
        a[0, 3] = np.nan   # NaN as the first element of column 3
        a[4, 0] = np.nan   # NaN as the first element of row 4
        a[2, 50] = np.nan  # NaN in the middle: never wins
        a[7, 69] = np.inf
        outs = []
        for ax in (0, 1):
            outs += [be.max_axis(a, ax), be.argmax_axis(a, ax)]
        return outs

    for shape in ((200, 132), (4100, 12), (70, 2052), (1000, 10), (513, 64), (66, 1028), (40000, 10)):
        @case(f"axis_reduce_wide_{shape[0]}x{shape[1]}")
        def _(be, shape=shape):
            # shapes of the vectorised float32 kernels: narrow rows staged in shared memory, a warp or
            # a block per row with 128-bit loads, columns cut into row slices; with the values that
            # decide the scan's semantics placed where slices, lanes and vectors meet
            rng = np.random.default_rng(40 + shape[0] + shape[1])
            a = np.round(_f(rng, shape, -3, 3) * 4) / 4      # many ties: the first maximum must win
            r, c = shape
            a[0, 1] = np.nan                                  # NaN seeds column 1 (axis 0) ...
            a[2, 0] = np.nan                                  # ... and row 2 (axis 1)
            a[r // 2, c // 2] = np.nan                        # a NaN that is no seed never wins
            a[:, 3] = -np.inf                                 # nothing exceeds the seed: index 0
            a[5, :] = -np.inf
            a[r - 1, 2] = np.inf
            a[7, c - 1] = np.inf
            a[1, 4], a[r - 2, 4] = 3.0, 3.0                   # equal maxima far apart
            a[6, 5], a[6, c - 2] = 3.0, 3.0
            a[0, 6], a[r - 1, 6] = -0.0, 0.0                  # +0 does not replace -0
            outs = []
            for ax in (0, 1):
                outs += [be.sum_axis(np.nan_to_num(a, nan=0.5, posinf=2.0, neginf=-2.0), ax), be.max_axis(a, ax),
                         be.argmax_axis(a, ax)]
            return outs

    @case("transpose_tiles")
    def _(be):
        rng = np.random.default_rng(41)
        return [be.transpose(_f(rng, shape)) for shape in ((64, 64), (128, 68), (4, 260), (132, 4), (200, 196), (60, 7))]

    @case("movement")
    def _(be):
        rng = np.random.default_rng(14)
        a, b = _f(rng, (37, 65)), _f(rng, (37, 65))
        c = _f(rng, (5, 65))
        i, j = rng.integers(-9, 9, (6, 3)), rng.integers(-9, 9, (6, 4))
        bo = rng.integers(0, 2, (33, 34)).astype(np.uint8)
        r3a, r3b = _f(rng, (3, 4, 5)), _f(rng, (3, 2, 5))
        return [be.transpose(a), be.transpose(i), be.transpose(bo), be.concat(a, b, 0), be.concat(a, b, 1),
                be.concat(a, c, 0), be.concat(i, j, 1), be.concat(r3a, r3b, 1), be.concat(bo, bo, 1),
                be.reshape(a, [65, 37]), be.reshape(r3a, [12, 5]), be.reshape(i, [18])]

    @case("constructors")
    def _(be):
        return [be.zeros([3, 5]), be.ones([2, 3, 4]), be.full([7], 2.5), be.full([2, 2], -1), be.full([3], True),
                be.eye(1), be.eye(9),
                be.range(0, 10, 1), be.range(2, 11, 3), be.range(10, 0, -3), be.range(5, 5, 1), be.zeros([0, 4])]

    # -- contractions: tolerance-checked on the GPU, bit-exact between the CPU checkers
    for (m, k, n) in ((1, 1, 1), (5, 7, 3), (33, 65, 10), (64, 64, 64), (128, 96, 160), (200, 300, 130),
                      (257, 129, 513)):
        @case(f"matmul_f32_{m}x{k}x{n}")
        def _(be, m=m, k=k, n=n):
            rng = np.random.default_rng(1000 + m + 7 * k + 13 * n)
            return [be.matmul(_f(rng, (m, k)), _f(rng, (k, n)))]

    @case("matmul_other_dtypes")
    def _(be):
        rng = np.random.default_rng(15)
        i, j = rng.integers(-5, 6, (17, 9)), rng.integers(-5, 6, (9, 21))
        bo = rng.integers(0, 2, (9, 21)).astype(np.uint8)
        f = _f(rng, (9, 21))
        return [be.matmul(i, j), be.matmul(i, bo), be.matmul(i, f), be.matmul(bo.T.copy(), f.reshape(9, 21)[:, :9].copy())]

    @case("softmax_rows")
    def _(be):
        rng = np.random.default_rng(16)
        outs = []
        for shape in ((1, 1), (4, 10), (33, 32), (9, 100), (5, 513), (3, 2049)):
            outs.append(be.softmax(_f(rng, shape, -6, 6)))
        big = _f(rng, (4, 10), -100, 100)  # widely spread logits: exp underflows to 0 for most
        outs.append(be.softmax(big))
        return outs

    @case("dense_layers")
    def _(be):
        rng = np.random.default_rng(17)
        outs = []
        for (m, k, n) in ((9, 20, 10), (130, 70, 200), (64, 128, 256)):
            x, w, b = _f(rng, (m, k), 0, 1), _f(rng, (k, n), -0.3, 0.3), _f(rng, (n,), -0.5, 0.5)
            outs += [be.dense(x, w, b, "none"), be.dense(x, w, b, "relu"), be.dense(x, w, None, "relu")]
        return outs

    # -- conv2d / maxpool2d: the reference has neither; its operators composed define them (see
    #    RefBackend).  Geometries of BASELINE configs 3 and 4 at small batch, plus ragged ones.
    conv_geoms = [
        # name,          n, c,  h,  w,  ko, kh, kw, stride, pad, act,   keep every k-th filter
        ("cfg3_geometry", 1, 64, 56, 56, 128, 3, 3, 1, 1, "relu", 8),
        ("cfg4_conv1", 3, 1, 28, 28, 32, 3, 3, 1, 1, "relu", 1),
        ("cfg4_conv2", 2, 32, 28, 28, 64, 3, 3, 1, 1, "relu", 1),
        ("stride2_5x5", 2, 16, 20, 20, 48, 5, 5, 2, 2, "none", 1),
        ("nopad_ragged", 2, 5, 9, 11, 7, 3, 2, 1, 0, "relu", 1),
        ("one_by_one", 1, 8, 6, 7, 4, 1, 1, 1, 0, "none", 1),
        ("empty_batch", 0, 3, 8, 8, 4, 3, 3, 1, 1, "relu", 1),
    ]
    for (gname, n, c, h, w, ko, kh, kw, stride, pad, act, keep) in conv_geoms:
        @case(f"conv2d_{gname}")
        def _(be, n=n, c=c, h=h, w=w, ko=ko, kh=kh, kw=kw, stride=stride, pad=pad, act=act, keep=keep):
            rng = np.random.default_rng(3000 + c * 7 + h + ko)
            x = rng.standard_normal((n, c, h, w)).astype(np.float32)
            wt = (rng.standard_normal((ko, c, kh, kw)) * np.sqrt(2.0 / (c * kh * kw))).astype(np.float32)
            b = rng.uniform(-0.1, 0.1, ko).astype(np.float32)
            # every output channel is an independent sum: the wide layer is checked on every keep-th filter
            wt, b = np.ascontiguousarray(wt[::keep]), np.ascontiguousarray(b[::keep])
            outs = [be.conv2d(x, wt, b, stride, pad, act)]
            if n and gname in ("cfg4_conv1", "nopad_ragged"):
                outs.append(be.conv2d(x, wt, None, stride, pad, "none"))
            return outs

    @case("maxpool2d_windows")
    def _(be):
        rng = np.random.default_rng(3100)
        outs = []
        for shape, win in (((2, 64, 28, 28), 2), ((2, 3, 9, 12), 3), ((1, 1, 7, 7), 2), ((2, 3, 10, 30), 2),
                           ((0, 2, 4, 4), 2)):
            x = rng.standard_normal(shape).astype(np.float32)
            if x.size:
                x[0, 0, 0, 0] = np.nan       # a NaN that opens a window stays
                x[-1, -1, 1, 1] = np.nan     # one that does not never wins
                x[0, 0, 2, 2:4] = (0.0, -0.0)  # among equal values the first one is kept
                x[0, 0, 3, 2:4] = (-1.0, -2.0)
            outs.append(be.maxpool2d(x, win))
        return outs

    return cases


CASES = build_cases()

# Cases whose outputs involve tensor-core contractions on the GPU (compared by tolerance there).
TOLERANCE_CASES = {name for name, _ in CASES if name.startswith(("matmul_f32", "dense_layers", "conv2d_"))}


# ---- the graph boundary: array literals in, host reads out ---------------------------------
#
# Calls that go through `backend.call(op, *args)` of oracle.Reference (the compiled reference, or
# the plugin's harness - same front end).  Each entry: (name, op, argument builder).  The golden
# file tests/golden/boundary.json holds what the compiled reference returned / printed.

def capture_stdout(fn):
    """Runs fn() and returns (its result, what the process wrote to file descriptor 1 meanwhile):
    `show` prints from C++."""
    import os
    import sys
    import tempfile

    sys.stdout.flush()
    saved = os.dup(1)
    with tempfile.TemporaryFile() as tmp:
        os.dup2(tmp.fileno(), 1)
        try:
            result = fn()
        finally:
            os.dup2(saved, 1)
            os.close(saved)
        tmp.seek(0)
        return result, tmp.read().decode()


def boundary_cases():
    from oracle import NestedArray

    lit = [[1.5, -2.0, 3.25], [4.0, 5.5, -0.0]]
    f = np.array([[1.5, -2.0, 3.0], [4.0, 5.5, 0.0]], np.float32)
    wide = (np.arange(40, dtype=np.float32).reshape(2, 20) - 7.5) * np.float32(1.0e3 / 3)
    cube = np.arange(24, dtype=np.float32).reshape(2, 3, 4) / 8
    return [
        # tensorFromArray (runtime.cpp:153-219, 1067-1077): dtype from the leaf type
        ("from_array_f64", "reshape", lambda: (NestedArray(lit, "f64"), IntArray([3, 2]))),
        ("from_array_f32", "reshape", lambda: (NestedArray(lit, "f32"), IntArray([6]))),
        ("from_array_i64", "reshape", lambda: (NestedArray([[1, 2], [3, 4], [5, 6]], "i64"), IntArray([2, 3]))),
        ("from_array_i32_rank3", "reshape", lambda: (NestedArray(np.arange(24).reshape(2, 3, 4), "i32"), IntArray([4, 6]))),
        ("from_array_bool", "reshape", lambda: (NestedArray([[1, 0, 1]], "bool"), IntArray([3]))),
        ("concat_arrays", "concat", lambda: (NestedArray(lit, "f64"), NestedArray([[7.0, 8.0, 9.0]], "f64"), 0)),
        # == with an array operand (operators.cpp:923-956)
        ("eq_tensor_array", "eq", lambda: (f, NestedArray(lit, "f64"))),
        ("eq_array_tensor", "eq", lambda: (NestedArray(lit, "f64"), f)),
        ("eq_array_scalar", "eq", lambda: (NestedArray([1, 2, 2, 3], "i64"), 2)),
        # host reads (runtime.cpp:1047-1065, 606-612)
        ("idx_1d", "idx", lambda: (np.array([0.5, 1.5, -2.5, 1e-3], np.float32), 2)),
        ("idx_1d_int", "idx", lambda: (np.arange(5) * 3, 4)),
        ("idx_2d", "idx2d", lambda: (f, 1, 2)),
        ("shape_rank3", "shape", lambda: (cube,)),
        # print (runtime.cpp:417-528): element formats, row wrapping at column 100, nesting
        ("show_f32", "show", lambda: (f,)),
        ("show_wrapped_rows", "show", lambda: (wide,)),
        ("show_rank3", "show", lambda: (cube,)),
        ("show_rank1_mixed", "show", lambda: (np.array([0.0, -0.0, 1e10, 12345.678, 1e-5, np.inf, np.nan, -1.0], np.float32),)),
        ("show_bool", "show", lambda: (np.array([[1, 0], [0, 1]], np.uint8),)),
        ("show_array_literal", "show", lambda: (NestedArray(lit, "f64"),)),
        ("show_empty", "show", lambda: (np.zeros((0, 3), np.float32),)),
    ]


def run_boundary_case(backend, op, build_args):
    """-> a JSON-able record of what the call returned and printed."""
    result, printed = capture_stdout(lambda: backend.call(op, *build_args()))
    if isinstance(result, np.ndarray):
        rec = {"dtype": str(result.dtype), "shape": list(result.shape), "hex": result.tobytes().hex()}
    else:
        rec = {"value": result}
    rec["printed"] = printed
    return rec
