/* TEST INFRASTRUCTURE, not product code.
 *
 * Plain-C restatement of the arithmetic of the reference tensor module (OpenCML/Camel,
 * modules/tensor).  Only tests, the smoke check and the bench's CPU-baseline leg may load it;
 * the GPU library never does.
 *
 * Pinning: every function that restates an existing reference operator is compared bit for bit
 * with the reference's own compiled code (oracle/_ref, built by the Makefile here) in
 * tests/test_oracle.py, and with the fixtures under tests/golden/ that were produced by that
 * compiled reference.  The operators that the reference does not have (relu, softmax, dense,
 * conv2d, maxpool2d) are pinned, bit for bit as well, by compositions of reference operators run
 * on the compiled reference (tests/cases.py, RefBackend): relu, softmax and dense by the .cml
 * idioms that define them; conv2d by one reference matmul per image over the gathered input
 * windows with the bias as the last term (the dense idiom); maxpool2d by the reference's
 * max(axis 0) over the gathered window elements.  In those two the gather is data movement
 * outside the reference; every arithmetic step is the reference's.
 *
 * The reference's convention, used by every function below: read each element as double
 * (TensorObject::getAsDouble, modules/tensor/runtime.cpp:298-310), compute in double, round
 * once into the output dtype (setFromDouble, runtime.cpp:340-355).
 *
 * dtype codes: 0 = float32, 1 = int64, 2 = bool stored as uint8.
 * Functions return 0 on success or a positive code naming the exception the reference throws:
 *   1 "Division by zero" (runtime.cpp:122-124), 2 "log: input must be positive"
 *   (runtime.cpp:1039-1041), 3 unsupported dtype for the operator.
 * Loops over independent output elements may run under OpenMP; the order of operations inside
 * one output element is always the reference's.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

enum { CTO_F32 = 0, CTO_I64 = 1, CTO_BOOL = 2 };
enum { CTO_ADD = 0, CTO_SUB = 1, CTO_MUL = 2, CTO_DIV = 3, CTO_POW = 4 };
enum { CTO_LT = 0, CTO_LE = 1, CTO_GT = 2, CTO_GE = 3, CTO_EQ = 4 };

/* runtime.cpp:298-310 */
static inline double get_d(int dtype, const void *p, uint64_t i) {
    switch (dtype) {
    case CTO_F32:
        return (double)((const float *)p)[i];
    case CTO_I64:
        return (double)((const int64_t *)p)[i];
    default:
        return ((const uint8_t *)p)[i] != 0 ? 1.0 : 0.0;
    }
}

/* runtime.cpp:340-355 */
static inline void set_d(int dtype, void *p, uint64_t i, double v) {
    switch (dtype) {
    case CTO_F32:
        ((float *)p)[i] = (float)v;
        break;
    case CTO_I64:
        ((int64_t *)p)[i] = (int64_t)v;
        break;
    default:
        ((uint8_t *)p)[i] = v != 0.0 ? 1 : 0;
        break;
    }
}

/* runtime.cpp:570-580, and the Divide/Power override at runtime.cpp:781-784 */
int cto_result_dtype(int op, int lhs, int rhs) {
    if (op == CTO_DIV || op == CTO_POW)
        return CTO_F32;
    if (lhs == CTO_F32 || rhs == CTO_F32)
        return CTO_F32;
    if (lhs == CTO_I64 || rhs == CTO_I64)
        return CTO_I64;
    return CTO_BOOL;
}

/* runtime.cpp:113-130; *err is set when the reference would throw. */
static inline double apply_binary(int op, double a, double b, int *err) {
    switch (op) {
    case CTO_ADD:
        return a + b;
    case CTO_SUB:
        return a - b;
    case CTO_MUL:
        return a * b;
    case CTO_DIV:
        if (b == 0.0) {
            *err = 1;
            return 0.0;
        }
        return a / b;
    default:
        return pow(a, b);
    }
}

/* runtime.cpp:132-146 */
static inline int apply_compare(int op, double a, double b) {
    switch (op) {
    case CTO_LT:
        return a < b;
    case CTO_LE:
        return a <= b;
    case CTO_GT:
        return a > b;
    case CTO_GE:
        return a >= b;
    default:
        return a == b;
    }
}

/* tensorBinary, runtime.cpp:775-793.  out has dtype cto_result_dtype(op, ldt, rdt). */
int cto_binary(int op, int ldt, const void *lhs, int rdt, const void *rhs, uint64_t n, void *out) {
    int odt = cto_result_dtype(op, ldt, rdt), err = 0;
    for (uint64_t i = 0; i < n; ++i) {
        set_d(odt, out, i, apply_binary(op, get_d(ldt, lhs, i), get_d(rdt, rhs, i), &err));
        if (err)
            return 1; /* the reference throws at the first zero divisor */
    }
    return 0;
}

/* tensorBinaryScalarRight / ScalarLeft, runtime.cpp:795-831.  sdt is the tensor dtype the
 * scalar's type normalises to (Float32/Float64 -> 0, Int32/Int64 -> 1, Bool -> 2); the scalar
 * value itself enters as double (scalarToDouble, runtime.cpp:62-77). */
int cto_binary_scalar(
    int op, int tdt, const void *t, double scalar, int sdt, int scalar_on_left, uint64_t n,
    void *out) {
    int odt = scalar_on_left ? cto_result_dtype(op, sdt, tdt) : cto_result_dtype(op, tdt, sdt);
    int err = 0;
    for (uint64_t i = 0; i < n; ++i) {
        double v = get_d(tdt, t, i);
        double r = scalar_on_left ? apply_binary(op, scalar, v, &err)
                                  : apply_binary(op, v, scalar, &err);
        if (err)
            return 1;
        set_d(odt, out, i, r);
    }
    return 0;
}

/* tensorCompare, runtime.cpp:863-877: Bool (uint8) output. */
int cto_compare(
    int op, int ldt, const void *lhs, int rdt, const void *rhs, uint64_t n, uint8_t *out) {
    for (uint64_t i = 0; i < n; ++i)
        out[i] = (uint8_t)apply_compare(op, get_d(ldt, lhs, i), get_d(rdt, rhs, i));
    return 0;
}

/* tensorCompareScalarRight / ScalarLeft, runtime.cpp:833-861. */
int cto_compare_scalar(
    int op, int tdt, const void *t, double scalar, int scalar_on_left, uint64_t n, uint8_t *out) {
    for (uint64_t i = 0; i < n; ++i) {
        double v = get_d(tdt, t, i);
        out[i]   = (uint8_t)(scalar_on_left ? apply_compare(op, scalar, v)
                                            : apply_compare(op, v, scalar));
    }
    return 0;
}

/* tensorSum, runtime.cpp:879-885: sequential double sum. */
double cto_sum(int dt, const void *t, uint64_t n) {
    double v = 0.0;
    for (uint64_t i = 0; i < n; ++i)
        v += get_d(dt, t, i);
    return v;
}

/* tensorSumAxis, runtime.cpp:887-922: rank 2, double accumulate, float32 out. */
int cto_sum_axis(int dt, const void *t, int64_t rows, int64_t cols, int axis, float *out) {
    if (axis == 0) {
        for (int64_t j = 0; j < cols; ++j) {
            double acc = 0.0;
            for (int64_t i = 0; i < rows; ++i)
                acc += get_d(dt, t, (uint64_t)(i * cols + j));
            out[j] = (float)acc;
        }
    } else {
        for (int64_t i = 0; i < rows; ++i) {
            double acc = 0.0;
            for (int64_t j = 0; j < cols; ++j)
                acc += get_d(dt, t, (uint64_t)(i * cols + j));
            out[i] = (float)acc;
        }
    }
    return 0;
}

/* tensorMaxAxis, runtime.cpp:924-963: strict '>' against the first element. */
int cto_max_axis(int dt, const void *t, int64_t rows, int64_t cols, int axis, float *out) {
    if (axis == 0) {
        for (int64_t j = 0; j < cols; ++j) {
            double best = get_d(dt, t, (uint64_t)j);
            for (int64_t i = 1; i < rows; ++i) {
                double v = get_d(dt, t, (uint64_t)(i * cols + j));
                if (v > best)
                    best = v;
            }
            out[j] = (float)best;
        }
    } else {
        for (int64_t i = 0; i < rows; ++i) {
            double best = get_d(dt, t, (uint64_t)(i * cols));
            for (int64_t j = 1; j < cols; ++j) {
                double v = get_d(dt, t, (uint64_t)(i * cols + j));
                if (v > best)
                    best = v;
            }
            out[i] = (float)best;
        }
    }
    return 0;
}

/* tensorArgmaxAxis, runtime.cpp:965-1011: first maximum wins, Int64 out. */
int cto_argmax_axis(int dt, const void *t, int64_t rows, int64_t cols, int axis, int64_t *out) {
    if (axis == 0) {
        for (int64_t j = 0; j < cols; ++j) {
            int64_t idx = 0;
            double best = get_d(dt, t, (uint64_t)j);
            for (int64_t i = 1; i < rows; ++i) {
                double v = get_d(dt, t, (uint64_t)(i * cols + j));
                if (v > best) {
                    best = v;
                    idx  = i;
                }
            }
            out[j] = idx;
        }
    } else {
        for (int64_t i = 0; i < rows; ++i) {
            int64_t idx = 0;
            double best = get_d(dt, t, (uint64_t)(i * cols));
            for (int64_t j = 1; j < cols; ++j) {
                double v = get_d(dt, t, (uint64_t)(i * cols + j));
                if (v > best) {
                    best = v;
                    idx  = j;
                }
            }
            out[i] = idx;
        }
    }
    return 0;
}

/* tensorExp, runtime.cpp:1013-1027: float tensors only. */
int cto_exp(const float *t, uint64_t n, float *out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i)
        out[i] = (float)exp((double)t[i]);
    return 0;
}

/* tensorLog, runtime.cpp:1029-1045: throws on the first element <= 0. */
int cto_log(const float *t, uint64_t n, float *out) {
    for (uint64_t i = 0; i < n; ++i) {
        double v = (double)t[i];
        if (v <= 0.0)
            return 2;
        out[i] = (float)log(v);
    }
    return 0;
}

/* tensorTranspose2D, runtime.cpp:704-720 (values pass through double unchanged). */
int cto_transpose(int dt, const void *t, int64_t rows, int64_t cols, void *out) {
    for (int64_t i = 0; i < rows; ++i)
        for (int64_t j = 0; j < cols; ++j)
            set_d(dt, out, (uint64_t)(j * rows + i), get_d(dt, t, (uint64_t)(i * cols + j)));
    return 0;
}

/* tensorConcat, runtime.cpp:722-773, on the (outer, axis, inner) view of the shapes. */
int cto_concat(
    int dt, const void *lhs, const void *rhs, uint64_t outer, uint64_t lhs_axis,
    uint64_t rhs_axis, uint64_t inner, void *out) {
    size_t item = dt == CTO_F32 ? 4 : (dt == CTO_I64 ? 8 : 1);
    for (uint64_t o = 0; o < outer; ++o) {
        char *dst = (char *)out + o * (lhs_axis + rhs_axis) * inner * item;
        memcpy(dst, (const char *)lhs + o * lhs_axis * inner * item, lhs_axis * inner * item);
        memcpy(
            dst + lhs_axis * inner * item, (const char *)rhs + o * rhs_axis * inner * item,
            rhs_axis * inner * item);
    }
    return 0;
}

/* __tensor_matmul__, modules/tensor/operators.cpp:740-769: C[i,j] rounds
 * sum_k double(A[i,k]) * double(B[k,j]), k ascending, into promote(adt, bdt). */
int cto_matmul(
    int adt, const void *a, int bdt, const void *b, int64_t m, int64_t k, int64_t n, void *out) {
    int odt = cto_result_dtype(CTO_ADD, adt, bdt);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m; ++i) {
        for (int64_t j = 0; j < n; ++j) {
            double acc = 0.0;
            for (int64_t kk = 0; kk < k; ++kk)
                acc += get_d(adt, a, (uint64_t)(i * k + kk)) * get_d(bdt, b, (uint64_t)(kk * n + j));
            set_d(odt, out, (uint64_t)(i * n + j), acc);
        }
    }
    return 0;
}

/* ---- operators the reference does not have; defined by composition of the ones above ---- */

/* relu(x) := multiply(x, gt(x, 0)), the idiom of test/run/nn/svm.cml:31.  Bit pattern
 * included: negative x gives -0.0, NaN stays NaN, -inf gives NaN (-inf * 0). */
int cto_relu(const float *t, uint64_t n, float *out) {
    for (uint64_t i = 0; i < n; ++i) {
        double v    = (double)t[i];
        double mask = v > 0.0 ? 1.0 : 0.0;
        out[i]      = (float)(v * mask);
    }
    return 0;
}

/* softmax over rows := the ten-operator function of test/run/nn/mnist.cml:13-25:
 * m = max(x,1); s = x - m (broadcast through a matmul with ones, which is exact);
 * e = exp(s); d = sum(e,1); e / d.  Each step rounds to float32 as its operator does. */
int cto_softmax_rows(const float *x, int64_t rows, int64_t cols, float *out) {
    int rc = 0;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < rows; ++i) {
        const float *r = x + i * cols;
        float *o       = out + i * cols;
        double best    = (double)r[0];
        for (int64_t j = 1; j < cols; ++j)
            if ((double)r[j] > best)
                best = (double)r[j];
        float m    = (float)best;
        double acc = 0.0;
        for (int64_t j = 0; j < cols; ++j) {
            float st = (float)((double)r[j] - (double)m);
            float e  = (float)exp((double)st);
            o[j]     = e;
            acc += (double)e;
        }
        float d = (float)acc;
        if ((double)d == 0.0) {
            rc = 1;
            continue;
        }
        for (int64_t j = 0; j < cols; ++j)
            o[j] = (float)((double)o[j] / (double)d);
    }
    return rc;
}

/* dense<w,b>(x) := concat(x, ones, 1) @ concat(w, b_row, 0), the bias idiom of
 * test/run/nn/lr.cml:19-21: the bias is the last term of the double sum.  activation: 0 none,
 * 1 relu as defined above.  bias may be NULL (plain matmul). */
int cto_dense(
    const float *x, const float *w, const float *bias, int64_t m, int64_t k, int64_t n,
    int activation, float *out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m; ++i) {
        for (int64_t j = 0; j < n; ++j) {
            double acc = 0.0;
            for (int64_t kk = 0; kk < k; ++kk)
                acc += (double)x[i * k + kk] * (double)w[kk * n + j];
            if (bias)
                acc += 1.0 * (double)bias[j];
            float v = (float)acc;
            if (activation == 1) {
                double dv = (double)v;
                v         = (float)(dv * (dv > 0.0 ? 1.0 : 0.0));
            }
            out[i * n + j] = v;
        }
    }
    return 0;
}

/* conv2d, NCHW input, OIHW weights, zero padding, square stride.  No reference body exists; the
 * definition is the reference matmul (operators.cpp:757-766) over the gathered input windows:
 * one double accumulator per output, terms in (c, kh, kw) ascending order, padded taps skipped
 * (they would add w * 0.0), bias last, one rounding, optional relu as y * (y > 0). */
int cto_conv2d(
    const float *x, const float *w, const float *bias, int64_t n, int64_t c, int64_t h,
    int64_t wd, int64_t ko, int64_t kh, int64_t kw, int64_t stride, int64_t pad, int activation,
    float *out) {
    int64_t ho = (h + 2 * pad - kh) / stride + 1;
    int64_t wo = (wd + 2 * pad - kw) / stride + 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t in = 0; in < n; ++in) {
        for (int64_t o = 0; o < ko; ++o) {
            for (int64_t y = 0; y < ho; ++y) {
                for (int64_t xo = 0; xo < wo; ++xo) {
                    double acc = 0.0;
                    for (int64_t ic = 0; ic < c; ++ic)
                        for (int64_t r = 0; r < kh; ++r) {
                            int64_t iy = y * stride - pad + r;
                            if (iy < 0 || iy >= h)
                                continue;
                            for (int64_t s = 0; s < kw; ++s) {
                                int64_t ix = xo * stride - pad + s;
                                if (ix < 0 || ix >= wd)
                                    continue;
                                acc += (double)x[((in * c + ic) * h + iy) * wd + ix] *
                                       (double)w[((o * c + ic) * kh + r) * kw + s];
                            }
                        }
                    if (bias)
                        acc += 1.0 * (double)bias[o];
                    float v = (float)acc;
                    if (activation == 1) {
                        double dv = (double)v;
                        v         = (float)(dv * (dv > 0.0 ? 1.0 : 0.0));
                    }
                    out[((in * ko + o) * ho + y) * wo + xo] = v;
                }
            }
        }
    }
    return 0;
}

/* maxpool2d, NCHW, window == stride, no padding.  No reference body exists; the definition is
 * tensorMaxAxis (runtime.cpp:924-963) over the window's elements: starts from the first element
 * and replaces on strict '>' scanning rows then columns. */
int cto_maxpool2d(
    const float *x, int64_t n, int64_t c, int64_t h, int64_t wd, int64_t win, float *out) {
    int64_t ho = h / win, wo = wd / win;
#pragma omp parallel for schedule(static)
    for (int64_t p = 0; p < n * c; ++p) {
        const float *src = x + p * h * wd;
        float *dst       = out + p * ho * wo;
        for (int64_t y = 0; y < ho; ++y)
            for (int64_t xo = 0; xo < wo; ++xo) {
                double best = (double)src[(y * win) * wd + xo * win];
                for (int64_t r = 0; r < win; ++r)
                    for (int64_t s = 0; s < win; ++s) {
                        double v = (double)src[(y * win + r) * wd + xo * win + s];
                        if (v > best)
                            best = v;
                    }
                dst[y * wo + xo] = (float)best;
            }
    }
    return 0;
}

/* Constructors, runtime.cpp:614-690. */
int cto_full(int dt, double value, uint64_t n, void *out) {
    for (uint64_t i = 0; i < n; ++i)
        set_d(dt, out, i, value);
    return 0;
}

int cto_eye(int64_t size, float *out) {
    memset(out, 0, (size_t)(size * size) * sizeof(float));
    for (int64_t i = 0; i < size; ++i)
        out[i * size + i] = 1.0f;
    return 0;
}

/* tensorArange, runtime.cpp:652-673: returns the count; writes when out != NULL. */
int64_t cto_arange(int64_t start, int64_t stop, int64_t step, int64_t *out) {
    int64_t cnt = 0;
    if (step > 0) {
        for (int64_t v = start; v < stop; v += step, ++cnt)
            if (out)
                out[cnt] = v;
    } else if (step < 0) {
        for (int64_t v = start; v > stop; v += step, ++cnt)
            if (out)
                out[cnt] = v;
    }
    return cnt;
}
