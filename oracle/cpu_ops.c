/*
 * CPU restatement of the loop nests DaCeML's "pure" expansions lower to, for the timed CPU baseline.
 *
 * TEST / BASELINE INFRASTRUCTURE ONLY: nothing in the product path links or loads this file.
 *
 * DaCe turns each pure expansion into OpenMP C++: one parallel loop nest per ONNX node, with the
 * tensor written back to memory between nodes (daceml/onnx/op_implementations/utils.py:43-102,
 * daceml/util/utils.py:205-235).  The functions below are those loop nests written by hand:
 *   conv2d_nchw      daceml/onnx/op_implementations/img_op_implementations.py:263-288 (7-deep nest,
 *                    parallel over (b, m, y, x), sequential (c, i, j) reduction), generalised with
 *                    stride / pad / group indexing as in the MaxPool expansion (:19-21)
 *   softmax_rows     pure_implementations.py:309-319 (max, exp, sum, divide as four passes)
 *   log_softmax_rows pure_implementations.py:649-656
 *   reduce_mean_rows pure_implementations.py:101-103
 *   ew_*             pure_implementations.py:24-108, 556-568, 741-743 (one pass per node)
 * GEMMs are not here: the reference hands them to a BLAS library node (OpenBLAS / MKL), and the
 * baseline does the same through the host BLAS.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* Sets the size of the OpenMP team the loop nests below use.  A launcher may export OMP_NUM_THREADS=1 for its worker
 * processes (torch.distributed.run does); the timed baseline asks for the host cores it is allowed to run on. */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void conv2d_nchw(const float* x, const float* w, const float* bias, float* y, int64_t n, int64_t c, int64_t h,
                 int64_t wd, int64_t m, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t pt, int64_t pl,
                 int64_t pb, int64_t pr, int64_t group) {
    const int64_t oh = (h + pt + pb - kh) / sh + 1, ow = (wd + pl + pr - kw) / sw + 1;
    const int64_t cg = c / group, mg = m / group;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < n; ++b)
        for (int64_t mm = 0; mm < m; ++mm) {
            const int64_t g = mm / mg;
            for (int64_t oy = 0; oy < oh; ++oy)
                for (int64_t ox = 0; ox < ow; ++ox) {
                    float acc = bias ? bias[mm] : 0.0f;
                    for (int64_t ci = 0; ci < cg; ++ci)
                        for (int64_t i = 0; i < kh; ++i) {
                            const int64_t iy = oy * sh - pt + i;
                            if (iy < 0 || iy >= h) continue;
                            for (int64_t j = 0; j < kw; ++j) {
                                const int64_t ix = ox * sw - pl + j;
                                if (ix < 0 || ix >= wd) continue;
                                acc += w[((mm * cg + ci) * kh + i) * kw + j] * x[((b * c + g * cg + ci) * h + iy) * wd + ix];
                            }
                        }
                    y[((b * m + mm) * oh + oy) * ow + ox] = acc;
                }
        }
}

void softmax_rows(const float* x, float* y, int64_t rows, int64_t cols, int is_log) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        float* yr = y + r * cols;
        float mx = xr[0];
        for (int64_t i = 1; i < cols; ++i) mx = xr[i] > mx ? xr[i] : mx;
        float sum = 0.0f;
        for (int64_t i = 0; i < cols; ++i) {
            yr[i] = expf(xr[i] - mx);
            sum += yr[i];
        }
        if (is_log) {
            const float ls = logf(sum);
            for (int64_t i = 0; i < cols; ++i) yr[i] = xr[i] - mx - ls;
        } else {
            for (int64_t i = 0; i < cols; ++i) yr[i] = yr[i] / sum;
        }
    }
}

void reduce_mean_rows(const float* x, float* y, int64_t rows, int64_t cols) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float s = 0.0f;
        for (int64_t i = 0; i < cols; ++i) s += x[r * cols + i];
        y[r] = s / (float)cols;
    }
}

/* y[r, i] = op(a[r, i], b) with b broadcast per row (mode 1), per column (mode 2), scalar (mode 3) or full (mode 0) */
void ew_binary(const float* a, const float* b, float* y, int64_t rows, int64_t cols, int op, int mode) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t i = 0; i < cols; ++i) {
            const float av = a[r * cols + i];
            const float bv = mode == 0 ? b[r * cols + i] : (mode == 1 ? b[r] : (mode == 2 ? b[i] : b[0]));
            float o;
            switch (op) {
                case 0: o = av + bv; break;
                case 1: o = av - bv; break;
                case 2: o = av * bv; break;
                case 3: o = av / bv; break;
                default: o = powf(av, bv); break;
            }
            y[r * cols + i] = o;
        }
}

/* op: 0 erf, 1 sqrt, 2 relu, 3 sigmoid, 4 exp, 5 tanh */
void ew_unary(const float* x, float* y, int64_t n, int op) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const float v = x[i];
        float o;
        switch (op) {
            case 0: o = erff(v); break;
            case 1: o = sqrtf(v); break;
            case 2: o = v > 0.0f ? v : 0.0f; break;
            case 3: o = 1.0f / (1.0f + expf(-v)); break;
            case 4: o = expf(v); break;
            default: o = tanhf(v); break;
        }
        y[i] = o;
    }
}

/* out[perm] = in: 4-D permutation, one pass (pure_implementations.py:322-326) */
void transpose4d(const float* x, float* y, const int64_t* shape, const int64_t* perm) {
    int64_t istr[4], oshape[4];
    istr[3] = 1;
    for (int d = 2; d >= 0; --d) istr[d] = istr[d + 1] * shape[d + 1];
    for (int d = 0; d < 4; ++d) oshape[d] = shape[perm[d]];
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t a = 0; a < oshape[0]; ++a)
        for (int64_t b = 0; b < oshape[1]; ++b)
            for (int64_t c = 0; c < oshape[2]; ++c)
                for (int64_t d = 0; d < oshape[3]; ++d)
                    y[((a * oshape[1] + b) * oshape[2] + c) * oshape[3] + d] =
                        x[a * istr[perm[0]] + b * istr[perm[1]] + c * istr[perm[2]] + d * istr[perm[3]]];
}
