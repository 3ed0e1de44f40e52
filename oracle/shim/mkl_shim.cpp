/*
 * Plain-loop implementations of the Intel MKL entry points named by the reference
 * (see mkl.h in this directory).  TEST INFRASTRUCTURE ONLY: the reference's CPU
 * tensor code is linked against this file to obtain an executable oracle and a
 * timed CPU baseline; the product library never links it.
 *
 * Semantics follow the published BLAS / Sparse BLAS / VML definitions:
 *   cblas_sgemm  : C = alpha*op(A)*op(B) + beta*C, row- or column-major
 *   mkl_scsrmm   : C = alpha*op(A)*B + beta*C with A in 4-array CSR; with
 *                  matdescra[3]=='C' (zero-based) B and C are row-major
 *   v?Exp etc.   : element-wise
 * Accumulation is single precision (for the s-variants), in ascending k / in the
 * stored order of a CSR row, one output element at a time.  MKL's own internal
 * summation order is unknown, which is why floating-point parity with the
 * reference is stated as a tolerance rather than bit equality.
 *
 * Threads: rows of C are split over OpenMP threads when s2v_shim_set_threads(n>1)
 * was called; each output element is still produced by one thread in the same
 * order, so results do not depend on the thread count.
 */
#include "mkl.h"

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

static int g_threads = 1;

extern "C" void s2v_shim_set_threads(int n)
{
    g_threads = n < 1 ? 1 : n;
}
extern "C" int s2v_shim_get_threads(void)
{
    return g_threads;
}

extern "C" void* mkl_malloc(size_t bytes, int alignment)
{
    size_t al = alignment < (int)sizeof(void*) ? sizeof(void*) : (size_t)alignment;
    void* p = nullptr;
    size_t padded = (bytes + al - 1) / al * al;
    if (padded == 0) padded = al;
    if (posix_memalign(&p, al, padded) != 0) return nullptr;
    return p;
}
extern "C" void mkl_free(void* p)
{
    free(p);
}

namespace
{

template <typename T>
T dot_(MKL_INT n, const T* x, MKL_INT incx, const T* y, MKL_INT incy)
{
    T s = 0;
    for (MKL_INT i = 0; i < n; ++i) s += x[(size_t)i * incx] * y[(size_t)i * incy];
    return s;
}

template <typename T>
CBLAS_INDEX iamax_(MKL_INT n, const T* x, MKL_INT incx)
{
    if (n <= 0) return 0;
    CBLAS_INDEX best = 0;
    T bv = std::fabs(x[0]);
    for (MKL_INT i = 1; i < n; ++i) {
        T v = std::fabs(x[(size_t)i * incx]);
        if (v > bv) { bv = v; best = (CBLAS_INDEX)i; }
    }
    return best;
}

template <typename T>
T asum_(MKL_INT n, const T* x, MKL_INT incx)
{
    T s = 0;
    for (MKL_INT i = 0; i < n; ++i) s += std::fabs(x[(size_t)i * incx]);
    return s;
}

template <typename T>
T nrm2_(MKL_INT n, const T* x, MKL_INT incx)
{
    T s = 0;
    for (MKL_INT i = 0; i < n; ++i) { T v = x[(size_t)i * incx]; s += v * v; }
    return std::sqrt(s);
}

template <typename T>
void axpby_(MKL_INT n, T a, const T* x, MKL_INT incx, T b, bool scale_y, T* y, MKL_INT incy)
{
    if (incx == 1 && incy == 1) {
        long nn = n;
#pragma omp parallel for num_threads(g_threads) if (g_threads > 1 && nn > (1 << 16)) schedule(static)
        for (long i = 0; i < nn; ++i) y[i] = scale_y ? a * x[i] + b * y[i] : a * x[i] + y[i];
        return;
    }
    for (MKL_INT i = 0; i < n; ++i) {
        T& yy = y[(size_t)i * incy];
        yy = scale_y ? a * x[(size_t)i * incx] + b * yy : a * x[(size_t)i * incx] + yy;
    }
}

template <typename T>
void ger_(CBLAS_LAYOUT layout, MKL_INT m, MKL_INT n, T alpha, const T* x, MKL_INT incx, const T* y, MKL_INT incy,
          T* a, MKL_INT lda)
{
    for (MKL_INT i = 0; i < m; ++i)
        for (MKL_INT j = 0; j < n; ++j) {
            size_t off = layout == CblasRowMajor ? (size_t)i * lda + j : (size_t)j * lda + i;
            a[off] += alpha * x[(size_t)i * incx] * y[(size_t)j * incy];
        }
}

template <typename T>
void gemv_(CBLAS_LAYOUT layout, CBLAS_TRANSPOSE trans, MKL_INT m, MKL_INT n, T alpha, const T* a, MKL_INT lda,
           const T* x, MKL_INT incx, T beta, T* y, MKL_INT incy)
{
    bool t = trans != CblasNoTrans;
    MKL_INT leny = t ? n : m, lenx = t ? m : n;
    for (MKL_INT i = 0; i < leny; ++i) {
        T s = 0;
        for (MKL_INT j = 0; j < lenx; ++j) {
            MKL_INT r = t ? j : i, c = t ? i : j;
            size_t off = layout == CblasRowMajor ? (size_t)r * lda + c : (size_t)c * lda + r;
            s += a[off] * x[(size_t)j * incx];
        }
        T& yy = y[(size_t)i * incy];
        yy = beta == (T)0 ? alpha * s : alpha * s + beta * yy;
    }
}

/* Row-major kernel; column-major is mapped onto it by the usual C^T = B^T A^T identity. */
template <typename T>
void gemm_rowmajor_(bool ta, bool tb, long m, long n, long k, T alpha, const T* a, long lda, const T* b, long ldb,
                    T beta, T* c, long ldc)
{
#pragma omp parallel num_threads(g_threads) if (g_threads > 1 && m * n * k > (1L << 18))
    {
        std::vector<T> acc((size_t)n);
#pragma omp for schedule(static)
        for (long i = 0; i < m; ++i) {
            T* accp = acc.data();
            for (long j = 0; j < n; ++j) accp[j] = 0;
            for (long p = 0; p < k; ++p) {
                const T av = ta ? a[p * lda + i] : a[i * lda + p];
                if (!tb) {
                    const T* brow = b + p * ldb;
                    for (long j = 0; j < n; ++j) accp[j] += av * brow[j];
                } else {
                    for (long j = 0; j < n; ++j) accp[j] += av * b[j * ldb + p];
                }
            }
            T* crow = c + i * ldc;
            if (beta == (T)0)
                for (long j = 0; j < n; ++j) crow[j] = alpha * accp[j];
            else
                for (long j = 0; j < n; ++j) crow[j] = alpha * accp[j] + beta * crow[j];
        }
    }
}

template <typename T>
void gemm_(CBLAS_LAYOUT layout, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, MKL_INT m, MKL_INT n, MKL_INT k, T alpha,
           const T* a, MKL_INT lda, const T* b, MKL_INT ldb, T beta, T* c, MKL_INT ldc)
{
    bool tA = ta != CblasNoTrans, tB = tb != CblasNoTrans;
    if (layout == CblasRowMajor)
        gemm_rowmajor_<T>(tA, tB, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
    else
        gemm_rowmajor_<T>(tB, tA, n, m, k, alpha, b, ldb, a, lda, beta, c, ldc);
}

template <typename T>
void omatadd_(char ordering, char transa, char transb, size_t m, size_t n, T alpha, const T* A, size_t lda, T beta,
              const T* B, size_t ldb, T* C, size_t ldc)
{
    bool row = ordering == 'R' || ordering == 'r';
    bool ta = !(transa == 'N' || transa == 'n'), tb = !(transb == 'N' || transb == 'n');
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j) {
            size_t ar = ta ? j : i, ac = ta ? i : j, br = tb ? j : i, bc = tb ? i : j;
            T av = row ? A[ar * lda + ac] : A[ac * lda + ar];
            T bv = row ? B[br * ldb + bc] : B[bc * ldb + br];
            (row ? C[i * ldc + j] : C[j * ldc + i]) = alpha * av + beta * bv;
        }
}

template <typename T>
void csrmm_(const char* transa, MKL_INT m, MKL_INT n, MKL_INT k, T alpha, const char* descr, const T* val,
            const MKL_INT* indx, const MKL_INT* pntrb, const MKL_INT* pntre, const T* b, MKL_INT ldb, T beta, T* c,
            MKL_INT ldc)
{
    const bool zero_based = descr[3] == 'C' || descr[3] == 'c';
    const MKL_INT base = zero_based ? 0 : 1;
    const bool trans = !(*transa == 'N' || *transa == 'n');
    /* zero-based indexing implies row-major dense operands, one-based implies column-major */
    auto B = [&](long r, long col) -> T { return zero_based ? b[r * (long)ldb + col] : b[col * (long)ldb + r]; };
    auto C = [&](long r, long col) -> T& { return zero_based ? c[r * (long)ldc + col] : c[col * (long)ldc + r]; };

    if (!trans) {
        if (zero_based) {
            const long mm = m, nn = n;
#pragma omp parallel num_threads(g_threads) if (g_threads > 1 && mm > 256)
            {
                std::vector<T> acc((size_t)nn);
#pragma omp for schedule(dynamic, 256)
                for (long i = 0; i < mm; ++i) {
                    T* accp = acc.data();
                    for (long j = 0; j < nn; ++j) accp[j] = 0;
                    for (MKL_INT t = pntrb[i] - base; t < pntre[i] - base; ++t) {
                        const T v = val[t];
                        const T* brow = b + (long)(indx[t] - base) * ldb;
                        for (long j = 0; j < nn; ++j) accp[j] += v * brow[j];
                    }
                    T* crow = c + i * (long)ldc;
                    if (beta == (T)0)
                        for (long j = 0; j < nn; ++j) crow[j] = alpha * accp[j];
                    else
                        for (long j = 0; j < nn; ++j) crow[j] = alpha * accp[j] + beta * crow[j];
                }
            }
            return;
        }
        for (long i = 0; i < m; ++i)
            for (long j = 0; j < n; ++j) {
                T s = 0;
                for (MKL_INT t = pntrb[i] - base; t < pntre[i] - base; ++t) s += val[t] * B(indx[t] - base, j);
                T& cc = C(i, j);
                cc = beta == (T)0 ? alpha * s : alpha * s + beta * cc;
            }
        return;
    }
    /* op(A) = A^T : A is m x k, C is k x n; scatter form, serial */
    for (long i = 0; i < k; ++i)
        for (long j = 0; j < n; ++j) {
            T& cc = C(i, j);
            cc = beta == (T)0 ? (T)0 : beta * cc;
        }
    for (long r = 0; r < m; ++r)
        for (MKL_INT t = pntrb[r] - base; t < pntre[r] - base; ++t) {
            long col = indx[t] - base;
            for (long j = 0; j < n; ++j) C(col, j) += alpha * val[t] * B(r, j);
        }
}

}  // namespace

extern "C" {

float cblas_sdot(MKL_INT n, const float* x, MKL_INT ix, const float* y, MKL_INT iy) { return dot_(n, x, ix, y, iy); }
double cblas_ddot(MKL_INT n, const double* x, MKL_INT ix, const double* y, MKL_INT iy) { return dot_(n, x, ix, y, iy); }
CBLAS_INDEX cblas_isamax(MKL_INT n, const float* x, MKL_INT ix) { return iamax_(n, x, ix); }
CBLAS_INDEX cblas_idamax(MKL_INT n, const double* x, MKL_INT ix) { return iamax_(n, x, ix); }
float cblas_sasum(MKL_INT n, const float* x, MKL_INT ix) { return asum_(n, x, ix); }
double cblas_dasum(MKL_INT n, const double* x, MKL_INT ix) { return asum_(n, x, ix); }
float cblas_snrm2(MKL_INT n, const float* x, MKL_INT ix) { return nrm2_(n, x, ix); }
double cblas_dnrm2(MKL_INT n, const double* x, MKL_INT ix) { return nrm2_(n, x, ix); }
void cblas_saxpy(MKL_INT n, float a, const float* x, MKL_INT ix, float* y, MKL_INT iy)
{
    axpby_<float>(n, a, x, ix, 1.f, false, y, iy);
}
void cblas_daxpy(MKL_INT n, double a, const double* x, MKL_INT ix, double* y, MKL_INT iy)
{
    axpby_<double>(n, a, x, ix, 1.0, false, y, iy);
}
void cblas_saxpby(MKL_INT n, float a, const float* x, MKL_INT ix, float b, float* y, MKL_INT iy)
{
    axpby_<float>(n, a, x, ix, b, true, y, iy);
}
void cblas_daxpby(MKL_INT n, double a, const double* x, MKL_INT ix, double b, double* y, MKL_INT iy)
{
    axpby_<double>(n, a, x, ix, b, true, y, iy);
}
void cblas_sger(CBLAS_LAYOUT l, MKL_INT m, MKL_INT n, float al, const float* x, MKL_INT ix, const float* y,
                MKL_INT iy, float* a, MKL_INT lda)
{
    ger_(l, m, n, al, x, ix, y, iy, a, lda);
}
void cblas_dger(CBLAS_LAYOUT l, MKL_INT m, MKL_INT n, double al, const double* x, MKL_INT ix, const double* y,
                MKL_INT iy, double* a, MKL_INT lda)
{
    ger_(l, m, n, al, x, ix, y, iy, a, lda);
}
void cblas_sgemv(CBLAS_LAYOUT l, CBLAS_TRANSPOSE t, MKL_INT m, MKL_INT n, float al, const float* a, MKL_INT lda,
                 const float* x, MKL_INT ix, float be, float* y, MKL_INT iy)
{
    gemv_(l, t, m, n, al, a, lda, x, ix, be, y, iy);
}
void cblas_dgemv(CBLAS_LAYOUT l, CBLAS_TRANSPOSE t, MKL_INT m, MKL_INT n, double al, const double* a, MKL_INT lda,
                 const double* x, MKL_INT ix, double be, double* y, MKL_INT iy)
{
    gemv_(l, t, m, n, al, a, lda, x, ix, be, y, iy);
}
void cblas_sgemm(CBLAS_LAYOUT l, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, MKL_INT m, MKL_INT n, MKL_INT k, float al,
                 const float* a, MKL_INT lda, const float* b, MKL_INT ldb, float be, float* c, MKL_INT ldc)
{
    gemm_(l, ta, tb, m, n, k, al, a, lda, b, ldb, be, c, ldc);
}
void cblas_dgemm(CBLAS_LAYOUT l, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, MKL_INT m, MKL_INT n, MKL_INT k, double al,
                 const double* a, MKL_INT lda, const double* b, MKL_INT ldb, double be, double* c, MKL_INT ldc)
{
    gemm_(l, ta, tb, m, n, k, al, a, lda, b, ldb, be, c, ldc);
}
void mkl_somatadd(char o, char ta, char tb, size_t m, size_t n, float al, const float* A, size_t lda, float be,
                  const float* B, size_t ldb, float* C, size_t ldc)
{
    omatadd_(o, ta, tb, m, n, al, A, lda, be, B, ldb, C, ldc);
}
void mkl_domatadd(char o, char ta, char tb, size_t m, size_t n, double al, const double* A, size_t lda, double be,
                  const double* B, size_t ldb, double* C, size_t ldc)
{
    omatadd_(o, ta, tb, m, n, al, A, lda, be, B, ldb, C, ldc);
}
void mkl_scsrmm(const char* ta, const MKL_INT* m, const MKL_INT* n, const MKL_INT* k, const float* al,
                const char* d, const float* val, const MKL_INT* indx, const MKL_INT* pb, const MKL_INT* pe,
                const float* b, const MKL_INT* ldb, const float* be, float* c, const MKL_INT* ldc)
{
    csrmm_(ta, *m, *n, *k, *al, d, val, indx, pb, pe, b, *ldb, *be, c, *ldc);
}
void mkl_dcsrmm(const char* ta, const MKL_INT* m, const MKL_INT* n, const MKL_INT* k, const double* al,
                const char* d, const double* val, const MKL_INT* indx, const MKL_INT* pb, const MKL_INT* pe,
                const double* b, const MKL_INT* ldb, const double* be, double* c, const MKL_INT* ldc)
{
    csrmm_(ta, *m, *n, *k, *al, d, val, indx, pb, pe, b, *ldb, *be, c, *ldc);
}

#define S2V_VML1(name, expr)                                                                     \
    void vs##name(MKL_INT n, const float* a, float* y) { for (MKL_INT i = 0; i < n; ++i) { float x = a[i]; y[i] = (expr); } } \
    void vd##name(MKL_INT n, const double* a, double* y) { for (MKL_INT i = 0; i < n; ++i) { double x = a[i]; y[i] = (expr); } }
S2V_VML1(Abs, std::fabs(x))
S2V_VML1(Sin, std::sin(x))
S2V_VML1(Cos, std::cos(x))
S2V_VML1(Exp, std::exp(x))
S2V_VML1(Ln, std::log(x))
S2V_VML1(Sqr, x * x)
S2V_VML1(Sqrt, std::sqrt(x))
S2V_VML1(InvSqrt, 1 / std::sqrt(x))
S2V_VML1(Inv, 1 / x)
#undef S2V_VML1
void vsMul(MKL_INT n, const float* a, const float* b, float* y) { for (MKL_INT i = 0; i < n; ++i) y[i] = a[i] * b[i]; }
void vdMul(MKL_INT n, const double* a, const double* b, double* y) { for (MKL_INT i = 0; i < n; ++i) y[i] = a[i] * b[i]; }
void vsDiv(MKL_INT n, const float* a, const float* b, float* y) { for (MKL_INT i = 0; i < n; ++i) y[i] = a[i] / b[i]; }
void vdDiv(MKL_INT n, const double* a, const double* b, double* y) { for (MKL_INT i = 0; i < n; ++i) y[i] = a[i] / b[i]; }
void vsPowx(MKL_INT n, const float* a, float b, float* y) { for (MKL_INT i = 0; i < n; ++i) y[i] = std::pow(a[i], b); }
void vdPowx(MKL_INT n, const double* a, double b, double* y) { for (MKL_INT i = 0; i < n; ++i) y[i] = std::pow(a[i], b); }

}  // extern "C"
