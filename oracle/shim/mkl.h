/*
 * Stand-in for Intel MKL's <mkl.h>, TEST INFRASTRUCTURE ONLY.
 *
 * The reference's CPU tensor layer calls Intel MKL (include/tensor/mkl_helper.h,
 * src/util/mem_holder.cpp:19,63).  MKL is a closed third-party dependency that is
 * not vendored with the reference and is not installed on the build machines, so
 * the reference's own C++ sources are compiled against this header instead.  It
 * declares exactly the entry points the reference names; mkl_shim.cpp implements
 * them from their published BLAS / Sparse BLAS / VML semantics with plain loops.
 *
 * Nothing in the product library includes or links this file.
 */
#ifndef S2V_ORACLE_MKL_SHIM_H
#define S2V_ORACLE_MKL_SHIM_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int MKL_INT;
typedef size_t CBLAS_INDEX;

typedef enum { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_LAYOUT;
typedef enum { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;

void* mkl_malloc(size_t bytes, int alignment);
void  mkl_free(void* p);

/* BLAS level 1 */
float  cblas_sdot(MKL_INT n, const float* x, MKL_INT incx, const float* y, MKL_INT incy);
double cblas_ddot(MKL_INT n, const double* x, MKL_INT incx, const double* y, MKL_INT incy);
CBLAS_INDEX cblas_isamax(MKL_INT n, const float* x, MKL_INT incx);
CBLAS_INDEX cblas_idamax(MKL_INT n, const double* x, MKL_INT incx);
float  cblas_sasum(MKL_INT n, const float* x, MKL_INT incx);
double cblas_dasum(MKL_INT n, const double* x, MKL_INT incx);
float  cblas_snrm2(MKL_INT n, const float* x, MKL_INT incx);
double cblas_dnrm2(MKL_INT n, const double* x, MKL_INT incx);
void cblas_saxpy(MKL_INT n, float a, const float* x, MKL_INT incx, float* y, MKL_INT incy);
void cblas_daxpy(MKL_INT n, double a, const double* x, MKL_INT incx, double* y, MKL_INT incy);
void cblas_saxpby(MKL_INT n, float a, const float* x, MKL_INT incx, float b, float* y, MKL_INT incy);
void cblas_daxpby(MKL_INT n, double a, const double* x, MKL_INT incx, double b, double* y, MKL_INT incy);

/* BLAS level 2 / 3 */
void cblas_sger(CBLAS_LAYOUT layout, MKL_INT m, MKL_INT n, float alpha, const float* x, MKL_INT incx,
                const float* y, MKL_INT incy, float* a, MKL_INT lda);
void cblas_dger(CBLAS_LAYOUT layout, MKL_INT m, MKL_INT n, double alpha, const double* x, MKL_INT incx,
                const double* y, MKL_INT incy, double* a, MKL_INT lda);
void cblas_sgemv(CBLAS_LAYOUT layout, CBLAS_TRANSPOSE trans, MKL_INT m, MKL_INT n, float alpha,
                 const float* a, MKL_INT lda, const float* x, MKL_INT incx, float beta, float* y, MKL_INT incy);
void cblas_dgemv(CBLAS_LAYOUT layout, CBLAS_TRANSPOSE trans, MKL_INT m, MKL_INT n, double alpha,
                 const double* a, MKL_INT lda, const double* x, MKL_INT incx, double beta, double* y, MKL_INT incy);
void cblas_sgemm(CBLAS_LAYOUT layout, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, MKL_INT m, MKL_INT n, MKL_INT k,
                 float alpha, const float* a, MKL_INT lda, const float* b, MKL_INT ldb,
                 float beta, float* c, MKL_INT ldc);
void cblas_dgemm(CBLAS_LAYOUT layout, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, MKL_INT m, MKL_INT n, MKL_INT k,
                 double alpha, const double* a, MKL_INT lda, const double* b, MKL_INT ldb,
                 double beta, double* c, MKL_INT ldc);

/* out-of-place matrix add: C = alpha*op(A) + beta*op(B) */
void mkl_somatadd(char ordering, char transa, char transb, size_t m, size_t n, float alpha, const float* A,
                  size_t lda, float beta, const float* B, size_t ldb, float* C, size_t ldc);
void mkl_domatadd(char ordering, char transa, char transb, size_t m, size_t n, double alpha, const double* A,
                  size_t lda, double beta, const double* B, size_t ldb, double* C, size_t ldc);

/* Sparse BLAS: C = alpha*op(A)*B + beta*C, A in 4-array CSR (val, indx, pntrb, pntre) */
void mkl_scsrmm(const char* transa, const MKL_INT* m, const MKL_INT* n, const MKL_INT* k, const float* alpha,
                const char* matdescra, const float* val, const MKL_INT* indx, const MKL_INT* pntrb,
                const MKL_INT* pntre, const float* b, const MKL_INT* ldb, const float* beta, float* c,
                const MKL_INT* ldc);
void mkl_dcsrmm(const char* transa, const MKL_INT* m, const MKL_INT* n, const MKL_INT* k, const double* alpha,
                const char* matdescra, const double* val, const MKL_INT* indx, const MKL_INT* pntrb,
                const MKL_INT* pntre, const double* b, const MKL_INT* ldb, const double* beta, double* c,
                const MKL_INT* ldc);

/* VML element-wise math: y[i] = f(a[i]) */
#define S2V_VML_DECL1(name) \
    void vs##name(MKL_INT n, const float* a, float* y); \
    void vd##name(MKL_INT n, const double* a, double* y);
#define S2V_VML_DECL2(name) \
    void vs##name(MKL_INT n, const float* a, const float* b, float* y); \
    void vd##name(MKL_INT n, const double* a, const double* b, double* y);
S2V_VML_DECL1(Abs) S2V_VML_DECL1(Sin) S2V_VML_DECL1(Cos) S2V_VML_DECL1(Exp) S2V_VML_DECL1(Ln)
S2V_VML_DECL1(Sqr) S2V_VML_DECL1(Sqrt) S2V_VML_DECL1(InvSqrt) S2V_VML_DECL1(Inv)
S2V_VML_DECL2(Mul) S2V_VML_DECL2(Div)
void vsPowx(MKL_INT n, const float* a, float b, float* y);
void vdPowx(MKL_INT n, const double* a, double b, double* y);
#undef S2V_VML_DECL1
#undef S2V_VML_DECL2

/* shim control (not part of MKL): number of OpenMP threads the shim may use, 1 = serial */
void s2v_shim_set_threads(int n);
int  s2v_shim_get_threads(void);

#ifdef __cplusplus
}
#endif
#endif
