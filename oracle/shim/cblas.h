/* Minimal CBLAS declarations for building the StreamBrain OpenMP kernel module
 * (BCPNN/backend/_kernels/kernels_openmp_internal.cc:2 includes <cblas.h>) on an
 * image that ships OpenBLAS only as a shared object inside a Python wheel.
 * Test infrastructure only: nothing in the product path includes this header.
 *
 * Only the two routines and two enums the StreamBrain forward pass uses are
 * declared (kernels_openmp_internal.cc:45-61).  When the library found is SciPy's
 * bundled OpenBLAS the symbols carry a `scipy_` prefix; -DSBB_CBLAS_SCIPY_PREFIX
 * maps the plain names onto them. */
#ifndef SBB_ORACLE_CBLAS_SHIM_H
#define SBB_ORACLE_CBLAS_SHIM_H

#ifdef SBB_CBLAS_SCIPY_PREFIX
#define cblas_sgemm scipy_cblas_sgemm
#define cblas_dgemm scipy_cblas_dgemm
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };

void cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, enum CBLAS_TRANSPOSE tb,
                 int m, int n, int k, float alpha, const float *a, int lda,
                 const float *b, int ldb, float beta, float *c, int ldc);
void cblas_dgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, enum CBLAS_TRANSPOSE tb,
                 int m, int n, int k, double alpha, const double *a, int lda,
                 const double *b, int ldb, double beta, double *c, int ldc);

#ifdef __cplusplus
}
#endif
#endif
