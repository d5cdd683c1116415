/* TEST INFRASTRUCTURE. Prototype-only stand-in for OpenBLAS's <cblas.h>, which the reference's generated
 * C++ programs include (e.g. src/out/NIPS18evaluation/evaluationCNN/Lantern/Lantern.cpp) and which this
 * image does not have. Only the two routines and the enums those programs use are declared. */
#ifndef LANTERN_ORACLE_CBLAS_SHIM_H
#define LANTERN_ORACLE_CBLAS_SHIM_H
#ifdef __cplusplus
extern "C" {
#endif
enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };
void cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, enum CBLAS_TRANSPOSE tb, int M, int N, int K,
                 float alpha, const float* A, int lda, const float* B, int ldb, float beta, float* C, int ldc);
void cblas_sgemv(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, int M, int N, float alpha, const float* A, int lda,
                 const float* X, int incX, float beta, float* Y, int incY);
#ifdef __cplusplus
}
#endif
#endif
