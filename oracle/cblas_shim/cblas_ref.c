/* TEST INFRASTRUCTURE. Straightforward row-major sgemm/sgemv with the BLAS contract, so that the reference's
 * generated programs link without OpenBLAS. Loop order i-k-j keeps the inner loop unit-stride. */
#include "cblas.h"
#include <stdlib.h>

void cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, enum CBLAS_TRANSPOSE tb, int M, int N, int K,
                 float alpha, const float* A, int lda, const float* B, int ldb, float beta, float* C, int ldc) {
  if (order != CblasRowMajor) abort();
  for (int i = 0; i < M; ++i) {
    float* c = C + (size_t)i * ldc;
    if (beta == 0.0f) for (int j = 0; j < N; ++j) c[j] = 0.0f;
    else if (beta != 1.0f) for (int j = 0; j < N; ++j) c[j] *= beta;
    if (tb == CblasNoTrans) {
      for (int k = 0; k < K; ++k) {
        float a = alpha * (ta == CblasNoTrans ? A[(size_t)i * lda + k] : A[(size_t)k * lda + i]);
        const float* b = B + (size_t)k * ldb;
        for (int j = 0; j < N; ++j) c[j] += a * b[j];
      }
    } else {
      for (int j = 0; j < N; ++j) {
        const float* b = B + (size_t)j * ldb;
        float s = 0.0f;
        if (ta == CblasNoTrans) { const float* a = A + (size_t)i * lda; for (int k = 0; k < K; ++k) s += a[k] * b[k]; }
        else for (int k = 0; k < K; ++k) s += A[(size_t)k * lda + i] * b[k];
        c[j] += alpha * s;
      }
    }
  }
}

void cblas_sgemv(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, int M, int N, float alpha, const float* A, int lda,
                 const float* X, int incX, float beta, float* Y, int incY) {
  if (order != CblasRowMajor) abort();
  if (ta == CblasNoTrans) {
    for (int i = 0; i < M; ++i) {
      float s = 0.0f;
      for (int j = 0; j < N; ++j) s += A[(size_t)i * lda + j] * X[(size_t)j * incX];
      Y[(size_t)i * incY] = alpha * s + (beta == 0.0f ? 0.0f : beta * Y[(size_t)i * incY]);
    }
  } else {
    for (int j = 0; j < N; ++j) {
      float s = 0.0f;
      for (int i = 0; i < M; ++i) s += A[(size_t)i * lda + j] * X[(size_t)i * incX];
      Y[(size_t)j * incY] = alpha * s + (beta == 0.0f ? 0.0f : beta * Y[(size_t)j * incY]);
    }
  }
}
