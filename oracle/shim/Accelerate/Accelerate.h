// TEST INFRASTRUCTURE ONLY. A stand-in for Apple's Accelerate umbrella header so
// that the reference's CPU QR (src/qr_cpu.mm) compiles unchanged on Linux against
// the OpenBLAS that ships inside the scipy wheel. Only the five symbols that file
// uses are mapped (src/qr_cpu.mm:54-56,79-117): sgeqrf_, sorgqr_, cblas_sgemm,
// vDSP_mtrans and the __LAPACK_int type.
#pragma once
#include <cstddef>

typedef int __LAPACK_int;

extern "C" {
void scipy_sgeqrf_(const int* m, const int* n, float* a, const int* lda, float* tau, float* work,
                   const int* lwork, int* info);
void scipy_sorgqr_(const int* m, const int* n, const int* k, float* a, const int* lda, const float* tau,
                   float* work, const int* lwork, int* info);
enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112 };
void scipy_cblas_sgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k,
                       float alpha, const float* a, int lda, const float* b, int ldb, float beta, float* c,
                       int ldc);
}

static inline void sgeqrf_(const int* m, const int* n, float* a, const int* lda, float* tau, float* work,
                           const int* lwork, int* info) {
    scipy_sgeqrf_(m, n, a, lda, tau, work, lwork, info);
}
static inline void sorgqr_(const int* m, const int* n, const int* k, float* a, const int* lda,
                           const float* tau, float* work, const int* lwork, int* info) {
    scipy_sorgqr_(m, n, k, a, lda, tau, work, lwork, info);
}
static inline void cblas_sgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k,
                               float alpha, const float* a, int lda, const float* b, int ldb, float beta,
                               float* c, int ldc) {
    scipy_cblas_sgemm(order, ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
}

// vDSP_mtrans(A, 1, C, 1, M, N): C (M x N) = transpose of A (N x M), both row-major.
static inline void vDSP_mtrans(const float* a, long, float* c, long, unsigned long m, unsigned long n) {
    for (unsigned long i = 0; i < m; ++i)
        for (unsigned long j = 0; j < n; ++j) c[i * n + j] = a[j * m + i];
}
