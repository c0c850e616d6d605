/* Fallback cblas_sgemm (row-major only) for hosts where no OpenBLAS binary is
 * available to link the reference CPU engine against. Plain fp32 dot products,
 * k innermost, OpenMP over output rows. Test infrastructure. */
#include "cblas.h"
void cblas_sgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb,
                 int M, int N, int K, float alpha, const float *A, int lda,
                 const float *B, int ldb, float beta, float *C, int ldc)
{
    (void)order;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < M; i++) {
        float *c = C + (long)i * ldc;
        for (int j = 0; j < N; j++) c[j] = (beta == 0.0f) ? 0.0f : beta * c[j];
        for (int k = 0; k < K; k++) {
            float a = alpha * (ta == CblasNoTrans ? A[(long)i * lda + k] : A[(long)k * lda + i]);
            if (tb == CblasNoTrans) {
                const float *b = B + (long)k * ldb;
                for (int j = 0; j < N; j++) c[j] += a * b[j];
            } else {
                for (int j = 0; j < N; j++) c[j] += a * B[(long)j * ldb + k];
            }
        }
    }
}
