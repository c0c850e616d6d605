/* Minimal CBLAS declarations used to compile the reference CPU engine
 * (engine/src/tensor_ops.cpp, engine/src/conv_ops.cpp include <cblas.h>) on an
 * image that ships an OpenBLAS binary but no development header.
 * Only the single routine the engine calls is declared. Test infrastructure. */
#ifndef SEERA_ORACLE_CBLAS_SHIM_H
#define SEERA_ORACLE_CBLAS_SHIM_H
#ifdef __cplusplus
extern "C" {
#endif
typedef enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_ORDER;
typedef enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;
void cblas_sgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb,
                 int M, int N, int K, float alpha, const float *A, int lda,
                 const float *B, int ldb, float beta, float *C, int ldc);
#ifdef __cplusplus
}
#endif
#endif
