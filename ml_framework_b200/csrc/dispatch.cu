// Public GEMM / convolution entries: choose the contraction engine by the precision mode.
//   mode 0    fp32 CUDA-core tiles (gemm_conv_simt.cu)
//   mode 1/2  tcgen05 tensor-core tiles (contraction_tc.cu): bf16 single pass / bf16x3
// Argument validation is shared: the CUDA-core entry checks are repeated by the tensor-core path through
// the same geometry tests before any launch.
#include "common.cuh"
#include "internal.h"
#include <cstring>

using namespace seera;

extern "C" {

int seera_set_option(const char *name, int value) {
    if (!name) return fail(SEERA_E_ARG, "set_option: null name");
    if (!strcmp(name, "dense_tma")) { rt().dense_tma = value != 0; return SEERA_OK; }
    if (!strcmp(name, "conv_tma")) { rt().conv_tma = value != 0; return SEERA_OK; }
    return fail(SEERA_E_ARG, "set_option: unknown option '%s'", name);
}

int seera_cuda_matmul(const float *A, const float *B, float *C, int M, int N, int K, int Nbatch) {
    return rt().precision ? (rt().dense_tma ? seera_tma_matmul(A, B, C, M, N, K, Nbatch) : seera_tc_matmul(A, B, C, M, N, K, Nbatch)) : seera_simt_matmul(A, B, C, M, N, K, Nbatch);
}
int seera_cuda_matmul_bwd(const float *A, const float *B, const float *dC, float *dA, float *dB, int M, int N, int K, int Nbatch) {
    return rt().precision ? (rt().dense_tma ? seera_tma_matmul_bwd(A, B, dC, dA, dB, M, N, K, Nbatch) : seera_tc_matmul_bwd(A, B, dC, dA, dB, M, N, K, Nbatch)) : seera_simt_matmul_bwd(A, B, dC, dA, dB, M, N, K, Nbatch);
}
int seera_cuda_conv2d_fwd(const float *image, const float *kernel, float *out, int batchN, int C, int H, int W, int F, int R, int S,
                          int pad_h, int pad_w, int stride_h, int stride_w) {
    return rt().precision ? (rt().conv_tma ? seera_tma_conv2d_fwd(image, kernel, out, batchN, C, H, W, F, R, S, pad_h, pad_w, stride_h, stride_w) : seera_tc_conv2d_fwd(image, kernel, out, batchN, C, H, W, F, R, S, pad_h, pad_w, stride_h, stride_w)) : seera_simt_conv2d_fwd(image, kernel, out, batchN, C, H, W, F, R, S, pad_h, pad_w, stride_h, stride_w);
}
int seera_cuda_conv2d_bwd(const float *W, const float *X, const float *dY, float *dX, float *dW, int batch, int C, int H, int W_in,
                          int F, int R, int S, int strideh, int stridew, int padh, int padw) {
    return rt().precision ? (rt().conv_tma ? seera_tma_conv2d_bwd(W, X, dY, dX, dW, batch, C, H, W_in, F, R, S, strideh, stridew, padh, padw) : seera_tc_conv2d_bwd(W, X, dY, dX, dW, batch, C, H, W_in, F, R, S, strideh, stridew, padh, padw)) : seera_simt_conv2d_bwd(W, X, dY, dX, dW, batch, C, H, W_in, F, R, S, strideh, stridew, padh, padw);
}
int seera_cuda_conv2DTranpose_fwd(const float *X, const float *W, float *out, int batch, int Cin, int Hin, int Win, int Cout,
                                  int KH, int KW, int strideh, int stridew, int padh, int padw) {
    return rt().precision ? (rt().conv_tma ? seera_tma_convT_fwd(X, W, out, batch, Cin, Hin, Win, Cout, KH, KW, strideh, stridew, padh, padw) : seera_tc_convT_fwd(X, W, out, batch, Cin, Hin, Win, Cout, KH, KW, strideh, stridew, padh, padw)) : seera_simt_convT_fwd(X, W, out, batch, Cin, Hin, Win, Cout, KH, KW, strideh, stridew, padh, padw);
}
int seera_cuda_conv2DTranspose_bwd(const float *W, const float *X, const float *dY, float *dX, float *dW, int batch, int Cin, int Hin,
                                   int Win, int Cout, int KH, int KW, int strideh, int stridew, int padh, int padw) {
    return rt().precision ? (rt().conv_tma ? seera_tma_convT_bwd(W, X, dY, dX, dW, batch, Cin, Hin, Win, Cout, KH, KW, strideh, stridew, padh, padw) : seera_tc_convT_bwd(W, X, dY, dX, dW, batch, Cin, Hin, Win, Cout, KH, KW, strideh, stridew, padh, padw)) : seera_simt_convT_bwd(W, X, dY, dX, dW, batch, Cin, Hin, Win, Cout, KH, KW, strideh, stridew, padh, padw);
}

}  // extern "C"
