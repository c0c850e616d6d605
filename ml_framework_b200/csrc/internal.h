// Entry points shared between translation units but not part of the public C ABI.
#pragma once
extern "C" {
int seera_simt_matmul(const float *A, const float *B, float *C, int M, int N, int K, int Nbatch);
int seera_simt_matmul_bwd(const float *A, const float *B, const float *dC, float *dA, float *dB, int M, int N, int K, int Nbatch);
int seera_simt_conv2d_fwd(const float *X, const float *Wt, float *Y, int NB, int C, int H, int W, int F, int R, int S,
                          int ph, int pw, int sh, int sw);
int seera_simt_conv2d_bwd(const float *Wt, const float *X, const float *dY, float *dX, float *dW, int NB, int C, int H, int W,
                          int F, int R, int S, int sh, int sw, int ph, int pw);
int seera_simt_convT_fwd(const float *X, const float *Wt, float *out, int NB, int Cin, int H, int W, int Cout, int KH, int KW,
                         int sh, int sw, int ph, int pw);
int seera_simt_convT_bwd(const float *Wt, const float *X, const float *dY, float *dX, float *dW, int NB, int Cin, int H, int W,
                         int Cout, int KH, int KW, int sh, int sw, int ph, int pw);
int seera_tma_matmul(const float *A, const float *B, float *C, int M, int N, int K, int Nbatch);
int seera_tma_matmul_bwd(const float *A, const float *B, const float *dC, float *dA, float *dB, int M, int N, int K, int Nbatch);
int seera_tma_conv2d_fwd(const float *X, const float *Wt, float *Y, int NB, int C, int H, int W, int F, int R, int S,
                         int ph, int pw, int sh, int sw);
int seera_tma_conv2d_bwd(const float *Wt, const float *X, const float *dY, float *dX, float *dW, int NB, int C, int H, int W,
                         int F, int R, int S, int sh, int sw, int ph, int pw);
int seera_tma_convT_fwd(const float *X, const float *Wt, float *out, int NB, int Cin, int H, int W, int Cout, int KH, int KW,
                        int sh, int sw, int ph, int pw);
int seera_tma_convT_bwd(const float *Wt, const float *X, const float *dY, float *dX, float *dW, int NB, int Cin, int H, int W,
                        int Cout, int KH, int KW, int sh, int sw, int ph, int pw);
int seera_tma_matmul_bias_act(const float *A, const float *B, const float *bias, float *C, int M, int N, int K, int Nbatch, int act);
int seera_tma_conv2d_bias_act_fwd(const float *X, const float *Wt, const float *bias, float *Y, int NB, int C, int H, int W, int F,
                                  int R, int S, int ph, int pw, int sh, int sw, int act);
int seera_tma_convT_bias_act_fwd(const float *X, const float *Wt, const float *bias, float *out, int NB, int Cin, int H, int W,
                                 int Cout, int KH, int KW, int sh, int sw, int ph, int pw, int act);
int seera_tc_matmul(const float *A, const float *B, float *C, int M, int N, int K, int Nbatch);
int seera_tc_matmul_bwd(const float *A, const float *B, const float *dC, float *dA, float *dB, int M, int N, int K, int Nbatch);
int seera_tc_conv2d_fwd(const float *X, const float *Wt, float *Y, int NB, int C, int H, int W, int F, int R, int S,
                        int ph, int pw, int sh, int sw);
int seera_tc_conv2d_bwd(const float *Wt, const float *X, const float *dY, float *dX, float *dW, int NB, int C, int H, int W,
                        int F, int R, int S, int sh, int sw, int ph, int pw);
int seera_tc_convT_fwd(const float *X, const float *Wt, float *out, int NB, int Cin, int H, int W, int Cout, int KH, int KW,
                       int sh, int sw, int ph, int pw);
int seera_tc_convT_bwd(const float *Wt, const float *X, const float *dY, float *dX, float *dW, int NB, int Cin, int H, int W,
                       int Cout, int KH, int KW, int sh, int sw, int ph, int pw);
}

#include "tc_epilogue.cuh"
namespace seera {
bool conv_first_pool_ok(int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw);
int conv_first_pool_fwd(const float *X, const float *Wt, const float *bias, const PoolOut &pool, int NB, int C, int H, int W, int F, int R,
                        int S, int ph, int pw, int sh, int sw, int act, const char *name);
// Dense products of at most 16 output columns, exact fp32 on the CUDA cores (gemm_skinny.cu).  rows = M * batch; bias, dA, dB and
// dbias may be null (dbias = the column sums of dC).
bool skinny_applies(int M, int N, int K, int Nbatch);
int skinny_fwd(const float *A, const float *B, const float *bias, float *C, int rows, int N, int K, int act, const char *name);
int skinny_bwd(const float *A, const float *B, const float *dC, float *dA, float *dB, float *dbias, int rows, int N, int K);
// Direct fp32 kernel for unit-stride (transposed) convolutions with 1, 2 or 4 output channels (conv_few.cu); bias may be null.
bool conv_few_applies(int NB, int C, int F, int R, int S, int OH, int OW);
int conv_few_fwd(const float *X, const float *Wt, const float *bias, float *Y, int NB, int C, int H, int W, int F, int R, int S, int PH,
                 int PW, int OH, int OW, int act, int transposed, const char *name);
// 3 x 3 unit-stride convolution with at most seven input channels + bias + activation + 2x2 max-pool, direct fp32 (conv_few.cu).
bool conv_pool_simt_applies(int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw);
int conv_pool_simt(const float *X, const float *Wt, const float *bias, const PoolOut &pool, int NB, int C, int H, int W, int F, int ph, int pw,
                   int act, const char *name);
// Forward of a "same" 3 x 3 unit-stride convolution with one input channel, direct fp32 (conv_few.cu); bias may be null.
bool conv_c1_fwd_applies(const float *X, const float *Y, int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw);
int conv_c1_fwd(const float *X, const float *Wt, const float *bias, float *Y, int NB, int H, int W, int F, int ph, int act, const char *name);
// Weight gradient of a convolution with one input channel and at most nine taps, direct fp32 (conv_few.cu).
bool wgrad_c1_applies(int NB, int C, int F, int R, int S, int OH, int OW);
int wgrad_c1(const float *A, const float *dY, float *dW, int NB, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw,
             const char *name);
// Direct fp32 kernels for convolutions with C*R*S <= 64 (conv_first.cu); bias may be null.
bool conv_first_applies(int C, int R, int S);
int conv_first_fwd(const float *X, const float *Wt, const float *bias, float *Y, int NB, int C, int H, int W, int F, int R, int S,
                   int ph, int pw, int sh, int sw, int act, const char *name);
bool conv_first_fuses_bias(int C, int R, int S);
int conv_first_act_wgrad(const float *X, const float *y, const float *g, const float *gp, const int *mask, const float *y_pooled,
                         float *dW, float *dbias, int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw,
                         int act, const char *name);
int conv_first_wgrad(const float *X, const float *dY, float *dW, int NB, int C, int H, int W, int F, int R, int S, int sh, int sw,
                     int ph, int pw, const char *name);
}
