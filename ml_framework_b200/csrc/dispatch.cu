// Public GEMM / convolution entries: choose the contraction engine by the precision mode.
//   mode 0      fp32 CUDA-core tiles (gemm_conv_simt.cu)
//   mode 1/2/3  tcgen05 tensor-core tiles fed by TMA (gemm_tma.cu, conv_tma.cu; short patches conv_first.cu, few channels
//               conv_few.cu): bf16 single pass / bf16x3 / bf16x6.  The in-kernel-gather kernel of contraction_tc.cu is the
//               fallback for geometries a tensor map cannot express and is selectable with the "dense_tma" / "conv_tma" options.
// Argument validation is shared: the CUDA-core entry checks are repeated by the tensor-core path through
// the same geometry tests before any launch.
#include "common.cuh"
#include "internal.h"
#include <cstring>

using namespace seera;

extern "C" {

int seera_set_option(const char *name, int value) {
    if (!name) return fail(SEERA_E_ARG, "set_option: null name");
    if (!strcmp(name, "mma_issuers")) {
        if (value != 0 && value != 1 && value != 2) return fail(SEERA_E_ARG, "set_option: mma_issuers must be 0, 1 or 2");
        rt().mma_issuers = value;
        return SEERA_OK;
    }
    if (!strcmp(name, "skinny_gemm")) { rt().skinny_gemm = value != 0; return SEERA_OK; }
    if (!strcmp(name, "dense_tma")) { rt().dense_tma = value != 0; return SEERA_OK; }
    if (!strcmp(name, "conv_tma")) { rt().conv_tma = value != 0; return SEERA_OK; }
    if (!strcmp(name, "pair_tiles")) { rt().pair_tiles = value != 0; return SEERA_OK; }
    if (!strcmp(name, "wgrad_single")) { rt().wgrad_single = value != 0; return SEERA_OK; }
    if (!strcmp(name, "tc_wait_ms")) {
        if (value < 1 || value > 60000) return fail(SEERA_E_ARG, "set_option: tc_wait_ms must be in [1, 60000]");
        rt().tc_wait_clocks = (unsigned long long)value * 2000000ull;
        return SEERA_OK;
    }
    if (!strcmp(name, "tc_test_skip_load")) { rt().tc_test_skip_load = value; return SEERA_OK; }
    if (!strcmp(name, "pool_short_patch")) { rt().pool_short_patch = value != 0; return SEERA_OK; }
    if (!strcmp(name, "sm_reserve")) {
        if (value < 0 || value >= rt().sm_physical) return fail(SEERA_E_ARG, "set_option: sm_reserve must be in [0, %d)", rt().sm_physical);
        rt().sm_count = rt().sm_physical - value;
        return SEERA_OK;
    }
    if (!strcmp(name, "tile_n_cap2") || !strcmp(name, "tile_n_cap3")) {
        if (value != 64 && value != 128 && value != 256) return fail(SEERA_E_ARG, "set_option: %s must be 64, 128 or 256", name);
        (name[10] == '2' ? rt().tile_n_cap2 : rt().tile_n_cap3) = value;
        return SEERA_OK;
    }
    return fail(SEERA_E_ARG, "set_option: unknown option '%s'", name);
}

// a product of at most 16 output columns runs as exact fp32 on the CUDA cores in every mode (gemm_skinny.cu)
static bool skinny_ok(const void *a, const void *b, const void *c, int M, int N, int K, int Nbatch) {
    return a && b && c && M >= 1 && Nbatch >= 1 && !seera::ensure_init() && seera::skinny_applies(M, N, K, Nbatch);
}
int seera_cuda_matmul(const float *A, const float *B, float *C, int M, int N, int K, int Nbatch) {
    if (skinny_ok(A, B, C, M, N, K, Nbatch)) return seera::skinny_fwd(A, B, nullptr, C, M * Nbatch, N, K, SEERA_ACT_NONE, "cuda_matmul");
    return rt().precision ? (rt().dense_tma ? seera_tma_matmul(A, B, C, M, N, K, Nbatch) : seera_tc_matmul(A, B, C, M, N, K, Nbatch)) : seera_simt_matmul(A, B, C, M, N, K, Nbatch);
}
int seera_cuda_matmul_bwd(const float *A, const float *B, const float *dC, float *dA, float *dB, int M, int N, int K, int Nbatch) {
    if (skinny_ok(A, B, dC, M, N, K, Nbatch)) return seera::skinny_bwd(A, B, dC, dA, dB, nullptr, M * Nbatch, N, K);
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


// ---- forward products with the bias and activation applied before the one store of the output ----------------
static int bias_act_after(int s, float *y, const float *bias, long long size, int channels, int inner, int act) {
    if (s || (!bias && !act)) return s;
    if (size > 0x7fffffff) return seera::fail(SEERA_E_LIMIT, "bias_act: tensor too large");
    return seera_bias_act_fwd(y, bias, y, (int)size, channels, inner, act);
}
int seera_matmul_bias_act_fwd(const float *A, const float *B, const float *bias, float *C, int M, int N, int K, int act) {
    if (skinny_ok(A, B, C, M, N, K, 1)) return seera::skinny_fwd(A, B, bias, C, M, N, K, act, "cuda_matmul");
    if (rt().precision && rt().dense_tma) return seera_tma_matmul_bias_act(A, B, bias, C, M, N, K, 1, act);
    return bias_act_after(seera_cuda_matmul(A, B, C, M, N, K, 1), C, bias, (long long)M * N, N, 1, act);
}
int seera_conv2d_bias_act_fwd(const float *image, const float *kernel, const float *bias, float *out, int batchN, int C, int H, int W,
                              int F, int R, int S, int pad_h, int pad_w, int stride_h, int stride_w, int act) {
    if (rt().precision && rt().conv_tma)
        return seera_tma_conv2d_bias_act_fwd(image, kernel, bias, out, batchN, C, H, W, F, R, S, pad_h, pad_w, stride_h, stride_w, act);
    int OH = (H + 2 * pad_h - R) / (stride_h > 0 ? stride_h : 1) + 1, OW = (W + 2 * pad_w - S) / (stride_w > 0 ? stride_w : 1) + 1;
    return bias_act_after(seera_cuda_conv2d_fwd(image, kernel, out, batchN, C, H, W, F, R, S, pad_h, pad_w, stride_h, stride_w), out, bias,
                          (long long)batchN * F * OH * OW, F, OH * OW, act);
}
int seera_conv2DTranspose_bias_act_fwd(const float *X, const float *W, const float *bias, float *out, int batch, int Cin, int Hin, int Win,
                                       int Cout, int KH, int KW, int strideh, int stridew, int padh, int padw, int act) {
    if (rt().precision && rt().conv_tma)
        return seera_tma_convT_bias_act_fwd(X, W, bias, out, batch, Cin, Hin, Win, Cout, KH, KW, strideh, stridew, padh, padw, act);
    int Ho = (Hin - 1) * strideh - 2 * padh + KH, Wo = (Win - 1) * stridew - 2 * padw + KW;
    return bias_act_after(seera_cuda_conv2DTranpose_fwd(X, W, out, batch, Cin, Hin, Win, Cout, KH, KW, strideh, stridew, padh, padw), out,
                          bias, (long long)batch * Cout * Ho * Wo, Cout, Ho * Wo, act);
}

}  // extern "C"
