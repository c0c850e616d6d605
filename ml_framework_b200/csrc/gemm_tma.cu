// Dense GEMMs fed by TMA: cp.async.bulk.tensor -> 128-byte-swizzled shared memory -> tcgen05.mma -> TMEM.
//
// Serves cuda_matmul and both products of cuda_matmul_bwd (reference: engine_cuda/src/GEMM.cu:13-225, which
// materialises B^T and A^T in HBM and runs one warp per 16x16 WMMA tile).  The boundary hands over fp32
// row-major matrices; TMA cannot convert, so each operand is first rounded to a bf16 "shadow" (plus the bf16
// residual for the bf16x3 mode) by one vectorised pass, in its NATURAL row-major layout.  No transpose is
// ever written: whether an operand is read along its rows or along its columns is a property of the tensor
// map box and of the matrix descriptor (K-major vs MN-major), so
//     C  = A  * B      A K-major,  B MN-major
//     dA = dC * B^T    dC K-major, B K-major
//     dB = A^T * dC    A MN-major, dC MN-major (contraction over the batch rows, split-K)
// all read the same three shadows.
//
// CTA = 192 threads: warp 0 issues TMA loads into a ring of stages (mbarrier expect_tx), warp 1 owns TMEM
// and issues the MMAs (tcgen05.commit releases a stage), warps 2-5 drain the 128 x BN fp32 accumulator
// with tcgen05.ld and store it.  Every mbarrier wait is bounded; on expiry a status word is set and the
// CTA still waits (bounded) for its copies in flight and frees TMEM before it exits.
#include "internal.h"
#include "tma_gemm_kernel.cuh"


using namespace seera;

extern "C" {

int seera_tma_matmul(const float *A, const float *B, float *C, int M, int N, int K, int Nbatch) {
    return seera_tma_matmul_bias_act(A, B, nullptr, C, M, N, K, Nbatch, SEERA_ACT_NONE);
}

// C = act(A * B + bias[column]); bias may be null.
int seera_tma_matmul_bias_act(const float *A, const float *B, const float *bias, float *C, int M, int N, int K, int Nbatch, int act) {
    SEERA_ENSURE();
    if (M < 1 || N < 1 || K < 1 || Nbatch < 1 || !A || !B || !C) return fail(SEERA_E_ARG, "cuda_matmul: bad argument");
    long long rows = (long long)M * Nbatch;
    if (rows > 0x7fffffff) return fail(SEERA_E_LIMIT, "cuda_matmul: batch*M too large");
    int ns = precision_copies();
    Shadow sa, sb;
    int s = make_shadow(A, (int)rows, K, ns, sa, CLS_ACT);
    if (!s) s = make_shadow(B, K, N, ns, sb, CLS_WEIGHT);
    if (!s) s = run_tma_gemm(sa, 0, sb, 1, StoreDense{C, N}, (int)rows, N, K, true, "cuda_matmul", bias, act);
    free_shadow(sa); free_shadow(sb);
    return s;
}

int seera_tma_matmul_bwd(const float *A, const float *B, const float *dC, float *dA, float *dB, int M, int N, int K, int Nbatch) {
    SEERA_ENSURE();
    if (M < 1 || N < 1 || K < 1 || Nbatch < 1 || !A || !B || !dC) return fail(SEERA_E_ARG, "cuda_matmul_bwd: bad argument");
    long long rows = (long long)M * Nbatch;
    if (rows > 0x7fffffff) return fail(SEERA_E_LIMIT, "cuda_matmul_bwd: batch*M too large");
    int ns = precision_copies();
    Shadow sd, sa, sb;
    int s = make_shadow(dC, (int)rows, N, ns, sd, CLS_GRAD);
    if (!s && dA) {      // dA[rows,K] = dC[rows,N] * B[K,N]^T : contraction over N, both operands read along their rows
        s = make_shadow(B, K, N, ns, sb, CLS_WEIGHT);
        if (!s) s = run_tma_gemm(sd, 0, sb, 0, StoreDense{dA, K}, (int)rows, K, N, true, "cuda_matmul_bwd(dA)");
    }
    if (!s && dB) {      // dB[K,N] = A[rows,K]^T * dC[rows,N] : contraction over rows, both operands read along their columns
        s = make_shadow(A, (int)rows, K, ns, sa, CLS_ACT);
        if (!s) s = run_tma_gemm(sa, 1, sd, 1, StoreDense{dB, N}, K, N, (int)rows, true, "cuda_matmul_bwd(dB)", nullptr, 0, wgrad_copies(ns));
    }
    free_shadow(sd); free_shadow(sa); free_shadow(sb);
    return s;
}

}  // extern "C"
