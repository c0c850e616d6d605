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


// ---- Dense layers that hand their 16-bit operand copies from call to call ------------------------------------------------
// Row-major copies of one [rows, cols] matrix (activations of a Dense layer, or its weight matrix), kept by the caller
// between the forward and the backward call of a layer, or written by one layer's epilogue for the next layer's forward.
struct seera_rows {
    seera::Shadow s;
    int ns;
};

namespace seera {

// C[m*ld + n] plus the 16-bit copies of the same values: the output of a Dense layer that feeds another Dense layer.
struct StoreDenseCopies {
    static constexpr bool kMContiguous = false;
    float *C; long long ld;
    __nv_bfloat16 *cp[3]; int cld, ns; Enc enc;
    __device__ void copy_out(int m, int n, float v) const {
        const long long o = (long long)m * cld + n;
        store_split1(v, ns, enc, cp[0] + o, cp[1] + o, cp[2] + o);
    }
    __device__ void operator()(int m, int n, float v) const { C[(long long)m * ld + n] = v; copy_out(m, n, v); }
    __device__ float *row(int m) const { return C + (long long)m * ld; }
    __device__ long long nstride() const { return 1; }
};

__device__ __forceinline__ float dense_slope(float y, int act) {
    switch (act) {
        case SEERA_ACT_RELU: return y > 0.f ? 1.f : 0.f;
        case SEERA_ACT_SIGMOID: return y * (1.f - y);
        case SEERA_ACT_TANH: return 1.f - y * y;
        default: return 1.f;
    }
}
// dz = g * act'(y) of a Dense layer, written ONLY as the 16-bit copies its two backward products read, plus per-block column
// sums for the bias gradient.  Block = 32 groups of 8 columns x 8 row lanes; grid (column blocks, row splits).
template <int NS>
__global__ void __launch_bounds__(256) dz_rows_kernel(const float *__restrict__ g, const float *__restrict__ y, int rows, int cols, int ld,
                                                      __nv_bfloat16 *__restrict__ d0, __nv_bfloat16 *__restrict__ d1,
                                                      __nv_bfloat16 *__restrict__ d2, Enc enc, float *__restrict__ partial, int act) {
    __shared__ float sm[8][32][9];
    const int cg = threadIdx.x & 31, lane_r = threadIdx.x >> 5;
    const int c0 = (blockIdx.x * 32 + cg) * 8, s = blockIdx.y, splits = gridDim.y;
    const bool vec = (cols & 3) == 0 && ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i] = 0.f;
    if (c0 < ld) {
        for (int r = s * 8 + lane_r; r < rows; r += splits * 8) {
            const long long base = (long long)r * cols + c0;
            float v[8], yv[8];
            if (vec && c0 + 8 <= cols) {
                const float4 a = __ldg(reinterpret_cast<const float4 *>(g + base)), b = __ldg(reinterpret_cast<const float4 *>(g + base) + 1);
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
                if (act) {
                    const float4 c = __ldg(reinterpret_cast<const float4 *>(y + base)), d = __ldg(reinterpret_cast<const float4 *>(y + base) + 1);
                    yv[0] = c.x; yv[1] = c.y; yv[2] = c.z; yv[3] = c.w; yv[4] = d.x; yv[5] = d.y; yv[6] = d.z; yv[7] = d.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const bool in = c0 + i < cols;
                    v[i] = in ? __ldg(g + base + i) : 0.f;
                    yv[i] = (in && act) ? __ldg(y + base + i) : 0.f;
                }
            }
            if (act) {
#pragma unroll
                for (int i = 0; i < 8; i++) v[i] *= dense_slope(yv[i], act);
            }
#pragma unroll
            for (int i = 0; i < 8; i++) acc[i] += v[i];
            const long long o = (long long)r * ld + c0;
            store_split8<NS>(v, enc, d0 + o, d1 + o, d2 + o);
        }
    }
    if (partial) {
#pragma unroll
        for (int i = 0; i < 8; i++) sm[lane_r][cg][i] = acc[i];
        __syncthreads();
        if (lane_r == 0 && c0 < ld) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                float t = 0.f;
#pragma unroll
                for (int k = 0; k < 8; k++) t += sm[k][cg][i];
                if (c0 + i < cols) partial[(long long)s * cols + c0 + i] = t;
            }
        }
    }
}
static const Shadow *rows_usable(const seera_rows *h, int ns, int rows, int cols, int cls) {
    const Enc want = enc_for(cls);
    if (!h || h->ns < ns || h->s.rows != rows || h->s.cols != cols || h->s.enc.fmt != want.fmt || h->s.enc.scale != want.scale ||
        h->s.enc.dscale != want.dscale) return nullptr;
    return &h->s;
}
static bool dense_keeps() { return rt().precision != 0 && rt().dense_tma; }

}  // namespace seera

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


void seera_rows_free(seera_rows_t *h) {
    if (!h) return;
    free_shadow(h->s);
    delete h;
}

int seera_matmul_bias_act_fwd_s(const float *A, const float *B, const float *bias, float *C, int M, int N, int K, int act,
                                seera_rows_t *a_in, seera_rows_t **a_keep, seera_rows_t **w_keep, seera_rows_t **c_copies) {
    SEERA_ENSURE();
    if (a_keep) *a_keep = nullptr;
    if (w_keep) *w_keep = nullptr;
    if (c_copies) *c_copies = nullptr;
    if (!dense_keeps() || skinny_applies(M, N, K, 1)) return seera_matmul_bias_act_fwd(A, B, bias, C, M, N, K, act);
    if (M < 1 || N < 1 || K < 1 || !A || !B || !C) return fail(SEERA_E_ARG, "matmul_bias_act_fwd: bad argument");
    const int ns = precision_copies();
    Shadow sa_local, sb, sc;
    const Shadow *sa = rows_usable(a_in, ns, M, K, CLS_ACT);
    int s = SEERA_OK;
    if (!sa) { s = make_shadow(A, M, K, ns, sa_local, CLS_ACT); sa = &sa_local; }
    if (!s) s = make_shadow(B, K, N, ns, sb, CLS_WEIGHT);
    if (!s && c_copies) {
        s = alloc_shadow(sc, M, N, ns);
        sc.enc = enc_for(CLS_ACT);
    }
    if (!s) {
        if (c_copies) {
            StoreDenseCopies cs{C, N, {sc.p[0], sc.p[1], sc.p[2]}, sc.ld, ns, sc.enc};
            s = run_tma_gemm(*sa, 0, sb, 1, cs, M, N, K, true, "cuda_matmul", bias, act);
        } else {
            s = run_tma_gemm(*sa, 0, sb, 1, StoreDense{C, N}, M, N, K, true, "cuda_matmul", bias, act);
        }
    }
    if (!s && a_keep && sa == &sa_local) { *a_keep = new seera_rows{sa_local, ns}; sa_local = Shadow{}; }
    if (!s && w_keep) { *w_keep = new seera_rows{sb, ns}; sb = Shadow{}; }
    if (!s && c_copies) { *c_copies = new seera_rows{sc, ns}; sc = Shadow{}; }
    free_shadow(sa_local); free_shadow(sb); free_shadow(sc);
    return s;
}

// Backward of y = act(A B + bias): dz = g * act'(y) goes straight into 16-bit copies (with the bias gradient), then
// dA = dz B^T and dB = A^T dz on the tensor cores, reading the copies of A and B the forward call kept.
int seera_matmul_act_bwd(const float *A, const float *B, const float *y, const float *g, float *dA, float *dB, float *dbias,
                         int M, int N, int K, int act, seera_rows_t *a_keep, seera_rows_t *w_keep) {
    SEERA_ENSURE();
    if (M < 1 || N < 1 || K < 1 || !A || !B || !g || (act != SEERA_ACT_NONE && !y))
        return fail(SEERA_E_ARG, "matmul_act_bwd: bad argument");
    if (act == SEERA_ACT_NONE && skinny_applies(M, N, K, 1)) return skinny_bwd(A, B, g, dA, dB, dbias, M, N, K);
    if (!dense_keeps() || skinny_applies(M, N, K, 1)) {          // composition of the separate entries
        float *dz = (float *)scratch_alloc((size_t)M * N * sizeof(float));
        if (!dz) return SEERA_E_OOM;
        int s = seera_act_bias_bwd(g, y, dz, dbias, M * N, N, 1, act);
        if (!s) s = seera_cuda_matmul_bwd(A, B, dz, dA, dB, M, N, K, 1);
        scratch_free(dz);
        return s;
    }
    const int ns = precision_copies();
    Shadow sd, sa_local, sb_local;
    int s = alloc_shadow(sd, M, N, ns);
    sd.enc = enc_for(CLS_GRAD);        // the dynamic factor is the one the loss head set for this backward pass
    float *partial = nullptr;
    if (!s) {
        const int colblocks = (sd.ld / 8 + 31) / 32;
        int splits = (rt().sm_count * 4 + colblocks - 1) / colblocks;
        const int maxs = (M + 7) / 8;
        if (splits > maxs) splits = maxs;
        if (splits < 1) splits = 1;
        if (dbias) { partial = (float *)scratch_alloc((size_t)splits * N * sizeof(float)); if (!partial) s = SEERA_E_OOM; }
        if (!s) {
            ProfBytes pb(4.0 * M * N * (act ? 2 : 1) + 2.0 * ns * M * sd.ld, "dz_rows");
            dim3 grid(colblocks, splits);
            cudaStream_t st = rt().stream;
            if (ns == 1) dz_rows_kernel<1><<<grid, 256, 0, st>>>(g, y, M, N, sd.ld, sd.p[0], sd.p[1], sd.p[2], sd.enc, partial, act);
            else if (ns == 2) dz_rows_kernel<2><<<grid, 256, 0, st>>>(g, y, M, N, sd.ld, sd.p[0], sd.p[1], sd.p[2], sd.enc, partial, act);
            else dz_rows_kernel<3><<<grid, 256, 0, st>>>(g, y, M, N, sd.ld, sd.p[0], sd.p[1], sd.p[2], sd.enc, partial, act);
            count_launch();
            cudaError_t e = cudaGetLastError();
            if (e == cudaSuccess && dbias) {
                launch_sum_splits(partial, dbias, N, splits, st);
                e = cudaGetLastError();
            }
            if (e != cudaSuccess) s = check_cuda(e, "matmul_act_bwd(dz)");
        }
        if (partial) scratch_free(partial);
    }
    if (!s && dA) {
        const Shadow *sb = rows_usable(w_keep, ns, K, N, CLS_WEIGHT);
        if (!sb) { s = make_shadow(B, K, N, ns, sb_local, CLS_WEIGHT); sb = &sb_local; }
        if (!s) s = run_tma_gemm(sd, 0, *sb, 0, StoreDense{dA, K}, M, K, N, true, "cuda_matmul_bwd(dA)");
    }
    if (!s && dB) {
        const Shadow *sa = rows_usable(a_keep, wgrad_copies(ns), M, K, CLS_ACT);
        if (!sa) { s = make_shadow(A, M, K, ns, sa_local, CLS_ACT); sa = &sa_local; }
        if (!s) s = run_tma_gemm(*sa, 1, sd, 1, StoreDense{dB, N}, K, N, M, true, "cuda_matmul_bwd(dB)", nullptr, 0, wgrad_copies(ns));
    }
    free_shadow(sd); free_shadow(sa_local); free_shadow(sb_local);
    return s;
}

}  // extern "C"
