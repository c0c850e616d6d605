// Dense products with at most 16 output columns (classifier heads: 256 -> 10, 784 -> 10, 1024 -> 10), exact fp32 on the
// CUDA cores, used in every precision mode.
//
// Such a product is a few MFLOP: on the tensor-core path it costs two operand conversions, a TMA pipeline fill for a handful
// of k-steps into a 32-column tile that is two thirds padding, and a split-K reduce - about 15 us per launch, three launches per
// layer and step - for well under a microsecond of arithmetic.  Here each of the three products of a layer (reference:
// engine_cuda/src/GEMM.cu:95-103 forward, :164-225 backward) is one or two small launches that read the fp32 operands in place:
//   C  = act(A B + bias)   a warp per pair of rows (a block per pair where rows are few), lanes stride over k, N running sums
//                          per lane and row, shuffle reduction
//   dA = dC B^T            one thread per element of dA, N multiply-adds
//   dB = A^T dC (+ dbias)  one thread per row of dB walks its share of the M rows; the shares are summed in a fixed order by a
//                          second small kernel, so the result does not depend on scheduling
#include "common.cuh"
#include "internal.h"
#include "tc_epilogue.cuh"

namespace seera {

constexpr int SK_MAXN = 16;

// k-extent of the slice of B a block keeps in shared memory: N * sk_kc(N) floats, at most 48 KB
__host__ __device__ constexpr int sk_kc(int n) { return n <= 12 ? 1024 : 768; }
constexpr int SK_ROWS = 64;          // most rows of dC a block stages at a time in the two backward kernels

// C = act(A B + bias).  A block keeps B^T (slice by slice when K exceeds it) in shared memory as bt[n][k], so that lane = k reads
// it without bank conflicts; a warp forms two rows of C at a time: lanes stride over k (coalesced reads of A), 2 * N running
// sums per lane, shuffle reduction at the end.  With more than one slice the later slices add into C and the last applies
// bias and activation.
template <int N>
__global__ void __launch_bounds__(256) skinny_fwd_kernel(const float *__restrict__ A, const float *__restrict__ B, const float *__restrict__ bias,
                                                         float *__restrict__ C, int rows, int K, int act) {
    constexpr int SK_KC = sk_kc(N);
    extern __shared__ float bt[];                                        // [N][SK_KC]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int k0 = 0; k0 < K; k0 += SK_KC) {
        const int kc = min(SK_KC, K - k0);
        __syncthreads();
        for (int e = threadIdx.x; e < kc * N; e += 256) {                 // e = k * N + n: consecutive floats of B
            const int k = e / N, n = e - k * N;
            bt[n * SK_KC + k] = __ldg(B + (long long)k0 * N + e);
        }
        __syncthreads();
        const bool first = k0 == 0, last = k0 + kc == K;
        for (int m = (blockIdx.x * 8 + warp) * 2; m < rows; m += gridDim.x * 16) {
            const bool two = m + 1 < rows;
            const float *a0 = A + (long long)m * K + k0, *a1 = a0 + (two ? K : 0);
            float acc0[N], acc1[N];
#pragma unroll
            for (int n = 0; n < N; n++) { acc0[n] = 0.f; acc1[n] = 0.f; }
#pragma unroll 8
            for (int k = lane; k < kc; k += 32) {
                const float x0 = __ldg(a0 + k), x1 = __ldg(a1 + k);
#pragma unroll
                for (int n = 0; n < N; n++) {
                    const float b = bt[n * SK_KC + k];
                    acc0[n] = fmaf(x0, b, acc0[n]);
                    acc1[n] = fmaf(x1, b, acc1[n]);
                }
            }
            float v0 = 0.f, v1 = 0.f;
#pragma unroll
            for (int n = 0; n < N; n++) {
                float t0 = acc0[n], t1 = acc1[n];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    t0 += __shfl_xor_sync(0xffffffffu, t0, o);
                    t1 += __shfl_xor_sync(0xffffffffu, t1, o);
                }
                if (lane == n) { v0 = t0; v1 = t1; }
            }
            if (lane < N) {
                float *c0 = C + (long long)m * N + lane;
                if (!first) { v0 += *c0; if (two) v1 += c0[N]; }
                if (last) {
                    const float bv = bias ? __ldg(bias + lane) : 0.f;
                    v0 = epilogue_act(v0 + bv, act);
                    v1 = epilogue_act(v1 + bv, act);
                }
                *c0 = v0;
                if (two) c0[N] = v1;
            }
        }
    }
}

// The same for few rows (at most a few blocks' worth per SM): one block per pair of rows, its eight warps take interleaved
// 32-wide pieces of k, B read in place (a warp's reads of B cover 32 * N consecutive floats over its n loop, served by L1), the
// warps' sums added in warp order through shared memory.  No staging of B, and a long contraction (a flattened feature map into
// ten classes) is spread over eight warps instead of walked by one.
template <int N>
__global__ void __launch_bounds__(256) skinny_fwd_small_kernel(const float *__restrict__ A, const float *__restrict__ B,
                                                               const float *__restrict__ bias, float *__restrict__ C, int rows, int K, int act) {
    __shared__ float red[8][2][N];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int m = blockIdx.x * 2;
    const bool two = m + 1 < rows;
    const float *a0 = A + (long long)m * K, *a1 = a0 + (two ? K : 0);
    float acc0[N], acc1[N];
#pragma unroll
    for (int n = 0; n < N; n++) { acc0[n] = 0.f; acc1[n] = 0.f; }
#pragma unroll 2
    for (int k = warp * 32 + lane; k < K; k += 256) {
        const float x0 = __ldg(a0 + k), x1 = __ldg(a1 + k);
        const float *b = B + (long long)k * N;
#pragma unroll
        for (int n = 0; n < N; n++) {
            const float bv = __ldg(b + n);
            acc0[n] = fmaf(x0, bv, acc0[n]);
            acc1[n] = fmaf(x1, bv, acc1[n]);
        }
    }
#pragma unroll
    for (int n = 0; n < N; n++) {
        float t0 = acc0[n], t1 = acc1[n];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            t0 += __shfl_xor_sync(0xffffffffu, t0, o);
            t1 += __shfl_xor_sync(0xffffffffu, t1, o);
        }
        if (lane == 0) { red[warp][0][n] = t0; red[warp][1][n] = t1; }
    }
    __syncthreads();
    if (threadIdx.x < 2 * N) {
        const int r = threadIdx.x / N, n = threadIdx.x - r * N;
        if (r == 0 || two) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) v += red[w][r][n];
            if (bias) v += __ldg(bias + n);
            C[(long long)(m + r) * N + n] = epilogue_act(v, act);
        }
    }
}

// Rows of dC staged in shared memory, padded to a multiple of four floats so that a row is read back with 128-bit broadcasts.
template <int N>
struct SkinnyRows {
    static constexpr int NP = (N + 3) / 4 * 4;
    float v[SK_ROWS][NP];
    __device__ void stage(const float *__restrict__ dC, int m0, int nrows) {
        for (int e = threadIdx.x; e < nrows * N; e += 256) {
            const int r = e / N, n = e - r * N;
            v[r][n] = __ldg(dC + (long long)m0 * N + e);
        }
    }
    __device__ void row(int r, float (&d)[NP]) const {
#pragma unroll
        for (int j = 0; j < NP; j += 4) {
            const float4 t = *reinterpret_cast<const float4 *>(&v[r][j]);
            d[j] = t.x; d[j + 1] = t.y; d[j + 2] = t.z; d[j + 3] = t.w;
        }
    }
};

// dA = dC B^T.  Grid (ceil(K / 256), row groups); thread = one column k of dA with its row of B in registers, walking the rows
// of its group: N multiply-adds per element against broadcast reads of the staged dC rows, stores coalesced over k.
template <int N>
__global__ void __launch_bounds__(256) skinny_dA_kernel(const float *__restrict__ dC, const float *__restrict__ B, float *__restrict__ dA,
                                                        int rows, int K, int chunk_rows) {
    __shared__ __align__(16) SkinnyRows<N> sd;
    constexpr int NP = SkinnyRows<N>::NP;
    const int k = blockIdx.x * 256 + threadIdx.x;
    float b[N];
#pragma unroll
    for (int n = 0; n < N; n++) b[n] = k < K ? __ldg(B + (long long)k * N + n) : 0.f;
    for (int m0 = blockIdx.y * chunk_rows; m0 < rows; m0 += gridDim.y * chunk_rows) {
        const int nrows = min(chunk_rows, rows - m0);
        __syncthreads();
        sd.stage(dC, m0, nrows);
        __syncthreads();
        if (k < K) {
#pragma unroll 4
            for (int r = 0; r < nrows; r++) {
                float d[NP];
                sd.row(r, d);
                float s = 0.f;
#pragma unroll
                for (int n = 0; n < N; n++) s = fmaf(d[n], b[n], s);
                dA[(long long)(m0 + r) * K + k] = s;
            }
        }
    }
}

// dB = A^T dC, dbias = column sums of dC.  Grid (ceil(K / 256), splits); thread = one row k of dB walking its split's rows of A
// (coalesced over k, eight loads in flight) against the staged dC rows.  The splits' sums are added up in index order by a second
// small kernel, so the result is the same on every run.
template <int N>
__global__ void __launch_bounds__(256) skinny_dB_kernel(const float *__restrict__ A, const float *__restrict__ dC, float *__restrict__ dB,
                                                        float *__restrict__ dbias, float *__restrict__ partial, int rows, int K, int chunk_rows) {
    __shared__ __align__(16) SkinnyRows<N> sd;
    constexpr int NP = SkinnyRows<N>::NP;
    const int k = blockIdx.x * 256 + threadIdx.x, s = blockIdx.y, splits = gridDim.y;
    const int chunks = (rows + chunk_rows - 1) / chunk_rows, per = (chunks + splits - 1) / splits;
    const int m_begin = (int)min((long long)rows, (long long)s * per * chunk_rows), m_end = (int)min((long long)rows, (long long)(s + 1) * per * chunk_rows);
    float acc[N], colsum = 0.f;
#pragma unroll
    for (int n = 0; n < N; n++) acc[n] = 0.f;
    for (int m0 = m_begin; m0 < m_end; m0 += chunk_rows) {
        const int nrows = min(chunk_rows, m_end - m0);
        __syncthreads();
        sd.stage(dC, m0, nrows);
        __syncthreads();
        if (blockIdx.x == 0 && threadIdx.x < N)
            for (int r = 0; r < nrows; r++) colsum += sd.v[r][threadIdx.x];
        if (k < K) {
            const float *a = A + (long long)m0 * K + k;
            int r = 0;
            for (; r + 8 <= nrows; r += 8) {
                float x[8];
#pragma unroll
                for (int j = 0; j < 8; j++) x[j] = __ldg(a + (long long)(r + j) * K);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    float d[NP];
                    sd.row(r + j, d);
#pragma unroll
                    for (int n = 0; n < N; n++) acc[n] = fmaf(x[j], d[n], acc[n]);
                }
            }
            for (; r < nrows; r++) {
                const float x = __ldg(a + (long long)r * K);
                float d[NP];
                sd.row(r, d);
#pragma unroll
                for (int n = 0; n < N; n++) acc[n] = fmaf(x, d[n], acc[n]);
            }
        }
    }
    // one split: the sums are the result; several: partial[split][k][n] (row K = the column sums), added up in index order below
    if (k < K) {
        float *p = splits == 1 ? dB + (long long)k * N : partial + ((long long)s * (K + 1) + k) * N;
#pragma unroll
        for (int n = 0; n < N; n++) p[n] = acc[n];
    }
    if (blockIdx.x == 0 && threadIdx.x < N) {
        if (splits > 1) partial[((long long)s * (K + 1) + K) * N + threadIdx.x] = colsum;
        else if (dbias) dbias[threadIdx.x] = colsum;
    }
}

bool skinny_applies(int M, int N, int K, int Nbatch) {
    return rt().precision != 0 && rt().skinny_gemm && N >= 1 && N <= SK_MAXN && K >= 1 && (long long)M * Nbatch < (1ll << 31) &&
           (long long)M * Nbatch * K < (1ll << 40);
}

#define SK_DISPATCH(N, CALL)                                                                          \
    switch (N) {                                                                                      \
        case 1: { constexpr int NN = 1; CALL; } break;   case 2: { constexpr int NN = 2; CALL; } break;   \
        case 3: { constexpr int NN = 3; CALL; } break;   case 4: { constexpr int NN = 4; CALL; } break;   \
        case 5: { constexpr int NN = 5; CALL; } break;   case 6: { constexpr int NN = 6; CALL; } break;   \
        case 7: { constexpr int NN = 7; CALL; } break;   case 8: { constexpr int NN = 8; CALL; } break;   \
        case 9: { constexpr int NN = 9; CALL; } break;   case 10: { constexpr int NN = 10; CALL; } break; \
        case 11: { constexpr int NN = 11; CALL; } break; case 12: { constexpr int NN = 12; CALL; } break; \
        case 13: { constexpr int NN = 13; CALL; } break; case 14: { constexpr int NN = 14; CALL; } break; \
        case 15: { constexpr int NN = 15; CALL; } break; default: { constexpr int NN = 16; CALL; } break; \
    }

int skinny_fwd(const float *A, const float *B, const float *bias, float *C, int rows, int N, int K, int act, const char *name) {
    cudaStream_t st = rt().stream;
    int grid = (rows + 15) / 16;
    if (grid > rt().sm_count * 2) grid = rt().sm_count * 2;
    const size_t smem = (size_t)N * sk_kc(N) * sizeof(float);
    const bool small = (rows + 1) / 2 <= rt().sm_count * 4;             // a block per pair of rows still fits a wave or so
    profile_begin();
    if (small) { SK_DISPATCH(N, (skinny_fwd_small_kernel<NN><<<(rows + 1) / 2, 256, 0, st>>>(A, B, bias, C, rows, K, act))) }
    else
    SK_DISPATCH(N, (skinny_fwd_kernel<NN><<<grid, 256, smem, st>>>(A, B, bias, C, rows, K, act)))
    count_launch();
    profile_end(2.0 * rows * N * (double)K, name);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

int skinny_bwd(const float *A, const float *B, const float *dC, float *dA, float *dB, float *dbias, int rows, int N, int K) {
    cudaStream_t st = rt().stream;
    cudaError_t e = cudaSuccess;
    const int kblocks = (K + 255) / 256;
    int groups = (rt().sm_count * 4 + kblocks - 1) / kblocks;            // about four blocks per SM
    // rows staged at a time: few where the rows are few, so that a small problem still spreads over many blocks (8 ... SK_ROWS)
    int chunk_rows = ((rows + groups - 1) / groups + 7) / 8 * 8;
    if (chunk_rows > SK_ROWS) chunk_rows = SK_ROWS;
    const int chunks = (rows + chunk_rows - 1) / chunk_rows;
    if (groups > chunks) groups = chunks;
    if (groups > 65535) groups = 65535;
    if (dA) {
        profile_begin();
        SK_DISPATCH(N, (skinny_dA_kernel<NN><<<dim3(kblocks, groups), 256, 0, st>>>(dC, B, dA, rows, K, chunk_rows)))
        count_launch();
        profile_end(2.0 * rows * N * (double)K, "cuda_matmul_bwd(dA)");
        e = cudaGetLastError();
    }
    if (e == cudaSuccess && (dB || dbias)) {
        const int splits = groups;
        float *partial = (float *)scratch_alloc((size_t)splits * (K + 1) * N * sizeof(float));
        float *db_out = dB;
        float *tmp = nullptr;
        if (!partial) return SEERA_E_OOM;
        if (!dB) { tmp = (float *)scratch_alloc((size_t)K * N * sizeof(float)); if (!tmp) { scratch_free(partial); return SEERA_E_OOM; } db_out = tmp; }
        profile_begin();
        SK_DISPATCH(N, (skinny_dB_kernel<NN><<<dim3(kblocks, splits), 256, 0, st>>>(A, dC, db_out, dbias, partial, rows, K, chunk_rows)))
        count_launch();
        if (splits > 1) {
            launch_sum_splits(partial, db_out, (K + 1) * N, splits, st, dbias, K * N);
        }
        profile_end(2.0 * rows * N * (double)K, "cuda_matmul_bwd(dB)");
        e = cudaGetLastError();
        scratch_free(partial);
        if (tmp) scratch_free(tmp);
    }
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, "cuda_matmul_bwd");
}

}  // namespace seera
