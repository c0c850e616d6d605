// fp32 CUDA-core contraction kernel behind Dense and the convolution family (precision mode 0), and the
// exact-fp32 reference for the tensor-core paths.
//
// One tiled kernel, C[M,N] = sum_k A(m,k) * B(k,n), whose operands are *functors*: the tile loaders ask
// the functor for element (m,k) / (k,n), so the same main loop serves
//   Dense forward / dA / dB             (engine_cuda/src/GEMM.cu:13-225; no materialised transposes, the batch
//                                        folds into the M or K extent because B is shared by all batches)
//   Conv2D forward, "fprop"             (engine_cuda/src/convolution.cu:15-101) im2col formed on the fly
//   Conv2D dX, "dgrad"                  (convolution.cu:144-265) gather form of col2im, no column scratch
//   Conv2D dW, "wgrad"                  (convolution.cu:268-366, :103-120) contraction over batch*pixels, split-K
//   ConvTranspose2D forward = dgrad, dX = fprop, dW = wgrad with the operand roles exchanged
//                                       (engine_cuda/src/upsampling.cu:15-401)
// The arithmetic is the CPU engine's (engine/src/conv_ops.cpp:95-287): dW is the SUM over the batch, padding
// taps contribute zero, Hout = (H-1)*stride - 2*pad + KH for the transposed convolution.
//
// Tile: BM x 128 x 16, 256 threads as 16x16, each thread (BM/16) x 8 outputs, register-staged global loads
// overlapped with the FMA loop.  Split-K writes fp32 partials [splits, M, N] to pooled scratch and a second
// kernel adds them in split order, so results are run-to-run deterministic.
#include "common.cuh"
#include "contraction_functors.cuh"

namespace seera {

constexpr int BN = 128, BK = 16, NT = 256;

// ---- the kernel -------------------------------------------------------------------------------------------------
// A_MFAST: adjacent threads load adjacent m (operand contiguous along m) instead of adjacent k.
// B_KFAST: adjacent threads load adjacent k (operand contiguous along k) instead of adjacent n.
template <int BM, bool A_MFAST, bool B_KFAST, class AL, class BL, class CS>
__global__ void __launch_bounds__(NT) contraction_kernel(AL al, BL bl, CS cs, float *__restrict__ partial,
                                                         int M, int N, int K, int kchunk) {
    constexpr int TM = BM / 16, PA = BM + 4, PB = BN + 4;
    __shared__ __align__(16) float As[BK][PA];
    __shared__ __align__(16) float Bs[BK][PB];
    const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int kbeg = blockIdx.z * kchunk, kend = min(K, kbeg + kchunk);

    // per-thread load assignments
    typename AL::Fx afx[A_MFAST ? 1 : TM];
    int a_m[A_MFAST ? 1 : TM], a_k[A_MFAST ? TM : 1];
    if (A_MFAST) {
        a_m[0] = t % BM; afx[0] = al.fix(m0 + a_m[0]);
#pragma unroll
        for (int i = 0; i < TM; i++) a_k[i] = t / BM + (NT / BM) * i;
    } else {
        a_k[0] = t & 15;
#pragma unroll
        for (int i = 0; i < TM; i++) { a_m[i] = (t >> 4) + 16 * i; afx[i] = al.fix(m0 + a_m[i]); }
    }
    typename BL::Fx bfx[B_KFAST ? 8 : 1];
    int b_n[B_KFAST ? 8 : 1], b_k[B_KFAST ? 1 : 8];
    if (B_KFAST) {
        b_k[0] = t & 15;
#pragma unroll
        for (int i = 0; i < 8; i++) { b_n[i] = (t >> 4) + 16 * i; bfx[i] = bl.fix(n0 + b_n[i]); }
    } else {
        b_n[0] = t & 127; bfx[0] = bl.fix(n0 + b_n[0]);
#pragma unroll
        for (int i = 0; i < 8; i++) b_k[i] = (t >> 7) + 2 * i;
    }

    float acc[TM][8];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.f;

    float ra[TM], rb[8];
    auto gload = [&](int k0) {
#pragma unroll
        for (int i = 0; i < TM; i++) {
            int kk = k0 + (A_MFAST ? a_k[i] : a_k[0]);
            ra[i] = kk < kend ? al.load(A_MFAST ? afx[0] : afx[i], kk) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            int kk = k0 + (B_KFAST ? b_k[0] : b_k[i]);
            rb[i] = kk < kend ? bl.load(B_KFAST ? bfx[i] : bfx[0], kk) : 0.f;
        }
    };

    if (kbeg < kend) gload(kbeg);
    for (int k0 = kbeg; k0 < kend; k0 += BK) {
#pragma unroll
        for (int i = 0; i < TM; i++) As[A_MFAST ? a_k[i] : a_k[0]][A_MFAST ? a_m[0] : a_m[i]] = ra[i];
#pragma unroll
        for (int i = 0; i < 8; i++) Bs[B_KFAST ? b_k[0] : b_k[i]][B_KFAST ? b_n[i] : b_n[0]] = rb[i];
        __syncthreads();
        if (k0 + BK < kend) gload(k0 + BK);
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[TM], b[8];
#pragma unroll
            for (int i = 0; i < TM; i++) a[i] = As[kk][ty * TM + i];
            float4 b0 = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
            float4 b1 = *reinterpret_cast<const float4 *>(&Bs[kk][64 + tx * 4]);
            b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w; b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; i++) {
        int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (n >= N) continue;
            if (partial) partial[((long long)blockIdx.z * M + m) * N + n] = acc[i][j];
            else cs(m, n, acc[i][j]);
        }
    }
}

template <class CS>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ partial, CS cs, int M, int N, int splits) {
    long long total = (long long)M * N;
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long i = tid; i < total; i += nthr) {
        float s = 0.f;
        for (int z = 0; z < splits; z++) s += partial[(long long)z * total + i];
        cs((int)(i / N), (int)(i % N), s);
    }
}

// Chooses BM and the split count, allocates partials from the pool when splitting, launches.
template <bool A_MFAST, bool B_KFAST, class AL, class BL, class CS>
int run_contraction(const AL &al, const BL &bl, const CS &cs, int M, int N, int K, bool allow_split, const char *name) {
    if (M < 1 || N < 1 || K < 1) return fail(SEERA_E_ARG, "%s: empty problem %dx%dx%d", name, M, N, K);
    int bm = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
    long long tiles = (long long)((M + bm - 1) / bm) * ((N + BN - 1) / BN);
    int splits = 1;
    if (allow_split) {
        long long want = (2LL * rt().sm_count + tiles - 1) / tiles;
        long long maxs = K / (BK * 8);
        splits = (int)(want < maxs ? want : maxs);
        if (splits < 1) splits = 1;
        if (splits > 512) splits = 512;
    }
    int kchunk = ((K + splits - 1) / splits + BK - 1) / BK * BK;
    splits = (K + kchunk - 1) / kchunk;
    float *partial = nullptr;
    if (splits > 1) {
        partial = (float *)scratch_alloc((size_t)splits * M * N * sizeof(float));
        if (!partial) return SEERA_E_OOM;
    }
    dim3 grid((N + BN - 1) / BN, (M + bm - 1) / bm, splits);
    if (grid.y > 65535 || grid.z > 65535) { if (partial) scratch_free(partial); return fail(SEERA_E_LIMIT, "%s: grid too large", name); }
    cudaStream_t st = rt().stream;
    profile_begin();
    if (bm == 32) contraction_kernel<32, A_MFAST, B_KFAST><<<grid, NT, 0, st>>>(al, bl, cs, partial, M, N, K, kchunk);
    else if (bm == 64) contraction_kernel<64, A_MFAST, B_KFAST><<<grid, NT, 0, st>>>(al, bl, cs, partial, M, N, K, kchunk);
    else contraction_kernel<128, A_MFAST, B_KFAST><<<grid, NT, 0, st>>>(al, bl, cs, partial, M, N, K, kchunk);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && partial) {
        splitk_reduce_kernel<<<stride_grid((long long)M * N), 256, 0, st>>>(partial, cs, M, N, splits);
        count_launch();
        e = cudaGetLastError();
    }
    if (partial) scratch_free(partial);
    profile_end(2.0 * M * N * (double)K, name);
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

// ---- the three convolution forms on explicit geometry ---------------------------------------------------------
// fprop:  Y[img,F,OH,OW] = conv(X[img,C,H,W], Wt[F,C,R,S])
int simt_conv_fprop(const float *X, const float *Wt, float *Y, int NB, int C, int H, int W, int F, int R, int S,
                    int sh, int sw, int ph, int pw, const char *name) {
    int OH = (H + 2 * ph - R) / sh + 1, OW = (W + 2 * pw - S) / sw + 1;
    if (OH < 1 || OW < 1) return fail(SEERA_E_ARG, "%s: kernel larger than padded input", name);
    int K = C * R * S, ncols = NB * OH * OW;
    ConvGeom g{C, H, W, OH, OW, R, S, sh, sw, ph, pw};
    Strided a{Wt, K, 1, F, K};
    StoreNCHW cs{Y, F, OH * OW};
    if (R == 3 && S == 3) return run_contraction<false, false>(a, Im2colByCol<9, 3>{X, g, ncols, K}, cs, F, ncols, K, false, name);
    return run_contraction<false, false>(a, Im2colByCol<0, 0>{X, g, ncols, K}, cs, F, ncols, K, false, name);
}

// dgrad:  dX[img,C,H,W] = sum_{f,r,s} dY[img,f,(h+ph-r)/sh,(w+pw-s)/sw] * Wt[f,c,r,s];  dY is [img,F,OH,OW]
int simt_conv_dgrad(const float *dY, const float *Wt, float *dX, int NB, int C, int H, int W, int F, int R, int S,
                    int sh, int sw, int ph, int pw, int OH, int OW, const char *name) {
    int K = F * R * S, ncols = NB * H * W;
    ConvGeom g{F, OH, OW, H, W, R, S, sh, sw, ph, pw};
    WeightByInChannel a{Wt, C, R * S, K};
    StoreNCHW cs{dX, C, H * W};
    if (R == 3 && S == 3) return run_contraction<false, false>(a, Col2imByPixel<9, 3>{dY, g, ncols, K}, cs, C, ncols, K, false, name);
    return run_contraction<false, false>(a, Col2imByPixel<0, 0>{dY, g, ncols, K}, cs, C, ncols, K, false, name);
}

// wgrad:  dW[F, C*R*S] = sum_{img,p} dY[img,f,p] * im2col(X)[img,(c,r,s),p];  dY is [img,F,OH,OW], X is [img,C,H,W]
int simt_conv_wgrad(const float *dY, const float *X, float *dW, int NB, int C, int H, int W, int F, int R, int S,
                    int sh, int sw, int ph, int pw, int OH, int OW, const char *name) {
    int K = NB * OH * OW, ncols = C * R * S;
    ConvGeom g{C, H, W, OH, OW, R, S, sh, sw, ph, pw};
    ByImagePixel a{dY, F, OH * OW, K};
    Im2colByTap b{X, g, ncols, K};
    StoreDense cs{dW, ncols};
    return run_contraction<false, true>(a, b, cs, F, ncols, K, true, name);
}

__global__ void __launch_bounds__(256) transpose_kernel(const float *__restrict__ in, float *__restrict__ out, int rows, int cols) {
    __shared__ float tile[32][33];
    const float *ib = in + (long long)blockIdx.z * rows * cols;
    float *ob = out + (long long)blockIdx.z * rows * cols;
    int c = blockIdx.x * 32 + (threadIdx.x & 31), r0 = blockIdx.y * 32;
    for (int i = threadIdx.x >> 5; i < 32; i += 8)
        if (r0 + i < rows && c < cols) tile[i][threadIdx.x & 31] = ib[(long long)(r0 + i) * cols + c];
    __syncthreads();
    int r = r0 + (threadIdx.x & 31), c0 = blockIdx.x * 32;
    for (int i = threadIdx.x >> 5; i < 32; i += 8)
        if (c0 + i < cols && r < rows) ob[(long long)(c0 + i) * rows + r] = tile[threadIdx.x & 31][i];
}

}  // namespace seera

using namespace seera;

extern "C" {

int seera_simt_matmul(const float *A, const float *B, float *C, int M, int N, int K, int Nbatch) {
    SEERA_ENSURE();
    if (M < 1 || N < 1 || K < 1 || Nbatch < 1 || !A || !B || !C) return fail(SEERA_E_ARG, "cuda_matmul: bad argument");
    long long rows = (long long)M * Nbatch;
    if (rows > 0x7fffffff) return fail(SEERA_E_LIMIT, "cuda_matmul: batch*M too large");
    Strided a{A, K, 1, (int)rows, K}, b{B, 1, N, N, K};
    return run_contraction<false, false>(a, b, StoreDense{C, N}, (int)rows, N, K, false, "cuda_matmul");
}

int seera_simt_matmul_bwd(const float *A, const float *B, const float *dC, float *dA, float *dB, int M, int N, int K, int Nbatch) {
    SEERA_ENSURE();
    if (M < 1 || N < 1 || K < 1 || Nbatch < 1 || !A || !B || !dC) return fail(SEERA_E_ARG, "cuda_matmul_bwd: bad argument");
    long long rows = (long long)M * Nbatch;
    if (rows > 0x7fffffff) return fail(SEERA_E_LIMIT, "cuda_matmul_bwd: batch*M too large");
    if (dA) {   // dA[rows,K] = dC[rows,N] * B^T : contraction over N; B^T(k'=n, j=k) = B[k*N + n] is contiguous along n
        Strided a{dC, N, 1, (int)rows, N}, b{B, N, 1, K, N};
        if (int s = run_contraction<false, true>(a, b, StoreDense{dA, K}, (int)rows, K, N, false, "cuda_matmul_bwd(dA)")) return s;
    }
    if (dB) {   // dB[K,N] = A^T[K,rows] * dC[rows,N] : contraction over rows; A^T(m=k, k'=row) = A[row*K + k] contiguous along m
        Strided a{A, 1, K, K, (int)rows}, b{dC, 1, N, N, (int)rows};
        if (int s = run_contraction<true, false>(a, b, StoreDense{dB, N}, K, N, (int)rows, true, "cuda_matmul_bwd(dB)")) return s;
    }
    return SEERA_OK;
}

int seera_cuda_transpose_2d(const float *in, float *out, int rows, int cols) { return seera_cuda_transpose_3d(in, out, 1, rows, cols); }
int seera_cuda_transpose_3d(const float *in, float *out, int Nbatch, int M, int K) {
    SEERA_ENSURE();
    if (Nbatch < 1 || M < 1 || K < 1 || !in || !out || Nbatch > 65535) return fail(SEERA_E_ARG, "cuda_transpose: bad argument");
    dim3 grid((K + 31) / 32, (M + 31) / 32, Nbatch);
    if (grid.y > 65535) return fail(SEERA_E_LIMIT, "cuda_transpose: too many rows");
    transpose_kernel<<<grid, 256, 0, rt().stream>>>(in, out, M, K);
    SEERA_LAUNCH_CHECK("cuda_transpose");
    return SEERA_OK;
}

static bool conv_args_ok(int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw) {
    return NB >= 1 && C >= 1 && H >= 1 && W >= 1 && F >= 1 && R >= 1 && S >= 1 && sh >= 1 && sw >= 1 && ph >= 0 && pw >= 0 &&
           (long long)NB * (C > F ? C : F) * H * W * (long long)(sh * sw) < (1LL << 31);
}

int seera_simt_conv2d_fwd(const float *X, const float *Wt, float *Y, int NB, int C, int H, int W, int F, int R, int S,
                          int ph, int pw, int sh, int sw) {
    SEERA_ENSURE();
    if (!conv_args_ok(NB, C, H, W, F, R, S, sh, sw, ph, pw) || !X || !Wt || !Y) return fail(SEERA_E_ARG, "cuda_conv2d_fwd: bad argument");
    return simt_conv_fprop(X, Wt, Y, NB, C, H, W, F, R, S, sh, sw, ph, pw, "cuda_conv2d_fwd");
}

int seera_simt_conv2d_bwd(const float *Wt, const float *X, const float *dY, float *dX, float *dW, int NB, int C, int H, int W,
                          int F, int R, int S, int sh, int sw, int ph, int pw) {
    SEERA_ENSURE();
    if (!conv_args_ok(NB, C, H, W, F, R, S, sh, sw, ph, pw) || !X || !Wt || !dY) return fail(SEERA_E_ARG, "cuda_conv2d_bwd: bad argument");
    int OH = (H + 2 * ph - R) / sh + 1, OW = (W + 2 * pw - S) / sw + 1;
    if (OH < 1 || OW < 1) return fail(SEERA_E_ARG, "cuda_conv2d_bwd: kernel larger than padded input");
    if (dX) if (int s = simt_conv_dgrad(dY, Wt, dX, NB, C, H, W, F, R, S, sh, sw, ph, pw, OH, OW, "cuda_conv2d_bwd(dX)")) return s;
    if (dW) if (int s = simt_conv_wgrad(dY, X, dW, NB, C, H, W, F, R, S, sh, sw, ph, pw, OH, OW, "cuda_conv2d_bwd(dW)")) return s;
    return SEERA_OK;
}

// Transposed convolution: X[NB,Cin,H,W], Wt[Cin,Cout,KH,KW], out[NB,Cout,Ho,Wo].  With the weight read as a
// convolution filter bank of Cin filters over Cout channels, the forward pass is that convolution's data
// gradient, dX is its forward pass applied to dY, and dW is its weight gradient with X in the dY role.
int seera_simt_convT_fwd(const float *X, const float *Wt, float *out, int NB, int Cin, int H, int W, int Cout, int KH, int KW,
                         int sh, int sw, int ph, int pw) {
    SEERA_ENSURE();
    int Ho = (H - 1) * sh - 2 * ph + KH, Wo = (W - 1) * sw - 2 * pw + KW;
    if (!conv_args_ok(NB, Cin, H, W, Cout, KH, KW, sh, sw, ph, pw) || Ho < 1 || Wo < 1 || !X || !Wt || !out)
        return fail(SEERA_E_ARG, "cuda_conv2DTranpose_fwd: bad argument");
    return simt_conv_dgrad(X, Wt, out, NB, Cout, Ho, Wo, Cin, KH, KW, sh, sw, ph, pw, H, W, "cuda_conv2DTranpose_fwd");
}

int seera_simt_convT_bwd(const float *Wt, const float *X, const float *dY, float *dX, float *dW, int NB, int Cin, int H, int W,
                         int Cout, int KH, int KW, int sh, int sw, int ph, int pw) {
    SEERA_ENSURE();
    int Ho = (H - 1) * sh - 2 * ph + KH, Wo = (W - 1) * sw - 2 * pw + KW;
    if (!conv_args_ok(NB, Cin, H, W, Cout, KH, KW, sh, sw, ph, pw) || Ho < 1 || Wo < 1 || !X || !Wt || !dY)
        return fail(SEERA_E_ARG, "cuda_conv2DTranspose_bwd: bad argument");
    if ((Ho + 2 * ph - KH) / sh + 1 != H || (Wo + 2 * pw - KW) / sw + 1 != W)
        return fail(SEERA_E_ARG, "cuda_conv2DTranspose_bwd: inconsistent geometry");
    if (dX) if (int s = simt_conv_fprop(dY, Wt, dX, NB, Cout, Ho, Wo, Cin, KH, KW, sh, sw, ph, pw, "cuda_conv2DTranspose_bwd(dX)")) return s;
    if (dW) if (int s = simt_conv_wgrad(X, dY, dW, NB, Cout, Ho, Wo, Cin, KH, KW, sh, sw, ph, pw, H, W, "cuda_conv2DTranspose_bwd(dW)")) return s;
    return SEERA_OK;
}

}  // extern "C"
