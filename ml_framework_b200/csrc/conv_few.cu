// Unit-stride convolution / transposed convolution with at most four output channels (the last layer of an
// autoencoder: 32 -> 1 channels).  On the tensor-core path such a layer fills one column of a 32-wide accumulator tile,
// so it pays for 32 columns of MMA issue and for a channels-last copy of its whole input.  It is really a
// memory-bound stencil: each output pixel is a dot product of C*R*S inputs.  Here one thread owns one output pixel,
// the filters sit in shared memory in (channel, tap, filter) order, the input is read in place (NCHW fp32, lanes walk
// the image row, so every load is one coalesced line that the eight neighbouring taps find again in L1) and the
// arithmetic is exact fp32.
//
// Replaces, for this shape, the forward of cuda_conv2DTranpose_fwd (engine_cuda/src/upsampling.cu:376-401: GEMM into a
// column buffer + col2im) followed by the bias broadcast and activation launches.
#include <cuda_runtime.h>

#include "common.cuh"
#include "internal.h"
#include "seera_b200.h"
#include "tc_epilogue.cuh"

namespace seera {

// y[n, f, oh, ow] = act(bias[f] + sum_{c, r, s} x[n, c, oh - PH + r, ow - PW + s] * wk[c][r][s][f])
// wk is filled from W[F][C][R][S] (convolution) or from W[C][F][R][S] read back to front (transposed convolution).
template <int F, int KS>
__global__ void __launch_bounds__(256) conv_few_kernel(const float *__restrict__ x, const float *__restrict__ Wt,
                                                       const float *__restrict__ bias, float *__restrict__ y, int NB, int C, int H,
                                                       int W, int OH, int OW, int Rr, int Sr, int PH, int PW, int act,
                                                       int transposed, FastDiv by_plane, FastDiv by_OW) {
    extern __shared__ float wk[];
    const int R = KS ? KS : Rr, S = KS ? KS : Sr;
    const int taps = R * S, nw = C * taps * F;
    for (int e = threadIdx.x; e < nw; e += blockDim.x) {
        const int f = e % F, k = e / F, c = k / taps, t = k - c * taps;
        const long long src = transposed ? ((long long)c * F + f) * taps + (taps - 1 - t) : ((long long)f * C + c) * taps + t;
        wk[e] = __ldg(Wt + src);
    }
    __syncthreads();
    float b[F];
#pragma unroll
    for (int f = 0; f < F; f++) b[f] = bias ? __ldg(bias + f) : 0.f;
    const int plane = OH * OW;
    const long long total = (long long)NB * plane;
    for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < total; p += (long long)gridDim.x * blockDim.x) {
        const int n = by_plane.div((int)p), rem = (int)(p - (long long)n * plane), oh = by_OW.div(rem), ow = rem - oh * OW;
        float acc[F];
#pragma unroll
        for (int f = 0; f < F; f++) acc[f] = b[f];
        const float *xn = x + (long long)n * C * H * W;
        const int ih0 = oh - PH, iw0 = ow - PW;
        for (int c = 0; c < C; c++) {
            const float *xc = xn + (long long)c * H * W;
            const float *wc = wk + c * taps * F;
#pragma unroll
            for (int r = 0; r < R; r++) {
                const int ih = ih0 + r;
                if ((unsigned)ih >= (unsigned)H) continue;
#pragma unroll
                for (int s = 0; s < S; s++) {
                    const int iw = iw0 + s;
                    if ((unsigned)iw < (unsigned)W) {
                        const float v = __ldg(xc + ih * W + iw);
#pragma unroll
                        for (int f = 0; f < F; f++) acc[f] = fmaf(v, wc[(r * S + s) * F + f], acc[f]);
                    }
                }
            }
        }
#pragma unroll
        for (int f = 0; f < F; f++) y[((long long)n * F + f) * plane + rem] = epilogue_act(acc[f], act);
    }
}

bool conv_few_applies(int NB, int C, int F, int R, int S, int OH, int OW) {
    return (F == 1 || F == 2 || F == 4) && (size_t)C * R * S * F * sizeof(float) <= 40 * 1024 && (long long)NB * OH * OW < (1ll << 31);
}

// Unit stride.  (PH, PW) are the lower paddings of the equivalent convolution: ph, pw for a convolution,
// R - 1 - ph, S - 1 - pw for a transposed one.
int conv_few_fwd(const float *X, const float *Wt, const float *bias, float *Y, int NB, int C, int H, int W, int F, int R, int S, int PH,
                 int PW, int OH, int OW, int act, int transposed, const char *name) {
    const size_t smem = (size_t)C * R * S * F * sizeof(float);
    const long long total = (long long)NB * OH * OW;
    const int grid = stride_grid(total);
    const FastDiv by_plane = fast_div(OH * OW), by_OW = fast_div(OW);
    cudaStream_t st = rt().stream;
    profile_begin();
#define SEERA_FEW(FV, KV) conv_few_kernel<FV, KV><<<grid, 256, smem, st>>>(X, Wt, bias, Y, NB, C, H, W, OH, OW, R, S, PH, PW, act, transposed, by_plane, by_OW)
    const bool k3 = R == 3 && S == 3;
    if (F == 1) { if (k3) SEERA_FEW(1, 3); else SEERA_FEW(1, 0); }
    else if (F == 2) { if (k3) SEERA_FEW(2, 3); else SEERA_FEW(2, 0); }
    else { if (k3) SEERA_FEW(4, 3); else SEERA_FEW(4, 0); }
#undef SEERA_FEW
    count_launch();
    cudaError_t e = cudaGetLastError();
    profile_end(2.0 * total * (double)F * C * R * S);
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

// ---- weight gradient of a convolution with ONE input channel and at most nine taps ----------------------------------
// dW[f][tap] = sum over (n, oh, ow) of dY[n, f, oh, ow] * A[n, 0, oh*sh - ph + r, ow*sw - pw + s]
// (also the weight gradient of a transposed convolution to one channel, with the roles of the two tensors exchanged, which
// is how cuda_conv2DTranspose_bwd calls it).  Per pixel this is 9 * F multiply-adds on 9 + F loaded values: a stencil
// reduction, far below what staging it for the tensor cores costs.  A warp owns four filters (36 running sums per lane)
// and walks 32-pixel tiles, lanes = consecutive pixels, so the F-channel tensor is read in place, once, in coalesced lines
// and the nine one-channel neighbours come from L1.  Sums are reduced in a fixed order (lanes by shuffle tree, then
// warps by a second kernel), so the result is deterministic.
constexpr int C1_FPW = 4;                // filters per warp
constexpr int C1_TAPS = 9;

__global__ void __launch_bounds__(256) wgrad_c1_kernel(const float *__restrict__ A, const float *__restrict__ dY, float *__restrict__ partial,
                                                       int NB, int H, int W, int F, int OH, int OW, int R, int S, int sh, int sw, int ph,
                                                       int pw, int ngroups, FastDiv by_plane, FastDiv by_OW, FastDiv by_S) {
    const int lane = threadIdx.x & 31;
    const int gw = blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = gridDim.x * 8;          // gridDim.x is a multiple of ngroups
    const int g = gw % ngroups, f0 = g * C1_FPW, taps = R * S;
    const int plane = OH * OW;
    const long long total = (long long)NB * plane;
    const long long tiles = (total + 31) / 32;
    float acc[C1_FPW][C1_TAPS];
#pragma unroll
    for (int i = 0; i < C1_FPW; i++)
#pragma unroll
        for (int t = 0; t < C1_TAPS; t++) acc[i][t] = 0.f;
    // tap -> (r, s), the same for every pixel
    int tr[C1_TAPS], ts[C1_TAPS];
#pragma unroll
    for (int t = 0; t < C1_TAPS; t++) { tr[t] = by_S.div(t); ts[t] = t - tr[t] * S; }
    for (long long tile = gw / ngroups; tile < tiles; tile += nwarps / ngroups) {
        const long long p = tile * 32 + lane;
        if (p < total) {
            const int n = by_plane.div((int)p), rem = (int)(p - (long long)n * plane), oh = by_OW.div(rem), ow = rem - oh * OW;
            const float *a = A + (long long)n * H * W;
            const int ih0 = oh * sh - ph, iw0 = ow * sw - pw;
            float av[C1_TAPS];
#pragma unroll
            for (int t = 0; t < C1_TAPS; t++) {
                const int ih = ih0 + tr[t], iw = iw0 + ts[t];
                av[t] = (t < taps && (unsigned)ih < (unsigned)H && (unsigned)iw < (unsigned)W) ? __ldg(a + ih * W + iw) : 0.f;
            }
#pragma unroll
            for (int i = 0; i < C1_FPW; i++) {
                const float d = f0 + i < F ? __ldg(dY + ((long long)n * F + f0 + i) * plane + rem) : 0.f;
#pragma unroll
                for (int t = 0; t < C1_TAPS; t++) acc[i][t] = fmaf(d, av[t], acc[i][t]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < C1_FPW; i++)
#pragma unroll
        for (int t = 0; t < C1_TAPS; t++) {
            float v = acc[i][t];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) partial[(long long)gw * (C1_FPW * C1_TAPS) + i * C1_TAPS + t] = v;
        }
}

// dW[f][t] = sum over the warps of group f / 4, in warp order: one warp per output, lanes stride over the group's warps.
__global__ void __launch_bounds__(256) wgrad_c1_reduce_kernel(const float *__restrict__ partial, float *__restrict__ dW, int F, int taps,
                                                              int ngroups, int nwarps) {
    const int lane = threadIdx.x & 31, o = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (o >= F * taps) return;
    const int f = o / taps, t = o - f * taps, g = f / C1_FPW, i = f - g * C1_FPW;
    float v = 0.f;
    for (int w = g + lane * ngroups; w < nwarps; w += 32 * ngroups) v += partial[(long long)w * (C1_FPW * C1_TAPS) + i * C1_TAPS + t];
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    if (lane == 0) dW[o] = v;
}

bool wgrad_c1_applies(int NB, int C, int F, int R, int S, int OH, int OW) {
    return C == 1 && R * S <= C1_TAPS && F >= 1 && (long long)NB * OH * OW < (1ll << 31);
}

int wgrad_c1(const float *A, const float *dY, float *dW, int NB, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw,
             const char *name) {
    const int OH = (H + 2 * ph - R) / sh + 1, OW = (W + 2 * pw - S) / sw + 1;
    const int ngroups = (F + C1_FPW - 1) / C1_FPW;
    const long long tiles = ((long long)NB * OH * OW + 31) / 32;
    // about four resident blocks per SM, rounded to a multiple of the group count; no more warps per group than tiles
    int blocks = rt().sm_count * 4 / ngroups;
    const long long need = (tiles + 7) / 8;
    if (blocks > need) blocks = (int)need;
    if (blocks < 1) blocks = 1;
    blocks *= ngroups;
    const int nwarps = blocks * 8;
    float *partial = (float *)scratch_alloc((size_t)nwarps * C1_FPW * C1_TAPS * sizeof(float));
    if (!partial) return SEERA_E_OOM;
    cudaStream_t st = rt().stream;
    profile_begin();
    wgrad_c1_kernel<<<blocks, 256, 0, st>>>(A, dY, partial, NB, H, W, F, OH, OW, R, S, sh, sw, ph, pw, ngroups, fast_div(OH * OW), fast_div(OW),
                                            fast_div(S));
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) {
        wgrad_c1_reduce_kernel<<<(F * R * S + 7) / 8, 256, 0, st>>>(partial, dW, F, R * S, ngroups, nwarps);
        count_launch();
        e = cudaGetLastError();
    }
    profile_end(2.0 * NB * OH * OW * (double)F * R * S);
    scratch_free(partial);
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

}  // namespace seera
