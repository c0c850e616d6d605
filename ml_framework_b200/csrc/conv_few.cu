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

}  // namespace seera
