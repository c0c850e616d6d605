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

// 3 x 3 filters: one thread owns FOUR consecutive pixels of an output row.  Per channel and filter row it loads the six
// inputs those pixels share (column validity is worked out once per thread, row validity once per row) and keeps the
// channel's nine weights per filter in registers: about a fifth of the instructions per output of the kernel above,
// which is instruction-bound.
template <int F>
__global__ void __launch_bounds__(256) conv_few3x3_kernel(const float *__restrict__ x, const float *__restrict__ Wt,
                                                          const float *__restrict__ bias, float *__restrict__ y, int NB, int C, int H,
                                                          int W, int OH, int OW, int PH, int PW, int act, int transposed,
                                                          FastDiv by_rowq, FastDiv by_OWq) {
    extern __shared__ float wk[];
    const int nw = C * 9 * F;
    for (int e = threadIdx.x; e < nw; e += blockDim.x) {
        const int f = e % F, k = e / F, c = k / 9, t = k - c * 9;
        const long long src = transposed ? ((long long)c * F + f) * 9 + (8 - t) : ((long long)f * C + c) * 9 + t;
        wk[e] = __ldg(Wt + src);
    }
    __syncthreads();
    float b[F];
#pragma unroll
    for (int f = 0; f < F; f++) b[f] = bias ? __ldg(bias + f) : 0.f;
    const int OWq = (OW + 3) >> 2, rowq = OH * OWq;              // items per row / per image
    const long long total = (long long)NB * rowq;
    const long long plane = (long long)OH * OW;
    for (long long it = (long long)blockIdx.x * blockDim.x + threadIdx.x; it < total; it += (long long)gridDim.x * blockDim.x) {
        const int n = by_rowq.div((int)it), rem = (int)(it - (long long)n * rowq), oh = by_OWq.div(rem), ow0 = (rem - oh * OWq) * 4;
        const int iw0 = ow0 - PW, ih0 = oh - PH;
        bool colok[6], rowok[3];
#pragma unroll
        for (int j = 0; j < 6; j++) colok[j] = (unsigned)(iw0 + j) < (unsigned)W;
#pragma unroll
        for (int r = 0; r < 3; r++) rowok[r] = (unsigned)(ih0 + r) < (unsigned)H;
        float acc[F][4];
#pragma unroll
        for (int f = 0; f < F; f++)
#pragma unroll
            for (int q = 0; q < 4; q++) acc[f][q] = b[f];
        const float *xp = x + (long long)n * C * H * W + (long long)ih0 * W + iw0;
        for (int c = 0; c < C; c++, xp += (long long)H * W) {
            float w[9][F];
#pragma unroll
            for (int t = 0; t < 9; t++)
#pragma unroll
                for (int f = 0; f < F; f++) w[t][f] = wk[(c * 9 + t) * F + f];
#pragma unroll
            for (int r = 0; r < 3; r++) {
                if (!rowok[r]) continue;
                float v[6];
#pragma unroll
                for (int j = 0; j < 6; j++) v[j] = colok[j] ? __ldg(xp + r * W + j) : 0.f;
#pragma unroll
                for (int s = 0; s < 3; s++)
#pragma unroll
                    for (int q = 0; q < 4; q++)
#pragma unroll
                        for (int f = 0; f < F; f++) acc[f][q] = fmaf(v[q + s], w[r * 3 + s][f], acc[f][q]);
            }
        }
#pragma unroll
        for (int f = 0; f < F; f++) {
            float *yo = y + ((long long)n * F + f) * plane + (long long)oh * OW + ow0;
#pragma unroll
            for (int q = 0; q < 4; q++)
                if (ow0 + q < OW) yo[q] = epilogue_act(acc[f][q], act);
        }
    }
}

// The usual case of that kernel, a "same" 3 x 3 filter (left padding 1, output as wide as the input, width a multiple of
// four): a lane reads its four inputs of a row as ONE 16-byte vector and gets the two outer columns from its neighbours
// by shuffle (lanes 0 and 31 load theirs).  The scalar form issues six loads per row that each use a quarter of the
// sectors they touch and is bound by L1 wavefronts; this one is bound by HBM.
template <int F>
__global__ void __launch_bounds__(256) conv_few3x3v_kernel(const float *__restrict__ x, const float *__restrict__ Wt,
                                                           const float *__restrict__ bias, float *__restrict__ y, int NB, int C, int H,
                                                           int W, int OH, int PH, int act, int transposed, FastDiv by_rowq,
                                                           FastDiv by_OWq) {
    extern __shared__ float wk[];
    const int nw = C * 9 * F;
    for (int e = threadIdx.x; e < nw; e += blockDim.x) {
        const int f = e % F, k = e / F, c = k / 9, t = k - c * 9;
        const long long src = transposed ? ((long long)c * F + f) * 9 + (8 - t) : ((long long)f * C + c) * 9 + t;
        wk[e] = __ldg(Wt + src);
    }
    __syncthreads();
    float b[F];
#pragma unroll
    for (int f = 0; f < F; f++) b[f] = bias ? __ldg(bias + f) : 0.f;
    const int lane = threadIdx.x & 31;
    const int OWq = W >> 2, rowq = OH * OWq;
    const long long total = (long long)NB * rowq;
    const long long plane = (long long)OH * W;
    // warp-uniform loop: every lane stays in it (the shuffles need all 32), lanes past the end compute on item 0 and store nothing
    for (long long base = ((long long)blockIdx.x * blockDim.x + threadIdx.x) - lane; base < total; base += (long long)gridDim.x * blockDim.x) {
        const bool live = base + lane < total;
        const int it = live ? (int)(base + lane) : 0;
        const int n = by_rowq.div(it), rem = it - n * rowq, oh = by_OWq.div(rem), ow0 = (rem - oh * OWq) * 4;
        const int ih0 = oh - PH;
        bool rowok[3];
#pragma unroll
        for (int r = 0; r < 3; r++) rowok[r] = (unsigned)(ih0 + r) < (unsigned)H;
        const bool has_left = ow0 > 0, has_right = ow0 + 4 < W;
        float acc[F][4];
#pragma unroll
        for (int f = 0; f < F; f++)
#pragma unroll
            for (int q = 0; q < 4; q++) acc[f][q] = b[f];
        const float *xp = x + (long long)n * C * H * W + (long long)ih0 * W + ow0;
        // Channels go in groups of four: all twelve row vectors of a group (and the edge lanes' outer columns) are requested
        // before the first is used.  One channel at a time, every channel costs the thread a full trip to HBM.
        constexpr int CG = 4;
        for (int c0 = 0; c0 < C; c0 += CG, xp += (long long)CG * H * W) {
            float4 m[CG][3];
            float edge[CG][3];
#pragma unroll
            for (int k = 0; k < CG; k++)
#pragma unroll
                for (int r = 0; r < 3; r++) {
                    const bool ok = rowok[r] && c0 + k < C;
                    const float *row = xp + (long long)k * H * W + r * W;
                    m[k][r] = ok ? __ldg(reinterpret_cast<const float4 *>(row)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    edge[k][r] = (ok && lane == 0 && has_left) ? __ldg(row - 1) : ((ok && lane == 31 && has_right) ? __ldg(row + 4) : 0.f);
                }
#pragma unroll
            for (int k = 0; k < CG; k++) {
                const int c = min(c0 + k, C - 1);                 // past the last channel the inputs are zero: any weights do
                float w[9][F];
#pragma unroll
                for (int t = 0; t < 9; t++)
#pragma unroll
                    for (int f = 0; f < F; f++) w[t][f] = wk[(c * 9 + t) * F + f];
#pragma unroll
                for (int r = 0; r < 3; r++) {
                    float left = __shfl_up_sync(0xffffffffu, m[k][r].w, 1), right = __shfl_down_sync(0xffffffffu, m[k][r].x, 1);
                    if (lane == 0) left = edge[k][r];
                    if (lane == 31) right = edge[k][r];
                    if (!has_left) left = 0.f;
                    if (!has_right) right = 0.f;
                    const float v[6] = {left, m[k][r].x, m[k][r].y, m[k][r].z, m[k][r].w, right};
#pragma unroll
                    for (int s = 0; s < 3; s++)
#pragma unroll
                        for (int q = 0; q < 4; q++)
#pragma unroll
                            for (int f = 0; f < F; f++) acc[f][q] = fmaf(v[q + s], w[r * 3 + s][f], acc[f][q]);
                }
            }
        }
        if (live) {
#pragma unroll
            for (int f = 0; f < F; f++)
                *reinterpret_cast<float4 *>(y + ((long long)n * F + f) * plane + (long long)oh * W + ow0) =
                    make_float4(epilogue_act(acc[f][0], act), epilogue_act(acc[f][1], act), epilogue_act(acc[f][2], act),
                                epilogue_act(acc[f][3], act));
        }
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
    if (R == 3 && S == 3 && PW == 1 && OW == W && (W & 3) == 0 && ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(Y)) & 15) == 0) {
        const int grid4 = stride_grid((long long)NB * OH * (W / 4));
        const FastDiv by_rowq = fast_div(OH * (W / 4)), by_OWq = fast_div(W / 4);
#define SEERA_FEW3V(FV) conv_few3x3v_kernel<FV><<<grid4, 256, smem, st>>>(X, Wt, bias, Y, NB, C, H, W, OH, PH, act, transposed, by_rowq, by_OWq)
        if (F == 1) SEERA_FEW3V(1); else if (F == 2) SEERA_FEW3V(2); else SEERA_FEW3V(4);
#undef SEERA_FEW3V
        count_launch();
        cudaError_t e3 = cudaGetLastError();
        profile_end(2.0 * total * (double)F * C * R * S, name);
        return e3 == cudaSuccess ? SEERA_OK : check_cuda(e3, name);
    }
    if (R == 3 && S == 3) {
        const int OWq = (OW + 3) / 4;
        const int grid4 = stride_grid((long long)NB * OH * OWq);
        const FastDiv by_rowq = fast_div(OH * OWq), by_OWq = fast_div(OWq);
#define SEERA_FEW3(FV) conv_few3x3_kernel<FV><<<grid4, 256, smem, st>>>(X, Wt, bias, Y, NB, C, H, W, OH, OW, PH, PW, act, transposed, by_rowq, by_OWq)
        if (F == 1) SEERA_FEW3(1); else if (F == 2) SEERA_FEW3(2); else SEERA_FEW3(4);
#undef SEERA_FEW3
        count_launch();
        cudaError_t e3 = cudaGetLastError();
        profile_end(2.0 * total * (double)F * C * R * S, name);
        return e3 == cudaSuccess ? SEERA_OK : check_cuda(e3, name);
    }
#define SEERA_FEW(FV, KV) conv_few_kernel<FV, KV><<<grid, 256, smem, st>>>(X, Wt, bias, Y, NB, C, H, W, OH, OW, R, S, PH, PW, act, transposed, by_plane, by_OW)
    if (F == 1) SEERA_FEW(1, 0); else if (F == 2) SEERA_FEW(2, 0); else SEERA_FEW(4, 0);
#undef SEERA_FEW
    count_launch();
    cudaError_t e = cudaGetLastError();
    profile_end(2.0 * total * (double)F * C * R * S, name);
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

// ---- 3 x 3 unit-stride convolution with a few input channels + bias + activation + 2x2 / stride-2 max-pool ------------------
// The first layer of an image network (3 -> 64 channels): 27 multiply-adds per output, which the tensor-core path can only
// reach by gathering and splitting patches in producer warps.  Here a lane owns one pool window (2 x 2 outputs, a 4 x 4 input
// patch per channel, read once with row / column validity worked out once) and a warp owns eight filters, whose 72 weights
// per channel come from shared memory as broadcast 16-byte reads.  The layer output is never stored: pooled values, the
// window-local argmax (scan order (0,0), (0,1), (1,0), (1,1), strict comparison: the first maximum wins, as in
// cuda_maxpool_fwd) and the channels-last bf16 copies of the pooled tensor for the next convolution are.  Exact fp32.
__global__ void __launch_bounds__(256, 3) conv3x3_pool_kernel(const float *__restrict__ x, const float *__restrict__ Wt,
                                                           const float *__restrict__ bias, PoolOut po, int NB, int C, int H, int W,
                                                           int F, int OH, int OW, int ph, int pw, int act, FastDiv by_Pq,
                                                           FastDiv by_OWq) {
    extern __shared__ float wk[];                         // [C][9][F], then [F] biases
    for (int e = threadIdx.x; e < C * 9 * F; e += blockDim.x) {
        const int f = e % F, k = e / F;                   // k = c * 9 + t
        wk[e] = __ldg(Wt + (long long)f * C * 9 + k);
    }
    for (int e = threadIdx.x; e < F; e += blockDim.x) wk[C * 9 * F + e] = bias ? __ldg(bias + e) : 0.f;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int OWq = OW >> 1, Pq = (OH >> 1) * OWq;
    const long long windows = (long long)NB * Pq;
    const long long tiles = (windows + 31) / 32;
    for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const long long wl = tile * 32 + lane;
        if (wl >= windows) continue;
        const int wi = (int)wl, n = by_Pq.div(wi), wrem = wi - n * Pq, ohq = by_OWq.div(wrem), owq = wrem - ohq * OWq;
        const int ih0 = 2 * ohq - ph, iw0 = 2 * owq - pw;
        bool rowok[4], colok[4];
#pragma unroll
        for (int i = 0; i < 4; i++) { rowok[i] = (unsigned)(ih0 + i) < (unsigned)H; colok[i] = (unsigned)(iw0 + i) < (unsigned)W; }
        const float *xn = x + (long long)n * C * H * W + (long long)ih0 * W + iw0;
        for (int fg = warp; fg * 8 < F; fg += 8) {
            const int f0 = fg * 8;
            float acc[4][8];
#pragma unroll
            for (int p = 0; p < 4; p++)
#pragma unroll
                for (int f = 0; f < 8; f++) acc[p][f] = 0.f;
            for (int c = 0; c < C; c++) {
                const float *xc = xn + (long long)c * H * W;
                float v[4][4];
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) v[i][j] = (rowok[i] && colok[j]) ? __ldg(xc + i * W + j) : 0.f;
#pragma unroll
                for (int t = 0; t < 9; t++) {
                    const float4 wa = *reinterpret_cast<const float4 *>(wk + (c * 9 + t) * F + f0);
                    const float4 wb = *reinterpret_cast<const float4 *>(wk + (c * 9 + t) * F + f0 + 4);
                    const float w8[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
                    const int r = t / 3, s = t - r * 3;
#pragma unroll
                    for (int p = 0; p < 4; p++) {
                        const float a = v[(p >> 1) + r][(p & 1) + s];
#pragma unroll
                        for (int f = 0; f < 8; f++) acc[p][f] = fmaf(a, w8[f], acc[p][f]);
                    }
                }
            }
            float mx[8];
#pragma unroll
            for (int f = 0; f < 8; f++) {
                const float b = wk[C * 9 * F + f0 + f];
                float m = -3.402823466e+38f;
                int id = 0;
#pragma unroll
                for (int p = 0; p < 4; p++) {
                    const float z = epilogue_act(acc[p][f] + b, act);
                    if (z > m) { m = z; id = p; }
                }
                const long long q = ((long long)n * F + f0 + f) * Pq + wrem;
                po.pooled[q] = m;
                po.mask[q] = id;
                mx[f] = m;
            }
            if (po.copy[0]) {
                const long long o = ((long long)n * Pq + wrem) * po.Cp + f0;
                if (po.ns == 1) store_split8<1>(mx, po.enc, po.copy[0] + o, nullptr, nullptr);
                else if (po.ns == 2) store_split8<2>(mx, po.enc, po.copy[0] + o, po.copy[1] + o, nullptr);
                else store_split8<3>(mx, po.enc, po.copy[0] + o, po.copy[1] + o, po.copy[2] + o);
            }
        }
    }
}

bool conv_pool_simt_applies(int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw) {
    const int OH = H + 2 * ph - 2, OW = W + 2 * pw - 2;
    return R == 3 && S == 3 && sh == 1 && sw == 1 && C >= 1 && C <= 7 && (F & 7) == 0 && F <= 512 && OH >= 2 && OW >= 2 && !(OH & 1) && !(OW & 1) &&
           (long long)NB * OH * OW < (1ll << 31) && (size_t)(C * 9 + 1) * F * sizeof(float) <= 40 * 1024;
}

int conv_pool_simt(const float *X, const float *Wt, const float *bias, const PoolOut &pool, int NB, int C, int H, int W, int F, int ph, int pw,
                   int act, const char *name) {
    const int OH = H + 2 * ph - 2, OW = W + 2 * pw - 2, Pq = (OH / 2) * (OW / 2);
    const long long tiles = ((long long)NB * Pq + 31) / 32;
    const int grid = (int)(tiles < (long long)rt().sm_count * 8 ? tiles : (long long)rt().sm_count * 8);
    cudaStream_t st = rt().stream;
    profile_begin();
    conv3x3_pool_kernel<<<grid, 256, (size_t)(C * 9 + 1) * F * sizeof(float), st>>>(X, Wt, bias, pool, NB, C, H, W, F, OH, OW, ph, pw, act,
                                                                               fast_div(Pq), fast_div(OW / 2));
    count_launch();
    cudaError_t e = cudaGetLastError();
    profile_end(2.0 * NB * OH * OW * (double)F * C * 9, name);
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

// ---- forward of a "same" 3 x 3 convolution with ONE input channel (a grey image into F filters; the data gradient of a
// transposed convolution to one channel) --------------------------------------------------------------------------------
// All output, almost no input: a lane reads the 3 x 6 inputs of its four pixels once (16-byte vector + neighbour shuffles,
// as above) and then walks the filters, nine weights from shared memory and one 16-byte store each.  Bound by the HBM
// writes of the output.
__global__ void __launch_bounds__(256) conv_c1_3x3v_kernel(const float *__restrict__ x, const float *__restrict__ Wt,
                                                           const float *__restrict__ bias, float *__restrict__ y, int NB, int H, int W,
                                                           int OH, int F, int PH, int act, FastDiv by_rowq, FastDiv by_OWq) {
    extern __shared__ float wk[];                         // [F][9] then [F] biases
    for (int e = threadIdx.x; e < F * 9; e += blockDim.x) wk[e] = __ldg(Wt + e);
    for (int e = threadIdx.x; e < F; e += blockDim.x) wk[F * 9 + e] = bias ? __ldg(bias + e) : 0.f;
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int OWq = W >> 2, rowq = OH * OWq;
    const long long total = (long long)NB * rowq;
    const long long plane = (long long)OH * W;
    for (long long base = ((long long)blockIdx.x * blockDim.x + threadIdx.x) - lane; base < total; base += (long long)gridDim.x * blockDim.x) {
        const bool live = base + lane < total;
        const int it = live ? (int)(base + lane) : 0;
        const int n = by_rowq.div(it), rem = it - n * rowq, oh = by_OWq.div(rem), ow0 = (rem - oh * OWq) * 4;
        const int ih0 = oh - PH;
        const bool has_left = ow0 > 0, has_right = ow0 + 4 < W;
        const float *xp = x + (long long)n * H * W + (long long)ih0 * W + ow0;
        float v[3][6];
#pragma unroll
        for (int r = 0; r < 3; r++) {
            const bool rowok = (unsigned)(ih0 + r) < (unsigned)H;
            const float *row = xp + r * W;
            const float4 m = rowok ? __ldg(reinterpret_cast<const float4 *>(row)) : make_float4(0.f, 0.f, 0.f, 0.f);
            float left = __shfl_up_sync(0xffffffffu, m.w, 1), right = __shfl_down_sync(0xffffffffu, m.x, 1);
            if (lane == 0) left = (rowok && has_left) ? __ldg(row - 1) : 0.f;
            if (lane == 31) right = (rowok && has_right) ? __ldg(row + 4) : 0.f;
            v[r][0] = has_left ? left : 0.f; v[r][1] = m.x; v[r][2] = m.y; v[r][3] = m.z; v[r][4] = m.w; v[r][5] = has_right ? right : 0.f;
        }
        if (!live) continue;
        float *yo = y + (long long)n * F * plane + (long long)oh * W + ow0;
        for (int f = 0; f < F; f++, yo += plane) {
            const float *w = wk + f * 9;
            const float b = wk[F * 9 + f];
            float a0 = b, a1 = b, a2 = b, a3 = b;
#pragma unroll
            for (int r = 0; r < 3; r++)
#pragma unroll
                for (int s2 = 0; s2 < 3; s2++) {
                    const float wv = w[r * 3 + s2];
                    a0 = fmaf(v[r][s2], wv, a0); a1 = fmaf(v[r][s2 + 1], wv, a1);
                    a2 = fmaf(v[r][s2 + 2], wv, a2); a3 = fmaf(v[r][s2 + 3], wv, a3);
                }
            *reinterpret_cast<float4 *>(yo) = make_float4(epilogue_act(a0, act), epilogue_act(a1, act), epilogue_act(a2, act), epilogue_act(a3, act));
        }
    }
}

bool conv_c1_fwd_applies(const float *X, const float *Y, int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw) {
    const int OH = H + 2 * ph - 2, OW = W + 2 * pw - 2;
    return C == 1 && R == 3 && S == 3 && sh == 1 && sw == 1 && pw == 1 && OW == W && OH >= 1 && (W & 3) == 0 && F >= 1 && F <= 1024 &&
           (long long)NB * OH * W < (1ll << 31) && ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(Y)) & 15) == 0;
}

int conv_c1_fwd(const float *X, const float *Wt, const float *bias, float *Y, int NB, int H, int W, int F, int ph, int act, const char *name) {
    const int OH = H + 2 * ph - 2;
    const long long items = (long long)NB * OH * (W / 4);
    cudaStream_t st = rt().stream;
    profile_begin();
    conv_c1_3x3v_kernel<<<stride_grid(items), 256, (size_t)F * 10 * sizeof(float), st>>>(X, Wt, bias, Y, NB, H, W, OH, F, ph, act,
                                                                                     fast_div(OH * (W / 4)), fast_div(W / 4));
    count_launch();
    cudaError_t e = cudaGetLastError();
    profile_end(2.0 * NB * OH * W * (double)F * 9, name);
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

template <int SW>          // filter width when it is 3 (tap -> (r, s) at compile time), 0: any width, worked out per tap
__global__ void __launch_bounds__(256, 2) wgrad_c1_kernel(const float *__restrict__ A, const float *__restrict__ dY, float *__restrict__ partial,
                                                       int NB, int H, int W, int F, int OH, int OW, int R, int S, int sh, int sw, int ph,
                                                       int pw, int ngroups, FastDiv by_plane, FastDiv by_OW, FastDiv by_S) {
    const int lane = threadIdx.x & 31;
    const int gw = blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = gridDim.x * 8;          // gridDim.x is a multiple of ngroups
    const int g = gw % ngroups, f0 = g * C1_FPW, taps = R * S;
    const int plane = OH * OW;
    const long long total = (long long)NB * plane;
    const long long tiles = (total + 63) / 64;
    float acc[C1_FPW][C1_TAPS];
#pragma unroll
    for (int i = 0; i < C1_FPW; i++)
#pragma unroll
        for (int t = 0; t < C1_TAPS; t++) acc[i][t] = 0.f;
    // two 32-pixel rows of loads are issued before either is consumed: with one, a warp has 13 loads in flight and the
    // kernel runs at the memory latency, not the bandwidth
    for (long long tile = gw / ngroups; tile < tiles; tile += nwarps / ngroups) {
        float av[2][C1_TAPS], d[2][C1_FPW];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const long long p = tile * 64 + h * 32 + lane;
            const bool live = p < total;
            const int pi = live ? (int)p : 0;
            const int n = by_plane.div(pi), rem = pi - n * plane, oh = by_OW.div(rem), ow = rem - oh * OW;
            const float *a = A + (long long)n * H * W;
            const int ih0 = oh * sh - ph, iw0 = ow * sw - pw;
#pragma unroll
            for (int t = 0; t < C1_TAPS; t++) {
                const int r = SW ? t / (SW ? SW : 1) : by_S.div(t), ih = ih0 + r, iw = iw0 + t - r * (SW ? SW : S);
                av[h][t] = (live && t < taps && (unsigned)ih < (unsigned)H && (unsigned)iw < (unsigned)W) ? __ldg(a + ih * W + iw) : 0.f;
            }
#pragma unroll
            for (int i = 0; i < C1_FPW; i++)
                d[h][i] = (live && f0 + i < F) ? __ldg(dY + ((long long)n * F + f0 + i) * plane + rem) : 0.f;
        }
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int i = 0; i < C1_FPW; i++)
#pragma unroll
                for (int t = 0; t < C1_TAPS; t++) acc[i][t] = fmaf(d[h][i], av[h][t], acc[i][t]);
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

// The same for filters three wide, unit stride along the row and an output width that is a multiple of four: a lane owns FOUR
// consecutive pixels, reads the four filters' gradients as 16-byte vectors and the 3 x 6 one-channel inputs they share.
// A quarter of the iterations for the same bytes: the kernel above runs at the memory latency, this one nearer the bandwidth.
__global__ void __launch_bounds__(256, 2) wgrad_c1x4_kernel(const float *__restrict__ A, const float *__restrict__ dY, float *__restrict__ partial,
                                                            int NB, int H, int W, int F, int OH, int OW, int R, int sh, int ph, int pw,
                                                            int ngroups, FastDiv by_rowq, FastDiv by_OWq) {
    const int lane = threadIdx.x & 31;
    const int gw = blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = gridDim.x * 8;
    const int g = gw % ngroups, f0 = g * C1_FPW;
    const int OWq = OW >> 2, rowq = OH * OWq, plane = OH * OW;
    const long long total = (long long)NB * rowq;
    const long long tiles = (total + 31) / 32;
    float acc[C1_FPW][C1_TAPS];
#pragma unroll
    for (int i = 0; i < C1_FPW; i++)
#pragma unroll
        for (int t = 0; t < C1_TAPS; t++) acc[i][t] = 0.f;
    for (long long tile = gw / ngroups; tile < tiles; tile += nwarps / ngroups) {
        const long long it = tile * 32 + lane;
        if (it >= total) continue;
        const int n = by_rowq.div((int)it), rem = (int)(it - (long long)n * rowq), oh = by_OWq.div(rem), ow0 = (rem - oh * OWq) * 4;
        const int ih0 = oh * sh - ph, iw0 = ow0 - pw;
        const float *a = A + (long long)n * H * W + (long long)ih0 * W + iw0;
        float av[3][6];
#pragma unroll
        for (int r = 0; r < 3; r++) {
            const bool rowok = r < R && (unsigned)(ih0 + r) < (unsigned)H;
#pragma unroll
            for (int j = 0; j < 6; j++) av[r][j] = (rowok && (unsigned)(iw0 + j) < (unsigned)W) ? __ldg(a + r * W + j) : 0.f;
        }
        float4 d[C1_FPW];
#pragma unroll
        for (int i = 0; i < C1_FPW; i++)
            d[i] = f0 + i < F ? __ldg(reinterpret_cast<const float4 *>(dY + ((long long)n * F + f0 + i) * plane + (long long)oh * OW + ow0))
                              : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < C1_FPW; i++)
#pragma unroll
            for (int r = 0; r < 3; r++)
#pragma unroll
                for (int s2 = 0; s2 < 3; s2++) {
                    float v = acc[i][r * 3 + s2];
                    v = fmaf(d[i].x, av[r][s2], v); v = fmaf(d[i].y, av[r][s2 + 1], v);
                    v = fmaf(d[i].z, av[r][s2 + 2], v); v = fmaf(d[i].w, av[r][s2 + 3], v);
                    acc[i][r * 3 + s2] = v;
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
    const bool quads = S == 3 && sw == 1 && (OW & 3) == 0 && (reinterpret_cast<uintptr_t>(dY) & 15) == 0;
    const long long tiles = quads ? ((long long)NB * OH * (OW / 4) + 31) / 32 : ((long long)NB * OH * OW + 63) / 64;
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
    if (quads)
        wgrad_c1x4_kernel<<<blocks, 256, 0, st>>>(A, dY, partial, NB, H, W, F, OH, OW, R, sh, ph, pw, ngroups, fast_div(OH * (OW / 4)),
                                                  fast_div(OW / 4));
    else if (S == 3)
        wgrad_c1_kernel<3><<<blocks, 256, 0, st>>>(A, dY, partial, NB, H, W, F, OH, OW, R, S, sh, sw, ph, pw, ngroups, fast_div(OH * OW),
                                                   fast_div(OW), fast_div(S));
    else
        wgrad_c1_kernel<0><<<blocks, 256, 0, st>>>(A, dY, partial, NB, H, W, F, OH, OW, R, S, sh, sw, ph, pw, ngroups, fast_div(OH * OW),
                                                   fast_div(OW), fast_div(S));
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) {
        wgrad_c1_reduce_kernel<<<(F * R * S + 7) / 8, 256, 0, st>>>(partial, dW, F, R * S, ngroups, nwarps);
        count_launch();
        e = cudaGetLastError();
    }
    profile_end(2.0 * NB * OH * OW * (double)F * R * S, name);
    scratch_free(partial);
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

}  // namespace seera
