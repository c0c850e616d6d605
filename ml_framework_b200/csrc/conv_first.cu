// Direct fp32 convolution for layers whose whole patch is short: C*R*S <= 64 (the first layer of an image model: one
// or three input channels under a 3x3 or 5x5 window).
//
// Such a layer has almost no arithmetic per byte: with 3 input channels and 64 filters it reads a few MB, writes
// hundreds, and spends 27 multiply-adds per output.  Staging it for the tensor cores would cost more HBM traffic
// (bf16 patch rows, channels-last copies of the output gradient) than the layer itself moves, so both directions
// run on the CUDA cores straight from the NCHW fp32 tensors, in exact fp32, with the bias and activation applied
// before the one store of the output:
//   forward   each thread gathers the patches of PIX output pixels into registers and sweeps the filters, read
//             from shared memory as float4 broadcasts; the output is written once, already activated.
//   dW        a block stages 64 pixels' patches and 64 filters' output gradients in shared memory and accumulates
//             a 64 x KP tile of dW in registers across all its pixel tiles (persistent grid); per-block partial
//             sums are then added in block order, so the result does not depend on scheduling.
// Replaces cuda_conv2d_fwd / the dW half of cuda_conv2d_bwd of the reference for these shapes
// (engine_cuda/src/conv_fwd.cu, conv_bwd.cu: im2col + WMMA GEMM there).
#include "common.cuh"
#include "internal.h"

namespace seera {

struct FirstGeom {
    int NB, C, H, W, F, R, S, sh, sw, ph, pw, OH, OW, K;
};

__device__ __forceinline__ float first_act(float z, int act) {
    switch (act) {
        case SEERA_ACT_RELU: return z > 0.f ? z : 0.f;
        case SEERA_ACT_SIGMOID: return 1.f / (1.f + expf(-z));
        case SEERA_ACT_TANH: return tanhf(z);
        default: return z;
    }
}

// Patch element table: for k = (c, r, s) the offset c*H*W + r*W + s and the window row / column, packed.
// krs[k] = -1 marks padding; -2 (only when ones_col is set) marks the column k == K whose patch value is the
// constant 1, so that the weight-gradient GEMM also yields the per-filter sum of the output gradient.
__device__ __forceinline__ void fill_patch_table(int *koff, int *krs, const FirstGeom &g, int KP, bool ones_col = false) {
    for (int k = threadIdx.x; k < KP; k += blockDim.x) {
        int c = k / (g.R * g.S), rs = k - c * g.R * g.S, r = rs / g.S, s = rs - r * g.S;
        koff[k] = c * g.H * g.W + r * g.W + s;
        krs[k] = k < g.K ? ((r << 16) | s) : ((ones_col && k == g.K) ? -2 : -1);
    }
}

// Where the weight gradient takes the output gradient dz[img][f][pixel] from: a stored fp32 tensor, or computed on the
// fly as dy * act'(y) with dy either a full-resolution gradient g or the gradient gp of a 2x2 / stride-2 max-pool of
// y routed through the pool's window-local argmax indices.
struct DzSource {
    const float *dz;            // stored gradient, or null
    const float *g, *gp;        // exactly one of these when dz is null
    const int *mask;
    const float *y;
    int act;
};
__device__ __forceinline__ float first_slope(float y, int act) {
    switch (act) {
        case SEERA_ACT_RELU: return y > 0.f ? 1.f : 0.f;
        case SEERA_ACT_SIGMOID: return y * (1.f - y);
        case SEERA_ACT_TANH: return 1.f - y * y;
        default: return 1.f;
    }
}

constexpr int FIRST_FC = 64;        // filters per block pass

// ---- forward ----------------------------------------------------------------------------------------------------
template <int KP, int PIX>
__global__ void __launch_bounds__(256) conv_first_fwd_kernel(const float *__restrict__ X, const float *__restrict__ Wt,
                                                             const float *__restrict__ bias, float *__restrict__ Y, FirstGeom g,
                                                             int act) {
    __shared__ __align__(16) float Ws[KP][FIRST_FC];
    __shared__ __align__(16) float bs[FIRST_FC];
    __shared__ int koff[KP], krs[KP];
    const int f0 = blockIdx.y * FIRST_FC;
    fill_patch_table(koff, krs, g, KP);
    for (int e = threadIdx.x; e < KP * FIRST_FC; e += 256) {
        int k = e / FIRST_FC, f = e - k * FIRST_FC;
        Ws[k][f] = (k < g.K && f0 + f < g.F) ? __ldg(Wt + (long long)(f0 + f) * g.K + k) : 0.f;
    }
    if (threadIdx.x < FIRST_FC) bs[threadIdx.x] = (bias && f0 + threadIdx.x < g.F) ? __ldg(bias + f0 + threadIdx.x) : 0.f;
    __syncthreads();

    const int P = g.OH * g.OW;
    const long long pixels = (long long)g.NB * P;
    const long long groups = (pixels + 256 * PIX - 1) / (256 * PIX);
  for (long long grp = blockIdx.x; grp < groups; grp += gridDim.x) {       // persistent: the filters above are staged once
    float x[PIX][KP];
    long long obase[PIX];
    bool live[PIX];
#pragma unroll
    for (int j = 0; j < PIX; j++) {
        long long pix = (grp * PIX + j) * 256 + threadIdx.x;
        live[j] = pix < pixels;
        int img = live[j] ? (int)(pix / P) : 0, rem = live[j] ? (int)(pix - (long long)img * P) : 0;
        int oh = rem / g.OW, ow = rem - oh * g.OW;
        int ih0 = oh * g.sh - g.ph, iw0 = ow * g.sw - g.pw;
        const float *xb = X + (long long)img * g.C * g.H * g.W + (long long)ih0 * g.W + iw0;
        obase[j] = (long long)img * g.F * P + rem;
#pragma unroll
        for (int k = 0; k < KP; k++) {
            int rs = krs[k];
            int ih = ih0 + (rs >> 16), iw = iw0 + (rs & 0xffff);
            bool ok = live[j] && rs >= 0 && (unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W;
            x[j][k] = ok ? __ldg(xb + koff[k]) : 0.f;
        }
    }
    const int fcount = min(FIRST_FC, g.F - f0);
    const long long P4 = P;
    float *yp[PIX];
#pragma unroll
    for (int j = 0; j < PIX; j++) yp[j] = Y + obase[j] + (long long)f0 * P4;
    for (int fg = 0; fg < fcount; fg += 4) {
        float4 acc[PIX];
        const float4 b4 = *reinterpret_cast<const float4 *>(&bs[fg]);
#pragma unroll
        for (int j = 0; j < PIX; j++) acc[j] = b4;
#pragma unroll
        for (int k = 0; k < KP; k++) {
            const float4 w = *reinterpret_cast<const float4 *>(&Ws[k][fg]);
#pragma unroll
            for (int j = 0; j < PIX; j++) {
                acc[j].x = fmaf(x[j][k], w.x, acc[j].x); acc[j].y = fmaf(x[j][k], w.y, acc[j].y);
                acc[j].z = fmaf(x[j][k], w.z, acc[j].z); acc[j].w = fmaf(x[j][k], w.w, acc[j].w);
            }
        }
        const int left = fcount - fg;
#pragma unroll
        for (int j = 0; j < PIX; j++) {
            float4 v = acc[j];
            if (act == SEERA_ACT_RELU) {          // same selection as first_act, without the switch per value
                v.x = v.x > 0.f ? v.x : 0.f; v.y = v.y > 0.f ? v.y : 0.f; v.z = v.z > 0.f ? v.z : 0.f; v.w = v.w > 0.f ? v.w : 0.f;
            } else if (act != SEERA_ACT_NONE) {
                v.x = first_act(v.x, act); v.y = first_act(v.y, act); v.z = first_act(v.z, act); v.w = first_act(v.w, act);
            }
            if (live[j]) {
                float *y = yp[j];
                if (left >= 4) { y[0] = v.x; y[P4] = v.y; y[2 * P4] = v.z; y[3 * P4] = v.w; }
                else { y[0] = v.x; if (left > 1) y[P4] = v.y; if (left > 2) y[2 * P4] = v.z; }
            }
            yp[j] += 4 * P4;
        }
    }
  }
}

// ---- weight gradient ----------------------------------------------------------------------------------------------
constexpr int FIRST_TP = 64;        // pixels per tile
constexpr int FIRST_DS = FIRST_TP + 4;

// Thread layout: KP/4 groups of four patch elements x 64/FT groups of FT filters x PS pixel halves = 256 threads.
template <int KP>
struct FirstWgradShape {
    static constexpr int FT = KP == 64 ? 4 : 2;
    static constexpr int PS = KP == 16 ? 2 : 1;
    static constexpr int KG = KP / 4;
    static constexpr int FG = FIRST_FC / FT;
};

template <int KP>
__global__ void __launch_bounds__(256) conv_first_wgrad_kernel(const float *__restrict__ X, DzSource src,
                                                               float *__restrict__ partial, FirstGeom g, int ntiles, int ones_col) {
    using Sh = FirstWgradShape<KP>;
    constexpr int FT = Sh::FT, PS = Sh::PS, KG = Sh::KG;
    __shared__ __align__(16) float Ps[FIRST_TP][KP + 4];      // + 4: staging stores of one warp spread over 8 banks
    __shared__ __align__(16) float Ds[FIRST_FC][FIRST_DS];
    __shared__ int koff[KP], krs[KP];
    const int f0 = blockIdx.y * FIRST_FC;
    const int fcount = min(FIRST_FC, g.F - f0);
    fill_patch_table(koff, krs, g, KP, ones_col != 0);
    __syncthreads();

    const int P = g.OH * g.OW;
    const int OWq = g.OW >> 1, Pq = (g.OH >> 1) * OWq;
    const long long pixels = (long long)g.NB * P;
    const int t = threadIdx.x;
    // compute role
    const int kg = t % KG, fgi = (t / KG) % Sh::FG, half = t / (KG * Sh::FG);
    const int p_lo = half * (FIRST_TP / PS), p_hi = p_lo + FIRST_TP / PS;
    // staging role: this thread's pixel of the tile and its quarter of the patch / of the filters
    const int sp = t % FIRST_TP, sq = t / FIRST_TP;     // sq in 0..3

    float acc[FT][4];
#pragma unroll
    for (int i = 0; i < FT; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        long long pix = (long long)tile * FIRST_TP + sp;
        bool live = pix < pixels;
        int img = live ? (int)(pix / P) : 0, rem = live ? (int)(pix - (long long)img * P) : 0;
        int oh = rem / g.OW, ow = rem - oh * g.OW;
        int ih0 = oh * g.sh - g.ph, iw0 = ow * g.sw - g.pw;
        const float *xb = X + (long long)img * g.C * g.H * g.W + (long long)ih0 * g.W + iw0;
#pragma unroll
        for (int i = 0; i < KP / 4; i++) {
            int k = sq * (KP / 4) + i;
            int rs = krs[k];
            int ih = ih0 + (rs >> 16), iw = iw0 + (rs & 0xffff);
            bool ok = live && rs >= 0 && (unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W;
            Ps[sp][k] = ok ? __ldg(xb + koff[k]) : ((rs == -2 && live) ? 1.f : 0.f);
        }
        const long long plane0 = (long long)img * g.F + f0;
        if (src.dz) {
            const float *db = src.dz + plane0 * P + rem;
#pragma unroll
            for (int i = 0; i < FIRST_FC / 4; i++) {
                int f = sq * (FIRST_FC / 4) + i;
                Ds[f][sp] = (live && f < fcount) ? __ldg(db + (long long)f * P) : 0.f;
            }
        } else {
            // all loads of a batch are issued before any is used: the tile is latency-bound otherwise
            const int win = (oh >> 1) * OWq + (ow >> 1), loc = ((oh & 1) << 1) | (ow & 1);
            constexpr int FB = 8;
#pragma unroll
            for (int i0 = 0; i0 < FIRST_FC / 4; i0 += FB) {
                float dy[FB], yv[FB];
                int mk[FB];
#pragma unroll
                for (int i = 0; i < FB; i++) {
                    const int f = min(sq * (FIRST_FC / 4) + i0 + i, fcount - 1);
                    const long long plane = plane0 + f;
                    if (src.gp) { mk[i] = __ldg(src.mask + plane * Pq + win); dy[i] = __ldg(src.gp + plane * Pq + win); }
                    else { mk[i] = loc; dy[i] = __ldg(src.g + plane * P + rem); }
                    yv[i] = src.act == SEERA_ACT_NONE ? 1.f : __ldg(src.y + plane * P + rem);
                }
#pragma unroll
                for (int i = 0; i < FB; i++) {
                    const int f = sq * (FIRST_FC / 4) + i0 + i;
                    float dz = mk[i] == loc ? dy[i] : 0.f;
                    if (src.act != SEERA_ACT_NONE) dz *= first_slope(yv[i], src.act);
                    Ds[f][sp] = (live && f < fcount) ? dz : 0.f;
                }
            }
        }
        __syncthreads();
#pragma unroll 4
        for (int p = p_lo; p < p_hi; p += 4) {
            float4 d[FT], q[4];
#pragma unroll
            for (int i = 0; i < FT; i++) d[i] = *reinterpret_cast<const float4 *>(&Ds[fgi * FT + i][p]);
#pragma unroll
            for (int j = 0; j < 4; j++) q[j] = *reinterpret_cast<const float4 *>(&Ps[p + j][kg * 4]);
#pragma unroll
            for (int i = 0; i < FT; i++) {
                acc[i][0] = fmaf(d[i].x, q[0].x, acc[i][0]); acc[i][1] = fmaf(d[i].x, q[0].y, acc[i][1]);
                acc[i][2] = fmaf(d[i].x, q[0].z, acc[i][2]); acc[i][3] = fmaf(d[i].x, q[0].w, acc[i][3]);
                acc[i][0] = fmaf(d[i].y, q[1].x, acc[i][0]); acc[i][1] = fmaf(d[i].y, q[1].y, acc[i][1]);
                acc[i][2] = fmaf(d[i].y, q[1].z, acc[i][2]); acc[i][3] = fmaf(d[i].y, q[1].w, acc[i][3]);
                acc[i][0] = fmaf(d[i].z, q[2].x, acc[i][0]); acc[i][1] = fmaf(d[i].z, q[2].y, acc[i][1]);
                acc[i][2] = fmaf(d[i].z, q[2].z, acc[i][2]); acc[i][3] = fmaf(d[i].z, q[2].w, acc[i][3]);
                acc[i][0] = fmaf(d[i].w, q[3].x, acc[i][0]); acc[i][1] = fmaf(d[i].w, q[3].y, acc[i][1]);
                acc[i][2] = fmaf(d[i].w, q[3].z, acc[i][2]); acc[i][3] = fmaf(d[i].w, q[3].w, acc[i][3]);
            }
        }
        __syncthreads();
    }
    // the two pixel halves (KP == 16 only) meet in shared memory, lower half first
    if (PS == 2) {
        float *red = &Ds[0][0];                     // 64 x 16 floats needed, 64 x 68 available
        if (half == 1) {
#pragma unroll
            for (int i = 0; i < FT; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) red[(fgi * FT + i) * KP + kg * 4 + j] = acc[i][j];
        }
        __syncthreads();
        if (half == 0) {
#pragma unroll
            for (int i = 0; i < FT; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] += red[(fgi * FT + i) * KP + kg * 4 + j];
        }
    }
    if (half == 0) {
        float *out = partial + ((long long)blockIdx.y * gridDim.x + blockIdx.x) * (FIRST_FC * KP);
#pragma unroll
        for (int i = 0; i < FT; i++)
            *reinterpret_cast<float4 *>(out + (fgi * FT + i) * KP + kg * 4) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    }
}

// dW[f][k] = sum over blocks of partial[chunk][block][f - f0][k].  A block of 8 warps owns 32 outputs (one per lane);
// warp w adds blocks w, w + 8, ... in order and the eight sums meet in shared memory in warp order: a fixed order.
__global__ void __launch_bounds__(256) conv_first_wgrad_reduce_kernel(const float *__restrict__ partial, float *__restrict__ dW,
                                                                      float *__restrict__ dbias, int F, int K, int KP, int nblocks) {
    __shared__ float part[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e = blockIdx.x * 32 + lane;                  // index into the padded [F rounded to 64][KP] grid
    const int f = e / KP, k = e - f * KP;
    const int chunk = f / FIRST_FC, fl = f - chunk * FIRST_FC;
    const float *p = partial + (long long)chunk * nblocks * (FIRST_FC * KP) + fl * KP + k;
    float s0 = 0.f, s1 = 0.f;
    int b = warp;
    for (; b + 8 < nblocks; b += 16) {
        s0 += p[(long long)b * (FIRST_FC * KP)];
        s1 += p[(long long)(b + 8) * (FIRST_FC * KP)];
    }
    if (b < nblocks) s0 += p[(long long)b * (FIRST_FC * KP)];
    part[warp][lane] = s0 + s1;
    __syncthreads();
    if (warp == 0 && f < F && (k < K || (dbias && k == K))) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) s += part[w][lane];
        if (k < K) dW[(long long)f * K + k] = s;
        else dbias[f] = s;                       // the column of ones: sum of the output gradient per filter
    }
}

// Blocks of `kernel` that one SM holds at once (256 threads, static shared memory only); a persistent grid of
// exactly SMs x this many blocks runs as a single round.
template <class K>
static int resident_blocks(K kernel) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, 256, 0) != cudaSuccess || n < 1) { cudaGetLastError(); n = 1; }
    return n;
}

static bool first_geom(FirstGeom &g, int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw) {
    g = FirstGeom{NB, C, H, W, F, R, S, sh, sw, ph, pw, (H + 2 * ph - R) / sh + 1, (W + 2 * pw - S) / sw + 1, C * R * S};
    return g.K <= 64 && R < 32768 && S < 32768 && (F + FIRST_FC - 1) / FIRST_FC <= 65535;
}

bool conv_first_applies(int C, int R, int S) { return C * R * S <= 64; }

int conv_first_fwd(const float *X, const float *Wt, const float *bias, float *Y, int NB, int C, int H, int W, int F, int R, int S,
                   int ph, int pw, int sh, int sw, int act, const char *name) {
    FirstGeom g;
    if (!first_geom(g, NB, C, H, W, F, R, S, sh, sw, ph, pw)) return fail(SEERA_E_LIMIT, "%s: shape outside the short-patch kernel", name);
    long long pixels = (long long)NB * g.OH * g.OW;
    unsigned chunks = (unsigned)((F + FIRST_FC - 1) / FIRST_FC);
    cudaStream_t st = rt().stream;
    const int sms = rt().sm_count;
    auto grid_for = [&](int per_sm, int pix_per_block) {
        long long groups = (pixels + pix_per_block - 1) / pix_per_block;
        long long blocks = (long long)sms * per_sm / chunks;
        if (blocks < 1) blocks = 1;
        return dim3((unsigned)(groups < blocks ? groups : blocks), chunks);
    };
    profile_begin();
    if (g.K <= 16) {
        static int occ = 0; if (!occ) occ = resident_blocks(conv_first_fwd_kernel<16, 2>);
        conv_first_fwd_kernel<16, 2><<<grid_for(occ, 512), 256, 0, st>>>(X, Wt, bias, Y, g, act);
    } else if (g.K <= 32) {
        static int occ = 0; if (!occ) occ = resident_blocks(conv_first_fwd_kernel<32, 2>);
        conv_first_fwd_kernel<32, 2><<<grid_for(occ, 512), 256, 0, st>>>(X, Wt, bias, Y, g, act);
    } else {
        static int occ = 0; if (!occ) occ = resident_blocks(conv_first_fwd_kernel<64, 1>);
        conv_first_fwd_kernel<64, 1><<<grid_for(occ, 256), 256, 0, st>>>(X, Wt, bias, Y, g, act);
    }
    count_launch();
    cudaError_t e = cudaGetLastError();
    profile_end(2.0 * pixels * (double)F * g.K);
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

static int first_wgrad_run(const float *X, const DzSource &src, float *dW, float *dbias, const FirstGeom &g, const char *name) {
    long long pixels = (long long)g.NB * g.OH * g.OW;
    int ntiles = (int)((pixels + FIRST_TP - 1) / FIRST_TP);
    int chunks = (g.F + FIRST_FC - 1) / FIRST_FC;
    int KP = g.K <= 16 ? 16 : g.K <= 32 ? 32 : 64;
    if (dbias && g.K >= KP) return fail(SEERA_E_LIMIT, "%s: no spare patch column for the bias gradient", name);
    static int occ[3] = {0, 0, 0};
    int &o = occ[KP == 16 ? 0 : KP == 32 ? 1 : 2];
    if (!o) o = KP == 16 ? resident_blocks(conv_first_wgrad_kernel<16>) : KP == 32 ? resident_blocks(conv_first_wgrad_kernel<32>)
                                                                                   : resident_blocks(conv_first_wgrad_kernel<64>);
    int nblocks = rt().sm_count * o / chunks;          // one round of resident blocks
    if (nblocks < 1) nblocks = 1;
    if (nblocks > ntiles) nblocks = ntiles;
    float *partial = (float *)scratch_alloc((size_t)chunks * nblocks * FIRST_FC * KP * sizeof(float));
    if (!partial) return SEERA_E_OOM;
    cudaStream_t st = rt().stream;
    dim3 grid((unsigned)nblocks, (unsigned)chunks);
    const int ones = dbias ? 1 : 0;
    profile_begin();
    if (KP == 16) conv_first_wgrad_kernel<16><<<grid, 256, 0, st>>>(X, src, partial, g, ntiles, ones);
    else if (KP == 32) conv_first_wgrad_kernel<32><<<grid, 256, 0, st>>>(X, src, partial, g, ntiles, ones);
    else conv_first_wgrad_kernel<64><<<grid, 256, 0, st>>>(X, src, partial, g, ntiles, ones);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) {
        conv_first_wgrad_reduce_kernel<<<chunks * FIRST_FC * KP / 32, 256, 0, st>>>(partial, dW, dbias, g.F, g.K, KP, nblocks);
        count_launch();
        e = cudaGetLastError();
    }
    profile_end(2.0 * pixels * (double)g.F * g.K);
    scratch_free(partial);
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

int conv_first_wgrad(const float *X, const float *dY, float *dW, int NB, int C, int H, int W, int F, int R, int S, int sh, int sw,
                     int ph, int pw, const char *name) {
    FirstGeom g;
    if (!first_geom(g, NB, C, H, W, F, R, S, sh, sw, ph, pw)) return fail(SEERA_E_LIMIT, "%s: shape outside the short-patch kernel", name);
    return first_wgrad_run(X, DzSource{dY, nullptr, nullptr, nullptr, nullptr, SEERA_ACT_NONE}, dW, nullptr, g, name);
}

// True when conv_first_act_wgrad can also produce the bias gradient (a spare column in the padded patch).
bool conv_first_fuses_bias(int C, int R, int S) {
    int K = C * R * S;
    return K <= 64 && K != 16 && K != 32 && K != 64;
}

// dW and dbias of y = act(conv(X, W) + b) from the gradient of y (g) or of its 2x2 / stride-2 max-pool (gp with the
// pool's argmax indices): dz = dy * act'(y) is formed while the tile is staged and never stored.
int conv_first_act_wgrad(const float *X, const float *y, const float *g, const float *gp, const int *mask, float *dW, float *dbias,
                         int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw, int act, const char *name) {
    FirstGeom geo;
    if (!first_geom(geo, NB, C, H, W, F, R, S, sh, sw, ph, pw)) return fail(SEERA_E_LIMIT, "%s: shape outside the short-patch kernel", name);
    if ((g == nullptr) == (gp == nullptr) || (gp && (!mask || (geo.OH & 1) || (geo.OW & 1))) || (act != SEERA_ACT_NONE && !y))
        return fail(SEERA_E_ARG, "%s: bad argument", name);
    return first_wgrad_run(X, DzSource{nullptr, g, gp, mask, y, act}, dW, dbias, geo, name);
}

}  // namespace seera
