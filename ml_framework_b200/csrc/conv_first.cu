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
#include "contraction_functors.cuh"
#include "internal.h"
#include "tc_epilogue.cuh"
#include "tma_gemm_kernel.cuh"

namespace seera {

struct FirstGeom {
    int NB, C, H, W, F, R, S, sh, sw, ph, pw, OH, OW, K;
    FastDiv by_P, by_OW, by_Pq, by_OWq;      // pixels per image, output width, and the same counted in 2x2 windows
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
    const float *yp;            // with gp: the pool's output (y at each window's argmax), or null
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


// =====================================================================================================================
// Tensor-core variants (precision modes 1-3).  The patch of a pixel is at most 64 values, i.e. ONE 128-byte row of a
// K-major operand tile, so the im2col matrix never needs to exist in HBM: producer warps gather the patches from the
// fp32 NCHW input (a few MB, L2-resident), split them into bf16 copies in registers and write them straight into shared
// memory in the 128-byte-swizzled layout tcgen05.mma reads (generic-proxy stores, fence.proxy.async, mbarrier).  The
// layer then costs its output traffic: the CUDA-core kernels above spend ~4600 issue slots per 128 pixels, these ~1000.
//
//   forward   D[128 pixels, F] = A[128, K] * B[F, K]^T, one k-step per tile (only the ceil(K/16) slices that hold
//             data are multiplied).  The filters are converted once per CTA and stay in shared memory.  4 producer
//             warps (thread = pixel), 1 MMA warp, 4 epilogue warps (bias + activation, coalesced NCHW store); A ring
//             and double-buffered TMEM accumulator as in the TMA kernel.
//   dW        D[F (padded to 128), 64] += dz[64 pixels, F]^T * patches[64 pixels, 64], both operands MN-major (rows =
//             pixels), accumulated in ONE TMEM tile per CTA over all its pixel steps; dz is formed by the producers
//             from the stored gradient or from (pooled gradient, pool mask, layer output).  A column of ones in the
//             patch matrix yields the bias gradient.  Per-CTA partial tiles are reduced in block order.
// Every mbarrier wait is bounded (status word as for the other tensor-core kernels).
constexpr int FT_PRODUCERS = 512;         // 16 producer warps: with one warp per scheduler the gathers' latency was the whole cost
constexpr int FT_EPI_WARPS = 8;           // two per TMEM lane quarter, each draining half of the tile's columns: the epilogue
                                          // shares its schedulers with the producers and was the slower side with four
constexpr int FTC_THREADS = FT_PRODUCERS + 32 + 32 * FT_EPI_WARPS;      // forward: warps 0-15 producers, 16 MMA, 17-24 epilogue
constexpr int FTW_PRODUCERS = 768;        // dW: 24 producer warps (the conversion work per pixel is several times the forward's)
constexpr int FTW_THREADS = FTW_PRODUCERS + 32;           // warps 0-23 producers, 24 MMA; warps 0-3 drain the accumulator at the end
constexpr int FTW_SLOTS = FTW_PRODUCERS / 64;             // pixel-ordered producers: job slots per pixel

__device__ __forceinline__ uint32_t sw128_offset(int row, int chunk) {        // 16-byte chunk `chunk` of 128-byte row `row`
    return (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}
template <int NS>
__device__ __forceinline__ void store_copies(unsigned char *base, uint32_t copy_stride, uint32_t off, float *v) {
    *reinterpret_cast<uint4 *>(base + off) = split_chunk(v);
    if (NS >= 2) *reinterpret_cast<uint4 *>(base + copy_stride + off) = split_chunk(v);
    if (NS >= 3) *reinterpret_cast<uint4 *>(base + 2 * copy_stride + off) = split_chunk(v);
}

template <int NS>
__global__ void __launch_bounds__(FTC_THREADS, 1)
first_tc_fwd_kernel(const float *__restrict__ X, const float *__restrict__ Wt, StorePixelRows cs, FirstGeom g,
                    const float *__restrict__ bias, int act, int bn, int stages, int nslices, int pool_on, PoolOut po, int *status) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * 8 + 4];      // full[8], empty[8], tfull[2], tempty[2]
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ int koff[64], krs[64];

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t a_bytes = TC_BM * 128, b_bytes = (uint32_t)bn * 128;
    unsigned char *b_base = smem;                                           // NS filter tiles
    unsigned char *a_base = smem + (size_t)NS * b_bytes;                    // stages x NS pixel tiles
    unsigned char *epi_smem = a_base + (size_t)stages * NS * a_bytes;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[8]), tfull0 = smem_u32(&bars[16]), tempty0 = smem_u32(&bars[18]);
    const uint32_t tmem_cols = (uint32_t)(2 * bn < 32 ? 32 : 2 * bn);
    const int chunks = nslices * 2;                                         // 16-byte chunks of a row that carry data

    if (t == 0) {
        abort_flag = 0;
        for (int s = 0; s < stages; s++) { mbar_init(full0 + 8 * s, FT_PRODUCERS / 32); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; b++) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, FT_EPI_WARPS); }
        fence_mbar_init();
    }
    fill_patch_table(koff, krs, g, 64);
    // filters: row f, k along the row; rows past F and k past K are zero
    for (int e = t; e < bn * chunks; e += FTC_THREADS) {
        const int row = e / chunks, kg = e - row * chunks;
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) { int k = kg * 8 + i; v[i] = (row < g.F && k < g.K) ? __ldg(Wt + (long long)row * g.K + k) : 0.f; }
        store_copies<NS>(b_base, b_bytes, sw128_offset(row, kg), v);
    }
    fence_async_smem();
    constexpr int MMA_WARP = FT_PRODUCERS / 32;
    if (warp == MMA_WARP) tmem_alloc(smem_u32(&tmem_base_slot), tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int *abortp = &abort_flag;

    const int P = g.OH * g.OW;
    const long long pixels = (long long)g.NB * P;
    // with the pool folded in, a tile is 32 pool windows and row = 4 * window + position inside the window (the number
    // of rows is the same: OH and OW are even)
    const int tiles = (int)((pixels + TC_BM - 1) / TC_BM);
    const int OWq = g.OW >> 1, Pq = P >> 2;

    if (warp < MMA_WARP) {
        // ---------------- producers: thread = (tile row = pixel, quarter of the row's chunks) ----------------
        const int row = t & 127, cg = t >> 7;
        // the patch elements this thread gathers (chunks cg and cg + 4) are the same for every tile: keep their
        // offsets and window positions in registers
        int off[2][8], wr[2][8], ws[2][8];
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int k = (cg + 4 * h) * 8 + i, rs = (cg + 4 * h) < chunks ? krs[k] : -1;
                off[h][i] = koff[k];
                wr[h][i] = rs >= 0 ? (rs >> 16) : -(1 << 20);          // a row far outside every image: the bounds test rejects it
                ws[h][i] = rs & 0xffff;
            }
        const bool second = cg + 4 < chunks;
        int s = 0;
        uint32_t ph = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
            if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abortp, status, 1)) break;
            const int pix = tile * TC_BM + row;                  // the launcher keeps the pixel count below 2^31
            const bool live = pix < (int)pixels;
            int img, oh, ow;
            if (pool_on) {
                const int wi = live ? pix >> 2 : 0, wimg = g.by_Pq.div(wi), wrem = wi - wimg * Pq, ohq = g.by_OWq.div(wrem), owq = wrem - ohq * OWq;
                img = wimg; oh = 2 * ohq + ((row >> 1) & 1); ow = 2 * owq + (row & 1);
            } else {
                img = live ? g.by_P.div(pix) : 0;
                const int rem = live ? pix - img * P : 0;
                oh = g.by_OW.div(rem); ow = rem - oh * g.OW;
            }
            const int ih0 = live ? oh * g.sh - g.ph : -(1 << 20), iw0 = ow * g.sw - g.pw;
            const float *xb = X + (long long)img * g.C * g.H * g.W + (long long)ih0 * g.W + iw0;
            unsigned char *a_stage = a_base + (size_t)s * NS * a_bytes;
            float v0[8], v1[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const bool ok = (unsigned)(ih0 + wr[0][i]) < (unsigned)g.H && (unsigned)(iw0 + ws[0][i]) < (unsigned)g.W;
                v0[i] = ok ? __ldg(xb + off[0][i]) : 0.f;
            }
            if (second) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const bool ok = (unsigned)(ih0 + wr[1][i]) < (unsigned)g.H && (unsigned)(iw0 + ws[1][i]) < (unsigned)g.W;
                    v1[i] = ok ? __ldg(xb + off[1][i]) : 0.f;
                }
            }
            if (cg < chunks) store_copies<NS>(a_stage, a_bytes, sw128_offset(row, cg), v0);
            if (second) store_copies<NS>(a_stage, a_bytes, sw128_offset(row, cg + 4), v1);
            fence_async_smem();                      // generic-proxy stores -> visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(full0 + 8 * s);        // one arrival per warp: 512 arrivals on one barrier serialise
            if (++s == stages) { s = 0; ph ^= 1u; }
        }
    } else if (warp == MMA_WARP && lane == 0) {
        // ---------------- MMA issuer ----------------
        const uint32_t idesc = umma_idesc_bf16(bn);
        constexpr int NPROD = NS == 1 ? 1 : (NS == 2 ? 3 : 6);
        const int pa[6] = {0, 0, 1, 0, 2, 1}, pb[6] = {0, 1, 0, 2, 0, 1};
        int it = 0, s = 0;
        uint32_t ph = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, it++) {
            const int buf = it & 1;
            if (!mbar_wait(tempty0 + 8 * buf, (((uint32_t)it >> 1) & 1u) ^ 1u, abortp, status, 4)) break;
            if (!mbar_wait(full0 + 8 * s, ph, abortp, status, 2)) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(buf * bn);
            const uint32_t a0 = smem_u32(a_base + (size_t)s * NS * a_bytes), b0 = smem_u32(b_base);
            uint32_t acc = 0;
            for (int j = 0; j < nslices; j++) {
                uint64_t da[NS], db[NS];
#pragma unroll
                for (int i = 0; i < NS; i++) {
                    da[i] = umma_desc_sw128(a0 + i * a_bytes + j * 32);
                    db[i] = umma_desc_sw128(b0 + i * b_bytes + j * 32);
                }
#pragma unroll
                for (int q = 0; q < NPROD; q++) { umma_bf16(d_tmem, da[pa[q]], db[pb[q]], idesc, acc); acc = 1; }
            }
            umma_commit(empty0 + 8 * s);
            umma_commit(tfull0 + 8 * buf);
            if (++s == stages) { s = 0; ph ^= 1u; }
        }
    } else if (warp > MMA_WARP) {
        // ---------------- epilogue: warp w drains TMEM lane quarter w % 4, columns of its half ----------------
        const int q = warp & 3, ew = warp - MMA_WARP - 1;
        const int half = bn >= 64 ? bn / 2 : bn;                  // a 32-column tile is not split: the second set of warps only arrives
        const int c0 = (ew >> 2) * half, c1 = min(bn, c0 + half);
        float *stage = reinterpret_cast<float *>(epi_smem + (size_t)ew * EPI_WARP_SMEM);
        int it = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, it++) {
            const int buf = it & 1;
            if (!mbar_wait(tfull0 + 8 * buf, ((uint32_t)it >> 1) & 1u, abortp, status, 3)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * bn + c0);
            if (c0 >= bn) {}
            else if (pool_on)
                drain_accumulator_pooled(taddr, tile * TC_BM + q * 32, c0, c1 - c0, (int)pixels, g.F, bias, act, po, stage);
            else
                drain_accumulator(taddr, tile * TC_BM + q * 32, 0, c0, c1, (int)pixels, g.F, cs, nullptr, 0, stage, bias, act);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * buf);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) tmem_dealloc(tmem_base, tmem_cols);
}

template <int NS>
__global__ void __launch_bounds__(FTW_THREADS, 1)
first_tc_wgrad_kernel(const float *__restrict__ X, DzSource src, float *__restrict__ partial, FirstGeom g, int nsteps, int stages,
                      int ones_col, int by_window, int *status) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * 8 + 1];      // full[8], empty[8], done
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ int koff[64], krs[64];

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr uint32_t A_BYTES = 16384, B_BYTES = 8192;              // dz: two boxes of 64 filters; patches: one box of 64 values
    const uint32_t stage_bytes = (uint32_t)NS * (A_BYTES + B_BYTES);
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[8]), done = smem_u32(&bars[16]);
    constexpr int MMA_WARP = FTW_PRODUCERS / 32;

    if (t == 0) {
        abort_flag = 0;
        // by_window: two groups of 4 producer warps per stage (dz rows, patch rows); otherwise all producer warps fill every stage
        for (int s = 0; s < stages; s++) { mbar_init(full0 + 8 * s, by_window ? 8 : FTW_PRODUCERS / 32); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(done, 1);
        fence_mbar_init();
    }
    fill_patch_table(koff, krs, g, 64, ones_col != 0);
    // chunks that no producer ever writes (filters past F, patch values past K) must read as zero
    for (uint32_t e = t; e < (uint32_t)stages * stage_bytes / 16; e += FTW_THREADS) reinterpret_cast<uint4 *>(smem)[e] = make_uint4(0, 0, 0, 0);
    fence_async_smem();
    if (warp == MMA_WARP) tmem_alloc(smem_u32(&tmem_base_slot), 64);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int *abortp = &abort_flag;

    const int P = g.OH * g.OW, OWq = g.OW >> 1, Pq = (g.OH >> 1) * OWq;
    const long long pixels = (long long)g.NB * P;
    const int kchunks = (g.K + (ones_col ? 1 : 0) + 7) / 8;          // patch chunks that carry data (<= 8)
    const int fchunks = (g.F + 7) / 8;                               // filter chunks that carry data (<= 16)

    if (warp < MMA_WARP && by_window) {
        // ---------------- producers, pooled gradient: a step is 16 pool windows = 64 pixels, row = 4 * window + position ----------------
        // A window's gradient, argmax index and pooled output are loaded ONCE for its four pixels (dz is zero at the other
        // three).  Stage s is filled by producer groups 2s (dz rows) and 2s + 1 (patch rows), 4 warps each, so up to
        // `stages` steps are being loaded and converted at once: a single warp converts slowly (dependent ALU chains), the
        // throughput comes from having many of them (at most 3 stages x 2 groups = 24 warps).
        const int group = t >> 7, tg = t & 127, s = group >> 1;
        const long long windows = (long long)g.NB * Pq;
        if (s < stages && (group & 1) == 0) {
            // ---- dz rows: thread = (window of the step, filter chunks fcg and fcg + 8) ----
            const bool slope = src.act != SEERA_ACT_NONE;
            const int wl = tg & 15, fcg = tg >> 4;
            uint32_t ph = 0;                                   // it advances by `stages`: the slot's phase flips every iteration
            for (int it = s;; it += stages, ph ^= 1u) {
                const long long step = blockIdx.x + (long long)it * gridDim.x;
                if (step >= nsteps) break;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abortp, status, 1)) break;
                unsigned char *a_stage = smem + (size_t)s * stage_bytes;
                const long long wj = step * 16 + wl;
                const bool wlive = wj < windows;
                const int wimg = wlive ? g.by_Pq.div((int)wj) : 0, wwrem = wlive ? (int)(wj - (long long)wimg * Pq) : 0;
                const long long wbase = (long long)wimg * g.F * Pq + wwrem;
                for (int fc = fcg; fc < fchunks; fc += 8) {
                    float gv[8], pv[8];
                    int mk[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {        // every load of the chunk is issued before any is used
                        const long long q = wbase + (long long)min(fc * 8 + i, g.F - 1) * Pq;
                        gv[i] = __ldg(src.gp + q);
                        mk[i] = __ldg(src.mask + q);
                        pv[i] = slope ? __ldg(src.yp + q) : 1.f;
                    }
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const float dz = slope ? gv[i] * first_slope(pv[i], src.act) : gv[i];
                        gv[i] = (wlive && fc * 8 + i < g.F) ? dz : 0.f;
                    }
#pragma unroll
                    for (int pos = 0; pos < 4; pos++) {
                        float v[8];
#pragma unroll
                        for (int i = 0; i < 8; i++) v[i] = mk[i] == pos ? gv[i] : 0.f;
                        store_copies<NS>(a_stage, A_BYTES, (uint32_t)(fc >> 3) * 8192u + sw128_offset(4 * wl + pos, fc & 7), v);
                    }
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(full0 + 8 * s);
            }
        } else if (s < stages) {
            // ---- patch rows: thread = (row of the step, patch chunks kq, kq + 2, ...) ----
            const int pr = tg & 63, kq = tg >> 6;
            int off[2][8], wr[2][8], ws[2][8];
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int kc = kq + 2 * h, k = (kc * 8 + i) & 63, rs = kc < kchunks ? krs[k] : -1;
                    off[h][i] = koff[k];
                    wr[h][i] = rs >= 0 ? (rs >> 16) : -(1 << 20);
                    ws[h][i] = rs == -2 ? -2 : (rs & 0xffff);
                }
            uint32_t ph = 0;                                   // it advances by `stages`: the slot's phase flips every iteration
            for (int it = s;; it += stages, ph ^= 1u) {
                const long long step = blockIdx.x + (long long)it * gridDim.x;
                if (step >= nsteps) break;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abortp, status, 1)) break;
                unsigned char *b_stage = smem + (size_t)s * stage_bytes + (size_t)NS * A_BYTES;
                const long long wi = step * 16 + (pr >> 2);
                const bool live = wi < windows;
                const int img = live ? g.by_Pq.div((int)wi) : 0, wrem = live ? (int)(wi - (long long)img * Pq) : 0;
                const int ohq = g.by_OWq.div(wrem), owq = wrem - ohq * OWq;
                const int oh = 2 * ohq + ((pr >> 1) & 1), ow = 2 * owq + (pr & 1);
                const int ih0 = live ? oh * g.sh - g.ph : -(1 << 20), iw0 = ow * g.sw - g.pw;
                const float *xb = X + (long long)img * g.C * g.H * g.W + (long long)ih0 * g.W + iw0;
                float v0[8], v1[8];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const bool ok = (unsigned)(ih0 + wr[0][i]) < (unsigned)g.H && (unsigned)(iw0 + ws[0][i]) < (unsigned)g.W && ws[0][i] != -2;
                    v0[i] = ok ? __ldg(xb + off[0][i]) : ((ws[0][i] == -2 && live) ? 1.f : 0.f);
                }
                if (kq + 2 < kchunks) {
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const bool ok = (unsigned)(ih0 + wr[1][i]) < (unsigned)g.H && (unsigned)(iw0 + ws[1][i]) < (unsigned)g.W && ws[1][i] != -2;
                        v1[i] = ok ? __ldg(xb + off[1][i]) : ((ws[1][i] == -2 && live) ? 1.f : 0.f);
                    }
                }
                if (kq < kchunks) store_copies<NS>(b_stage, B_BYTES, sw128_offset(pr, kq), v0);
                if (kq + 2 < kchunks) store_copies<NS>(b_stage, B_BYTES, sw128_offset(pr, kq + 2), v1);
                for (int kc = kq + 4; kc < kchunks; kc += 2) {          // patches longer than 32 values: tables from shared memory
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int k = kc * 8 + i, rs = krs[k];
                        const int ih = ih0 + (rs >> 16), iw = iw0 + (rs & 0xffff);
                        const bool ok = live && rs >= 0 && (unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W;
                        v[i] = ok ? __ldg(xb + koff[k]) : ((rs == -2 && live) ? 1.f : 0.f);
                    }
                    store_copies<NS>(b_stage, B_BYTES, sw128_offset(pr, kc), v);
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(full0 + 8 * s);
            }
        }
    } else if (warp < MMA_WARP) {
        // ---------------- producers, stored or full-resolution gradient: thread = (pixel of the step, job slot) ----------------
        // Jobs per pixel: the 8-filter chunks of dz first, then the 8-value chunks of the patch; slot takes jobs slot, slot + 12, ...
        const int p = t & 63, slot = t >> 6;
        const int mode = src.dz ? 0 : (src.gp ? 2 : 1);               // stored dz | full-resolution gradient | pooled gradient
        const float *grad = src.dz ? src.dz : (src.gp ? src.gp : src.g);
        const bool slope = mode != 0 && src.act != SEERA_ACT_NONE;
        int s = 0;
        uint32_t ph = 0;
        for (int step = blockIdx.x; step < nsteps; step += gridDim.x, s = (s + 1 == stages ? 0 : s + 1), ph ^= (s == 0 ? 1u : 0u)) {
            if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abortp, status, 1)) break;
            unsigned char *a_stage = smem + (size_t)s * stage_bytes, *b_stage = a_stage + (size_t)NS * A_BYTES;
            const int pix = step * 64 + p;
            const bool live = pix < (int)pixels;
            const int img = live ? g.by_P.div(pix) : 0, rem = live ? pix - img * P : 0;
            const int oh = g.by_OW.div(rem), ow = rem - oh * g.OW;
            for (int job = slot; job < fchunks + kchunks; job += FTW_SLOTS) {
                if (job < fchunks) {
                    const int fc = job;
                    const int win = (oh >> 1) * OWq + (ow >> 1), loc = ((oh & 1) << 1) | (ow & 1);
                    const long long ybase = (long long)img * g.F * P + rem;                       // + f * P
                    const long long gbase = mode == 2 ? (long long)img * g.F * Pq + win : ybase;   // + f * (Pq or P)
                    const int gstride = mode == 2 ? Pq : P;
                    float dy[8], yv[8];
                    int mk[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {            // every load of the chunk is issued before any is used
                        const int f = min(fc * 8 + i, g.F - 1);
                        dy[i] = __ldg(grad + gbase + (long long)f * gstride);
                        mk[i] = mode == 2 ? __ldg(src.mask + gbase + (long long)f * gstride) : loc;
                        yv[i] = slope ? __ldg(src.y + ybase + (long long)f * P) : 1.f;
                    }
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        float dz = mk[i] == loc ? dy[i] : 0.f;
                        if (slope) dz *= first_slope(yv[i], src.act);
                        dy[i] = (live && fc * 8 + i < g.F) ? dz : 0.f;
                    }
                    store_copies<NS>(a_stage, A_BYTES, (uint32_t)(fc >> 3) * 8192u + sw128_offset(p, fc & 7), dy);
                } else {
                    const int kc = job - fchunks;
                    const int ih0 = oh * g.sh - g.ph, iw0 = ow * g.sw - g.pw;
                    const float *xb = X + (long long)img * g.C * g.H * g.W + (long long)ih0 * g.W + iw0;
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int k = kc * 8 + i, rs = krs[k];
                        const int ih = ih0 + (rs >> 16), iw = iw0 + (rs & 0xffff);
                        const bool ok = live && rs >= 0 && (unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W;
                        v[i] = ok ? __ldg(xb + koff[k]) : ((rs == -2 && live) ? 1.f : 0.f);
                    }
                    store_copies<NS>(b_stage, B_BYTES, sw128_offset(p, kc), v);
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(full0 + 8 * s);
        }
    } else if (lane == 0) {
        // ---------------- MMA issuer: one accumulator for the whole CTA ----------------
        const uint32_t idesc = umma_idesc_bf16(64) | (1u << 15) | (1u << 16);       // both operands MN-major
        constexpr int NPROD = NS == 1 ? 1 : (NS == 2 ? 3 : 6);
        const int pa[6] = {0, 0, 1, 0, 2, 1}, pb[6] = {0, 1, 0, 2, 0, 1};
        uint32_t acc = 0;
        int s = 0;
        uint32_t ph = 0;
        bool alive = true;
        for (int step = blockIdx.x; step < nsteps && alive; step += gridDim.x, s = (s + 1 == stages ? 0 : s + 1), ph ^= (s == 0 ? 1u : 0u)) {
            alive = mbar_wait(full0 + 8 * s, ph, abortp, status, 2);
            if (!alive) break;
            tc_fence_after();
            const uint32_t a0 = smem_u32(smem + (size_t)s * stage_bytes), b0 = a0 + (uint32_t)NS * A_BYTES;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint64_t da[NS], db[NS];
#pragma unroll
                for (int i = 0; i < NS; i++) {
                    da[i] = umma_desc_sw128_mn(a0 + i * A_BYTES + j * 2048, 8192);
                    db[i] = umma_desc_sw128_mn(b0 + i * B_BYTES + j * 2048, 8192);
                }
#pragma unroll
                for (int q = 0; q < NPROD; q++) { umma_bf16(tmem_base, da[pa[q]], db[pb[q]], idesc, acc); acc = 1; }
            }
            umma_commit(empty0 + 8 * s);
        }
        if (alive) umma_commit(done);
    }
    __syncwarp();
    if (warp < 4) {
        // ---------------- accumulator -> this CTA's partial tile, laid out [filter box][block][64 filters][64] ----------------
        if (mbar_wait(done, 0, abortp, status, 3)) {
            tc_fence_after();
            const int f = warp * 32 + lane;
            float *out = partial + (((long long)(f >> 6) * gridDim.x + blockIdx.x) * 64 + (f & 63)) * 64;
#pragma unroll
            for (int c = 0; c < 64; c += 32) {
                float v[32];
                tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c, v);
                if (f < ((g.F + 63) / 64) * 64) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4 *>(out + c + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) tmem_dealloc(tmem_base, 64);
}

// Dynamic shared memory limit raised once per kernel instantiation and device.
template <class K>
static cudaError_t raise_smem_limit(K kernel, int *done_flags) {
    const int dev = rt().device & 63;
    if (done_flags[dev]) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
    if (e == cudaSuccess) done_flags[dev] = 1;
    return e;
}

static bool first_tc_fwd_ok(const FirstGeom &g) { return rt().precision >= 1 && g.F <= 128 && (long long)g.NB * g.OH * g.OW < (1LL << 31) - 256; }
static bool first_tc_wgrad_ok(const FirstGeom &g, bool want_bias) {
    return rt().precision >= 1 && g.F <= 128 && (!want_bias || g.K < 64) && (long long)g.NB * g.OH * g.OW < (1LL << 31) - 256;
}

static int first_tc_fwd(const float *X, const float *Wt, const float *bias, float *Y, const FirstGeom &g, int act, const char *name,
                        const PoolOut *pool = nullptr) {
    const int ns = rt().precision == 5 ? 2 : precision_copies();   // these kernels split into bf16 themselves: the fp16 modes 4 and 5 run as bf16x3
    const int bn = g.F <= 32 ? 32 : (g.F <= 64 ? 64 : 128);
    const int nslices = (g.K + 15) / 16;
    const long long pixels = (long long)g.NB * g.OH * g.OW;
    const int tiles = (int)((pixels + TC_BM - 1) / TC_BM);
    const size_t fixed = (size_t)ns * bn * 128 + FT_EPI_WARPS * EPI_WARP_SMEM + 1024;
    int stages = (int)((225 * 1024 - fixed) / ((size_t)ns * TC_BM * 128));
    if (stages > 4) stages = 4;
    if (stages < 2) return fail(SEERA_E_LIMIT, "%s: tile does not fit shared memory", name);
    const size_t smem = fixed + (size_t)stages * ns * TC_BM * 128;
    const dim3 grid((unsigned)(tiles < rt().sm_count ? tiles : rt().sm_count));
    StorePixelRows cs{Y, g.F, g.OH * g.OW};
    PoolOut po{};
    const int pool_on = pool ? 1 : 0;
    if (pool) { po = *pool; pool_out_geometry(po, g.OH * g.OW, g.OW, 1); }
    cudaStream_t st = rt().stream;
    cudaError_t e;
    static int f1[64], f2[64], f3[64];
    profile_begin();
    if (ns == 1) { e = raise_smem_limit(first_tc_fwd_kernel<1>, f1); if (e == cudaSuccess) first_tc_fwd_kernel<1><<<grid, FTC_THREADS, smem, st>>>(X, Wt, cs, g, bias, act, bn, stages, nslices, pool_on, po, tc_status_word()); }
    else if (ns == 2) { e = raise_smem_limit(first_tc_fwd_kernel<2>, f2); if (e == cudaSuccess) first_tc_fwd_kernel<2><<<grid, FTC_THREADS, smem, st>>>(X, Wt, cs, g, bias, act, bn, stages, nslices, pool_on, po, tc_status_word()); }
    else { e = raise_smem_limit(first_tc_fwd_kernel<3>, f3); if (e == cudaSuccess) first_tc_fwd_kernel<3><<<grid, FTC_THREADS, smem, st>>>(X, Wt, cs, g, bias, act, bn, stages, nslices, pool_on, po, tc_status_word()); }
    count_launch();
    if (e == cudaSuccess) e = cudaGetLastError();
    profile_end(2.0 * pixels * (double)g.F * g.K, name);
    rt().tc_used = true;
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

static int first_tc_wgrad(const float *X, const DzSource &src, float *dW, float *dbias, const FirstGeom &g, const char *name) {
    const int ns = rt().precision == 5 ? 2 : precision_copies();   // these kernels split into bf16 themselves: the fp16 modes 4 and 5 run as bf16x3
    const long long pixels = (long long)g.NB * g.OH * g.OW;
    // pooled gradient with the pool's output at hand: steps of 16 pool windows, one producer group per stage
    const int by_window = (src.gp && (src.yp || src.act == SEERA_ACT_NONE)) ? 1 : 0;
    const int nsteps = by_window ? (int)(((long long)g.NB * (g.OH / 2) * (g.OW / 2) + 15) / 16) : (int)((pixels + 63) / 64);
    const size_t stage = (size_t)ns * (16384 + 8192);
    int stages = (int)((220 * 1024) / stage);
    if (stages > (by_window ? 3 : 4)) stages = by_window ? 3 : 4;       // by window: two groups of 4 producer warps per stage, 24 warps
    const size_t smem = stage * stages + 1024;
    const int nblocks = nsteps < rt().sm_count ? nsteps : rt().sm_count;
    const int boxes = (g.F + 63) / 64;
    float *partial = (float *)scratch_alloc((size_t)boxes * nblocks * 64 * 64 * sizeof(float));
    if (!partial) return SEERA_E_OOM;
    cudaStream_t st = rt().stream;
    cudaError_t e;
    static int f1[64], f2[64], f3[64];
    const int ones = dbias ? 1 : 0;
    profile_begin();
    if (ns == 1) { e = raise_smem_limit(first_tc_wgrad_kernel<1>, f1); if (e == cudaSuccess) first_tc_wgrad_kernel<1><<<nblocks, FTW_THREADS, smem, st>>>(X, src, partial, g, nsteps, stages, ones, by_window, tc_status_word()); }
    else if (ns == 2) { e = raise_smem_limit(first_tc_wgrad_kernel<2>, f2); if (e == cudaSuccess) first_tc_wgrad_kernel<2><<<nblocks, FTW_THREADS, smem, st>>>(X, src, partial, g, nsteps, stages, ones, by_window, tc_status_word()); }
    else { e = raise_smem_limit(first_tc_wgrad_kernel<3>, f3); if (e == cudaSuccess) first_tc_wgrad_kernel<3><<<nblocks, FTW_THREADS, smem, st>>>(X, src, partial, g, nsteps, stages, ones, by_window, tc_status_word()); }
    count_launch();
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e == cudaSuccess) {
        conv_first_wgrad_reduce_kernel<<<boxes * 64 * 64 / 32, 256, 0, st>>>(partial, dW, dbias, g.F, g.K, 64, nblocks);
        count_launch();
        e = cudaGetLastError();
    }
    profile_end(2.0 * pixels * (double)g.F * g.K, name);
    scratch_free(partial);
    rt().tc_used = true;
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

static bool first_geom(FirstGeom &g, int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw) {
    g = FirstGeom{NB, C, H, W, F, R, S, sh, sw, ph, pw, (H + 2 * ph - R) / sh + 1, (W + 2 * pw - S) / sw + 1, C * R * S};
    g.by_P = fast_div(g.OH * g.OW); g.by_OW = fast_div(g.OW);
    g.by_Pq = fast_div((g.OH * g.OW) >> 2); g.by_OWq = fast_div(g.OW >> 1);
    return g.K <= 64 && R < 32768 && S < 32768 && (F + FIRST_FC - 1) / FIRST_FC <= 65535;
}

bool conv_first_applies(int C, int R, int S) { return C * R * S <= 64; }

// The forward with the 2x2 max-pool of its output folded into the epilogue (tensor-core variant only).
bool conv_first_pool_ok(int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw) {
    FirstGeom g;
    if (conv_pool_simt_applies(NB, C, H, W, F, R, S, sh, sw, ph, pw)) return true;
    return first_geom(g, NB, C, H, W, F, R, S, sh, sw, ph, pw) && first_tc_fwd_ok(g) && g.OH >= 2 && g.OW >= 2 && !(g.OH & 1) && !(g.OW & 1);
}
int conv_first_pool_fwd(const float *X, const float *Wt, const float *bias, const PoolOut &pool, int NB, int C, int H, int W, int F, int R,
                        int S, int ph, int pw, int sh, int sw, int act, const char *name) {
    if (!conv_first_pool_ok(NB, C, H, W, F, R, S, sh, sw, ph, pw)) return fail(SEERA_E_LIMIT, "%s: shape outside the fused pool path", name);
    if (conv_pool_simt_applies(NB, C, H, W, F, R, S, sh, sw, ph, pw))       // 3 x 3, unit stride: fp32 stencil with the pool folded in
        return conv_pool_simt(X, Wt, bias, pool, NB, C, H, W, F, ph, pw, act, name);
    FirstGeom g;
    first_geom(g, NB, C, H, W, F, R, S, sh, sw, ph, pw);
    return first_tc_fwd(X, Wt, bias, nullptr, g, act, name, &pool);
}

int conv_first_fwd(const float *X, const float *Wt, const float *bias, float *Y, int NB, int C, int H, int W, int F, int R, int S,
                   int ph, int pw, int sh, int sw, int act, const char *name) {
    FirstGeom g;
    if (!first_geom(g, NB, C, H, W, F, R, S, sh, sw, ph, pw)) return fail(SEERA_E_LIMIT, "%s: shape outside the short-patch kernel", name);
    if (conv_c1_fwd_applies(X, Y, NB, C, H, W, F, R, S, sh, sw, ph, pw))       // one input channel, "same" 3 x 3: output-bound stencil
        return conv_c1_fwd(X, Wt, bias, Y, NB, H, W, F, ph, act, name);
    if (first_tc_fwd_ok(g)) return first_tc_fwd(X, Wt, bias, Y, g, act, name);
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
    profile_end(2.0 * pixels * (double)F * g.K, name);
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

static int first_wgrad_run(const float *X, const DzSource &src, float *dW, float *dbias, const FirstGeom &g, const char *name) {
    if (first_tc_wgrad_ok(g, dbias != nullptr)) return first_tc_wgrad(X, src, dW, dbias, g, name);
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
    profile_end(2.0 * pixels * (double)g.F * g.K, name);
    scratch_free(partial);
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

int conv_first_wgrad(const float *X, const float *dY, float *dW, int NB, int C, int H, int W, int F, int R, int S, int sh, int sw,
                     int ph, int pw, const char *name) {
    FirstGeom g;
    if (!first_geom(g, NB, C, H, W, F, R, S, sh, sw, ph, pw)) return fail(SEERA_E_LIMIT, "%s: shape outside the short-patch kernel", name);
    if (wgrad_c1_applies(NB, C, F, R, S, g.OH, g.OW))          // one input channel, <= 9 taps: a stencil reduction in fp32
        return wgrad_c1(X, dY, dW, NB, H, W, F, R, S, sh, sw, ph, pw, name);
    return first_wgrad_run(X, DzSource{dY, nullptr, nullptr, nullptr, nullptr, SEERA_ACT_NONE, nullptr}, dW, nullptr, g, name);
}

// True when conv_first_act_wgrad can also produce the bias gradient (a spare column in the padded patch).
bool conv_first_fuses_bias(int C, int R, int S) {
    int K = C * R * S;
    return K <= 64 && K != 16 && K != 32 && K != 64;         // holds for the CUDA-core kernel; the tensor-core one needs only K < 64
}

// dW and dbias of y = act(conv(X, W) + b) from the gradient of y (g) or of its 2x2 / stride-2 max-pool (gp with the
// pool's argmax indices): dz = dy * act'(y) is formed while the tile is staged and never stored.
int conv_first_act_wgrad(const float *X, const float *y, const float *g, const float *gp, const int *mask, const float *y_pooled,
                         float *dW, float *dbias, int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw,
                         int act, const char *name) {
    FirstGeom geo;
    if (!first_geom(geo, NB, C, H, W, F, R, S, sh, sw, ph, pw)) return fail(SEERA_E_LIMIT, "%s: shape outside the short-patch kernel", name);
    if ((g == nullptr) == (gp == nullptr) || (gp && (!mask || (geo.OH & 1) || (geo.OW & 1))) ||
        (act != SEERA_ACT_NONE && !y && !(gp && y_pooled && first_tc_wgrad_ok(geo, dbias != nullptr))))
        return fail(SEERA_E_ARG, "%s: bad argument", name);
    return first_wgrad_run(X, DzSource{nullptr, g, gp, mask, y, act, y_pooled}, dW, dbias, geo, name);
}

}  // namespace seera
