// Convolution family as implicit GEMM on the tensor cores, operands fetched by TMA in im2col mode.
//
// Replaces engine_cuda/src/convolution.cu:15-453 and upsampling.cu:15-401 (explicit fp32 column buffers of up
// to 1.85 GB and per-sample dW scratch of up to 2.4 GB, one warp per 16x16 WMMA tile).  Nothing here writes an
// im2col matrix: the TMA unit walks the filter windows of a channels-last activation tensor and lands each
// (tap, 64-channel) slice in shared memory already in the swizzled layout tcgen05.mma reads.
//
// The boundary hands over fp32 NCHW, so each call first makes bf16 channels-last shadows (one transposing pass;
// 1, 2 or 3 copies by precision mode) and small re-ordered weight shadows:
//     forward   Y[pix, f]   = sum_{tap,c} X_nhwc[window(pix)+tap, c] * Wf[f][tap][c]        A im2col, B rows
//     dX        dX[pix, c]  = sum_{tap,f} dY_nhwc[window'(pix)+tap, f] * Wd[c][tap'][f]     same kernel on dY with the
//               (stride 1)                                                                  taps flipped, pad' = K-1-pad
//     dW        dW[f][tap,c] = sum_pix dY_nhwc[pix, f] * X_nhwc[window(pix)+tap, c]         A = (tap,c) boxes by im2col,
//                                                                                          B = dY columns, split over pixels
// A transposed convolution is the same three kernels with the roles exchanged (its forward is a dX, its dX a
// forward, its dW a dW with X and dY swapped).  Data gradients with stride > 1 go to the kernel that gathers in
// its producer warps (contraction_tc.cu).  Outputs are written fp32 NCHW straight from TMEM (lanes run along
// pixels, so stores are coalesced).  Arithmetic follows engine/src/conv_ops.cpp:95-287.
#include <cfloat>

#include "internal.h"
#include "tma_gemm_kernel.cuh"

namespace seera {

typedef CUresult (*EncodeIm2colFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                   const int *, const int *, cuuint32_t, cuuint32_t, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeIm2colFn encode_im2col_fn() {
    static EncodeIm2colFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &p, cudaEnableDefault, &q) != cudaSuccess || !p) {
            cudaGetLastError();
            return nullptr;
        }
        fn = reinterpret_cast<EncodeIm2colFn>(p);
    }
    return fn;
}

// Channels-last bf16 tensor [NB, H, W, Cp]; windows of R x S taps, lower padding (ph, pw), traversal stride (sh, sw).
// The box of valid window corners runs from (-pw, -ph) to (W + pw_up - S, H + ph_up - R) with symmetric padding.
static int make_map_im2col_box(CUtensorMap *m, const void *base, int NB, int H, int W, int Cp, int sh, int sw, int lower_w, int lower_h,
                               int upper_w, int upper_h, int channels_per_pixel, int pixels_per_column);

static int make_map_im2col(CUtensorMap *m, const void *base, int NB, int H, int W, int Cp, int R, int S, int sh, int sw, int ph, int pw,
                           int channels_per_pixel, int pixels_per_column) {
    return make_map_im2col_box(m, base, NB, H, W, Cp, sh, sw, -pw, -ph, pw - (S - 1), ph - (R - 1), channels_per_pixel, pixels_per_column);
}

// General form: window corners run over w in [lower_w, W + upper_w), h in [lower_h, H + upper_h), stepping by (sw, sh).
static int make_map_im2col_box(CUtensorMap *m, const void *base, int NB, int H, int W, int Cp, int sh, int sw, int lower_w, int lower_h,
                               int upper_w, int upper_h, int channels_per_pixel, int pixels_per_column) {
    const int R = 0, S = 0, ph = -lower_h, pw = -lower_w;
    EncodeIm2colFn enc = encode_im2col_fn();
    if (!enc) return fail(SEERA_E_CUDA, "cuTensorMapEncodeIm2col is not available from this driver");
    cuuint64_t dims[4] = {(cuuint64_t)Cp, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)NB};
    cuuint64_t strides[3] = {(cuuint64_t)Cp * 2, (cuuint64_t)W * Cp * 2, (cuuint64_t)H * W * Cp * 2};
    int lower[2] = {lower_w, lower_h};
    int upper[2] = {upper_w, upper_h};
    cuuint32_t estr[4] = {1, (cuuint32_t)sw, (cuuint32_t)sh, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, lower, upper,
                     (cuuint32_t)channels_per_pixel, (cuuint32_t)pixels_per_column, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(SEERA_E_CUDA, "cuTensorMapEncodeIm2col failed (%d) for %dx%dx%dx%d window %dx%d stride %d,%d pad %d,%d", (int)r, NB, H, W,
                    Cp, R, S, sh, sw, ph, pw);
    // Known driver defect, documented in the CUTLASS sources (include/cute/atom/copy_traits_sm90_im2col.hpp, the note beside
    // cuTensorMapEncodeIm2col): drivers up to CUDA 13.1 set bit 21 of the second 64-bit word of an IM2COL descriptor when the
    // whole tensor is smaller than 128 KiB, and a load through such a descriptor returns wrong pixels.  Clearing the bit is
    // the published remedy for that driver range.  tests/test_gpu_tensorcore.py::test_im2col_maps_of_tensors_below_128_kib
    // runs convolutions on both sides of the 128 KiB boundary.
    int drv = 0;
    if (cudaDriverGetVersion(&drv) == cudaSuccess && drv <= 13010 && (size_t)NB * H * W * Cp * 2 < 131072)
        reinterpret_cast<uint64_t *>(m)[1] &= ~(1ull << 21);
    return SEERA_OK;
}

// ---- fp32 NCHW -> bf16 channels-last shadows: [NB, C, P] -> [NB, P, Cp] ---------------------------------------
// Tile of 64 channels x 32 pixels through shared memory: reads are coalesced along pixels (128 bytes per warp
// row), writes are 16-byte chunks of 8 channels, 8 threads covering the 128 contiguous bytes of one pixel.
template <int NS>
__global__ void __launch_bounds__(256) shadow_nhwc_kernel(const float *__restrict__ src, int C, int P, int Cp,
                                                          __nv_bfloat16 *__restrict__ d0, __nv_bfloat16 *__restrict__ d1,
                                                          __nv_bfloat16 *__restrict__ d2, Enc enc) {
    __shared__ float tile[64][33];
    const int img = blockIdx.z, c0 = blockIdx.y * 64, p0 = blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const float *s = src + (long long)img * C * P;
    for (int i = ty; i < 64; i += 8) {
        int c = c0 + i, p = p0 + tx;
        tile[i][tx] = (c < C && p < P) ? __ldg(s + (long long)c * P + p) : 0.f;
    }
    __syncthreads();
    const int cg = threadIdx.x & 7, pl = threadIdx.x >> 3;      // channel group of 8, pixel within the tile
    const int p = p0 + pl, c = c0 + cg * 8;
    if (p < P && c < Cp) {                                      // Cp is a multiple of 8: a group is all in or all out
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = tile[cg * 8 + i][pl];
        long long o = ((long long)img * P + p) * Cp + c;
        store_split8<NS>(v, enc, d0 + o, d1 + o, d2 + o);
    }
}

// The same for planes whose pixel count is a multiple of 4 (16-byte aligned source): a block walks tiles of 64 channels x 64 pixels,
// every thread with four 128-bit loads in flight per tile (the small-tile kernel above keeps eight 4-byte loads in flight and
// starts a block per 8 KB: 0.40 of the HBM peak; this one is bound by the traffic itself).
template <int NS>
__global__ void __launch_bounds__(256) shadow_nhwc_wide_kernel(const float *__restrict__ src, int C, int P, int Cp, int ptiles, int ctiles,
                                                               long long tiles, __nv_bfloat16 *__restrict__ d0,
                                                               __nv_bfloat16 *__restrict__ d1, __nv_bfloat16 *__restrict__ d2, Enc enc) {
    __shared__ float tile[64][65];
    const int q = threadIdx.x & 15, r0 = threadIdx.x >> 4;          // read side: 16-byte piece q of rows r0, r0 + 16, ...
    const int cg = threadIdx.x & 7, pl = threadIdx.x >> 3;          // write side: channel group of 8, pixels pl and pl + 32
    for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int pt = (int)(t % ptiles);
        const long long rest = t / ptiles;
        const int ct = (int)(rest % ctiles), img = (int)(rest / ctiles);
        const int c0 = ct * 64, p0 = pt * 64;
        const float *s = src + (long long)img * C * P;
        float4 v[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int c = c0 + r0 + 16 * i, p = p0 + 4 * q;
            v[i] = (c < C && p < P) ? __ldg(reinterpret_cast<const float4 *>(s + (long long)c * P + p)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        __syncthreads();                                            // the previous tile has been read out
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float *row = &tile[r0 + 16 * i][4 * q];
            row[0] = v[i].x; row[1] = v[i].y; row[2] = v[i].z; row[3] = v[i].w;
        }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int p = p0 + pl + 32 * h, c = c0 + cg * 8;
            if (p < P && c < Cp) {
                float o8[8];
#pragma unroll
                for (int i = 0; i < 8; i++) o8[i] = tile[cg * 8 + i][pl + 32 * h];
                const long long o = ((long long)img * P + p) * Cp + c;
                store_split8<NS>(o8, enc, d0 + o, d1 + o, d2 + o);
            }
        }
    }
}

struct NhwcShadow {
    __nv_bfloat16 *p[3] = {nullptr, nullptr, nullptr};
    int NB = 0, H = 0, W = 0, C = 0, Cp = 0;
    Enc enc{0, 1.f, nullptr};
};
static void free_nhwc(NhwcShadow &s) {
    for (int i = 0; i < 3; i++) { if (s.p[i]) scratch_free(s.p[i]); s.p[i] = nullptr; }
}
static int make_nhwc(const float *src, int NB, int C, int H, int W, int ns, NhwcShadow &s, int cls) {
    s.NB = NB; s.H = H; s.W = W; s.C = C; s.Cp = (C + 7) / 8 * 8;
    s.enc = enc_for(cls);
    if (s.enc.dscale)          // an fp32 gradient tensor handed in from outside: its own largest entry sets the dynamic factor
        if (int e = seera_grad_scale_update(src, (long long)NB * C * H * W)) return e;
    size_t bytes = (size_t)NB * H * W * s.Cp * 2;
    for (int i = 0; i < ns; i++) { s.p[i] = (__nv_bfloat16 *)scratch_alloc(bytes); if (!s.p[i]) return SEERA_E_OOM; }
    int P = H * W;
    dim3 grid((P + 31) / 32, (s.Cp + 63) / 64, NB);
    if (grid.z > 65535 || grid.y > 65535) return fail(SEERA_E_LIMIT, "channels-last shadow: batch or channel count too large");
    cudaStream_t st = rt().stream;
    ProfBytes pb(4.0 * NB * C * P + (double)ns * bytes, "shadow_nhwc");
    if ((P & 3) == 0 && P >= 64 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        const int ptiles = (P + 63) / 64, ctiles = (s.Cp + 63) / 64;
        const long long tiles = (long long)NB * ctiles * ptiles;
        const int blocks = stride_grid(tiles * 256);
        if (ns == 1) shadow_nhwc_wide_kernel<1><<<blocks, 256, 0, st>>>(src, C, P, s.Cp, ptiles, ctiles, tiles, s.p[0], s.p[1], s.p[2], s.enc);
        else if (ns == 2) shadow_nhwc_wide_kernel<2><<<blocks, 256, 0, st>>>(src, C, P, s.Cp, ptiles, ctiles, tiles, s.p[0], s.p[1], s.p[2], s.enc);
        else shadow_nhwc_wide_kernel<3><<<blocks, 256, 0, st>>>(src, C, P, s.Cp, ptiles, ctiles, tiles, s.p[0], s.p[1], s.p[2], s.enc);
    } else
    if (ns == 1) shadow_nhwc_kernel<1><<<grid, 256, 0, st>>>(src, C, P, s.Cp, s.p[0], s.p[1], s.p[2], s.enc);
    else if (ns == 2) shadow_nhwc_kernel<2><<<grid, 256, 0, st>>>(src, C, P, s.Cp, s.p[0], s.p[1], s.p[2], s.enc);
    else shadow_nhwc_kernel<3><<<grid, 256, 0, st>>>(src, C, P, s.Cp, s.p[0], s.p[1], s.p[2], s.enc);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, "shadow_nhwc");
}

// ---- weight shadows: out[o][tap][ip] = W[o*so + i*si + (flip ? taps-1-tap : tap)], zero for i >= I --------------
template <int NS>
__global__ void __launch_bounds__(256) shadow_weight_kernel(const float *__restrict__ Wt, int O, int I, int Ip, int taps, long long so,
                                                            long long si, int flip, __nv_bfloat16 *__restrict__ d0,
                                                            __nv_bfloat16 *__restrict__ d1, __nv_bfloat16 *__restrict__ d2, Enc enc) {
    long long total = (long long)O * taps * Ip;
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    const bool small = total < (1ll << 31);       // 32-bit index arithmetic then (a 64-bit division is ~10x the instructions)
    for (long long e = tid; e < total; e += nthr) {
        int i, tap, o;
        if (small) {
            const unsigned t2 = (unsigned)e / (unsigned)Ip;
            i = (int)((unsigned)e - t2 * (unsigned)Ip);
            o = (int)(t2 / (unsigned)taps);
            tap = (int)(t2 - (unsigned)o * (unsigned)taps);
        } else {
            i = (int)(e % Ip); long long t2 = e / Ip;
            tap = (int)(t2 % taps); o = (int)(t2 / taps);
        }
        float v = i < I ? __ldg(Wt + o * so + i * si + (flip ? taps - 1 - tap : tap)) : 0.f;
        store_split1(v, NS, enc, d0 + e, d1 + e, d2 + e);
    }
}
// Result is a row-major matrix [O, taps*Ip] (Shadow with ld = cols).
static int make_weight_shadow(const float *Wt, int O, int I, int taps, long long so, long long si, int flip, int ns, Shadow &s) {
    int Ip = (I + 7) / 8 * 8;
    if (int e = alloc_shadow(s, O, taps * Ip, ns)) return e;
    s.enc = enc_for(CLS_WEIGHT);
    long long total = (long long)O * taps * Ip;
    int grid = stride_grid(total);
    cudaStream_t st = rt().stream;
    if (ns == 1) shadow_weight_kernel<1><<<grid, 256, 0, st>>>(Wt, O, I, Ip, taps, so, si, flip, s.p[0], s.p[1], s.p[2], s.enc);
    else if (ns == 2) shadow_weight_kernel<2><<<grid, 256, 0, st>>>(Wt, O, I, Ip, taps, so, si, flip, s.p[0], s.p[1], s.p[2], s.enc);
    else shadow_weight_kernel<3><<<grid, 256, 0, st>>>(Wt, O, I, Ip, taps, so, si, flip, s.p[0], s.p[1], s.p[2], s.enc);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, "shadow_weight");
}

// Filter shadow of one output phase of a strided data gradient: out[o][(t',u')][ip] = W[o*so + i*si + r*S + s] with
// r = r0 + sh*(Ta-1-t'), s = s0 + sw*(Ub-1-u')  (the taps that reach this phase, flipped), zero for i >= I.
template <int NS>
__global__ void __launch_bounds__(256) shadow_weight_phase_kernel(const float *__restrict__ Wt, int O, int I, int Ip, long long so, long long si,
                                                                  int S, int r0, int sh, int Ta, int s0, int sw, int Ub,
                                                                  __nv_bfloat16 *__restrict__ d0, __nv_bfloat16 *__restrict__ d1,
                                                                  __nv_bfloat16 *__restrict__ d2, Enc enc) {
    const int taps = Ta * Ub;
    long long total = (long long)O * taps * Ip;
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long e = tid; e < total; e += nthr) {
        int i = (int)(e % Ip); long long t2 = e / Ip;
        int tap = (int)(t2 % taps); int o = (int)(t2 / taps);
        int tp = tap / Ub, up = tap - tp * Ub;
        int r = r0 + sh * (Ta - 1 - tp), sx = s0 + sw * (Ub - 1 - up);
        float v = i < I ? __ldg(Wt + o * so + i * si + r * S + sx) : 0.f;
        store_split1(v, NS, enc, d0 + e, d1 + e, d2 + e);
    }
}

// Output of one phase: row m = (img, i, j) of the phase grid is pixel (a + sh*i, b + sw*j) of the full-resolution tensor.
struct StorePhaseRows {
    static constexpr bool kMContiguous = true;
    float *out; int Nch, H, W, Hg, Wg, a, b, sh, sw;
    __device__ float *row(int m) const {
        int pg = Hg * Wg, img = m / pg, rem = m - img * pg, i = rem / Wg, j = rem - i * Wg;
        return out + (long long)img * Nch * H * W + (long long)(a + sh * i) * W + (b + sw * j);
    }
    __device__ long long nstride() const { return (long long)H * W; }
    __device__ void operator()(int m, int n, float v) const { row(m)[n * nstride()] = v; }
};

// dW element for accumulator row m = (tap, channel) and column n = output-side channel: dW[(n*C + c)*taps + tap]
struct StoreWgrad {
    static constexpr bool kMContiguous = true;
    float *dW; int C, taps, c64;
    __device__ void operator()(int m, int n, float v) const {
        int tap = m / c64, c = m - tap * c64;
        if (c < C) dW[((long long)n * C + c) * taps + tap] = v;
    }
    __device__ float *row(int m) const { int tap = m / c64, c = m - tap * c64; return c < C ? dW + (long long)c * taps + tap : nullptr; }
    __device__ long long nstride() const { return (long long)C * taps; }
};

// Y[NB, F, OH, OW] = conv(X_nhwc, weights Wk[F][tap][Cp]) with window R x S, stride, lower padding.
static int tma_fprop(const NhwcShadow &x, const Shadow &wk, float *Y, int F, int R, int S, int sh, int sw, int ph, int pw,
                     int OH, int OW, int ns, const char *name, const float *bias = nullptr, int act = 0, const PoolOut *pool = nullptr) {
    TmaGemmParams p{};
    p.bias = bias; p.act = act;
    if (pool) { p.pool_on = 1; p.pool = *pool; pool_out_geometry(p.pool, OH * OW, OW, 0); }
    p.a_mode = TMA_A_IM2COL; p.b_mn = 0;
    p.a_fp16 = x.enc.fmt; p.b_fp16 = wk.enc.fmt; p.out_scale = 1.f / (x.enc.scale * wk.enc.scale); p.dinv = enc_dinv(x.enc, wk.enc);
    p.M = x.NB * OH * OW; p.N = F;
    p.cchunks = (x.Cp + 63) / 64; p.cpad = x.Cp; p.taps = R * S; p.S = S;
    p.K = p.taps * p.cchunks * 64;
    p.OW = OW; p.OHW = OH * OW; p.sw = sw; p.sh = sh; p.pw = pw; p.ph = ph;
    tma_plan(p, ns, false);
    TmaMaps maps;
    for (int i = 0; i < 3; i++) {
        int j = i < ns ? i : 0;
        if (int s = make_map_im2col(&maps.a[i], x.p[j], x.NB, x.H, x.W, x.Cp, R, S, sh, sw, ph, pw, 64, TC_BM)) return s;
        if (int s = make_map_2d(&maps.b[i], wk.p[j], wk.rows, wk.cols, wk.ld, 64, p.pair ? p.bn / 2 : p.bn)) return s;
    }
    double flops = 2.0 * p.M * (double)F * x.C * R * S;
    return launch_tma_gemm(maps, p, StorePixelRows{Y, F, OH * OW}, ns, false, flops, name);
}

// dW[Fo][C][R][S] = sum over output pixels of dY_nhwc[pix, f] * X_nhwc[window(pix)+tap, c]
static int tma_wgrad(const NhwcShadow &x, const NhwcShadow &dy, float *dW, int R, int S, int sh, int sw, int ph, int pw, int ns,
                     const char *name) {
    const int OH = dy.H, OW = dy.W, F = dy.C;
    TmaGemmParams p{};
    p.a_mode = TMA_A_TAPS; p.b_mn = 1;
    p.a_fp16 = x.enc.fmt; p.b_fp16 = dy.enc.fmt; p.out_scale = 1.f / (x.enc.scale * dy.enc.scale); p.dinv = enc_dinv(x.enc, dy.enc);
    p.cchunks = (x.Cp + 63) / 64; p.cpad = x.Cp; p.taps = R * S; p.S = S;
    p.M = p.taps * p.cchunks * 64; p.N = F;
    p.K = x.NB * OH * OW;
    p.OW = OW; p.OHW = OH * OW; p.sw = sw; p.sh = sh; p.pw = pw; p.ph = ph;
    tma_plan(p, ns, true);
    TmaMaps maps;
    for (int i = 0; i < 3; i++) {
        int j = i < ns ? i : 0;
        if (int s = make_map_im2col(&maps.a[i], x.p[j], x.NB, x.H, x.W, x.Cp, R, S, sh, sw, ph, pw, 64, 64)) return s;
        if (int s = make_map_2d(&maps.b[i], dy.p[j], dy.NB * OH * OW, dy.Cp, dy.Cp, 64, 64)) return s;
    }
    double flops = 2.0 * p.K * (double)F * x.C * R * S;
    return launch_tma_gemm(maps, p, StoreWgrad{dW, x.C, R * S, p.cchunks * 64}, ns, true, flops, name);
}

// ---- strided data gradient by output phase ---------------------------------------------------------------------
// out[n, c, h, w] = sum over (f, r, s) with (h + ph - r) % sh == 0 and (w + pw - s) % sw == 0 of
//                   g[n, f, (h + ph - r)/sh, (w + pw - s)/sw] * Wt[o = c, i = f, r, s].
// Output pixels with h % sh == a and w % sw == b see only the taps r = r0 + sh*t, s = s0 + sw*u (r0 = (a + ph) % sh,
// s0 = (b + pw) % sw), and over the phase grid (i, j) = (h / sh, w / sw) the sum is a unit-stride convolution of g with
// those taps: window corner (i + qa - (Ta-1), j + qb - (Ub-1)), qa = (a + ph - r0)/sh.  Each phase is one TMA
// implicit-GEMM launch with its own window box and filter shadow, scattering into the full-resolution tensor.
struct PhaseAxis { int r0, T, q, lower, upper, G; };
static PhaseAxis phase_axis(int a, int pad, int stride, int K, int full, int gdim) {
    PhaseAxis x;
    x.r0 = (a + pad) % stride;
    x.T = x.r0 < K ? (K - x.r0 + stride - 1) / stride : 0;
    x.q = (a + pad - x.r0) / stride;
    x.G = a < full ? (full - a + stride - 1) / stride : 0;
    x.lower = x.q - (x.T - 1);
    x.upper = x.G - gdim + x.lower;
    return x;
}
static bool phases_supported(int H, int W, int GH, int GW, int R, int S, int sh, int sw, int ph, int pw) {
    for (int a = 0; a < sh; a++) {
        PhaseAxis y = phase_axis(a, ph, sh, R, H, GH);
        if (y.T && y.G && (y.lower < -128 || y.lower > 127 || y.upper > 0 || y.upper < -128)) return false;
    }
    for (int b = 0; b < sw; b++) {
        PhaseAxis x = phase_axis(b, pw, sw, S, W, GW);
        if (x.T && x.G && (x.lower < -128 || x.lower > 127 || x.upper > 0 || x.upper < -128)) return false;
    }
    return true;
}
static int tma_dgrad_phases(const NhwcShadow &g, const float *Wt, long long so, long long si, float *out, int Nch, int H, int W,
                            int R, int S, int sh, int sw, int ph, int pw, int ns, const char *name, const float *bias = nullptr,
                            int act = 0) {
    cudaStream_t st = rt().stream;
    bool hole = false;
    for (int a = 0; a < sh; a++) hole |= phase_axis(a, ph, sh, R, H, g.H).T == 0;
    for (int b = 0; b < sw; b++) hole |= phase_axis(b, pw, sw, S, W, g.W).T == 0;
    if (hole) {       // stride larger than the filter: some output pixels receive nothing from the sum
        if (bias || act) return fail(SEERA_E_LIMIT, "%s: fused bias/activation needs every output pixel under some tap", name);
        cudaError_t e = cudaMemsetAsync(out, 0, (size_t)g.NB * Nch * H * W * sizeof(float), st);
        if (e != cudaSuccess) return check_cuda(e, name);
    }
    const int Ip = g.Cp;
    for (int a = 0; a < sh; a++) {
        PhaseAxis y = phase_axis(a, ph, sh, R, H, g.H);
        if (!y.T || !y.G) continue;
        for (int b = 0; b < sw; b++) {
            PhaseAxis x = phase_axis(b, pw, sw, S, W, g.W);
            if (!x.T || !x.G) continue;
            Shadow wk;
            const int taps = y.T * x.T;
            if (int e = alloc_shadow(wk, Nch, taps * Ip, ns)) return e;
            wk.enc = enc_for(CLS_WEIGHT);
            long long total = (long long)Nch * taps * Ip;
            int grid = stride_grid(total);
            if (ns == 1) shadow_weight_phase_kernel<1><<<grid, 256, 0, st>>>(Wt, Nch, g.C, Ip, so, si, S, y.r0, sh, y.T, x.r0, sw, x.T, wk.p[0], wk.p[1], wk.p[2], wk.enc);
            else if (ns == 2) shadow_weight_phase_kernel<2><<<grid, 256, 0, st>>>(Wt, Nch, g.C, Ip, so, si, S, y.r0, sh, y.T, x.r0, sw, x.T, wk.p[0], wk.p[1], wk.p[2], wk.enc);
            else shadow_weight_phase_kernel<3><<<grid, 256, 0, st>>>(Wt, Nch, g.C, Ip, so, si, S, y.r0, sh, y.T, x.r0, sw, x.T, wk.p[0], wk.p[1], wk.p[2], wk.enc);
            count_launch();
            cudaError_t ce = cudaGetLastError();
            if (ce != cudaSuccess) { free_shadow(wk); return check_cuda(ce, "shadow_weight_phase"); }

            TmaGemmParams p{};
            p.bias = bias; p.act = act;
            p.a_mode = TMA_A_IM2COL; p.b_mn = 0;
            p.a_fp16 = g.enc.fmt; p.b_fp16 = wk.enc.fmt; p.out_scale = 1.f / (g.enc.scale * wk.enc.scale); p.dinv = enc_dinv(g.enc, wk.enc);
            p.M = g.NB * y.G * x.G; p.N = Nch;
            p.cchunks = (g.Cp + 63) / 64; p.cpad = g.Cp; p.taps = taps; p.S = x.T;
            p.K = p.taps * p.cchunks * 64;
            p.OW = x.G; p.OHW = y.G * x.G; p.sw = 1; p.sh = 1; p.pw = -x.lower; p.ph = -y.lower;
            tma_plan(p, ns, false);
            TmaMaps maps;
            int e = SEERA_OK;
            for (int i = 0; i < 3 && !e; i++) {
                int j = i < ns ? i : 0;
                e = make_map_im2col_box(&maps.a[i], g.p[j], g.NB, g.H, g.W, g.Cp, 1, 1, x.lower, y.lower, x.upper, y.upper, 64, TC_BM);
                if (!e) e = make_map_2d(&maps.b[i], wk.p[j], wk.rows, wk.cols, wk.ld, 64, p.pair ? p.bn / 2 : p.bn);
            }
            double flops = 2.0 * p.M * (double)Nch * g.C * taps;
            if (!e) e = launch_tma_gemm(maps, p, StorePhaseRows{out, Nch, H, W, y.G, x.G, a, b, sh, sw}, ns, false, flops, name);
            free_shadow(wk);
            if (e) return e;
        }
    }
    return SEERA_OK;
}

// ---- activation backward written straight into channels-last shadows ------------------------------------------
// dz = dy * act'(y) for a layer output y[NB, C, H, W]; dy is either the full-resolution gradient g or, when gp is
// given, the gradient gp[NB, C, H/2, W/2] of a 2x2 / stride-2 max-pool of y routed through the pool's window-local
// argmax indices (the pool backward folded in).  The fp32 dz never reaches HBM: each 64-channel x 32-pixel tile is
// transposed in shared memory and stored as bf16 copies [NB, H*W, Cp], which is what the convolution backward
// reads.  Per-channel sums of dz (the bias gradient) are accumulated per thread in a fixed order, reduced by warp
// shuffles and written as one partial row per block.
__device__ __forceinline__ float slope_from_output(float y, int act) {
    switch (act) {
        case SEERA_ACT_RELU: return y > 0.f ? 1.f : 0.f;
        case SEERA_ACT_SIGMOID: return y * (1.f - y);
        case SEERA_ACT_TANH: return 1.f - y * y;
        default: return 1.f;
    }
}
template <int NS>
__global__ void __launch_bounds__(256, 4) dz_shadow_kernel(const float *__restrict__ g, const float *__restrict__ gp, const int *__restrict__ mask,
                                                        const float *__restrict__ y, const float *__restrict__ yp, int C, int H, int W,
                                                        int Cp, int items, int ptiles,
                                                        int act, __nv_bfloat16 *__restrict__ d0, __nv_bfloat16 *__restrict__ d1,
                                                        __nv_bfloat16 *__restrict__ d2, float *__restrict__ partial, Enc enc) {
    // Read side: warp = group of 8 consecutive channels, lane = pixel: every load is one 128-byte line of a channel plane.
    // Write side: the 32-pixel x 64-channel tile goes through shared memory so that 8 consecutive lanes write the 128 bytes one
    // pixel owns in the channels-last copies and a warp writes four whole pixels per store.
    __shared__ __align__(16) float sdz[32][64 + 4];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int cb = blockIdx.y * 64 + warp * 8;
    const int P = H * W, Wq = W >> 1, Pq = (H >> 1) * Wq;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i] = 0.f;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int img = item / ptiles, p0 = (item - img * ptiles) * 32, p = p0 + lane;
        if (cb < Cp) {
            float dy[8], yv[8];
            bool sloped = false;
            if (p >= P) {
#pragma unroll
                for (int i = 0; i < 8; i++) dy[i] = 0.f;
            } else {
            if (gp) {
                const int h = p / W, w = p - h * W;
                const int win = (h >> 1) * Wq + (w >> 1), loc = ((h & 1) << 1) | (w & 1);
                int mk[8];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const long long q = ((long long)img * C + min(cb + i, C - 1)) * Pq + win;
                    mk[i] = __ldg(mask + q);
                    dy[i] = __ldg(gp + q);
                    // the pool's output is y at the window's argmax, the only pixel of the window where dz is not zero
                    yv[i] = (yp && act != SEERA_ACT_NONE) ? __ldg(yp + q) : 1.f;
                }
#pragma unroll
                for (int i = 0; i < 8; i++) dy[i] = mk[i] == loc ? dy[i] : 0.f;
                if (yp && act != SEERA_ACT_NONE) {
                    sloped = true;
#pragma unroll
                    for (int i = 0; i < 8; i++) dy[i] *= slope_from_output(yv[i], act);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) dy[i] = __ldg(g + ((long long)img * C + min(cb + i, C - 1)) * P + p);
            }
            if (act != SEERA_ACT_NONE && !sloped) {
#pragma unroll
                for (int i = 0; i < 8; i++) yv[i] = __ldg(y + ((long long)img * C + min(cb + i, C - 1)) * P + p);
#pragma unroll
                for (int i = 0; i < 8; i++) dy[i] *= slope_from_output(yv[i], act);
            }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                if (cb + i >= C) dy[i] = 0.f;          // padding channels of the last group
                acc[i] += dy[i];
            }
            }
            *reinterpret_cast<float4 *>(&sdz[lane][warp * 8]) = make_float4(dy[0], dy[1], dy[2], dy[3]);
            *reinterpret_cast<float4 *>(&sdz[lane][warp * 8 + 4]) = make_float4(dy[4], dy[5], dy[6], dy[7]);
        }
        __syncthreads();
        const int ch = threadIdx.x & 7, c8 = blockIdx.y * 64 + ch * 8, pp = p0 + (threadIdx.x >> 3);
        if (c8 < Cp && pp < P) {
            const float4 a = *reinterpret_cast<const float4 *>(&sdz[threadIdx.x >> 3][ch * 8]);
            const float4 b = *reinterpret_cast<const float4 *>(&sdz[threadIdx.x >> 3][ch * 8 + 4]);
            float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            const long long o = ((long long)img * P + pp) * Cp + c8;
            store_split8<NS>(v, enc, d0 + o, d1 + o, d2 + o);
        }
        __syncthreads();
    }
    if (partial) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float t = acc[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            if (lane == 0 && cb + i < C) partial[(long long)blockIdx.x * C + cb + i] = t;
        }
    }
}
// The same for a pooled gradient with the pool's output at hand, organised by pool window: lane = window, so the
// quarter-resolution tensors (gradient, argmax index, pooled output) are read as full 128-byte lines, once per window
// instead of once per pixel, and each thread writes the channels-last chunks of its window's four pixels.
template <int NS>
__global__ void __launch_bounds__(256, 4) dz_shadow_window_kernel(const float *__restrict__ gp, const int *__restrict__ mask,
                                                                  const float *__restrict__ yp, int C, int H, int W, int Cp, int items,
                                                                  int wtiles, int act, __nv_bfloat16 *__restrict__ d0,
                                                                  __nv_bfloat16 *__restrict__ d1, __nv_bfloat16 *__restrict__ d2,
                                                                  float *__restrict__ partial, Enc enc) {
    // Tile = 32 windows x 64 channels.  Read side: lane = window, warp = 8 channels (full lines of the channel-major pooled
    // tensors).  Write side: the tile goes through shared memory so that 8 consecutive lanes write the 128 bytes one pixel owns
    // in the channels-last copies (a lane-per-window store touches 32 different lines per instruction).
    __shared__ __align__(16) float sval[32][64 + 4];
    __shared__ __align__(16) int smk[32][64 + 4];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int cb = blockIdx.y * 64 + warp * 8;
    const int P = H * W, Wq = W >> 1, Pq = (H >> 1) * Wq;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i] = 0.f;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int img = item / wtiles, q0 = (item - img * wtiles) * 32, q = q0 + lane;
        if (cb < Cp) {
            float val[8];
            int mk[8];
            if (q < Pq) {
                float pv[8];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const long long o = ((long long)img * C + min(cb + i, C - 1)) * Pq + q;
                    val[i] = __ldg(gp + o);
                    mk[i] = __ldg(mask + o);
                    pv[i] = act != SEERA_ACT_NONE ? __ldg(yp + o) : 1.f;
                }
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    if (act != SEERA_ACT_NONE) val[i] *= slope_from_output(pv[i], act);
                    if (cb + i >= C) val[i] = 0.f;
                    acc[i] += ((unsigned)mk[i] < 4u) ? val[i] : 0.f;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) { val[i] = 0.f; mk[i] = -1; }
            }
            *reinterpret_cast<float4 *>(&sval[lane][warp * 8]) = make_float4(val[0], val[1], val[2], val[3]);
            *reinterpret_cast<float4 *>(&sval[lane][warp * 8 + 4]) = make_float4(val[4], val[5], val[6], val[7]);
            *reinterpret_cast<int4 *>(&smk[lane][warp * 8]) = make_int4(mk[0], mk[1], mk[2], mk[3]);
            *reinterpret_cast<int4 *>(&smk[lane][warp * 8 + 4]) = make_int4(mk[4], mk[5], mk[6], mk[7]);
        }
        __syncthreads();
        // thread = (window w, 8-channel chunk ch): its window's four pixels, 16 bytes of each copy per pixel
        const int ch = threadIdx.x & 7, c8 = blockIdx.y * 64 + ch * 8, w = threadIdx.x >> 3, qq = q0 + w;
        if (c8 < Cp && qq < Pq) {
            const float4 a = *reinterpret_cast<const float4 *>(&sval[w][ch * 8]), b = *reinterpret_cast<const float4 *>(&sval[w][ch * 8 + 4]);
            const int4 ma = *reinterpret_cast<const int4 *>(&smk[w][ch * 8]), mb = *reinterpret_cast<const int4 *>(&smk[w][ch * 8 + 4]);
            const float vv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            const int mm[8] = {ma.x, ma.y, ma.z, ma.w, mb.x, mb.y, mb.z, mb.w};
            const int ohq = qq / Wq, owq = qq - ohq * Wq;
#pragma unroll
            for (int pos = 0; pos < 4; pos++) {
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; i++) v[i] = mm[i] == pos ? vv[i] : 0.f;
                const int p = (2 * ohq + (pos >> 1)) * W + 2 * owq + (pos & 1);
                const long long o = ((long long)img * P + p) * Cp + c8;
                store_split8<NS>(v, enc, d0 + o, d1 + o, d2 + o);
            }
        }
        __syncthreads();
    }
    if (partial) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float t = acc[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            if (lane == 0 && cb + i < C) partial[(long long)blockIdx.x * C + cb + i] = t;
        }
    }
}

// The same for layers whose pooled image holds fewer than 32 windows (a power of two of them: 4 x 4, 2 x 2, 4 x 2 ... pooled
// images deep in a network).  With lane = window most lanes of the kernel above would idle.  Here a tile is 32 / Pq whole images
// x 64 channels: per image those are 64 * Pq CONSECUTIVE floats of each quarter-resolution tensor, read flat (fully coalesced),
// turned to (window, channel) order in shared memory and written like above.  The bias gradient is summed on the write side.
template <int NS>
__global__ void __launch_bounds__(256, 3) dz_shadow_window_small_kernel(const float *__restrict__ gp, const int *__restrict__ mask,
                                                                        const float *__restrict__ yp, int NB, int C, int H, int W, int Cp,
                                                                        int items, int lgPq, int act, __nv_bfloat16 *__restrict__ d0,
                                                                        __nv_bfloat16 *__restrict__ d1, __nv_bfloat16 *__restrict__ d2,
                                                                        float *__restrict__ partial, Enc enc) {
    __shared__ __align__(16) float sval[32][64 + 4];
    __shared__ __align__(16) int smk[32][64 + 4];
    const int P = H * W, Wq = W >> 1, Pq = 1 << lgPq, ipt = 32 >> lgPq, cb0 = blockIdx.y * 64;
    const int ch = threadIdx.x & 7, c8 = cb0 + ch * 8, w = threadIdx.x >> 3;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i] = 0.f;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        float val[8], pv[8];
        int mk[8];
#pragma unroll
        for (int it = 0; it < 8; it++) {
            const int e = it * 256 + threadIdx.x, q = e & (Pq - 1), cl = (e >> lgPq) & 63, img = item * ipt + (e >> (lgPq + 6));
            const bool ok = img < NB && cb0 + cl < C;
            const long long o = ((long long)min(img, NB - 1) * C + min(cb0 + cl, C - 1)) * Pq + q;
            val[it] = ok ? __ldg(gp + o) : 0.f;
            mk[it] = ok ? __ldg(mask + o) : -1;
            pv[it] = (ok && act != SEERA_ACT_NONE) ? __ldg(yp + o) : 1.f;
        }
#pragma unroll
        for (int it = 0; it < 8; it++) {
            const int e = it * 256 + threadIdx.x, q = e & (Pq - 1), cl = (e >> lgPq) & 63, il = e >> (lgPq + 6);
            if (act != SEERA_ACT_NONE) val[it] *= slope_from_output(pv[it], act);
            sval[il * Pq + q][cl] = val[it];
            smk[il * Pq + q][cl] = mk[it];
        }
        __syncthreads();
        const int img = item * ipt + (w >> lgPq), qq = w & (Pq - 1);
        if (c8 < Cp && img < NB) {
            const float4 a = *reinterpret_cast<const float4 *>(&sval[w][ch * 8]), b = *reinterpret_cast<const float4 *>(&sval[w][ch * 8 + 4]);
            const int4 ma = *reinterpret_cast<const int4 *>(&smk[w][ch * 8]), mb = *reinterpret_cast<const int4 *>(&smk[w][ch * 8 + 4]);
            const float vv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            const int mm[8] = {ma.x, ma.y, ma.z, ma.w, mb.x, mb.y, mb.z, mb.w};
            const int ohq = qq / Wq, owq = qq - ohq * Wq;
#pragma unroll
            for (int i = 0; i < 8; i++) acc[i] += ((unsigned)mm[i] < 4u) ? vv[i] : 0.f;
#pragma unroll
            for (int pos = 0; pos < 4; pos++) {
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; i++) v[i] = mm[i] == pos ? vv[i] : 0.f;
                const int p = (2 * ohq + (pos >> 1)) * W + 2 * owq + (pos & 1);
                const long long o = ((long long)img * P + p) * Cp + c8;
                store_split8<NS>(v, enc, d0 + o, d1 + o, d2 + o);
            }
        }
        __syncthreads();
    }
    if (partial) {
        // threads with the same ch hold sums of the same eight channels: lanes ch, ch + 8, ch + 16, ch + 24 of each warp
        float *red = &sval[0][0];                      // [8 warps][8 chunks][8 channels]
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float t = acc[i];
            t += __shfl_xor_sync(0xffffffffu, t, 8);
            t += __shfl_xor_sync(0xffffffffu, t, 16);
            if (lane < 8) red[(warp * 8 + lane) * 8 + i] = t;
        }
        __syncthreads();
        if (threadIdx.x < 64) {
            float t = 0.f;
#pragma unroll
            for (int wv = 0; wv < 8; wv++) t += red[wv * 64 + threadIdx.x];
            if (cb0 + threadIdx.x < C) partial[(long long)blockIdx.x * C + cb0 + threadIdx.x] = t;
        }
    }
}
// ---- 2x2 / stride-2 max-pool that also writes the channels-last copies of its output ---------------------------
// Same thread layout as dz_shadow_kernel (warp = 8 channels, lane = output pixel).  The scan order and the strict
// comparison match cuda_maxpool_fwd, so values and window-local argmax indices are the same bit for bit.
template <int NS>
__global__ void __launch_bounds__(256, 4) pool2x2_shadow_kernel(const float *__restrict__ y, float *__restrict__ out, int *__restrict__ mask,
                                                             int C, int H, int W, int Cp, int items, int ptiles,
                                                             __nv_bfloat16 *__restrict__ d0, __nv_bfloat16 *__restrict__ d1,
                                                             __nv_bfloat16 *__restrict__ d2, Enc enc) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int cb = blockIdx.y * 64 + warp * 8;
    const int OW = W >> 1, Pq = (H >> 1) * OW;
    if (cb >= Cp) return;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int img = item / ptiles, q = (item - img * ptiles) * 32 + lane;
        if (q >= Pq) continue;
        const int oh = q / OW, ow = q - oh * OW;
        float2 a[8], b[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float *r = y + (((long long)img * C + min(cb + i, C - 1)) * H + 2 * oh) * W + 2 * ow;
            a[i] = __ldg(reinterpret_cast<const float2 *>(r));
            b[i] = __ldg(reinterpret_cast<const float2 *>(r + W));
        }
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float m = -FLT_MAX; int idx = 0;
            if (a[i].x > m) { m = a[i].x; idx = 0; } if (a[i].y > m) { m = a[i].y; idx = 1; }
            if (b[i].x > m) { m = b[i].x; idx = 2; } if (b[i].y > m) { m = b[i].y; idx = 3; }
            if (cb + i < C) {
                const long long o = ((long long)img * C + cb + i) * Pq + q;
                out[o] = m; mask[o] = idx;
            }
            v[i] = cb + i < C ? m : 0.f;
        }
        const long long o = ((long long)img * Pq + q) * Cp + cb;
        store_split8<NS>(v, enc, d0 + o, d1 + o, d2 + o);
    }
}

static bool conv_ok(int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw) {
    return NB >= 1 && C >= 1 && H >= 1 && W >= 1 && F >= 1 && R >= 1 && S >= 1 && sh >= 1 && sw >= 1 && ph >= 0 && pw >= 0 &&
           (long long)NB * (C > F ? C : F) * H * W * (long long)(sh * sw) < (1LL << 31);
}
// limits of the im2col descriptor: traversal strides <= 8, corner offsets within [-128, 127], batch <= 65535 for the shadow grid
static bool tma_conv_supported(int NB, int R, int S, int sh, int sw, int ph, int pw) {
    return sh <= 8 && sw <= 8 && ph <= 127 && pw <= 127 && R - 1 - ph <= 127 && S - 1 - pw <= 127 && ph <= R - 1 && pw <= S - 1 &&
           NB <= 65535;
}

}  // namespace seera

// Channels-last bf16 copies of one NCHW tensor, handed across calls (forward -> backward, activation backward ->
// convolution backward) so that they are produced once.
struct seera_shadow {
    seera::NhwcShadow s;
    int ns;
};

namespace seera {

static const NhwcShadow *usable(const seera_shadow *h, int ns, int NB, int C, int H, int W, int cls) {
    const Enc want = enc_for(cls);            // copies made under another encoding (bf16 against fp16) cannot be mixed in
    if (!h || h->ns < ns || h->s.NB != NB || h->s.C != C || h->s.H != H || h->s.W != W || h->s.enc.fmt != want.fmt ||
        h->s.enc.scale != want.scale || h->s.enc.dscale != want.dscale) return nullptr;
    return &h->s;
}

// Convolution backward; xk / dyk are optional kept shadows of X / dY (dY itself may then be null unless the short-patch
// weight gradient or a fallback needs the fp32 tensor).
static int tma_conv2d_bwd_kept(const float *Wt, const float *X, const float *dY, float *dX, float *dW, int NB, int C, int H, int W,
                               int F, int R, int S, int sh, int sw, int ph, int pw, const seera_shadow *xk, const seera_shadow *dyk) {
    SEERA_ENSURE();
    if (!conv_ok(NB, C, H, W, F, R, S, sh, sw, ph, pw) || !X || !Wt || (!dY && !dyk)) return fail(SEERA_E_ARG, "cuda_conv2d_bwd: bad argument");
    int OH = (H + 2 * ph - R) / sh + 1, OW = (W + 2 * pw - S) / sw + 1;
    if (OH < 1 || OW < 1) return fail(SEERA_E_ARG, "cuda_conv2d_bwd: kernel larger than padded input");
    const bool first = conv_first_applies(C, R, S);
    const bool phases = !(sh == 1 && sw == 1) && phases_supported(H, W, OH, OW, R, S, sh, sw, ph, pw);
    const bool need_fp32_dy = !tma_conv_supported(NB, R, S, sh, sw, ph, pw) || (dW && first) || (dX && !(sh == 1 && sw == 1) && !phases);
    if (need_fp32_dy && !dY) return fail(SEERA_E_ARG, "cuda_conv2d_bwd: this shape needs the fp32 output gradient");
    if (!tma_conv_supported(NB, R, S, sh, sw, ph, pw)) return seera_tc_conv2d_bwd(Wt, X, dY, dX, dW, NB, C, H, W, F, R, S, sh, sw, ph, pw);
    int ns = precision_copies();
    NhwcShadow dys_local, xs_local; Shadow wd;
    const NhwcShadow *dys = usable(dyk, ns, NB, F, OH, OW, CLS_GRAD), *xs = usable(xk, ns, NB, C, H, W, CLS_ACT);
    int s = SEERA_OK;
    if (!dys && (dX || (dW && !first))) {
        if (!dY) return fail(SEERA_E_ARG, "cuda_conv2d_bwd: kept gradient copies do not fit this call and no fp32 gradient was given");
        s = make_nhwc(dY, NB, F, OH, OW, ns, dys_local, CLS_GRAD);
        dys = &dys_local;
    }
    if (!s && dX) {
        if (sh == 1 && sw == 1) {     // dX = forward convolution of dY with flipped taps and swapped channel roles, pad' = K-1-pad
            s = make_weight_shadow(Wt, C, F, R * S, R * S, (long long)C * R * S, 1, ns, wd);
            if (!s) s = tma_fprop(*dys, wd, dX, C, R, S, 1, 1, R - 1 - ph, S - 1 - pw, H, W, ns, "cuda_conv2d_bwd(dX)");
        } else if (phases) {
            s = tma_dgrad_phases(*dys, Wt, R * S, (long long)C * R * S, dX, C, H, W, R, S, sh, sw, ph, pw, ns, "cuda_conv2d_bwd(dX)");
        } else {
            s = seera_tc_conv2d_bwd(Wt, X, dY, dX, nullptr, NB, C, H, W, F, R, S, sh, sw, ph, pw);
        }
    }
    if (!s && dW) {
        if (first) {                  // short patch: direct fp32 kernel on the NCHW tensors
            s = conv_first_wgrad(X, dY, dW, NB, C, H, W, F, R, S, sh, sw, ph, pw, "cuda_conv2d_bwd(dW)");
        } else {
            if (!xs) { s = make_nhwc(X, NB, C, H, W, ns, xs_local, CLS_ACT); xs = &xs_local; }
            if (!s) s = tma_wgrad(*xs, *dys, dW, R, S, sh, sw, ph, pw, wgrad_copies(ns), "cuda_conv2d_bwd(dW)");
        }
    }
    free_nhwc(dys_local); free_nhwc(xs_local); free_shadow(wd);
    return s;
}

}  // namespace seera

using namespace seera;

extern "C" {

int seera_tma_conv2d_fwd(const float *X, const float *Wt, float *Y, int NB, int C, int H, int W, int F, int R, int S,
                         int ph, int pw, int sh, int sw) {
    return seera_tma_conv2d_bias_act_fwd(X, Wt, nullptr, Y, NB, C, H, W, F, R, S, ph, pw, sh, sw, SEERA_ACT_NONE);
}

// Y = act(conv(X, Wt) + bias[f]); bias may be null.
int seera_tma_conv2d_bias_act_fwd(const float *X, const float *Wt, const float *bias, float *Y, int NB, int C, int H, int W, int F,
                                  int R, int S, int ph, int pw, int sh, int sw, int act) {
    SEERA_ENSURE();
    if (!conv_ok(NB, C, H, W, F, R, S, sh, sw, ph, pw) || !X || !Wt || !Y) return fail(SEERA_E_ARG, "cuda_conv2d_fwd: bad argument");
    int OH = (H + 2 * ph - R) / sh + 1, OW = (W + 2 * pw - S) / sw + 1;
    if (OH < 1 || OW < 1) return fail(SEERA_E_ARG, "cuda_conv2d_fwd: kernel larger than padded input");
    if (conv_first_applies(C, R, S))  // short patch: direct fp32 kernel
        return conv_first_fwd(X, Wt, bias, Y, NB, C, H, W, F, R, S, ph, pw, sh, sw, act, "cuda_conv2d_fwd");
    if (sh == 1 && sw == 1 && conv_few_applies(NB, C, F, R, S, OH, OW))       // a few filters: a stencil, not a GEMM
        return conv_few_fwd(X, Wt, bias, Y, NB, C, H, W, F, R, S, ph, pw, OH, OW, act, 0, "cuda_conv2d_fwd");
    if (!tma_conv_supported(NB, R, S, sh, sw, ph, pw)) {
        int s = seera_tc_conv2d_fwd(X, Wt, Y, NB, C, H, W, F, R, S, ph, pw, sh, sw);
        if (!s && (bias || act)) s = seera_bias_act_fwd(Y, bias, Y, NB * F * OH * OW, F, OH * OW, act);
        return s;
    }
    int ns = precision_copies();
    NhwcShadow xs; Shadow wk;
    int s = make_nhwc(X, NB, C, H, W, ns, xs, CLS_ACT);
    if (!s) s = make_weight_shadow(Wt, F, C, R * S, (long long)C * R * S, R * S, 0, ns, wk);
    if (!s) s = tma_fprop(xs, wk, Y, F, R, S, sh, sw, ph, pw, OH, OW, ns, "cuda_conv2d_fwd", bias, act);
    free_nhwc(xs); free_shadow(wk);
    return s;
}

int seera_tma_conv2d_bwd(const float *Wt, const float *X, const float *dY, float *dX, float *dW, int NB, int C, int H, int W,
                         int F, int R, int S, int sh, int sw, int ph, int pw) {
    return tma_conv2d_bwd_kept(Wt, X, dY, dX, dW, NB, C, H, W, F, R, S, sh, sw, ph, pw, nullptr, nullptr);
}

// ---- entries that hand channels-last copies from one call to the next ---------------------------------------------
static bool keeps_shadows(int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw) {
    return rt().precision && rt().conv_tma && conv_ok(NB, C, H, W, F, R, S, sh, sw, ph, pw) && tma_conv_supported(NB, R, S, sh, sw, ph, pw) &&
           !conv_first_applies(C, R, S);
}

void seera_shadow_free(seera_shadow_t *h) {
    if (!h) return;
    free_nhwc(h->s);
    delete h;
}

int seera_conv2d_bias_act_fwd_s(const float *X, const float *Wt, const float *bias, float *Y, int NB, int C, int H, int W, int F,
                                int R, int S, int ph, int pw, int sh, int sw, int act, seera_shadow_t *x_in, seera_shadow_t **x_keep) {
    SEERA_ENSURE();
    if (x_keep) *x_keep = nullptr;
    if (!keeps_shadows(NB, C, H, W, F, R, S, sh, sw, ph, pw))
        return seera_conv2d_bias_act_fwd(X, Wt, bias, Y, NB, C, H, W, F, R, S, ph, pw, sh, sw, act);
    if (!X || !Wt || !Y) return fail(SEERA_E_ARG, "cuda_conv2d_fwd: bad argument");
    int OH = (H + 2 * ph - R) / sh + 1, OW = (W + 2 * pw - S) / sw + 1;
    if (OH < 1 || OW < 1) return fail(SEERA_E_ARG, "cuda_conv2d_fwd: kernel larger than padded input");
    if (sh == 1 && sw == 1 && conv_few_applies(NB, C, F, R, S, OH, OW))       // reads X in place: no copies made, none kept
        return conv_few_fwd(X, Wt, bias, Y, NB, C, H, W, F, R, S, ph, pw, OH, OW, act, 0, "cuda_conv2d_fwd");
    int ns = precision_copies();
    NhwcShadow local; Shadow wk;
    const NhwcShadow *xs = usable(x_in, ns, NB, C, H, W, CLS_ACT);
    int s = SEERA_OK;
    if (!xs) { s = make_nhwc(X, NB, C, H, W, ns, local, CLS_ACT); xs = &local; }
    if (!s) s = make_weight_shadow(Wt, F, C, R * S, (long long)C * R * S, R * S, 0, ns, wk);
    if (!s) s = tma_fprop(*xs, wk, Y, F, R, S, sh, sw, ph, pw, OH, OW, ns, "cuda_conv2d_fwd", bias, act);
    free_shadow(wk);
    if (!s && x_keep && xs == &local) {
        *x_keep = new seera_shadow{local, ns};          // ownership of the device copies moves to the handle
    } else {
        free_nhwc(local);
    }
    return s;
}

int seera_maxpool2x2_fwd_s(const float *X, float *out, int *mask, int N, int C, int H, int W, seera_shadow_t **out_shadow) {
    SEERA_ENSURE();
    if (out_shadow) *out_shadow = nullptr;
    if (N < 1 || C < 1 || H < 2 || W < 2 || (H & 1) || (W & 1) || !X || !out || !mask) return fail(SEERA_E_ARG, "maxpool2x2_fwd: bad argument");
    const int Pq = (H / 2) * (W / 2), ptiles = (Pq + 31) / 32;
    const long long items = (long long)N * ptiles;
    if (!out_shadow || !rt().precision || !rt().conv_tma || N > 65535 || items > 0x7fffffff || (reinterpret_cast<uintptr_t>(X) & 7))
        return seera_cuda_maxpool_fwd(X, out, mask, N, C, H, W, 2, 2, 0, 0, 2, 2);
    const int ns = precision_copies();
    NhwcShadow sh;
    sh.NB = N; sh.H = H / 2; sh.W = W / 2; sh.C = C; sh.Cp = (C + 7) / 8 * 8;
    sh.enc = enc_for(CLS_ACT);
    size_t bytes = (size_t)N * Pq * sh.Cp * 2;
    for (int i = 0; i < ns; i++) { sh.p[i] = (__nv_bfloat16 *)scratch_alloc(bytes); if (!sh.p[i]) { free_nhwc(sh); return SEERA_E_OOM; } }
    const int cchunks = (sh.Cp + 63) / 64;
    int blocks = rt().sm_count * 4 / cchunks;           // one round of resident blocks (4 per SM)
    if (blocks < 1) blocks = 1;
    if (blocks > items) blocks = (int)items;
    dim3 grid((unsigned)blocks, (unsigned)cchunks);
    cudaStream_t st = rt().stream;
    // input read once; pooled values and argmax mask written; ns channels-last copies of the pooled tensor written
    ProfBytes pb(4.0 * N * C * H * W + 8.0 * N * C * Pq + (double)ns * bytes, "pool2x2_shadow");
    if (ns == 1) pool2x2_shadow_kernel<1><<<grid, 256, 0, st>>>(X, out, mask, C, H, W, sh.Cp, (int)items, ptiles, sh.p[0], sh.p[1], sh.p[2], sh.enc);
    else if (ns == 2) pool2x2_shadow_kernel<2><<<grid, 256, 0, st>>>(X, out, mask, C, H, W, sh.Cp, (int)items, ptiles, sh.p[0], sh.p[1], sh.p[2], sh.enc);
    else pool2x2_shadow_kernel<3><<<grid, 256, 0, st>>>(X, out, mask, C, H, W, sh.Cp, (int)items, ptiles, sh.p[0], sh.p[1], sh.p[2], sh.enc);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { free_nhwc(sh); return check_cuda(e, "maxpool2x2_fwd"); }
    *out_shadow = new seera_shadow{sh, ns};
    return SEERA_OK;
}

// ---- convolution + bias + activation + 2x2 max-pool in one launch ----------------------------------------------------
// In raster row order a 2x2 window must lie inside one epilogue warp's 32 rows: OW a power of two <= 16 and an even OH.
static bool pool_in_epilogue_ok(int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw) {
    if (!rt().precision || !rt().conv_tma || !conv_ok(NB, C, H, W, F, R, S, sh, sw, ph, pw)) return false;
    if (conv_first_applies(C, R, S))       // the fp32 stencil kernel always; the tensor-core short-patch kernel's pooled epilogue only on request
        return conv_pool_simt_applies(NB, C, H, W, F, R, S, sh, sw, ph, pw) || (rt().pool_short_patch && conv_first_pool_ok(NB, C, H, W, F, R, S, sh, sw, ph, pw));
    if (!tma_conv_supported(NB, R, S, sh, sw, ph, pw)) return false;
    const int OH = (H + 2 * ph - R) / sh + 1, OW = (W + 2 * pw - S) / sw + 1;
    return OH >= 2 && !(OH & 1) && (OW == 2 || OW == 4 || OW == 8 || OW == 16);
}
int seera_conv2d_pool_fusable(int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw) {
    if (ensure_init()) return 0;
    return pool_in_epilogue_ok(NB, C, H, W, F, R, S, sh, sw, ph, pw) ? 1 : 0;
}

int seera_conv2d_bias_act_pool_fwd_s(const float *X, const float *Wt, const float *bias, float *pooled, int *mask, int NB, int C, int H,
                                     int W, int F, int R, int S, int ph, int pw, int sh, int sw, int act, seera_shadow_t *x_in,
                                     seera_shadow_t **x_keep, seera_shadow_t **pooled_copies) {
    SEERA_ENSURE();
    if (x_keep) *x_keep = nullptr;
    if (pooled_copies) *pooled_copies = nullptr;
    if (!X || !Wt || !pooled || !mask) return fail(SEERA_E_ARG, "conv2d_pool_fwd: bad argument");
    if (!pool_in_epilogue_ok(NB, C, H, W, F, R, S, sh, sw, ph, pw))
        return fail(SEERA_E_LIMIT, "conv2d_pool_fwd: this shape or mode does not fold the pool in (see seera_conv2d_pool_fusable)");
    const int OH = (H + 2 * ph - R) / sh + 1, OW = (W + 2 * pw - S) / sw + 1;
    const int ns = precision_copies();
    PoolOut po{};
    po.pooled = pooled; po.mask = mask;
    NhwcShadow pc;                                     // copies of the pooled tensor, when the caller wants them
    if (pooled_copies) {
        pc.NB = NB; pc.H = OH / 2; pc.W = OW / 2; pc.C = F; pc.Cp = (F + 7) / 8 * 8;
        pc.enc = enc_for(CLS_ACT);
        size_t bytes = (size_t)NB * pc.H * pc.W * pc.Cp * 2;
        for (int i = 0; i < ns; i++) { pc.p[i] = (__nv_bfloat16 *)scratch_alloc(bytes); if (!pc.p[i]) { free_nhwc(pc); return SEERA_E_OOM; } }
        for (int i = 0; i < 3; i++) po.copy[i] = pc.p[i];
        po.ns = ns; po.Cp = pc.Cp; po.enc = pc.enc;
    }
    int s;
    if (conv_first_applies(C, R, S)) {
        s = conv_first_pool_fwd(X, Wt, bias, po, NB, C, H, W, F, R, S, ph, pw, sh, sw, act, "conv2d_pool_fwd");
    } else {
        NhwcShadow local; Shadow wk;
        const NhwcShadow *xs = usable(x_in, ns, NB, C, H, W, CLS_ACT);
        s = SEERA_OK;
        if (!xs) { s = make_nhwc(X, NB, C, H, W, ns, local, CLS_ACT); xs = &local; }
        if (!s) s = make_weight_shadow(Wt, F, C, R * S, (long long)C * R * S, R * S, 0, ns, wk);
        if (!s) s = tma_fprop(*xs, wk, nullptr, F, R, S, sh, sw, ph, pw, OH, OW, ns, "conv2d_pool_fwd", bias, act, &po);
        free_shadow(wk);
        if (!s && x_keep && xs == &local) *x_keep = new seera_shadow{local, ns};
        else free_nhwc(local);
    }
    if (!s && pooled_copies) *pooled_copies = new seera_shadow{pc, ns};
    else free_nhwc(pc);
    return s;
}

// dz = dy * act'(y) as channels-last copies plus dbias; dy = g, or gp through a 2x2 / stride-2 max-pool mask.
static int make_dz_shadow(const float *g, const float *gp, const int *mask, const float *y, const float *yp, float *dbias, int NB, int C,
                          int H, int W, int act, int ns, NhwcShadow &out) {
    out.NB = NB; out.H = H; out.W = W; out.C = C; out.Cp = (C + 7) / 8 * 8;
    out.enc = enc_for(CLS_GRAD);
    size_t bytes = (size_t)NB * H * W * out.Cp * 2;
    for (int i = 0; i < ns; i++) { out.p[i] = (__nv_bfloat16 *)scratch_alloc(bytes); if (!out.p[i]) return SEERA_E_OOM; }
    const bool by_window = gp && (yp || act == SEERA_ACT_NONE);
    const int Pq = (H / 2) * (W / 2);
    const bool small = by_window && Pq >= 1 && Pq < 32 && (Pq & (Pq - 1)) == 0;     // several whole images per 32-window tile
    int lgPq = 0;
    while (small && (1 << lgPq) < Pq) lgPq++;
    const int P = H * W, ptiles = by_window ? (Pq + 31) / 32 : (P + 31) / 32, cchunks = (out.Cp + 63) / 64;
    const long long items = small ? (NB + (32 / Pq) - 1) / (32 / Pq) : (long long)NB * ptiles;
    int splits = rt().sm_count * 4 / cchunks;           // one round of resident blocks (4 per SM)
    if (splits < 1) splits = 1;
    if (splits > items) splits = (int)items;
    if (items > 0x7fffffff || cchunks > 65535) return fail(SEERA_E_LIMIT, "activation backward: tensor too large");
    float *partial = nullptr;
    if (dbias) { partial = (float *)scratch_alloc((size_t)splits * C * sizeof(float)); if (!partial) return SEERA_E_OOM; }
    dim3 grid((unsigned)splits, (unsigned)cchunks);
    cudaStream_t st = rt().stream;
    // by window: pooled gradient + mask (+ pooled output) read at a quarter of the layer's resolution; otherwise the
    // full-resolution gradient (or pooled gradient + mask) and the layer output; ns copies of dz written either way
    const double in_bytes = by_window ? 4.0 * NB * C * (P / 4) * (2 + (yp ? 1 : 0))
                                      : 4.0 * NB * C * ((g ? (double)P : 2.0 * (P / 4)) + (act ? (double)P : 0.0));
    ProfBytes pb(in_bytes + (double)ns * bytes, by_window ? "dz_shadow_window" : "dz_shadow");
    if (small) {
        if (ns == 1) dz_shadow_window_small_kernel<1><<<grid, 256, 0, st>>>(gp, mask, yp, NB, C, H, W, out.Cp, (int)items, lgPq, act, out.p[0], out.p[1], out.p[2], partial, out.enc);
        else if (ns == 2) dz_shadow_window_small_kernel<2><<<grid, 256, 0, st>>>(gp, mask, yp, NB, C, H, W, out.Cp, (int)items, lgPq, act, out.p[0], out.p[1], out.p[2], partial, out.enc);
        else dz_shadow_window_small_kernel<3><<<grid, 256, 0, st>>>(gp, mask, yp, NB, C, H, W, out.Cp, (int)items, lgPq, act, out.p[0], out.p[1], out.p[2], partial, out.enc);
    } else if (by_window) {
        if (ns == 1) dz_shadow_window_kernel<1><<<grid, 256, 0, st>>>(gp, mask, yp, C, H, W, out.Cp, (int)items, ptiles, act, out.p[0], out.p[1], out.p[2], partial, out.enc);
        else if (ns == 2) dz_shadow_window_kernel<2><<<grid, 256, 0, st>>>(gp, mask, yp, C, H, W, out.Cp, (int)items, ptiles, act, out.p[0], out.p[1], out.p[2], partial, out.enc);
        else dz_shadow_window_kernel<3><<<grid, 256, 0, st>>>(gp, mask, yp, C, H, W, out.Cp, (int)items, ptiles, act, out.p[0], out.p[1], out.p[2], partial, out.enc);
    } else
    if (ns == 1) dz_shadow_kernel<1><<<grid, 256, 0, st>>>(g, gp, mask, y, yp, C, H, W, out.Cp, (int)items, ptiles, act, out.p[0], out.p[1], out.p[2], partial, out.enc);
    else if (ns == 2) dz_shadow_kernel<2><<<grid, 256, 0, st>>>(g, gp, mask, y, yp, C, H, W, out.Cp, (int)items, ptiles, act, out.p[0], out.p[1], out.p[2], partial, out.enc);
    else dz_shadow_kernel<3><<<grid, 256, 0, st>>>(g, gp, mask, y, yp, C, H, W, out.Cp, (int)items, ptiles, act, out.p[0], out.p[1], out.p[2], partial, out.enc);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && dbias) {
        launch_sum_splits(partial, dbias, C, splits, st);
        e = cudaGetLastError();
    }
    if (partial) scratch_free(partial);
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, "activation backward (channels-last)");
}

int seera_conv2d_act_bwd(const float *Wt, const float *X, const float *y, const float *g, const float *gp, const int *pool_mask,
                         const float *y_pooled, float *dX, float *dW, float *dbias, int NB, int C, int H, int W, int F, int R, int S, int sh, int sw,
                         int ph, int pw, int act, seera_shadow_t *x_shadow) {
    SEERA_ENSURE();
    if (!conv_ok(NB, C, H, W, F, R, S, sh, sw, ph, pw) || !X || !Wt || (g == nullptr) == (gp == nullptr) || (gp && !pool_mask) ||
        (act != SEERA_ACT_NONE && !y && !(gp && y_pooled)))
        return fail(SEERA_E_ARG, "conv2d_act_bwd: bad argument");
    int OH = (H + 2 * ph - R) / sh + 1, OW = (W + 2 * pw - S) / sw + 1;
    if (OH < 1 || OW < 1) return fail(SEERA_E_ARG, "conv2d_act_bwd: kernel larger than padded input");
    if (gp && ((OH & 1) || (OW & 1))) return fail(SEERA_E_ARG, "conv2d_act_bwd: pooled gradient needs even output height and width");
    const long long out_elems = (long long)NB * F * OH * OW;
    if (keeps_shadows(NB, C, H, W, F, R, S, sh, sw, ph, pw) &&
        (sh == 1 && sw == 1 ? true : phases_supported(H, W, OH, OW, R, S, sh, sw, ph, pw) || !dX)) {
        seera_shadow dz{NhwcShadow{}, precision_copies()};
        int s = make_dz_shadow(g, gp, pool_mask, y, gp ? y_pooled : nullptr, dbias, NB, F, OH, OW, act, dz.ns, dz.s);
        if (!s) s = tma_conv2d_bwd_kept(Wt, X, nullptr, dX, dW, NB, C, H, W, F, R, S, sh, sw, ph, pw, x_shadow, &dz);
        free_nhwc(dz.s);
        return s;
    }
    if (rt().precision && rt().conv_tma && conv_first_applies(C, R, S) && !dX && dW && (!dbias || conv_first_fuses_bias(C, R, S)))
        return conv_first_act_wgrad(X, y, g, gp, pool_mask, gp ? y_pooled : nullptr, dW, dbias, NB, C, H, W, F, R, S, sh, sw, ph, pw, act,
                                    "conv2d_act_bwd");
    // composition of the separate entries
    if (act != SEERA_ACT_NONE && !y && !(gp && y_pooled)) return fail(SEERA_E_ARG, "conv2d_act_bwd: this shape needs the layer output");
    float *dy_full = nullptr, *dz = nullptr, *gq = nullptr;
    int s = SEERA_OK;
    dz = (float *)scratch_alloc((size_t)out_elems * sizeof(float));
    if (!dz) return SEERA_E_OOM;
    if (gp && (y_pooled || act == SEERA_ACT_NONE)) {
        // slope and bias sums at pooled resolution (the pool's output is y wherever the routed gradient is not zero),
        // then the pool backward spreads the result
        gq = (float *)scratch_alloc((size_t)(out_elems / 4) * sizeof(float));
        if (!gq) s = SEERA_E_OOM;
        if (!s) s = seera_act_bias_bwd(gp, y_pooled, gq, dbias, (int)(out_elems / 4), F, (OH / 2) * (OW / 2), act);
        if (!s) s = seera_cuda_maxpool_bwd(gq, pool_mask, dz, NB, F, OH, OW, 2, 2, 0, 0, 2, 2);
    } else {
        if (gp) {
            dy_full = (float *)scratch_alloc((size_t)out_elems * sizeof(float));
            if (!dy_full) s = SEERA_E_OOM;
            if (!s) s = seera_cuda_maxpool_bwd(gp, pool_mask, dy_full, NB, F, OH, OW, 2, 2, 0, 0, 2, 2);
        }
        if (!s) s = seera_act_bias_bwd(gp ? dy_full : g, y, dz, dbias, (int)out_elems, F, OH * OW, act);
    }
    if (!s) s = seera_cuda_conv2d_bwd(Wt, X, dz, dX, dW, NB, C, H, W, F, R, S, sh, sw, ph, pw);
    if (dy_full) scratch_free(dy_full);
    if (gq) scratch_free(gq);
    scratch_free(dz);
    return s;
}

// Transposed convolution X[NB,Cin,H,W], Wt[Cin,Cout,KH,KW] -> out[NB,Cout,Ho,Wo]: the data gradient of the convolution
// whose filter bank has Cin filters over Cout channels.
int seera_tma_convT_fwd(const float *X, const float *Wt, float *out, int NB, int Cin, int H, int W, int Cout, int KH, int KW,
                        int sh, int sw, int ph, int pw) {
    return seera_tma_convT_bias_act_fwd(X, Wt, nullptr, out, NB, Cin, H, W, Cout, KH, KW, sh, sw, ph, pw, SEERA_ACT_NONE);
}

// out = act(convT(X, Wt) + bias[cout]); bias may be null.
int seera_tma_convT_bias_act_fwd(const float *X, const float *Wt, const float *bias, float *out, int NB, int Cin, int H, int W,
                                 int Cout, int KH, int KW, int sh, int sw, int ph, int pw, int act) {
    SEERA_ENSURE();
    int Ho = (H - 1) * sh - 2 * ph + KH, Wo = (W - 1) * sw - 2 * pw + KW;
    if (!conv_ok(NB, Cin, H, W, Cout, KH, KW, sh, sw, ph, pw) || Ho < 1 || Wo < 1 || !X || !Wt || !out)
        return fail(SEERA_E_ARG, "cuda_conv2DTranpose_fwd: bad argument");
    const bool unit = sh == 1 && sw == 1;
    if (unit && conv_few_applies(NB, Cin, Cout, KH, KW, Ho, Wo))        // a few output channels: a stencil, not a GEMM
        return conv_few_fwd(X, Wt, bias, out, NB, Cin, H, W, Cout, KH, KW, KH - 1 - ph, KW - 1 - pw, Ho, Wo, act, 1, "cuda_conv2DTranpose_fwd");
    if (!tma_conv_supported(NB, KH, KW, sh, sw, ph, pw) || (!unit && !phases_supported(Ho, Wo, H, W, KH, KW, sh, sw, ph, pw)) ||
        (!unit && (bias || act) && (sh > KH || sw > KW))) {
        int s = seera_tc_convT_fwd(X, Wt, out, NB, Cin, H, W, Cout, KH, KW, sh, sw, ph, pw);
        if (!s && (bias || act)) s = seera_bias_act_fwd(out, bias, out, NB * Cout * Ho * Wo, Cout, Ho * Wo, act);
        return s;
    }
    int ns = precision_copies();
    NhwcShadow xs; Shadow wd;
    int taps = KH * KW;
    int s = make_nhwc(X, NB, Cin, H, W, ns, xs, CLS_ACT);
    if (!s && unit) {
        s = make_weight_shadow(Wt, Cout, Cin, taps, taps, (long long)Cout * taps, 1, ns, wd);
        if (!s) s = tma_fprop(xs, wd, out, Cout, KH, KW, 1, 1, KH - 1 - ph, KW - 1 - pw, Ho, Wo, ns, "cuda_conv2DTranpose_fwd", bias, act);
    } else if (!s) {
        s = tma_dgrad_phases(xs, Wt, taps, (long long)Cout * taps, out, Cout, Ho, Wo, KH, KW, sh, sw, ph, pw, ns, "cuda_conv2DTranpose_fwd",
                             bias, act);
    }
    free_nhwc(xs); free_shadow(wd);
    return s;
}

int seera_tma_convT_bwd(const float *Wt, const float *X, const float *dY, float *dX, float *dW, int NB, int Cin, int H, int W,
                        int Cout, int KH, int KW, int sh, int sw, int ph, int pw) {
    SEERA_ENSURE();
    int Ho = (H - 1) * sh - 2 * ph + KH, Wo = (W - 1) * sw - 2 * pw + KW;
    if (!conv_ok(NB, Cin, H, W, Cout, KH, KW, sh, sw, ph, pw) || Ho < 1 || Wo < 1 || !X || !Wt || !dY ||
        (Ho + 2 * ph - KH) / sh + 1 != H || (Wo + 2 * pw - KW) / sw + 1 != W)
        return fail(SEERA_E_ARG, "cuda_conv2DTranspose_bwd: bad argument");
    if (!tma_conv_supported(NB, KH, KW, sh, sw, ph, pw))
        return seera_tc_convT_bwd(Wt, X, dY, dX, dW, NB, Cin, H, W, Cout, KH, KW, sh, sw, ph, pw);
    if (conv_first_applies(Cout, KH, KW)) {      // short patch on the output side (e.g. a one-channel image): direct fp32 kernels
        int s = SEERA_OK;
        if (dX) s = conv_first_fwd(dY, Wt, nullptr, dX, NB, Cout, Ho, Wo, Cin, KH, KW, ph, pw, sh, sw, SEERA_ACT_NONE, "cuda_conv2DTranspose_bwd(dX)");
        if (!s && dW) s = conv_first_wgrad(dY, X, dW, NB, Cout, Ho, Wo, Cin, KH, KW, sh, sw, ph, pw, "cuda_conv2DTranspose_bwd(dW)");
        return s;
    }
    int ns = precision_copies();
    int taps = KH * KW;
    NhwcShadow dys, xs; Shadow wk;
    int s = make_nhwc(dY, NB, Cout, Ho, Wo, ns, dys, CLS_GRAD);
    if (!s && dX) {      // dX[NB,Cin,H,W] = convolution of dY with Wt read as [F = Cin][C = Cout][KH][KW]
        s = make_weight_shadow(Wt, Cin, Cout, taps, (long long)Cout * taps, taps, 0, ns, wk);
        if (!s) s = tma_fprop(dys, wk, dX, Cin, KH, KW, sh, sw, ph, pw, H, W, ns, "cuda_conv2DTranspose_bwd(dX)");
    }
    if (!s && dW) {      // dW[Cin][Cout][KH][KW]: weight gradient of that convolution with dY as its input and X as its output gradient
        s = make_nhwc(X, NB, Cin, H, W, ns, xs, CLS_ACT);
        if (!s) s = tma_wgrad(dys, xs, dW, KH, KW, sh, sw, ph, pw, wgrad_copies(ns), "cuda_conv2DTranspose_bwd(dW)");
    }
    free_nhwc(dys); free_nhwc(xs); free_shadow(wk);
    return s;
}

}  // extern "C"
