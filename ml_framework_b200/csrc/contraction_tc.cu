// Tensor-core contraction for sm_100a: tcgen05.mma with the accumulator in tensor memory (TMEM).
//
// One kernel serves every GEMM-shaped op of the training step (Dense forward / dA / dB, Conv2D forward /
// dX / dW, ConvTranspose2D forward / dX / dW; reference: engine_cuda/src/GEMM.cu, convolution.cu,
// upsampling.cu, all WMMA 16x16x16 with one warp per tile).  The boundary hands over fp32 NCHW tensors,
// so the operand tiles cannot come straight from a bulk copy: producer warps read the fp32 operands
// through the same functors as the CUDA-core kernel (plain strides, im2col, col2im, per-tap views),
// round them to bf16 and write them into shared memory in the K-major 128-byte-swizzled layout the
// tensor core reads.  Roles inside a CTA of 288 threads:
//
//   warps 0-7  producers  fill a ring of smem stages (A: 128 x 64, B: BN x 64 bf16), then
//                         fence.proxy.async + mbarrier arrive on full[stage]
//   warp 8     MMA        one thread waits full[stage], issues 4 (bf16) or 12 (bf16x3) tcgen05.mma
//                         of K=16 per stage into TMEM, tcgen05.commit -> empty[stage]
//   warps 0-7  epilogue   after the last commit, tcgen05.ld the 128 x BN fp32 accumulator (warp w reads
//                         lane quarter w%4, column half w/4) and store through the output functor
//
// Precision: mode 1 rounds both operands to bf16 once (fp32 accumulate).  Mode 2 ("bf16x3") splits every
// operand into hi = bf16(x) and lo = bf16(x - hi) and accumulates hi*hi + hi*lo + lo*hi, which keeps
// ~16 mantissa bits per operand and brings results to fp32-class accuracy at three MMAs per product.
//
// Every wait on an mbarrier is bounded by a clock budget; on expiry the kernel records a status word,
// all roles leave their loops, and TMEM is still released before the CTA exits.
#include "common.cuh"
#include "contraction_functors.cuh"
#include "tc_epilogue.cuh"
#include "tc_ptx.cuh"

namespace seera {

// Writes 8 consecutive-k values of one tile row as a 16-byte chunk (and, for bf16x3, the chunk of the
// rounding residuals) at the swizzled position of (row, kgroup).
template <bool SPLIT>
__device__ __forceinline__ void store_chunk(unsigned char *tile_hi, unsigned char *tile_lo, int row, int kg, const float *v) {
    uint32_t off = (uint32_t)row * 128u + (uint32_t)((kg ^ (row & 7)) << 4);
    uint4 h;
    h.x = pack_bf16x2(v[0], v[1]); h.y = pack_bf16x2(v[2], v[3]); h.z = pack_bf16x2(v[4], v[5]); h.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4 *>(tile_hi + off) = h;
    if (SPLIT) {
        float r[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            uint32_t word = (i & 1) ? ((&h.x)[i >> 1] & 0xFFFF0000u) : ((&h.x)[i >> 1] << 16);
            r[i] = v[i] - __uint_as_float(word);
        }
        uint4 l;
        l.x = pack_bf16x2(r[0], r[1]); l.y = pack_bf16x2(r[2], r[3]); l.z = pack_bf16x2(r[4], r[5]); l.w = pack_bf16x2(r[6], r[7]);
        *reinterpret_cast<uint4 *>(tile_lo + off) = l;
    }
}

// Fills one operand tile (ROWS x 64) of a stage.  KFAST: the 8 lanes of a row take its 8 k-groups
// (operand contiguous along k); otherwise lanes run along rows (operand contiguous along the row index).
template <bool SPLIT, bool KFAST, class L>
__device__ __forceinline__ void produce_tile(const L &ld, const typename L::Fx &fx_row, unsigned char *hi, unsigned char *lo,
                                             int rows, int row0, int k0, int kend, int t) {
    const int items = rows >> 5;                       // rows * 8 k-groups / 256 producer threads
    for (int j = 0; j < items; j++) {
        int row, kg;
        float v[8];
        if (KFAST) {
            kg = t & 7; row = (t >> 3) + 32 * j;
            typename L::Fx fx = ld.fix(row0 + row);
#pragma unroll
            for (int i = 0; i < 8; i++) { int k = k0 + kg * 8 + i; v[i] = k < kend ? ld.load(fx, k) : 0.f; }
        } else {
            row = t % rows; kg = t / rows + (TC_PRODUCERS / rows) * j;
#pragma unroll
            for (int i = 0; i < 8; i++) { int k = k0 + kg * 8 + i; v[i] = k < kend ? ld.load(fx_row, k) : 0.f; }
        }
        store_chunk<SPLIT>(hi, lo, row, kg, v);
    }
}

struct TcParams {
    int M, N, K, kchunk, bn, stages;
    float *partial;          // split-K partials [splits][M][N] or null
    int *status;             // device status word: 0 ok, otherwise the code of the wait that expired
};

template <bool SPLIT, bool A_KFAST, bool B_KFAST, class AL, class BL, class CS>
__global__ void __launch_bounds__(TC_THREADS, 1) tc_contraction_kernel(AL al, BL bl, CS cs, TcParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * 8 + 1];      // full[8], empty[8], accumulator
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int bn = p.bn, stages = p.stages;
    const int m0 = blockIdx.x * TC_BM, n0 = blockIdx.y * bn;
    const int kbeg = blockIdx.z * p.kchunk, kend = min(p.K, kbeg + p.kchunk);
    const int ktiles = (kend - kbeg + TC_BK - 1) / TC_BK;

    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t a_bytes = TC_BM * 128, b_bytes = (uint32_t)bn * 128;
    const uint32_t stage_bytes = (SPLIT ? 2u : 1u) * (a_bytes + b_bytes);
    auto a_hi = [&](int s) { return smem + (size_t)s * stage_bytes; };
    auto a_lo = [&](int s) { return a_hi(s) + a_bytes; };                       // only with SPLIT
    auto b_hi = [&](int s) { return a_hi(s) + (SPLIT ? 2u : 1u) * a_bytes; };
    auto b_lo = [&](int s) { return b_hi(s) + b_bytes; };
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[8]), accum = smem_u32(&bars[16]);

    if (t == 0) {
        abort_flag = 0;
        for (int s = 0; s < stages; s++) { mbar_init(full0 + 8 * s, TC_PRODUCERS); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(accum, 1);
        fence_mbar_init();
        fence_async_smem();
    }
    if (warp == 8) tmem_alloc(smem_u32(&tmem_base_slot), (uint32_t)(bn < 32 ? 32 : bn));
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int *abortp = &abort_flag;

    if (warp < 8) {
        // ---------------- producers ----------------
        typename AL::Fx afx = al.fix(m0 + (A_KFAST ? 0 : t % TC_BM));
        typename BL::Fx bfx = bl.fix(n0 + (B_KFAST ? 0 : t % bn));
        bool alive = true;
        for (int kt = 0; kt < ktiles && alive; kt++) {
            int s = kt % stages;
            uint32_t ph = (uint32_t)(kt / stages) & 1u;
            alive = mbar_wait(empty0 + 8 * s, ph ^ 1u, abortp, p.status, 1);
            if (!alive) break;
            int k0 = kbeg + kt * TC_BK;
            produce_tile<SPLIT, A_KFAST>(al, afx, a_hi(s), a_lo(s), TC_BM, m0, k0, kend, t);
            produce_tile<SPLIT, B_KFAST>(bl, bfx, b_hi(s), b_lo(s), bn, n0, k0, kend, t);
            fence_async_smem();                     // generic-proxy stores -> visible to the tensor core's reads
            mbar_arrive(full0 + 8 * s);
        }
    } else if (lane == 0) {
        // ---------------- MMA issuer ----------------
        const uint32_t idesc = umma_idesc_bf16(bn);
        bool alive = true;
        uint32_t first = 0;                          // 0 -> overwrite the accumulator, 1 -> accumulate
        for (int kt = 0; kt < ktiles && alive; kt++) {
            int s = kt % stages;
            uint32_t ph = (uint32_t)(kt / stages) & 1u;
            alive = mbar_wait(full0 + 8 * s, ph, abortp, p.status, 2);
            if (!alive) break;
            tc_fence_after();
            uint64_t da = umma_desc_sw128(smem_u32(a_hi(s))), db = umma_desc_sw128(smem_u32(b_hi(s)));
            uint64_t dal = 0, dbl = 0;
            if (SPLIT) { dal = umma_desc_sw128(smem_u32(a_lo(s))); dbl = umma_desc_sw128(smem_u32(b_lo(s))); }
#pragma unroll
            for (int j = 0; j < TC_BK / 16; j++) {   // K = 16 per instruction: 32 bytes along the swizzled row
                umma_bf16(tmem_base, da + 2 * j, db + 2 * j, idesc, first);
                first = 1;
                if (SPLIT) {
                    umma_bf16(tmem_base, da + 2 * j, dbl + 2 * j, idesc, 1);
                    umma_bf16(tmem_base, dal + 2 * j, db + 2 * j, idesc, 1);
                }
            }
            umma_commit(empty0 + 8 * s);             // the stage may be refilled once these MMAs have read it
        }
        if (alive) umma_commit(accum);               // accumulator complete
    }

    // ---------------- epilogue: TMEM -> registers -> output functor ----------------
    if (warp < 8 && ktiles > 0) {
        bool ok = mbar_wait(accum, 0, abortp, p.status, 3);
        tc_fence_after();
        if (ok) {
            const int q = warp & 3, half = warp >> 2;
            const int cols_per_half = bn >= 64 ? bn / 2 : bn;          // bn = 32: the second warp group has nothing to do
            if (bn >= 64 || half == 0) {
                // every MMA has completed, so the operand stages are free: reuse them as per-warp staging
                float *stage = reinterpret_cast<float *>(smem + (size_t)warp * EPI_WARP_SMEM);
                int cb = half * cols_per_half;
                drain_accumulator(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)cb, m0 + q * 32, n0, cb, cb + cols_per_half,
                                  p.M, p.N, cs, p.partial, (long long)blockIdx.z * p.M * p.N, stage);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) tmem_dealloc(tmem_base, (uint32_t)(bn < 32 ? 32 : bn));
}

template <class CS>
__global__ void __launch_bounds__(256) tc_splitk_reduce_kernel(const float *__restrict__ partial, CS cs, int M, int N, int splits) {
    long long total = (long long)M * N;
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long i = tid; i < total; i += nthr) {
        float s = 0.f;
        for (int z = 0; z < splits; z++) s += partial[(long long)z * total + i];
        cs((int)(i / N), (int)(i % N), s);
    }
}

int *tc_status_word() {
    static int *w = nullptr;
    if (!w) {
        if (cudaMalloc(&w, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        cudaMemsetAsync(w, 0, sizeof(int), rt().stream);
    }
    return w;
}

template <bool A_KFAST, bool B_KFAST, class AL, class BL, class CS>
int run_tc(const AL &al, const BL &bl, const CS &cs, int M, int N, int K, bool allow_split, const char *name) {
    if (M < 1 || N < 1 || K < 1) return fail(SEERA_E_ARG, "%s: empty problem %dx%dx%d", name, M, N, K);
    const bool split3 = rt().precision >= 2;      // mode 3 (three-way split) runs as the two-way split here
    int bn = N <= 32 ? 32 : (N <= 64 ? 64 : (N <= 128 ? 128 : 256));
    if (split3 && bn > 128) bn = 128;
    size_t stage = (size_t)(split3 ? 2 : 1) * (TC_BM * 128 + (size_t)bn * 128);
    int stages = (int)((200 * 1024) / stage);
    if (stages > 6) stages = 6;
    if (stages < 2) return fail(SEERA_E_LIMIT, "%s: tile does not fit shared memory", name);
    size_t smem = stage * stages + 1024;
    long long tiles = (long long)((M + TC_BM - 1) / TC_BM) * ((N + bn - 1) / bn);
    int splits = 1;
    if (allow_split) {
        long long want = (2LL * rt().sm_count + tiles - 1) / tiles;
        long long maxs = K / (TC_BK * 8);
        splits = (int)(want < maxs ? want : maxs);
        if (splits < 1) splits = 1;
        if (splits > 512) splits = 512;
    }
    int kchunk = ((K + splits - 1) / splits + TC_BK - 1) / TC_BK * TC_BK;
    splits = (K + kchunk - 1) / kchunk;
    float *partial = nullptr;
    if (splits > 1) {
        partial = (float *)scratch_alloc((size_t)splits * M * N * sizeof(float));
        if (!partial) return SEERA_E_OOM;
    }
    dim3 grid((M + TC_BM - 1) / TC_BM, (N + bn - 1) / bn, splits);
    if (grid.y > 65535 || grid.z > 65535) { if (partial) scratch_free(partial); return fail(SEERA_E_LIMIT, "%s: grid too large", name); }
    TcParams p{M, N, K, kchunk, bn, stages, partial, tc_status_word()};
    cudaStream_t st = rt().stream;
    cudaError_t e;
    profile_begin();
    if (split3) {
        auto kern = tc_contraction_kernel<true, A_KFAST, B_KFAST, AL, BL, CS>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) { kern<<<grid, TC_THREADS, smem, st>>>(al, bl, cs, p); e = cudaGetLastError(); }
    } else {
        auto kern = tc_contraction_kernel<false, A_KFAST, B_KFAST, AL, BL, CS>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) { kern<<<grid, TC_THREADS, smem, st>>>(al, bl, cs, p); e = cudaGetLastError(); }
    }
    count_launch();
    if (e == cudaSuccess && partial) {
        tc_splitk_reduce_kernel<<<stride_grid((long long)M * N), 256, 0, st>>>(partial, cs, M, N, splits);
        count_launch();
        e = cudaGetLastError();
    }
    if (partial) scratch_free(partial);
    profile_end(2.0 * M * N * (double)K, name);
    rt().tc_used = true;
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

// ---- convolution forms, M = output pixels ------------------------------------------------------------------
static int tc_conv_fprop(const float *X, const float *Wt, float *Y, int NB, int C, int H, int W, int F, int R, int S,
                         int sh, int sw, int ph, int pw, const char *name) {
    int OH = (H + 2 * ph - R) / sh + 1, OW = (W + 2 * pw - S) / sw + 1;
    if (OH < 1 || OW < 1) return fail(SEERA_E_ARG, "%s: kernel larger than padded input", name);
    int K = C * R * S, rows = NB * OH * OW;
    ConvGeom g{C, H, W, OH, OW, R, S, sh, sw, ph, pw};
    Strided b{Wt, K, 1, F, K};
    StorePixelRows cs{Y, F, OH * OW};
    if (R == 3 && S == 3) return run_tc<false, true>(Im2colByCol<9, 3>{X, g, rows, K}, b, cs, rows, F, K, false, name);
    return run_tc<false, true>(Im2colByCol<0, 0>{X, g, rows, K}, b, cs, rows, F, K, false, name);
}
static int tc_conv_dgrad(const float *dY, const float *Wt, float *dX, int NB, int C, int H, int W, int F, int R, int S,
                         int sh, int sw, int ph, int pw, int OH, int OW, const char *name) {
    int K = F * R * S, rows = NB * H * W;
    ConvGeom g{F, OH, OW, H, W, R, S, sh, sw, ph, pw};
    WeightByInChannel b{Wt, C, R * S, K};
    StorePixelRows cs{dX, C, H * W};
    if (R == 3 && S == 3) return run_tc<false, false>(Col2imByPixel<9, 3>{dY, g, rows, K}, b, cs, rows, C, K, false, name);
    return run_tc<false, false>(Col2imByPixel<0, 0>{dY, g, rows, K}, b, cs, rows, C, K, false, name);
}
// dW[f][(c,r,s)]: M = taps (c,r,s), N = F, contraction over (img, pixel); both operands are contiguous along it
static int tc_conv_wgrad(const float *dY, const float *X, float *dW, int NB, int C, int H, int W, int F, int R, int S,
                         int sh, int sw, int ph, int pw, int OH, int OW, const char *name) {
    int K = NB * OH * OW, taps = C * R * S;
    ConvGeom g{C, H, W, OH, OW, R, S, sh, sw, ph, pw};
    Im2colByTap a{X, g, taps, K};
    ByImagePixel b{dY, F, OH * OW, K};
    StoreDenseT cs{dW, taps};
    return run_tc<true, true>(a, b, cs, taps, F, K, true, name);
}

}  // namespace seera

using namespace seera;

extern "C" {

int seera_tc_matmul(const float *A, const float *B, float *C, int M, int N, int K, int Nbatch) {
    SEERA_ENSURE();
    if (M < 1 || N < 1 || K < 1 || Nbatch < 1 || !A || !B || !C) return fail(SEERA_E_ARG, "cuda_matmul: bad argument");
    long long rows = (long long)M * Nbatch;
    if (rows > 0x7fffffff) return fail(SEERA_E_LIMIT, "cuda_matmul: batch*M too large");
    Strided a{A, K, 1, (int)rows, K}, b{B, 1, N, N, K};                 // B(n,k) = B[k*N + n]: contiguous along n
    return run_tc<true, false>(a, b, StoreDense{C, N}, (int)rows, N, K, false, "cuda_matmul");
}

int seera_tc_matmul_bwd(const float *A, const float *B, const float *dC, float *dA, float *dB, int M, int N, int K, int Nbatch) {
    SEERA_ENSURE();
    if (M < 1 || N < 1 || K < 1 || Nbatch < 1 || !A || !B || !dC) return fail(SEERA_E_ARG, "cuda_matmul_bwd: bad argument");
    long long rows = (long long)M * Nbatch;
    if (rows > 0x7fffffff) return fail(SEERA_E_LIMIT, "cuda_matmul_bwd: batch*M too large");
    if (dA) {   // dA[rows,K] = dC[rows,N] * B^T: both operands contiguous along the contraction index n
        Strided a{dC, N, 1, (int)rows, N}, b{B, N, 1, K, N};
        if (int s = run_tc<true, true>(a, b, StoreDense{dA, K}, (int)rows, K, N, false, "cuda_matmul_bwd(dA)")) return s;
    }
    if (dB) {   // dB[K,N] = A^T * dC: M = K, contraction over rows; both operands contiguous along their row index
        Strided a{A, 1, K, K, (int)rows}, b{dC, 1, N, N, (int)rows};
        if (int s = run_tc<false, false>(a, b, StoreDense{dB, N}, K, N, (int)rows, true, "cuda_matmul_bwd(dB)")) return s;
    }
    return SEERA_OK;
}

static bool tc_conv_ok(int NB, int C, int H, int W, int F, int R, int S, int sh, int sw, int ph, int pw) {
    return NB >= 1 && C >= 1 && H >= 1 && W >= 1 && F >= 1 && R >= 1 && S >= 1 && sh >= 1 && sw >= 1 && ph >= 0 && pw >= 0 &&
           (long long)NB * (C > F ? C : F) * H * W * (long long)(sh * sw) < (1LL << 31);
}

int seera_tc_conv2d_fwd(const float *X, const float *Wt, float *Y, int NB, int C, int H, int W, int F, int R, int S,
                        int ph, int pw, int sh, int sw) {
    SEERA_ENSURE();
    if (!tc_conv_ok(NB, C, H, W, F, R, S, sh, sw, ph, pw) || !X || !Wt || !Y) return fail(SEERA_E_ARG, "cuda_conv2d_fwd: bad argument");
    return tc_conv_fprop(X, Wt, Y, NB, C, H, W, F, R, S, sh, sw, ph, pw, "cuda_conv2d_fwd");
}
int seera_tc_conv2d_bwd(const float *Wt, const float *X, const float *dY, float *dX, float *dW, int NB, int C, int H, int W,
                        int F, int R, int S, int sh, int sw, int ph, int pw) {
    SEERA_ENSURE();
    if (!tc_conv_ok(NB, C, H, W, F, R, S, sh, sw, ph, pw) || !X || !Wt || !dY) return fail(SEERA_E_ARG, "cuda_conv2d_bwd: bad argument");
    int OH = (H + 2 * ph - R) / sh + 1, OW = (W + 2 * pw - S) / sw + 1;
    if (OH < 1 || OW < 1) return fail(SEERA_E_ARG, "cuda_conv2d_bwd: kernel larger than padded input");
    if (dX) if (int s = tc_conv_dgrad(dY, Wt, dX, NB, C, H, W, F, R, S, sh, sw, ph, pw, OH, OW, "cuda_conv2d_bwd(dX)")) return s;
    if (dW) if (int s = tc_conv_wgrad(dY, X, dW, NB, C, H, W, F, R, S, sh, sw, ph, pw, OH, OW, "cuda_conv2d_bwd(dW)")) return s;
    return SEERA_OK;
}
int seera_tc_convT_fwd(const float *X, const float *Wt, float *out, int NB, int Cin, int H, int W, int Cout, int KH, int KW,
                       int sh, int sw, int ph, int pw) {
    SEERA_ENSURE();
    int Ho = (H - 1) * sh - 2 * ph + KH, Wo = (W - 1) * sw - 2 * pw + KW;
    if (!tc_conv_ok(NB, Cin, H, W, Cout, KH, KW, sh, sw, ph, pw) || Ho < 1 || Wo < 1 || !X || !Wt || !out)
        return fail(SEERA_E_ARG, "cuda_conv2DTranpose_fwd: bad argument");
    return tc_conv_dgrad(X, Wt, out, NB, Cout, Ho, Wo, Cin, KH, KW, sh, sw, ph, pw, H, W, "cuda_conv2DTranpose_fwd");
}
int seera_tc_convT_bwd(const float *Wt, const float *X, const float *dY, float *dX, float *dW, int NB, int Cin, int H, int W,
                       int Cout, int KH, int KW, int sh, int sw, int ph, int pw) {
    SEERA_ENSURE();
    int Ho = (H - 1) * sh - 2 * ph + KH, Wo = (W - 1) * sw - 2 * pw + KW;
    if (!tc_conv_ok(NB, Cin, H, W, Cout, KH, KW, sh, sw, ph, pw) || Ho < 1 || Wo < 1 || !X || !Wt || !dY ||
        (Ho + 2 * ph - KH) / sh + 1 != H || (Wo + 2 * pw - KW) / sw + 1 != W)
        return fail(SEERA_E_ARG, "cuda_conv2DTranspose_bwd: bad argument");
    if (dX) if (int s = tc_conv_fprop(dY, Wt, dX, NB, Cout, Ho, Wo, Cin, KH, KW, sh, sw, ph, pw, "cuda_conv2DTranspose_bwd(dX)")) return s;
    if (dW) if (int s = tc_conv_wgrad(X, dY, dW, NB, Cout, Ho, Wo, Cin, KH, KW, sh, sw, ph, pw, H, W, "cuda_conv2DTranspose_bwd(dW)")) return s;
    return SEERA_OK;
}

// Reads and clears the device status word of the tensor-core kernels (0 = every wait completed).
int seera_tc_device_status(void) {
    int *w = tc_status_word();
    if (!w) return -1;
    int v = 0;
    if (cudaMemcpyAsync(&v, w, sizeof(int), cudaMemcpyDeviceToHost, rt().stream) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(rt().stream) != cudaSuccess) return -1;
    if (v) cudaMemsetAsync(w, 0, sizeof(int), rt().stream);
    return v;
}

}  // extern "C"
