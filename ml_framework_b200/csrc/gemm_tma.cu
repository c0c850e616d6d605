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
#include <cuda.h>

#include "common.cuh"
#include "contraction_functors.cuh"
#include "internal.h"
#include "tc_epilogue.cuh"
#include "tc_ptx.cuh"

namespace seera {

// ---- tensor maps -----------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) {
            cudaGetLastError();
            return nullptr;
        }
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// bf16 row-major matrix [rows, cols] with pitch ld (elements, multiple of 8): 2-D map, inner dimension = cols.
// Box = box_inner x box_outer elements, 128-byte swizzle, out-of-range elements read as zero.
static int make_map_2d(CUtensorMap *m, const void *base, int rows, int cols, int ld, int box_inner, int box_outer) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(SEERA_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SEERA_E_CUDA, "cuTensorMapEncodeTiled failed (%d) for %dx%d ld %d box %dx%d", (int)r, rows, cols, ld,
                                       box_inner, box_outer);
    return SEERA_OK;
}

// ---- fp32 -> bf16 shadow (hi, and the residual lo = bf16(x - hi) for bf16x3) -------------------------------
template <bool SPLIT>
__global__ void __launch_bounds__(256) shadow_rows_kernel(const float *__restrict__ src, long long src_ld, int rows, int cols,
                                                          __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo, int ld) {
    // one thread per 8 consecutive elements of a row; ld is a multiple of 8 so the 16-byte stores are aligned
    long long groups_per_row = ld >> 3, total = (long long)rows * groups_per_row;
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long g = tid; g < total; g += nthr) {
        int r = (int)(g / groups_per_row), c0 = (int)(g - (long long)r * groups_per_row) * 8;
        const float *s = src + (long long)r * src_ld + c0;
        float v[8];
        if (c0 + 8 <= cols && ((reinterpret_cast<uintptr_t>(s) & 15) == 0)) {
            float4 a = __ldg(reinterpret_cast<const float4 *>(s)), b = __ldg(reinterpret_cast<const float4 *>(s) + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = (c0 + i < cols) ? __ldg(s + i) : 0.f;
        }
        uint4 h;
        h.x = pack_bf16x2(v[0], v[1]); h.y = pack_bf16x2(v[2], v[3]); h.z = pack_bf16x2(v[4], v[5]); h.w = pack_bf16x2(v[6], v[7]);
        *reinterpret_cast<uint4 *>(hi + (long long)r * ld + c0) = h;
        if (SPLIT) {
            const uint32_t w[4] = {h.x, h.y, h.z, h.w};
            float e[8];
#pragma unroll
            for (int i = 0; i < 8; i++) e[i] = v[i] - __uint_as_float((i & 1) ? (w[i >> 1] & 0xFFFF0000u) : (w[i >> 1] << 16));
            uint4 l;
            l.x = pack_bf16x2(e[0], e[1]); l.y = pack_bf16x2(e[2], e[3]); l.z = pack_bf16x2(e[4], e[5]); l.w = pack_bf16x2(e[6], e[7]);
            *reinterpret_cast<uint4 *>(lo + (long long)r * ld + c0) = l;
        }
    }
}

struct Shadow {
    __nv_bfloat16 *hi = nullptr, *lo = nullptr;
    int rows = 0, cols = 0, ld = 0;
};

static int make_shadow(const float *src, int rows, int cols, bool split, Shadow &s) {
    s.rows = rows; s.cols = cols; s.ld = (cols + 7) / 8 * 8;
    size_t bytes = (size_t)rows * s.ld * 2;
    s.hi = (__nv_bfloat16 *)scratch_alloc(bytes);
    if (!s.hi) return SEERA_E_OOM;
    if (split) { s.lo = (__nv_bfloat16 *)scratch_alloc(bytes); if (!s.lo) return SEERA_E_OOM; }
    long long groups = (long long)rows * (s.ld / 8);
    if (split) shadow_rows_kernel<true><<<stride_grid(groups), 256, 0, rt().stream>>>(src, cols, rows, cols, s.hi, s.lo, s.ld);
    else shadow_rows_kernel<false><<<stride_grid(groups), 256, 0, rt().stream>>>(src, cols, rows, cols, s.hi, s.lo, s.ld);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, "shadow_rows");
}
static void free_shadow(Shadow &s) {
    if (s.hi) scratch_free(s.hi);
    if (s.lo) scratch_free(s.lo);
    s.hi = s.lo = nullptr;
}

// ---- TMA + mbarrier PTX -------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}

// MN-major operand tile: 64 contiguous row-index elements (128 bytes) per k line, 8 k lines per 1024-byte
// atom; atoms of the next 64 row indices start box_bytes later.
__device__ __forceinline__ uint64_t umma_desc_sw128_mn(uint32_t addr, uint32_t box_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((box_bytes >> 4) & 0x3FFF) << 16;   // leading byte offset: next 64 elements along M/N
    d |= (uint64_t)(1024 >> 4) << 32;                   // stride byte offset: next 8 k lines
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

struct TmaGemmParams {
    int M, N, K, kchunk, bn, stages;
    int a_mn, b_mn;          // 1: operand is read along its contiguous row index (MN-major), 0: K-major
    float *partial;
    int *status;
};

constexpr int TG_THREADS = 192;

template <bool SPLIT, class CS>
__global__ void __launch_bounds__(TG_THREADS, 1)
tma_gemm_kernel(const __grid_constant__ CUtensorMap mapAh, const __grid_constant__ CUtensorMap mapAl,
                const __grid_constant__ CUtensorMap mapBh, const __grid_constant__ CUtensorMap mapBl, CS cs, TmaGemmParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * 8 + 1];
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
    const uint32_t smem0 = smem_u32(smem);
    auto a_hi = [&](int s) { return smem0 + (uint32_t)s * stage_bytes; };
    auto a_lo = [&](int s) { return a_hi(s) + a_bytes; };
    auto b_hi = [&](int s) { return a_hi(s) + (SPLIT ? 2u : 1u) * a_bytes; };
    auto b_lo = [&](int s) { return b_hi(s) + b_bytes; };
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[8]), accum = smem_u32(&bars[16]);
    const uint32_t tmem_cols = (uint32_t)(bn < 32 ? 32 : bn);

    if (t == 0) {
        abort_flag = 0;
        for (int s = 0; s < stages; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(accum, 1);
        fence_mbar_init();
        fence_async_smem();
    }
    if (warp == 1) tmem_alloc(smem_u32(&tmem_base_slot), tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int *abortp = &abort_flag;

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ----------------
        int issued = 0;
        for (int kt = 0; kt < ktiles; kt++) {
            int s = kt % stages;
            uint32_t ph = (uint32_t)(kt / stages) & 1u;
            if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abortp, p.status, 1)) break;
            int k0 = kbeg + kt * TC_BK;
            uint32_t bar = full0 + 8 * s;
            mbar_expect_tx(bar, stage_bytes);
            if (p.a_mn) {
                for (int b = 0; b < TC_BM / 64; b++) {
                    tma_load_2d(a_hi(s) + b * 8192, &mapAh, m0 + 64 * b, k0, bar);
                    if (SPLIT) tma_load_2d(a_lo(s) + b * 8192, &mapAl, m0 + 64 * b, k0, bar);
                }
            } else {
                tma_load_2d(a_hi(s), &mapAh, k0, m0, bar);
                if (SPLIT) tma_load_2d(a_lo(s), &mapAl, k0, m0, bar);
            }
            if (p.b_mn) {
                for (int b = 0; b < bn / 64; b++) {
                    tma_load_2d(b_hi(s) + b * 8192, &mapBh, n0 + 64 * b, k0, bar);
                    if (SPLIT) tma_load_2d(b_lo(s) + b * 8192, &mapBl, n0 + 64 * b, k0, bar);
                }
            } else {
                tma_load_2d(b_hi(s), &mapBh, k0, n0, bar);
                if (SPLIT) tma_load_2d(b_lo(s), &mapBl, k0, n0, bar);
            }
            issued = kt + 1;
        }
        if (*abortp) {
            // give copies already in flight a bounded chance to land before the CTA's shared memory goes away
            for (int kt = max(0, issued - stages); kt < issued; kt++) {
                unsigned long long t0 = clock64();
                while (!mbar_try_wait(full0 + 8 * (kt % stages), (uint32_t)(kt / stages) & 1u) && clock64() - t0 < TC_WAIT_CLOCKS) {}
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer ----------------
        const uint32_t idesc = umma_idesc_bf16(bn) | ((uint32_t)p.a_mn << 15) | ((uint32_t)p.b_mn << 16);
        const uint32_t a_step = p.a_mn ? 2048u : 32u, b_step = p.b_mn ? 2048u : 32u;   // bytes per K=16 slice
        bool alive = true;
        uint32_t acc = 0;
        for (int kt = 0; kt < ktiles && alive; kt++) {
            int s = kt % stages;
            uint32_t ph = (uint32_t)(kt / stages) & 1u;
            alive = mbar_wait(full0 + 8 * s, ph, abortp, p.status, 2);
            if (!alive) break;
            tc_fence_after();
#pragma unroll
            for (int j = 0; j < TC_BK / 16; j++) {
                uint32_t ao = j * a_step, bo = j * b_step;
                uint64_t da = p.a_mn ? umma_desc_sw128_mn(a_hi(s) + ao, 8192) : umma_desc_sw128(a_hi(s) + ao);
                uint64_t db = p.b_mn ? umma_desc_sw128_mn(b_hi(s) + bo, 8192) : umma_desc_sw128(b_hi(s) + bo);
                umma_bf16(tmem_base, da, db, idesc, acc);
                acc = 1;
                if (SPLIT) {
                    uint64_t dal = p.a_mn ? umma_desc_sw128_mn(a_lo(s) + ao, 8192) : umma_desc_sw128(a_lo(s) + ao);
                    uint64_t dbl = p.b_mn ? umma_desc_sw128_mn(b_lo(s) + bo, 8192) : umma_desc_sw128(b_lo(s) + bo);
                    umma_bf16(tmem_base, da, dbl, idesc, 1);
                    umma_bf16(tmem_base, dal, db, idesc, 1);
                }
            }
            umma_commit(empty0 + 8 * s);
        }
        if (alive) umma_commit(accum);
    } else if (warp >= 2) {
        // ---------------- epilogue: warp w drains TMEM lane quarter w % 4 ----------------
        bool ok = mbar_wait(accum, 0, abortp, p.status, 3);
        tc_fence_after();
        if (ok) {
            // every MMA has completed, so the operand stages are free: reuse them as per-warp staging
            const int q = warp & 3;
            float *stage = reinterpret_cast<float *>(smem + (size_t)(warp - 2) * EPI_WARP_SMEM);
            drain_accumulator(tmem_base + ((uint32_t)(q * 32) << 16), m0 + q * 32, n0, 0, bn, p.M, p.N, cs, p.partial,
                              (long long)blockIdx.z * p.M * p.N, stage);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

template <class CS>
__global__ void __launch_bounds__(256) tma_splitk_reduce_kernel(const float *__restrict__ partial, CS cs, int M, int N, int splits) {
    long long total = (long long)M * N;
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long i = tid; i < total; i += nthr) {
        float s = 0.f;
        for (int z = 0; z < splits; z++) s += partial[(long long)z * total + i];
        cs((int)(i / N), (int)(i % N), s);
    }
}

int *tc_status_word();

// A operand: shadow `sa`; a_mn = 0: sa is [M, K] (read along its rows); a_mn = 1: sa is [K, M].  Likewise B with N.
template <class CS>
static int run_tma_gemm(const Shadow &sa, int a_mn, const Shadow &sb, int b_mn, const CS &cs, int M, int N, int K,
                        bool allow_split, const char *name) {
    const bool split3 = rt().precision == 2;
    int bn = N <= 32 ? 32 : (N <= 64 ? 64 : (N <= 128 ? 128 : 256));
    if (b_mn && bn < 64) bn = 64;
    if (split3 && bn > 128) bn = 128;
    size_t stage = (size_t)(split3 ? 2 : 1) * (TC_BM * 128 + (size_t)bn * 128);
    int stages = (int)((200 * 1024) / stage);
    if (stages > 8) stages = 8;
    if (stages < 2) return fail(SEERA_E_LIMIT, "%s: tile does not fit shared memory", name);
    size_t smem = stage * stages + 1024;
    long long tiles = (long long)((M + TC_BM - 1) / TC_BM) * ((N + bn - 1) / bn);
    int splits = 1;
    if (allow_split) {
        long long want = (rt().sm_count + tiles - 1) / tiles;
        long long maxs = K / (TC_BK * 4);
        splits = (int)(want < maxs ? want : maxs);
        if (splits < 1) splits = 1;
        if (splits > 256) splits = 256;
    }
    int kchunk = ((K + splits - 1) / splits + TC_BK - 1) / TC_BK * TC_BK;
    splits = (K + kchunk - 1) / kchunk;

    CUtensorMap mAh, mAl, mBh, mBl;
    int s;
    // K-major: inner dimension = K (cols of the shadow), box 64 x rows-of-tile; MN-major: inner = M/N, box 64 x 64 k lines
    if ((s = make_map_2d(&mAh, sa.hi, sa.rows, sa.cols, sa.ld, 64, a_mn ? 64 : TC_BM))) return s;
    if ((s = make_map_2d(&mBh, sb.hi, sb.rows, sb.cols, sb.ld, 64, b_mn ? 64 : bn))) return s;
    mAl = mAh; mBl = mBh;
    if (split3) {
        if ((s = make_map_2d(&mAl, sa.lo, sa.rows, sa.cols, sa.ld, 64, a_mn ? 64 : TC_BM))) return s;
        if ((s = make_map_2d(&mBl, sb.lo, sb.rows, sb.cols, sb.ld, 64, b_mn ? 64 : bn))) return s;
    }
    float *partial = nullptr;
    if (splits > 1) {
        partial = (float *)scratch_alloc((size_t)splits * M * N * sizeof(float));
        if (!partial) return SEERA_E_OOM;
    }
    dim3 grid((M + TC_BM - 1) / TC_BM, (N + bn - 1) / bn, splits);
    TmaGemmParams p{M, N, K, kchunk, bn, stages, a_mn, b_mn, partial, tc_status_word()};
    cudaStream_t st = rt().stream;
    cudaError_t e;
    profile_begin();
    if (split3) {
        auto kern = tma_gemm_kernel<true, CS>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) { kern<<<grid, TG_THREADS, smem, st>>>(mAh, mAl, mBh, mBl, cs, p); e = cudaGetLastError(); }
    } else {
        auto kern = tma_gemm_kernel<false, CS>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) { kern<<<grid, TG_THREADS, smem, st>>>(mAh, mAl, mBh, mBl, cs, p); e = cudaGetLastError(); }
    }
    count_launch();
    if (e == cudaSuccess && partial) {
        tma_splitk_reduce_kernel<<<stride_grid((long long)M * N), 256, 0, st>>>(partial, cs, M, N, splits);
        count_launch();
        e = cudaGetLastError();
    }
    if (partial) scratch_free(partial);
    profile_end(2.0 * M * N * (double)K);
    rt().tc_used = true;
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

}  // namespace seera

using namespace seera;

extern "C" {

int seera_tma_matmul(const float *A, const float *B, float *C, int M, int N, int K, int Nbatch) {
    SEERA_ENSURE();
    if (M < 1 || N < 1 || K < 1 || Nbatch < 1 || !A || !B || !C) return fail(SEERA_E_ARG, "cuda_matmul: bad argument");
    long long rows = (long long)M * Nbatch;
    if (rows > 0x7fffffff) return fail(SEERA_E_LIMIT, "cuda_matmul: batch*M too large");
    bool split = rt().precision == 2;
    Shadow sa, sb;
    int s = make_shadow(A, (int)rows, K, split, sa);
    if (!s) s = make_shadow(B, K, N, split, sb);
    if (!s) s = run_tma_gemm(sa, 0, sb, 1, StoreDense{C, N}, (int)rows, N, K, false, "cuda_matmul");
    free_shadow(sa); free_shadow(sb);
    return s;
}

int seera_tma_matmul_bwd(const float *A, const float *B, const float *dC, float *dA, float *dB, int M, int N, int K, int Nbatch) {
    SEERA_ENSURE();
    if (M < 1 || N < 1 || K < 1 || Nbatch < 1 || !A || !B || !dC) return fail(SEERA_E_ARG, "cuda_matmul_bwd: bad argument");
    long long rows = (long long)M * Nbatch;
    if (rows > 0x7fffffff) return fail(SEERA_E_LIMIT, "cuda_matmul_bwd: batch*M too large");
    bool split = rt().precision == 2;
    Shadow sd, sa, sb;
    int s = make_shadow(dC, (int)rows, N, split, sd);
    if (!s && dA) {      // dA[rows,K] = dC[rows,N] * B[K,N]^T : contraction over N, both operands read along their rows
        s = make_shadow(B, K, N, split, sb);
        if (!s) s = run_tma_gemm(sd, 0, sb, 0, StoreDense{dA, K}, (int)rows, K, N, false, "cuda_matmul_bwd(dA)");
    }
    if (!s && dB) {      // dB[K,N] = A[rows,K]^T * dC[rows,N] : contraction over rows, both operands read along their columns
        s = make_shadow(A, (int)rows, K, split, sa);
        if (!s) s = run_tma_gemm(sa, 1, sd, 1, StoreDense{dB, N}, K, N, (int)rows, true, "cuda_matmul_bwd(dB)");
    }
    free_shadow(sd); free_shadow(sa); free_shadow(sb);
    return s;
}

}  // extern "C"
