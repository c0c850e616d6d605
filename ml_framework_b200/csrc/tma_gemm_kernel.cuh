// TMA-fed tcgen05 GEMM kernel, tensor-map helpers and bf16 shadow conversion shared by the Dense and the
// convolution entry points.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "contraction_functors.cuh"
#include "tc_epilogue.cuh"
#include "tc_ptx.cuh"

namespace seera {


// ---- tensor maps -----------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
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
inline int make_map_2d(CUtensorMap *m, const void *base, int rows, int cols, int ld, int box_inner, int box_outer) {
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

// ---- fp32 -> bf16 shadows -----------------------------------------------------------------------------------
// NS = 1: hi = bf16(x).  NS = 2: plus lo = bf16(x - hi).  NS = 3: plus lo2 = bf16(x - hi - lo) (24 mantissa bits).
struct Shadow {
    __nv_bfloat16 *p[3] = {nullptr, nullptr, nullptr};      // 16-bit containers: bf16 or fp16 by `enc`
    int rows = 0, cols = 0, ld = 0;
    Enc enc{0, 1.f, nullptr};
};

// Classes of tensor, for the scale of an fp16 encoding: activations are O(1) after He / Glorot initialisation, weights a
// few hundredths, gradients of a batch-mean loss 1e-6 .. 1e-2.  With the factors 2^4 / 2^8 / 2^12 the second copy of a
// value stays a normal fp16 number down to a magnitude of 2^-7 / 2^-11 / 2^-15 (below that its absolute error is
// 2^-29 / 2^-33 / 2^-37, far under the products' own rounding); values saturate at 4094 / 255.9 / 15.99 - data beyond
// that belongs in the bf16 modes 2 and 3, which keep fp32's exponent range.
enum { CLS_ACT = 0, CLS_WEIGHT = 1, CLS_GRAD = 2 };

template <int NS>
__global__ void __launch_bounds__(256) shadow_rows_kernel(const float *__restrict__ src, long long src_ld, int rows, int cols,
                                                          __nv_bfloat16 *__restrict__ d0, __nv_bfloat16 *__restrict__ d1,
                                                          __nv_bfloat16 *__restrict__ d2, int ld, Enc enc, FastDiv by_groups) {
    // one thread per 8 consecutive elements of a row; ld is a multiple of 8 so the 16-byte stores are aligned
    long long groups_per_row = ld >> 3, total = (long long)rows * groups_per_row;
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    const bool small = total < (1ll << 31);       // then the row index is one multiply and a shift instead of a 64-bit division
    for (long long g = tid; g < total; g += nthr) {
        int r = small ? by_groups.div((int)g) : (int)(g / groups_per_row), c0 = (int)(g - (long long)r * groups_per_row) * 8;
        const float *s = src + (long long)r * src_ld + c0;
        float v[8];
        if (c0 + 8 <= cols && ((reinterpret_cast<uintptr_t>(s) & 15) == 0)) {
            float4 a = __ldg(reinterpret_cast<const float4 *>(s)), b = __ldg(reinterpret_cast<const float4 *>(s) + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = (c0 + i < cols) ? __ldg(s + i) : 0.f;
        }
        long long o = (long long)r * ld + c0;
        store_split8<NS>(v, enc, d0 + o, d1 + o, d2 + o);
    }
}

// Precision modes 1 / 2 / 3: one, two, three bf16 copies (1, 3, 6 products).  Mode 4: two fp16 copies (3 products).
// Mode 5: one fp16 copy (1 product) - the first copy of a mode-4 set, so copies kept by a mode-4 forward serve a mode-5 backward.
inline int precision_copies() { int m = rt().precision; return m == 4 ? 2 : (m == 5 ? 1 : (m < 1 ? 1 : (m > 3 ? 3 : m))); }
inline Enc enc_for(int cls) {
    if (rt().precision != 4 && rt().precision != 5) return Enc{0, 1.f, nullptr};
    static const float scale[3] = {16.f, 256.f, 4096.f};
    return Enc{1, scale[cls], cls == CLS_GRAD ? grad_scale_words() : nullptr};
}
// Copies a weight-gradient product uses.  Its rounding stays in that one tensor (nothing downstream of dW in the backward
// pass reads it), so with the "wgrad_single" option the fp16 split mode forms dW from the first copy of each operand alone:
// one product instead of three, 2e-4 of rounding in dW.
inline int wgrad_copies(int ns) { return (rt().wgrad_single && rt().precision == 4) ? 1 : ns; }
// The inverse of an operand's dynamic factor, for the epilogue (null: none).
inline const float *enc_dinv(const Enc &a, const Enc &b) { return (a.dscale || b.dscale) ? grad_scale_words() + 1 : nullptr; }

inline int alloc_shadow(Shadow &s, int rows, int cols, int ns) {
    s.rows = rows; s.cols = cols; s.ld = (cols + 7) / 8 * 8;
    for (int i = 0; i < ns; i++) {
        s.p[i] = (__nv_bfloat16 *)scratch_alloc((size_t)rows * s.ld * 2);
        if (!s.p[i]) return SEERA_E_OOM;
    }
    return SEERA_OK;
}
inline void free_shadow(Shadow &s) {
    for (int i = 0; i < 3; i++) { if (s.p[i]) scratch_free(s.p[i]); s.p[i] = nullptr; }
}
// Row-major fp32 [rows, cols] -> bf16 shadows of the same layout (pitch rounded up to 8 elements).
inline int make_shadow(const float *src, int rows, int cols, int ns, Shadow &s, int cls) {
    if (int e = alloc_shadow(s, rows, cols, ns)) return e;
    s.enc = enc_for(cls);
    if (s.enc.dscale)          // an fp32 gradient tensor handed in from outside: its own largest entry sets the dynamic factor
        if (int e = seera_grad_scale_update(src, (long long)rows * cols)) return e;
    long long groups = (long long)rows * (s.ld / 8);
    int grid = stride_grid(groups);
    cudaStream_t st = rt().stream;
    ProfBytes pb(4.0 * rows * cols + 2.0 * ns * rows * s.ld, "shadow_rows");
    if (ns == 1) shadow_rows_kernel<1><<<grid, 256, 0, st>>>(src, cols, rows, cols, s.p[0], s.p[1], s.p[2], s.ld, s.enc, fast_div(s.ld / 8));
    else if (ns == 2) shadow_rows_kernel<2><<<grid, 256, 0, st>>>(src, cols, rows, cols, s.p[0], s.p[1], s.p[2], s.ld, s.enc, fast_div(s.ld / 8));
    else shadow_rows_kernel<3><<<grid, 256, 0, st>>>(src, cols, rows, cols, s.p[0], s.p[1], s.p[2], s.ld, s.enc, fast_div(s.ld / 8));
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, "shadow_rows");
}

// ---- TMA + mbarrier PTX -------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}
// im2col-mode load from an NHWC tensor: {c, w, h, n} is the channel offset and the position of the filter
// window's corner for the FIRST pixel of the column; {off_w, off_h} selects the filter tap.  The copy walks
// pixelsPerColumn window positions (w fastest, then h, then n) and fetches channelsPerPixel channels of each.
__device__ __forceinline__ void tma_load_im2col(uint32_t dst_smem, const CUtensorMap *map, int c, int w, int h, int n,
                                                int off_w, int off_h, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6], {%7, %8};"
                 ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(c), "r"(w), "r"(h), "r"(n), "r"(bar),
                   "h"((unsigned short)off_w), "h"((unsigned short)off_h) : "memory");
}

// ---- CTA pairs (tcgen05 cta_group::2): two CTAs of a cluster share one 256-row accumulator tile -------------------------
// Each CTA stages its own 128 rows of A and its own half of B's columns; the MMA, issued by the even CTA alone, reads the
// shared memory of both, and each CTA's TMEM receives its 128 rows of the result.  Per CTA and k-step that is
// (128 + N/2) operand rows loaded for 128 x N of output instead of (128 + N): the L2 -> shared-memory stream, which bounds
// the split-product kernels, shrinks by a quarter to a third.  No multicast load is involved: every CTA issues plain
// tensor copies into its own shared memory; only their completion is counted on the even CTA's barrier, and the
// tcgen05.commit that frees a stage or publishes an accumulator arrives on both CTAs' barriers.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();        // the single-thread roles left their warps diverged
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
// shared::cluster address of the same variable in the CTA of rank `rank`
__device__ __forceinline__ uint32_t mapa_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair once the MMAs issued so far have finished
__device__ __forceinline__ void umma2_commit_both(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short)3) : "memory");
}
// tensor copies of a CTA of a pair: into its own shared memory, completion counted on `bar`, a shared::cluster address
__device__ __forceinline__ void tma2_load_2d(uint32_t dst_smem, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma2_load_im2col(uint32_t dst_smem, const CUtensorMap *map, int c, int w, int h, int n,
                                                 int off_w, int off_h, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.im2col.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6], {%7, %8};"
                 ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(c), "r"(w), "r"(h), "r"(n), "r"(bar),
                   "h"((unsigned short)off_w), "h"((unsigned short)off_h) : "memory");
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

// How the producer thread forms the A tile of a stage:
//   TMA_A_ROWS    2-D map of a row-major matrix [M, K], read along its rows (K-major)
//   TMA_A_COLS    2-D map of a row-major matrix [K, M], read along its columns (MN-major, two 64-wide boxes)
//   TMA_A_IM2COL  im2col map of an NHWC tensor; M = output pixels, K = (tap, channel): one tap x 64 channels
//                 per stage (K-major).  B is then [N, (tap, channel)] read along its rows.
//   TMA_A_TAPS    im2col map of an NHWC tensor; M = (tap, channel), K = output pixels: 64 pixels per stage,
//                 two boxes of 64 channels (MN-major).  B is then [pixels, N] read along its columns.
enum { TMA_A_ROWS = 0, TMA_A_COLS = 1, TMA_A_IM2COL = 2, TMA_A_TAPS = 3 };

struct TmaGemmParams {
    int M, N, K, kchunk, splits, bn, stages;
    int a_mode, b_mn;        // b_mn = 1: B read along its contiguous row index (MN-major)
    int pair;                // 1: launched as clusters of two CTAs sharing 256-row tiles (tcgen05 cta_group::2)
    int issuers;             // 1 or 2 threads issue the MMAs of a k-step (the K = 16 slices dealt round robin), each into its own
                             // accumulator; the epilogue adds the accumulators up
    // convolution geometry for the im2col modes
    int OW, OHW;             // output width and pixels per image of the traversal
    int sw, sh, pw, ph;      // window stride and lower padding
    int S, taps;             // filter width and R*S
    int cpad, cchunks;       // channel pitch of the weight rows / channels rounded up to 64, in chunks of 64
    float *partial;
    int *status;
    unsigned long long wait_clocks;   // budget of every bounded wait in the kernel
    int skip_load;           // test hook: the producer of CTA 0 leaves out the loads of this k-step (-1: none), so that the
                             // waits downstream of it run out and the kernel has to report and unwind
    const float *dinv;       // device word holding the inverse of the gradient operand's dynamic factor (null: none)
    float out_scale;         // the accumulator is multiplied by this before bias / activation / store: 1 / (scale_a * scale_b)
    int a_fp16, b_fp16;      // operand formats: 0 bf16, 1 fp16
    const float *bias;       // per-column bias added before the store, or null
    int act;                 // activation applied before the store (0 = none)
    int pool_on;             // 1: rows are pixels of a layer output that is only consumed through a 2x2 max-pool: store that instead
    PoolOut pool;
    FastDiv by_mtiles, by_ntiles, by_OHW, by_OW, by_S, by_cchunks;      // filled by launch_tma_gemm
};

// warp 0: TMA producer; warps 1-2: MMA issuers (the first p.issuers of them); warp 3 allocates TMEM; warps 4-7: epilogue.
// (Eight warps: with a ninth the register file would be shared out as for twelve, 168 registers per thread, and the epilogue spills.)
constexpr int TG_THREADS = 256, TG_EPI_WARP0 = 4;

// Persistent kernel: each CTA walks tiles  id = blockIdx.x, blockIdx.x + gridDim.x, ...  (m-tile fastest, then n-tile,
// then K split).  The operand ring keeps streaming across tile boundaries and the accumulator is double-buffered in
// TMEM, so the epilogue of tile i overlaps the main loop of tile i+1.
//
// One thread can issue a tcgen05.mma only every 80-90 clocks, whatever the instruction's size (measured: 88 clocks per MMA at
// N = 64 from one thread, the same MMAs from two threads at twice the rate), while a 128 x N x 16 instruction occupies the
// tensor pipe for N / 2 clocks.  With N <= 128 a single issuing thread therefore leaves the pipe idle half of the time or more.
// So two threads (lane 0 of warps 1 and 2) issue where the accumulators fit: they wait for the same stage, take the K = 16 slices
// of the k-step alternately, each into an accumulator of its own (MMAs of different threads are not ordered among themselves), and each commits
// to the stage's "empty" barrier and to the tile's "accumulator full" barrier, which count `issuers` arrivals.  TMEM holds
// 2 buffers x issuers x bn columns (at most 512); the epilogue adds the accumulators of a buffer while it drains them.
template <int NS, class CS, bool PAIR>
__global__ void __launch_bounds__(TG_THREADS, 1)
tma_gemm_kernel(const __grid_constant__ CUtensorMap mapA0, const __grid_constant__ CUtensorMap mapA1,
                const __grid_constant__ CUtensorMap mapA2, const __grid_constant__ CUtensorMap mapB0,
                const __grid_constant__ CUtensorMap mapB1, const __grid_constant__ CUtensorMap mapB2, CS cs, TmaGemmParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * 8 + 4];      // full[8], empty[8], tfull[2], tempty[2]
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int bn = p.bn, stages = p.stages;
    // PAIR: the two CTAs of a cluster work on one tile of 256 rows; `rank` 0 (the even CTA) issues its MMAs
    constexpr int TM = PAIR ? 2 * TC_BM : TC_BM;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, nworkers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int bh = PAIR ? bn >> 1 : bn;                       // columns of B this CTA stages
    const int mtiles = (p.M + TM - 1) / TM, ntiles = (p.N + bn - 1) / bn;
    const int total_tiles = mtiles * ntiles * p.splits;
    const bool a_mn = p.a_mode == TMA_A_COLS || p.a_mode == TMA_A_TAPS;

    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t a_bytes = TC_BM * 128, b_bytes = (uint32_t)bh * 128;
    const uint32_t stage_bytes = (uint32_t)NS * (a_bytes + b_bytes);
    const uint32_t smem0 = smem_u32(smem);
    auto a_tile = [&](int s, int i) { return smem0 + (uint32_t)s * stage_bytes + (uint32_t)i * a_bytes; };
    auto b_tile = [&](int s, int i) { return smem0 + (uint32_t)s * stage_bytes + (uint32_t)NS * a_bytes + (uint32_t)i * b_bytes; };
    unsigned char *epi_smem = smem + (size_t)stages * stage_bytes;   // 4 x EPI_WARP_SMEM after the ring
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[8]), tfull0 = smem_u32(&bars[16]), tempty0 = smem_u32(&bars[18]);
    const int issuers = PAIR ? 1 : p.issuers;
    const uint32_t tmem_cols = (uint32_t)(2 * issuers * bn < 32 ? 32 : 2 * issuers * bn);

    if (t == 0) {
        abort_flag = 0;
        for (int s = 0; s < stages; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, issuers); }
        for (int b = 0; b < 2; b++) { mbar_init(tfull0 + 8 * b, issuers); mbar_init(tempty0 + 8 * b, PAIR ? 8 : 4); }
        fence_mbar_init();
        fence_async_smem();
    }
    if (warp == 3) { if (PAIR) tmem_alloc2(smem_u32(&tmem_base_slot), tmem_cols); else tmem_alloc(smem_u32(&tmem_base_slot), tmem_cols); }
    tc_fence_before();
    if (PAIR) cluster_sync_all(); else __syncthreads();        // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int *abortp = &abort_flag;

    // tile id -> origin and K range
    auto tile_origin = [&](int id, int &m0, int &n0, int &kbeg, int &ktiles, int &z) {
        int rest = p.by_mtiles.div(id), mt = id - rest * mtiles;
        z = p.by_ntiles.div(rest);
        int nt = rest - z * ntiles;
        m0 = mt * TM + (int)rank * TC_BM; n0 = nt * bn;         // this CTA's own 128 rows
        kbeg = z * p.kchunk;
        int kend = min(p.K, kbeg + p.kchunk);
        ktiles = (kend - kbeg + TC_BK - 1) / TC_BK;
    };

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ----------------
        const CUtensorMap *mA[3] = {&mapA0, &mapA1, &mapA2};
        const CUtensorMap *mB[3] = {&mapB0, &mapB1, &mapB2};
        auto ld2d = [&](uint32_t dst, const CUtensorMap *m, int x, int y, uint32_t bar) {
            if (PAIR) tma2_load_2d(dst, m, x, y, bar); else tma_load_2d(dst, m, x, y, bar);
        };
        auto ldim = [&](uint32_t dst, const CUtensorMap *m, int c, int w, int h, int n, int ow, int oh, uint32_t bar) {
            if (PAIR) tma2_load_im2col(dst, m, c, w, h, n, ow, oh, bar); else tma_load_im2col(dst, m, c, w, h, n, ow, oh, bar);
        };
        int it = 0, issued_from = 0;
        int s = 0;                                            // ring slot and its phase, carried across tiles
        uint32_t ph = 0;
        bool alive = true;
        for (int id = worker; id < total_tiles && alive; id += nworkers) {
            int m0, n0, kbeg, ktiles, z;
            tile_origin(id, m0, n0, kbeg, ktiles, z);
            const int nb0 = n0 + (int)rank * bh;               // this CTA's own columns of B
            // im2col, M = pixels: window corner of this tile's first output pixel
            int pix_img = 0, pix_w = 0, pix_h = 0;
            if (p.a_mode == TMA_A_IM2COL) {
                pix_img = p.by_OHW.div(m0);
                int rem = m0 - pix_img * p.OHW, oh = p.by_OW.div(rem), ow = rem - oh * p.OW;
                pix_w = ow * p.sw - p.pw; pix_h = oh * p.sh - p.ph;
            }
            // im2col, M = (tap, channel): the two 64-channel boxes of this tile
            int box_c[2] = {0, 0}, box_s[2] = {0, 0}, box_r[2] = {0, 0};
            bool box_ok[2] = {true, true};
            uint32_t tx_bytes = PAIR ? 2u * stage_bytes : stage_bytes;     // a pair counts both CTAs' bytes on the even CTA's barrier
            if (p.a_mode == TMA_A_TAPS) {
                int c64 = p.cchunks * 64;
                for (int b = 0; b < 2; b++) {
                    int mb = m0 + 64 * b, tap = p.by_cchunks.div(mb >> 6);
                    box_ok[b] = tap < p.taps;
                    box_c[b] = mb - tap * c64; box_r[b] = p.by_S.div(tap); box_s[b] = tap - box_r[b] * p.S;
                    if (!box_ok[b]) tx_bytes -= (uint32_t)NS * 8192u;
                }
                if (PAIR && rank == 0) {                       // the peer's boxes beyond the last tap are not loaded either
                    for (int b = 0; b < 2; b++) {
                        int mb = m0 + TC_BM + 64 * b, tap = p.by_cchunks.div(mb >> 6);
                        if (tap >= p.taps) tx_bytes -= (uint32_t)NS * 8192u;
                    }
                }
            }
            for (int kt = 0; kt < ktiles; kt++, it++) {
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abortp, p.status, 1, p.wait_clocks)) { alive = false; break; }
                int k0 = kbeg + kt * TC_BK;
                const uint32_t bar = PAIR ? mapa_rank(full0 + 8 * s, 0) : full0 + 8 * s;
                if (p.skip_load >= 0 && blockIdx.x == 0 && it == p.skip_load) {      // test hook: this stage never fills
                    if (++s == stages) { s = 0; ph ^= 1u; }
                    continue;
                }
                if (rank == 0) mbar_expect_tx(full0 + 8 * s, tx_bytes);
                int bk = k0;                                  // B's coordinate along the contraction
                if (p.a_mode == TMA_A_ROWS) {
#pragma unroll
                    for (int i = 0; i < NS; i++) ld2d(a_tile(s, i), mA[i], k0, m0, bar);
                } else if (p.a_mode == TMA_A_COLS) {
#pragma unroll
                    for (int i = 0; i < NS; i++)
                        for (int b = 0; b < 2; b++) ld2d(a_tile(s, i) + b * 8192, mA[i], m0 + 64 * b, k0, bar);
                } else if (p.a_mode == TMA_A_IM2COL) {
                    int ktile = k0 >> 6, tap = p.by_cchunks.div(ktile), c0 = (ktile - tap * p.cchunks) * 64;
                    int r = p.by_S.div(tap), sx = tap - r * p.S;
#pragma unroll
                    for (int i = 0; i < NS; i++) ldim(a_tile(s, i), mA[i], c0, pix_w, pix_h, pix_img, sx, r, bar);
                    bk = tap * p.cpad + c0;
                } else {
                    int img = p.by_OHW.div(k0), rem = k0 - img * p.OHW, oh = p.by_OW.div(rem), ow = rem - oh * p.OW;
                    int w = ow * p.sw - p.pw, h = oh * p.sh - p.ph;
#pragma unroll
                    for (int i = 0; i < NS; i++)
                        for (int b = 0; b < 2; b++)
                            if (box_ok[b]) ldim(a_tile(s, i) + b * 8192, mA[i], box_c[b], w, h, img, box_s[b], box_r[b], bar);
                }
                if (p.b_mn) {
#pragma unroll
                    for (int i = 0; i < NS; i++)
                        for (int b = 0; b < bh / 64; b++) ld2d(b_tile(s, i) + b * 8192, mB[i], nb0 + 64 * b, bk, bar);
                } else {
#pragma unroll
                    for (int i = 0; i < NS; i++) ld2d(b_tile(s, i), mB[i], bk, nb0, bar);
                }
                if (++s == stages) { s = 0; ph ^= 1u; }
            }
        }
        if (*abortp && rank == 0) {
            // give copies already in flight a bounded chance to land before the CTA's shared memory goes away
            issued_from = it - stages < 0 ? 0 : it - stages;
            for (int k = issued_from; k < it; k++) {
                unsigned long long t0 = clock64();
                if (p.skip_load >= 0 && blockIdx.x == 0 && k == p.skip_load) continue;      // nothing was issued for it
                while (!mbar_try_wait(full0 + 8 * (k % stages), (uint32_t)(k / stages) & 1u) && clock64() - t0 < p.wait_clocks) {}
            }
        }
    } else if (warp >= 1 && warp <= issuers && lane == 0 && rank == 0) {
        // ---------------- MMA issuers (in the even CTA of a pair) ----------------
        const int me = warp - 1;
        uint32_t idesc = umma_idesc_16bit(bn, p.a_fp16, p.b_fp16) | ((uint32_t)(a_mn ? 1 : 0) << 15) | ((uint32_t)p.b_mn << 16);
        if (PAIR) idesc = (idesc & ~(31u << 24)) | ((uint32_t)(TM >> 4) << 24);          // M = 256 over the two CTAs
        const uint32_t a_step = a_mn ? 2048u : 32u, b_step = p.b_mn ? 2048u : 32u;   // bytes per K=16 slice
        // split products kept: hi*hi | + hi*lo, lo*hi | + hi*lo2, lo2*hi, lo*lo
        constexpr int NPROD = NS == 1 ? 1 : (NS == 2 ? 3 : 6);
        const int pa[6] = {0, 0, 1, 0, 2, 1}, pb[6] = {0, 1, 0, 2, 0, 1};
        bool alive = true;
        int local = 0;
        int s = 0;                                            // ring slot and its phase, carried across tiles
        uint32_t ph = 0;
        // descriptors of copy 0 / slice 0 in slot 0; the others differ only in the start-address field (16-byte units),
        // which never carries out of its 14 bits for addresses inside the CTA's shared memory
        const uint32_t a_step16 = a_step >> 4, b_step16 = b_step >> 4, a_copy16 = a_bytes >> 4, b_copy16 = b_bytes >> 4;
        const uint64_t da0 = (a_mn ? umma_desc_sw128_mn(a_tile(0, 0), 8192) : umma_desc_sw128(a_tile(0, 0))) + (uint32_t)me * a_step16;
        const uint64_t db0 = (p.b_mn ? umma_desc_sw128_mn(b_tile(0, 0), 8192) : umma_desc_sw128(b_tile(0, 0))) + (uint32_t)me * b_step16;
        const uint32_t stage16 = stage_bytes >> 4;
        for (int id = worker; id < total_tiles && alive; id += nworkers, local++) {
            int m0, n0, kbeg, ktiles, z;
            tile_origin(id, m0, n0, kbeg, ktiles, z);
            const int buf = local & 1;
            // the epilogue must have drained this accumulator buffer (two tiles ago)
            alive = mbar_wait(tempty0 + 8 * buf, (((uint32_t)local >> 1) & 1u) ^ 1u, abortp, p.status, 4, p.wait_clocks);
            if (!alive) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)((buf * issuers + me) * bn);
            uint32_t acc = 0;
            for (int kt = 0; kt < ktiles && alive; kt++) {
                alive = mbar_wait(full0 + 8 * s, ph, abortp, p.status, 2, p.wait_clocks);
                if (!alive) break;
                tc_fence_after();
                const uint64_t das = da0 + (uint32_t)s * stage16, dbs = db0 + (uint32_t)s * stage16;
                // the K = 16 slices of this thread (da0 / db0 already point at its first one), fully unrolled either way: the
                // issuing thread's own instruction stream is what limits the MMA rate
                auto slice = [&](uint64_t dsa, uint64_t dsb) {
                    uint64_t da[NS], db[NS];
#pragma unroll
                    for (int i = 0; i < NS; i++) { da[i] = dsa + (uint32_t)i * a_copy16; db[i] = dsb + (uint32_t)i * b_copy16; }
#pragma unroll
                    for (int q = 0; q < NPROD; q++) {
                        if (PAIR) umma2_bf16(d_tmem, da[pa[q]], db[pb[q]], idesc, acc); else umma_bf16(d_tmem, da[pa[q]], db[pb[q]], idesc, acc);
                        acc = 1;
                    }
                };
                if (issuers == 2) {
#pragma unroll
                    for (int jj = 0; jj < TC_BK / 32; jj++) slice(das + (uint32_t)(2 * jj) * a_step16, dbs + (uint32_t)(2 * jj) * b_step16);
                } else {
#pragma unroll
                    for (int jj = 0; jj < TC_BK / 16; jj++) slice(das + (uint32_t)jj * a_step16, dbs + (uint32_t)jj * b_step16);
                }
                if (PAIR) umma2_commit_both(empty0 + 8 * s); else umma_commit(empty0 + 8 * s);
                if (++s == stages) { s = 0; ph ^= 1u; }
            }
            if (alive) { if (PAIR) umma2_commit_both(tfull0 + 8 * buf); else umma_commit(tfull0 + 8 * buf); }   // accumulator complete
        }
    } else if (warp >= TG_EPI_WARP0) {
        // ---------------- epilogue: warp w drains TMEM lane quarter w % 4 ----------------
        const int q = warp & 3;
        float *stage = reinterpret_cast<float *>(epi_smem + (size_t)(warp - TG_EPI_WARP0) * EPI_WARP_SMEM);
        const float out_scale = p.dinv ? p.out_scale * __ldg(p.dinv) : p.out_scale;
        int local = 0;
        const uint32_t tempty_at = PAIR ? mapa_rank(tempty0, 0) : tempty0;      // the even CTA's barrier counts both epilogues
        for (int id = worker; id < total_tiles; id += nworkers, local++) {
            int m0, n0, kbeg, ktiles, z;
            tile_origin(id, m0, n0, kbeg, ktiles, z);
            const int buf = local & 1;
            if (!mbar_wait(tfull0 + 8 * buf, ((uint32_t)local >> 1) & 1u, abortp, p.status, 3, p.wait_clocks)) break;
            tc_fence_after();
            if (p.pool_on)
                drain_accumulator_pooled(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * issuers * bn), m0 + q * 32, n0, bn, p.M, p.N,
                                         p.bias, p.act, p.pool, stage, out_scale, issuers, (uint32_t)bn);
            else
                drain_accumulator(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * issuers * bn), m0 + q * 32, n0, 0, bn, p.M, p.N, cs,
                                  p.partial, (long long)z * p.M * p.N, stage, p.bias, p.act, out_scale, issuers, (uint32_t)bn);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { if (PAIR) mbar_arrive_cluster(tempty_at + 8 * buf); else mbar_arrive(tempty0 + 8 * buf); }
        }
    }
    tc_fence_before();
    if (PAIR) cluster_sync_all(); else __syncthreads();        // neither CTA's shared memory or TMEM goes away while the other still uses it
    if (warp == 3) { if (PAIR) tmem_dealloc2(tmem_base, tmem_cols); else tmem_dealloc(tmem_base, tmem_cols); }
}

template <class CS>
__global__ void __launch_bounds__(256) tma_splitk_reduce_kernel(const float *__restrict__ partial, CS cs, int M, int N, int splits,
                                                                const float *__restrict__ bias, int act, float scale,
                                                                const float *__restrict__ dinv) {
    if (dinv) scale *= __ldg(dinv);
    long long total = (long long)M * N;
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    const bool small = total < (1ll << 31);       // 32-bit index arithmetic then: the 64-bit division costs more than the loads
    for (long long i = tid; i < total; i += nthr) {
        float s = 0.f;
#pragma unroll 4
        for (int z = 0; z < splits; z++) s += __ldg(partial + (long long)z * total + i);
        s *= scale;
        const int m = small ? (int)((unsigned)i / (unsigned)N) : (int)(i / N);
        const int n = (int)(i - (long long)m * N);
        if (bias) s += __ldg(bias + n);
        cs(m, n, epilogue_act(s, act));
    }
}

int *tc_status_word();

struct TmaMaps { CUtensorMap a[3], b[3]; };

inline int tma_pick_bn(int N, int ns, int b_mn) {
    int bn = N <= 32 ? 32 : (N <= 64 ? 64 : (N <= 128 ? 128 : 256));
    if (b_mn && bn < 64) bn = 64;
    if (ns == 2 && bn > rt().tile_n_cap2) bn = rt().tile_n_cap2;
    if (ns >= 3 && bn > rt().tile_n_cap3) bn = rt().tile_n_cap3;
    // at least two stages of ns * (128 + bn) * 128 bytes must fit beside the epilogue staging
    while (bn > 32 && 2 * (size_t)ns * (TC_BM + bn) * 128 > 225 * 1024 - 4 * EPI_WARP_SMEM - 1024) bn >>= 1;
    return bn;
}

// Chooses the accumulator width and whether the launch runs as CTA pairs; sets p.bn and p.pair from p.M, p.N, p.b_mn.
// Pairs pay when the operand stream bounds the kernel (the split modes: per CTA and k-step 128 + N/2 operand rows instead of
// 128 + N) and there are enough 256-row tiles to keep 74 pairs busy; a launch that may split its contraction always has.
inline void tma_plan(TmaGemmParams &p, int ns, bool allow_split) {
    p.bn = tma_pick_bn(p.N, ns, p.b_mn);
    p.pair = 0;
    // MMA-issuing threads: two where TMEM has room for their accumulators (2 buffers x issuers x bn <= 512 columns); one thread
    // keeps up with 256-column instructions by itself
    p.issuers = p.bn <= 128 ? 2 : 1;
    if (rt().mma_issuers && rt().mma_issuers < p.issuers) p.issuers = rt().mma_issuers;
    if (!rt().pair_tiles || ns > 2 || rt().sm_count < 4) return;
    int bn = p.bn;
    if (ns == 2 && p.N > 128) bn = 256;               // a pair stages half of B per CTA: 2 x (16 + 16) KB per stage, three stages
    if (bn < 64 || (p.b_mn && bn < 128) || p.M < 2 * TC_BM) return;
    const long long pair_tiles = (long long)((p.M + 2 * TC_BM - 1) / (2 * TC_BM)) * ((p.N + bn - 1) / bn);
    if (!allow_split && pair_tiles < rt().sm_count / 2) return;
    p.bn = bn;
    p.pair = 1;
}

// Launches the kernel on prepared tensor maps.  p.M, p.N, p.K (contraction length in elements), a_mode, b_mn, bn
// and the geometry fields must be set; kchunk, stages, partial and status are filled here.
template <class CS>
int launch_tma_gemm(const TmaMaps &maps, TmaGemmParams p, const CS &cs, int ns, bool allow_split, double flops, const char *name) {
    if (p.issuers != 2 || p.pair || 4 * p.bn > 512) p.issuers = 1;      // TMEM has 512 columns
    const int tm = p.pair ? 2 * TC_BM : TC_BM;
    size_t stage = (size_t)ns * (TC_BM * 128 + (size_t)(p.pair ? p.bn / 2 : p.bn) * 128);
    // 227 KB per CTA on sm_100a; keep 2 KB for the kernel's static shared memory and alignment slack
    int stages = (int)((225 * 1024 - 4 * EPI_WARP_SMEM - 1024) / stage);
    if (stages > 8) stages = 8;
    if (stages < 2) return fail(SEERA_E_LIMIT, "%s: tile does not fit shared memory", name);
    size_t smem = stage * stages + 4 * EPI_WARP_SMEM + 1024;
    long long tiles = (long long)((p.M + tm - 1) / tm) * ((p.N + p.bn - 1) / p.bn);
    // Split of the contraction: every (tile, split) item is one pass of a persistent CTA, so the launch takes
    // ceil(items / SMs) rounds of ceil(ksteps / splits) k-steps each, plus a fixed cost per item (pipeline fill, the
    // partial tile written out, worth about four k-steps).  A split also pays for the reduce launch (eight k-steps) and
    // for moving the partial sums: splits x M x N floats written and read back, M x N written, priced at 5 TB/s against
    // a k-step of about 0.25 us per product at N = 128 (small outputs stay in L2 and cost nothing; a 4096 x 4096 output
    // split in two would cost more than the idle SMs it fills).  Take the split count with the smallest such estimate;
    // ties go to fewer splits.
    int splits = 1;
    const long long ksteps = (p.K + TC_BK - 1) / TC_BK;
    if (allow_split) {
        const long long sms = p.pair ? rt().sm_count / 2 : rt().sm_count;      // workers: CTAs, or pairs of them
        const double kstep_us = 0.25 * (ns == 1 ? 1 : (ns == 2 ? 3 : 6)) * p.bn / 128.0;
        const double partial_ksteps = (double)p.M * p.N * 4.0 / 5e6 / kstep_us;      // one pass over M x N floats, in k-steps
        long long maxs = ksteps / 2;                  // at least two k-steps per item
        if (maxs > 256) maxs = 256;
        long long best = -1;
        for (long long sp = 1; sp <= maxs || sp == 1; sp++) {
            long long per = (ksteps + sp - 1) / sp, eff = (ksteps + per - 1) / per;
            long long rounds = (tiles * eff + sms - 1) / sms;
            long long cost = rounds * (per + 4);
            if (sp > 1) cost += 8 + (long long)((2.0 * eff + 1.0) * partial_ksteps);
            if (best < 0 || cost < best) { best = cost; splits = (int)eff; }
        }
    }
    p.kchunk = (int)((ksteps + splits - 1) / splits) * TC_BK;
    splits = (p.K + p.kchunk - 1) / p.kchunk;
    p.splits = splits;
    p.stages = stages;
    p.by_mtiles = fast_div((p.M + tm - 1) / tm); p.by_ntiles = fast_div((p.N + p.bn - 1) / p.bn);
    p.by_OHW = fast_div(p.OHW); p.by_OW = fast_div(p.OW); p.by_S = fast_div(p.S); p.by_cchunks = fast_div(p.cchunks);
    p.status = tc_status_word();
    p.wait_clocks = rt().tc_wait_clocks;
    p.skip_load = rt().tc_test_skip_load;
    rt().tc_test_skip_load = -1;                 // one launch only
    p.partial = nullptr;
    if (splits > 1) {
        p.partial = (float *)scratch_alloc((size_t)splits * p.M * p.N * sizeof(float));
        if (!p.partial) return SEERA_E_OOM;
    }
    long long all_tiles = tiles * splits;
    const long long workers = p.pair ? rt().sm_count / 2 : rt().sm_count;
    dim3 grid((unsigned)((all_tiles < workers ? all_tiles : workers) * (p.pair ? 2 : 1)));     // persistent: one CTA per SM at most
    cudaStream_t st = rt().stream;
    cudaError_t e;
    profile_begin();
#define SEERA_TMA_LAUNCH(NSV, PAIRV)                                                                                       \
    {                                                                                                                      \
        auto kern = tma_gemm_kernel<NSV, CS, PAIRV>;                                                                       \
        static int smem_set[64];                     /* per instantiation and device: raise the limit once */              \
        const int dev = rt().device & 63;                                                                                  \
        e = cudaSuccess;                                                                                                   \
        if (!smem_set[dev]) {                                                                                              \
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);                       \
            if (e == cudaSuccess) smem_set[dev] = 1;                                                                       \
        }                                                                                                                  \
        if (e == cudaSuccess) {                                                                                            \
            cudaLaunchConfig_t cfg = {};                                                                                   \
            cfg.gridDim = grid; cfg.blockDim = dim3(TG_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;             \
            cudaLaunchAttribute attr[1];                                                                                   \
            attr[0].id = cudaLaunchAttributeClusterDimension;                                                              \
            attr[0].val.clusterDim.x = PAIRV ? 2 : 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;          \
            cfg.attrs = attr; cfg.numAttrs = PAIRV ? 1 : 0;                                                                \
            e = cudaLaunchKernelEx(&cfg, kern, maps.a[0], maps.a[1], maps.a[2], maps.b[0], maps.b[1], maps.b[2], cs, p);   \
            if (e == cudaSuccess) e = cudaGetLastError();                                                                  \
        }                                                                                                                  \
    }
    if (p.pair) { if (ns == 1) SEERA_TMA_LAUNCH(1, true) else SEERA_TMA_LAUNCH(2, true) }
    else if (ns == 1) SEERA_TMA_LAUNCH(1, false) else if (ns == 2) SEERA_TMA_LAUNCH(2, false) else SEERA_TMA_LAUNCH(3, false)
#undef SEERA_TMA_LAUNCH
    count_launch();
    if (e == cudaSuccess && p.partial) {
        tma_splitk_reduce_kernel<<<stride_grid((long long)p.M * p.N), 256, 0, st>>>(p.partial, cs, p.M, p.N, splits, p.bias, p.act, p.out_scale, p.dinv);
        count_launch();
        e = cudaGetLastError();
    }
    if (p.partial) scratch_free(p.partial);
    profile_end(flops, name);
    rt().tc_used = true;
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, name);
}

// Dense: A operand shadow `sa`; a_mn = 0: sa is [M, K] (read along its rows); a_mn = 1: sa is [K, M].  Likewise B with N.
template <class CS>
int run_tma_gemm(const Shadow &sa, int a_mn, const Shadow &sb, int b_mn, const CS &cs, int M, int N, int K,
                 bool allow_split, const char *name, const float *bias = nullptr, int act = 0, int copies = 0) {
    const int ns = copies ? copies : precision_copies();
    TmaGemmParams p{};
    p.bias = bias; p.act = act;
    p.M = M; p.N = N; p.K = K; p.a_mode = a_mn ? TMA_A_COLS : TMA_A_ROWS; p.b_mn = b_mn;
    p.a_fp16 = sa.enc.fmt; p.b_fp16 = sb.enc.fmt; p.out_scale = 1.f / (sa.enc.scale * sb.enc.scale);
    p.dinv = enc_dinv(sa.enc, sb.enc);
    tma_plan(p, ns, allow_split);
    TmaMaps maps;
    for (int i = 0; i < 3; i++) {
        int j = i < ns ? i : 0;
        // K-major: inner dimension = K (cols of the shadow), box 64 x rows-of-tile; MN-major: inner = M/N, box 64 x 64 k lines
        if (int s = make_map_2d(&maps.a[i], sa.p[j], sa.rows, sa.cols, sa.ld, 64, a_mn ? 64 : TC_BM)) return s;
        if (int s = make_map_2d(&maps.b[i], sb.p[j], sb.rows, sb.cols, sb.ld, 64, b_mn ? 64 : (p.pair ? p.bn / 2 : p.bn))) return s;
    }
    return launch_tma_gemm(maps, p, cs, ns, allow_split, 2.0 * M * N * (double)K, name);
}

}  // namespace seera
