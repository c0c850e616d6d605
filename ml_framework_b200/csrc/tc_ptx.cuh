// Inline-PTX wrappers for the sm_100a tensor-core path: mbarrier, proxy fences, TMEM allocation,
// tcgen05.mma / commit / ld, shared-memory matrix descriptors and the instruction descriptor.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace seera {

constexpr int TC_BM = 128, TC_BK = 64, TC_PRODUCERS = 256, TC_THREADS = 288;
constexpr unsigned long long TC_WAIT_CLOCKS = 4000000000ull;      // ~2 s at 2 GHz

// Division by a launch constant as one wide multiply and a shift: the producer and the MMA issuer are single threads
// with nothing to hide an integer division's ~100 dependent clocks behind, and they divide several times per k-step.
// Exact for 0 <= n < 2^31 (shift = 31 + ceil(log2 d), mul = ceil(2^shift / d) < 2^32).
struct FastDiv {
    uint32_t mul, shift;
    int d;
    __device__ __forceinline__ int div(int n) const { return (int)(((unsigned long long)(uint32_t)n * mul) >> shift); }
};
inline FastDiv fast_div(int d) {
    if (d < 1) d = 1;
    uint32_t l = 0;
    while ((1ll << l) < d) l++;
    FastDiv f;
    f.shift = 31 + l;
    f.mul = (uint32_t)(((1ull << f.shift) + (unsigned long long)d - 1) / (unsigned long long)d);
    f.d = d;
    return f;
}

// ---- PTX wrappers ----------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false when the budget (in clocks) ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status, int code,
                                          unsigned long long budget = TC_WAIT_CLOCKS) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (*abort_flag) return false;
        if (clock64() - t0 > budget) {
            *abort_flag = 1;
            if (status) atomicCAS(status, 0, code);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 inputs, fp32 accumulate, one CTA.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// mbarrier arrives once every MMA issued so far by this thread has finished reading smem / writing TMEM
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float *v) {
    uint32_t *r = reinterpret_cast<uint32_t *>(v);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                   "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                   "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// The same over `nacc` accumulators that sit `acc_stride` columns apart and hold partial sums of one tile (one per MMA-issuing
// thread): their sum, added in index order.
__device__ __forceinline__ void tmem_ld32_sum(uint32_t taddr, float *v, int nacc, uint32_t acc_stride) {
    tmem_ld32(taddr, v);
    for (int i = 1; i < nacc; i++) {
        float w[32];
        tmem_ld32(taddr + (uint32_t)i * acc_stride, w);
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] += w[j];
    }
}

// Shared-memory matrix descriptor: K-major tile whose rows are 128 bytes (64 bf16) with the 128-byte
// swizzle; 8-row groups are 1024 bytes apart.  `addr` must be 1024-byte aligned plus a multiple of 32
// bytes selecting the K=16 slice inside the row.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);          // start address, 16-byte units
    d |= (uint64_t)1 << 16;                           // leading byte offset (unused for this layout)
    d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                           // descriptor version for sm_100
    d |= (uint64_t)2 << 61;                           // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D fp32, A and B bf16, both K-major, M = 128, N = bn.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}
// The same with the operand formats chosen: field value 1 = bf16, 0 = fp16 (bits 7-9 for A, 10-12 for B).
__device__ __forceinline__ uint32_t umma_idesc_16bit(int bn, int a_fp16, int b_fp16) {
    return (1u << 4) | ((a_fp16 ? 0u : 1u) << 7) | ((b_fp16 ? 0u : 1u) << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t packed, int odd) {
    return __uint_as_float(odd ? (packed & 0xFFFF0000u) : (packed << 16));
}
// How a tensor's 16-bit operand copies are encoded.  fmt 0: bf16 (fp32's exponent range, 8-bit mantissa).  fmt 1: fp16
// (11-bit mantissa, so a two-copy split carries 22 bits and three products give an fp32-class result where bf16 needs six)
// with the values multiplied by `scale`, a power of two chosen per class of tensor so that the SECOND copy - 2^-11 of the
// first - stays in fp16's normal range for the values that matter; conversion saturates instead of producing infinities.
// The product's epilogue multiplies by 1 / (scale_a * scale_b), which is exact.
// Gradients have no fixed magnitude (they shrink by orders of magnitude as training converges), so their factor has a
// second, dynamic part: `dscale` points at a power of two in device memory that the loss head refreshes every step from
// the largest entry of the loss gradient (seera_grad_scale_update); null means 1.
struct Enc {
    int fmt;
    float scale;
    const float *dscale;
};
__device__ __forceinline__ float enc_factor(const Enc &e) { return e.dscale ? e.scale * __ldg(e.dscale) : e.scale; }

__device__ __forceinline__ uint32_t pack_f16x2_sat(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float f16_bits_to_float(uint32_t packed, int odd) {
    return __half2float(__ushort_as_half((unsigned short)(odd ? (packed >> 16) : (packed & 0xFFFFu))));
}
// Rounds 8 values to bf16 and returns them as one 16-byte chunk; `v` is replaced by the residuals, so calling it again
// yields the next copy of a split (hi, then mid, then lo).
__device__ __forceinline__ uint4 split_chunk(float *v) {
    uint4 h;
    h.x = pack_bf16x2(v[0], v[1]); h.y = pack_bf16x2(v[2], v[3]); h.z = pack_bf16x2(v[4], v[5]); h.w = pack_bf16x2(v[6], v[7]);
    const uint32_t w[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] -= bf16_bits_to_float(w[i >> 1], i & 1);
    return h;
}
__device__ __forceinline__ uint4 split_chunk_f16(float *v) {
    uint4 h;
    h.x = pack_f16x2_sat(v[0], v[1]); h.y = pack_f16x2_sat(v[2], v[3]); h.z = pack_f16x2_sat(v[4], v[5]); h.w = pack_f16x2_sat(v[6], v[7]);
    const uint32_t w[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] -= f16_bits_to_float(w[i >> 1], i & 1);
    return h;
}
// Writes the NS copies of 8 consecutive values (16-byte chunks at d0, d1, d2) in the encoding `e`; v is consumed.
template <int NS>
__device__ __forceinline__ void store_split8(float *v, const Enc &e, void *d0, void *d1, void *d2) {
    if (e.fmt) {
        const float f = enc_factor(e);
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] *= f;
        *reinterpret_cast<uint4 *>(d0) = split_chunk_f16(v);
        if (NS >= 2) *reinterpret_cast<uint4 *>(d1) = split_chunk_f16(v);
        if (NS >= 3) *reinterpret_cast<uint4 *>(d2) = split_chunk_f16(v);
    } else {
        *reinterpret_cast<uint4 *>(d0) = split_chunk(v);
        if (NS >= 2) *reinterpret_cast<uint4 *>(d1) = split_chunk(v);
        if (NS >= 3) *reinterpret_cast<uint4 *>(d2) = split_chunk(v);
    }
}
// The same for one value (ns known at run time).
__device__ __forceinline__ void store_split1(float v, int ns, const Enc &e, __nv_bfloat16 *d0, __nv_bfloat16 *d1, __nv_bfloat16 *d2) {
    unsigned short *u0 = reinterpret_cast<unsigned short *>(d0), *u1 = reinterpret_cast<unsigned short *>(d1),
                   *u2 = reinterpret_cast<unsigned short *>(d2);
    if (e.fmt) {
        v *= enc_factor(e);
        uint32_t p = pack_f16x2_sat(v, 0.f);
        *u0 = (unsigned short)p;
        if (ns >= 2) {
            v -= f16_bits_to_float(p, 0); p = pack_f16x2_sat(v, 0.f); *u1 = (unsigned short)p;
            if (ns >= 3) { v -= f16_bits_to_float(p, 0); *u2 = (unsigned short)pack_f16x2_sat(v, 0.f); }
        }
    } else {
        __nv_bfloat16 h = __float2bfloat16_rn(v);
        *d0 = h;
        if (ns >= 2) {
            v -= __bfloat162float(h); h = __float2bfloat16_rn(v); *d1 = h;
            if (ns >= 3) { v -= __bfloat162float(h); *d2 = __float2bfloat16_rn(v); }
        }
    }
}

}  // namespace seera
