// Accumulator drain shared by the tensor-core kernels: one warp moves its 32 TMEM lanes (rows) x `ncols`
// columns to global memory through the output functor.
#pragma once
#include "tc_ptx.cuh"

namespace seera {

constexpr int EPI_WARP_SMEM = 32 * 33 * 4;      // bytes of staging per epilogue warp (N-contiguous outputs)

// taddr: TMEM address of (first lane of this warp's quarter, column c_begin); row_base: global row of lane 0.
// Outputs contiguous along m (NCHW pixels, transposed dense) are stored straight from registers: lanes hold
// consecutive rows, so each store instruction is one coalesced line.  Outputs contiguous along n (row-major
// C, split-K partials) go through a 32x33 shared-memory transpose so that lanes hold consecutive columns.
// Per-column bias and activation applied on the way out (bias == nullptr and act == 0: plain store).  Split-K partial
// sums are stored untouched; their reduction applies the same transform.
__device__ __forceinline__ float epilogue_act(float z, int act) {
    switch (act) {
        case 1: return z > 0.f ? z : 0.f;               // SEERA_ACT_RELU
        case 2: return 1.f / (1.f + expf(-z));          // SEERA_ACT_SIGMOID
        case 3: return tanhf(z);                        // SEERA_ACT_TANH
        default: return z;
    }
}

// Output functors that also keep 16-bit copies of what they store expose copy_out(m, n, value); the others do not.
template <class CS>
__device__ __forceinline__ auto maybe_copy_out(const CS &cs, int m, int n, float v, int) -> decltype(cs.copy_out(m, n, v), void()) {
    cs.copy_out(m, n, v);
}
template <class CS>
__device__ __forceinline__ void maybe_copy_out(const CS &, int, int, float, long) {}

template <class CS>
__device__ __forceinline__ void drain_accumulator(uint32_t taddr, int row_base, int col_base, int c_begin, int c_end,
                                                  int M, int N, const CS &cs, float *partial, long long partial_off,
                                                  float *stage /* EPI_WARP_SMEM bytes, this warp's own */,
                                                  const float *bias = nullptr, int act = 0, float scale = 1.f,
                                                  int nacc = 1, uint32_t acc_stride = 0 /* partial accumulators to add up */) {
    const int lane = threadIdx.x & 31;
    const bool transpose = partial != nullptr || !CS::kMContiguous;
    const long long sn = cs.nstride();
    // direct path: this lane owns row m; its address part is computed once, not per element
    const int m_own = row_base + lane;
    float *own = (!transpose && m_own < M) ? cs.row(m_own) : nullptr;
    for (int c = c_begin; c < c_end; c += 32) {
        float v[32];
        tmem_ld32_sum(taddr + (uint32_t)(c - c_begin), v, nacc, acc_stride);
        if (scale != 1.f && !partial) {            // operand copies carried power-of-two factors: take them out (exact)
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] *= scale;
        }
        const bool fuse = !partial && (bias || act);
        if (!transpose) {
            if (fuse) {            // lanes hold rows here: the 32 column biases go through this warp's staging buffer
                const int n = col_base + c + lane;
                __syncwarp();
                stage[lane] = (bias && n < N) ? __ldg(bias + n) : 0.f;
                __syncwarp();
                if (act == 1) {    // relu: the common case without a switch per value
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 b4 = *reinterpret_cast<const float4 *>(stage + j);
                        float z;
                        z = v[j] + b4.x; v[j] = z > 0.f ? z : 0.f;
                        z = v[j + 1] + b4.y; v[j + 1] = z > 0.f ? z : 0.f;
                        z = v[j + 2] + b4.z; v[j + 2] = z > 0.f ? z : 0.f;
                        z = v[j + 3] + b4.w; v[j + 3] = z > 0.f ? z : 0.f;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 b4 = *reinterpret_cast<const float4 *>(stage + j);
                        v[j] = epilogue_act(v[j] + b4.x, act); v[j + 1] = epilogue_act(v[j + 1] + b4.y, act);
                        v[j + 2] = epilogue_act(v[j + 2] + b4.z, act); v[j + 3] = epilogue_act(v[j + 3] + b4.w, act);
                    }
                }
            }
            if (own) {
                float *q = own + (long long)(col_base + c) * sn;       // one pointer, advanced by the column stride
                const int nvalid = N - (col_base + c);
                if (nvalid >= 32) {
#pragma unroll
                    for (int j = 0; j < 32; j++) { *q = v[j]; q += sn; }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        if (j < nvalid) *q = v[j];
                        q += sn;
                    }
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++) stage[lane * 33 + j] = v[j];
            __syncwarp();
            const int n = col_base + c + lane;
            if (n < N) {
                if (partial) {
                    float *q = partial + partial_off + (long long)row_base * N + n;
                    const int rows = min(32, M - row_base);
                    for (int r = 0; r < rows; r++) q[(long long)r * N] = stage[r * 33 + lane];
                } else {
                    const float b = (fuse && bias) ? __ldg(bias + n) : 0.f;      // lanes hold columns here
#pragma unroll 4
                    for (int r = 0; r < 32; r++) {
                        if (row_base + r < M) {
                            float *rp = cs.row(row_base + r);
                            const float val = fuse ? epilogue_act(stage[r * 33 + lane] + b, act) : stage[r * 33 + lane];
                            if (rp) { rp[n * sn] = val; maybe_copy_out(cs, row_base + r, n, val, 0); }
                        }
                    }
                }
            }
            __syncwarp();
        }
    }
}

// ---- epilogue with a 2x2 / stride-2 max-pool folded in --------------------------------------------------------------
// The accumulator rows are output pixels of y = act(conv + bias); instead of storing y, each warp reduces the 2x2
// windows that lie inside its 32 rows with shuffles and stores only the pooled value, the window-local argmax (scan
// order (0,0), (0,1), (1,0), (1,1), strict comparison: the first maximum wins, as in cuda_maxpool_fwd) and the bf16
// channels-last copies of the pooled tensor for the next convolution.  y itself never reaches HBM.
// Row order: raster (row = pixel index; needs OW a power of two <= 16 so that a window's rows are lanes l, l^1, l^OW,
// l^(OW+1)) or window-major (row = 4 * window + position; partners are lanes l^1, l^2, l^3).
struct PoolOut {
    float *pooled;                 // [NB, F, OH/2, OW/2]
    int *mask;                     // same shape
    __nv_bfloat16 *copy[3];        // [NB, (OH/2)*(OW/2), Cp] or null
    int ns, Cp;
    Enc enc;                       // encoding of the copies
    int P, OW;                     // pixels per image and width of y
    int window_major;
    FastDiv by_P, by_OW, by_Pq;    // set by pool_out_geometry
};
inline void pool_out_geometry(PoolOut &po, int P, int OW, int window_major) {
    po.P = P; po.OW = OW; po.window_major = window_major;
    po.by_P = fast_div(P); po.by_OW = fast_div(OW); po.by_Pq = fast_div(P >> 2);
}

__device__ __forceinline__ void drain_accumulator_pooled(uint32_t taddr, int row_base, int col_base, int ncols, int M, int N,
                                                         const float *bias, int act, const PoolOut &po, float *stage, float scale = 1.f,
                                                         int nacc = 1, uint32_t acc_stride = 0) {
    // The warp's 32 rows hold exactly 8 windows.  Each 32-column chunk gets bias + activation while lanes still hold rows,
    // then goes through the warp's 32 x 33 staging buffer so that lanes hold COLUMNS (filters): a lane reads the four
    // values of a window from shared memory (no shuffles), and the 8 windows of its filter are 8 consecutive floats of the
    // pooled plane.
    const int lane = threadIdx.x & 31;
    const int Pq = po.P >> 2, OWq = po.OW >> 1;
    const int d2 = po.window_major ? 2 : po.OW;
    // first row of window w inside the warp's rows, its image and its index inside the image (the same for every lane)
    int r0[8], wimg[8], wrem[8];
#pragma unroll
    for (int w = 0; w < 8; w++) {
        if (po.window_major) {
            r0[w] = 4 * w;
            const int wi = (row_base >> 2) + w;
            wimg[w] = po.by_Pq.div(wi); wrem[w] = wi - wimg[w] * Pq;
        } else {
            const int wr = w / OWq, wc = w - wr * OWq;            // window row / column inside the warp's rows
            r0[w] = 2 * wr * po.OW + 2 * wc;
            const int m = row_base + r0[w], img = po.by_P.div(m), rem = m - img * po.P, oh = po.by_OW.div(rem), ow = rem - oh * po.OW;
            wimg[w] = img; wrem[w] = (oh >> 1) * OWq + (ow >> 1);
        }
    }
    // runs of four windows that are four consecutive floats of one pooled plane are stored as one 16-byte vector
    bool run[2];
#pragma unroll
    for (int h = 0; h < 2; h++)
        run[h] = wimg[4 * h + 3] == wimg[4 * h] && wrem[4 * h + 3] == wrem[4 * h] + 3 && (wrem[4 * h] & 3) == 0 && (Pq & 3) == 0 &&
                 row_base + r0[4 * h + 3] < M;
    const bool aligned = ((reinterpret_cast<uintptr_t>(po.pooled) | reinterpret_cast<uintptr_t>(po.mask)) & 15) == 0;
    for (int c = 0; c < ncols; c += 32) {
        float v[32];
        tmem_ld32_sum(taddr + (uint32_t)c, v, nacc, acc_stride);
        if (scale != 1.f) {
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] *= scale;
        }
        const int n = col_base + c + lane;                          // this lane's filter once lanes hold columns
        __syncwarp();
        stage[lane] = (bias && n < N) ? __ldg(bias + n) : 0.f;
        __syncwarp();
        if (act == 1) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                const float4 b4 = *reinterpret_cast<const float4 *>(stage + j);
                float z;
                z = v[j] + b4.x; v[j] = z > 0.f ? z : 0.f;
                z = v[j + 1] + b4.y; v[j + 1] = z > 0.f ? z : 0.f;
                z = v[j + 2] + b4.z; v[j + 2] = z > 0.f ? z : 0.f;
                z = v[j + 3] + b4.w; v[j + 3] = z > 0.f ? z : 0.f;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                const float4 b4 = *reinterpret_cast<const float4 *>(stage + j);
                v[j] = epilogue_act(v[j] + b4.x, act); v[j + 1] = epilogue_act(v[j + 1] + b4.y, act);
                v[j + 2] = epilogue_act(v[j + 2] + b4.z, act); v[j + 3] = epilogue_act(v[j + 3] + b4.w, act);
            }
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 32; j++) stage[lane * 33 + j] = v[j];
        __syncwarp();
        float mx[8];
        int ix[8];
#pragma unroll
        for (int w = 0; w < 8; w++) {
            const float a0 = stage[r0[w] * 33 + lane], a1 = stage[(r0[w] + 1) * 33 + lane];
            const float a2 = stage[(r0[w] + d2) * 33 + lane], a3 = stage[(r0[w] + d2 + 1) * 33 + lane];
            float m = -3.402823466e+38f; int id = 0;               // -FLT_MAX, strict comparisons: the first maximum wins
            if (a0 > m) { m = a0; id = 0; }
            if (a1 > m) { m = a1; id = 1; }
            if (a2 > m) { m = a2; id = 2; }
            if (a3 > m) { m = a3; id = 3; }
            mx[w] = m; ix[w] = id;
        }
        if (n < N) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const long long o = ((long long)wimg[4 * h] * N + n) * Pq + wrem[4 * h];
                if (run[h] && aligned) {
                    *reinterpret_cast<float4 *>(po.pooled + o) = make_float4(mx[4 * h], mx[4 * h + 1], mx[4 * h + 2], mx[4 * h + 3]);
                    *reinterpret_cast<int4 *>(po.mask + o) = make_int4(ix[4 * h], ix[4 * h + 1], ix[4 * h + 2], ix[4 * h + 3]);
                } else {
#pragma unroll
                    for (int w = 4 * h; w < 4 * h + 4; w++) {
                        if (row_base + r0[w] >= M) continue;
                        const long long q = ((long long)wimg[w] * N + n) * Pq + wrem[w];
                        po.pooled[q] = mx[w];
                        po.mask[q] = ix[w];
                    }
                }
            }
        }
        if (po.copy[0] && n < po.Cp) {                              // channels-last copies: lanes = consecutive channels
#pragma unroll
            for (int w = 0; w < 8; w++) {
                if (row_base + r0[w] >= M) continue;
                float r = n < N ? mx[w] : 0.f;
                const long long o = ((long long)wimg[w] * Pq + wrem[w]) * po.Cp + n;
                store_split1(r, po.ns, po.enc, po.copy[0] + o, po.copy[1] + o, po.copy[2] + o);
            }
        }
    }
}

}  // namespace seera
