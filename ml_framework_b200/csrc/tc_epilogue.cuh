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

template <class CS>
__device__ __forceinline__ void drain_accumulator(uint32_t taddr, int row_base, int col_base, int c_begin, int c_end,
                                                  int M, int N, const CS &cs, float *partial, long long partial_off,
                                                  float *stage /* EPI_WARP_SMEM bytes, this warp's own */,
                                                  const float *bias = nullptr, int act = 0) {
    const int lane = threadIdx.x & 31;
    const bool transpose = partial != nullptr || !CS::kMContiguous;
    const long long sn = cs.nstride();
    // direct path: this lane owns row m; its address part is computed once, not per element
    const int m_own = row_base + lane;
    float *own = (!transpose && m_own < M) ? cs.row(m_own) : nullptr;
    for (int c = c_begin; c < c_end; c += 32) {
        float v[32];
        tmem_ld32(taddr + (uint32_t)(c - c_begin), v);
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
                            if (rp) rp[n * sn] = fuse ? epilogue_act(stage[r * 33 + lane] + b, act) : stage[r * 33 + lane];
                        }
                    }
                }
            }
            __syncwarp();
        }
    }
}

}  // namespace seera
