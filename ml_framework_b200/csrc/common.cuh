// Shared host-side state and helpers for the engine's translation units.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include "seera_b200.h"

namespace seera {

struct Runtime {
    int device = -1;
    int sm_count = 148;                 // SMs the kernels size their grids for (physical count minus the "sm_reserve" option)
    int sm_physical = 148;
    cudaStream_t stream = nullptr;      // the stream every kernel is enqueued on
    cudaStream_t own_stream = nullptr;
    int precision = 0;                  // set from SEERA_PRECISION (default 3) when the runtime is created
    unsigned long long tc_wait_clocks = 4000000000ull;      // budget of a bounded wait inside a tensor-core kernel (~2 s)
    int tc_test_skip_load = -1;         // test hook ("tc_test_skip_load" option): see TmaGemmParams::skip_load
    bool dense_tma = true;              // Dense GEMMs in modes 1/2: TMA-fed kernel (false: in-kernel conversion kernel)
    int tile_n_cap2 = 128;              // widest accumulator tile with two operand copies per stage (bf16x3)
    int tile_n_cap3 = 128;              // ... with three (bf16x6)
    bool pool_short_patch = false;      // fold a 2x2 max-pool into the tensor-core short-patch forward kernel too (its epilogue warps become the
                                        // bottleneck: off; 3 x 3 unit-stride layers fold it into the fp32 stencil kernel regardless)
    bool wgrad_single = true;           // precision mode 4: weight gradients from the first fp16 copy of each operand alone
    bool skinny_gemm = true;            // Dense products of at most 16 output columns: exact fp32 on the CUDA cores in every mode
    int mma_issuers = 0;                // cap on the MMA-issuing threads of the TMA-fed GEMM kernel (0: none; 1 or 2)
    bool pair_tiles = false;            // TMA-fed GEMMs as clusters of two CTAs on 256-row tiles where the plan finds it pays
    bool conv_tma = true;               // convolutions in modes 1-3: TMA im2col kernel (false: in-kernel gather kernel)
    bool capturing = false;             // a stream capture (seera_graph_begin) is open
    bool tc_used = false;               // a tensor-core kernel ran since the status word was last read
    int status = 0;
    uint64_t launches = 0;
    char err[512] = {0};
};
Runtime &rt();
int fail(int code, const char *fmt, ...);       // records the status + message, returns code
int check_cuda(cudaError_t e, const char *what);
int ensure_init();

// Grid for a grid-stride kernel over `work_items` with `threads` per block: enough blocks to cover
// the work once, capped at a whole number of waves (8 resident 256-thread CTAs per SM).
inline int stride_grid(long long work_items, int threads = 256) {
    long long need = (work_items + threads - 1) / threads;
    long long cap = (long long)rt().sm_count * 8;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

inline void count_launch(int n = 1) { rt().launches += n; }

// out[c] = sum over s < splits of partial[s * n + c], added in a fixed order (the same bits on every run).  A block owns 32
// consecutive columns; its eight warps take the splits w, w + 8, ... (128-byte coalesced reads, splits / 8 dependent loads
// instead of `splits`), then the eight sums are added in warp order.  Columns at or beyond n_first go to out2 (may be null).
static __global__ void __launch_bounds__(256) sum_splits_kernel(const float *__restrict__ partial, float *__restrict__ out,
                                                                float *__restrict__ out2, int n_first, int n, int splits) {
    __shared__ float sm[8][33];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, c = blockIdx.x * 32 + lane;
    float t = 0.f;
    if (c < n) {
#pragma unroll 4
        for (int s = warp; s < splits; s += 8) t += __ldg(partial + (long long)s * n + c);
    }
    sm[warp][lane] = t;
    __syncthreads();
    if (warp == 0 && c < n) {
        float r = sm[0][lane];
#pragma unroll
        for (int w = 1; w < 8; w++) r += sm[w][lane];
        if (c < n_first) out[c] = r;
        else if (out2) out2[c - n_first] = r;
    }
}
inline void launch_sum_splits(const float *partial, float *out, int n, int splits, cudaStream_t st, float *out2 = nullptr, int n_first = -1) {
    sum_splits_kernel<<<(n + 31) / 32, 256, 0, st>>>(partial, out, out2, n_first < 0 ? n : n_first, n, splits);
    count_launch();
}

#define SEERA_ENSURE()                      \
    do {                                    \
        int _s = seera::ensure_init();      \
        if (_s) return _s;                  \
    } while (0)

#define SEERA_LAUNCH_CHECK(name)                                                   \
    do {                                                                           \
        seera::count_launch();                                                     \
        cudaError_t _e = cudaGetLastError();                                       \
        if (_e != cudaSuccess) return seera::check_cuda(_e, name);                 \
    } while (0)

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Contraction profile (seera_profile_enable): bracket a launch sequence with events and book its FLOPs.
void profile_begin();
void profile_end_bytes(double bytes, const char *tag);      // a bandwidth-bound pass: its algorithmic bytes
void profile_end(double flops, const char *name = nullptr);    // name ending in (dX)/(dA) or (dW)/(dB) books the launch as a backward product

// Brackets the launches of a bandwidth-bound pass for the profile: constructed before them, destroyed after them.
struct ProfBytes {
    double bytes;
    const char *tag;
    ProfBytes(double b, const char *t) : bytes(b), tag(t) { profile_begin(); }
    ~ProfBytes() { profile_end_bytes(bytes, tag); }
};

// Device float[2]: {dynamic factor of the fp16 gradient copies, its inverse}; both 1 until a loss head sets them (fused.cu).
float *grad_scale_words();

// Pool-backed scratch for internal use (split-K partials, operand shadows).
void graph_note_collective();              // runtime.cu: the open capture records a collective
void graphs_with_collectives_release();     // runtime.cu: destroy the executable graphs that hold collectives (before the communicator goes)
void *scratch_alloc(size_t bytes);
void scratch_free(void *p);

}  // namespace seera
