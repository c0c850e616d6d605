// Max-pool (argmax-index mask), nearest-neighbour unpooling and the single-axis reductions.
//
// Replaces engine_cuda/src/maxPool.cu:9-129, unpooling.cu:7-97 and reductionKernels.cu:12-379.
// Semantics follow the reference CPU engine, the parity oracle:
//   max-pool forward   engine/src/pool_ops.cpp:10-43   scan starts at -FLT_MAX, strict >, so the FIRST
//                      maximum wins; taps in the padding count as 0.0; mask = kh*KW + kw
//   max-pool backward  engine/src/pool_ops.cpp:45-71   add dout at the argmax tap, dropped if that tap is padding
//   unpooling          engine/src/pool_ops.cpp:74-109
// The reference GPU kernels differ (last maximum wins, 0/1 mask at input resolution, racy for overlapping
// windows: maxPool.cu:37-50, :63-64); the CPU engine's rule is the one implemented.
#include "common.cuh"
#include <cfloat>

namespace seera {

// ---- max-pool, general shape: one thread per output element ----------------------------------------
__global__ void __launch_bounds__(256) maxpool_fwd_kernel(const float *__restrict__ X, float *__restrict__ out, int *__restrict__ mask,
                                                          long long total, int H, int W, int OH, int OW,
                                                          int KH, int KW, int sh, int sw, int ph, int pw) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long o = tid; o < total; o += nthr) {
        int ow = (int)(o % OW); long long t = o / OW;
        int oh = (int)(t % OH); long long nc = t / OH;
        const float *xp = X + nc * H * W;
        float mx = -FLT_MAX; int idx = 0;
        for (int kh = 0; kh < KH; kh++) {
            int h = oh * sh + kh - ph;
            for (int kw = 0; kw < KW; kw++) {
                int w = ow * sw + kw - pw;
                float v = (h >= 0 && h < H && w >= 0 && w < W) ? __ldg(xp + (long long)h * W + w) : 0.0f;
                if (v > mx) { mx = v; idx = kh * KW + kw; }
            }
        }
        out[o] = mx; mask[o] = idx;
    }
}

// 2x2 window, stride 2, no padding, even H and W, W % 4 == 0: each thread produces two adjacent outputs
// from two float4 loads (rows 2*oh and 2*oh+1), so reads and writes are all 64/128-bit and coalesced.
__global__ void __launch_bounds__(256) maxpool2x2_fwd_kernel(const float4 *__restrict__ X, float2 *__restrict__ out,
                                                             int2 *__restrict__ mask, long long pairs, int OH, int OW2) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long q = tid; q < pairs; q += nthr) {
        int j = (int)(q % OW2); long long t = q / OW2;
        int oh = (int)(t % OH); long long nc = t / OH;
        long long row0 = (nc * (2 * OH) + 2 * oh) * OW2 + j;           // float4 index: a row holds OW2 float4
        float4 a = __ldg(X + row0), b = __ldg(X + row0 + OW2);
        float m0 = -FLT_MAX, m1 = -FLT_MAX; int i0 = 0, i1 = 0;
        if (a.x > m0) { m0 = a.x; i0 = 0; } if (a.y > m0) { m0 = a.y; i0 = 1; }
        if (b.x > m0) { m0 = b.x; i0 = 2; } if (b.y > m0) { m0 = b.y; i0 = 3; }
        if (a.z > m1) { m1 = a.z; i1 = 0; } if (a.w > m1) { m1 = a.w; i1 = 1; }
        if (b.z > m1) { m1 = b.z; i1 = 2; } if (b.w > m1) { m1 = b.w; i1 = 3; }
        out[q] = make_float2(m0, m1);
        mask[q] = make_int2(i0, i1);
    }
}

// Backward for the same 2x2/2 case: windows tile the input exactly, so each thread WRITES the two 2x2
// blocks of its output pair (no atomics, no zero-fill pass).
__global__ void __launch_bounds__(256) maxpool2x2_bwd_kernel(const float2 *__restrict__ dout, const int2 *__restrict__ mask,
                                                             float4 *__restrict__ dX, long long pairs, int OH, int OW2) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long q = tid; q < pairs; q += nthr) {
        int j = (int)(q % OW2); long long t = q / OW2;
        int oh = (int)(t % OH); long long nc = t / OH;
        float2 d = __ldg(dout + q); int2 m = __ldg(mask + q);
        float4 a, b;
        a.x = m.x == 0 ? d.x : 0.f; a.y = m.x == 1 ? d.x : 0.f; b.x = m.x == 2 ? d.x : 0.f; b.y = m.x == 3 ? d.x : 0.f;
        a.z = m.y == 0 ? d.y : 0.f; a.w = m.y == 1 ? d.y : 0.f; b.z = m.y == 2 ? d.y : 0.f; b.w = m.y == 3 ? d.y : 0.f;
        long long row0 = (nc * (2 * OH) + 2 * oh) * OW2 + j;
        dX[row0] = a; dX[row0 + OW2] = b;
    }
}

// General backward, gather form: one thread per INPUT element sums dout over every window whose argmax
// tap is this element.  No atomics, deterministic, dX fully written.
__global__ void __launch_bounds__(256) maxpool_bwd_kernel(const float *__restrict__ dout, const int *__restrict__ mask,
                                                          float *__restrict__ dX, long long total, int H, int W, int OH, int OW,
                                                          int KH, int KW, int sh, int sw, int ph, int pw) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long i = tid; i < total; i += nthr) {
        int w = (int)(i % W); long long t = i / W;
        int h = (int)(t % H); long long nc = t / H;
        float acc = 0.f;
        for (int kh = 0; kh < KH; kh++) {
            int hh = h + ph - kh;
            if (hh < 0 || hh % sh) continue;
            int oh = hh / sh; if (oh >= OH) continue;
            for (int kw = 0; kw < KW; kw++) {
                int ww = w + pw - kw;
                if (ww < 0 || ww % sw) continue;
                int ow = ww / sw; if (ow >= OW) continue;
                long long o = (nc * OH + oh) * OW + ow;
                if (__ldg(mask + o) == kh * KW + kw) acc += __ldg(dout + o);
            }
        }
        dX[i] = acc;
    }
}

// ---- nearest-neighbour unpooling ----------------------------------------------------------------------
__global__ void __launch_bounds__(256) unpool_fwd_kernel(const float *__restrict__ x, float *__restrict__ out, long long total,
                                                         int H, int W, int sh, int sw) {
    int Ho = H * sh, Wo = W * sw;
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long o = tid; o < total; o += nthr) {
        int w = (int)(o % Wo); long long t = o / Wo;
        int h = (int)(t % Ho); long long nc = t / Ho;
        out[o] = __ldg(x + (nc * H + h / sh) * W + w / sw);
    }
}
__global__ void __launch_bounds__(256) unpool_bwd_kernel(const float *__restrict__ dout, float *__restrict__ dx, long long total,
                                                         int H, int W, int sh, int sw) {
    int Wo = W * sw;
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long i = tid; i < total; i += nthr) {
        int w = (int)(i % W); long long t = i / W;
        int h = (int)(t % H); long long nc = t / H;
        float s = 0.f;
        for (int a = h * sh; a < (h + 1) * sh; a++)
            for (int b = w * sw; b < (w + 1) * sw; b++) s += __ldg(dout + (nc * H * sh + a) * Wo + b);
        dx[i] = s;
    }
}

// Fast paths for tensors under 2^31 elements: 32-bit index arithmetic (the 64-bit divisions above cost more than the
// memory traffic) and, when the output width is a multiple of 4, one 16-byte store per thread.
template <bool V4>
__global__ void __launch_bounds__(256) unpool_fwd32_kernel(const float *__restrict__ x, float *__restrict__ out, unsigned items,
                                                           unsigned H, unsigned W, unsigned sh, unsigned sw) {
    const unsigned Ho = H * sh, Wo = W * sw, Wq = V4 ? Wo / 4 : Wo;
    for (unsigned q = blockIdx.x * blockDim.x + threadIdx.x; q < items; q += gridDim.x * blockDim.x) {
        unsigned row = q / Wq, wq = q - row * Wq;
        unsigned nc = row / Ho, h = row - nc * Ho;
        const float *src = x + ((size_t)nc * H + h / sh) * W;
        if (V4) {
            unsigned w0 = wq * 4;
            float4 v = make_float4(__ldg(src + w0 / sw), __ldg(src + (w0 + 1) / sw), __ldg(src + (w0 + 2) / sw), __ldg(src + (w0 + 3) / sw));
            *reinterpret_cast<float4 *>(out + (size_t)q * 4) = v;
        } else {
            out[q] = __ldg(src + wq / sw);
        }
    }
}
__global__ void __launch_bounds__(256) unpool_bwd32_kernel(const float *__restrict__ dout, float *__restrict__ dx, unsigned total,
                                                           unsigned H, unsigned W, unsigned sh, unsigned sw) {
    const unsigned Wo = W * sw;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        unsigned row = i / W, w = i - row * W;             // row = nc * H + h
        const float *src = dout + (size_t)row * sh * Wo + w * sw;
        float s = 0.f;
        for (unsigned a = 0; a < sh; a++)
            for (unsigned b = 0; b < sw; b++) s += __ldg(src + (size_t)a * Wo + b);
        dx[i] = s;
    }
}

// ---- reductions over a tensor viewed as [outer, n, inner] ------------------------------------------------
enum { R_SUM = 0, R_MEAN = 1, R_MAX = 2, R_MIN = 3 };

// inner > 1, or short rows: one thread per output element walks the axis (threads adjacent in `inner`
// read adjacent addresses).
template <int OP>
__global__ void __launch_bounds__(256) reduce_strided_kernel(const float *__restrict__ A, float *__restrict__ out,
                                                             long long outputs, int n, long long inner) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long o = tid; o < outputs; o += nthr) {
        const float *p = A + (o / inner) * n * inner + (o % inner);
        float acc = (OP <= R_MEAN) ? 0.f : p[0];
        for (int k = 0; k < n; k++) {
            float v = __ldg(p + (long long)k * inner);
            if (OP <= R_MEAN) acc += v; else if (OP == R_MAX) acc = v > acc ? v : acc; else acc = v < acc ? v : acc;
        }
        out[o] = OP == R_MEAN ? acc / (float)n : acc;
    }
}

// inner == 1 and long rows: one warp per row, lanes stride the row, shuffle tree at the end.
template <int OP>
__global__ void __launch_bounds__(256) reduce_rows_kernel(const float *__restrict__ A, float *__restrict__ out, long long rows, int n) {
    long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    long long nwarp = (long long)gridDim.x * (blockDim.x >> 5);
    int lane = threadIdx.x & 31;
    for (; row < rows; row += nwarp) {
        const float *p = A + row * n;
        float acc = (OP <= R_MEAN) ? 0.f : p[0];
        for (int k = lane; k < n; k += 32) {
            float v = __ldg(p + k);
            if (OP <= R_MEAN) acc += v; else if (OP == R_MAX) acc = v > acc ? v : acc; else acc = v < acc ? v : acc;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float v = __shfl_xor_sync(0xffffffffu, acc, o);
            if (OP <= R_MEAN) acc += v; else if (OP == R_MAX) acc = v > acc ? v : acc; else acc = v < acc ? v : acc;
        }
        if (lane == 0) out[row] = OP == R_MEAN ? acc / (float)n : acc;
    }
}

// Sum over the OUTER axis of [n, inner] with few outputs and a long axis (bias-gradient shape):
// grid (ceil(inner/32), splits), block 32 columns x 8 row lanes; partial[s][col] then a second pass.
__global__ void __launch_bounds__(256) reduce_outer_partial_kernel(const float *__restrict__ A, float *__restrict__ partial,
                                                                   int n, long long inner) {
    __shared__ float sm[8][33];
    long long col = (long long)blockIdx.x * 32 + (threadIdx.x & 31);
    int lane_r = threadIdx.x >> 5, s = blockIdx.y, splits = gridDim.y;
    float acc = 0.f;
    if (col < inner)
        for (int r = s * 8 + lane_r; r < n; r += splits * 8) acc += __ldg(A + (long long)r * inner + col);
    sm[lane_r][threadIdx.x & 31] = acc;
    __syncthreads();
    if (lane_r == 0 && col < inner) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; k++) t += sm[k][threadIdx.x];
        partial[(long long)s * inner + col] = t;
    }
}
__global__ void __launch_bounds__(256) reduce_outer_final_kernel(const float *__restrict__ partial, float *__restrict__ out,
                                                                 long long inner, int splits, float scale) {
    long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= inner) return;
    float t = 0.f;
    for (int s = 0; s < splits; s++) t += partial[(long long)s * inner + c];
    out[c] = t * scale;
}

template <bool MAX>
__global__ void __launch_bounds__(256) argreduce_kernel(const float *__restrict__ A, int *__restrict__ out,
                                                        long long outputs, int n, long long inner) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long o = tid; o < outputs; o += nthr) {
        const float *p = A + (o / inner) * n * inner + (o % inner);
        float best = p[0]; int bi = 0;
        for (int k = 1; k < n; k++) {
            float v = __ldg(p + (long long)k * inner);
            if (MAX ? v > best : v < best) { best = v; bi = k; }     // strict: first extremum wins
        }
        out[o] = bi;
    }
}

__global__ void __launch_bounds__(256) reduce_bwd_kernel(const float *__restrict__ dOut, float *__restrict__ dA,
                                                         long long total, int n, long long inner, float scale) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long i = tid; i < total; i += nthr) {
        long long o = (i / (inner * n)) * inner + (i % inner);
        dA[i] = __ldg(dOut + o) * scale;
    }
}

// max/min backward: the first element along the axis equal to the forward output receives dOut (added
// into dA, which the caller zero-fills: Seera_Engine.py:457-462).
__global__ void __launch_bounds__(256) extremum_bwd_kernel(const float *__restrict__ dOut, const float *__restrict__ A,
                                                           const float *__restrict__ fo, float *__restrict__ dA,
                                                           long long outputs, int n, long long inner) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long o = tid; o < outputs; o += nthr) {
        long long base = (o / inner) * n * inner + (o % inner);
        float target = fo[o];
        for (int k = 0; k < n; k++) {
            if (A[base + (long long)k * inner] == target) { dA[base + (long long)k * inner] += dOut[o]; break; }
        }
    }
}

struct AxisView { long long outer, inner; int n; };

static int axis_view(int ndims, int dim, const int *dimarr, AxisView &v, const char *name) {
    if (ndims < 1 || ndims > 16 || !dimarr) return fail(SEERA_E_ARG, "%s: ndims %d", name, ndims);
    if (dim < 0) dim += ndims;
    if (dim < 0 || dim >= ndims) return fail(SEERA_E_ARG, "%s: dim out of range", name);
    v.outer = 1; v.inner = 1;
    for (int i = 0; i < ndims; i++) {
        if (dimarr[i] < 1) return fail(SEERA_E_ARG, "%s: empty dimension", name);
        if (i < dim) v.outer *= dimarr[i]; else if (i > dim) v.inner *= dimarr[i];
    }
    v.n = dimarr[dim];
    return SEERA_OK;
}

template <int OP>
static int reduce_fwd(const float *A, float *out, int ndims, int dim, const int *dimarr, const char *name) {
    SEERA_ENSURE();
    AxisView v;
    if (int s = axis_view(ndims, dim, dimarr, v, name)) return s;
    if (!A || !out) return fail(SEERA_E_ARG, "%s: null pointer", name);
    long long outputs = v.outer * v.inner;
    cudaStream_t st = rt().stream;
    if (OP <= R_MEAN && v.outer == 1 && v.inner <= 65536 && v.n >= 256) {
        int colblocks = (int)((v.inner + 31) / 32);
        int splits = (rt().sm_count * 4 + colblocks - 1) / colblocks;
        int maxs = (v.n + 7) / 8; if (splits > maxs) splits = maxs; if (splits < 1) splits = 1;
        float *partial = (float *)scratch_alloc((size_t)splits * v.inner * sizeof(float));
        if (!partial) return SEERA_E_OOM;
        reduce_outer_partial_kernel<<<dim3(colblocks, splits), 256, 0, st>>>(A, partial, v.n, v.inner);
        SEERA_LAUNCH_CHECK(name);
        reduce_outer_final_kernel<<<(int)((v.inner + 255) / 256), 256, 0, st>>>(partial, out, v.inner, splits,
                                                                               OP == R_MEAN ? 1.0f / (float)v.n : 1.0f);
        scratch_free(partial);
        SEERA_LAUNCH_CHECK(name);
    } else if (v.inner == 1 && v.n >= 64) {
        reduce_rows_kernel<OP><<<stride_grid(outputs * 32), 256, 0, st>>>(A, out, outputs, v.n);
        SEERA_LAUNCH_CHECK(name);
    } else {
        reduce_strided_kernel<OP><<<stride_grid(outputs), 256, 0, st>>>(A, out, outputs, v.n, v.inner);
        SEERA_LAUNCH_CHECK(name);
    }
    return SEERA_OK;
}

}  // namespace seera

using namespace seera;

extern "C" {

int seera_cuda_maxpool_fwd(const float *X, float *out, int *mask, int N, int C, int H, int W, int R, int S,
                           int ph, int pw, int sh, int sw) {
    SEERA_ENSURE();
    if (N < 1 || C < 1 || H < 1 || W < 1 || R < 1 || S < 1 || sh < 1 || sw < 1 || ph < 0 || pw < 0 || !X || !out || !mask)
        return fail(SEERA_E_ARG, "cuda_maxpool_fwd: bad argument");
    int OH = (H + 2 * ph - R) / sh + 1, OW = (W + 2 * pw - S) / sw + 1;
    if (OH < 1 || OW < 1) return fail(SEERA_E_ARG, "cuda_maxpool_fwd: window larger than padded input");
    if ((long long)OH * OW > (long long)H * W)
        return fail(SEERA_E_ARG, "cuda_maxpool_fwd: %dx%d outputs do not fit the caller's %dx%d mask buffer", OH, OW, H, W);
    long long total = (long long)N * C * OH * OW;
    ProfBytes pb(4.0 * N * C * H * W + 8.0 * total, "maxpool_fwd");
    if (R == 2 && S == 2 && sh == 2 && sw == 2 && ph == 0 && pw == 0 && H % 2 == 0 && W % 4 == 0 &&
        aligned16(X) && aligned16(out) && aligned16(mask)) {
        long long pairs = total / 2;
        maxpool2x2_fwd_kernel<<<stride_grid(pairs), 256, 0, rt().stream>>>(reinterpret_cast<const float4 *>(X),
            reinterpret_cast<float2 *>(out), reinterpret_cast<int2 *>(mask), pairs, OH, OW / 2);
    } else {
        maxpool_fwd_kernel<<<stride_grid(total), 256, 0, rt().stream>>>(X, out, mask, total, H, W, OH, OW, R, S, sh, sw, ph, pw);
    }
    SEERA_LAUNCH_CHECK("cuda_maxpool_fwd");
    return SEERA_OK;
}

int seera_cuda_maxpool_bwd(const float *dout, const int *mask, float *dX, int N, int C, int H, int W, int R, int S,
                           int ph, int pw, int sh, int sw) {
    SEERA_ENSURE();
    if (N < 1 || C < 1 || H < 1 || W < 1 || R < 1 || S < 1 || sh < 1 || sw < 1 || ph < 0 || pw < 0 || !dout || !dX || !mask)
        return fail(SEERA_E_ARG, "cuda_maxpool_bwd: bad argument");
    int OH = (H + 2 * ph - R) / sh + 1, OW = (W + 2 * pw - S) / sw + 1;
    if (OH < 1 || OW < 1) return fail(SEERA_E_ARG, "cuda_maxpool_bwd: window larger than padded input");
    ProfBytes pb(4.0 * N * C * H * W + 8.0 * N * C * OH * OW, "maxpool_bwd");
    if (R == 2 && S == 2 && sh == 2 && sw == 2 && ph == 0 && pw == 0 && H % 2 == 0 && W % 4 == 0 &&
        aligned16(dX) && aligned16(dout) && aligned16(mask)) {
        long long pairs = (long long)N * C * OH * OW / 2;
        maxpool2x2_bwd_kernel<<<stride_grid(pairs), 256, 0, rt().stream>>>(reinterpret_cast<const float2 *>(dout),
            reinterpret_cast<const int2 *>(mask), reinterpret_cast<float4 *>(dX), pairs, OH, OW / 2);
    } else {
        long long total = (long long)N * C * H * W;
        maxpool_bwd_kernel<<<stride_grid(total), 256, 0, rt().stream>>>(dout, mask, dX, total, H, W, OH, OW, R, S, sh, sw, ph, pw);
    }
    SEERA_LAUNCH_CHECK("cuda_maxpool_bwd");
    return SEERA_OK;
}

int seera_cuda_unpooling_fwd(const float *inp, float *out, int N, int C, int H, int W, int sh, int sw) {
    SEERA_ENSURE();
    if (N < 1 || C < 1 || H < 1 || W < 1 || sh < 1 || sw < 1 || !inp || !out) return fail(SEERA_E_ARG, "cuda_unpooling_fwd: bad argument");
    long long total = (long long)N * C * H * sh * W * sw;
    ProfBytes pb(4.0 * N * C * H * W + 4.0 * total, "unpool_fwd");
    if (total < (1LL << 31)) {
        const bool v4 = (W * sw) % 4 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
        unsigned items = (unsigned)(v4 ? total / 4 : total);
        if (v4) unpool_fwd32_kernel<true><<<stride_grid(items), 256, 0, rt().stream>>>(inp, out, items, H, W, sh, sw);
        else unpool_fwd32_kernel<false><<<stride_grid(items), 256, 0, rt().stream>>>(inp, out, items, H, W, sh, sw);
    } else {
        unpool_fwd_kernel<<<stride_grid(total), 256, 0, rt().stream>>>(inp, out, total, H, W, sh, sw);
    }
    SEERA_LAUNCH_CHECK("cuda_unpooling_fwd");
    return SEERA_OK;
}
int seera_cuda_unpooling_bwd(const float *dout, float *dx, int N, int C, int H, int W, int sh, int sw) {
    SEERA_ENSURE();
    if (N < 1 || C < 1 || H < 1 || W < 1 || sh < 1 || sw < 1 || !dout || !dx) return fail(SEERA_E_ARG, "cuda_unpooling_bwd: bad argument");
    long long total = (long long)N * C * H * W;
    ProfBytes pb(4.0 * total + 4.0 * total * sh * sw, "unpool_bwd");
    if (total * sh * sw < (1LL << 31)) unpool_bwd32_kernel<<<stride_grid(total), 256, 0, rt().stream>>>(dout, dx, (unsigned)total, H, W, sh, sw);
    else unpool_bwd_kernel<<<stride_grid(total), 256, 0, rt().stream>>>(dout, dx, total, H, W, sh, sw);
    SEERA_LAUNCH_CHECK("cuda_unpooling_bwd");
    return SEERA_OK;
}

int seera_cuda_sum_fwd(const float *A, float *out, int nd, int dim, const int *da)  { return reduce_fwd<R_SUM>(A, out, nd, dim, da, "cuda_sum_fwd"); }
int seera_cuda_mean_fwd(const float *A, float *out, int nd, int dim, const int *da) { return reduce_fwd<R_MEAN>(A, out, nd, dim, da, "cuda_mean_fwd"); }
int seera_cuda_max_fwd(const float *A, float *out, int nd, int dim, const int *da)  { return reduce_fwd<R_MAX>(A, out, nd, dim, da, "cuda_max_fwd"); }
int seera_cuda_min_fwd(const float *A, float *out, int nd, int dim, const int *da)  { return reduce_fwd<R_MIN>(A, out, nd, dim, da, "cuda_min_fwd"); }

static int arg_fwd(const float *A, int *out, int nd, int dim, const int *da, bool mx, const char *name) {
    SEERA_ENSURE();
    AxisView v;
    if (int s = axis_view(nd, dim, da, v, name)) return s;
    if (!A || !out) return fail(SEERA_E_ARG, "%s: null pointer", name);
    long long outputs = v.outer * v.inner;
    if (mx) argreduce_kernel<true><<<stride_grid(outputs), 256, 0, rt().stream>>>(A, out, outputs, v.n, v.inner);
    else argreduce_kernel<false><<<stride_grid(outputs), 256, 0, rt().stream>>>(A, out, outputs, v.n, v.inner);
    SEERA_LAUNCH_CHECK(name);
    return SEERA_OK;
}
int seera_cuda_argmax_fwd(const float *A, int *out, int nd, int dim, const int *da) { return arg_fwd(A, out, nd, dim, da, true, "cuda_argmax_fwd"); }
int seera_cuda_argmin_fwd(const float *A, int *out, int nd, int dim, const int *da) { return arg_fwd(A, out, nd, dim, da, false, "cuda_argmin_fwd"); }

static int bcast_bwd(const float *dOut, float *dA, int nd, int dim, const int *da, bool mean, const char *name) {
    SEERA_ENSURE();
    AxisView v;
    if (int s = axis_view(nd, dim, da, v, name)) return s;
    if (!dOut || !dA) return fail(SEERA_E_ARG, "%s: null pointer", name);
    long long total = v.outer * v.n * v.inner;
    reduce_bwd_kernel<<<stride_grid(total), 256, 0, rt().stream>>>(dOut, dA, total, v.n, v.inner, mean ? 1.0f / (float)v.n : 1.0f);
    SEERA_LAUNCH_CHECK(name);
    return SEERA_OK;
}
int seera_cuda_sum_bwd(const float *dOut, float *dA, int nd, int dim, const int *da)  { return bcast_bwd(dOut, dA, nd, dim, da, false, "cuda_sum_bwd"); }
int seera_cuda_mean_bwd(const float *dOut, float *dA, int nd, int dim, const int *da) { return bcast_bwd(dOut, dA, nd, dim, da, true, "cuda_mean_bwd"); }

static int ext_bwd(const float *dOut, const float *fi, const float *fo, float *dA, int nd, int dim, const int *da, const char *name) {
    SEERA_ENSURE();
    AxisView v;
    if (int s = axis_view(nd, dim, da, v, name)) return s;
    if (!dOut || !fi || !fo || !dA) return fail(SEERA_E_ARG, "%s: null pointer", name);
    long long outputs = v.outer * v.inner;
    extremum_bwd_kernel<<<stride_grid(outputs), 256, 0, rt().stream>>>(dOut, fi, fo, dA, outputs, v.n, v.inner);
    SEERA_LAUNCH_CHECK(name);
    return SEERA_OK;
}
int seera_cuda_max_bwd(const float *dOut, const float *fi, const float *fo, float *dA, int nd, int dim, const int *da) { return ext_bwd(dOut, fi, fo, dA, nd, dim, da, "cuda_max_bwd"); }
int seera_cuda_min_bwd(const float *dOut, const float *fi, const float *fo, float *dA, int nd, int dim, const int *da) { return ext_bwd(dOut, fi, fo, dA, nd, dim, da, "cuda_min_bwd"); }

}  // extern "C"
