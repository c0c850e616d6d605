// Batch normalisation, forward and backward, for [N, C] and [N, C, H, W] tensors.
//
// The reference runs this layer on the CPU only, even in its GPU path (Seera_init.py:870-921 forward,
// Seera_Engine.py:381-415 backward, engine/src/batchnorm_ops.cpp:12-138 the arithmetic): every batch goes device -> host
// -> device around it.  Here it is two bandwidth-bound passes over the tensor forward (statistics, normalise) and two backward
// (sums of dout and dout * x_hat, dx), each with a C-thread finalise between them.
//
// Statistics.  The reference takes the mean first and the variance from the differences to it (two passes over x).  Here every
// thread walks its share of a channel ONCE, accumulating sum (x - K) and sum (x - K)^2 around the first value K it meets - a
// sample of the same distribution, so the subtraction in  M2 = s2 - s1^2 / n  cancels a few bits at most - and the per-thread
// triples (n, mean, M2) are merged pairwise with Chan's update  mean = mean_a + d * n_b / n,  M2 = M2_a + M2_b + d^2 * n_a * n_b / n
// (d = mean_b - mean_a) in a fixed order: lanes, warps, then the split rows.  That is as accurate as the two-pass form (both are
// within a few ulp of the fp64 result; the parity tests hold the outputs to 1e-5 of the CPU engine's) for one read less.
// Every other reduction has a fixed order too: per-thread strided partials, a block tree, then the partial rows summed in split
// order.  x_hat is not stored: the backward recomputes it from the layer input, the saved mean and 1/std (one multiply-add
// against a second activation-sized buffer of traffic).
//
// Layout [N, C, S] with S = H*W (1 for the 1-D form).  S > 1: a block owns one channel and a stripe of images and reads
// its planes contiguously.  S == 1: a block owns 32 adjacent channels x a stripe of rows, so warps read rows contiguously.
#include "common.cuh"

namespace seera {

constexpr int BN_MAX_SPLITS = 64;

__device__ __forceinline__ float bn_block_sum(float v, float *sm /* 8 floats */) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) r += sm[w];
    return r;
}
// sum over the split rows of a [splits, C] partial table, in split order
__device__ __forceinline__ float bn_sum_partials(const float *partial, int c, int C, int splits) {
    float t = 0.f;
    for (int s = 0; s < splits; s++) t += partial[(long long)s * C + c];
    return t;
}

// ---- one-pass statistics -------------------------------------------------------------------------------------------
struct BnMoments { float n, mean, m2; };
__device__ __forceinline__ BnMoments bn_merge(const BnMoments &a, const BnMoments &b) {
    const float n = a.n + b.n;
    if (n == 0.f) return BnMoments{0.f, 0.f, 0.f};
    const float d = b.mean - a.mean, w = b.n / n;
    return BnMoments{n, a.mean + d * w, a.m2 + b.m2 + d * d * a.n * w};
}
struct BnShifted {                 // a thread's running sums around its first value
    float k, s1, s2, n;
    __device__ __forceinline__ void add(float v) {
        if (n == 0.f) k = v;
        const float d = v - k;
        s1 += d; s2 += d * d; n += 1.f;
    }
    __device__ __forceinline__ BnMoments done() const {
        if (n == 0.f) return BnMoments{0.f, 0.f, 0.f};
        return BnMoments{n, k + s1 / n, fmaxf(s2 - s1 * s1 / n, 0.f)};
    }
};
__device__ __forceinline__ BnMoments bn_warp_merge(BnMoments m) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {              // lane l merges (l, l ^ o) with the lower lane first: every lane ends with the same bits
        BnMoments other{__shfl_xor_sync(0xffffffffu, m.n, o), __shfl_xor_sync(0xffffffffu, m.mean, o), __shfl_xor_sync(0xffffffffu, m.m2, o)};
        m = ((threadIdx.x & o) == 0) ? bn_merge(m, other) : bn_merge(other, m);
    }
    return m;
}
// partial[(split * C + c) * 3 + {0, 1, 2}] = (n, mean, M2) of channel c over the images split, split + splits, ...
__global__ void __launch_bounds__(256) bn_stats_planes_kernel(const float *__restrict__ x, float *__restrict__ partial, int N, int C, int S,
                                                              int splits, int vec) {
    __shared__ float sm[8][3];
    const int c = blockIdx.x, split = blockIdx.y;
    BnShifted acc{0.f, 0.f, 0.f, 0.f};
    for (int n = split; n < N; n += splits) {
        const float *plane = x + ((long long)n * C + c) * S;
        if (vec) {
            const float4 *p4 = reinterpret_cast<const float4 *>(plane);
            for (int s = threadIdx.x; s < (S >> 2); s += 256) {
                const float4 v = __ldg(p4 + s);
                acc.add(v.x); acc.add(v.y); acc.add(v.z); acc.add(v.w);
            }
        } else {
            for (int s = threadIdx.x; s < S; s += 256) acc.add(__ldg(plane + s));
        }
    }
    BnMoments m = bn_warp_merge(acc.done());
    if ((threadIdx.x & 31) == 0) { sm[threadIdx.x >> 5][0] = m.n; sm[threadIdx.x >> 5][1] = m.mean; sm[threadIdx.x >> 5][2] = m.m2; }
    __syncthreads();
    if (threadIdx.x == 0) {
        BnMoments t{sm[0][0], sm[0][1], sm[0][2]};
#pragma unroll
        for (int w = 1; w < 8; w++) t = bn_merge(t, BnMoments{sm[w][0], sm[w][1], sm[w][2]});
        float *o = partial + ((long long)split * C + c) * 3;
        o[0] = t.n; o[1] = t.mean; o[2] = t.m2;
    }
}
// [N, C] rows: a block owns 32 adjacent channels and the rows split * 8 + ry, + splits * 8, ...
__global__ void __launch_bounds__(256) bn_stats_rows_kernel(const float *__restrict__ x, float *__restrict__ partial, int N, int C, int splits) {
    __shared__ float sm[8][32][3];
    const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + cx, split = blockIdx.y;
    BnShifted acc{0.f, 0.f, 0.f, 0.f};
    if (c < C)
        for (int n = split * 8 + ry; n < N; n += splits * 8) acc.add(__ldg(x + (long long)n * C + c));
    const BnMoments m = acc.done();
    sm[ry][cx][0] = m.n; sm[ry][cx][1] = m.mean; sm[ry][cx][2] = m.m2;
    __syncthreads();
    if (ry == 0 && c < C) {
        BnMoments t{sm[0][cx][0], sm[0][cx][1], sm[0][cx][2]};
#pragma unroll
        for (int r = 1; r < 8; r++) t = bn_merge(t, BnMoments{sm[r][cx][0], sm[r][cx][1], sm[r][cx][2]});
        float *o = partial + ((long long)split * C + c) * 3;
        o[0] = t.n; o[1] = t.mean; o[2] = t.m2;
    }
}

// ---- backward sums: per channel  sum dy -> out0  and  sum dy * x_hat -> out1,  x_hat = (x - mean[c]) * std_inv[c] ----------
__global__ void __launch_bounds__(256) bn_reduce_planes_kernel(const float *__restrict__ x, const float *__restrict__ dy,
                                                               const float *__restrict__ mean,
                                                               const float *__restrict__ std_inv, float *__restrict__ out0,
                                                               float *__restrict__ out1, int N, int C, int S, int splits) {
    __shared__ float sm[8];
    const int c = blockIdx.x, split = blockIdx.y;
    const float mu = mean[c], si = std_inv[c];
    float a0 = 0.f, a1 = 0.f;
    const bool vec = (S & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy)) & 15) == 0;
    for (int n = split; n < N; n += splits) {
        const long long base = ((long long)n * C + c) * S;
        if (vec) {
            const float4 *x4 = reinterpret_cast<const float4 *>(x + base), *g4 = reinterpret_cast<const float4 *>(dy + base);
            for (int s = threadIdx.x; s < (S >> 2); s += 256) {
                const float4 v = __ldg(x4 + s), g = __ldg(g4 + s);
                a0 += (g.x + g.y) + (g.z + g.w);
                a1 += (g.x * ((v.x - mu) * si) + g.y * ((v.y - mu) * si)) + (g.z * ((v.z - mu) * si) + g.w * ((v.w - mu) * si));
            }
            continue;
        }
        for (int s = threadIdx.x; s < S; s += 256) {
            const float v = __ldg(x + base + s);
            const float g = __ldg(dy + base + s);
            a0 += g; a1 += g * ((v - mu) * si);
        }
    }
    a0 = bn_block_sum(a0, sm);
    a1 = bn_block_sum(a1, sm);
    if (threadIdx.x == 0) {
        out0[(long long)split * C + c] = a0;
        out1[(long long)split * C + c] = a1;
    }
}
__global__ void __launch_bounds__(256) bn_reduce_rows_kernel(const float *__restrict__ x, const float *__restrict__ dy,
                                                             const float *__restrict__ mean,
                                                             const float *__restrict__ std_inv, float *__restrict__ out0,
                                                             float *__restrict__ out1, int N, int C, int splits) {
    __shared__ float s0[8][32], s1[8][32];
    const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + cx, split = blockIdx.y;
    const bool live = c < C;
    const float mu = live ? mean[c] : 0.f, si = live ? std_inv[c] : 0.f;
    float a0 = 0.f, a1 = 0.f;
    if (live) {
        for (int n = split * 8 + ry; n < N; n += splits * 8) {
            const float v = __ldg(x + (long long)n * C + c);
            const float g = __ldg(dy + (long long)n * C + c);
            a0 += g; a1 += g * ((v - mu) * si);
        }
    }
    s0[ry][cx] = a0; s1[ry][cx] = a1;
    __syncthreads();
    if (ry == 0 && live) {
        float t0 = 0.f, t1 = 0.f;
#pragma unroll
        for (int r = 0; r < 8; r++) { t0 += s0[r][cx]; t1 += s1[r][cx]; }
        out0[(long long)split * C + c] = t0;
        out1[(long long)split * C + c] = t1;
    }
}

// mean, 1/std and the running statistics of every channel (training: the split rows' moments merged in split order), or the
// running statistics as they are (inference)
__global__ void __launch_bounds__(256) bn_finalize_fwd_kernel(const float *__restrict__ moments, float *__restrict__ running_mean,
                                                              float *__restrict__ running_var, float *__restrict__ mean_out,
                                                              float *__restrict__ std_inv_out, int C, int splits, float M, float momentum,
                                                              float eps, int training) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    if (training) {
        BnMoments t{0.f, 0.f, 0.f};
        for (int s = 0; s < splits; s++) {
            const float *p = moments + ((long long)s * C + c) * 3;
            t = bn_merge(t, BnMoments{p[0], p[1], p[2]});
        }
        const float mu = t.mean, var = t.m2 / (M > 0.f ? M : t.n);        // M <= 0: the count comes with the moments (shards of several ranks)
        mean_out[c] = mu;
        std_inv_out[c] = 1.0f / sqrtf(var + eps);
        running_mean[c] = (1.0f - momentum) * running_mean[c] + momentum * mu;
        running_var[c] = (1.0f - momentum) * running_var[c] + momentum * var;
    } else {
        mean_out[c] = running_mean[c];
        std_inv_out[c] = 1.0f / sqrtf(running_var[c] + eps);
    }
}
// Cross-rank statistics: this rank's moments (its split rows merged in split order) into its slot of a [world, C, 3] table whose
// other slots are zero; the table is then summed over the ranks - adding zeros is exact, so every rank ends with every rank's
// moments - and bn_finalize_fwd_kernel merges the `world` rows in rank order like split rows.
__global__ void __launch_bounds__(256) bn_merge_local_kernel(const float *__restrict__ moments, float *__restrict__ slot, int C, int splits) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    BnMoments t{0.f, 0.f, 0.f};
    for (int s = 0; s < splits; s++) {
        const float *p = moments + ((long long)s * C + c) * 3;
        t = bn_merge(t, BnMoments{p[0], p[1], p[2]});
    }
    slot[c * 3] = t.n; slot[c * 3 + 1] = t.mean; slot[c * 3 + 2] = t.m2;
}
// Backward across ranks: sums[0..C) = sum dy, sums[C..2C) = sum dy * x_hat of this rank, sums[2C] = its element count per channel;
// summed over the ranks before bn_dx reads them.
__global__ void __launch_bounds__(256) bn_pack_sums_kernel(const float *__restrict__ dbeta, const float *__restrict__ dgamma,
                                                           float *__restrict__ sums, int C, float count) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < C) { sums[c] = dbeta[c]; sums[C + c] = dgamma[c]; }
    if (c == 0) sums[2 * C] = count;
}
__global__ void __launch_bounds__(256) bn_finalize_bwd_kernel(const float *__restrict__ p0, const float *__restrict__ p1,
                                                              float *__restrict__ dbeta, float *__restrict__ dgamma, int C, int splits) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    dbeta[c] = bn_sum_partials(p0, c, C, splits);
    dgamma[c] = bn_sum_partials(p1, c, C, splits);
}

// y = gamma * (x - mean) * std_inv + beta
__global__ void __launch_bounds__(256) bn_normalize_kernel(const float *__restrict__ x, const float *__restrict__ mean,
                                                           const float *__restrict__ std_inv, const float *__restrict__ gamma,
                                                           const float *__restrict__ beta, float *__restrict__ y, long long total, int C,
                                                           int S) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    if (total < (1LL << 31)) {                  // 32-bit index arithmetic: the 64-bit divisions cost more than the traffic
        for (unsigned e = (unsigned)tid; e < (unsigned)total; e += (unsigned)nthr) {
            const unsigned c = (e / (unsigned)S) % (unsigned)C;
            y[e] = __ldg(gamma + c) * ((__ldg(x + e) - __ldg(mean + c)) * __ldg(std_inv + c)) + __ldg(beta + c);
        }
        return;
    }
    for (long long e = tid; e < total; e += nthr) {
        const int c = (int)((e / S) % C);
        y[e] = __ldg(gamma + c) * ((__ldg(x + e) - __ldg(mean + c)) * __ldg(std_inv + c)) + __ldg(beta + c);
    }
}
// dx = (1/M) * std_inv * (M * dxh - sum dxh - x_hat * sum dxh * x_hat), dxh = dy * gamma; the sums are gamma * dbeta and gamma * dgamma
__global__ void __launch_bounds__(256) bn_dx_kernel(const float *__restrict__ dy, const float *__restrict__ x, const float *__restrict__ mean,
                                                    const float *__restrict__ std_inv, const float *__restrict__ gamma,
                                                    const float *__restrict__ dbeta, const float *__restrict__ dgamma,
                                                    float *__restrict__ dx, long long total, int C, int S, float M,
                                                    const float *__restrict__ M_dev) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    if (M_dev) M = __ldg(M_dev);                    // the count over all ranks' shards
    const float inv_M = 1.0f / M;
    const bool small = total < (1LL << 31);
    for (long long e = tid; e < total; e += nthr) {
        const int c = small ? (int)(((unsigned)e / (unsigned)S) % (unsigned)C) : (int)((e / S) % C);
        const float g = __ldg(gamma + c), si = __ldg(std_inv + c);
        const float xh = (__ldg(x + e) - __ldg(mean + c)) * si;
        const float dxh = __ldg(dy + e) * g;
        dx[e] = inv_M * si * (M * dxh - g * __ldg(dbeta + c) - xh * (g * __ldg(dgamma + c)));
    }
}

// The same two passes for planes of at least 256 floats (a multiple of 4, 16-byte aligned): a block takes whole planes, reads the
// channel's scalars once per plane and moves 128-bit words - no division per element.
__global__ void __launch_bounds__(256) bn_normalize_planes_kernel(const float *__restrict__ x, const float *__restrict__ mean,
                                                                  const float *__restrict__ std_inv, const float *__restrict__ gamma,
                                                                  const float *__restrict__ beta, float *__restrict__ y, long long planes,
                                                                  int C, int S) {
    for (long long p = blockIdx.x; p < planes; p += gridDim.x) {
        const int c = (int)(p % C);
        const float mu = __ldg(mean + c), g = __ldg(gamma + c), si = __ldg(std_inv + c), b = __ldg(beta + c);
        const float4 *x4 = reinterpret_cast<const float4 *>(x + p * S);
        float4 *y4 = reinterpret_cast<float4 *>(y + p * S);
        for (int s = threadIdx.x; s < (S >> 2); s += 256) {
            const float4 v = __ldg(x4 + s);
            y4[s] = make_float4(g * ((v.x - mu) * si) + b, g * ((v.y - mu) * si) + b, g * ((v.z - mu) * si) + b, g * ((v.w - mu) * si) + b);
        }
    }
}
__global__ void __launch_bounds__(256) bn_dx_planes_kernel(const float *__restrict__ dy, const float *__restrict__ x, const float *__restrict__ mean,
                                                           const float *__restrict__ std_inv, const float *__restrict__ gamma,
                                                           const float *__restrict__ dbeta, const float *__restrict__ dgamma,
                                                           float *__restrict__ dx, long long planes, int C, int S, float M,
                                                           const float *__restrict__ M_dev) {
    if (M_dev) M = __ldg(M_dev);
    const float inv_M = 1.0f / M;
    for (long long p = blockIdx.x; p < planes; p += gridDim.x) {
        const int c = (int)(p % C);
        const float g = __ldg(gamma + c), si = __ldg(std_inv + c), mu = __ldg(mean + c);
        const float sb = g * __ldg(dbeta + c), sg = g * __ldg(dgamma + c);
        const float4 *x4 = reinterpret_cast<const float4 *>(x + p * S), *g4 = reinterpret_cast<const float4 *>(dy + p * S);
        float4 *d4 = reinterpret_cast<float4 *>(dx + p * S);
        for (int s = threadIdx.x; s < (S >> 2); s += 256) {
            const float4 v = __ldg(x4 + s), u = __ldg(g4 + s);
            float4 o;
            o.x = inv_M * si * (M * (u.x * g) - sb - ((v.x - mu) * si) * sg);
            o.y = inv_M * si * (M * (u.y * g) - sb - ((v.y - mu) * si) * sg);
            o.z = inv_M * si * (M * (u.z * g) - sb - ((v.z - mu) * si) * sg);
            o.w = inv_M * si * (M * (u.w * g) - sb - ((v.w - mu) * si) * sg);
            d4[s] = o;
        }
    }
}
static bool bn_planes_ok(int S, const void *a, const void *b, const void *c) {
    return S >= 256 && (S & 3) == 0 && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15) == 0;
}

static int bn_splits(int N, int C, int S) {
    long long blocks = S > 1 ? C : (C + 31) / 32;
    long long rows = S > 1 ? N : (N + 7) / 8;
    long long s = ((long long)rt().sm_count * 4 + blocks - 1) / blocks;
    if (s > rows) s = rows;
    if (s > BN_MAX_SPLITS) s = BN_MAX_SPLITS;
    return s < 1 ? 1 : (int)s;
}
static cudaError_t bn_reduce(const float *x, const float *dy, const float *mean, const float *std_inv, float *out0, float *out1, int N, int C,
                             int S, int splits) {
    cudaStream_t st = rt().stream;
    if (S > 1) bn_reduce_planes_kernel<<<dim3(C, splits), 256, 0, st>>>(x, dy, mean, std_inv, out0, out1, N, C, S, splits);
    else bn_reduce_rows_kernel<<<dim3((C + 31) / 32, splits), 256, 0, st>>>(x, dy, mean, std_inv, out0, out1, N, C, splits);
    count_launch();
    return cudaGetLastError();
}

}  // namespace seera

using namespace seera;

extern "C" {

// cross != 0 and a data-parallel communicator of more than one rank: statistics (forward) and the two sums of the dx formula
// (backward) over the shards of all ranks; dgamma / dbeta stay this rank's own sums (the gradient exchange averages them like
// every other parameter gradient).
static int bn_fwd_impl(const float *x, const float *gamma, const float *beta, float *running_mean, float *running_var, float *y,
                       float *mean_out, float *std_inv_out, int N, int C, int S, float momentum, float eps, int training, int cross) {
    SEERA_ENSURE();
    if (N < 1 || C < 1 || S < 1 || C > 65535 || !x || !gamma || !beta || !running_mean || !running_var || !y || !mean_out || !std_inv_out)
        return fail(SEERA_E_ARG, "batchnorm_fwd: bad argument");
    const long long total = (long long)N * C * S;
    const int world = cross ? seera_dp_world() : 1;
    cudaStream_t st = rt().stream;
    cudaError_t e = cudaSuccess;
    float *sums = nullptr, *table = nullptr;      // [splits, C, 3] moments of the split rows; [world, C, 3] moments of the ranks
    int splits = 1, status = SEERA_OK;
    if (training) {
        splits = bn_splits(N, C, S);
        sums = (float *)scratch_alloc((size_t)3 * splits * C * sizeof(float));
        if (!sums) return SEERA_E_OOM;
        if (S > 1) {
            const int vec = (S & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
            bn_stats_planes_kernel<<<dim3(C, splits), 256, 0, st>>>(x, sums, N, C, S, splits, vec);
        } else {
            bn_stats_rows_kernel<<<dim3((C + 31) / 32, splits), 256, 0, st>>>(x, sums, N, C, splits);
        }
        count_launch();
        e = cudaGetLastError();
        if (e == cudaSuccess && world > 1) {
            const size_t tn = (size_t)world * C * 3;
            table = (float *)scratch_alloc(tn * sizeof(float));
            if (!table) { scratch_free(sums); return SEERA_E_OOM; }
            e = cudaMemsetAsync(table, 0, tn * sizeof(float), st);
            if (e == cudaSuccess) {
                bn_merge_local_kernel<<<(C + 255) / 256, 256, 0, st>>>(sums, table + (size_t)seera_dp_rank() * C * 3, C, splits);
                count_launch();
                e = cudaGetLastError();
            }
            if (e == cudaSuccess) status = seera_dp_allreduce(table, (long long)tn, 0);
        }
    }
    if (e == cudaSuccess && status == SEERA_OK) {
        if (table) bn_finalize_fwd_kernel<<<(C + 255) / 256, 256, 0, st>>>(table, running_mean, running_var, mean_out, std_inv_out, C, world,
                                                                           0.f, momentum, eps, training);
        else bn_finalize_fwd_kernel<<<(C + 255) / 256, 256, 0, st>>>(sums, running_mean, running_var, mean_out, std_inv_out, C, splits,
                                                                     (float)((long long)N * S), momentum, eps, training);
        count_launch();
        e = cudaGetLastError();
    }
    if (e == cudaSuccess && status == SEERA_OK) {
        if (bn_planes_ok(S, x, y, x)) {
            const long long planes = (long long)N * C;
            bn_normalize_planes_kernel<<<stride_grid(planes * 256), 256, 0, st>>>(x, mean_out, std_inv_out, gamma, beta, y, planes, C, S);
        } else {
            bn_normalize_kernel<<<stride_grid(total), 256, 0, st>>>(x, mean_out, std_inv_out, gamma, beta, y, total, C, S);
        }
        count_launch();
        e = cudaGetLastError();
    }
    if (sums) scratch_free(sums);
    if (table) scratch_free(table);
    if (status != SEERA_OK) return status;
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, "batchnorm_fwd");
}

static int bn_bwd_impl(const float *dy, const float *x, const float *mean, const float *std_inv, const float *gamma, float *dx,
                       float *dgamma, float *dbeta, int N, int C, int S, int cross) {
    SEERA_ENSURE();
    if (N < 1 || C < 1 || S < 1 || C > 65535 || !dy || !x || !mean || !std_inv || !gamma || !dx || !dgamma || !dbeta)
        return fail(SEERA_E_ARG, "batchnorm_bwd: bad argument");
    const long long total = (long long)N * C * S;
    const int world = cross ? seera_dp_world() : 1;
    const int splits = bn_splits(N, C, S);
    float *p0 = (float *)scratch_alloc((size_t)2 * splits * C * sizeof(float));
    if (!p0) return SEERA_E_OOM;
    float *p1 = p0 + (size_t)splits * C;
    float *all = nullptr;                          // [2C + 1]: the two sums and the element count over every rank's shard
    cudaStream_t st = rt().stream;
    int status = SEERA_OK;
    cudaError_t e = bn_reduce(x, dy, mean, std_inv, p0, p1, N, C, S, splits);
    if (e == cudaSuccess) {
        bn_finalize_bwd_kernel<<<(C + 255) / 256, 256, 0, st>>>(p0, p1, dbeta, dgamma, C, splits);
        count_launch();
        e = cudaGetLastError();
    }
    if (e == cudaSuccess && world > 1) {
        all = (float *)scratch_alloc((size_t)(2 * C + 1) * sizeof(float));
        if (!all) { scratch_free(p0); return SEERA_E_OOM; }
        bn_pack_sums_kernel<<<(C + 255) / 256, 256, 0, st>>>(dbeta, dgamma, all, C, (float)((long long)N * S));
        count_launch();
        e = cudaGetLastError();
        if (e == cudaSuccess) status = seera_dp_allreduce(all, 2 * C + 1, 0);
    }
    if (e == cudaSuccess && status == SEERA_OK) {
        const float *sb = all ? all : dbeta, *sg = all ? all + C : dgamma, *md = all ? all + 2 * C : nullptr;
        const float M = (float)((long long)N * S);
        if (bn_planes_ok(S, x, dy, dx)) {
            const long long planes = (long long)N * C;
            bn_dx_planes_kernel<<<stride_grid(planes * 256), 256, 0, st>>>(dy, x, mean, std_inv, gamma, sb, sg, dx, planes, C, S, M, md);
        } else {
            bn_dx_kernel<<<stride_grid(total), 256, 0, st>>>(dy, x, mean, std_inv, gamma, sb, sg, dx, total, C, S, M, md);
        }
        count_launch();
        e = cudaGetLastError();
    }
    scratch_free(p0);
    if (all) scratch_free(all);
    if (status != SEERA_OK) return status;
    return e == cudaSuccess ? SEERA_OK : check_cuda(e, "batchnorm_bwd");
}

int seera_batchnorm_fwd(const float *x, const float *gamma, const float *beta, float *running_mean, float *running_var, float *y,
                        float *mean_out, float *std_inv_out, int N, int C, int S, float momentum, float eps, int training) {
    return bn_fwd_impl(x, gamma, beta, running_mean, running_var, y, mean_out, std_inv_out, N, C, S, momentum, eps, training, 0);
}
int seera_batchnorm_bwd(const float *dy, const float *x, const float *mean, const float *std_inv, const float *gamma, float *dx,
                        float *dgamma, float *dbeta, int N, int C, int S) {
    return bn_bwd_impl(dy, x, mean, std_inv, gamma, dx, dgamma, dbeta, N, C, S, 0);
}
int seera_batchnorm_fwd_sync(const float *x, const float *gamma, const float *beta, float *running_mean, float *running_var, float *y,
                             float *mean_out, float *std_inv_out, int N, int C, int S, float momentum, float eps, int training) {
    return bn_fwd_impl(x, gamma, beta, running_mean, running_var, y, mean_out, std_inv_out, N, C, S, momentum, eps, training, 1);
}
int seera_batchnorm_bwd_sync(const float *dy, const float *x, const float *mean, const float *std_inv, const float *gamma, float *dx,
                             float *dgamma, float *dbeta, int N, int C, int S) {
    return bn_bwd_impl(dy, x, mean, std_inv, gamma, dx, dgamma, dbeta, N, C, S, 1);
}

}  // extern "C"
