// Fused bandwidth-bound passes of the training step: bias + activation forward, activation gradient +
// bias gradient backward, row softmax and its VJP, softmax/cross-entropy and MSE loss heads, and the
// Adam / SGD-momentum updates.
//
// The reference runs each of these as a chain of separate launches with intermediates in HBM:
//   bias add + activation   broadcast_add_4d then cuda_*_fwd writing out AND grad   (Seera.py:136-137, :255-258)
//   activation backward     cuda_elemmult(local_grad, cp) then cuda_elemadd        (Seera_Engine.py:571-583)
//   bias gradient           broadcast_mul_4d + up to three cuda_sum_fwd            (Seera_Engine.py:43-65)
//   softmax / VJP           one 256-thread block per row                           (engine_cuda/src/activations.cu:87-157)
//   Adam / SGD              ~30 cuten operator launches per parameter tensor       (Seera.py:1038-1063, :992-1001)
// Arithmetic follows the CPU engine, the parity oracle (engine/src/activation_ops.cpp:84-115,
// Seera.py:1069-1084, :1006-1008).
#include "common.cuh"

namespace seera {

__device__ __forceinline__ float act_fwd(float z, int act) {
    switch (act) {
        case SEERA_ACT_RELU: return z > 0.f ? z : 0.f;
        case SEERA_ACT_SIGMOID: return 1.f / (1.f + expf(-z));
        case SEERA_ACT_TANH: return tanhf(z);
        default: return z;
    }
}
// derivative expressed through the output y = act(z)
__device__ __forceinline__ float act_grad_from_out(float y, int act) {
    switch (act) {
        case SEERA_ACT_RELU: return y > 0.f ? 1.f : 0.f;
        case SEERA_ACT_SIGMOID: return y * (1.f - y);
        case SEERA_ACT_TANH: return 1.f - y * y;
        default: return 1.f;
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over a 256-thread block; result valid in thread 0. `sm` holds 8 floats.
__device__ __forceinline__ float block_sum_256(float v, float *sm) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
    if (threadIdx.x < 32) {
        r = threadIdx.x < (blockDim.x >> 5) ? sm[threadIdx.x] : 0.f;
        r = warp_sum(r);
    }
    __syncthreads();
    return r;
}

// ---- y = act(z + bias[channel]) ------------------------------------------------------------------
// mode 0: scalar; mode 1: inner % 4 == 0 (one channel per float4); mode 2: inner == 1 and
// channels % 4 == 0 (four consecutive channels per float4).
__global__ void __launch_bounds__(256) bias_act_kernel(const float *__restrict__ z, const float *__restrict__ bias,
                                                       float *__restrict__ y, long long n, int channels, int inner,
                                                       int act, int mode) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    if (mode == 0) {
        for (long long i = tid; i < n; i += nthr) {
            float b = bias ? __ldg(bias + (i / inner) % channels) : 0.f;
            y[i] = act_fwd(z[i] + b, act);
        }
        return;
    }
    long long n4 = n >> 2;
    const float4 *z4 = reinterpret_cast<const float4 *>(z);
    float4 *y4 = reinterpret_cast<float4 *>(y);
    for (long long i = tid; i < n4; i += nthr) {
        float4 v = z4[i], b;
        if (!bias) b = make_float4(0.f, 0.f, 0.f, 0.f);
        else if (mode == 1) { float s = __ldg(bias + ((i << 2) / inner) % channels); b = make_float4(s, s, s, s); }
        else b = __ldg(reinterpret_cast<const float4 *>(bias) + ((i << 2) % channels >> 2));
        v.x = act_fwd(v.x + b.x, act); v.y = act_fwd(v.y + b.y, act);
        v.z = act_fwd(v.z + b.z, act); v.w = act_fwd(v.w + b.w, act);
        y4[i] = v;
    }
}

// ---- dz = dy * act'(y); per-channel partial sums of dz ----------------------------------------------
// Channel-major case (inner > 1, NCHW): grid (channels, splits); block (c, s) walks samples
// n = s, s + splits, ... and the contiguous `inner` run of channel c in each; writes partial[s*channels + c].
__global__ void __launch_bounds__(256) act_bias_bwd_nchw_kernel(const float *__restrict__ dy, const float *__restrict__ y,
                                                                float *__restrict__ dz, float *__restrict__ partial,
                                                                int outer, int channels, int inner, int act, bool vec) {
    __shared__ float sm[8];
    int c = blockIdx.x, s = blockIdx.y, splits = gridDim.y;
    float acc = 0.f;
    // this block's samples are n = s, s + splits, ...; walk (sample, element) pairs flattened so that all threads
    // stay busy when a channel plane is smaller than the block
    const int cnt = (outer - s + splits - 1) / splits;
    if (vec) {
        const int q = inner >> 2;
        const bool small = (long long)cnt * q < (1ll << 31);       // 32-bit division then
        for (long long j = threadIdx.x; j < (long long)cnt * q; j += blockDim.x) {
            int k = small ? (int)((unsigned)j / (unsigned)q) : (int)(j / q), i = (int)(j - (long long)k * q);
            long long base = ((long long)(s + k * splits) * channels + c) * inner;
            float4 d = reinterpret_cast<const float4 *>(dy + base)[i], yy = reinterpret_cast<const float4 *>(y + base)[i], r;
            r.x = d.x * act_grad_from_out(yy.x, act); r.y = d.y * act_grad_from_out(yy.y, act);
            r.z = d.z * act_grad_from_out(yy.z, act); r.w = d.w * act_grad_from_out(yy.w, act);
            reinterpret_cast<float4 *>(dz + base)[i] = r;
            acc += (r.x + r.y) + (r.z + r.w);
        }
    } else {
        const bool small = (long long)cnt * inner < (1ll << 31);
        for (long long j = threadIdx.x; j < (long long)cnt * inner; j += blockDim.x) {
            int k = small ? (int)((unsigned)j / (unsigned)inner) : (int)(j / inner), i = (int)(j - (long long)k * inner);
            long long at = ((long long)(s + k * splits) * channels + c) * inner + i;
            float r = dy[at] * act_grad_from_out(y[at], act);
            dz[at] = r;
            acc += r;
        }
    }
    float tot = block_sum_256(acc, sm);
    if (threadIdx.x == 0 && partial) partial[(long long)s * channels + c] = tot;
}

// Row-major case (inner == 1, [rows, channels]): block = 32 columns x 8 row lanes; grid (ceil(channels/32), splits).
__global__ void __launch_bounds__(256) act_bias_bwd_rows_kernel(const float *__restrict__ dy, const float *__restrict__ y,
                                                                float *__restrict__ dz, float *__restrict__ partial,
                                                                int rows, int channels, int act) {
    __shared__ float sm[8][33];
    int col = blockIdx.x * 32 + (threadIdx.x & 31), lane_r = threadIdx.x >> 5;
    int s = blockIdx.y, splits = gridDim.y;
    float acc = 0.f;
    if (col < channels) {
        for (int r = s * 8 + lane_r; r < rows; r += splits * 8) {
            long long i = (long long)r * channels + col;
            float v = dy[i] * act_grad_from_out(y[i], act);
            dz[i] = v;
            acc += v;
        }
    }
    sm[lane_r][threadIdx.x & 31] = acc;
    __syncthreads();
    if (lane_r == 0 && col < channels && partial) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; k++) t += sm[k][threadIdx.x];
        partial[(long long)s * channels + col] = t;
    }
}

// out[i][c] = (labels[i] == c): labels outside [0, classes) give an all-zero row
__global__ void __launch_bounds__(256) onehot_kernel(const int *__restrict__ labels, float *__restrict__ out, int total, int classes) {
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        const int i = e / classes, c = e - i * classes;
        out[e] = __ldg(labels + i) == c ? 1.f : 0.f;
    }
}

// ---- row softmax: one warp per row --------------------------------------------------------------------
__global__ void __launch_bounds__(256) softmax_fwd_kernel(const float *__restrict__ x, float *__restrict__ out, int N, int C) {
    int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    int nwarp = gridDim.x * (blockDim.x >> 5);
    for (; row < N; row += nwarp) {
        const float *r = x + (long long)row * C;
        float *o = out + (long long)row * C;
        float mx = -INFINITY;
        for (int c = lane; c < C; c += 32) mx = fmaxf(mx, r[c]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int c = lane; c < C; c += 32) { float e = expf(r[c] - mx); o[c] = e; sum += e; }
        sum = warp_sum(sum);
        float inv = 1.f / sum;
        for (int c = lane; c < C; c += 32) o[c] *= inv;
    }
}

__global__ void __launch_bounds__(256) softmax_vjp_kernel(const float *__restrict__ s, const float *__restrict__ d,
                                                          float *__restrict__ dx, int N, int C) {
    int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    int nwarp = gridDim.x * (blockDim.x >> 5);
    for (; row < N; row += nwarp) {
        const float *sr = s + (long long)row * C, *dr = d + (long long)row * C;
        float dot = 0.f;
        for (int c = lane; c < C; c += 32) dot += dr[c] * sr[c];
        dot = warp_sum(dot);
        for (int c = lane; c < C; c += 32) dx[(long long)row * C + c] = sr[c] * (dr[c] - dot);
    }
}

// softmax -> clip -> log -> -y* -> sum(-1), and the gradient of inv_count * sum_rows w.r.t. z
__global__ void __launch_bounds__(256) softmax_cce_kernel(const float *__restrict__ z, const float *__restrict__ yhot,
                                                          float *__restrict__ p, float *__restrict__ loss_rows,
                                                          float *__restrict__ dz, int N, int C, float eps, float inv_count) {
    int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    int nwarp = gridDim.x * (blockDim.x >> 5);
    float hi = 1.0f - eps;
    for (; row < N; row += nwarp) {
        const float *r = z + (long long)row * C, *yr = yhot + (long long)row * C;
        float *pr = p + (long long)row * C, *dr = dz + (long long)row * C;
        float mx = -INFINITY;
        for (int c = lane; c < C; c += 32) mx = fmaxf(mx, r[c]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int c = lane; c < C; c += 32) { float e = expf(r[c] - mx); pr[c] = e; sum += e; }
        sum = warp_sum(sum);
        float inv = 1.f / sum, loss = 0.f, dot = 0.f;
        for (int c = lane; c < C; c += 32) {
            float pv = pr[c] * inv;
            pr[c] = pv;
            float pc = pv < eps ? eps : (pv > hi ? hi : pv);
            float negy = yr[c] * -1.0f;
            loss += negy * logf(pc);
            float g = (pv >= eps && pv <= hi) ? (1.0f / pc) * (negy * inv_count) : 0.f;   // d loss / d p
            dr[c] = g;
            dot += g * pv;
        }
        loss = warp_sum(loss);
        dot = warp_sum(dot);
        for (int c = lane; c < C; c += 32) dr[c] = pr[c] * (dr[c] - dot);
        if (lane == 0) loss_rows[row] = loss;
    }
}

// Deterministic single-block sum of n floats times scale.
__global__ void __launch_bounds__(1024) scaled_sum_kernel(const float *__restrict__ v, float *__restrict__ out, int n, float scale) {
    __shared__ float sm[32];
    float acc = 0.f;
#pragma unroll 4
    for (int i = threadIdx.x; i < n; i += blockDim.x) acc += v[i];
    float t = block_sum_256(acc, sm);
    if (threadIdx.x == 0) *out = t * scale;
}

// Element-wise losses with their gradient in the same pass.  KIND 0: (p-y)^2 (Seera.py:943-945); 1: |p-y| with the sign
// convention of abs_fwd, 0 at 0 (Seera.py:947-949, engine/src/activation_ops.cpp:50-56); 2: binary cross-entropy
// -y log(p+eps) - (1-y) log(1-p+eps) (Seera.py:951-953).  dp = dloss/dp * inv_count; per-block sums go to `partials`.
template <int KIND>
__global__ void __launch_bounds__(256) elem_loss_kernel(const float *__restrict__ p, const float *__restrict__ y,
                                                        float *__restrict__ partials, float *__restrict__ dp,
                                                        long long n, float inv_count, float eps) {
    __shared__ float sm[8];
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    float acc = 0.f;
    for (long long i = tid; i < n; i += nthr) {
        if (KIND == 0) {
            float d = p[i] + y[i] * -1.0f;
            acc += d * d;
            dp[i] = (2.0f * d) * inv_count;
        } else if (KIND == 1) {
            float d = p[i] + y[i] * -1.0f;
            acc += fabsf(d);
            dp[i] = (d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f)) * inv_count;
        } else {
            const float pv = p[i], yv = y[i], a = pv + eps, b = (1.f - pv) + eps;
            acc += -yv * logf(a) - (1.f - yv) * logf(b);
            dp[i] = (-yv / a + (1.f - yv) / b) * inv_count;
        }
    }
    float t = block_sum_256(acc, sm);
    if (threadIdx.x == 0) partials[blockIdx.x] = t;
}

// ---- optimizers -------------------------------------------------------------------------------------------
struct AdamArgs { float lr, b1, omb1, b2, omb2, eps, c1, c2, gs; };

__device__ __forceinline__ void adam_one(float &w, float g, float &m, float &v, const AdamArgs &a) {
    g *= a.gs;
    m = a.b1 * m + a.omb1 * g;
    v = a.b2 * v + a.omb2 * (g * g);
    float mh = m / a.c1, vh = v / a.c2;
    w -= (a.lr * mh) / (sqrtf(vh) + a.eps);
}

template <class Args>
__device__ __forceinline__ void adam_range(float *__restrict__ w, const float *__restrict__ g, float *__restrict__ m,
                                           float *__restrict__ v, long long n, bool vec, const Args &a) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    if (vec) {                 // 128-bit accesses: 28 bytes per parameter move as 7 vector transactions per 4 parameters
        long long n4 = n >> 2;
        float4 *w4 = reinterpret_cast<float4 *>(w), *m4 = reinterpret_cast<float4 *>(m), *v4 = reinterpret_cast<float4 *>(v);
        const float4 *g4 = reinterpret_cast<const float4 *>(g);
        for (long long i = tid; i < n4; i += nthr) {
            float4 ww = w4[i], gg = g4[i], mm = m4[i], vv = v4[i];
            adam_one(ww.x, gg.x, mm.x, vv.x, a); adam_one(ww.y, gg.y, mm.y, vv.y, a);
            adam_one(ww.z, gg.z, mm.z, vv.z, a); adam_one(ww.w, gg.w, mm.w, vv.w, a);
            w4[i] = ww; m4[i] = mm; v4[i] = vv;
        }
        for (long long i = (n4 << 2) + tid; i < n; i += nthr) adam_one(w[i], g[i], m[i], v[i], a);
    } else {
        for (long long i = tid; i < n; i += nthr) adam_one(w[i], g[i], m[i], v[i], a);
    }
}
__device__ __forceinline__ void sgd_range(float *__restrict__ w, const float *__restrict__ g, float *__restrict__ vel, long long n,
                                          bool vec, float lr, float mu, float gs) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    if (vec) {
        long long n4 = n >> 2;
        float4 *w4 = reinterpret_cast<float4 *>(w), *v4 = reinterpret_cast<float4 *>(vel);
        const float4 *g4 = reinterpret_cast<const float4 *>(g);
        for (long long i = tid; i < n4; i += nthr) {
            float4 ww = w4[i], gg = g4[i], vv = v4[i];
            vv.x = mu * vv.x + lr * (gg.x * gs); vv.y = mu * vv.y + lr * (gg.y * gs);
            vv.z = mu * vv.z + lr * (gg.z * gs); vv.w = mu * vv.w + lr * (gg.w * gs);
            ww.x -= vv.x; ww.y -= vv.y; ww.z -= vv.z; ww.w -= vv.w;
            w4[i] = ww; v4[i] = vv;
        }
        for (long long i = (n4 << 2) + tid; i < n; i += nthr) { vel[i] = mu * vel[i] + lr * (g[i] * gs); w[i] -= vel[i]; }
    } else {
        for (long long i = tid; i < n; i += nthr) { vel[i] = mu * vel[i] + lr * (g[i] * gs); w[i] -= vel[i]; }
    }
}

__global__ void __launch_bounds__(256) adam_kernel(float *__restrict__ w, const float *__restrict__ g, float *__restrict__ m,
                                                   float *__restrict__ v, long long n, bool vec, AdamArgs a) {
    adam_range(w, g, m, v, n, vec, a);
}
// The same update with its scalars read from device memory, so that a captured step graph can be replayed with a new
// step count (the host refreshes the nine floats before each replay).
__global__ void __launch_bounds__(256) adam_dev_kernel(float *__restrict__ w, const float *__restrict__ g, float *__restrict__ m,
                                                       float *__restrict__ v, long long n, bool vec, const float *__restrict__ h) {
    AdamArgs a{h[0], h[1], h[2], h[3], h[4], h[5], h[6], h[7], h[8]};
    adam_range(w, g, m, v, n, vec, a);
}
__global__ void __launch_bounds__(256) sgd_dev_kernel(float *__restrict__ w, const float *__restrict__ g, float *__restrict__ vel,
                                                      long long n, bool vec, const float *__restrict__ h) {
    sgd_range(w, g, vel, n, vec, h[0], h[1], h[2]);
}
__global__ void __launch_bounds__(256) sgd_kernel(float *__restrict__ w, const float *__restrict__ g, float *__restrict__ vel,
                                                  long long n, bool vec, float lr, float mu, float gs) {
    sgd_range(w, g, vel, n, vec, lr, mu, gs);
}

// ---- dynamic factor of the fp16 gradient copies -------------------------------------------------------------------
__global__ void grad_scale_reset_kernel(float *w) {
    if (threadIdx.x == 0) { w[0] = 1.f; w[1] = 1.f; reinterpret_cast<unsigned *>(w)[2] = 0u; w[3] = 0.f; }
}
__global__ void __launch_bounds__(256) grad_amax_kernel(const float *__restrict__ g, long long n, unsigned *__restrict__ amax_bits) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    float m = 0.f;
    for (long long i = tid; i < n; i += nthr) {
        const float a = fabsf(g[i]);
        if (a < 3.0e38f) m = fmaxf(m, a);              // infinities and NaNs do not steer the scale
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(amax_bits, __float_as_uint(m));
}
// factor = 2^(-4 - e) with amax = m * 2^e, m in [0.5, 1): together with the static 2^12 of the gradient class the largest
// entry of the loss gradient lands in [128, 256) - eight binades of headroom below fp16's maximum for gradients that grow
// on the way down the network, twenty-one binades of normal range below it for those that shrink.
__global__ void grad_scale_finalize_kernel(float *w) {
    if (threadIdx.x != 0) return;
    unsigned *bits = reinterpret_cast<unsigned *>(w) + 2;
    const float amax = __uint_as_float(*bits);
    *bits = 0u;
    int e = 0;
    if (amax > 0.f) frexpf(amax, &e);
    e = max(-100, min(30, e));
    w[0] = amax > 0.f ? ldexpf(1.f, -4 - e) : 1.f;
    w[1] = amax > 0.f ? ldexpf(1.f, 4 + e) : 1.f;
}

float *grad_scale_words() {
    static float *w = nullptr;
    if (!w) {
        if (cudaMalloc(&w, 4 * sizeof(float)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        grad_scale_reset_kernel<<<1, 32, 0, rt().stream>>>(w);
        count_launch();
    }
    return w;
}

}  // namespace seera

using namespace seera;

extern "C" {

int seera_bias_act_fwd(const float *z, const float *bias, float *y, int size, int channels, int inner, int act) {
    SEERA_ENSURE();
    if (size < 0 || channels < 1 || inner < 1 || (size > 0 && (!z || !y))) return fail(SEERA_E_ARG, "bias_act_fwd: bad argument");
    if (size == 0) return SEERA_OK;
    int mode = 0;
    if (aligned16(z) && aligned16(y) && size % 4 == 0) {
        if (inner % 4 == 0) mode = 1;
        else if (inner == 1 && channels % 4 == 0 && (!bias || aligned16(bias))) mode = 2;
    }
    ProfBytes pb(8.0 * size, "bias_act_fwd");
    bias_act_kernel<<<stride_grid(mode ? size / 4 : size), 256, 0, rt().stream>>>(z, bias, y, size, channels, inner, act, mode);
    SEERA_LAUNCH_CHECK("bias_act_fwd");
    return SEERA_OK;
}

// Split count of the activation-backward pass: enough blocks for ~4 waves, never more than the rows available.
static int act_bias_splits(int outer, int channels, int inner) {
    int splits;
    if (inner == 1) {
        int colblocks = (channels + 31) / 32;
        splits = (rt().sm_count * 4 + colblocks - 1) / colblocks;
        int maxs = (outer + 7) / 8;
        if (splits > maxs) splits = maxs;
    } else {
        splits = (rt().sm_count * 4 + channels - 1) / channels;
        if (splits > outer) splits = outer;
        if (splits > 65535) splits = 65535;
    }
    return splits < 1 ? 1 : splits;
}

// Launches dz = dy * act'(y) and, when dbias is wanted, the two-stage per-channel sum through `partial`
// (splits * channels floats of scratch owned by the caller of this helper).
static int act_bias_bwd_launch(const float *dy, const float *y, float *dz, float *dbias, float *partial, int outer, int channels,
                               int inner, int act, int splits) {
    // dy and (with an activation) y read, dz written unless it is dy itself
    ProfBytes pb(4.0 * outer * channels * inner * (1 + (act ? 1 : 0) + (dz != dy ? 1 : 0)), "act_bias_bwd");
    if (inner == 1) {
        int colblocks = (channels + 31) / 32;
        act_bias_bwd_rows_kernel<<<dim3(colblocks, splits), 256, 0, rt().stream>>>(dy, y, dz, partial, outer, channels, act);
        SEERA_LAUNCH_CHECK("act_bias_bwd(rows)");
    } else {
        bool vec = (inner % 4 == 0) && aligned16(dy) && aligned16(y) && aligned16(dz);
        act_bias_bwd_nchw_kernel<<<dim3(channels, splits), 256, 0, rt().stream>>>(dy, y, dz, partial, outer, channels, inner, act, vec);
        SEERA_LAUNCH_CHECK("act_bias_bwd(nchw)");
    }
    if (dbias) {
        launch_sum_splits(partial, dbias, channels, splits, rt().stream);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return check_cuda(e, "act_bias_bwd(sum)");
    }
    return SEERA_OK;
}

static int act_bias_bwd_check(const float *dy, const float *y, float *dz, int size, int channels, int inner, int act, const char *name) {
    const long long per_outer = (long long)channels * inner;      // in 64 bits: channels * inner may not fit an int
    if (size < 0 || channels < 1 || inner < 1 || (size > 0 && (!dy || !dz)) || (act != SEERA_ACT_NONE && !y) ||
        per_outer > 0x7fffffffLL || (long long)size % per_outer != 0)
        return fail(SEERA_E_ARG, "%s: bad argument", name);
    return SEERA_OK;
}

int seera_act_bias_bwd(const float *dy, const float *y, float *dz, float *dbias, int size, int channels, int inner, int act) {
    SEERA_ENSURE();
    if (int s = act_bias_bwd_check(dy, y, dz, size, channels, inner, act, "act_bias_bwd")) return s;
    if (size == 0) return SEERA_OK;
    if (!y) y = dy;   // act == NONE never reads it
    int outer = size / (channels * inner);
    int splits = act_bias_splits(outer, channels, inner);
    float *partial = nullptr;
    if (dbias) { partial = (float *)scratch_alloc((size_t)splits * channels * sizeof(float)); if (!partial) return SEERA_E_OOM; }
    int s = act_bias_bwd_launch(dy, y, dz, dbias, partial, outer, channels, inner, act, splits);
    if (partial) scratch_free(partial);
    return s;
}

// ---- activation backward without any allocation -------------------------------------------------------------
// Scratch for the per-channel partial sums lives in this fixed device array instead of the pool.  It is part of
// the library image: every GPU that loads the library carries these 256 KiB until the process exits.
#define SEERA_STATIC_PARTIALS 65536
static __device__ __align__(256) float g_act_bias_partials[SEERA_STATIC_PARTIALS];

// In host code the array's name is only a handle for the runtime, not a device address; the address a kernel can
// use has to be asked for, once per device, while that device is current.
static float *static_partials_for_current_device(int *status) {
    static float *per_device[64] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { *status = fail(SEERA_E_CUDA, "act_bias_bwd_noalloc: cannot identify the current device"); return nullptr; }
    if (!per_device[dev]) {
        float *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&p, g_act_bias_partials);
        if (e != cudaSuccess || !p) { *status = check_cuda(e == cudaSuccess ? cudaErrorInvalidSymbol : e, "cudaGetSymbolAddress(act_bias partials)"); return nullptr; }
        per_device[dev] = p;
    }
    return per_device[dev];
}

int seera_act_bias_bwd_noalloc(const float *dy, const float *y, float *dz, float *dbias, int size, int channels, int inner, int act) {
    SEERA_ENSURE();
    if (int s = act_bias_bwd_check(dy, y, dz, size, channels, inner, act, "act_bias_bwd_noalloc")) return s;
    if (size == 0) return SEERA_OK;
    if (!y) y = dy;
    int outer = size / (channels * inner);
    if (channels > SEERA_STATIC_PARTIALS)
        return fail(SEERA_E_LIMIT, "act_bias_bwd_noalloc: %d channels exceed the fixed scratch of %d partial sums", channels, SEERA_STATIC_PARTIALS);
    int splits = act_bias_splits(outer, channels, inner);
    if ((long long)splits * channels > SEERA_STATIC_PARTIALS) splits = SEERA_STATIC_PARTIALS / channels;   // (not reached with 148 SMs)
    int st = SEERA_OK;
    float *partial = dbias ? static_partials_for_current_device(&st) : nullptr;
    if (dbias && !partial) return st;
    // every partial that is read is written first by this call, so nothing needs clearing
    return act_bias_bwd_launch(dy, y, dz, dbias, partial, outer, channels, inner, act, splits);
}

int seera_cuda_softmax_fwd(const float *x, float *out, int N, int C) {
    SEERA_ENSURE();
    if (N < 0 || C < 1 || (N > 0 && (!x || !out))) return fail(SEERA_E_ARG, "cuda_softmax_fwd: bad argument");
    if (N == 0) return SEERA_OK;
    softmax_fwd_kernel<<<stride_grid((long long)N * 32), 256, 0, rt().stream>>>(x, out, N, C);
    SEERA_LAUNCH_CHECK("cuda_softmax_fwd");
    return SEERA_OK;
}

int seera_cuda_softmax_vjp(const float *s, const float *dout, float *dx, int N, int C) {
    SEERA_ENSURE();
    if (N < 0 || C < 1 || (N > 0 && (!s || !dout || !dx))) return fail(SEERA_E_ARG, "cuda_softmax_vjp: bad argument");
    if (N == 0) return SEERA_OK;
    softmax_vjp_kernel<<<stride_grid((long long)N * 32), 256, 0, rt().stream>>>(s, dout, dx, N, C);
    SEERA_LAUNCH_CHECK("cuda_softmax_vjp");
    return SEERA_OK;
}

int seera_onehot_f32(const int *labels, float *out, int n, int classes) {
    SEERA_ENSURE();
    if (n < 0 || classes < 1 || (n > 0 && (!labels || !out)) || (long long)n * classes > 0x7fffffffLL)
        return fail(SEERA_E_ARG, "onehot_f32: bad argument");
    if (n == 0) return SEERA_OK;
    onehot_kernel<<<stride_grid((long long)n * classes), 256, 0, rt().stream>>>(labels, out, n * classes, classes);
    SEERA_LAUNCH_CHECK("onehot_f32");
    return SEERA_OK;
}

int seera_softmax_cce_fwd_bwd(const float *z, const float *onehot, float *p, float *loss_rows, float *loss_mean,
                              float *dz, int N, int C, float eps, float inv_count) {
    SEERA_ENSURE();
    if (N < 1 || C < 1 || !z || !onehot || !p || !loss_rows || !loss_mean || !dz)
        return fail(SEERA_E_ARG, "softmax_cce_fwd_bwd: bad argument");
    ProfBytes pb(16.0 * N * C, "softmax_cce");
    softmax_cce_kernel<<<stride_grid((long long)N * 32), 256, 0, rt().stream>>>(z, onehot, p, loss_rows, dz, N, C, eps, inv_count);
    SEERA_LAUNCH_CHECK("softmax_cce");
    scaled_sum_kernel<<<1, N > 1024 ? 1024 : 256, 0, rt().stream>>>(loss_rows, loss_mean, N, inv_count);
    SEERA_LAUNCH_CHECK("softmax_cce(sum)");
    return SEERA_OK;
}

int seera_mse_partials(int size) {
    int g = size > 0 ? stride_grid(size) : 1;
    return g;
}

static int elem_loss(int kind, const float *p, const float *y, float *partials, float *loss_mean, float *dp, int size,
                     float inv_count, float eps, const char *name) {
    SEERA_ENSURE();
    if (size < 1 || !p || !y || !partials || !loss_mean || !dp) return fail(SEERA_E_ARG, "%s: bad argument", name);
    int g = stride_grid(size);
    cudaStream_t st = rt().stream;
    ProfBytes pb(12.0 * size, name);
    if (kind == 0) elem_loss_kernel<0><<<g, 256, 0, st>>>(p, y, partials, dp, size, inv_count, eps);
    else if (kind == 1) elem_loss_kernel<1><<<g, 256, 0, st>>>(p, y, partials, dp, size, inv_count, eps);
    else elem_loss_kernel<2><<<g, 256, 0, st>>>(p, y, partials, dp, size, inv_count, eps);
    SEERA_LAUNCH_CHECK(name);
    scaled_sum_kernel<<<1, g > 1024 ? 1024 : 256, 0, st>>>(partials, loss_mean, g, inv_count);
    SEERA_LAUNCH_CHECK(name);
    return SEERA_OK;
}
int seera_mse_fwd_bwd(const float *p, const float *y, float *partials, float *loss_mean, float *dp, int size, float inv_count) {
    return elem_loss(0, p, y, partials, loss_mean, dp, size, inv_count, 0.f, "mse_fwd_bwd");
}
int seera_mae_fwd_bwd(const float *p, const float *y, float *partials, float *loss_mean, float *dp, int size, float inv_count) {
    return elem_loss(1, p, y, partials, loss_mean, dp, size, inv_count, 0.f, "mae_fwd_bwd");
}
int seera_bce_fwd_bwd(const float *p, const float *y, float *partials, float *loss_mean, float *dp, int size, float inv_count,
                      float eps) {
    return elem_loss(2, p, y, partials, loss_mean, dp, size, inv_count, eps, "bce_fwd_bwd");
}

// ---- dynamic factor of the fp16 gradient copies (precision modes 4 and 5) -------------------------------------------
// words[0] = factor, words[1] = 1 / factor, words[2] = bits of the running maximum |g| (as an unsigned: positive floats
// order like their bit patterns).
int seera_grad_scale_update(const float *g, long long n) {
    SEERA_ENSURE();
    if (n < 0 || (n > 0 && !g)) return fail(SEERA_E_ARG, "grad_scale_update: bad argument");
    float *w = grad_scale_words();
    if (!w) return fail(SEERA_E_OOM, "grad_scale_update: no device memory for the scale words");
    if (n == 0) return SEERA_OK;
    grad_amax_kernel<<<stride_grid(n), 256, 0, rt().stream>>>(g, n, reinterpret_cast<unsigned *>(w) + 2);
    SEERA_LAUNCH_CHECK("grad_scale_update(amax)");
    grad_scale_finalize_kernel<<<1, 32, 0, rt().stream>>>(w);
    SEERA_LAUNCH_CHECK("grad_scale_update");
    return SEERA_OK;
}

int seera_adam_step(float *w, const float *g, float *m, float *v, int n, float lr, float beta1, float omb1,
                    float beta2, float omb2, float eps, float c1, float c2, float grad_scale) {
    SEERA_ENSURE();
    if (n < 0 || (n > 0 && (!w || !g || !m || !v))) return fail(SEERA_E_ARG, "adam_step: bad argument");
    if (n == 0) return SEERA_OK;
    bool vec = aligned16(w) && aligned16(g) && aligned16(m) && aligned16(v);
    AdamArgs a{lr, beta1, omb1, beta2, omb2, eps, c1, c2, grad_scale};
    ProfBytes pb(28.0 * n, "adam");
    adam_kernel<<<stride_grid(vec ? (n + 3) / 4 : n), 256, 0, rt().stream>>>(w, g, m, v, n, vec, a);
    SEERA_LAUNCH_CHECK("adam_step");
    return SEERA_OK;
}

int seera_adam_step_dev(float *w, const float *g, float *m, float *v, int n, const float *hyper) {
    SEERA_ENSURE();
    if (n < 0 || (n > 0 && (!w || !g || !m || !v || !hyper))) return fail(SEERA_E_ARG, "adam_step_dev: bad argument");
    if (n == 0) return SEERA_OK;
    bool vec = aligned16(w) && aligned16(g) && aligned16(m) && aligned16(v);
    ProfBytes pb(28.0 * n, "adam");
    adam_dev_kernel<<<stride_grid(vec ? (n + 3) / 4 : n), 256, 0, rt().stream>>>(w, g, m, v, n, vec, hyper);
    SEERA_LAUNCH_CHECK("adam_step_dev");
    return SEERA_OK;
}
int seera_sgd_step_dev(float *w, const float *g, float *vel, int n, const float *hyper) {
    SEERA_ENSURE();
    if (n < 0 || (n > 0 && (!w || !g || !vel || !hyper))) return fail(SEERA_E_ARG, "sgd_step_dev: bad argument");
    if (n == 0) return SEERA_OK;
    bool vec = aligned16(w) && aligned16(g) && aligned16(vel);
    ProfBytes pb(20.0 * n, "sgd");
    sgd_dev_kernel<<<stride_grid(vec ? (n + 3) / 4 : n), 256, 0, rt().stream>>>(w, g, vel, n, vec, hyper);
    SEERA_LAUNCH_CHECK("sgd_step_dev");
    return SEERA_OK;
}

int seera_sgd_step(float *w, const float *g, float *vel, int n, float lr, float momentum, float grad_scale) {
    SEERA_ENSURE();
    if (n < 0 || (n > 0 && (!w || !g || !vel))) return fail(SEERA_E_ARG, "sgd_step: bad argument");
    if (n == 0) return SEERA_OK;
    bool vec = aligned16(w) && aligned16(g) && aligned16(vel);
    ProfBytes pb(20.0 * n, "sgd");
    sgd_kernel<<<stride_grid(vec ? (n + 3) / 4 : n), 256, 0, rt().stream>>>(w, g, vel, n, vec, lr, momentum, grad_scale);
    SEERA_LAUNCH_CHECK("sgd_step");
    return SEERA_OK;
}

}  // extern "C"
