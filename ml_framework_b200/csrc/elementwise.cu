// Bandwidth-bound element-wise kernels: unary ops with local gradients, flat binary ops,
// in-place scalar ops, fills and the 4-D broadcast add/mul.
//
// Replaces engine_cuda/src/activations.cu:9-83, elemops.cu:14-40, cuTen_essentails.cu:8-78 and
// broadcast.cu:12-65 (one element per thread, blocking after every launch).  Here every kernel is a
// grid-stride loop over 128-bit vectors (scalar tail and an unaligned-pointer path kept because the
// caller may do byte arithmetic on device addresses), sized to whole waves of the device.
// Arithmetic follows the reference CPU engine (engine/src/activation_ops.cpp:7-81), which is the
// parity oracle: strict x > 0 for ReLU, closed interval for the clip gradient, 0.5/(s+1e-12) for sqrt.
#include "common.cuh"

namespace seera {

// ---- op functors: value and local gradient --------------------------------------------------
struct OpRelu    { __device__ void operator()(float x, float &o, float &g) const { o = x > 0.f ? x : 0.f; g = x > 0.f ? 1.f : 0.f; } };
struct OpSigmoid { __device__ void operator()(float x, float &o, float &g) const { float s = 1.f / (1.f + expf(-x)); o = s; g = s * (1.f - s); } };
struct OpTanh    { __device__ void operator()(float x, float &o, float &g) const { float t = tanhf(x); o = t; g = 1.f - t * t; } };
struct OpLog     { __device__ void operator()(float x, float &o, float &g) const { o = logf(x); g = 1.f / x; } };
struct OpExp     { __device__ void operator()(float x, float &o, float &g) const { float e = expf(x); o = e; g = e; } };
struct OpAbs     { __device__ void operator()(float x, float &o, float &g) const { o = fabsf(x); g = x > 0.f ? 1.f : (x < 0.f ? -1.f : 0.f); } };
struct OpSqrt    { __device__ void operator()(float x, float &o, float &g) const { float s = sqrtf(x); o = s; g = 0.5f / (s + 1e-12f); } };
struct OpPow     { float e; __device__ void operator()(float x, float &o, float &g) const { o = powf(x, e); g = e * powf(x, e - 1.f); } };
struct OpClip    { float lo, hi; __device__ void operator()(float x, float &o, float &g) const { o = x < lo ? lo : (x > hi ? hi : x); g = (x >= lo && x <= hi) ? 1.f : 0.f; } };

template <class Op>
__global__ void __launch_bounds__(256) unary_kernel(const float *__restrict__ x, float *__restrict__ out,
                                                    float *__restrict__ grad, long long n, bool vec, Op op) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    if (vec) {
        long long n4 = n >> 2;
        const float4 *x4 = reinterpret_cast<const float4 *>(x);
        float4 *o4 = reinterpret_cast<float4 *>(out), *g4 = reinterpret_cast<float4 *>(grad);
        for (long long i = tid; i < n4; i += nthr) {
            float4 v = __ldg(x4 + i), o, g;
            op(v.x, o.x, g.x); op(v.y, o.y, g.y); op(v.z, o.z, g.z); op(v.w, o.w, g.w);
            o4[i] = o; g4[i] = g;
        }
        for (long long i = (n4 << 2) + tid; i < n; i += nthr) op(x[i], out[i], grad[i]);
    } else {
        for (long long i = tid; i < n; i += nthr) op(x[i], out[i], grad[i]);
    }
}

template <class Op>
int launch_unary(const float *x, float *out, float *grad, int size, Op op, const char *name) {
    SEERA_ENSURE();
    if (size < 0 || (size > 0 && (!x || !out || !grad))) return fail(SEERA_E_ARG, "%s: bad argument", name);
    if (size == 0) return SEERA_OK;
    bool vec = aligned16(x) && aligned16(out) && aligned16(grad);
    unary_kernel<Op><<<stride_grid(vec ? (size + 3) / 4 : size), 256, 0, rt().stream>>>(x, out, grad, size, vec, op);
    SEERA_LAUNCH_CHECK(name);
    return SEERA_OK;
}

// ---- flat binary ---------------------------------------------------------------------------
struct BAdd { __device__ float operator()(float a, float b) const { return a + b; } };
struct BSub { __device__ float operator()(float a, float b) const { return a - b; } };
struct BMul { __device__ float operator()(float a, float b) const { return a * b; } };
struct BDiv { __device__ float operator()(float a, float b) const { return a / b; } };

template <class Op>
__global__ void __launch_bounds__(256) binary_kernel(const float *__restrict__ a, const float *__restrict__ b,
                                                     float *__restrict__ c, long long n, bool vec, Op op) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    if (vec) {
        long long n4 = n >> 2;
        const float4 *a4 = reinterpret_cast<const float4 *>(a), *b4 = reinterpret_cast<const float4 *>(b);
        float4 *c4 = reinterpret_cast<float4 *>(c);
        for (long long i = tid; i < n4; i += nthr) {
            float4 u = a4[i], v = b4[i], r;
            r.x = op(u.x, v.x); r.y = op(u.y, v.y); r.z = op(u.z, v.z); r.w = op(u.w, v.w);
            c4[i] = r;
        }
        for (long long i = (n4 << 2) + tid; i < n; i += nthr) c[i] = op(a[i], b[i]);
    } else {
        for (long long i = tid; i < n; i += nthr) c[i] = op(a[i], b[i]);
    }
}

template <class Op>
int launch_binary(const float *a, const float *b, float *c, int size, Op op, const char *name) {
    SEERA_ENSURE();
    if (size < 0 || (size > 0 && (!a || !b || !c))) return fail(SEERA_E_ARG, "%s: bad argument", name);
    if (size == 0) return SEERA_OK;
    bool vec = aligned16(a) && aligned16(b) && aligned16(c);
    binary_kernel<Op><<<stride_grid(vec ? (size + 3) / 4 : size), 256, 0, rt().stream>>>(a, b, c, size, vec, op);
    SEERA_LAUNCH_CHECK(name);
    return SEERA_OK;
}

// ---- in-place scalar ops and fills ------------------------------------------------------------
struct SMul  { float k; __device__ float operator()(float a) const { return a * k; } };
struct SAdd  { float k; __device__ float operator()(float a) const { return a + k; } };
struct SPow  { float k; __device__ float operator()(float a) const { return powf(a, k); } };
struct SFill { float k; __device__ float operator()(float) const { return k; } };

template <class Op, bool READ>
__global__ void __launch_bounds__(256) inplace_kernel(float *__restrict__ a, long long n, bool vec, Op op) {
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    if (vec) {
        long long n4 = n >> 2;
        float4 *a4 = reinterpret_cast<float4 *>(a);
        for (long long i = tid; i < n4; i += nthr) {
            float4 u = READ ? a4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            u.x = op(u.x); u.y = op(u.y); u.z = op(u.z); u.w = op(u.w);
            a4[i] = u;
        }
        for (long long i = (n4 << 2) + tid; i < n; i += nthr) a[i] = op(READ ? a[i] : 0.f);
    } else {
        for (long long i = tid; i < n; i += nthr) a[i] = op(READ ? a[i] : 0.f);
    }
}

template <class Op, bool READ>
int launch_inplace(float *a, int size, Op op, const char *name) {
    SEERA_ENSURE();
    if (size < 0 || (size > 0 && !a)) return fail(SEERA_E_ARG, "%s: bad argument", name);
    if (size == 0) return SEERA_OK;
    bool vec = aligned16(a);
    inplace_kernel<Op, READ><<<stride_grid(vec ? (size + 3) / 4 : size), 256, 0, rt().stream>>>(a, size, vec, op);
    SEERA_LAUNCH_CHECK(name);
    return SEERA_OK;
}

// ---- NumPy-rule broadcast of two 4-D shapes ------------------------------------------------------
// Output dims are the element-wise maximum; an operand dim of 1 gets stride 0.  Each thread walks
// the innermost output axis in order, so the div/mod runs once per row segment.
template <class Op>
__global__ void __launch_bounds__(256) broadcast_kernel(const float *__restrict__ A, const float *__restrict__ B,
                                                        float *__restrict__ C, int oN, int oC, int oH, int oW,
                                                        int4 sa, int4 sb, Op op) {
    long long total = (long long)oN * oC * oH * oW;
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long i = tid; i < total; i += nthr) {
        int w = (int)(i % oW); long long t = i / oW;
        int h = (int)(t % oH); t /= oH;
        int c = (int)(t % oC); int n = (int)(t / oC);
        long long ia = (long long)n * sa.x + (long long)c * sa.y + (long long)h * sa.z + (long long)w * sa.w;
        long long ib = (long long)n * sb.x + (long long)c * sb.y + (long long)h * sb.z + (long long)w * sb.w;
        C[i] = op(A[ia], B[ib]);
    }
}

template <class Op>
int launch_broadcast(const float *A, const float *B, float *C, const int a[4], const int b[4], Op op, const char *name) {
    SEERA_ENSURE();
    int o[4];
    for (int i = 0; i < 4; i++) {
        if (a[i] < 1 || b[i] < 1 || (a[i] != b[i] && a[i] != 1 && b[i] != 1))
            return fail(SEERA_E_ARG, "%s: shapes (%d,%d,%d,%d) and (%d,%d,%d,%d) do not broadcast", name,
                        a[0], a[1], a[2], a[3], b[0], b[1], b[2], b[3]);
        o[i] = a[i] > b[i] ? a[i] : b[i];
    }
    if (!A || !B || !C) return fail(SEERA_E_ARG, "%s: null pointer", name);
    auto strides = [](const int d[4]) {
        int4 s;
        s.w = d[3] == 1 ? 0 : 1;
        s.z = d[2] == 1 ? 0 : d[3];
        s.y = d[1] == 1 ? 0 : d[2] * d[3];
        s.x = d[0] == 1 ? 0 : d[1] * d[2] * d[3];
        return s;
    };
    long long total = (long long)o[0] * o[1] * o[2] * o[3];
    broadcast_kernel<Op><<<stride_grid(total), 256, 0, rt().stream>>>(A, B, C, o[0], o[1], o[2], o[3], strides(a), strides(b), op);
    SEERA_LAUNCH_CHECK(name);
    return SEERA_OK;
}

}  // namespace seera

using namespace seera;

// element e of the joined [N, n1 + n2] matrix lives in part a (column < n1) or part b; JOIN copies parts -> joined, else joined -> parts
template <bool JOIN, class V>
__global__ void __launch_bounds__(256) concat_kernel(const float *a_, const float *b_, float *joined_, long long total, int n1, int n2) {
    V *a = reinterpret_cast<V *>(const_cast<float *>(a_)), *b = reinterpret_cast<V *>(const_cast<float *>(b_));
    V *joined = reinterpret_cast<V *>(joined_);
    const int n = n1 + n2;
    long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    for (long long e = tid; e < total; e += nthr) {
        const long long row = e / n;
        const int col = (int)(e - row * n);
        V *part = col < n1 ? a + row * n1 + col : b + row * n2 + (col - n1);
        if (JOIN) joined[e] = *part;
        else *part = joined[e];
    }
}

extern "C" {
int seera_cuda_relu_fwd(const float *x, float *o, float *g, int n)    { return launch_unary(x, o, g, n, OpRelu{}, "cuda_relu_fwd"); }
int seera_cuda_sigmoid_fwd(const float *x, float *o, float *g, int n) { return launch_unary(x, o, g, n, OpSigmoid{}, "cuda_sigmoid_fwd"); }
int seera_cuda_tanh_fwd(const float *x, float *o, float *g, int n)    { return launch_unary(x, o, g, n, OpTanh{}, "cuda_tanh_fwd"); }
int seera_cuda_log_fwd(const float *x, float *o, float *g, int n)     { return launch_unary(x, o, g, n, OpLog{}, "cuda_log_fwd"); }
int seera_cuda_exp_fwd(const float *x, float *o, float *g, int n)     { return launch_unary(x, o, g, n, OpExp{}, "cuda_exp_fwd"); }
int seera_cuda_abs_fwd(const float *x, float *o, float *g, int n)     { return launch_unary(x, o, g, n, OpAbs{}, "cuda_abs_fwd"); }
int seera_cuda_sqrt_fwd(const float *x, float *o, float *g, int n)    { return launch_unary(x, o, g, n, OpSqrt{}, "cuda_sqrt_fwd"); }
int seera_cuda_pow_fwd(const float *x, float e, float *o, float *g, int n) { return launch_unary(x, o, g, n, OpPow{e}, "cuda_pow_fwd"); }
int seera_cuda_clip_fwd(const float *x, float lo, float hi, float *o, float *g, int n) { return launch_unary(x, o, g, n, OpClip{lo, hi}, "cuda_clip_fwd"); }

int seera_cuda_elemadd_gputogpu(const float *A, const float *B, float *C, int n)  { return launch_binary(A, B, C, n, BAdd{}, "cuda_elemadd"); }
int seera_cuda_elemsub_gputogpu(const float *A, const float *B, float *C, int n)  { return launch_binary(A, B, C, n, BSub{}, "cuda_elemsub"); }
int seera_cuda_elemmult_gputogpu(const float *A, const float *B, float *C, int n) { return launch_binary(A, B, C, n, BMul{}, "cuda_elemmult"); }
int seera_cuda_elemdiv_gputogpu(const float *A, const float *B, float *C, int n)  { return launch_binary(A, B, C, n, BDiv{}, "cuda_elemdiv"); }

int seera_cuda_scaler_multiply_f(float *a, float k, int n) { return launch_inplace<SMul, true>(a, n, SMul{k}, "cuda_scaler_multiply_f"); }
int seera_cuda_scaler_add_f(float *a, float k, int n)      { return launch_inplace<SAdd, true>(a, n, SAdd{k}, "cuda_scaler_add_f"); }
int seera_cuda_scaler_power_f(float *a, float k, int n)    { return launch_inplace<SPow, true>(a, n, SPow{k}, "cuda_scaler_power_f"); }
int seera_cuda_ones_f(float *a, int n)                     { return launch_inplace<SFill, false>(a, n, SFill{1.f}, "cuda_ones_f"); }
int seera_cuda_zeros_f(float *a, int n)                    { return launch_inplace<SFill, false>(a, n, SFill{0.f}, "cuda_zeros_f"); }

int seera_broadcast_add_4d(const float *A, const float *B, float *C, int aN, int aC, int aH, int aW, int bN, int bC, int bH, int bW) {
    int a[4] = {aN, aC, aH, aW}, b[4] = {bN, bC, bH, bW};
    return launch_broadcast(A, B, C, a, b, BAdd{}, "broadcast_add_4d");
}
int seera_broadcast_mul_4d(const float *A, const float *B, float *C, int aN, int aC, int aH, int aW, int bN, int bC, int bH, int bW) {
    int a[4] = {aN, aC, aH, aW}, b[4] = {bN, bC, bH, bW};
    return launch_broadcast(A, B, C, a, b, BMul{}, "broadcast_mul_4d");
}

// ---- concatenation along axis 1 of [N, n1] and [N, n2] rows (n = C*H*W per sample), and its backward split ---------
// The reference issues two cudaMemcpy per sample from a Python loop (cuTen.py:688-796); here each direction is one launch.
int seera_concat_fwd(const float *a, const float *b, float *out, int N, int n1, int n2) {
    SEERA_ENSURE();
    if (N < 0 || n1 < 0 || n2 < 0 || (N > 0 && ((n1 > 0 && !a) || (n2 > 0 && !b) || !out))) return fail(SEERA_E_ARG, "concat_fwd: bad argument");
    const long long total = (long long)N * (n1 + n2);
    if (total == 0) return SEERA_OK;
    const bool v4 = n1 % 4 == 0 && n2 % 4 == 0 && aligned16(a) && aligned16(b) && aligned16(out);
    if (v4) concat_kernel<true, float4><<<stride_grid(total / 4), 256, 0, rt().stream>>>(a, b, out, total / 4, n1 / 4, n2 / 4);
    else concat_kernel<true, float><<<stride_grid(total), 256, 0, rt().stream>>>(a, b, out, total, n1, n2);
    SEERA_LAUNCH_CHECK("concat_fwd");
    return SEERA_OK;
}
int seera_concat_bwd(const float *dout, float *da, float *db, int N, int n1, int n2) {
    SEERA_ENSURE();
    if (N < 0 || n1 < 0 || n2 < 0 || (N > 0 && ((n1 > 0 && !da) || (n2 > 0 && !db) || !dout))) return fail(SEERA_E_ARG, "concat_bwd: bad argument");
    const long long total = (long long)N * (n1 + n2);
    if (total == 0) return SEERA_OK;
    const bool v4 = n1 % 4 == 0 && n2 % 4 == 0 && aligned16(da) && aligned16(db) && aligned16(dout);
    if (v4) concat_kernel<false, float4><<<stride_grid(total / 4), 256, 0, rt().stream>>>(da, db, const_cast<float *>(dout), total / 4, n1 / 4, n2 / 4);
    else concat_kernel<false, float><<<stride_grid(total), 256, 0, rt().stream>>>(da, db, const_cast<float *>(dout), total, n1, n2);
    SEERA_LAUNCH_CHECK("concat_bwd");
    return SEERA_OK;
}

}  // extern "C"
