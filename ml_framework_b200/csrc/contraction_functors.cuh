// Operand and output functors shared by the contraction kernels (CUDA-core tiles and tensor-core tiles).
//
// A contraction is C[M,N] = sum_k A(m,k) * B(k,n).  An operand functor exposes
//     Fx    fix(int fixed_index)          work done once per thread (row m for A, column n for B)
//     float load(const Fx&, int k)        one element, zero outside the operand
// so one main loop serves Dense (plain strides, either operand transposed), the im2col view of a
// convolution input, the col2im gather of a data gradient and the per-tap view of a weight gradient.
#pragma once
#include "common.cuh"

namespace seera {

// ---- operand functors ------------------------------------------------------------------------------------
// Every functor exposes  Fx fix(int fixed_index)  (work done once per thread) and
// float load(const Fx&, int k)  (per k-step).  For A the fixed index is the row m, for B the column n.

// element (fixed f, varying k) at p[f*fs + k*ks], zero outside [0,nf) x [0,nk)
struct Strided {
    const float *p; long long fs, ks; int nf, nk;
    struct Fx { const float *q; bool ok; };
    __device__ Fx fix(int f) const { return {p + (long long)f * fs, f < nf}; }
    __device__ float load(const Fx &x, int k) const { return (x.ok && k < nk) ? __ldg(x.q + (long long)k * ks) : 0.f; }
};

struct ConvGeom {
    int C, H, W;          // the tensor being gathered from: channels and spatial size
    int OH, OW;           // the spatial size of the other side (outputs of the forward convolution)
    int R, S, sh, sw, ph, pw;
};

// im2col(X)[k = (c,r,s)][n = (img,oh,ow)] : fixed = column n, varying = k.   (fprop B operand)
template <int RS_, int S_>
struct Im2colByCol {
    const float *X; ConvGeom g; int ncols, K;
    struct Fx { const float *base; int ih0, iw0; bool ok; };
    __device__ Fx fix(int n) const {
        int P = g.OH * g.OW, img = n / P, p = n - img * P, oh = p / g.OW, ow = p - oh * g.OW;
        return {X + (long long)img * g.C * g.H * g.W, oh * g.sh - g.ph, ow * g.sw - g.pw, n < ncols};
    }
    __device__ float load(const Fx &x, int k) const {
        int RS = RS_ ? RS_ : g.R * g.S, S = S_ ? S_ : g.S;
        int c = k / RS, rs = k - c * RS, r = rs / S, s = rs - r * S;
        int ih = x.ih0 + r, iw = x.iw0 + s;
        bool v = x.ok && k < K && (unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W;
        return v ? __ldg(x.base + ((long long)c * g.H + ih) * g.W + iw) : 0.f;
    }
};

// im2col(X)[k = (img,oh,ow)][n = (c,r,s)] : fixed = column n = (c,r,s), varying = k.   (wgrad B operand)
struct Im2colByTap {
    const float *X; ConvGeom g; int ncols, K;
    struct Fx { int coff, dr, ds; bool ok; };
    __device__ Fx fix(int n) const {
        int RS = g.R * g.S, c = n / RS, rs = n - c * RS, r = rs / g.S, s = rs - r * g.S;
        return {c * g.H * g.W, r - g.ph, s - g.pw, n < ncols};
    }
    __device__ float load(const Fx &x, int k) const {
        int P = g.OH * g.OW, img = k / P, p = k - img * P, oh = p / g.OW, ow = p - oh * g.OW;
        int ih = oh * g.sh + x.dr, iw = ow * g.sw + x.ds;
        bool v = x.ok && k < K && (unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W;
        return v ? __ldg(X + (long long)img * g.C * g.H * g.W + x.coff + ih * g.W + iw) : 0.f;
    }
};

// dY[img][f][p] seen as A(m = f, k = (img,p))   (wgrad A operand); F channels of P pixels
struct ByImagePixel {
    const float *Y; int F, P, K;
    struct Fx { long long off; bool ok; };
    __device__ Fx fix(int f) const { return {(long long)f * P, f < F}; }
    __device__ float load(const Fx &x, int k) const {
        int img = k / P, p = k - img * P;
        return (x.ok && k < K) ? __ldg(Y + (long long)img * F * P + x.off + p) : 0.f;
    }
};

// W[f][c][r][s] seen as A(m = c, k = (f,r,s))   (dgrad A operand)
struct WeightByInChannel {
    const float *Wt; int C, RS, K;
    struct Fx { const float *q; bool ok; };
    __device__ Fx fix(int c) const { return {Wt + (long long)c * RS, c < C}; }
    __device__ float load(const Fx &x, int k) const {
        int f = k / RS, rs = k - f * RS;
        return (x.ok && k < K) ? __ldg(x.q + (long long)f * C * RS + rs) : 0.f;
    }
};

// col2im gather: B(k = (f,r,s), n = (img,h,w)) = dY[img][f][(h+ph-r)/sh][(w+pw-s)/sw] when divisible and in range.
// Here g.C = F (channels of dY), g.H x g.W = spatial size of dY, g.OH x g.OW = spatial size of dX.   (dgrad B operand)
template <int RS_, int S_>
struct Col2imByPixel {
    const float *Y; ConvGeom g; int ncols, K;
    struct Fx { const float *base; int hh, ww; bool ok; };
    __device__ Fx fix(int n) const {
        int P = g.OH * g.OW, img = n / P, p = n - img * P, h = p / g.OW, w = p - h * g.OW;
        return {Y + (long long)img * g.C * g.H * g.W, h + g.ph, w + g.pw, n < ncols};
    }
    __device__ float load(const Fx &x, int k) const {
        int RS = RS_ ? RS_ : g.R * g.S, S = S_ ? S_ : g.S;
        int f = k / RS, rs = k - f * RS, r = rs / S, s = rs - r * S;
        int a = x.hh - r, b = x.ww - s;
        bool v = x.ok && k < K && a >= 0 && b >= 0;
        int oh = a, ow = b;
        if (g.sh != 1) { oh = a / g.sh; v = v && (oh * g.sh == a); }
        if (g.sw != 1) { ow = b / g.sw; v = v && (ow * g.sw == b); }
        v = v && oh < g.H && ow < g.W;
        return v ? __ldg(x.base + ((long long)f * g.H + oh) * g.W + ow) : 0.f;
    }
};

// ---- output functors -----------------------------------------------------------------------------------------
struct StoreDense {        // C[m*ld + n]
    static constexpr bool kMContiguous = false;
    float *C; long long ld;
    __device__ void operator()(int m, int n, float v) const { C[(long long)m * ld + n] = v; }
    // every output functor is affine in n: element (m, n) lives at row(m)[n * nstride()]; row(m) == nullptr skips the row
    __device__ float *row(int m) const { return C + (long long)m * ld; }
    __device__ long long nstride() const { return 1; }
};
struct StoreNCHW {         // n = (img, p): out[(img*M + m)*P + p]
    static constexpr bool kMContiguous = false;
    float *out; int M, P;
    __device__ void operator()(int m, int n, float v) const {
        int img = n / P, p = n - img * P;
        out[((long long)img * M + m) * P + p] = v;
    }
};   // (used by the CUDA-core kernel only, whose N index is the pixel)


// Output functors for kernels whose M index is the long (pixel / batch-row) dimension.
struct StoreDenseT {       // C[n*ld + m]
    static constexpr bool kMContiguous = true;
    float *C; long long ld;
    __device__ void operator()(int m, int n, float v) const { C[(long long)n * ld + m] = v; }
    __device__ float *row(int m) const { return C + m; }
    __device__ long long nstride() const { return ld; }
};
struct StorePixelRows {    // m = (img, p): out[(img*Nch + n)*P + p]
    static constexpr bool kMContiguous = true;
    float *out; int Nch, P;
    __device__ void operator()(int m, int n, float v) const {
        int img = m / P, p = m - img * P;
        out[((long long)img * Nch + n) * P + p] = v;
    }
    __device__ float *row(int m) const { int img = m / P, p = m - img * P; return out + (long long)img * Nch * P + p; }
    __device__ long long nstride() const { return P; }
};

}  // namespace seera
