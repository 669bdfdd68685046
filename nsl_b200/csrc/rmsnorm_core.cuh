// RMSNorm with the reference's f64 semantics at fp32 cost.
//
// nsl_tensor_rmsnorm (crates/nsl-runtime/src/tensor/mod.rs:3016-3035) computes, per row,
//   rms = sqrt(sum_k x_k^2 / K + eps)      in f64
//   h_k = (f32)(x_k / rms * w_k)           in f64, rounded once to f32.
// This GPU issues an f64 instruction of a warp every 16 clocks per scheduler (measured: a row of 3200
// normalised with f64 arithmetic cost 3.4 us of a CTA's time, more than a decode projection's whole
// multiply), so the f64 work is reduced to a dozen instructions per row and none per element:
//
//  * sum of squares: x^2 = p + e exactly (p = fl(x*x), e = fma(x, x, -p)); p and e are accumulated in a
//    float-float pair (TwoSum), 48 bits; partial sums are combined in f64.  The result differs from the
//    reference's sequential f64 sum by a few units of 2^-46, which moves a normalised value across an f32
//    rounding boundary about once in 10^7 elements (a tree of f64 partial sums, the form used before,
//    already differed from the sequential sum in the last bits).
//  * 1/rms: f32 rsqrt seed and two Newton steps in f64 (within 3 ulp), split into rh + rl (f32 each).
//  * element: x*w = p + e exactly, (p + e)(rh + rl) = q + low with relative error < 2^-45 (three fmas), and
//    r = fl(q + low).  r equals the reference's (f32)((double)x / rms * (double)w) -- whose own f64 value is
//    within 2 ulp(f64) of the same ideal -- unless the ideal lies within 2^-45 of an f32 rounding boundary.
//    The distance of q + low from the boundaries of r's rounding interval is hu - |t|, t = (q - r) + low,
//    hu = half an ulp of r; elements with |t| >= hu (1 - 2^-17), i.e. closer than 2^-42 relative (8.5e-6 of
//    random inputs), and elements outside the safe exponent ranges, zero excepted, take the f64 expression.
//    Checked on the CPU against that expression on 4.7e7 random elements (K = 256, 3200, 8640, amplitudes
//    e^-10 .. e^10, with outliers): no difference.
//  * rows whose squares leave [2^-80, 2^100) or whose mean square leaves (2^-60, 2^60) are summed and
//    normalised in f64 throughout (the caller's fallback).
#pragma once
#include "common.cuh"

namespace nslq {

struct FF { float h, l; };      // the value h + l

// a += x^2; bad: the square left the range in which e is exact and a cannot overflow
static __device__ __forceinline__ void ff_add_sq(FF &a, float x, bool &bad)
{
    const float p = __fmul_rn(x, x), e = __fmaf_rn(x, x, -p);
    bad |= !(p < 0x1p100f) || (p < 0x1p-80f && x != 0.0f);
    const float t = __fadd_rn(a.h, p), bb = __fsub_rn(t, a.h);
    const float err = __fadd_rn(__fsub_rn(a.h, __fsub_rn(t, bb)), __fsub_rn(p, bb));
    a.h = t;
    a.l = __fadd_rn(a.l, __fadd_rn(err, e));
}

static __device__ __forceinline__ void ff_add(FF &a, const FF b)
{
    const float t = __fadd_rn(a.h, b.h), bb = __fsub_rn(t, a.h);
    const float err = __fadd_rn(__fsub_rn(a.h, __fsub_rn(t, bb)), __fsub_rn(b.h, bb));
    a.h = t;
    a.l = __fadd_rn(__fadd_rn(a.l, b.l), err);
}

// Sum over the warp; a row marked bad comes back with h = NaN in every lane.
static __device__ __forceinline__ FF ff_warp_sum(FF a, bool bad)
{
    if (bad) a.h = __int_as_float(0x7fc00000);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        FF b;
        b.h = __shfl_xor_sync(0xffffffffu, a.h, o);
        b.l = __shfl_xor_sync(0xffffffffu, a.l, o);
        ff_add(a, b);
    }
    return a;
}

// The warps' partial sums added as a tree of fixed shape (three dependent f64 additions for eight warps
// instead of eight: an f64 instruction's latency is part of every row's critical path).
template <int N>
static __device__ __forceinline__ double sum_partials(const double *part, int stride)
{
    double t[N];
#pragma unroll
    for (int i = 0; i < N; ++i) t[i] = part[i * stride];
#pragma unroll
    for (int n = N; n > 1; n = (n + 1) / 2)
#pragma unroll
        for (int i = 0; i < n / 2; ++i) t[i] = t[i] + t[n - 1 - i];
    return t[0];
}

struct RmsScale {
    double tot, k, eps;     // for the f64 expression
    float rh, rl;           // 1/rms = rh + rl
    bool fast;
};

// tot: the row's sum of squares; inv_k = 1.0 / K rounded to f64 (from the host).
static __device__ __forceinline__ RmsScale rms_scale(double tot, double k, double inv_k, double eps)
{
    RmsScale s;
    s.tot = tot; s.k = k; s.eps = eps;
    const double ms = fma(tot, inv_k, eps);
    s.fast = ms > 0x1p-60 && ms < 0x1p60;              // false for NaN
    double y = (double)rsqrtf((float)ms);
#pragma unroll
    for (int it = 0; it < 2; ++it) {
        const double t = __dmul_rn(ms, y), e = __fma_rn(-t, y, 1.0), h = __dmul_rn(y, 0.5);
        y = __fma_rn(h, e, y);
    }
    s.rh = (float)y;
    s.rl = (float)(y - (double)s.rh);
    return s;
}

// The reference's expression, for the elements (and rows) the fp32 path hands over.
static __device__ __noinline__ float norm_exact(float x, float w, double tot, double k, double eps)
{
    const double rms = sqrt(tot / k + eps);
    return (float)(__dmul_rn(__ddiv_rn((double)x, rms), (double)w));
}

static __device__ __forceinline__ float norm_ff(float x, float w, const RmsScale &s)
{
    if (!s.fast) return norm_exact(x, w, s.tot, s.k, s.eps);
    const float p = __fmul_rn(x, w);
    if (x == 0.0f || w == 0.0f) return p;              // +-0 with the product's sign, as the reference
    const float e = __fmaf_rn(x, w, -p);
    const float q = __fmul_rn(p, s.rh), qe = __fmaf_rn(p, s.rh, -q);
    const float low = __fmaf_rn(p, s.rl, __fmaf_rn(e, s.rh, qe));
    const float r = __fadd_rn(q, low), t = __fadd_rn(__fsub_rn(q, r), low);
    const uint32_t rb = __float_as_uint(r), eb = rb & 0x7f800000u, pb = __float_as_uint(p) & 0x7f800000u;
    const float hu = __uint_as_float(eb - (24u << 23));
    const bool ok = fabsf(t) < __fmul_rn(hu, 0.99999237060546875f) && eb >= (40u << 23) && eb <= (230u << 23) &&
                    pb >= (40u << 23) && pb <= (214u << 23) && (rb & 0x007fffffu) != 0u;
    return ok ? r : norm_exact(x, w, s.tot, s.k, s.eps);
}

}  // namespace nslq
