// Pack-at-load: the reference's weight quantisers on the GPU, producing the reference's bytes.
//
//  * ternary (BitNet b1.58): per-tensor absmean scale, trit = round_half_away(clamp(w/scale,-1,1)),
//    four trits per byte HIGH-BITS-FIRST  (crates/nsl-codegen/src/bitnet/loader.rs:126-193,
//    crates/nsl-codegen/src/bitnet/pack.rs:38-43).  The reference sums |w| sequentially in f32,
//    and a float sum depends on its order, so the scale kernel keeps that order: one thread adds,
//    the rest of its CTA only stages the data through shared memory.  It is a load-time cost
//    (~60 ms for a 27.6 M-element tensor), paid once per weight.
//  * INT4 per-group RTN in the QuantizedTensor form, shape [N,K], groups along K
//    (crates/nsl-runtime/src/quantize.rs:224-266, :366-417): f64 arithmetic like the reference,
//    min/max are order-independent, so one warp per group is exact.
//  * AWQ 4-bit, shape [K,N], groups along K per column (crates/nsl-runtime/src/awq.rs:53-144).
#include <climits>

#include "common.cuh"

namespace nslq {

constexpr int SEQ_THREADS = 256;
constexpr int SEQ_CHUNK = SEQ_THREADS * 4;

template <typename T>
__global__ void __launch_bounds__(SEQ_THREADS)
absmean_sequential_kernel(const T *__restrict__ w, int64_t numel, float *__restrict__ scale_out)
{
    __shared__ float buf[2][SEQ_CHUNK];
    float acc = 0.0f;
    const int64_t nchunks = (numel + SEQ_CHUNK - 1) / SEQ_CHUNK;
    auto stage = [&](int64_t c, int b) {
        const int64_t base = c * SEQ_CHUNK;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t k = base + i * SEQ_THREADS + threadIdx.x;
            buf[b][i * SEQ_THREADS + threadIdx.x] = (k < numel) ? fabsf(Elem<T>::to_f32(w[k])) : 0.0f;
        }
    };
    if (nchunks > 0) stage(0, 0);
    __syncthreads();
    for (int64_t c = 0; c < nchunks; ++c) {
        const int b = (int)(c & 1);
        if (c + 1 < nchunks && threadIdx.x != 0) stage(c + 1, b ^ 1);      // the others fetch the next chunk
        if (threadIdx.x == 0) {
            const int64_t left = numel - c * SEQ_CHUNK;
            const int n = left < SEQ_CHUNK ? (int)left : SEQ_CHUNK;
            for (int i = 0; i < n; ++i) acc = __fadd_rn(acc, buf[b][i]);   // the reference's order
            if (c + 1 < nchunks) {                                          // thread 0's own share of the next chunk
                const int64_t base = (c + 1) * SEQ_CHUNK;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int64_t k = base + i * SEQ_THREADS;
                    buf[b ^ 1][i * SEQ_THREADS] = (k < numel) ? fabsf(Elem<T>::to_f32(w[k])) : 0.0f;
                }
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) scale_out[0] = __fdiv_rn(acc, (float)numel);
}

template <typename T>
__global__ void __launch_bounds__(256)
ternary_pack_kernel(const T *__restrict__ w, int64_t nbytes, const float *__restrict__ scale_in, uint8_t *__restrict__ packed)
{
    const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nbytes) return;
    const float scale = scale_in[0];
    const float eff = scale > 0.0f ? scale : 1.0f;
    uint32_t byte = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float s = __fdiv_rn(Elem<T>::to_f32(w[4 * b + i]), eff);
        float t = truncf(s);
        if (fabsf(s - t) >= 0.5f) t += copysignf(1.0f, s);
        const int trit = max(-1, min(1, __float2int_rz(t)));              // clamp commutes with the rounding; NaN -> 0
        byte |= (uint32_t)(trit + 1) << (6 - 2 * i);
    }
    packed[b] = (uint8_t)byte;
}

// ---- INT4 RTN, QuantizedTensor [N,K], per-group along axis 1: one warp per (row, group)
static __device__ __forceinline__ double warp_min(double v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmin(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
static __device__ __forceinline__ double warp_max(double v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmax(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
static __device__ __forceinline__ double clampd(double v, double lo, double hi) { return v < lo ? lo : (v > hi ? hi : v); }
// Rust `f64 as u8`: saturating, NaN -> 0
static __device__ __forceinline__ uint32_t sat_u8(double v) { return (v != v || v <= 0.0) ? 0u : (v >= 255.0 ? 255u : (uint32_t)v); }

template <typename T>
__global__ void __launch_bounds__(256)
int4_group_quantize_nk_kernel(const T *__restrict__ w, int64_t N, int64_t K, int gs, int G, uint8_t *__restrict__ codes,
                              float *__restrict__ scale_out, uint8_t *__restrict__ zp_out)
{
    const int64_t grp_id = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (grp_id >= N * G) return;
    const int64_t n = grp_id / G;
    const int g = (int)(grp_id % G);
    const int64_t k0 = (int64_t)g * gs, k1 = (k0 + gs < K) ? k0 + gs : K;
    const T *row = w + n * K;
    double mn = INFINITY, mx = -INFINITY;
    for (int64_t k = k0 + lane; k < k1; k += 32) {
        const double v = (double)row[k];
        if (v < mn) mn = v;                      // same comparisons as the reference's loop (NaN never wins)
        if (v > mx) mx = v;
    }
    mn = warp_min(mn);
    mx = warp_max(mx);
    const double qmin = 0.0, qmax = 15.0;
    float scale;
    uint32_t zp;
    const double range = mx - mn;
    if (range < 1e-7) {                          // quantize.rs:236-248: constant group
        const double mid_q = round((qmin + qmax) / 2.0);
        const double abs_val = fmax(fabs(mn), 1e-7);
        const double sc = abs_val / mid_q;
        zp = sat_u8(clampd(round(mid_q - mn / sc), qmin, qmax));
        scale = (float)sc;
    } else {
        const double sc = range / (qmax - qmin);
        zp = sat_u8(clampd(round(-mn / sc), qmin, qmax));
        scale = (float)sc;
    }
    if (lane == 0) { scale_out[grp_id] = scale; zp_out[grp_id] = (uint8_t)zp; }
    // two codes per byte over the flat index n*K+k; K and the group size are even (host check), so a
    // byte never straddles rows or groups
    for (int64_t k = k0 + 2 * lane; k < k1; k += 64) {
        const uint32_t q0 = sat_u8(clampd(round((double)row[k] / (double)scale + (double)zp), qmin, qmax));
        const uint32_t q1 = sat_u8(clampd(round((double)row[k + 1] / (double)scale + (double)zp), qmin, qmax));
        codes[(n * K + k) >> 1] = (uint8_t)((q0 & 15u) | ((q1 & 15u) << 4));
    }
}

// ---- AWQ [K,N]: one thread per (group, column); groups along K
template <typename T>
__global__ void __launch_bounds__(256)
awq_quantize_kn_kernel(const T *__restrict__ w, int64_t K, int64_t N, int gs, int G, uint8_t *__restrict__ data,
                       double *__restrict__ scales, double *__restrict__ zeros)
{
    const int64_t id = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= (int64_t)G * N) return;
    const int g = (int)(id / N);
    const int64_t col = id % N;
    const int64_t k0 = (int64_t)g * gs, k1 = (k0 + gs < K) ? k0 + gs : K;
    double mn = INFINITY, mx = -INFINITY;
    for (int64_t k = k0; k < k1; ++k) { const double v = (double)w[k * N + col]; mn = fmin(mn, v); mx = fmax(mx, v); }
    double scale, zero = mn;
    if (fabs(mx - mn) < 1e-10) scale = 1.0; else scale = (mx - mn) / 15.0;
    scales[id] = scale;
    zeros[id] = zero;
    for (int64_t k = k0; k < k1; ++k) {
        const double r = round(((double)w[k * N + col] - zero) / scale);
        int q = (r != r) ? 0 : (r <= -2147483648.0 ? INT_MIN : (r >= 2147483647.0 ? INT_MAX : (int)r));
        q = max(0, min(15, q));
        const int64_t flat = k * N + col;
        // neighbouring columns share a byte and are written by other threads: merge with an atomic OR
        atomicOr(reinterpret_cast<unsigned int *>(data + ((flat >> 1) & ~(int64_t)3)),
                 (unsigned int)q << (8 * ((flat >> 1) & 3) + 4 * (flat & 1)));
    }
}

template <typename T>
static int ternary_quantize_pack_t(const void *w, int64_t numel, uint8_t *packed, float *scale, cudaStream_t st)
{
    absmean_sequential_kernel<T><<<1, SEQ_THREADS, 0, st>>>((const T *)w, numel, scale);
    int rc = check_launch("absmean_sequential_kernel");
    if (rc) return rc;
    const int64_t nbytes = numel / 4;
    ternary_pack_kernel<T><<<(unsigned)((nbytes + 255) / 256), 256, 0, st>>>((const T *)w, nbytes, scale, packed);
    return check_launch("ternary_pack_kernel");
}

int ternary_quantize_pack_dispatch(const void *w, int w_dtype, int64_t numel, uint8_t *packed, float *scale, cudaStream_t st)
{
    switch (w_dtype) {
    case NSLQ_DTYPE_F32: return ternary_quantize_pack_t<float>(w, numel, packed, scale, st);
    case NSLQ_DTYPE_FP16: return ternary_quantize_pack_t<__half>(w, numel, packed, scale, st);
    case NSLQ_DTYPE_BF16: return ternary_quantize_pack_t<__nv_bfloat16>(w, numel, packed, scale, st);
    default: return fail(NSLQ_ERR_ARG, "nslq_ternary_quantize_pack: dtype %d not in {F32,FP16,BF16}", w_dtype);
    }
}

int int4_quantize_nk_dispatch(const void *w, int w_dtype, int64_t N, int64_t K, int64_t gs, uint8_t *codes, float *scale,
                              uint8_t *zp, cudaStream_t st)
{
    const int G = (int)((K + gs - 1) / gs);
    if (cudaMemsetAsync(codes, 0, (size_t)(N * K / 2), st) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "nslq_int4_quantize_nk: %s", cudaGetErrorString(cudaGetLastError()));
    const int64_t groups = N * G;
    const unsigned blocks = (unsigned)((groups + 7) / 8);
    if (w_dtype == NSLQ_DTYPE_F64) int4_group_quantize_nk_kernel<double><<<blocks, 256, 0, st>>>((const double *)w, N, K, (int)gs, G, codes, scale, zp);
    else if (w_dtype == NSLQ_DTYPE_F32) int4_group_quantize_nk_kernel<float><<<blocks, 256, 0, st>>>((const float *)w, N, K, (int)gs, G, codes, scale, zp);
    else return fail(NSLQ_ERR_ARG, "nslq_int4_quantize_nk: dtype %d not in {F64,F32}", w_dtype);
    return check_launch("int4_group_quantize_nk_kernel");
}

int awq_quantize_kn_dispatch(const void *w, int w_dtype, int64_t K, int64_t N, int64_t gs, uint8_t *data, double *scales, double *zeros,
                             cudaStream_t st)
{
    const int G = (int)((K + gs - 1) / gs);
    if (cudaMemsetAsync(data, 0, (size_t)(K * N / 2), st) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "nslq_awq_quantize_kn: %s", cudaGetErrorString(cudaGetLastError()));
    const int64_t n = (int64_t)G * N;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (w_dtype == NSLQ_DTYPE_F64) awq_quantize_kn_kernel<double><<<blocks, 256, 0, st>>>((const double *)w, K, N, (int)gs, G, data, scales, zeros);
    else if (w_dtype == NSLQ_DTYPE_F32) awq_quantize_kn_kernel<float><<<blocks, 256, 0, st>>>((const float *)w, K, N, (int)gs, G, data, scales, zeros);
    else return fail(NSLQ_ERR_ARG, "nslq_awq_quantize_kn: dtype %d not in {F64,F32}", w_dtype);
    return check_launch("awq_quantize_kn_kernel");
}

// ---------------------------------------------------------------- nsl_qtensor_quantize / _dequantize, every form
// crates/nsl-runtime/src/quantize.rs:283-426 and :436-537: INT8 or INT4, per tensor / per channel / per
// group along any axis of an n-dimensional tensor.  The tensor is seen as [outer][axis][inner]; the scale
// index of an element follows the reference's loops (per channel: the channel; per group: outer * groups +
// channel / group_size).  Minimum and maximum are order-independent, everything else is per element, so the
// reference's bytes come out whatever the thread order.
struct QtGeom {
    int64_t total, axis_size, inner, ngroups;
    int gran, gs, int4;
};

static __device__ __forceinline__ int64_t qt_scale_index(const QtGeom &g, int64_t flat)
{
    if (g.gran == 0) return 0;
    const int64_t block = g.axis_size * g.inner;
    const int64_t o = flat / block, ch = (flat - o * block) / g.inner;
    return g.gran == 1 ? ch : o * g.ngroups + ch / g.gs;
}

// doubles as keys whose unsigned order is the numeric order (for atomicMin / atomicMax)
static __device__ __forceinline__ unsigned long long dkey(double v)
{
    const unsigned long long b = (unsigned long long)__double_as_longlong(v);
    return (b >> 63) ? ~b : (b | 0x8000000000000000ull);
}
static __device__ __forceinline__ double dunkey(unsigned long long k)
{
    return __longlong_as_double((long long)((k >> 63) ? (k & 0x7fffffffffffffffull) : ~k));
}

__global__ void qt_init_minmax_kernel(unsigned long long *mn, unsigned long long *mx, int64_t n)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { mn[i] = dkey(INFINITY); mx[i] = dkey(-INFINITY); }
}

template <typename T>
__global__ void __launch_bounds__(256) qt_minmax_kernel(const T *__restrict__ src, QtGeom g, unsigned long long *mn, unsigned long long *mx)
{
    // Whole warps stay in the loop (the tail is padded with NaNs, which never win), so that a warp whose 32
    // consecutive elements share one scale -- the common case: rows, groups along the last axis, per tensor --
    // reduces by shuffles and issues one pair of atomics instead of 32 to the same address.
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t rounds = (g.total + stride - 1) / stride;
    for (int64_t r = 0; r < rounds; ++r) {
        const int64_t i = r * stride + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
        const bool in = i < g.total;
        const double v = in ? (double)src[i] : NAN;
        const int64_t si = in ? qt_scale_index(g, i) : -1;
        const bool live = v == v;                   // the reference's comparisons never let a NaN win
        const int64_t s0 = __shfl_sync(0xffffffffu, si, 0);
        if (__all_sync(0xffffffffu, si == s0)) {
            if (s0 < 0) continue;
            double lo = live ? v : INFINITY, hi = live ? v : -INFINITY;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                lo = fmin(lo, __shfl_xor_sync(0xffffffffu, lo, o));
                hi = fmax(hi, __shfl_xor_sync(0xffffffffu, hi, o));
            }
            if ((threadIdx.x & 31) == 0 && lo <= hi) {
                atomicMin(mn + s0, dkey(lo));
                atomicMax(mx + s0, dkey(hi));
            }
        } else if (live && in) {
            atomicMin(mn + si, dkey(v));
            atomicMax(mx + si, dkey(v));
        }
    }
}

__global__ void qt_scale_zp_kernel(const unsigned long long *mn_k, const unsigned long long *mx_k, int64_t n, double qmax,
                                   float *__restrict__ scale_out, uint8_t *__restrict__ zp_out)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const double qmin = 0.0, mn = dunkey(mn_k[i]), mx = dunkey(mx_k[i]);
    const double range = mx - mn;
    if (range < 1e-7) {                             // quantize.rs:236-248: constant group
        const double mid_q = round((qmin + qmax) / 2.0);
        const double abs_val = fmax(fabs(mn), 1e-7);
        const double sc = abs_val / mid_q;
        zp_out[i] = (uint8_t)sat_u8(clampd(round(mid_q - mn / sc), qmin, qmax));
        scale_out[i] = (float)sc;
    } else {
        const double sc = range / (qmax - qmin);
        zp_out[i] = (uint8_t)sat_u8(clampd(round(-mn / sc), qmin, qmax));
        scale_out[i] = (float)sc;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) qt_quantize_kernel(const T *__restrict__ src, QtGeom g, const float *__restrict__ scale,
                                                          const uint8_t *__restrict__ zp, uint8_t *__restrict__ data)
{
    const double qmax = g.int4 ? 15.0 : 255.0;
    const int64_t nbytes = g.int4 ? (g.total + 1) / 2 : g.total;
    for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < nbytes; b += (int64_t)gridDim.x * blockDim.x) {
        uint32_t out = 0;
        const int per = g.int4 ? 2 : 1;
        for (int e = 0; e < per; ++e) {
            const int64_t i = b * per + e;
            if (i >= g.total) break;
            const int64_t si = qt_scale_index(g, i);
            const uint32_t q = sat_u8(clampd(round((double)src[i] / (double)scale[si] + (double)zp[si]), 0.0, qmax));
            out |= g.int4 ? ((q & 15u) << (4 * e)) : q;
        }
        data[b] = (uint8_t)out;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) qt_dequantize_kernel(const uint8_t *__restrict__ data, QtGeom g, const float *__restrict__ scale,
                                                            const uint8_t *__restrict__ zp, T *__restrict__ out)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < g.total; i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t q = g.int4 ? ((i & 1) ? (data[i >> 1] >> 4) : (data[i >> 1] & 15u)) : data[i];
        const int64_t si = qt_scale_index(g, i);
        out[i] = (T)(((double)q - (double)zp[si]) * (double)scale[si]);     // quantize.rs:263-266, f64
    }
}

// *nscales = the length the reference gives scale and zero_point (compute_num_scales, quantize.rs:72-96: for
// per-group it multiplies every other dimension, the inner ones too); *nused = the entries its loops write
// (outer * groups, quantize.rs:375-420).  The entries past *nused are zero here (the reference leaves the
// scales there uninitialised and the zero points 0).
static int qt_geometry(const char *who, const int64_t *shape, int ndim, int dtype, int gran, int axis, int64_t gs, QtGeom *g, int64_t *nscales,
                       int64_t *nused)
{
    if (!shape || ndim <= 0 || ndim > 8) return fail(NSLQ_ERR_SHAPE, "%s: ndim=%d (1..8)", who, ndim);
    if (dtype != 0 && dtype != 1) return fail(NSLQ_ERR_ARG, "%s: unknown quantization dtype %d", who, dtype);
    if (gran < 0 || gran > 2) return fail(NSLQ_ERR_ARG, "%s: unknown quantization granularity %d", who, gran);
    if (gran != 0 && (axis < 0 || axis >= ndim)) return fail(NSLQ_ERR_ARG, "%s: axis %d of a %d-dimensional tensor", who, axis, ndim);
    if (gran == 2 && gs <= 0) return fail(NSLQ_ERR_ARG, "%s: group size %lld", who, (long long)gs);
    int64_t total = 1;
    for (int i = 0; i < ndim; ++i) { if (shape[i] <= 0) return fail(NSLQ_ERR_SHAPE, "%s: dimension %d is %lld", who, i, (long long)shape[i]); total *= shape[i]; }
    g->total = total; g->gran = gran; g->int4 = dtype == 1; g->gs = gran == 2 ? (int)gs : 1;
    g->axis_size = gran ? shape[axis] : total; g->inner = 1;
    for (int d = axis + 1; gran && d < ndim; ++d) g->inner *= shape[d];
    g->ngroups = gran == 2 ? (g->axis_size + gs - 1) / gs : 1;
    const int64_t outer = gran ? total / (g->axis_size * g->inner) : 1;
    *nused = gran == 0 ? 1 : (gran == 1 ? g->axis_size : outer * g->ngroups);
    *nscales = gran == 2 ? (total / g->axis_size) * g->ngroups : *nused;
    return NSLQ_OK;
}

int qtensor_quantize_dispatch(const void *src, int src_dtype, const int64_t *shape, int ndim, int dtype, int gran, int axis, int64_t gs,
                              uint8_t *data, float *scale, uint8_t *zp, cudaStream_t st)
{
    QtGeom g;
    int64_t ns = 0, nall = 0;
    int rc = qt_geometry("nslq_qtensor_quantize", shape, ndim, dtype, gran, axis, gs, &g, &nall, &ns);
    if (rc) return rc;
    if (src_dtype != NSLQ_DTYPE_F64 && src_dtype != NSLQ_DTYPE_F32) return fail(NSLQ_ERR_ARG, "nslq_qtensor_quantize: dtype %d not in {F64,F32}", src_dtype);
    unsigned long long *mm = nullptr;                 // load-time call: a scratch of two keys per scale
    if (cudaMalloc(&mm, (size_t)ns * 16) != cudaSuccess) return fail(NSLQ_ERR_CUDA, "nslq_qtensor_quantize: %s", cudaGetErrorString(cudaGetLastError()));
    const unsigned sb = (unsigned)((ns + 255) / 256);
    const unsigned eb = (unsigned)(g.total / 256 + 1 < 4736 ? g.total / 256 + 1 : 4736);
    if (nall > ns) {
        cudaMemsetAsync(scale + ns, 0, (size_t)(nall - ns) * 4, st);
        cudaMemsetAsync(zp + ns, 0, (size_t)(nall - ns), st);
    }
    qt_init_minmax_kernel<<<sb, 256, 0, st>>>(mm, mm + ns, ns);
    if (src_dtype == NSLQ_DTYPE_F64) qt_minmax_kernel<double><<<eb, 256, 0, st>>>((const double *)src, g, mm, mm + ns);
    else qt_minmax_kernel<float><<<eb, 256, 0, st>>>((const float *)src, g, mm, mm + ns);
    qt_scale_zp_kernel<<<sb, 256, 0, st>>>(mm, mm + ns, ns, g.int4 ? 15.0 : 255.0, scale, zp);
    if (src_dtype == NSLQ_DTYPE_F64) qt_quantize_kernel<double><<<eb, 256, 0, st>>>((const double *)src, g, scale, zp, data);
    else qt_quantize_kernel<float><<<eb, 256, 0, st>>>((const float *)src, g, scale, zp, data);
    rc = check_launch("qt_quantize_kernel");
    cudaStreamSynchronize(st);
    cudaFree(mm);
    return rc;
}

int qtensor_dequantize_dispatch(const uint8_t *data, const float *scale, const uint8_t *zp, const int64_t *shape, int ndim, int dtype,
                                int gran, int axis, int64_t gs, void *out, int out_dtype, cudaStream_t st)
{
    QtGeom g;
    int64_t ns = 0, nall = 0;
    int rc = qt_geometry("nslq_qtensor_dequantize", shape, ndim, dtype, gran, axis, gs, &g, &nall, &ns);
    if (rc) return rc;
    const unsigned eb = (unsigned)(g.total / 256 + 1 < 4736 ? g.total / 256 + 1 : 4736);
    if (out_dtype == NSLQ_DTYPE_F64) qt_dequantize_kernel<double><<<eb, 256, 0, st>>>(data, g, scale, zp, (double *)out);
    else if (out_dtype == NSLQ_DTYPE_F32) qt_dequantize_kernel<float><<<eb, 256, 0, st>>>(data, g, scale, zp, (float *)out);
    else return fail(NSLQ_ERR_ARG, "nslq_qtensor_dequantize: out dtype %d not in {F64,F32}", out_dtype);
    return check_launch("qt_dequantize_kernel");
}

int64_t qtensor_num_scales(const int64_t *shape, int ndim, int gran, int axis, int64_t gs)
{
    QtGeom g;
    int64_t ns = 0, nall = 0;
    return qt_geometry("nslq_qtensor_num_scales", shape, ndim, 0, gran, axis, gs, &g, &nall, &ns) == NSLQ_OK ? nall : -1;
}

}  // namespace nslq
