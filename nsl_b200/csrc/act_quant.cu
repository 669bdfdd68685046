// Stage 1: per-token absmax int8 activation quantisation.
//
// One CTA per token row.  The row is read once into registers; max|x| is reduced
// with warp shuffles (then across warps through shared memory); the row is then
// quantised from registers with the reference's exact arithmetic and written in the
// natural order and/or the order the matmul kernels consume, plus scale and sum.
//
// Arithmetic follows crates/nsl-codegen/tests/bitnet_reference_impl.rs:46-70 of
// NSL: inv = 127/scale (IEEE divide), v = x*inv, clamp to [-127,127], round half
// away from zero, NaN -> 0.
#include "common.cuh"

namespace nslq {

constexpr int AQ_THREADS = 256;

static __device__ __forceinline__ float block_max(float v, float *smem)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) smem[w] = v;
    __syncthreads();
    float r = (l < AQ_THREADS / 32) ? smem[l] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
    return r;  // every thread holds the block maximum
}

static __device__ __forceinline__ int block_sum(int v, int *smem)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) smem[w] = v;
    __syncthreads();
    int r = (l < AQ_THREADS / 32) ? smem[l] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

// VEC = true: K % 16 == 0 and 16-byte aligned rows; four elements per thread per
// iteration, quads of lanes cover one group of 16 k (needed for q_perm).
template <typename T, bool VEC, int XV>
__global__ void __launch_bounds__(AQ_THREADS)
act_quant_kernel(const T *__restrict__ x, int64_t K, int8_t *__restrict__ q_plain,
                 int8_t *__restrict__ q_perm, float *__restrict__ scale_out,
                 int32_t *__restrict__ rowsum_out)
{
    __shared__ float smax[AQ_THREADS / 32];
    __shared__ int ssum[AQ_THREADS / 32];
    const int64_t r = blockIdx.x;
    const T *row = x + r * K;
    pdl_wait();

    // VEC path: the thread's share of the row stays in registers between the absmax pass and
    // the rounding pass (XV float4 per thread: K <= XV*4*AQ_THREADS; longer rows re-read the
    // tail, which is still in L1/L2).  XV is 4 or 12: short rows keep registers low so that more
    // rows are in flight per SM.
    const int nvec = VEC ? (int)(K >> 2) : 0;
    float4 xv[VEC ? XV : 1];
    float m = 0.0f;
    if (VEC) {
#pragma unroll
        for (int i = 0; i < XV; ++i) {
            const int v = i * AQ_THREADS + threadIdx.x;
            xv[i] = (v < nvec) ? Vec4<T>::load(row, v) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < XV; ++i)
            m = fmaxf(m, fmaxf(fmaxf(fabsf(xv[i].x), fabsf(xv[i].y)), fmaxf(fabsf(xv[i].z), fabsf(xv[i].w))));
        for (int v = XV * AQ_THREADS + threadIdx.x; v < nvec; v += AQ_THREADS) {
            const float4 f = Vec4<T>::load(row, v);
            m = fmaxf(m, fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w))));
        }
    } else {
        for (int64_t k = threadIdx.x; k < K; k += AQ_THREADS) m = fmaxf(m, fabsf(Elem<T>::to_f32(row[k])));
    }
    const float scale = block_max(m, smax);
    pdl_launch_dependents();
    const float inv = __fdiv_rn(127.0f, scale);
    const bool zero_row = (scale == 0.0f);

    int sum = 0;
    if (VEC) {
        // K/4 is a multiple of 4 and AQ_THREADS is a multiple of 4, so the four lanes of a quad
        // are always inside the row together; `mask` names exactly the lanes inside.
        auto quant_store = [&](const float4 &f, int v, unsigned mask) {
            // An all-zero row has scale 0 and inv = +inf: 0 * inf and NaN * inf are NaN, which
            // quant_one maps to 0 like the reference, so the row needs no special case here.  (The
            // kernel is bound by issued instructions -- about 25 per element at 1.4 IPC -- not by
            // HBM, so the selects and the four adds of the row sum are worth removing.)
            const int q0 = quant_one(f.x, inv), q1 = quant_one(f.y, inv);
            const int q2 = quant_one(f.z, inv), q3 = quant_one(f.w, inv);
            const uint32_t w = pack4_i8(q0, q1, q2, q3);
            sum = __dp4a((int)w, 0x01010101, sum);
            if (q_plain) reinterpret_cast<uint32_t *>(q_plain + r * K)[v] = w;
            if (q_perm) reinterpret_cast<uint32_t *>(q_perm + r * K)[v] = quad_transpose(w, mask);
        };
#pragma unroll
        for (int i = 0; i < XV; ++i) {
            const int v = i * AQ_THREADS + threadIdx.x;
            const bool in = v < nvec;
            const unsigned mask = __ballot_sync(0xffffffffu, in);
            if (in) quant_store(xv[i], v, mask);
        }
        for (int base = XV * AQ_THREADS; base < nvec; base += AQ_THREADS) {
            const int v = base + threadIdx.x;
            const bool in = v < nvec;
            const unsigned mask = __ballot_sync(0xffffffffu, in);
            if (in) quant_store(Vec4<T>::load(row, v), v, mask);
        }
    } else {
        for (int64_t k = threadIdx.x; k < K; k += AQ_THREADS) {
            int q = zero_row ? 0 : quant_one(Elem<T>::to_f32(row[k]), inv);
            sum += q;
            if (q_plain) q_plain[r * K + k] = (int8_t)q;
        }
    }
    if (rowsum_out) {
        int tot = block_sum(sum, ssum);
        if (threadIdx.x == 0) rowsum_out[r] = tot;
    }
    if (threadIdx.x == 0) scale_out[r] = scale;
}

static __device__ __forceinline__ double block_sum_f64(double v, double *smem)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) smem[w] = v;
    __syncthreads();
    double r = (l < AQ_THREADS / 32) ? smem[l] : 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

// RMSNorm fused in front of the quantisation (the prologue NSL's BitNet kernel config names
// `fused_rmsnorm` but never emits, crates/nsl-codegen/src/bitnet/config.rs:23-31): one CTA per row,
//   rms = sqrt(sum_k x^2 / K + eps)                 in f64
//   h   = (f32)(x / rms * weight)                   in f64, rounded once
// exactly the arithmetic of nsl_tensor_rmsnorm (crates/nsl-runtime/src/tensor/mod.rs:3016-3035),
// except that the sum of squares is a tree reduction instead of a sequential loop (it can differ
// in the last bits of the f64); h never goes to memory unless h_out is given.  Then the row is
// quantised from registers like act_quant_kernel.
template <typename T, int XV>
__global__ void __launch_bounds__(AQ_THREADS)
rmsnorm_act_quant_kernel(const T *__restrict__ x, const float *__restrict__ weight, double eps, int64_t K,
                         float *__restrict__ h_out, int8_t *__restrict__ q_plain, int8_t *__restrict__ q_perm,
                         float *__restrict__ scale_out, int32_t *__restrict__ rowsum_out)
{
    __shared__ float smax[AQ_THREADS / 32];
    __shared__ int ssum[AQ_THREADS / 32];
    __shared__ double ssq[AQ_THREADS / 32];
    const int64_t r = blockIdx.x;
    const T *row = x + r * K;
    pdl_wait();
    const int nvec = (int)(K >> 2);
    float4 xv[XV];
    double sq = 0.0;
#pragma unroll
    for (int i = 0; i < XV; ++i) {
        const int v = i * AQ_THREADS + threadIdx.x;
        xv[i] = (v < nvec) ? Vec4<T>::load(row, v) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < XV; ++i)
        sq += (double)xv[i].x * xv[i].x + (double)xv[i].y * xv[i].y + (double)xv[i].z * xv[i].z + (double)xv[i].w * xv[i].w;
    const double rms = sqrt(block_sum_f64(sq, ssq) / (double)K + eps);
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < XV; ++i) {
        const int v = i * AQ_THREADS + threadIdx.x;
        if (v < nvec) {
            const float4 w = reinterpret_cast<const float4 *>(weight)[v];
            float4 h;
            h.x = (float)((double)xv[i].x / rms * (double)w.x); h.y = (float)((double)xv[i].y / rms * (double)w.y);
            h.z = (float)((double)xv[i].z / rms * (double)w.z); h.w = (float)((double)xv[i].w / rms * (double)w.w);
            xv[i] = h;
            if (h_out) reinterpret_cast<float4 *>(h_out + r * K)[v] = h;
            m = fmaxf(m, fmaxf(fmaxf(fabsf(h.x), fabsf(h.y)), fmaxf(fabsf(h.z), fabsf(h.w))));
        }
    }
    const float scale = block_max(m, smax);
    pdl_launch_dependents();
    const float inv = __fdiv_rn(127.0f, scale);
    int sum = 0;
#pragma unroll
    for (int i = 0; i < XV; ++i) {
        const int v = i * AQ_THREADS + threadIdx.x;
        const bool in = v < nvec;
        const unsigned mask = __ballot_sync(0xffffffffu, in);          // whole quads: K % 16 == 0
        if (in) {
            const float4 f = xv[i];
            const uint32_t w = pack4_i8(quant_one(f.x, inv), quant_one(f.y, inv), quant_one(f.z, inv), quant_one(f.w, inv));
            sum = __dp4a((int)w, 0x01010101, sum);
            if (q_plain) reinterpret_cast<uint32_t *>(q_plain + r * K)[v] = w;
            if (q_perm) reinterpret_cast<uint32_t *>(q_perm + r * K)[v] = quad_transpose(w, mask);
        }
    }
    if (rowsum_out) {
        const int tot = block_sum(sum, ssum);
        if (threadIdx.x == 0) rowsum_out[r] = tot;
    }
    if (threadIdx.x == 0) scale_out[r] = scale;
}

template <typename T>
static int launch_rmsnorm_quant(const void *x, const float *weight, double eps, int64_t M, int64_t K, float *h_out,
                                int8_t *q_plain, int8_t *q_perm, float *scale, int32_t *rowsum, cudaStream_t st)
{
    dim3 grid((unsigned)M), block(AQ_THREADS);
    cudaError_t e;
    if (K <= 4 * 4 * AQ_THREADS)
        e = launch_kernel(rmsnorm_act_quant_kernel<T, 4>, grid, block, 0, st, (const T *)x, weight, eps, K, h_out, q_plain, q_perm, scale, rowsum);
    else
        e = launch_kernel(rmsnorm_act_quant_kernel<T, 12>, grid, block, 0, st, (const T *)x, weight, eps, K, h_out, q_plain, q_perm, scale, rowsum);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "rmsnorm_act_quant_kernel: %s", cudaGetErrorString(e));
    return check_launch("rmsnorm_act_quant_kernel");
}

int rmsnorm_act_quant_dispatch(const void *x, int x_dtype, const float *weight, double eps, int64_t M, int64_t K,
                               float *h_out, int8_t *q_plain, int8_t *q_perm, float *scale, int32_t *rowsum, cudaStream_t st)
{
    if (!x || !weight || !scale) return fail(NSLQ_ERR_ARG, "nslq_rmsnorm_act_quant_i8: null x, weight or scale");
    if (M < 0 || K <= 0 || M > 0x7fffffffLL) return fail(NSLQ_ERR_SHAPE, "nslq_rmsnorm_act_quant_i8: bad M=%lld K=%lld", (long long)M, (long long)K);
    if (K % 16 != 0 || K > 12 * 4 * AQ_THREADS)
        return fail(NSLQ_ERR_SHAPE, "nslq_rmsnorm_act_quant_i8: K=%lld must be a multiple of 16 and at most %d", (long long)K, 12 * 4 * AQ_THREADS);
    if (!aligned16(x) || !aligned16(weight) || (h_out && !aligned16(h_out)) || (q_plain && !aligned16(q_plain)) || (q_perm && !aligned16(q_perm)))
        return fail(NSLQ_ERR_ARG, "nslq_rmsnorm_act_quant_i8: buffers must be 16-byte aligned");
    if (M == 0) return NSLQ_OK;
    switch (x_dtype) {
    case NSLQ_DTYPE_F32: return launch_rmsnorm_quant<float>(x, weight, eps, M, K, h_out, q_plain, q_perm, scale, rowsum, st);
    case NSLQ_DTYPE_FP16: return launch_rmsnorm_quant<__half>(x, weight, eps, M, K, h_out, q_plain, q_perm, scale, rowsum, st);
    case NSLQ_DTYPE_BF16: return launch_rmsnorm_quant<__nv_bfloat16>(x, weight, eps, M, K, h_out, q_plain, q_perm, scale, rowsum, st);
    default: return fail(NSLQ_ERR_ARG, "nslq_rmsnorm_act_quant_i8: x_dtype %d not in {F32,FP16,BF16}", x_dtype);
    }
}

// SiLU(gate) * up fused in front of the quantisation of the down projection's input (the other
// "fused neighbour" of the linear: gate and up never make a round trip as an activation tensor):
//   h = (f32)( g / (1 + exp(-g)) * u )    computed in fp32 from the f32/fp16/bf16 inputs,
// then quantised from registers like act_quant_kernel.  One CTA per row.
template <typename T, int XV>
__global__ void __launch_bounds__(AQ_THREADS)
swiglu_act_quant_kernel(const T *__restrict__ gate, const T *__restrict__ up, int64_t K, int64_t ld_g, int64_t ld_u,
                        float *__restrict__ h_out,
                        int8_t *__restrict__ q_plain, int8_t *__restrict__ q_perm, float *__restrict__ scale_out,
                        int32_t *__restrict__ rowsum_out)
{
    __shared__ float smax[AQ_THREADS / 32];
    __shared__ int ssum[AQ_THREADS / 32];
    const int64_t r = blockIdx.x;
    pdl_wait();
    const int nvec = (int)(K >> 2);
    float4 hv[XV];
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < XV; ++i) {
        const int v = i * AQ_THREADS + threadIdx.x;
        hv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (v < nvec) {
            const float4 g = Vec4<T>::load(gate + r * ld_g, v), u = Vec4<T>::load(up + r * ld_u, v);
            float4 h;
            h.x = __fdiv_rn(g.x, 1.0f + expf(-g.x)) * u.x; h.y = __fdiv_rn(g.y, 1.0f + expf(-g.y)) * u.y;
            h.z = __fdiv_rn(g.z, 1.0f + expf(-g.z)) * u.z; h.w = __fdiv_rn(g.w, 1.0f + expf(-g.w)) * u.w;
            hv[i] = h;
            if (h_out) reinterpret_cast<float4 *>(h_out + r * K)[v] = h;
            m = fmaxf(m, fmaxf(fmaxf(fabsf(h.x), fabsf(h.y)), fmaxf(fabsf(h.z), fabsf(h.w))));
        }
    }
    const float scale = block_max(m, smax);
    pdl_launch_dependents();
    const float inv = __fdiv_rn(127.0f, scale);
    int sum = 0;
#pragma unroll
    for (int i = 0; i < XV; ++i) {
        const int v = i * AQ_THREADS + threadIdx.x;
        const bool in = v < nvec;
        const unsigned mask = __ballot_sync(0xffffffffu, in);          // whole quads: K % 16 == 0
        if (in) {
            const float4 f = hv[i];
            const uint32_t w = pack4_i8(quant_one(f.x, inv), quant_one(f.y, inv), quant_one(f.z, inv), quant_one(f.w, inv));
            sum = __dp4a((int)w, 0x01010101, sum);
            if (q_plain) reinterpret_cast<uint32_t *>(q_plain + r * K)[v] = w;
            if (q_perm) reinterpret_cast<uint32_t *>(q_perm + r * K)[v] = quad_transpose(w, mask);
        }
    }
    if (rowsum_out) {
        const int tot = block_sum(sum, ssum);
        if (threadIdx.x == 0) rowsum_out[r] = tot;
    }
    if (threadIdx.x == 0) scale_out[r] = scale;
}

template <typename T>
static int launch_swiglu_quant(const void *gate, const void *up, int64_t M, int64_t K, int64_t ld_g, int64_t ld_u, float *h_out, int8_t *q_plain,
                               int8_t *q_perm, float *scale, int32_t *rowsum, cudaStream_t st)
{
    dim3 grid((unsigned)M), block(AQ_THREADS);
    cudaError_t e;
    if (K <= 4 * 4 * AQ_THREADS)
        e = launch_kernel(swiglu_act_quant_kernel<T, 4>, grid, block, 0, st, (const T *)gate, (const T *)up, K, ld_g, ld_u, h_out, q_plain, q_perm, scale, rowsum);
    else
        e = launch_kernel(swiglu_act_quant_kernel<T, 12>, grid, block, 0, st, (const T *)gate, (const T *)up, K, ld_g, ld_u, h_out, q_plain, q_perm, scale, rowsum);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "swiglu_act_quant_kernel: %s", cudaGetErrorString(e));
    return check_launch("swiglu_act_quant_kernel");
}

int swiglu_act_quant_dispatch(const void *gate, const void *up, int dtype, int64_t M, int64_t K, int64_t ld_g, int64_t ld_u,
                              float *h_out,
                              int8_t *q_plain, int8_t *q_perm, float *scale, int32_t *rowsum, cudaStream_t st)
{
    if (!gate || !up || !scale) return fail(NSLQ_ERR_ARG, "nslq_swiglu_act_quant_i8: null gate, up or scale");
    if (M < 0 || K <= 0 || M > 0x7fffffffLL) return fail(NSLQ_ERR_SHAPE, "nslq_swiglu_act_quant_i8: bad M=%lld K=%lld", (long long)M, (long long)K);
    if (K % 16 != 0 || K > 12 * 4 * AQ_THREADS)
        return fail(NSLQ_ERR_SHAPE, "nslq_swiglu_act_quant_i8: K=%lld must be a multiple of 16 and at most %d", (long long)K, 12 * 4 * AQ_THREADS);
    if (!aligned16(gate) || !aligned16(up) || (h_out && !aligned16(h_out)) || (q_plain && !aligned16(q_plain)) || (q_perm && !aligned16(q_perm)))
        return fail(NSLQ_ERR_ARG, "nslq_swiglu_act_quant_i8: buffers must be 16-byte aligned");
    const int64_t es = dtype == NSLQ_DTYPE_F32 ? 4 : 2;
    if (ld_g < K || ld_u < K || (ld_g * es) % 16 != 0 || (ld_u * es) % 16 != 0)
        return fail(NSLQ_ERR_SHAPE, "nslq_swiglu_act_quant_i8: row strides must be at least K and keep rows 16-byte aligned");
    if (M == 0) return NSLQ_OK;
    switch (dtype) {
    case NSLQ_DTYPE_F32: return launch_swiglu_quant<float>(gate, up, M, K, ld_g, ld_u, h_out, q_plain, q_perm, scale, rowsum, st);
    case NSLQ_DTYPE_FP16: return launch_swiglu_quant<__half>(gate, up, M, K, ld_g, ld_u, h_out, q_plain, q_perm, scale, rowsum, st);
    case NSLQ_DTYPE_BF16: return launch_swiglu_quant<__nv_bfloat16>(gate, up, M, K, ld_g, ld_u, h_out, q_plain, q_perm, scale, rowsum, st);
    default: return fail(NSLQ_ERR_ARG, "nslq_swiglu_act_quant_i8: dtype %d not in {F32,FP16,BF16}", dtype);
    }
}

template <typename T>
static int launch_act_quant(const void *x, int64_t M, int64_t K, int8_t *q_plain, int8_t *q_perm,
                            float *scale, int32_t *rowsum, cudaStream_t st)
{
    const bool vec = (K % 16 == 0) && aligned16(x) && (!q_plain || aligned16(q_plain)) &&
                     (!q_perm || aligned16(q_perm));
    if (q_perm && !vec)
        return fail(NSLQ_ERR_SHAPE, "nslq_act_quant_i8: q_perm needs K %% 16 == 0 and 16-byte aligned buffers (K=%lld)",
                    (long long)K);
    dim3 grid((unsigned)M), block(AQ_THREADS);
    cudaError_t e;
    if (!vec) e = launch_kernel(act_quant_kernel<T, false, 1>, grid, block, 0, st, (const T *)x, K, q_plain, q_perm, scale, rowsum);
    else if (K <= 4 * 4 * AQ_THREADS) e = launch_kernel(act_quant_kernel<T, true, 4>, grid, block, 0, st, (const T *)x, K, q_plain, q_perm, scale, rowsum);
    else e = launch_kernel(act_quant_kernel<T, true, 12>, grid, block, 0, st, (const T *)x, K, q_plain, q_perm, scale, rowsum);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "act_quant_kernel: %s", cudaGetErrorString(e));
    return check_launch("act_quant_kernel");
}

int act_quant_dispatch(const void *x, int x_dtype, int64_t M, int64_t K, int8_t *q_plain, int8_t *q_perm,
                       float *scale, int32_t *rowsum, cudaStream_t st)
{
    if (!x || !scale) return fail(NSLQ_ERR_ARG, "nslq_act_quant_i8: null x or scale");
    if (M < 0 || K <= 0 || M > 0x7fffffffLL) return fail(NSLQ_ERR_SHAPE, "nslq_act_quant_i8: bad M=%lld K=%lld", (long long)M, (long long)K);
    if (M == 0) return NSLQ_OK;
    switch (x_dtype) {
    case NSLQ_DTYPE_F32: return launch_act_quant<float>(x, M, K, q_plain, q_perm, scale, rowsum, st);
    case NSLQ_DTYPE_FP16: return launch_act_quant<__half>(x, M, K, q_plain, q_perm, scale, rowsum, st);
    case NSLQ_DTYPE_BF16: return launch_act_quant<__nv_bfloat16>(x, M, K, q_plain, q_perm, scale, rowsum, st);
    default: return fail(NSLQ_ERR_ARG, "nslq_act_quant_i8: x_dtype %d not in {F32,FP16,BF16}", x_dtype);
    }
}

}  // namespace nslq
