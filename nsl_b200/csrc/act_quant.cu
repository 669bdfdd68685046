// Stage 1: per-token absmax int8 activation quantisation.
//
// One CTA per token row.  The row is read once into registers, each thread holding whole
// groups of 16 consecutive elements; max|x| is reduced with warp shuffles (then across warps
// through shared memory); the row is then quantised from registers with the reference's exact
// arithmetic and written in the natural order and/or the order the matmul kernels consume
// (16-byte stores assembled in registers), plus scale and sum.
//
// Arithmetic follows crates/nsl-codegen/tests/bitnet_reference_impl.rs:46-70 of
// NSL: inv = 127/scale (IEEE divide), v = x*inv, clamp to [-127,127], round half
// away from zero, NaN -> 0.
#include <cooperative_groups.h>

#include "common.cuh"
#include "quant_core.cuh"

namespace nslq {

namespace cg = cooperative_groups;

constexpr int AQ_THREADS = 256;

static __device__ __forceinline__ float block_max(float v, float *smem)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) smem[w] = v;
    __syncthreads();
    float r = (l < (int)(blockDim.x >> 5)) ? smem[l] : 0.0f;
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
    int r = (l < (int)(blockDim.x >> 5)) ? smem[l] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

// One group of 16 quantised and stored: natural order and/or the order the matmul kernels consume
// (position 4i+j of the group holds k = 4j+i), one 16-byte store each; returns the sum of the 16.
// FAST: inv is finite, so |x*inv| <= 127*(1+2^-23) for every element of the row and
//   trunc(s + copysign(0.49999997, s)) == round-half-away(s)
// holds for every float |s| <= 200 (checked over all of them on the CPU): below 0.5 the sum stays
// below 1, at a tie k+0.5 it rounds up to k+1 exactly, elsewhere it stays inside [k, k+1).  Four
// instructions per element, no compare, no clamp.  The other rows (scale 0, or so small that
// 127/scale overflows) take quant_one, which saturates and maps NaN to 0 like the reference.
template <bool FAST>
static __device__ __forceinline__ int quant_group(const float (&f)[16], float inv, int8_t *q_plain_row, int8_t *q_perm_row, int g)
{
    int q[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        if (FAST) {
            const float s = __fmul_rn(f[e], inv);
            const float h = __int_as_float((__float_as_int(s) & 0x80000000) | 0x3effffff);
            q[e] = __float2int_rz(__fadd_rn(s, h));
        } else {
            q[e] = quant_one(f[e], inv);
        }
    }
    uint4 pw;
    pw.x = pack4_sat(q[0], q[4], q[8], q[12]);
    pw.y = pack4_sat(q[1], q[5], q[9], q[13]);
    pw.z = pack4_sat(q[2], q[6], q[10], q[14]);
    pw.w = pack4_sat(q[3], q[7], q[11], q[15]);
    if (q_perm_row) reinterpret_cast<uint4 *>(q_perm_row)[g] = pw;
    if (q_plain_row) {
        uint4 nw;
        nw.x = pack4_sat(q[0], q[1], q[2], q[3]);
        nw.y = pack4_sat(q[4], q[5], q[6], q[7]);
        nw.z = pack4_sat(q[8], q[9], q[10], q[11]);
        nw.w = pack4_sat(q[12], q[13], q[14], q[15]);
        reinterpret_cast<uint4 *>(q_plain_row)[g] = nw;
    }
    int sum = __dp4a((int)pw.x, 0x01010101, 0);
    sum = __dp4a((int)pw.y, 0x01010101, sum);
    sum = __dp4a((int)pw.z, 0x01010101, sum);
    return __dp4a((int)pw.w, 0x01010101, sum);
}

// VEC = true: K % 16 == 0 and 16-byte aligned rows; a thread owns whole groups of 16 consecutive
// elements, so both output orders are assembled in registers and stored 16 bytes at a time: no
// shuffles, no lane masks.  (The kernel is bound by issued instructions, not by HBM, as long as it
// spends more than about eight per element.)
template <typename T, bool VEC, int XG, int NT = AQ_THREADS>
__global__ void __launch_bounds__(NT)
act_quant_kernel(const T *__restrict__ x, int64_t K, int8_t *__restrict__ q_plain,
                 int8_t *__restrict__ q_perm, float *__restrict__ scale_out,
                 int32_t *__restrict__ rowsum_out)
{
    __shared__ float smax[NT / 32];
    __shared__ int ssum[NT / 32];
    const int64_t r = blockIdx.x;
    const T *row = x + r * K;
    pdl_wait();

    // VEC path: the thread's groups stay in registers between the absmax pass and the rounding pass
    // (XG groups per thread: K <= XG*16*NT; longer rows re-read the tail, which is still in
    // L1/L2).  XG is 1 or 3: short rows keep registers low so that more rows are in flight per SM.
    const int ngrp = VEC ? (int)(K >> 4) : 0;
    float xv[VEC ? XG : 1][16];
    float m = 0.0f;
    if (VEC) {
#pragma unroll
        for (int i = 0; i < XG; ++i) {
            const int g = i * NT + threadIdx.x;
            if (g < ngrp) Group16<T>::load(row, g, xv[i]);
            else {
#pragma unroll
                for (int e = 0; e < 16; ++e) xv[i][e] = 0.0f;
            }
        }
#pragma unroll
        for (int i = 0; i < XG; ++i) m = absmax16(xv[i], m);
        for (int g = XG * NT + threadIdx.x; g < ngrp; g += NT) {
            float f[16];
            Group16<T>::load(row, g, f);
            m = absmax16(f, m);
        }
    } else {
        for (int64_t k = threadIdx.x; k < K; k += NT) m = fmaxf(m, fabsf(Elem<T>::to_f32(row[k])));
    }
    const float scale = block_max(m, smax);
    pdl_launch_dependents();
    const float inv = __fdiv_rn(127.0f, scale);
    const bool zero_row = (scale == 0.0f);

    int sum = 0;
    if (VEC) {
        int8_t *pl = q_plain ? q_plain + r * K : nullptr, *pp = q_perm ? q_perm + r * K : nullptr;
        if (inv < INFINITY) {                              // CTA-uniform; false for inf and NaN
#pragma unroll
            for (int i = 0; i < XG; ++i) {
                const int g = i * NT + threadIdx.x;
                if (g < ngrp) sum += quant_group<true>(xv[i], inv, pl, pp, g);
            }
            for (int g = XG * NT + threadIdx.x; g < ngrp; g += NT) {
                float f[16];
                Group16<T>::load(row, g, f);
                sum += quant_group<true>(f, inv, pl, pp, g);
            }
        } else {
            for (int g = threadIdx.x; g < ngrp; g += NT) {
                float f[16];
                Group16<T>::load(row, g, f);
                sum += quant_group<false>(f, inv, pl, pp, g);
            }
        }
    } else {
        for (int64_t k = threadIdx.x; k < K; k += NT) {
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
    // Short rows: the norm weights are fetched now, not behind the reduction (a second memory round trip
    // in a kernel that is one latency chain).  Long rows have no registers to spare for that.
    constexpr bool WPRE = XV <= 4;
    float4 wv[WPRE ? XV : 1];
    if (WPRE) {
#pragma unroll
        for (int i = 0; i < XV; ++i) {
            const int v = i * AQ_THREADS + threadIdx.x;
            wv[i] = (v < nvec) ? __ldg(reinterpret_cast<const float4 *>(weight) + v) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
#pragma unroll
    for (int i = 0; i < XV; ++i)
        sq += (double)xv[i].x * xv[i].x + (double)xv[i].y * xv[i].y + (double)xv[i].z * xv[i].z + (double)xv[i].w * xv[i].w;
    const double rms = sqrt(block_sum_f64(sq, ssq) / (double)K + eps);
    const double rinv = __drcp_rn(rms);
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < XV; ++i) {
        const int v = i * AQ_THREADS + threadIdx.x;
        if (v < nvec) {
            const float4 w = WPRE ? wv[WPRE ? i : 0] : reinterpret_cast<const float4 *>(weight)[v];
            const float4 h = norm_four(xv[i], rms, rinv, w);
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
//   h = (f32)( g / (1 + exp(-g)) * u )    computed in fp32 from the f32/fp16/bf16 inputs (swiglu_one),
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
            h.x = swiglu_one(g.x, u.x); h.y = swiglu_one(g.y, u.y);
            h.z = swiglu_one(g.z, u.z); h.w = swiglu_one(g.w, u.w);
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

// Up to 64 rows (decode): one CTA per row is a long serial chain (K exp/divide pairs on 256 threads)
// on one of 148 SMs.  Here a cluster of CL CTAs shares a row: every CTA forms and keeps K/CL products
// (at most one group of 16 per thread), the row maximum is exchanged through the cluster's shared
// memory, and rank 0 adds up the partial row sums.  Same arithmetic, same bits as the kernel above.
constexpr int SQC_THREADS = 128;
template <typename T, int CL>
__global__ void __launch_bounds__(SQC_THREADS)
swiglu_act_quant_cluster_kernel(const T *__restrict__ gate, const T *__restrict__ up, int64_t K, int64_t ld_g, int64_t ld_u,
                                float *__restrict__ h_out, int8_t *__restrict__ q_plain, int8_t *__restrict__ q_perm,
                                float *__restrict__ scale_out, int32_t *__restrict__ rowsum_out)
{
    __shared__ float wmax[SQC_THREADS / 32];
    __shared__ int wsum[SQC_THREADS / 32];
    __shared__ float cmax;                // this CTA's maximum, read by its peers
    __shared__ int csum[CL];              // rank 0's copy collects every CTA's partial row sum
    cg::cluster_group cl = cg::this_cluster();
    const int64_t r = blockIdx.x / CL;
    const int rank = blockIdx.x % CL, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_wait();
    const int ngrp = (int)(K >> 4), per = (ngrp + CL - 1) / CL;          // per <= SQC_THREADS (checked by the host)
    const int g = rank * per + (int)threadIdx.x;
    const bool active = (int)threadIdx.x < per && g < ngrp;
    float h[16];
    float m = 0.0f;
    if (active) {
        float gv[16], uv[16];
        Group16<T>::load(gate + r * ld_g, g, gv);
        Group16<T>::load(up + r * ld_u, g, uv);
#pragma unroll
        for (int e = 0; e < 16; ++e) h[e] = swiglu_one(gv[e], uv[e]);
        if (h_out) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                reinterpret_cast<float4 *>(h_out + r * K)[4 * g + j] = make_float4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
        }
        m = absmax16(h, m);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) wmax[warp] = m;
    __syncthreads();
    if (threadIdx.x == 0) cmax = fmaxf(fmaxf(wmax[0], wmax[1]), fmaxf(wmax[2], wmax[3]));
    cl.sync();                            // every CTA's maximum is published (and every CTA is running)
    float scale = 0.0f;
#pragma unroll
    for (int c = 0; c < CL; ++c) scale = fmaxf(scale, *cl.map_shared_rank(&cmax, c));
    pdl_launch_dependents();
    const float inv = __fdiv_rn(127.0f, scale);
    int sum = 0;
    if (active) {
        int8_t *pl = q_plain ? q_plain + r * K : nullptr, *pp = q_perm ? q_perm + r * K : nullptr;
        sum = inv < INFINITY ? quant_group<true>(h, inv, pl, pp, g) : quant_group<false>(h, inv, pl, pp, g);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) wsum[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) *cl.map_shared_rank(&csum[rank], 0) = wsum[0] + wsum[1] + wsum[2] + wsum[3];
    cl.sync();                            // peers stay alive until every remote read of cmax is done; partial sums have landed
    if (rank == 0 && threadIdx.x == 0) {
        int tot = 0;
#pragma unroll
        for (int c = 0; c < CL; ++c) tot += csum[c];
        if (rowsum_out) rowsum_out[r] = tot;
        scale_out[r] = scale;
    }
}

template <typename T>
static int launch_swiglu_quant(const void *gate, const void *up, int64_t M, int64_t K, int64_t ld_g, int64_t ld_u, float *h_out, int8_t *q_plain,
                               int8_t *q_perm, float *scale, int32_t *rowsum, cudaStream_t st)
{
    dim3 grid((unsigned)M), block(AQ_THREADS);
    cudaError_t e;
    constexpr int CL = 8;
    if (M <= 64 && K <= (int64_t)16 * SQC_THREADS * CL) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(M * CL));
        cfg.blockDim = dim3(SQC_THREADS);
        cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = CL;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = g_use_pdl ? 2 : 1;
        e = cudaLaunchKernelEx(&cfg, swiglu_act_quant_cluster_kernel<T, CL>, (const T *)gate, (const T *)up, K, ld_g, ld_u, h_out, q_plain,
                               q_perm, scale, rowsum);
        if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "swiglu_act_quant_cluster_kernel: %s", cudaGetErrorString(e));
        return check_launch("swiglu_act_quant_cluster_kernel");
    }
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
    else if (M >= 1024 && K > 16 * 128 && K <= 2 * 16 * 128)
        // many medium rows (a prefill): CTAs of 128 threads with two groups per thread keep more rows in flight per SM and
        // halve the block reductions per byte
        e = launch_kernel(act_quant_kernel<T, true, 2, 128>, grid, dim3(128), 0, st, (const T *)x, K, q_plain, q_perm, scale, rowsum);
    else if (M >= 1024 && K > 2 * 16 * 192 && K <= 3 * 16 * 192)
        e = launch_kernel(act_quant_kernel<T, true, 3, 192>, grid, dim3(192), 0, st, (const T *)x, K, q_plain, q_perm, scale, rowsum);
    else if (K <= 16 * AQ_THREADS) e = launch_kernel(act_quant_kernel<T, true, 1>, grid, block, 0, st, (const T *)x, K, q_plain, q_perm, scale, rowsum);
    else e = launch_kernel(act_quant_kernel<T, true, 3>, grid, block, 0, st, (const T *)x, K, q_plain, q_perm, scale, rowsum);
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
