// The launches around the quantized linears and the attention of a decoder: for a decode step the embedding
// rows of the current tokens, the RMSNorm in front of the output head and the greedy choice of the next
// token, so that a step of the harness is library launches from the first to the last (the head's bf16 GEMM
// aside); for the prompt the rotary embedding and the cache writes.  Each restates a runtime function of NSL
// as one launch:
//
//   nslq_embed_gather   nsl_tensor_embedding_lookup  crates/nsl-runtime/src/tensor/mod.rs:2592-2680
//   nslq_rmsnorm_rows   nsl_tensor_rmsnorm           crates/nsl-runtime/src/tensor/mod.rs:3016-3035
//   nslq_argmax_rows    nsl_tensor_argmax            crates/nsl-runtime/src/sampling.rs:322-400
//
//   nslq_rope_kv_prefill  RotaryEmbedding.forward + the cache writes of a prompt   stdlib/nsl/nn/rope.nsl:41-68
//
// The first three are one CTA per row and bound by launch latency at decode sizes; the last is one CTA per prompt token.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "quant_core.cuh"

namespace nslq {

static __device__ int g_glue_status = 0;      // 0xA01: a token id outside the embedding table

template <typename T> static __device__ __forceinline__ float elem_to_float(T v);
template <> __device__ __forceinline__ float elem_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float elem_to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float elem_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// out[r, :] = (f32) table[tokens[r], :].  The reference checks host-resident ids and aborts; ids that live
// on the device cannot be checked by the host without a synchronisation, so the kernel checks them: a row
// whose id is out of range becomes zeros and the status word says so.
template <typename T>
__global__ void __launch_bounds__(256) embed_gather_kernel(const T *__restrict__ table, int64_t V, int64_t H,
                                                           const int64_t *__restrict__ tokens, float *__restrict__ out)
{
    pdl_wait();
    const int64_t r = blockIdx.x;
    const int64_t tok = tokens[r];
    const bool ok = tok >= 0 && tok < V;
    if (!ok && threadIdx.x == 0) atomicCAS(&g_glue_status, 0, 0xA01);
    const T *row = table + (ok ? tok : 0) * H;
    for (int64_t i = threadIdx.x; i < H; i += blockDim.x) out[r * H + i] = ok ? elem_to_float(row[i]) : 0.0f;
    pdl_launch_dependents();
}

// y[r, k] = (out dtype)(f32)(x[r,k] / rms * w[k]), rms = sqrt(mean x^2 + eps) in f64: the arithmetic of
// nslq_rmsnorm_act_quant_i8's normalisation (tree sum of squares), rounded once more when y is 16-bit.
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float *__restrict__ x, const float *__restrict__ w, double eps,
                                                           int64_t K, void *__restrict__ y, int y_dtype)
{
    __shared__ double part[8];
    pdl_wait();
    const int64_t r = blockIdx.x;
    const float *row = x + r * K;
    double sq = 0.0;
    for (int64_t i = threadIdx.x; i < K; i += 256) sq += (double)row[i] * (double)row[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = sq;
    __syncthreads();
    const double tot = sum_partials<8>(part, 1);
    const double rms = sqrt(tot / (double)K + eps), rinv = __drcp_rn(rms);
    for (int64_t i = threadIdx.x; i < K; i += 256) store_out(y, y_dtype, r * K + i, norm_one(row[i], rms, rinv, w[i]));
    pdl_launch_dependents();
}

// out[r] = the lowest index of the largest element of row r; a NaN never wins and a row without any
// element above -inf gives 0 (the reference's loop: `if v > best` from -inf, index 0).  `counter`, when
// given, is advanced by one by the first CTA: the position of a decode loop, which lives on the device.
constexpr int AM_THREADS = 1024;
template <typename T>
__global__ void __launch_bounds__(AM_THREADS) argmax_rows_kernel(const T *__restrict__ x, int64_t V, int64_t ld, int64_t *__restrict__ out,
                                                                 int64_t *__restrict__ counter)
{
    __shared__ float sval[AM_THREADS / 32];
    __shared__ int64_t sidx[AM_THREADS / 32];
    pdl_wait();
    const int64_t r = blockIdx.x;
    const T *row = x + r * ld;
    float best = -INFINITY;
    int64_t bi = INT64_MAX;
    for (int64_t i = threadIdx.x; i < V; i += AM_THREADS) {
        const float v = elem_to_float(row[i]);
        if (v > best) { best = v; bi = i; }
    }
    auto merge = [&](float ov, int64_t oi) {
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int64_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        merge(ov, oi);
    }
    if ((threadIdx.x & 31) == 0) { sval[threadIdx.x >> 5] = best; sidx[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = sval[threadIdx.x];
        bi = sidx[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int64_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            merge(ov, oi);
        }
        if (threadIdx.x == 0) {
            out[r] = bi == INT64_MAX ? 0 : bi;
            if (counter && r == 0) *counter += 1;
        }
    }
    pdl_launch_dependents();
}

// Prefill: RoPE of the prompt's queries (in place) and keys, and the keys and values written into the cache, one
// launch instead of the framework's slice / multiply / concatenate / copy kernels.  x * cos + rotate_half(x) * sin
// with table = concat(freqs, freqs) (stdlib/nsl/nn/rope.nsl:41-68): for i < D/2
//   out[i]       = x[i] * cos[t, i]       - x[i + D/2] * sin[t, i]
//   out[i + D/2] = x[i + D/2] * cos[t, i] + x[i]       * sin[t, i]
// each product and the sum rounded separately in fp32, then once to bf16 (the same bits as the expression
// evaluated operation by operation on fp32 tensors).  One CTA per token; q, k, v are token rows [B*T, heads*D].
// One rotated pair (d, d + D/2) from the inputs x1 = x[d], x2 = x[d + D/2].
static __device__ __forceinline__ void rope_pair(float x1, float x2, float c, float sn, float &lo, float &hi)
{
    lo = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, sn));
    hi = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, sn));
}

// VEC: D/2 and the row strides are even and every base pointer 4-byte aligned, so a thread takes two neighbouring
// dimensions with 4-byte accesses (8-byte for the tables).
template <bool VEC>
__global__ void __launch_bounds__(256) rope_kv_prefill_kernel(__nv_bfloat16 *__restrict__ q, const __nv_bfloat16 *__restrict__ k,
                                                              const __nv_bfloat16 *__restrict__ v, int64_t q_ld, int64_t k_ld, int64_t v_ld,
                                                              __nv_bfloat16 *__restrict__ k_cache, __nv_bfloat16 *__restrict__ v_cache,
                                                              const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                                                              int T, int64_t pos0, int H, int Hkv, int D, int64_t max_ctx)
{
    pdl_wait();
    const int64_t row = blockIdx.x;
    const int64_t b = row / T, t = pos0 + row % T;
    const int half = D >> 1;
    const float *cr = cos_t + t * half, *sr = sin_t + t * half;
    __nv_bfloat16 *qr = q + row * q_ld;
    const __nv_bfloat16 *kr = k + row * k_ld, *vr = v + row * v_ld;
    if (VEC) {
        const int hp = half >> 1;                             // pairs of neighbouring dimensions per half
        for (int i = threadIdx.x; i < (H + Hkv) * hp; i += 256) {
            const int h = i / hp, d = 2 * (i % hp);
            const bool isq = h < H;
            const __nv_bfloat16 *src = isq ? qr + h * D : kr + (h - H) * D;
            __nv_bfloat16 *dst = isq ? qr + h * D : k_cache + ((b * Hkv + (h - H)) * max_ctx + t) * D;
            const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(src + d));
            const float2 x2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(src + d + half));
            const float2 c = *reinterpret_cast<const float2 *>(cr + d), sn = *reinterpret_cast<const float2 *>(sr + d);
            float2 lo, hi;
            rope_pair(x1.x, x2.x, c.x, sn.x, lo.x, hi.x);
            rope_pair(x1.y, x2.y, c.y, sn.y, lo.y, hi.y);
            *reinterpret_cast<__nv_bfloat162 *>(dst + d) = __floats2bfloat162_rn(lo.x, lo.y);
            *reinterpret_cast<__nv_bfloat162 *>(dst + d + half) = __floats2bfloat162_rn(hi.x, hi.y);
        }
        for (int i = threadIdx.x; i < Hkv * half; i += 256) {  // values: 4-byte copies (D is a multiple of 4 here)
            const int h = i / half, d = 2 * (i % half);
            *reinterpret_cast<uint32_t *>(v_cache + ((b * Hkv + h) * max_ctx + t) * D + d) =
                *reinterpret_cast<const uint32_t *>(vr + h * D + d);
        }
    } else {
        for (int i = threadIdx.x; i < (H + Hkv) * half; i += 256) {
            const int h = i / half, d = i % half;
            const bool isq = h < H;
            const __nv_bfloat16 *src = isq ? qr + h * D : kr + (h - H) * D;
            __nv_bfloat16 *dst = isq ? qr + h * D : k_cache + ((b * Hkv + (h - H)) * max_ctx + t) * D;
            float lo, hi;
            rope_pair(__bfloat162float(src[d]), __bfloat162float(src[d + half]), cr[d], sr[d], lo, hi);
            dst[d] = __float2bfloat16_rn(lo);
            dst[d + half] = __float2bfloat16_rn(hi);
        }
        for (int i = threadIdx.x; i < Hkv * D; i += 256) {
            const int h = i / D, d = i % D;
            v_cache[((b * Hkv + h) * max_ctx + t) * D + d] = vr[i];
        }
    }
    pdl_launch_dependents();
}

int decode_glue_status(int *out)
{
    int v = 0;
    const int zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_glue_status, sizeof(int)) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "decode_glue_status: %s", cudaGetErrorString(cudaGetLastError()));
    if (v != 0) cudaMemcpyToSymbol(g_glue_status, &zero, sizeof(int));
    *out = v;
    return NSLQ_OK;
}

}  // namespace nslq

using namespace nslq;

extern "C" {

int nslq_embed_gather(const void *table, int table_dtype, int64_t V, int64_t H, const int64_t *tokens, int64_t B, float *out, void *stream)
{
    if (!table || !tokens || !out) return fail(NSLQ_ERR_ARG, "nslq_embed_gather: null argument");
    if (V <= 0 || H <= 0 || B < 0 || B > 0x7fffffffLL) return fail(NSLQ_ERR_SHAPE, "nslq_embed_gather: V=%lld H=%lld B=%lld", (long long)V, (long long)H, (long long)B);
    if (B == 0) return NSLQ_OK;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    switch (table_dtype) {
    case NSLQ_DTYPE_F32: e = launch_kernel(embed_gather_kernel<float>, dim3((unsigned)B), dim3(256), 0, st, (const float *)table, V, H, tokens, out); break;
    case NSLQ_DTYPE_FP16: e = launch_kernel(embed_gather_kernel<__half>, dim3((unsigned)B), dim3(256), 0, st, (const __half *)table, V, H, tokens, out); break;
    case NSLQ_DTYPE_BF16: e = launch_kernel(embed_gather_kernel<__nv_bfloat16>, dim3((unsigned)B), dim3(256), 0, st, (const __nv_bfloat16 *)table, V, H, tokens, out); break;
    default: return fail(NSLQ_ERR_ARG, "nslq_embed_gather: table dtype %d not in {F32,FP16,BF16}", table_dtype);
    }
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "embed_gather_kernel: %s", cudaGetErrorString(e));
    return check_launch("embed_gather_kernel");
}

int nslq_rmsnorm_rows(const float *x, const float *weight, double eps, int64_t M, int64_t K, void *y, int y_dtype, void *stream)
{
    if (!x || !weight || !y) return fail(NSLQ_ERR_ARG, "nslq_rmsnorm_rows: null argument");
    if (M < 0 || K <= 0 || M > 0x7fffffffLL) return fail(NSLQ_ERR_SHAPE, "nslq_rmsnorm_rows: M=%lld K=%lld", (long long)M, (long long)K);
    if (y_dtype != NSLQ_DTYPE_F32 && y_dtype != NSLQ_DTYPE_FP16 && y_dtype != NSLQ_DTYPE_BF16)
        return fail(NSLQ_ERR_ARG, "nslq_rmsnorm_rows: y dtype %d not in {F32,FP16,BF16}", y_dtype);
    if (M == 0) return NSLQ_OK;
    const cudaError_t e = launch_kernel(rmsnorm_rows_kernel, dim3((unsigned)M), dim3(256), 0, (cudaStream_t)stream, x, weight, eps, K, y, y_dtype);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "rmsnorm_rows_kernel: %s", cudaGetErrorString(e));
    return check_launch("rmsnorm_rows_kernel");
}

int nslq_rope_kv_prefill(void *q, const void *k, const void *v, int64_t q_ld, int64_t k_ld, int64_t v_ld, void *k_cache, void *v_cache,
                         const float *cos_t, const float *sin_t, int64_t B, int64_t T, int64_t pos0, int64_t H, int64_t Hkv, int64_t D,
                         int64_t max_ctx, void *stream)
{
    if (!q || !k || !v || !k_cache || !v_cache || !cos_t || !sin_t) return fail(NSLQ_ERR_ARG, "nslq_rope_kv_prefill: null argument");
    if (B <= 0 || T <= 0 || H <= 0 || Hkv <= 0 || D <= 0 || D % 2 != 0 || pos0 < 0 || pos0 + T > max_ctx || B * T > 0x7fffffffLL ||
        q_ld < H * D || k_ld < Hkv * D || v_ld < Hkv * D)
        return fail(NSLQ_ERR_SHAPE, "nslq_rope_kv_prefill: B=%lld T=%lld pos0=%lld H=%lld Hkv=%lld D=%lld (even) max_ctx=%lld, row strides %lld %lld %lld",
                    (long long)B, (long long)T, (long long)pos0, (long long)H, (long long)Hkv, (long long)D, (long long)max_ctx,
                    (long long)q_ld, (long long)k_ld, (long long)v_ld);
    auto al = [](const void *p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; };
    const bool vec = D % 4 == 0 && q_ld % 2 == 0 && k_ld % 2 == 0 && v_ld % 2 == 0 && al(q, 4) && al(k, 4) && al(v, 4) && al(k_cache, 4) &&
                     al(v_cache, 4) && al(cos_t, 8) && al(sin_t, 8);
    const cudaError_t e = launch_kernel(vec ? rope_kv_prefill_kernel<true> : rope_kv_prefill_kernel<false>, dim3((unsigned)(B * T)), dim3(256),
                                        0, (cudaStream_t)stream, (__nv_bfloat16 *)q, (const __nv_bfloat16 *)k, (const __nv_bfloat16 *)v, q_ld,
                                        k_ld, v_ld, (__nv_bfloat16 *)k_cache, (__nv_bfloat16 *)v_cache, cos_t, sin_t, (int)T, pos0, (int)H,
                                        (int)Hkv, (int)D, max_ctx);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "rope_kv_prefill_kernel: %s", cudaGetErrorString(e));
    return check_launch("rope_kv_prefill_kernel");
}

int nslq_argmax_rows(const void *x, int x_dtype, int64_t M, int64_t V, int64_t ld, int64_t *out, int64_t *counter, void *stream)
{
    if (!x || !out) return fail(NSLQ_ERR_ARG, "nslq_argmax_rows: null argument");
    if (M < 0 || V <= 0 || ld < V || M > 0x7fffffffLL) return fail(NSLQ_ERR_SHAPE, "nslq_argmax_rows: M=%lld V=%lld ld=%lld", (long long)M, (long long)V, (long long)ld);
    if (M == 0) return NSLQ_OK;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    switch (x_dtype) {
    case NSLQ_DTYPE_F32: e = launch_kernel(argmax_rows_kernel<float>, dim3((unsigned)M), dim3(AM_THREADS), 0, st, (const float *)x, V, ld, out, counter); break;
    case NSLQ_DTYPE_FP16: e = launch_kernel(argmax_rows_kernel<__half>, dim3((unsigned)M), dim3(AM_THREADS), 0, st, (const __half *)x, V, ld, out, counter); break;
    case NSLQ_DTYPE_BF16: e = launch_kernel(argmax_rows_kernel<__nv_bfloat16>, dim3((unsigned)M), dim3(AM_THREADS), 0, st, (const __nv_bfloat16 *)x, V, ld, out, counter); break;
    default: return fail(NSLQ_ERR_ARG, "nslq_argmax_rows: dtype %d not in {F32,FP16,BF16}", x_dtype);
    }
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "argmax_rows_kernel: %s", cudaGetErrorString(e));
    return check_launch("argmax_rows_kernel");
}

}  // extern "C"
