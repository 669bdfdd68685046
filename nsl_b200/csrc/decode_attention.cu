// Decoder step around the linears: RoPE + KV-cache append + single-query attention, one launch.
//
// For every (sequence b, head h) of a decode step:
//   q, k_new  <- rotate-half RoPE at position pos (NSL's convention: the frequency table is
//               concat(freqs, freqs), stdlib/nsl/nn/rope.nsl:10-17; x*cos + rotate_half(x)*sin)
//   K[b,hk,pos] <- k_new (rounded to the cache dtype), V[b,hk,pos] <- v_new
//   out[b,h]  <- softmax_j( q . K[b,hk,j] * sm_scale,  j <= pos ) @ V[b,hk,:]
// which is what GroupedQueryAttention.forward computes for the newest token with a causal mask
// (stdlib/nsl/nn/gqa.nsl:66-95; hk = h / (H / Hkv)).  It replaces about fifteen framework kernels
// per layer of the decoder harness; the position is read from device memory so that a CUDA graph
// of the step can advance it itself.
//
// HBM-bound on the cache reads: one CTA per (b, h), sixteen warps, a warp per key, lanes 0..D/4-1 each holding
// four head dimensions, so a key or value row is one coalesced read of 2*D bytes; scores live in
// shared memory (ctx floats); fp32 arithmetic throughout, bf16 in and out.
#include "common.cuh"

namespace nslq {

// CTA width: 16 warps when there are few (b, h) pairs (batch 1 has only H CTAs, so each must be wide),
// 4 warps when there are enough CTAs to fill the machine several times over.
constexpr int DA_UNROLL = 8;               // key / value rows in flight per warp

static __device__ __forceinline__ float4 ld_bf16x4(const __nv_bfloat16 *p)
{
    const uint2 r = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
static __device__ __forceinline__ void st_bf16x4(__nv_bfloat16 *p, float4 v)
{
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2 *>(p) = make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
}
static __device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

struct AttnParams {
    const __nv_bfloat16 *q, *k_new, *v_new;   // [B,H,D], [B,Hkv,D], [B,Hkv,D]; rows of a sequence contiguous
    int64_t q_bs, k_bs, v_bs;                 // elements between consecutive sequences of q, k_new, v_new
    __nv_bfloat16 *k_cache, *v_cache;         // [B,Hkv,max_ctx,D]
    const float *cos_t, *sin_t;               // [max_ctx, D/2]
    const int64_t *pos;                       // device scalar: index the new token is written at
    __nv_bfloat16 *out;                       // [B,H,D]
    int H, Hkv, D, max_ctx;
    float sm_scale;
};

template <int DA_THREADS>
__global__ void __launch_bounds__(DA_THREADS)
decode_attention_kernel(const AttnParams p)
{
    constexpr int DA_WARPS = DA_THREADS / 32;
    extern __shared__ __align__(16) float sm[];
    float *scores = sm;                                   // [max_ctx]
    float *xrow = sm + p.max_ctx;                         // [2][D]: q then k_new before rotation
    float *part = xrow + 2 * p.D;                         // [DA_WARPS][D] partial outputs, then reductions
    __shared__ float red[DA_WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x / p.H, h = blockIdx.x % p.H, hk = h / (p.H / p.Hkv);
    pdl_wait();
    const int pos = (int)*p.pos;
    if (pos < 0 || pos >= p.max_ctx) return;              // nothing sensible to do; the host checks the range it can see
    const int half = p.D >> 1, nl = p.D >> 2;             // lanes that hold four dimensions each
    const __nv_bfloat16 *qg = p.q + (int64_t)b * p.q_bs + (int64_t)h * p.D;
    const __nv_bfloat16 *kg = p.k_new + (int64_t)b * p.k_bs + (int64_t)hk * p.D;
    const __nv_bfloat16 *vg = p.v_new + (int64_t)b * p.v_bs + (int64_t)hk * p.D;
    __nv_bfloat16 *kc = p.k_cache + ((int64_t)b * p.Hkv + hk) * p.max_ctx * p.D;
    __nv_bfloat16 *vc = p.v_cache + ((int64_t)b * p.Hkv + hk) * p.max_ctx * p.D;

    // ---- RoPE of q and k_new; append k, v (every head of a KV group writes the same bytes)
    for (int d = threadIdx.x; d < 2 * p.D; d += DA_THREADS)
        xrow[d] = __bfloat162float(d < p.D ? qg[d] : kg[d - p.D]);
    __syncthreads();
    float4 qv = make_float4(0.f, 0.f, 0.f, 0.f);         // this lane's four dimensions of the rotated, scaled query
    if (lane < nl) {
        float qr[4], kr[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int d = 4 * lane + e, i = d < half ? d : d - half;
            const float c = p.cos_t[(int64_t)pos * half + i], s = p.sin_t[(int64_t)pos * half + i];
            const float qa = xrow[d], qb = xrow[d < half ? d + half : d - half];
            const float ka = xrow[p.D + d], kb = xrow[p.D + (d < half ? d + half : d - half)];
            qr[e] = d < half ? qa * c - qb * s : qa * c + qb * s;
            kr[e] = d < half ? ka * c - kb * s : ka * c + kb * s;
        }
        // the query is rounded to bf16 like the keys it meets (the framework path does the same)
        qv = make_float4(__bfloat162float(__float2bfloat16_rn(qr[0])), __bfloat162float(__float2bfloat16_rn(qr[1])),
                         __bfloat162float(__float2bfloat16_rn(qr[2])), __bfloat162float(__float2bfloat16_rn(qr[3])));
        if (warp == 0) {
            st_bf16x4(kc + (int64_t)pos * p.D + 4 * lane, make_float4(kr[0], kr[1], kr[2], kr[3]));
            *reinterpret_cast<uint2 *>(vc + (int64_t)pos * p.D + 4 * lane) = *reinterpret_cast<const uint2 *>(vg + 4 * lane);
        }
    }
    __syncthreads();                                      // the new row is in the cache for this CTA's own reads

    // ---- scores: a warp per key, DA_UNROLL keys in flight
    const int n = pos + 1;
    float mx = -INFINITY;
    for (int j0 = warp * DA_UNROLL; j0 < n; j0 += DA_WARPS * DA_UNROLL) {
        float4 kv[DA_UNROLL];
#pragma unroll
        for (int u = 0; u < DA_UNROLL; ++u)
            kv[u] = (lane < nl && j0 + u < n) ? ld_bf16x4(kc + (int64_t)(j0 + u) * p.D + 4 * lane) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < DA_UNROLL; ++u) {
            const float s = warp_sum(qv.x * kv[u].x + qv.y * kv[u].y + qv.z * kv[u].z + qv.w * kv[u].w) * p.sm_scale;
            if (j0 + u < n) {
                if (lane == 0) scores[j0 + u] = s;
                mx = fmaxf(mx, s);
            }
        }
    }
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < DA_WARPS; ++w) mx = fmaxf(mx, red[w]);
    float sum = 0.0f;
    for (int j = threadIdx.x; j < n; j += DA_THREADS) {
        const float e = __expf(scores[j] - mx);
        scores[j] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    __syncthreads();
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < DA_WARPS; ++w) tot += red[w];
    const float inv = 1.0f / tot;

    // ---- out = P @ V: a warp per value row, lanes over the head dimensions
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j0 = warp * DA_UNROLL; j0 < n; j0 += DA_WARPS * DA_UNROLL) {
        float4 vv[DA_UNROLL];
#pragma unroll
        for (int u = 0; u < DA_UNROLL; ++u)
            vv[u] = (lane < nl && j0 + u < n) ? ld_bf16x4(vc + (int64_t)(j0 + u) * p.D + 4 * lane) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < DA_UNROLL; ++u) {
            const float pj = j0 + u < n ? scores[j0 + u] : 0.0f;
            acc.x += pj * vv[u].x; acc.y += pj * vv[u].y; acc.z += pj * vv[u].z; acc.w += pj * vv[u].w;
        }
    }
    if (lane < nl) *reinterpret_cast<float4 *>(part + warp * p.D + 4 * lane) = acc;
    __syncthreads();
    if (warp == 0 && lane < nl) {
        float4 o = *reinterpret_cast<const float4 *>(part + 4 * lane);
#pragma unroll
        for (int w = 1; w < DA_WARPS; ++w) {
            const float4 t = *reinterpret_cast<const float4 *>(part + w * p.D + 4 * lane);
            o.x += t.x; o.y += t.y; o.z += t.z; o.w += t.w;
        }
        st_bf16x4(p.out + ((int64_t)b * p.H + h) * p.D + 4 * lane, make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv));
    }
}

int decode_attention_dispatch(const void *q, const void *k_new, const void *v_new, int64_t q_bs, int64_t k_bs, int64_t v_bs,
                              void *k_cache, void *v_cache,
                              const float *cos_t, const float *sin_t, const int64_t *pos, int64_t B, int64_t H, int64_t Hkv,
                              int64_t D, int64_t max_ctx, float sm_scale, void *out, cudaStream_t st)
{
    if (!q || !k_new || !v_new || !k_cache || !v_cache || !cos_t || !sin_t || !pos || !out)
        return fail(NSLQ_ERR_ARG, "nslq_decode_attention: null argument");
    if (B <= 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0 || D <= 0 || D > 128 || D % 4 != 0 || max_ctx <= 0 || max_ctx % 4 != 0 || B * H > 0x7fffffffLL)
        return fail(NSLQ_ERR_SHAPE, "nslq_decode_attention: B=%lld H=%lld Hkv=%lld D=%lld (D %% 4 == 0, D <= 128) max_ctx=%lld (a multiple of 4)",
                    (long long)B, (long long)H, (long long)Hkv, (long long)D, (long long)max_ctx);
    const bool wide = B * H < 1024;
    const int warps = wide ? 16 : 4;
    const size_t smem = (size_t)(max_ctx + 2 * D + warps * D) * sizeof(float);
    if (smem > 200 * 1024) return fail(NSLQ_ERR_UNSUPPORTED, "nslq_decode_attention: max_ctx=%lld does not fit shared memory", (long long)max_ctx);
    static size_t reserved = 48 * 1024;
    if (smem > reserved) {
        if (cudaFuncSetAttribute(decode_attention_kernel<512>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
            cudaFuncSetAttribute(decode_attention_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return fail(NSLQ_ERR_CUDA, "decode_attention_kernel: cannot reserve %zu bytes of shared memory: %s", smem,
                        cudaGetErrorString(cudaGetLastError()));
        reserved = smem;
    }
    if (q_bs % 4 != 0 || k_bs % 4 != 0 || v_bs % 4 != 0 || q_bs < H * D || k_bs < Hkv * D || v_bs < Hkv * D)
        return fail(NSLQ_ERR_SHAPE, "nslq_decode_attention: batch strides must be multiples of 4 elements and cover a sequence's rows");
    AttnParams p{(const __nv_bfloat16 *)q, (const __nv_bfloat16 *)k_new, (const __nv_bfloat16 *)v_new, q_bs, k_bs, v_bs,
                 (__nv_bfloat16 *)k_cache, (__nv_bfloat16 *)v_cache, cos_t, sin_t, pos, (__nv_bfloat16 *)out,
                 (int)H, (int)Hkv, (int)D, (int)max_ctx, sm_scale};
    cudaError_t e = wide ? launch_kernel(decode_attention_kernel<512>, dim3((unsigned)(B * H)), dim3(512), smem, st, p)
                         : launch_kernel(decode_attention_kernel<128>, dim3((unsigned)(B * H)), dim3(128), smem, st, p);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "decode_attention_kernel: %s", cudaGetErrorString(e));
    return check_launch("decode_attention_kernel");
}

}  // namespace nslq
