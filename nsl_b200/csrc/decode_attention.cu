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
// HBM-bound on the cache reads: one CTA per (b, h).  q.K runs on the tensor pipe (mma.sync m16n8k16,
// the query as row 0 of A, eight keys per MMA column set, fp32 accumulation); P@V is fp32 FMAs with a
// warp per value row, lanes 0..D/4-1 each holding four head dimensions.  Scores live in shared memory
// (ctx floats); bf16 in and out.
#include <cooperative_groups.h>

#include "common.cuh"

namespace nslq {

namespace cg = cooperative_groups;

// CTA width: 8 warps while two CTAs per SM hold every (b, h) pair, 4 warps beyond that; with fewer pairs
// than resident CTAs a cluster of CTAs splits each pair's context (batch 1 has only H pairs).
constexpr int DA_UNROLL = 16;              // value rows in flight per warp
constexpr int DA_KU = 2;                   // groups of eight key rows in flight per warp

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

// 0 = ok; 0x901 = a launch found its position outside [0, max_ctx) and did nothing.
static __device__ int g_attn_status = 0;

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

// SPLIT > 1: a cluster of SPLIT CTAs shares one (sequence, head); CTA `rank` takes a contiguous slice of
// the context and rank 0 merges the partial softmax results (running maximum, sum, unnormalised output)
// that the others write into its shared memory.
template <int DA_THREADS, int SPLIT>
__global__ void __launch_bounds__(DA_THREADS)
decode_attention_kernel(const AttnParams p)
{
    constexpr int DA_WARPS = DA_THREADS / 32;
    __shared__ __align__(16) float merge[SPLIT > 1 ? SPLIT : 1][132];    // per rank: max, sum, out[D <= 128]
    extern __shared__ __align__(16) float sm[];
    float *scores = sm;                                   // [max_ctx + DA_UNROLL]
    float *xrow = sm + p.max_ctx + DA_UNROLL;                         // [2][D]: q then k_new before rotation
    float *part = xrow + 2 * p.D;                         // [DA_WARPS][D] partial outputs, then reductions
    __shared__ float red[DA_WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bh = blockIdx.x / SPLIT, rank = blockIdx.x % SPLIT;     // the cluster spans SPLIT consecutive CTAs
    const int b = bh / p.H, h = bh % p.H, hk = h / (p.H / p.Hkv);
    pdl_wait();
    // q and k_new do not depend on the position: their loads go out before the position is read, not
    // behind the branch on it (2 D <= 256 values, at most two per thread).
    const __nv_bfloat16 *qg = p.q + (int64_t)b * p.q_bs + (int64_t)h * p.D;
    const __nv_bfloat16 *kg = p.k_new + (int64_t)b * p.k_bs + (int64_t)hk * p.D;
    float xin[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int d = (int)threadIdx.x + u * DA_THREADS;
        xin[u] = d < 2 * p.D ? __bfloat162float(d < p.D ? qg[d] : kg[d - p.D]) : 0.0f;
    }
    const int pos = (int)*p.pos;
    if (pos < 0 || pos >= p.max_ctx) {                    // every CTA of a cluster takes this exit together
        // Nothing sensible to do -- but not silently: a decode loop replayed past the end of its cache would
        // otherwise keep emitting tokens from stale outputs.  The status word is read by nslq_device_status.
        if (threadIdx.x == 0) atomicCAS(&g_attn_status, 0, 0x901);
        return;
    }
    if (SPLIT > 1) cg::this_cluster().sync();             // every CTA of the cluster runs before anyone writes into rank 0's shared memory
    const int half = p.D >> 1, nl = p.D >> 2;             // lanes that hold four dimensions each
    // this CTA's slice [jb, je) of the n = pos + 1 keys (whole groups of 16; later ranks may be empty)
    const int n = pos + 1;
    const int chunk = SPLIT > 1 ? (((n + SPLIT - 1) / SPLIT + 15) & ~15) : n;
    const int jb = rank * chunk, je = min(n, jb + chunk);
    const bool owns_new = SPLIT == 1 || (jb <= pos && pos < je);         // the slice that holds the new row writes it
    const __nv_bfloat16 *vg = p.v_new + (int64_t)b * p.v_bs + (int64_t)hk * p.D;
    __nv_bfloat16 *kc = p.k_cache + ((int64_t)b * p.Hkv + hk) * p.max_ctx * p.D;
    __nv_bfloat16 *vc = p.v_cache + ((int64_t)b * p.Hkv + hk) * p.max_ctx * p.D;

    // ---- RoPE of q and k_new; append k, v (every head of a KV group writes the same bytes)
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int d = (int)threadIdx.x + u * DA_THREADS;
        if (d < 2 * p.D) xrow[d] = xin[u];
    }
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
        if (warp == 0 && owns_new) {
            st_bf16x4(kc + (int64_t)pos * p.D + 4 * lane, make_float4(kr[0], kr[1], kr[2], kr[3]));
            *reinterpret_cast<uint2 *>(vc + (int64_t)pos * p.D + 4 * lane) = *reinterpret_cast<const uint2 *>(vg + 4 * lane);
        }
    }
    __syncthreads();                                      // the new row is in the cache for this CTA's own reads

    // ---- scores on the tensor pipe: mma.sync.m16n8k16 with the query as row 0 of A (the other fifteen
    // rows are zero) and eight keys as the columns of B, read straight from the cache: lane (g, t)
    // loads dims 2t, 2t+1 and 2t+8, 2t+9 of key j0+g for every 16 dims.  About 2.6 issued
    // instructions per key instead of 17 for a per-key shuffle reduction; the kernel was bound by
    // issued instructions, not by HBM.
    const int g = lane >> 2, t = lane & 3;
    constexpr int KSTEPS = 8;                              // 16 dims each: D <= 128
    uint32_t qa0[KSTEPS], qa2[KSTEPS];                     // A fragment registers of row 0 (zero elsewhere)
    {
        // the rotated query goes through shared memory once, as bf16 pairs
        __nv_bfloat16 *qs = reinterpret_cast<__nv_bfloat16 *>(xrow);          // [D], reuses the staging rows (all reads of them are behind the barrier above)
        if (warp == 0 && lane < nl) st_bf16x4(qs + 4 * lane, qv);
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int d0 = 16 * ks + 2 * t, d2 = d0 + 8;
            qa0[ks] = (g == 0 && d0 < p.D) ? *reinterpret_cast<const uint32_t *>(qs + d0) : 0u;
            qa2[ks] = (g == 0 && d2 < p.D) ? *reinterpret_cast<const uint32_t *>(qs + d2) : 0u;
        }
    }
    const int ksteps = (p.D + 15) >> 4;
    // Loads carry no predicates: a dimension past D reads dimension D-2 instead (its query register is
    // zero) and a key past the slice reads its last key (its score is never stored), so every address is
    // inside initialised cache rows and a warp keeps DA_KU * 8 key rows in flight per iteration.
    // Only the last 16 dimensions can reach past D.
    const int last0 = min(16 * (ksteps - 1) + 2 * t, p.D - 2) - 2 * t, last2 = min(16 * (ksteps - 1) + 2 * t + 8, p.D - 2) - 2 * t;
    float mx = -INFINITY;
    for (int j0 = jb + warp * (8 * DA_KU); j0 < je; j0 += DA_WARPS * (8 * DA_KU)) {
        uint32_t b0[DA_KU][KSTEPS], b1[DA_KU][KSTEPS];
#pragma unroll
        for (int u = 0; u < DA_KU; ++u) {
            const __nv_bfloat16 *krow = kc + (int64_t)min(j0 + 8 * u + g, je - 1) * p.D + 2 * t;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                if (ks < ksteps - 1) {                     // warp-uniform
                    b0[u][ks] = *reinterpret_cast<const uint32_t *>(krow + 16 * ks);
                    b1[u][ks] = *reinterpret_cast<const uint32_t *>(krow + 16 * ks + 8);
                } else if (ks == ksteps - 1) {
                    b0[u][ks] = *reinterpret_cast<const uint32_t *>(krow + last0);
                    b1[u][ks] = *reinterpret_cast<const uint32_t *>(krow + last2);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < DA_KU; ++u) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks)
                if (ks < ksteps)
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                                 : "r"(qa0[ks]), "r"(0u), "r"(qa2[ks]), "r"(0u), "r"(b0[u][ks]), "r"(b1[u][ks]));
            if (g == 0) {                                  // row 0 of C: keys j, j + 1
                const int j = j0 + 8 * u + 2 * t;
                if (j < je) { const float sv = c[0] * p.sm_scale; scores[j] = sv; mx = fmaxf(mx, sv); }
                if (j + 1 < je) { const float sv = c[1] * p.sm_scale; scores[j + 1] = sv; mx = fmaxf(mx, sv); }
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < DA_WARPS; ++w) mx = fmaxf(mx, red[w]);
    float sum = 0.0f;
    for (int j = jb + threadIdx.x; j < je; j += DA_THREADS) {
        const float e = __expf(scores[j] - mx);
        scores[j] = e;
        sum += e;
    }
    if (je > jb)
        for (int j = je + threadIdx.x; j < je + DA_UNROLL; j += DA_THREADS) scores[j] = 0.0f;     // the array has DA_UNROLL spare floats
    sum = warp_sum(sum);
    __syncthreads();
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < DA_WARPS; ++w) tot += red[w];
    const float inv = 1.0f / tot;

    // ---- out = P @ V: a warp per value row, lanes over the head dimensions
    // Probabilities past the slice are zero (written above its last key by the softmax loop), rows past
    // it read its last row and lanes past D/4 read the row's last four dimensions: no predicates.
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const int voff = 4 * min(lane, nl - 1);
    for (int j0 = jb + warp * DA_UNROLL; j0 < je; j0 += DA_WARPS * DA_UNROLL) {
        uint2 vv[DA_UNROLL];
#pragma unroll
        for (int u = 0; u < DA_UNROLL; ++u)
            vv[u] = *reinterpret_cast<const uint2 *>(vc + (int64_t)min(j0 + u, je - 1) * p.D + voff);
#pragma unroll
        for (int u = 0; u < DA_UNROLL; u += 4) {
            const float4 pj = *reinterpret_cast<const float4 *>(scores + j0 + u);   // j0 is a multiple of 4
            const float pp[4] = {pj.x, pj.y, pj.z, pj.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint2 r = vv[u + e];
                acc.x += pp[e] * __uint_as_float(r.x << 16); acc.y += pp[e] * __uint_as_float(r.x & 0xffff0000u);
                acc.z += pp[e] * __uint_as_float(r.y << 16); acc.w += pp[e] * __uint_as_float(r.y & 0xffff0000u);
            }
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
        if (SPLIT == 1) {
            st_bf16x4(p.out + ((int64_t)b * p.H + h) * p.D + 4 * lane, make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv));
        } else {
            // this slice's (maximum, sum, unnormalised output) into rank 0's shared memory
            float *dst = cg::this_cluster().map_shared_rank(&merge[0][0], 0) + rank * 132;
            *reinterpret_cast<float4 *>(dst + 4 + 4 * lane) = o;
            if (lane == 0) { dst[0] = mx; dst[1] = tot; }
        }
    }
    if (SPLIT > 1) {
        cg::this_cluster().sync();                        // release/acquire at cluster scope: the slots are visible
        if (rank == 0 && warp == 0 && lane < nl) {
            float big = merge[0][0];
#pragma unroll
            for (int r = 1; r < SPLIT; ++r) big = fmaxf(big, merge[r][0]);
            float den = 0.0f;
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int r = 0; r < SPLIT; ++r) {
                const float w = __expf(merge[r][0] - big);            // an empty slice has maximum -inf: weight 0
                const float4 t = *reinterpret_cast<const float4 *>(&merge[r][4 + 4 * lane]);
                den += w * merge[r][1];
                o.x += w * t.x; o.y += w * t.y; o.z += w * t.z; o.w += w * t.w;
            }
            const float id = 1.0f / den;
            st_bf16x4(p.out + ((int64_t)b * p.H + h) * p.D + 4 * lane, make_float4(o.x * id, o.y * id, o.z * id, o.w * id));
        }
    }
}

// `split` consecutive CTAs form a cluster (one (b, h) pair); dependent launch as everywhere else.
static cudaError_t launch_attention(void (*kernel)(const AttnParams), int64_t pairs, int threads, int split, size_t smem,
                                    cudaStream_t st, const AttnParams &p)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(pairs * split));
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (split > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = (unsigned)split;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (g_use_pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kernel, p);
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
    // About 640 threads fit an SM at this kernel's register count, i.e. two CTAs of 256 threads: 296 CTAs are
    // resident at once.  Fewer (b, h) pairs than that: a cluster of 2, 4 or 8 CTAs splits each pair's context.
    const int64_t BH = B * H;
    const int split = BH <= 37 ? 8 : (BH <= 74 ? 4 : (BH <= 148 ? 2 : 1));
    const int threads = BH <= 296 ? 256 : 128;
    const int warps = threads / 32;
    const size_t smem = (size_t)(max_ctx + DA_UNROLL + 2 * D + warps * D) * sizeof(float);
    if (smem > 200 * 1024) return fail(NSLQ_ERR_UNSUPPORTED, "nslq_decode_attention: max_ctx=%lld does not fit shared memory", (long long)max_ctx);
    static std::atomic<size_t> r8[kMaxDevices], r4[kMaxDevices], r2[kMaxDevices], r1[kMaxDevices], r0[kMaxDevices];
    if (reserve_smem(decode_attention_kernel<256, 8>, r8, smem) != cudaSuccess ||
        reserve_smem(decode_attention_kernel<256, 4>, r4, smem) != cudaSuccess ||
        reserve_smem(decode_attention_kernel<256, 2>, r2, smem) != cudaSuccess ||
        reserve_smem(decode_attention_kernel<256, 1>, r1, smem) != cudaSuccess ||
        reserve_smem(decode_attention_kernel<128, 1>, r0, smem) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "decode_attention_kernel: cannot reserve %zu bytes of shared memory: %s", smem,
                    cudaGetErrorString(cudaGetLastError()));
    if (q_bs % 4 != 0 || k_bs % 4 != 0 || v_bs % 4 != 0 || q_bs < H * D || k_bs < Hkv * D || v_bs < Hkv * D)
        return fail(NSLQ_ERR_SHAPE, "nslq_decode_attention: batch strides must be multiples of 4 elements and cover a sequence's rows");
    AttnParams p{(const __nv_bfloat16 *)q, (const __nv_bfloat16 *)k_new, (const __nv_bfloat16 *)v_new, q_bs, k_bs, v_bs,
                 (__nv_bfloat16 *)k_cache, (__nv_bfloat16 *)v_cache, cos_t, sin_t, pos, (__nv_bfloat16 *)out,
                 (int)H, (int)Hkv, (int)D, (int)max_ctx, sm_scale};
    cudaError_t e;
    switch (threads == 128 ? 0 : split) {
    case 0: e = launch_attention(decode_attention_kernel<128, 1>, BH, 128, 1, smem, st, p); break;
    case 1: e = launch_attention(decode_attention_kernel<256, 1>, BH, 256, 1, smem, st, p); break;
    case 2: e = launch_attention(decode_attention_kernel<256, 2>, BH, 256, 2, smem, st, p); break;
    case 4: e = launch_attention(decode_attention_kernel<256, 4>, BH, 256, 4, smem, st, p); break;
    default: e = launch_attention(decode_attention_kernel<256, 8>, BH, 256, 8, smem, st, p); break;
    }
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "decode_attention_kernel: %s", cudaGetErrorString(e));
    return check_launch("decode_attention_kernel");
}

int decode_attention_status(int *out)
{
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int)) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "nslq_device_status: %s", cudaGetErrorString(cudaGetLastError()));
    if (v != 0) cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(int));
    *out = v;
    return NSLQ_OK;
}

}  // namespace nslq
