// Stage 2: BitLinear decode GEMV/skinny GEMM for M <= 16 tokens.
//
// HBM-bound weight streaming.  The packed weight is read in NSL's own layout
// ([N][K/4] bytes, 4 consecutive-k trits per byte, HIGH-BITS-FIRST, code = trit+1;
// crates/nsl-codegen/src/bitnet/pack.rs:38-43) with 128-bit loads that are all
// issued before any arithmetic, unpacked in registers and multiplied on the
// integer tensor pipe:
//
//   * a CTA owns 16 output rows; its warps split K in steps of 256 (4 lanes of a
//     quad x 64 trits = one uint4 each, for rows g and g+8 of the tile);
//   * a 32-bit word w of packed bytes b0..b3 yields, for i = 0..3,
//     w & (0x03030303 << (6-2i)) = the codes of k = 4j+i for byte j, times 4^(3-i):
//     four u8x4 MMA operand registers per word for one AND each, no per-trit work.
//     The quantised activations are stored in the matching order (position 4i+j of
//     every 16 holds k = 4j+i), so registers line up with no shuffles;
//   * mma.sync.m16n8k32.u8.s8 accumulates sum_k q*code*4^(3-i) exactly in int32, one
//     accumulator per position class i, for up to 8 tokens per MMA; the classes are
//     shifted back (exact) and summed; acc = that - rowsum(q) because code = trit + 1;
//   * the K-split partials are reduced through shared memory and finalised as
//     ((scale/127) * (float)acc) * weight_scale with separately rounded steps
//     (crates/nsl-codegen/src/bitnet/phases/finalize.rs:39-53).
//
// For one token the activation quantisation is fused in (the bulk-copy kernel below, or
// ternary_gemv_fused_kernel -- written for up to four -- where a CTA's slab does not fit): each
// CTA issues its weight loads, then -- while they are in flight -- quantises the token
// rows itself (absmax by warp shuffles, the reference's exact rounding) into shared memory
// in the consumption order, so a decode-time linear is one launch and one trip to HBM.
//
// Also here: a scalar kernel for shapes the streaming kernel cannot take
// (K % 64 != 0 or unaligned rows); same arithmetic, natural-order activations.
#include "quant_core.cuh"
#include "sm100_common.cuh"
#include "ternary_mma.cuh"

namespace nslq {

constexpr int GEMV_MAX_LAYERS = 4;
struct GemvParams {
    const uint8_t *w;      // [N][K/4]
    const int8_t *q;       // [M][K] permuted order
    const float *scale;    // [M]
    const int32_t *rowsum; // [M]
    void *y;               // [M][N]
    int32_t *acc_out;      // [M][N] or null
    const float *bias;     // [N] or null
    const float *residual; // [M][N] or null
    int64_t N, K;
    int M, y_dtype;
    float weight_scale;
    // Sibling projections of the same quantised rows (q/k/v, gate/up) in the same launch: CTAs from
    // sib[i].first_cta on multiply sibling i's weights.  acc_out, bias and residual are null then.
    int nsib;
    struct Sibling {
        const uint8_t *w;
        void *y;
        int64_t N;
        float weight_scale;
        unsigned first_cta;
    } sib[GEMV_MAX_LAYERS - 1];
};

// KW warps per CTA split K; NT = token tiles of 8; UNROLL = steps whose weight
// loads are in flight together per warp.
template <int KW, int NT, int UNROLL>
__global__ void __launch_bounds__(KW * 32)
ternary_gemv_kernel(const GemvParams p)
{
    __shared__ int red[KW][NT][32][4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    // this CTA's projection: the first one, or the last sibling whose range the CTA index has reached
    const uint8_t *lw = p.w;
    void *ly = p.y;
    int64_t lN = p.N;
    float lws = p.weight_scale;
    unsigned cta0 = 0;
#pragma unroll
    for (int i = 0; i < GEMV_MAX_LAYERS - 1; ++i) {
        if (i < p.nsib && blockIdx.x >= p.sib[i].first_cta) {
            lw = p.sib[i].w; ly = p.sib[i].y; lN = p.sib[i].N; lws = p.sib[i].weight_scale; cta0 = p.sib[i].first_cta;
        }
    }
    const int64_t n0 = (int64_t)(blockIdx.x - cta0) * 16;
    const int64_t row_bytes = p.K >> 2;
    const int nchunks = (int)(p.K >> 6);            // 64 trits = 16 bytes per chunk
    const int nsteps = (nchunks + 3) >> 2;
    const bool rowa_ok = (n0 + g) < lN, rowb_ok = (n0 + g + 8) < lN;
    const uint8_t *wa = lw + (n0 + g) * row_bytes;
    const uint8_t *wb = lw + (n0 + g + 8) * row_bytes;

    Acc4 acc[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc_zero(acc[nt]);

    bool waited = false;
    for (int s0 = warp; s0 < nsteps; s0 += KW * UNROLL) {
        uint4 ra[UNROLL], rb[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int c = 4 * (s0 + u * KW) + t;
            const bool ok = c < nchunks;
            ra[u] = (ok && rowa_ok) ? ld_stream_u4(wa + (int64_t)c * 16) : make_uint4(0, 0, 0, 0);
            rb[u] = (ok && rowb_ok) ? ld_stream_u4(wb + (int64_t)c * 16) : make_uint4(0, 0, 0, 0);
        }
        // Weights do not depend on the preceding kernel; the activations do.
        if (!waited) { pdl_launch_dependents(); pdl_wait(); waited = true; }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int c = 4 * (s0 + u * KW) + t;
            if (4 * (s0 + u * KW) >= nchunks) break;   // warp-uniform
            const bool ok = c < nchunks;
            uint4 xq[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int tok = nt * 8 + g;
                const uint4 *src = reinterpret_cast<const uint4 *>(p.q + (int64_t)tok * p.K + (int64_t)c * 64);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    xq[nt][j] = (ok && tok < p.M) ? __ldg(src + j) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) chunk_mma(acc[nt], ra[u], rb[u], xq[nt]);
        }
    }
    if (!waited) pdl_wait();

#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int r = 0; r < 4; ++r) red[warp][nt][lane][r] = acc_value(acc[nt], r);
    __syncthreads();

    // One output per thread-iteration; consecutive threads take consecutive rows.
    for (int e = threadIdx.x; e < 16 * 8 * NT; e += KW * 32) {
        const int row = e & 15, tok = e >> 4;
        if (tok >= p.M || n0 + row >= lN) continue;
        const int nt = tok >> 3, tl = tok & 7;
        const int src_lane = (row & 7) * 4 + (tl >> 1);
        const int src_reg = ((row >> 3) << 1) | (tl & 1);
        int a = 0;
#pragma unroll
        for (int w = 0; w < KW; ++w) a += red[w][nt][src_lane][src_reg];
        a -= p.rowsum[tok];
        const int64_t o = (int64_t)tok * lN + n0 + row;
        if (p.acc_out) p.acc_out[o] = a;
        float v = bitlinear_finalize(a, p.scale[tok], lws);
        if (p.bias) v = __fadd_rn(v, p.bias[n0 + row]);
        if (p.residual) v = __fadd_rn(v, p.residual[o]);
        store_out(ly, p.y_dtype, o, v);
    }
}


struct FusedParams {
    const uint8_t *w;      // [N][K/4]
    const void *x;         // [M][K] fp32 / fp16 / bf16
    void *y;               // [M][N]
    int32_t *acc_out;      // [M][N] or null
    const float *bias;     // [N] or null
    const float *residual; // [M][N] or null
    int64_t N, K;
    int M, y_dtype;
    float weight_scale;
};

constexpr int FUSED_MAX_M = 4;

// Decode kernel with the activation quantisation fused in (up to four tokens; the library calls it
// for one: beyond that the CTAs' repeated quantisation costs more than a second launch).  A CTA owns TPC row tiles
// of 16 output rows; each tile's K range is split over KW warps (threads = TPC*KW*32).  The
// token rows are quantised once per CTA, so a wider CTA repeats less of that work.
// Dynamic shared memory: [M*K int8 activations, consumption order][TPC*KW*32*4 int reduce]
// [small per-token arrays].
template <typename T, int KW, int TPC, int UNROLL>
__global__ void __launch_bounds__(KW * TPC * 32)
ternary_gemv_fused_kernel(const FusedParams p)
{
    constexpr int NW = KW * TPC, NTHR = NW * 32;
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = warp / KW, kw = warp % KW;
    const int g = lane >> 2, t = lane & 3;
    int8_t *q_s = reinterpret_cast<int8_t *>(smem);
    int *red = reinterpret_cast<int *>(smem + (((size_t)p.M * p.K + 15) & ~(size_t)15));
    float *part_f = reinterpret_cast<float *>(red + NW * 32 * 4);       // [NW][FUSED_MAX_M]
    int *part_i = reinterpret_cast<int *>(part_f + NW * FUSED_MAX_M);    // [NW][FUSED_MAX_M]
    float *scale_s = reinterpret_cast<float *>(part_i + NW * FUSED_MAX_M);
    int *rowsum_s = reinterpret_cast<int *>(scale_s + FUSED_MAX_M);

    const int64_t n0 = ((int64_t)blockIdx.x * TPC + tile) * 16;
    const int64_t row_bytes = p.K >> 2;
    const int nchunks = (int)(p.K >> 6);
    const int nsteps = (nchunks + 3) >> 2;
    const bool rowa_ok = (n0 + g) < p.N, rowb_ok = (n0 + g + 8) < p.N;
    const uint8_t *wa = p.w + (n0 + g) * row_bytes;
    const uint8_t *wb = p.w + (n0 + g + 8) * row_bytes;

    uint4 ra[UNROLL], rb[UNROLL];
    auto load_batch = [&](int s0) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int c = 4 * (s0 + u * KW) + t;
            const bool ok = c < nchunks;
            ra[u] = (ok && rowa_ok) ? ld_stream_u4(wa + (int64_t)c * 16) : make_uint4(0, 0, 0, 0);
            rb[u] = (ok && rowb_ok) ? ld_stream_u4(wb + (int64_t)c * 16) : make_uint4(0, 0, 0, 0);
        }
    };
    // Weights never depend on the preceding kernel: get them moving, let the next kernel of
    // the stream start doing the same, and only then wait for our own inputs.
    load_batch(kw);
    pdl_launch_dependents();
    pdl_wait();

    // ---- quantise the M token rows into shared memory (same arithmetic as act_quant_kernel).
    // Each thread keeps its share of a row in registers between the absmax pass and the
    // rounding pass (XV float4 per thread covers K <= XV*4*NTHR; longer rows are re-read).
    const T *x = reinterpret_cast<const T *>(p.x);
    const int nvec = (int)(p.K >> 2);
    constexpr int XV = (NTHR >= 512) ? 4 : 8;
    for (int m = 0; m < p.M; ++m) {
        const T *xr = x + (int64_t)m * p.K;
        float4 xv[XV];
        float mx = 0.0f;
#pragma unroll
        for (int i = 0; i < XV; ++i) {
            const int v = i * NTHR + threadIdx.x;
            xv[i] = (v < nvec) ? Vec4<T>::load(xr, v) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < XV; ++i)
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(xv[i].x), fabsf(xv[i].y)), fmaxf(fabsf(xv[i].z), fabsf(xv[i].w))));
        for (int v = XV * NTHR + threadIdx.x; v < nvec; v += NTHR) {
            const float4 f = Vec4<T>::load(xr, v);
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w))));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) part_f[warp * FUSED_MAX_M + m] = mx;
        __syncthreads();
        float scale = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; ++w) scale = fmaxf(scale, part_f[w * FUSED_MAX_M + m]);
        const float inv = __fdiv_rn(127.0f, scale);
        const bool zero_row = (scale == 0.0f);
        if (threadIdx.x == 0) scale_s[m] = scale;
        int sum = 0;
        uint32_t *q_row = reinterpret_cast<uint32_t *>(q_s + (int64_t)m * p.K);
        auto quant_store = [&](const float4 &f, int v, unsigned mask) {
            const int q0 = zero_row ? 0 : quant_one(f.x, inv), q1 = zero_row ? 0 : quant_one(f.y, inv);
            const int q2 = zero_row ? 0 : quant_one(f.z, inv), q3 = zero_row ? 0 : quant_one(f.w, inv);
            sum += q0 + q1 + q2 + q3;
            q_row[v] = quad_transpose(pack4_i8(q0, q1, q2, q3), mask);
        };
#pragma unroll
        for (int i = 0; i < XV; ++i) {
            const int v = i * NTHR + threadIdx.x;
            const bool in = v < nvec;
            const unsigned mask = __ballot_sync(0xffffffffu, in);   // whole quads: K % 64 == 0
            if (in) quant_store(xv[i], v, mask);
        }
        for (int base = XV * NTHR; base < nvec; base += NTHR) {
            const int v = base + threadIdx.x;
            const bool in = v < nvec;
            const unsigned mask = __ballot_sync(0xffffffffu, in);
            if (in) quant_store(Vec4<T>::load(xr, v), v, mask);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) part_i[warp * FUSED_MAX_M + m] = sum;
    }
    __syncthreads();
    if (threadIdx.x < p.M) {
        int tot = 0;
#pragma unroll
        for (int w = 0; w < NW; ++w) tot += part_i[w * FUSED_MAX_M + threadIdx.x];
        rowsum_s[threadIdx.x] = tot;
    }

    // ---- stream K.  A lane whose token does not exist reads a block of zeros with stride 0, so
    // the loop has no selects; a chunk index past the row only meets zero weights.
    uint4 *zero_blk = reinterpret_cast<uint4 *>(rowsum_s + FUSED_MAX_M);
    if (threadIdx.x < 4) zero_blk[threadIdx.x] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    const uint4 *qrow = (g < p.M) ? reinterpret_cast<const uint4 *>(q_s + (size_t)g * p.K) + t * 4 : zero_blk;
    const int qstride = (g < p.M) ? 16 : 0;
    Acc4 acc;
    acc_zero(acc);
    for (int s0 = kw; s0 < nsteps; s0 += KW * UNROLL) {
        if (s0 != kw) load_batch(s0);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int sidx = s0 + u * KW;
            if (4 * sidx >= nchunks) break;   // warp-uniform
            uint4 xq[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) xq[j] = qrow[sidx * qstride + j];
            chunk_mma(acc, ra[u], rb[u], xq);
        }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) red[(warp * 32 + lane) * 4 + r] = acc_value(acc, r);
    __syncthreads();

    // 16 rows x up to 4 tokens per tile; consecutive threads take consecutive rows
    for (int e = threadIdx.x; e < TPC * 16 * FUSED_MAX_M; e += NTHR) {
        const int tl = e / (16 * FUSED_MAX_M), row = e & 15, tok = (e >> 4) & (FUSED_MAX_M - 1);
        const int64_t n = ((int64_t)blockIdx.x * TPC + tl) * 16 + row;
        if (tok >= p.M || n >= p.N) continue;
        const int src_lane = (row & 7) * 4 + (tok >> 1);
        const int src_reg = ((row >> 3) << 1) | (tok & 1);
        int a = 0;
#pragma unroll
        for (int w = 0; w < KW; ++w) a += red[((tl * KW + w) * 32 + src_lane) * 4 + src_reg];
        a -= rowsum_s[tok];
        const int64_t o = (int64_t)tok * p.N + n;
        if (p.acc_out) p.acc_out[o] = a;
        float v = bitlinear_finalize(a, scale_s[tok], p.weight_scale);
        if (p.bias) v = __fadd_rn(v, p.bias[n]);
        if (p.residual) v = __fadd_rn(v, p.residual[o]);
        store_out(p.y, p.y_dtype, o, v);
    }
}

// ---------------------------------------------------------------- bulk-copy decode kernel (one token row)
// The same product with the weight slab brought in by the copy engine.  A CTA owns ROWS
// consecutive output rows; in NSL's layout their packed bytes are ONE contiguous range of the
// weight (ROWS * K/4 bytes), so the CTA's first instruction issues a handful of cp.async.bulk
// copies (one per tile of 16 rows, each with its own mbarrier) that land the whole slab in
// shared memory without occupying a register or an issue slot.  Only then does it wait for the
// preceding kernel (the weights never depend on it) and quantise the token rows.  A CTA needs
// ~70 KB and 256 threads, so three are resident per SM: with dependent launch the next two
// calls of a decode chain already have their weights in flight while this one does arithmetic,
// which is what a 7 MB matrix needs to approach HBM speed (the whole matrix is in flight at once).
// (An mma.sync form of this CTA served three and four tokens; quantising four token rows in every
// CTA made it 7.3 us where the separate quantiser plus the pre-quantised kernel take 1.7 + 2.9, so
// those token counts are two launches now and the form is gone.)
constexpr int BULK_MAX_LAYERS = 4;
struct BulkParams {
    const uint8_t *w;      // [N][K/4]
    const void *x;         // [M][K] fp32 / fp16 / bf16
    void *y;               // [M][N]
    int32_t *acc_out;      // [M][N] or null
    const float *bias;     // [N] or null
    const float *residual; // [M][N] or null
    int64_t N, K;
    int M, y_dtype;
    float weight_scale;
    // What the token rows are made of before they are quantised (the launches in front of a decode
    // projection, done by every CTA for itself instead):
    //   SRC_PLAIN    x
    //   SRC_RMSNORM  (f32)(x / rms * norm_w), rms = sqrt(mean x^2 + eps) in f64  (nslq_rmsnorm_act_quant_i8)
    //   SRC_SWIGLU   silu(x) * x2 in fp32                                        (nslq_swiglu_act_quant_i8)
    int src;               // (a template argument of the kernels; kept here for the dispatch)
    const void *x2;        // [M][K], SRC_SWIGLU
    const float *norm_w;   // [K], SRC_RMSNORM
    double eps;
    // Sibling projections of the same token rows (q/k/v, gate/up) in the same launch: CTAs from
    // sib[i].first_cta on multiply sibling i's weights instead.  Every CTA quantises the rows for itself
    // anyway, so siblings cost nothing but their own CTAs, and one launch replaces a fork onto side
    // streams and its join.  acc_out and residual are null when there are siblings.
    int nsib;
    struct Sibling {
        const uint8_t *w;
        void *y;
        const float *bias;
        int64_t N;
        float weight_scale;
        unsigned first_cta;
    } sib[BULK_MAX_LAYERS - 1];
};
enum { SRC_PLAIN = 0, SRC_RMSNORM = 1, SRC_SWIGLU = 2 };

// Group gi of token m before normalisation: x, or silu(x) * x2.
template <typename T, int SRC>
static __device__ __forceinline__ void src_load(const BulkParams &p, int m, int gi, float (&f)[16])
{
    Group16<T>::load(reinterpret_cast<const T *>(p.x) + (int64_t)m * p.K, gi, f);
    if (SRC == SRC_SWIGLU) {
        float u[16];
        Group16<T>::load(reinterpret_cast<const T *>(p.x2) + (int64_t)m * p.K, gi, u);
#pragma unroll
        for (int e = 0; e < 16; ++e) f[e] = swiglu_one(f[e], u[e]);
    }
}

constexpr int BULK_THREADS = 256;

// acc + sum_b (unsigned byte b of a) * (signed byte b of x)
static __device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t x, int acc)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(x), "r"(acc));
    return d;
}

static __device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// SRC_RMSNORM / SRC_SWIGLU: form, measure and quantise token row m.  The formed row is staged in shared
// memory (h_s, K floats, quarter j of group gi at float4 index j * ngroups + gi so that a warp's accesses are
// consecutive; every thread reads back only the groups it wrote) so that each transform exists
// once, in a rolled loop: kept in registers and unrolled, the prologue was several thousand instructions that
// a CTA executes exactly once, and fetching them cost more than executing them.
// part_d / part_f / part_i: [NW][FUSED_MAX_M] partials of the warps; the caller synchronises after the last row.
// put(q, gi, sum) packs a quantised group into the kernel's own layout.
template <typename T, int SRC, int NW, typename Put>
static __device__ __forceinline__ void src_quantise_row(const BulkParams &p, int m, float *h_s, double *part_d, float *part_f,
                                                        int *part_i, Put put)
{
    constexpr int NTHR = NW * 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ngroups = (int)(p.K >> 4);
    float mx = 0.0f;
    double sq = 0.0;
#pragma unroll 1
    for (int gi = threadIdx.x; gi < ngroups; gi += NTHR) {
        float f[16];
        src_load<T, SRC>(p, m, gi, f);
        if (SRC == SRC_RMSNORM) {
            // the norm weights of this group are needed behind two reductions: have them fetched meanwhile
            asm volatile("prefetch.global.L1 [%0];" ::"l"(p.norm_w + 16 * (int64_t)gi));
#pragma unroll
            for (int e = 0; e < 16; ++e) sq += (double)f[e] * (double)f[e];
        } else {
            mx = absmax16(f, mx);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) reinterpret_cast<float4 *>(h_s)[j * ngroups + gi] = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
    }
    if (SRC == SRC_RMSNORM) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) part_d[warp * FUSED_MAX_M + m] = sq;
        __syncthreads();
        const double tot = sum_partials<NW>(part_d + m, FUSED_MAX_M);
        const double rms = sqrt(tot / (double)p.K + p.eps), rinv = __drcp_rn(rms);
#pragma unroll 1
        for (int gi = threadIdx.x; gi < ngroups; gi += NTHR) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float4 v = reinterpret_cast<const float4 *>(h_s)[j * ngroups + gi];
                const float4 w = __ldg(reinterpret_cast<const float4 *>(p.norm_w) + 4 * gi + j);
                v = norm_four(v, rms, rinv, w);
                mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                reinterpret_cast<float4 *>(h_s)[j * ngroups + gi] = v;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) part_f[warp * FUSED_MAX_M + m] = mx;
    __syncthreads();
    float scale = 0.0f;
#pragma unroll
    for (int w = 0; w < NW; ++w) scale = fmaxf(scale, part_f[w * FUSED_MAX_M + m]);
    const float inv = __fdiv_rn(127.0f, scale);
    const bool fast = inv < INFINITY;                         // CTA-uniform; false for inf and NaN
    int sum = 0;
#pragma unroll 1
    for (int gi = threadIdx.x; gi < ngroups; gi += NTHR) {
        float f[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float4 v = reinterpret_cast<const float4 *>(h_s)[j * ngroups + gi];
            f[4 * j] = v.x; f[4 * j + 1] = v.y; f[4 * j + 2] = v.z; f[4 * j + 3] = v.w;
        }
        int q[16];
        if (fast) quant16<true>(f, inv, q); else quant16<false>(f, inv, q);
        put(q, gi, sum);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) part_i[warp * FUSED_MAX_M + m] = sum;
}

// The same CTA with the products on the integer ALUs (dp4a) instead of mma.sync: the form used for
// one token (the MT = 2 form of the template is kept but no longer dispatched).  Measured on this part: with eight warps and at most sixteen accumulator
// chains per warp the mma.sync form spends 1.5-2 us multiplying a 64-row slab (one sub-step of
// 16 MMAs, their 64 ANDs and 8 shared-memory loads takes ~800 cycles at two warps per scheduler),
// twice the time of this form, and its registers allow two CTAs per SM where this one fits three.
//
// Warp w owns rows 8w..8w+7 of the slab.  A lane owns one 32-bit word of packed weights (16 trits)
// per pass, the same word index for all eight rows: it loads the 16 bytes of quantised activations
// that belong to that word once per pass (consumption order: four words, one per position class)
// and then, per row, one 4-byte word of weights -- a warp reads 128 consecutive bytes of a row, so
// the unpadded slab is conflict-free -- and per class one AND (w & (0x03030303 << 2i) = the four
// codes of the class, scaled by 4^i) and one dp4a.u32.s32.  Row sums are reduced by shuffles.
template <typename T, int ROWS, int MT, int SRC>
__global__ void __launch_bounds__(BULK_THREADS, 3)
ternary_gemv_bulk_dp4a_kernel(const BulkParams p)
{
    using namespace sm100;
    static_assert(ROWS == 64 || ROWS == 32, "rows per CTA");
    constexpr int RT = ROWS / 16;                             // copy chunks (16 rows each)
    constexpr int KW = 64 / ROWS;                             // warps sharing a row set split the passes
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row_bytes = (int)(p.K >> 2);
    const int nwords = row_bytes >> 2;                        // 32-bit words (16 trits) per row
    const int qrow = (int)p.K;                                // bytes of one quantised token row, unpadded
    uint8_t *w_s = smem;
    uint8_t *q_s = smem + (size_t)ROWS * row_bytes;
    int *red = reinterpret_cast<int *>(q_s + (((size_t)p.M * qrow + 15) & ~(size_t)15));   // [8 warps][8 rows][FUSED_MAX_M] (KW > 1 only)
    float *part_f = reinterpret_cast<float *>(red + 8 * 32 * 4);          // [8][FUSED_MAX_M]
    int *part_i = reinterpret_cast<int *>(part_f + 8 * FUSED_MAX_M);      // [8][FUSED_MAX_M]
    uint64_t *bars = reinterpret_cast<uint64_t *>(part_i + 8 * FUSED_MAX_M);   // [RT]
    double *part_d = reinterpret_cast<double *>(bars + 4);                // [8][FUSED_MAX_M]
    // this CTA's projection: the first one, or the last sibling whose range the CTA index has reached
    const uint8_t *lw = p.w;
    void *ly = p.y;
    const float *lbias = p.bias;
    int64_t lN = p.N;
    float lws = p.weight_scale;
    unsigned cta0 = 0;
#pragma unroll
    for (int i = 0; i < BULK_MAX_LAYERS - 1; ++i) {
        if (i < p.nsib && blockIdx.x >= p.sib[i].first_cta) {
            lw = p.sib[i].w; ly = p.sib[i].y; lbias = p.sib[i].bias; lN = p.sib[i].N; lws = p.sib[i].weight_scale; cta0 = p.sib[i].first_cta;
        }
    }
    const int64_t n0 = (int64_t)(blockIdx.x - cta0) * ROWS;

    if (threadIdx.x == 0) {
#pragma unroll
        for (int r = 0; r < RT; ++r) mbar_init(smem_u32(bars + r), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            const int64_t first = n0 + 16 * r;
            const int64_t rows = lN - first < 16 ? lN - first : 16;
            if (rows > 0) {
                const uint32_t bytes = (uint32_t)(rows * row_bytes);
                mbar_arrive_expect_tx(smem_u32(bars + r), bytes);
                bulk_load(smem_u32(w_s + (size_t)16 * r * row_bytes), lw + first * row_bytes, bytes, smem_u32(bars + r));
            } else {
                mbar_arrive(smem_u32(bars + r));
            }
        }
    }
    // (The next kernel of the stream is released late, after the multiply: measured in chains of these
    // calls, an early release made the chain 25 % slower -- the dependents' CTAs and copies then crowd
    // this grid's own -- while a late one still hides their launch and prefetch under this grid's tail.)
    pdl_wait();

    // ---- quantise the token rows
    const int ngroups = (int)(p.K >> 4);
    float scale[MT];
    if (SRC == SRC_PLAIN) {                                   // registers hold a thread's groups between the two passes
        const T *x = reinterpret_cast<const T *>(p.x);
        constexpr int XG = MT == 1 ? 2 : 1;                   // groups per thread and token kept in registers
        float xv[MT][XG][16];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float mx = 0.0f;
            if (m < p.M) {
#pragma unroll
                for (int i = 0; i < XG; ++i) {
                    const int gi = i * BULK_THREADS + threadIdx.x;
                    if (gi < ngroups) { Group16<T>::load(x + (int64_t)m * p.K, gi, xv[m][i]); mx = absmax16(xv[m][i], mx); }
                }
                for (int gi = XG * BULK_THREADS + threadIdx.x; gi < ngroups; gi += BULK_THREADS) {
                    float f[16];
                    Group16<T>::load(x + (int64_t)m * p.K, gi, f);
                    mx = absmax16(f, mx);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            if (lane == 0) part_f[warp * FUSED_MAX_M + m] = mx;
        }
        __syncthreads();                                      // also publishes the barrier initialisation
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            scale[m] = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; ++w) scale[m] = fmaxf(scale[m], part_f[w * FUSED_MAX_M + m]);
            int sum = 0;
            if (m < p.M) {
                const float inv = __fdiv_rn(127.0f, scale[m]);
                const bool fast = inv < INFINITY;             // CTA-uniform; false for inf and NaN
                auto put = [&](const float (&f)[16], int gi) {
                    int q[16];
                    if (fast) quant16<true>(f, inv, q); else quant16<false>(f, inv, q);
                    *reinterpret_cast<uint4 *>(q_s + (size_t)m * qrow + (size_t)gi * 16) = pack_perm16(q, sum);
                };
#pragma unroll
                for (int i = 0; i < XG; ++i) {
                    const int gi = i * BULK_THREADS + threadIdx.x;
                    if (gi < ngroups) put(xv[m][i], gi);
                }
                for (int gi = XG * BULK_THREADS + threadIdx.x; gi < ngroups; gi += BULK_THREADS) {
                    float f[16];
                    Group16<T>::load(x + (int64_t)m * p.K, gi, f);
                    put(f, gi);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (lane == 0) part_i[warp * FUSED_MAX_M + m] = sum;
        }
        __syncthreads();
    } else {
        float *h_s = reinterpret_cast<float *>(part_d + 8 * FUSED_MAX_M);
#pragma unroll 1
        for (int m = 0; m < p.M; ++m)
            src_quantise_row<T, SRC, 8>(p, m, h_s, part_d, part_f, part_i, [&](const int (&q)[16], int gi, int &sum) {
                *reinterpret_cast<uint4 *>(q_s + (size_t)m * qrow + (size_t)gi * 16) = pack_perm16(q, sum);
            });
        __syncthreads();                                      // (the first one inside also published the barrier initialisation)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            scale[m] = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; ++w) scale[m] = fmaxf(scale[m], part_f[w * FUSED_MAX_M + m]);
        }
    }

    // ---- multiply: warp -> rows 8*(warp / KW) .. +7, passes warp % KW, + KW, ... (32 words per pass)
    const int rset = warp / KW, kw = warp % KW;
    const uint8_t *wr_s = w_s + (size_t)(8 * rset) * row_bytes;
    const int npass = (nwords + 31) >> 5;
    int tot[MT][8];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int r = 0; r < 8; ++r) tot[m][r] = 0;
    const bool landed = mbar_wait_warp(smem_u32(bars + (8 * rset) / 16), 0, 0x801);
    if (landed) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m >= p.M) break;
            int acc[8][4];
#pragma unroll
            for (int r = 0; r < 8; ++r)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[r][i] = 0;
            for (int ps = kw; ps < npass; ps += KW) {
                const int wi = 32 * ps + lane;
                if (wi < nwords) {
                    const uint4 xw = *reinterpret_cast<const uint4 *>(q_s + (size_t)m * qrow + (size_t)wi * 16);
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        const uint32_t ww = *reinterpret_cast<const uint32_t *>(wr_s + (size_t)r * row_bytes + (size_t)wi * 4);
                        acc[r][0] = dp4a_us(ww & 0xc0c0c0c0u, xw.x, acc[r][0]);
                        acc[r][1] = dp4a_us(ww & 0x30303030u, xw.y, acc[r][1]);
                        acc[r][2] = dp4a_us(ww & 0x0c0c0c0cu, xw.z, acc[r][2]);
                        acc[r][3] = dp4a_us(ww & 0x03030303u, xw.w, acc[r][3]);
                    }
                }
            }
            // class sums are exact multiples of 64, 16, 4, 1
#pragma unroll
            for (int r = 0; r < 8; ++r) tot[m][r] = (acc[r][0] >> 6) + (acc[r][1] >> 4) + (acc[r][2] >> 2) + acc[r][3];
        }
    }
    pdl_launch_dependents();
    // The 32 lanes of a warp hold partial sums of the same eight rows.  Transposing butterfly: at each of
    // the first three steps a lane keeps half of its rows and hands the other half to its partner, so the
    // eight sums cost 4 + 2 + 1 + 1 + 1 shuffles instead of forty (shuffles share one unit per SM and all
    // eight warps arrive here together).  Afterwards lane l holds the total of row 4*b4 + 2*b3 + b2 of l.
    int rowtot[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        int v4[4], v2[2];
        const bool hi16 = lane & 16, hi8 = lane & 8, hi4 = lane & 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int keep = hi16 ? tot[m][4 + i] : tot[m][i], give = hi16 ? tot[m][i] : tot[m][4 + i];
            v4[i] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int keep = hi8 ? v4[2 + i] : v4[i], give = hi8 ? v4[i] : v4[2 + i];
            v2[i] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
        }
        const int keep = hi4 ? v2[1] : v2[0], give = hi4 ? v2[0] : v2[1];
        int v = keep + __shfl_xor_sync(0xffffffffu, give, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        rowtot[m] = v;
    }
    const int myrow = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
    if (KW > 1) {                                             // K was split over KW warps: add through shared memory
        if ((lane & 3) == 0) {
#pragma unroll
            for (int m = 0; m < MT; ++m) red[(warp * 8 + myrow) * FUSED_MAX_M + m] = rowtot[m];
        }
        __syncthreads();
        if (kw != 0) return;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            rowtot[m] = 0;
#pragma unroll
            for (int w = 0; w < KW; ++w) rowtot[m] += red[((rset * KW + w) * 8 + myrow) * FUSED_MAX_M + m];
        }
    }
    // of the four lanes that hold a row's total, lane (l & 3) == m stores token m
    const int64_t n = n0 + 8 * rset + myrow;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        if ((lane & 3) == m && m < p.M && n < lN) {
            int rs = 0;
#pragma unroll
            for (int w = 0; w < 8; ++w) rs += part_i[w * FUSED_MAX_M + m];
            const int a = rowtot[m] - rs;
            const int64_t o = (int64_t)m * lN + n;
            if (p.acc_out) p.acc_out[o] = a;
            float v = bitlinear_finalize(a, scale[m], lws);
            if (lbias) v = __fadd_rn(v, lbias[n]);
            if (p.residual) v = __fadd_rn(v, p.residual[o]);
            store_out(ly, p.y_dtype, o, v);
        }
    }
}

// Scalar kernel for any K % 4 == 0: one thread per (token, output row), natural
// order int8 activations, byte loads.  Correctness path for odd shapes only.
__global__ void __launch_bounds__(128)
ternary_scalar_kernel(const uint8_t *__restrict__ w, const int8_t *__restrict__ q_plain,
                      const float *__restrict__ scale, void *y, int32_t *acc_out,
                      const float *bias, const float *residual, int64_t N, int64_t K, int y_dtype,
                      float weight_scale)
{
    pdl_wait();
    const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t tok = blockIdx.y;
    if (n >= N) return;
    const uint8_t *wr = w + n * (K >> 2);
    const int8_t *qr = q_plain + tok * K;
    int acc = 0;
    for (int64_t b = 0; b < (K >> 2); ++b) {
        const uint32_t by = wr[b];
        acc += (int)qr[4 * b + 0] * ((int)((by >> 6) & 3u) - 1);
        acc += (int)qr[4 * b + 1] * ((int)((by >> 4) & 3u) - 1);
        acc += (int)qr[4 * b + 2] * ((int)((by >> 2) & 3u) - 1);
        acc += (int)qr[4 * b + 3] * ((int)(by & 3u) - 1);
    }
    const int64_t o = tok * N + n;
    if (acc_out) acc_out[o] = acc;
    float v = bitlinear_finalize(acc, scale[tok], weight_scale);
    if (bias) v = __fadd_rn(v, bias[n]);
    if (residual) v = __fadd_rn(v, residual[o]);
    store_out(y, y_dtype, o, v);
}

template <int KW, int NT>
static int launch_gemv(const GemvParams &p, cudaStream_t st)
{
    GemvParams q = p;
    unsigned tiles = (unsigned)((p.N + 15) / 16);
    for (int i = 0; i < q.nsib; ++i) {
        q.sib[i].first_cta = tiles;
        tiles += (unsigned)((q.sib[i].N + 15) / 16);
    }
    cudaError_t e = launch_kernel(ternary_gemv_kernel<KW, NT, 4>, dim3(tiles), dim3(KW * 32), 0, st, q);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "ternary_gemv_kernel: %s", cudaGetErrorString(e));
    return check_launch("ternary_gemv_kernel");
}

// True when the streaming kernel can take the problem.
bool ternary_gemv_supported(const void *w, const void *q_perm, int64_t K)
{
    return (K % 64 == 0) && aligned16(w) && aligned16(q_perm);
}

// M <= 16 tokens, permuted-order activations.
int ternary_gemv_dispatch(const uint8_t *w, const int8_t *q_perm, const float *scale,
                          const int32_t *rowsum, int M, int64_t N, int64_t K, float weight_scale,
                          void *y, int y_dtype, int32_t *acc_out, const float *bias,
                          const float *residual, cudaStream_t st)
{
    GemvParams p{w, q_perm, scale, rowsum, y, acc_out, bias, residual, N, K, M, y_dtype, weight_scale, 0, {}};
    const int nsteps = (int)((K / 64 + 3) / 4);
    const bool wide = nsteps > 16;   // long rows: 8 warps split K
    if (M <= 8) return wide ? launch_gemv<8, 1>(p, st) : launch_gemv<4, 1>(p, st);
    return wide ? launch_gemv<8, 2>(p, st) : launch_gemv<4, 2>(p, st);
}

// Up to four projections of the same quantised rows in one launch (q/k/v, gate/up): ws[i] [Ns[i]][K/4], ys[i] [M][Ns[i]].
int ternary_gemv_multi_dispatch_q(int nl, const uint8_t *const *ws, const int64_t *Ns, const float *weight_scales, void *const *ys,
                                  const int8_t *q_perm, const float *scale, const int32_t *rowsum, int M, int64_t K, int y_dtype,
                                  cudaStream_t st)
{
    if (nl < 1 || nl > GEMV_MAX_LAYERS) return fail(NSLQ_ERR_ARG, "BitLinear: %d projections in one launch, at most %d", nl, GEMV_MAX_LAYERS);
    GemvParams p{ws[0], q_perm, scale, rowsum, ys[0], nullptr, nullptr, nullptr, Ns[0], K, M, y_dtype, weight_scales[0], nl - 1, {}};
    for (int i = 1; i < nl; ++i) p.sib[i - 1] = GemvParams::Sibling{ws[i], ys[i], Ns[i], weight_scales[i], 0u};
    const int nsteps = (int)((K / 64 + 3) / 4);
    const bool wide = nsteps > 16;
    if (M <= 8) return wide ? launch_gemv<8, 1>(p, st) : launch_gemv<4, 1>(p, st);
    return wide ? launch_gemv<8, 2>(p, st) : launch_gemv<4, 2>(p, st);
}

template <typename T, int KW, int TPC, int UNROLL = 4>
static int launch_fused(const FusedParams &p, cudaStream_t st)
{
    constexpr int NW = KW * TPC;
    const size_t smem = (((size_t)p.M * p.K + 15) & ~(size_t)15) + (size_t)NW * 32 * 4 * 4 + (size_t)NW * FUSED_MAX_M * 8 + FUSED_MAX_M * 8 + 64;
    static std::atomic<size_t> reserved[kMaxDevices];
    if (reserve_smem(ternary_gemv_fused_kernel<T, KW, TPC, UNROLL>, reserved, smem) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "ternary_gemv_fused_kernel: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(cudaGetLastError()));
    const unsigned ctas = (unsigned)((p.N + 16 * TPC - 1) / (16 * TPC));
    cudaError_t e = launch_kernel(ternary_gemv_fused_kernel<T, KW, TPC, UNROLL>, dim3(ctas), dim3(NW * 32), smem, st, p);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "ternary_gemv_fused_kernel: %s", cudaGetErrorString(e));
    return check_launch("ternary_gemv_fused_kernel");
}

template <typename T>
static int pick_fused(const FusedParams &p, cudaStream_t st)
{
    const int nsteps = (int)((p.K / 64 + 3) / 4);
    const bool wide = nsteps > 16;                    // long rows: 8 warps split K
    const int64_t tiles = (p.N + 15) / 16;
    // widest CTA that still leaves about one CTA per SM
    if (!wide) {
        if (tiles >= 4 * 120) return launch_fused<T, 4, 4>(p, st);
        if (tiles >= 2 * 120) return launch_fused<T, 4, 2>(p, st);
        return launch_fused<T, 4, 1>(p, st);
    }
    if (tiles >= 2 * 120) return launch_fused<T, 8, 2>(p, st);
    return launch_fused<T, 8, 1>(p, st);
}

static int bulk_rows(int64_t K)
{
    const int64_t row_bytes = K / 4;
    if (64 * row_bytes <= 64 * 1024) return 64;
    if (32 * row_bytes <= 96 * 1024) return 32;
    return 0;
}

static size_t bulk_smem(int rows, int M, int64_t K, bool staged_row = false)
{
    constexpr size_t nw = 8;
    return (size_t)rows * (K / 4) + (((size_t)M * K + 15) & ~(size_t)15) + nw * 32 * 4 * 4 + nw * FUSED_MAX_M * 8 + 4 * 8 +
           nw * FUSED_MAX_M * 8 + (staged_row ? (size_t)K * 4 : 0) + 64;
}

template <typename T, int ROWS, int MT, int SRC>
static int launch_bulk_dp4a(const BulkParams &p, cudaStream_t st)
{
    const size_t smem = bulk_smem(ROWS, p.M, p.K, SRC != SRC_PLAIN);
    static std::atomic<size_t> reserved[kMaxDevices];
    static std::atomic<int> carved[kMaxDevices];
    if (!carved[device_index()].load(std::memory_order_acquire)) {
        cudaFuncSetAttribute(ternary_gemv_bulk_dp4a_kernel<T, ROWS, MT, SRC>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        carved[device_index()].store(1, std::memory_order_release);
    }
    if (reserve_smem(ternary_gemv_bulk_dp4a_kernel<T, ROWS, MT, SRC>, reserved, smem) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "ternary_gemv_bulk_dp4a_kernel: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(cudaGetLastError()));
    BulkParams q = p;
    unsigned ctas = (unsigned)((p.N + ROWS - 1) / ROWS);
    for (int i = 0; i < q.nsib; ++i) {
        q.sib[i].first_cta = ctas;
        ctas += (unsigned)((q.sib[i].N + ROWS - 1) / ROWS);
    }
    cudaError_t e = launch_kernel(ternary_gemv_bulk_dp4a_kernel<T, ROWS, MT, SRC>, dim3(ctas), dim3(BULK_THREADS), smem, st, q);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "ternary_gemv_bulk_dp4a_kernel: %s", cudaGetErrorString(e));
    return check_launch("ternary_gemv_bulk_dp4a_kernel");
}

template <typename T, int SRC>
static int pick_bulk_src(const BulkParams &p, cudaStream_t st)
{
    // one token row in every form (see the callers for the measurements)
    if (p.M != 1) return fail(NSLQ_ERR_UNSUPPORTED, "BitLinear: the bulk-copy kernel takes one token row, not %d", p.M);
    return bulk_rows(p.K) == 64 ? launch_bulk_dp4a<T, 64, 1, SRC>(p, st) : launch_bulk_dp4a<T, 32, 1, SRC>(p, st);
}

template <typename T>
static int pick_bulk(const BulkParams &p, cudaStream_t st)
{
    if (p.src == SRC_RMSNORM) return pick_bulk_src<T, SRC_RMSNORM>(p, st);
    if (p.src == SRC_SWIGLU) return pick_bulk_src<T, SRC_SWIGLU>(p, st);
    return pick_bulk_src<T, SRC_PLAIN>(p, st);
}

// The bulk-copy kernel takes the call when the slab of its CTA and the quantised rows fit shared memory.
static bool bulk_supported(int M, int64_t K, bool staged_row = false)
{
    const int rows = bulk_rows(K);
    return M == 1 && rows != 0 && bulk_smem(rows, M, K, staged_row) <= 160 * 1024;
}

// Whether one token row goes to the bulk-copy kernel (and not to the older register-staged one) in ternary_gemv_fused_dispatch.
bool ternary_gemv_bulk_takes_one_row(int64_t K) { return bulk_supported(1, K); }

int ternary_gemv_status(int *out) { return sm100::read_wait_status(out); }

// x [M][K] in its own dtype, M <= 4 (callers pass M = 1), K % 64 == 0, 16-byte aligned x and w, M*K <= 160 KiB.
bool ternary_gemv_fused_supported(const void *w, const void *x, int64_t M, int64_t K)
{
    return M >= 1 && M <= FUSED_MAX_M && (K % 64 == 0) && aligned16(w) && aligned16(x) && M * K <= 160 * 1024;
}

static int bulk_by_dtype(const BulkParams &b, int x_dtype, cudaStream_t st)
{
    switch (x_dtype) {
    case NSLQ_DTYPE_F32: return pick_bulk<float>(b, st);
    case NSLQ_DTYPE_FP16: return pick_bulk<__half>(b, st);
    case NSLQ_DTYPE_BF16: return pick_bulk<__nv_bfloat16>(b, st);
    default: return fail(NSLQ_ERR_ARG, "BitLinear: x_dtype %d not in {F32,FP16,BF16}", x_dtype);
    }
}

// One token row whose RMSNorm (norm_w != null) or SiLU(x) * x2 (x2 != null) the CTAs form for themselves.
bool ternary_gemv_src_supported(const void *w, const void *x, const void *x2, const float *norm_w, int64_t M, int64_t K)
{
    return M == 1 && (K % 64 == 0) && aligned16(w) && aligned16(x) && (!x2 || aligned16(x2)) &&
           (!norm_w || aligned16(norm_w)) && bulk_supported((int)M, K, true);
}

int ternary_gemv_src_dispatch(const uint8_t *w, const void *x, const void *x2, const float *norm_w, double eps, int x_dtype,
                              int M, int64_t N, int64_t K, float weight_scale, void *y, int y_dtype, int32_t *acc_out,
                              const float *bias, const float *residual, cudaStream_t st)
{
    BulkParams b{w, x, y, acc_out, bias, residual, N, K, M, y_dtype, weight_scale,
                 norm_w ? SRC_RMSNORM : (x2 ? SRC_SWIGLU : SRC_PLAIN), x2, norm_w, eps, 0, {}};
    return bulk_by_dtype(b, x_dtype, st);
}

// The same for up to four projections of the same token rows in one launch (q/k/v, gate/up): ws[i] [N[i]][K/4],
// ys[i] [M][N[i]]; no accumulator output and no residual.  The callers have checked ternary_gemv_src_supported
// for every weight pointer.
int ternary_gemv_multi_dispatch(int nl, const uint8_t *const *ws, const int64_t *Ns, const float *weight_scales, const float *const *biases,
                                void *const *ys, const void *x, const float *norm_w, double eps, int x_dtype, int M, int64_t K,
                                int y_dtype, cudaStream_t st)
{
    if (nl < 1 || nl > BULK_MAX_LAYERS) return fail(NSLQ_ERR_ARG, "BitLinear: %d projections in one launch, at most %d", nl, BULK_MAX_LAYERS);
    BulkParams b{ws[0], x, ys[0], nullptr, biases[0], nullptr, Ns[0], K, M, y_dtype, weight_scales[0],
                 norm_w ? SRC_RMSNORM : SRC_PLAIN, nullptr, norm_w, eps, nl - 1, {}};
    for (int i = 1; i < nl; ++i) b.sib[i - 1] = BulkParams::Sibling{ws[i], ys[i], biases[i], Ns[i], weight_scales[i], 0u};
    return bulk_by_dtype(b, x_dtype, st);
}

int ternary_gemv_fused_dispatch(const uint8_t *w, const void *x, int x_dtype, int M, int64_t N, int64_t K,
                                float weight_scale, void *y, int y_dtype, int32_t *acc_out, const float *bias,
                                const float *residual, cudaStream_t st)
{
    if (bulk_supported(M, K)) {
        BulkParams b{w, x, y, acc_out, bias, residual, N, K, M, y_dtype, weight_scale, SRC_PLAIN, nullptr, nullptr, 0.0, 0, {}};
        return bulk_by_dtype(b, x_dtype, st);
    }
    FusedParams p{w, x, y, acc_out, bias, residual, N, K, M, y_dtype, weight_scale};
    switch (x_dtype) {
    case NSLQ_DTYPE_F32: return pick_fused<float>(p, st);
    case NSLQ_DTYPE_FP16: return pick_fused<__half>(p, st);
    case NSLQ_DTYPE_BF16: return pick_fused<__nv_bfloat16>(p, st);
    default: return fail(NSLQ_ERR_ARG, "BitLinear: x_dtype %d not in {F32,FP16,BF16}", x_dtype);
    }
}

int ternary_scalar_dispatch(const uint8_t *w, const int8_t *q_plain, const float *scale, int64_t M,
                            int64_t N, int64_t K, float weight_scale, void *y, int y_dtype,
                            int32_t *acc_out, const float *bias, const float *residual,
                            cudaStream_t st)
{
    dim3 grid((unsigned)((N + 127) / 128), (unsigned)M);
    if (M > 65535) return fail(NSLQ_ERR_UNSUPPORTED, "scalar BitLinear kernel: M=%lld > 65535", (long long)M);
    cudaError_t e = launch_kernel(ternary_scalar_kernel, grid, dim3(128), 0, st, w, q_plain, scale, y, acc_out, bias, residual,
                                  N, K, y_dtype, weight_scale);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "ternary_scalar_kernel: %s", cudaGetErrorString(e));
    return check_launch("ternary_scalar_kernel");
}

}  // namespace nslq
