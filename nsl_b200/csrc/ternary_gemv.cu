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
// For M <= 4 the activation quantisation is fused in (ternary_gemv_fused_kernel): each
// CTA issues its weight loads, then -- while they are in flight -- quantises the token
// rows itself (absmax by warp shuffles, the reference's exact rounding) into shared memory
// in the consumption order, so a decode-time linear is one launch and one trip to HBM.
//
// Also here: a scalar kernel for shapes the streaming kernel cannot take
// (K % 64 != 0 or unaligned rows); same arithmetic, natural-order activations.
#include "common.cuh"
#include "ternary_mma.cuh"

namespace nslq {

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
    const int64_t n0 = (int64_t)blockIdx.x * 16;
    const int64_t row_bytes = p.K >> 2;
    const int nchunks = (int)(p.K >> 6);            // 64 trits = 16 bytes per chunk
    const int nsteps = (nchunks + 3) >> 2;
    const bool rowa_ok = (n0 + g) < p.N, rowb_ok = (n0 + g + 8) < p.N;
    const uint8_t *wa = p.w + (n0 + g) * row_bytes;
    const uint8_t *wb = p.w + (n0 + g + 8) * row_bytes;

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
        if (tok >= p.M || n0 + row >= p.N) continue;
        const int nt = tok >> 3, tl = tok & 7;
        const int src_lane = (row & 7) * 4 + (tl >> 1);
        const int src_reg = ((row >> 3) << 1) | (tl & 1);
        int a = 0;
#pragma unroll
        for (int w = 0; w < KW; ++w) a += red[w][nt][src_lane][src_reg];
        a -= p.rowsum[tok];
        const int64_t o = (int64_t)tok * p.N + n0 + row;
        if (p.acc_out) p.acc_out[o] = a;
        float v = bitlinear_finalize(a, p.scale[tok], p.weight_scale);
        if (p.bias) v = __fadd_rn(v, p.bias[n0 + row]);
        if (p.residual) v = __fadd_rn(v, p.residual[o]);
        store_out(p.y, p.y_dtype, o, v);
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

// Decode kernel with the activation quantisation fused in (M <= 4).  A CTA owns TPC row tiles
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
    const unsigned tiles = (unsigned)((p.N + 15) / 16);
    cudaError_t e = launch_kernel(ternary_gemv_kernel<KW, NT, 4>, dim3(tiles), dim3(KW * 32), 0, st, p);
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
    GemvParams p{w, q_perm, scale, rowsum, y, acc_out, bias, residual, N, K, M, y_dtype, weight_scale};
    const int nsteps = (int)((K / 64 + 3) / 4);
    const bool wide = nsteps > 16;   // long rows: 8 warps split K
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

// x [M][K] in its own dtype, M <= 4, K % 64 == 0, 16-byte aligned x and w, M*K <= 160 KiB.
bool ternary_gemv_fused_supported(const void *w, const void *x, int64_t M, int64_t K)
{
    return M >= 1 && M <= FUSED_MAX_M && (K % 64 == 0) && aligned16(w) && aligned16(x) && M * K <= 160 * 1024;
}

int ternary_gemv_fused_dispatch(const uint8_t *w, const void *x, int x_dtype, int M, int64_t N, int64_t K,
                                float weight_scale, void *y, int y_dtype, int32_t *acc_out, const float *bias,
                                const float *residual, cudaStream_t st)
{
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
