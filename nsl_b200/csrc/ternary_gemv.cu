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
//     (w >> (6-2i)) & 0x03030303 = codes of k = 4j+i for byte j: four u8x4 MMA
//     operand registers per word, no per-trit work.  The quantised activations
//     are stored in the matching order (position 4i+j of every 16 holds k = 4j+i),
//     so registers line up with no shuffles;
//   * mma.sync.m16n8k32.u8.s8 accumulates sum_k q*code exactly in int32 for up to
//     8 tokens per MMA; acc = that - rowsum(q) because code = trit + 1;
//   * the K-split partials are reduced through shared memory and finalised as
//     ((scale/127) * (float)acc) * weight_scale with separately rounded steps
//     (crates/nsl-codegen/src/bitnet/phases/finalize.rs:39-53).
//
// Also here: a scalar kernel for shapes the streaming kernel cannot take
// (K % 64 != 0 or unaligned rows); same arithmetic, natural-order activations.
#include "common.cuh"

namespace nslq {

static __device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

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

    int acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[nt][r] = 0;

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
        if (!waited) { pdl_wait(); waited = true; }
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
            const uint32_t wwa[4] = {ra[u].x, ra[u].y, ra[u].z, ra[u].w};
            const uint32_t wwb[4] = {rb[u].x, rb[u].y, rb[u].z, rb[u].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t a_i0 = (wwa[j] >> 6) & 0x03030303u, a_i1 = (wwa[j] >> 4) & 0x03030303u;
                const uint32_t a_i2 = (wwa[j] >> 2) & 0x03030303u, a_i3 = wwa[j] & 0x03030303u;
                const uint32_t b_i0 = (wwb[j] >> 6) & 0x03030303u, b_i1 = (wwb[j] >> 4) & 0x03030303u;
                const uint32_t b_i2 = (wwb[j] >> 2) & 0x03030303u, b_i3 = wwb[j] & 0x03030303u;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint32_t x0 = xq[nt][j].x, x1 = xq[nt][j].y, x2 = xq[nt][j].z, x3 = xq[nt][j].w;
                    mma_u8s8(acc[nt], a_i0, b_i0, a_i1, b_i1, x0, x1);
                    mma_u8s8(acc[nt], a_i2, b_i2, a_i3, b_i3, x2, x3);
                }
            }
        }
    }
    if (!waited) pdl_wait();
    pdl_launch_dependents();

#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int r = 0; r < 4; ++r) red[warp][nt][lane][r] = acc[nt][r];
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
    ternary_gemv_kernel<KW, NT, 4><<<tiles, KW * 32, 0, st>>>(p);
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

int ternary_scalar_dispatch(const uint8_t *w, const int8_t *q_plain, const float *scale, int64_t M,
                            int64_t N, int64_t K, float weight_scale, void *y, int y_dtype,
                            int32_t *acc_out, const float *bias, const float *residual,
                            cudaStream_t st)
{
    dim3 grid((unsigned)((N + 127) / 128), (unsigned)M);
    if (M > 65535) return fail(NSLQ_ERR_UNSUPPORTED, "scalar BitLinear kernel: M=%lld > 65535", (long long)M);
    ternary_scalar_kernel<<<grid, 128, 0, st>>>(w, q_plain, scale, y, acc_out, bias, residual, N, K,
                                                y_dtype, weight_scale);
    return check_launch("ternary_scalar_kernel");
}

}  // namespace nslq
