// Stage 2: W4A16 decode GEMV/skinny GEMM for M <= 16 tokens.
//
// HBM-bound weight streaming, same skeleton as the ternary GEMV: a CTA owns 16
// output rows, its warps split K in steps of 128 (4 lanes of a quad x 32 codes =
// one uint4 each, rows g and g+8), all weight loads of a batch are issued before
// any arithmetic.  Codes are [N][K/2] bytes, low nibble = even k
// (crates/nsl-runtime/src/quantize.rs:187-216).
//
// In-register unpack: for a 32-bit word w (8 codes), ((w >> 4i) & 0x000F000F) |
// MAGIC is a pair of 16-bit floats (BIAS+q[i], BIAS+q[i+4]) -- BIAS = 128 for
// bf16 (0x4300), 1024 for fp16 (0x6400) -- i.e. a ready MMA A register for one
// lop3.  The matching activation pair (x[i], x[i+4]) is one byte-permute of the
// 16-bit activations as they sit in memory.  mma.sync.m16n8k16 accumulates
// D = sum (BIAS+q)*x in fp32 and, with an all-ones A operand, X = sum x; per
// 128-k step   y += scale * (D - (BIAS + zp) * X)
// which is sum (q - zp) * scale * x, the reference dequantisation
// (crates/nsl-runtime/src/quantize.rs:263-266) with fp32 accumulation.
//
// Also here: a scalar kernel for any group size / K / activation dtype (f64
// accumulation), the correctness path for shapes the streaming kernel cannot take.
#include "common.cuh"

namespace nslq {

template <typename T> struct W4Traits;
template <> struct W4Traits<__nv_bfloat16> {
    static constexpr uint32_t MAGIC = 0x43004300u, ONES = 0x3F803F80u;
    static constexpr float BIAS = 128.0f;
    static __device__ __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
};
template <> struct W4Traits<__half> {
    static constexpr uint32_t MAGIC = 0x64006400u, ONES = 0x3C003C00u;
    static constexpr float BIAS = 1024.0f;
    static __device__ __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
};

struct W4Params {
    const uint8_t *codes;  // [N][K/2]
    const float *scale;    // [N][G]
    const float *zc;       // [N][G] zero point in code units
    const void *x;         // [M][K] 16-bit
    void *y;               // [M][N]
    int64_t N, K;
    int G, gs, M, y_dtype;
};

template <typename T, int KW, int NT, int UNROLL>
__global__ void __launch_bounds__(KW * 32)
w4a16_gemv_kernel(const W4Params p)
{
    using TR = W4Traits<T>;
    __shared__ float red[KW][NT][32][4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t n0 = (int64_t)blockIdx.x * 16;
    const int64_t row_bytes = p.K >> 1;
    const int nsteps = (int)(p.K >> 7);             // 128 k per step
    const int64_t ra_n = n0 + g, rb_n = n0 + g + 8;
    const bool rowa_ok = ra_n < p.N, rowb_ok = rb_n < p.N;
    const uint8_t *wa = p.codes + ra_n * row_bytes;
    const uint8_t *wb = p.codes + rb_n * row_bytes;
    const uint16_t *xbase = reinterpret_cast<const uint16_t *>(p.x);

    float yacc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int r = 0; r < 4; ++r) yacc[nt][r] = 0.0f;

    bool waited = false;
    for (int s0 = warp; s0 < nsteps; s0 += KW * UNROLL) {
        uint4 ra[UNROLL], rb[UNROLL];
        float sa[UNROLL], sb[UNROLL], za[UNROLL], zb[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int s = s0 + u * KW;
            const bool ok = s < nsteps;
            const int64_t off = ((int64_t)(4 * s + t)) * 16;
            ra[u] = (ok && rowa_ok) ? ld_stream_u4(wa + off) : make_uint4(0, 0, 0, 0);
            rb[u] = (ok && rowb_ok) ? ld_stream_u4(wb + off) : make_uint4(0, 0, 0, 0);
            const int grp = ok ? (s * 128) / p.gs : 0;
            sa[u] = (ok && rowa_ok) ? __ldg(p.scale + ra_n * p.G + grp) : 0.0f;
            sb[u] = (ok && rowb_ok) ? __ldg(p.scale + rb_n * p.G + grp) : 0.0f;
            za[u] = (ok && rowa_ok) ? __ldg(p.zc + ra_n * p.G + grp) : 0.0f;
            zb[u] = (ok && rowb_ok) ? __ldg(p.zc + rb_n * p.G + grp) : 0.0f;
        }
        if (!waited) { pdl_wait(); waited = true; }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int s = s0 + u * KW;
            if (s >= nsteps) break;   // warp-uniform
            uint4 xv[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int tok = nt * 8 + g;
                const uint4 *src = reinterpret_cast<const uint4 *>(xbase + (int64_t)tok * p.K + (int64_t)(4 * s + t) * 32);
#pragma unroll
                for (int j = 0; j < 4; ++j) xv[nt][j] = (tok < p.M) ? __ldg(src + j) : make_uint4(0, 0, 0, 0);
            }
            float d[NT][4], xs[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int r = 0; r < 4; ++r) { d[nt][r] = 0.0f; xs[nt][r] = 0.0f; }
            const uint32_t wwa[4] = {ra[u].x, ra[u].y, ra[u].z, ra[u].w};
            const uint32_t wwb[4] = {rb[u].x, rb[u].y, rb[u].z, rb[u].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t a[4], b[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    a[i] = ((wwa[j] >> (4 * i)) & 0x000F000Fu) | TR::MAGIC;
                    b[i] = ((wwb[j] >> (4 * i)) & 0x000F000Fu) | TR::MAGIC;
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint32_t xw[4] = {xv[nt][j].x, xv[nt][j].y, xv[nt][j].z, xv[nt][j].w};
                    // pair i = (x[8j+i], x[8j+i+4])
                    const uint32_t x0 = __byte_perm(xw[0], xw[2], 0x5410), x1 = __byte_perm(xw[0], xw[2], 0x7632);
                    const uint32_t x2 = __byte_perm(xw[1], xw[3], 0x5410), x3 = __byte_perm(xw[1], xw[3], 0x7632);
                    TR::mma(d[nt], a[0], b[0], a[1], b[1], x0, x1);
                    TR::mma(d[nt], a[2], b[2], a[3], b[3], x2, x3);
                    TR::mma(xs[nt], TR::ONES, TR::ONES, TR::ONES, TR::ONES, x0, x1);
                    TR::mma(xs[nt], TR::ONES, TR::ONES, TR::ONES, TR::ONES, x2, x3);
                }
            }
            const float zba = TR::BIAS + za[u], zbb = TR::BIAS + zb[u];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                yacc[nt][0] = fmaf(sa[u], d[nt][0] - zba * xs[nt][0], yacc[nt][0]);
                yacc[nt][1] = fmaf(sa[u], d[nt][1] - zba * xs[nt][1], yacc[nt][1]);
                yacc[nt][2] = fmaf(sb[u], d[nt][2] - zbb * xs[nt][2], yacc[nt][2]);
                yacc[nt][3] = fmaf(sb[u], d[nt][3] - zbb * xs[nt][3], yacc[nt][3]);
            }
        }
    }
    if (!waited) pdl_wait();
    pdl_launch_dependents();

#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int r = 0; r < 4; ++r) red[warp][nt][lane][r] = yacc[nt][r];
    __syncthreads();

    for (int e = threadIdx.x; e < 16 * 8 * NT; e += KW * 32) {
        const int row = e & 15, tok = e >> 4;
        if (tok >= p.M || n0 + row >= p.N) continue;
        const int nt = tok >> 3, tl = tok & 7;
        const int src_lane = (row & 7) * 4 + (tl >> 1);
        const int src_reg = ((row >> 3) << 1) | (tl & 1);
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < KW; ++w) v += red[w][nt][src_lane][src_reg];
        store_out(p.y, p.y_dtype, (int64_t)tok * p.N + n0 + row, v);
    }
}

// Note on the pair order above: pair index i of word j is (code 8j+i, code 8j+i+4);
// the activations x[8j .. 8j+7] sit in words xw[0..3] = (x0,x1),(x2,x3),(x4,x5),(x6,x7),
// so pair 0 = low halves of xw[0],xw[2]; pair 1 = high halves of xw[0],xw[2];
// pair 2 = low halves of xw[1],xw[3]; pair 3 = high halves of xw[1],xw[3].

// Scalar kernel: any K, any group size, x in F32/FP16/BF16, f64 accumulation.
template <typename T>
__global__ void __launch_bounds__(128)
w4a16_scalar_kernel(const uint8_t *__restrict__ codes, const float *__restrict__ scale,
                    const float *__restrict__ zc, const T *__restrict__ x, void *y, int64_t N,
                    int64_t K, int G, int gs, int y_dtype)
{
    pdl_wait();
    const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t tok = blockIdx.y;
    if (n >= N) return;
    double acc = 0.0;
    for (int64_t k = 0; k < K; ++k) {
        const int64_t flat = n * K + k;
        const uint8_t by = codes[flat >> 1];
        const int q = (flat & 1) ? (by >> 4) : (by & 15);
        const int gi = (int)(k / gs);
        const double wv = ((double)q - (double)zc[n * G + gi]) * (double)scale[n * G + gi];
        acc += (double)Elem<T>::to_f32(x[tok * K + k]) * wv;
    }
    store_out(y, y_dtype, tok * N + n, (float)acc);
}

bool w4a16_gemv_supported(const void *codes, const void *x, int x_dtype, int64_t K, int64_t gs)
{
    return (x_dtype == NSLQ_DTYPE_BF16 || x_dtype == NSLQ_DTYPE_FP16) && (K % 128 == 0) &&
           (gs % 128 == 0) && aligned16(codes) && aligned16(x);
}

template <typename T>
static int launch_w4(const W4Params &p, cudaStream_t st)
{
    const unsigned tiles = (unsigned)((p.N + 15) / 16);
    const int nsteps = (int)(p.K / 128);
    if (p.M <= 8) {
        if (nsteps > 32) w4a16_gemv_kernel<T, 8, 1, 4><<<tiles, 256, 0, st>>>(p);
        else w4a16_gemv_kernel<T, 4, 1, 4><<<tiles, 128, 0, st>>>(p);
    } else {
        if (nsteps > 32) w4a16_gemv_kernel<T, 8, 2, 4><<<tiles, 256, 0, st>>>(p);
        else w4a16_gemv_kernel<T, 4, 2, 4><<<tiles, 128, 0, st>>>(p);
    }
    return check_launch("w4a16_gemv_kernel");
}

int w4a16_gemv_dispatch(const uint8_t *codes, const float *scale, const float *zc, int64_t N, int64_t K,
                        int G, int gs, const void *x, int x_dtype, int M, void *y, int y_dtype,
                        cudaStream_t st)
{
    W4Params p{codes, scale, zc, x, y, N, K, G, gs, M, y_dtype};
    if (x_dtype == NSLQ_DTYPE_BF16) return launch_w4<__nv_bfloat16>(p, st);
    return launch_w4<__half>(p, st);
}

int w4a16_scalar_dispatch(const uint8_t *codes, const float *scale, const float *zc, int64_t N, int64_t K,
                          int G, int gs, const void *x, int x_dtype, int64_t M, void *y, int y_dtype,
                          cudaStream_t st)
{
    if (M > 65535) return fail(NSLQ_ERR_UNSUPPORTED, "scalar W4A16 kernel: M=%lld > 65535", (long long)M);
    dim3 grid((unsigned)((N + 127) / 128), (unsigned)M);
    switch (x_dtype) {
    case NSLQ_DTYPE_F32: w4a16_scalar_kernel<float><<<grid, 128, 0, st>>>(codes, scale, zc, (const float *)x, y, N, K, G, gs, y_dtype); break;
    case NSLQ_DTYPE_FP16: w4a16_scalar_kernel<__half><<<grid, 128, 0, st>>>(codes, scale, zc, (const __half *)x, y, N, K, G, gs, y_dtype); break;
    case NSLQ_DTYPE_BF16: w4a16_scalar_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(codes, scale, zc, (const __nv_bfloat16 *)x, y, N, K, G, gs, y_dtype); break;
    default: return fail(NSLQ_ERR_ARG, "W4A16: x_dtype %d not in {F32,FP16,BF16}", x_dtype);
    }
    return check_launch("w4a16_scalar_kernel");
}

}  // namespace nslq
