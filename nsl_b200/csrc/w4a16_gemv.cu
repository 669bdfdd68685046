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

static __device__ __forceinline__ void cp_async_4(void *smem_dst, const void *gsrc)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
static __device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Decode kernel, persistent and software-pipelined (used when M*K*2 bytes of activations fit
// in shared memory).  Each CTA (8 warps splitting K) walks over row tiles of 16 outputs:
//   * once per CTA, while the first tile's weight loads are in flight, x is copied into shared
//     memory in the pair order the MMA B operand wants -- (x[i], x[i+4]) for i = 0..3 of every
//     8 -- and every 128-k step of every token is summed in fp32, so the main loop has no
//     byte-permutes and no all-ones MMAs:
//         y += scale * (D - (BIAS + zp) * xsum[step])     with D = sum (BIAS+q) * x  from the MMA;
//   * per tile, the next tile's weight loads (registers) and group tables (cp.async into the
//     other shared-memory buffer) are issued before the current tile's arithmetic, so HBM keeps
//     streaming while the tensor pipe works.
// Dynamic shared memory: [M*K 16-bit, pair order][nsteps][MT] xsum | [8][NT][32][4] reduce |
// 2 x [16][G] scale | 2 x [16][G] zero point | 64 zero bytes.
template <typename T, int NT, int UNROLL>
__global__ void __launch_bounds__(256, (NT == 1) ? 2 : 1)
w4a16_gemv_persistent_kernel(const W4Params p, const int ntiles)
{
    using TR = W4Traits<T>;
    constexpr int KW = 8, NTHR = 256, MT = 8 * NT;
    extern __shared__ __align__(16) uint8_t smem[];
    const int kw = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int nsteps = (int)(p.K >> 7);
    uint4 *x_s = reinterpret_cast<uint4 *>(smem);                                   // [M][K/8] uint4
    float *xsum_s = reinterpret_cast<float *>(smem + (size_t)p.M * p.K * 2);        // [nsteps][MT]
    float *red = xsum_s + (size_t)nsteps * MT;                                      // [KW][NT][32][4]
    float *scale_s = red + KW * NT * 32 * 4;                                        // [2][16][G]
    float *zc_s = scale_s + 2 * 16 * p.G;                                           // [2][16][G]
    uint4 *zero_s = reinterpret_cast<uint4 *>(zc_s + 2 * 16 * p.G);                 // 64 bytes of zeros
    const int64_t row_bytes = p.K >> 1;
    if (threadIdx.x < 4) zero_s[threadIdx.x] = make_uint4(0, 0, 0, 0);

    uint4 ra[UNROLL], rb[UNROLL], na[UNROLL], nb[UNROLL];
    auto load_weights = [&](int tile, int s0, uint4 (&da)[UNROLL], uint4 (&db)[UNROLL]) {
        const int64_t ra_n = (int64_t)tile * 16 + g, rb_n = ra_n + 8;
        const uint8_t *wa = p.codes + ra_n * row_bytes, *wb = p.codes + rb_n * row_bytes;
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int s = s0 + u * KW;
            const bool ok = s < nsteps;
            const int64_t off = ((int64_t)(4 * s + t)) * 16;
            da[u] = (ok && ra_n < p.N) ? ld_stream_u4(wa + off) : make_uint4(0, 0, 0, 0);
            db[u] = (ok && rb_n < p.N) ? ld_stream_u4(wb + off) : make_uint4(0, 0, 0, 0);
        }
    };
    auto load_tables = [&](int tile, int buf) {       // asynchronous: lands in shared memory on its own
        for (int i = threadIdx.x; i < 16 * p.G; i += NTHR) {
            const int64_t n = (int64_t)tile * 16 + i / p.G;
            if (n < p.N) {
                cp_async_4(scale_s + buf * 16 * p.G + i, p.scale + n * p.G + (i % p.G));
                cp_async_4(zc_s + buf * 16 * p.G + i, p.zc + n * p.G + (i % p.G));
            }
        }
    };

    int tile = blockIdx.x;
    load_weights(tile, kw, ra, rb);
    load_tables(tile, 0);
    pdl_launch_dependents();
    pdl_wait();

    // ---- stage x once: pair order + per-step sums (16 consecutive lanes cover one 128-k step)
    for (int i = threadIdx.x; i < nsteps * MT; i += NTHR) xsum_s[i] = 0.0f;   // tokens >= M stay 0
    const int vec_per_row = (int)(p.K >> 3);
    const int nvec = p.M * vec_per_row;
    const uint4 *xg = reinterpret_cast<const uint4 *>(p.x);
    __syncthreads();
    for (int base = 0; base < nvec; base += NTHR) {
        const int v = base + threadIdx.x;
        const bool in = v < nvec;
        const unsigned mask = __ballot_sync(0xffffffffu, in);   // whole half-warps: K % 128 == 0
        if (!in) continue;
        const uint4 xw = __ldg(xg + v);
        uint4 o;
        o.x = __byte_perm(xw.x, xw.z, 0x5410); o.y = __byte_perm(xw.x, xw.z, 0x7632);   // (x0,x4) (x1,x5)
        o.z = __byte_perm(xw.y, xw.w, 0x5410); o.w = __byte_perm(xw.y, xw.w, 0x7632);   // (x2,x6) (x3,x7)
        x_s[v] = o;
        const T *e = reinterpret_cast<const T *>(&xw);
        float sum = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) sum += Elem<T>::to_f32(e[k]);
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(mask, sum, off);
        if ((lane & 15) == 0) xsum_s[((v % vec_per_row) >> 4) * MT + v / vec_per_row] = sum;
    }
    cp_async_wait_all();
    __syncthreads();

    // Per-thread constants of the main loop.  A lane whose token does not exist reads a block of
    // zeros with stride 0, so the loop has no selects; steps and groups do not depend on the tile.
    const uint4 *xrow[NT];
    int xstride[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int tok = nt * 8 + g;
        const bool valid = tok < p.M;
        xrow[nt] = valid ? x_s + tok * vec_per_row + t * 4 : zero_s;
        xstride[nt] = valid ? 16 : 0;
    }
    const int spg_shift = 31 - __clz(p.gs >> 7);        // steps per group is a power of two (host check)
    const float2 *xsum2 = reinterpret_cast<const float2 *>(xsum_s) + t;

    int buf = 0;
    for (; tile < ntiles; tile += gridDim.x, buf ^= 1) {
        const int next = tile + gridDim.x;
        if (next < ntiles) {               // keep HBM busy during this tile's arithmetic
            load_weights(next, kw, na, nb);
            load_tables(next, buf ^ 1);
        }
        float yacc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int r = 0; r < 4; ++r) yacc[nt][r] = 0.0f;
        const float *sca = scale_s + (buf * 16 + g) * p.G, *scb = sca + 8 * p.G;
        const float *zca = zc_s + (buf * 16 + g) * p.G, *zcb = zca + 8 * p.G;

        for (int s0 = kw; s0 < nsteps; s0 += KW * UNROLL) {
            if (s0 != kw) load_weights(tile, s0, ra, rb);      // rows longer than one batch: not pipelined
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int s = s0 + u * KW;
                if (s >= nsteps) break;   // warp-uniform
                float d0[NT][4], d1[NT][4];    // two chains per token tile: consecutive MMAs do not wait on each other
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int r = 0; r < 4; ++r) { d0[nt][r] = 0.0f; d1[nt][r] = 0.0f; }
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
                        const uint4 xp = xrow[nt][s * xstride[nt] + j];
                        TR::mma(d0[nt], a[0], b[0], a[1], b[1], xp.x, xp.y);
                        TR::mma(d1[nt], a[2], b[2], a[3], b[3], xp.z, xp.w);
                    }
                }
                const int grp = s >> spg_shift;
                const float sa = sca[grp], sb = scb[grp];
                const float za = TR::BIAS + zca[grp], zb = TR::BIAS + zcb[grp];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const float2 xs = xsum2[(s * MT + nt * 8) >> 1];
                    yacc[nt][0] = fmaf(sa, (d0[nt][0] + d1[nt][0]) - za * xs.x, yacc[nt][0]);
                    yacc[nt][1] = fmaf(sa, (d0[nt][1] + d1[nt][1]) - za * xs.y, yacc[nt][1]);
                    yacc[nt][2] = fmaf(sb, (d0[nt][2] + d1[nt][2]) - zb * xs.x, yacc[nt][2]);
                    yacc[nt][3] = fmaf(sb, (d0[nt][3] + d1[nt][3]) - zb * xs.y, yacc[nt][3]);
                }
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int r = 0; r < 4; ++r) red[((kw * NT + nt) * 32 + lane) * 4 + r] = yacc[nt][r];
        __syncthreads();
        for (int e = threadIdx.x; e < 16 * MT; e += NTHR) {
            const int row = e & 15, tok = e >> 4;
            const int64_t n = (int64_t)tile * 16 + row;
            if (tok >= p.M || n >= p.N) continue;
            const int nt = tok >> 3, tk = tok & 7;
            const int src_lane = (row & 7) * 4 + (tk >> 1);
            const int src_reg = ((row >> 3) << 1) | (tk & 1);
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < KW; ++w) v += red[((w * NT + nt) * 32 + src_lane) * 4 + src_reg];
            store_out(p.y, p.y_dtype, (int64_t)tok * p.N + n, v);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) { ra[u] = na[u]; rb[u] = nb[u]; }
        cp_async_wait_all();               // the next tile's tables have landed
        __syncthreads();                   // ... for every thread; and the reduce area is free again
    }
}

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

static int sm_count_cached() { return sm_count_current(); }

template <typename T, int NT>
static int launch_w4_persistent(const W4Params &p, size_t smem, cudaStream_t st)
{
    static std::atomic<size_t> reserved[kMaxDevices];
    if (reserve_smem(w4a16_gemv_persistent_kernel<T, NT, 4>, reserved, smem) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "w4a16_gemv_persistent_kernel: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(cudaGetLastError()));
    const int ntiles = (int)((p.N + 15) / 16);
    const int per_sm = (NT == 1 && smem <= 100 * 1024) ? 2 : 1;
    const int slots = sm_count_cached() * per_sm;
    const int grid = ntiles < slots ? ntiles : slots;
    cudaError_t e = launch_kernel(w4a16_gemv_persistent_kernel<T, NT, 4>, dim3(grid), dim3(256), smem, st, p, ntiles);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "w4a16_gemv_persistent_kernel: %s", cudaGetErrorString(e));
    return check_launch("w4a16_gemv_persistent_kernel");
}

// Persistent kernel when the activations (and the small tables) fit in shared memory; else the
// kernel that reads them from global memory.
template <typename T>
static int pick_w4(const W4Params &p, cudaStream_t st)
{
    const int nsteps = (int)(p.K / 128);
    const int NT = p.M > 8 ? 2 : 1;
    const size_t smem = (size_t)p.M * p.K * 2 + (size_t)nsteps * 8 * NT * 4 + (size_t)8 * NT * 32 * 4 * 4 +
                        (size_t)4 * 16 * p.G * 4 + 64;
    const int spg = p.gs / 128;
    if (smem <= 200 * 1024 && p.N < (1ll << 31) && (spg & (spg - 1)) == 0)
        return NT == 1 ? launch_w4_persistent<T, 1>(p, smem, st) : launch_w4_persistent<T, 2>(p, smem, st);
    return launch_w4<T>(p, st);
}

int w4a16_gemv_dispatch(const uint8_t *codes, const float *scale, const float *zc, int64_t N, int64_t K,
                        int G, int gs, const void *x, int x_dtype, int M, void *y, int y_dtype,
                        cudaStream_t st)
{
    W4Params p{codes, scale, zc, x, y, N, K, G, gs, M, y_dtype};
    if (x_dtype == NSLQ_DTYPE_BF16) return pick_w4<__nv_bfloat16>(p, st);
    return pick_w4<__half>(p, st);
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
