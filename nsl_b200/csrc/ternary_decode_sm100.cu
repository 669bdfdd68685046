// Stage 2 on the 5th-generation tensor cores: BitLinear decode (M <= 16 tokens) as a weight stream.
//
//   acc[m,n] = sum_k q[m,k] * W[n,k]        int8 x ternary, exact int32
//
// A decode-time linear reads every packed weight byte once; what limits it on this part is not
// HBM but the instructions spent per byte.  The mma.sync formulation costs ~200 issued
// instructions per KiB of packed weights (the legacy MMA expands to several instructions each,
// plus one AND per operand register); this kernel spends ~40: the packed bytes are expanded with
// one AND per 32-bit word and class, stored to TENSOR memory with tcgen05.st and multiplied by
// tcgen05.mma with the weights as the 128-row M-side operand and the (at most 16) tokens as N.
//
//   w & (0x03030303 << (6-2i)) is the four codes {0,1,2} of trit position i of the word's four
//   bytes, times 4^(3-i): still a valid u8.  The four position classes go to four separate
//   accumulators (4 x 16 TMEM columns), each the exact sum times its scale; the epilogue shifts
//   them back and adds them.  The token operand is laid out to match: inside a block of 128 k,
//   position 32i + 4g + b holds k = 16g + 4b + i, so MMA number i of the block (K = 32) sees
//   class i of all eight packed words.
//
// Persistent, warp-specialised, one CTA per SM, tiles of 128 weight rows:
//   warp 0      TMA producer: per step ONE cp.async.bulk.tensor copy (this CTA only) of 128 rows x
//               128 packed bytes (512 k), SWIZZLE_128B so that the per-row reads of the unpack
//               threads are conflict-free; a ring of up to 8 stages (128 KiB in flight per SM).
//   warps 8-15  unpack, two groups of four warps on alternate steps: a thread owns a weight row,
//               reads its 128 bytes, ANDs out 4 x 32 words per 128 k and stores them to its TMEM
//               lane (tcgen05.st.x32 four times).
//   warp 1      MMA issuer (converged warp, elected lane): 16 tcgen05.mma.kind::i8 (M=128, N=16,
//               K=32) per step, A = codes in TMEM, B = tokens resident in shared memory
//               (K-major, 128-byte swizzle), one commit per step.
//   warps 4-7   epilogue: tcgen05.ld the four class accumulators (double-buffered), combine,
//               subtract the token's row sum (code = trit + 1), ((scale/127)*acc)*weight_scale
//               with separately rounded steps, store (32 lanes = 32 consecutive n of one token).
//   warps 1,3-7 first stage the tokens: either copy already-quantised int8 (consumption order) or
//               (one or two tokens) quantise fp32/fp16/bf16 rows in place (absmax, the reference's
//               rounding, row sums), while the weights are already streaming and being unpacked
//               -- only the MMAs wait for them.
//
// Every mbarrier wait is bounded in time; on expiry the kernel records a status word and falls
// through to the common teardown, which frees its TMEM.
#include <type_traits>

#include "sm100_common.cuh"

namespace nslq {

namespace dec {

using namespace sm100;

constexpr int BW = 128;                  // weight rows per tile = MMA M = TMEM lanes
constexpr int NTOK = 16;                 // MMA N: token slots
constexpr int THREADS = 512;
constexpr int KS = 4;                    // 128-k blocks per pipeline step
constexpr int PK_ROW = KS * 32;          // packed bytes per row and step = one swizzle line
constexpr int P_BYTES = BW * PK_ROW;     // 16 KiB per stage
constexpr int A_COLS = KS * 32;          // TMEM columns per operand stage
constexpr int AS = 3;                    // operand stages: columns 128..511
constexpr int ACC_COLS = 4 * NTOK;       // four classes; two buffers at columns 0 and 64
constexpr int MAX_TS = 8;
constexpr int ND = 16;                   // ring of "step retired" barriers, > MAX_TS
constexpr int XB_BYTES = NTOK * 128;     // token operand of one 128-k block: 2 KiB
constexpr int SWARPS = 6;                // warps 1 and 3..7 stage the tokens (warp 2 allocates TMEM meanwhile)
constexpr int FUSED_MAX_M = 2;           // beyond that every CTA repeating the quantisation costs more than a launch
constexpr int SW = SWARPS * 32;
constexpr uint32_t IDESC = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(NTOK >> 3) << 17) | ((uint32_t)(BW >> 4) << 24);

struct Params {
    const uint8_t *w;        // [N][K/4]
    const void *x;           // [M][K] fp32/fp16/bf16 (fused quantisation) or null
    const int8_t *q;         // [M][K] consumption order (position 4i+j of every 16 holds k = 4j+i), when x is null
    const float *scale;      // [M], when x is null
    const int32_t *rowsum;   // [M], when x is null
    void *y;                 // [M][N]
    int32_t *acc_out;        // [M][N] or null
    const float *bias;       // [N] or null
    const float *residual;   // [M][N] or null
    int64_t N, K;
    int M, y_dtype;
    float weight_scale;
    int ts, nkb, nsteps, ntiles;
    int off_ring, off_misc, off_bar;
};

static __device__ __forceinline__ void stage_sync() { asm volatile("bar.sync 1, %0;" ::"n"(SW) : "memory"); }

// byte offset of position p (multiple of 4) of token r in the token operand of one 128-k block
static __device__ __forceinline__ int xs_off(int r, int p)
{
    return (r >> 3) * 1024 + (r & 7) * 128 + ((((p >> 4) ^ (r & 7)) << 4) | (p & 15));
}

template <typename XT>
__global__ void __launch_bounds__(THREADS, 1)
ternary_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                  // 1024-byte aligned (swizzle atom)
    uint8_t *base_ptr = smem_raw + (base - raw);
    // [token operand: nkb x 2 KiB][ring: ts x 16 KiB][misc][barriers]
    const uint32_t ring = base + p.off_ring;
    float *scale_s = reinterpret_cast<float *>(base_ptr + p.off_misc);
    int *rowsum_s = reinterpret_cast<int *>(scale_s + NTOK);
    float *part_f = reinterpret_cast<float *>(rowsum_s + NTOK);     // [16 warps]
    int *part_i = reinterpret_cast<int *>(part_f + 16);
    const uint32_t bars = base + p.off_bar;
    auto raw_bar = [&](int t) { return bars + 8u * t; };
    auto pfree_bar = [&](int t) { return bars + 8u * (MAX_TS + t); };
    auto afull_bar = [&](int a) { return bars + 8u * (2 * MAX_TS + a); };
    auto done_bar = [&](uint32_t i) { return bars + 8u * (2 * MAX_TS + AS + (i & (ND - 1))); };
    auto done_par = [&](uint32_t i) { return (i / ND) & 1u; };
    auto accf_bar = [&](int b) { return bars + 8u * (2 * MAX_TS + AS + ND + b); };
    auto acce_bar = [&](int b) { return bars + 8u * (2 * MAX_TS + AS + ND + 2 + b); };
    const uint32_t tmem_bar = bars + 8u * (2 * MAX_TS + AS + ND + 4);      // TMEM allocated, address published
    constexpr int NBAR = 2 * MAX_TS + AS + ND + 5;
    const uint32_t slot = bars + 8u * NBAR;
    volatile uint32_t *slot_ptr = reinterpret_cast<volatile uint32_t *>(base_ptr + p.off_bar + 8 * NBAR);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int my_tiles = (int)blockIdx.x < p.ntiles ? (p.ntiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (threadIdx.x == 0) {
        for (int t = 0; t < p.ts; ++t) { mbar_init(raw_bar(t), 1); mbar_init(pfree_bar(t), 4); }
        for (int a = 0; a < AS; ++a) mbar_init(afull_bar(a), 4);
        for (int i = 0; i < ND; ++i) mbar_init(done_bar(i), 1);
        for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), 128); }
        mbar_init(tmem_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // The allocation takes ~1000 cycles; warp 2 does nothing else, while the producer already
    // streams and the staging warps already load the tokens.  Whoever touches TMEM waits for tmem_bar first.
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(slot) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tmem_bar);
    }
    uint32_t tmem_base = 0;
    bool tmem_ok = true;
    auto get_tmem = [&]() {                                          // warp-uniform
        tmem_ok = mbar_wait_warp(tmem_bar, 0, 0x640);
        tc_fence_after();
        tmem_base = *slot_ptr;
    };

    if (warp == 0) {
        // ---------------- TMA producer.  The weights do not depend on the preceding kernel of the
        // stream, so this warp neither waits for it nor delays the next one.
        pdl_launch_dependents();
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0, it = 0;
            bool ok = true;
            for (int j = 0; j < my_tiles && ok; ++j) {
                const int n0 = ((int)blockIdx.x + j * (int)gridDim.x) * BW;
                for (int st = 0; st < p.nsteps; ++st, ++it) {
                    if (it >= (uint32_t)p.ts) {        // the stage's previous user: step it - ts
                        if (!(ok = mbar_wait(done_bar(it - p.ts), done_par(it - p.ts), 0x601))) break;
                        if (!(ok = mbar_wait(pfree_bar(s), ph ^ 1u, 0x602))) break;
                    }
                    mbar_arrive_expect_tx(raw_bar(s), P_BYTES);
                    tma_load_2d(ring + s * P_BYTES, &tmap_w, st * PK_ROW, n0, raw_bar(s));
                    if (++s == p.ts) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else {
        if (warp < 8 && warp != 2) {
            // ---------------- the tokens into shared memory (warps 1, 3..7)
            pdl_wait();
            const int wq = warp == 1 ? 0 : warp - 2, tq = wq * 32 + lane;
            if constexpr (std::is_void<XT>::value) {
                // q holds, per group of 16 k, four words: word i = class i of the group's four bytes
                const int groups16 = (int)(p.K >> 4), all = groups16 * p.M;
                const uint4 *src = reinterpret_cast<const uint4 *>(p.q);
                // (token, group) of this thread's element, advanced by SW per element: no division in the loop
                int m = tq / groups16, gg = tq - m * groups16;
                const int adv_m = SW / groups16, adv_g = SW - adv_m * groups16;
#pragma unroll 4
                for (int e = tq; e < all; e += SW) {
                    const int kb = gg >> 3, g = gg & 7;
                    const uint4 v = __ldg(src + e);
                    uint8_t *blk = base_ptr + (size_t)kb * XB_BYTES;
                    *reinterpret_cast<uint32_t *>(blk + xs_off(m, 4 * g)) = v.x;
                    *reinterpret_cast<uint32_t *>(blk + xs_off(m, 32 + 4 * g)) = v.y;
                    *reinterpret_cast<uint32_t *>(blk + xs_off(m, 64 + 4 * g)) = v.z;
                    *reinterpret_cast<uint32_t *>(blk + xs_off(m, 96 + 4 * g)) = v.w;
                    m += adv_m;
                    gg += adv_g;
                    if (gg >= groups16) { gg -= groups16; ++m; }
                }
                if (tq < p.M) { scale_s[tq] = p.scale[tq]; rowsum_s[tq] = p.rowsum[tq]; }
            } else {
                // same arithmetic as act_quant_kernel
                const XT *x = reinterpret_cast<const XT *>(p.x);
                const int nvec = (int)(p.K >> 2);
                // quantise vec4 v of token m (lane i of a quad gets class i of the quad's four bytes,
                // k = 16g + 4b + i) and return the four values' sum
                auto quant_f4 = [&](const float4 &f, int m, int v, float inv, bool zero_row, unsigned mask) {
                    const int q0 = zero_row ? 0 : quant_one(f.x, inv), q1 = zero_row ? 0 : quant_one(f.y, inv);
                    const int q2 = zero_row ? 0 : quant_one(f.z, inv), q3 = zero_row ? 0 : quant_one(f.w, inv);
                    const uint32_t wcls = quad_transpose(pack4_i8(q0, q1, q2, q3), mask);
                    const int kb = v >> 5, g = (v & 31) >> 2, i = v & 3;
                    *reinterpret_cast<uint32_t *>(base_ptr + (size_t)kb * XB_BYTES + xs_off(m, 32 * i + 4 * g)) = wcls;
                    return q0 + q1 + q2 + q3;
                };
                auto quant_vec = [&](const XT *xr, int m, int v, float inv, bool zero_row, unsigned mask) {
                    return quant_f4(Vec4<XT>::load(xr, v), m, v, inv, zero_row, mask);
                };
                auto absmax4 = [&](const XT *xr, int v0, int step) {   // several loads in flight per lane
                    float mx = 0.0f;
                    int v = v0;
                    for (; v + 3 * step < nvec; v += 4 * step) {
                        float4 f[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) f[i] = Vec4<XT>::load(xr, v + i * step);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(f[i].x), fabsf(f[i].y)), fmaxf(fabsf(f[i].z), fabsf(f[i].w))));
                    }
                    for (; v < nvec; v += step) {
                        const float4 f = Vec4<XT>::load(xr, v);
                        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w))));
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                    return mx;
                };
                if (p.M <= 2) {
                    // all six staging warps on a row; the first XV vec4 of every thread stay in registers
                    // between the absmax pass and the rounding pass (K <= XV*4*SW: the whole row)
                    constexpr int XV = 4;
                    for (int m = 0; m < p.M; ++m) {
                        const XT *xr = x + (int64_t)m * p.K;
                        float4 xv[XV];
                        float mx = 0.0f;
#pragma unroll
                        for (int i = 0; i < XV; ++i) {
                            const int v = i * SW + tq;
                            xv[i] = v < nvec ? Vec4<XT>::load(xr, v) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
#pragma unroll
                        for (int i = 0; i < XV; ++i)
                            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(xv[i].x), fabsf(xv[i].y)), fmaxf(fabsf(xv[i].z), fabsf(xv[i].w))));
                        if (nvec > XV * SW) mx = fmaxf(mx, absmax4(xr, XV * SW + tq, SW));
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                        if (lane == 0) part_f[wq] = mx;
                        stage_sync();
                        float scale = 0.0f;
#pragma unroll
                        for (int w = 0; w < SWARPS; ++w) scale = fmaxf(scale, part_f[w]);
                        const float inv = __fdiv_rn(127.0f, scale);
                        const bool zero_row = (scale == 0.0f);
                        int sum = 0;
#pragma unroll
                        for (int i = 0; i < XV; ++i) {
                            const int v = i * SW + tq;
                            const bool in = v < nvec;
                            const unsigned mask = __ballot_sync(0xffffffffu, in);     // whole quads: K % 64 == 0
                            if (in) sum += quant_f4(xv[i], m, v, inv, zero_row, mask);
                        }
                        for (int vb = XV * SW; vb < nvec; vb += SW) {
                            const int v = vb + tq;
                            const bool in = v < nvec;
                            const unsigned mask = __ballot_sync(0xffffffffu, in);
                            if (in) sum += quant_f4(Vec4<XT>::load(xr, v), m, v, inv, zero_row, mask);
                        }
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                        if (lane == 0) part_i[wq] = sum;
                        stage_sync();
                        if (tq == 0) {
                            int tot = 0;
                            for (int w = 0; w < SWARPS; ++w) tot += part_i[w];
                            rowsum_s[m] = tot;
                            scale_s[m] = scale;
                        }
                    }
                } else {
                    for (int m = wq; m < p.M; m += SWARPS) {         // a warp per row, no exchange between warps
                        const XT *xr = x + (int64_t)m * p.K;
                        const float scale = absmax4(xr, lane, 32);
                        const float inv = __fdiv_rn(127.0f, scale);
                        const bool zero_row = (scale == 0.0f);
                        int sum = 0;
                        for (int vb = 0; vb < nvec; vb += 32) {
                            const int v = vb + lane;
                            const bool in = v < nvec;
                            const unsigned mask = __ballot_sync(0xffffffffu, in);     // whole quads: K % 64 == 0
                            if (in) sum += quant_vec(xr, m, v, inv, zero_row, mask);
                        }
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                        if (lane == 0) { rowsum_s[m] = sum; scale_s[m] = scale; }
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the tensor core reads the tokens
            stage_sync();
        }

        if (warp == 1) {
            // ---------------- MMA issuer (whole warp in the loop, one elected lane issues)
            const bool leader = elect_one();
            uint32_t a = 0, aph = 0, it = 0;
            get_tmem();
            bool ok = tmem_ok;
            for (int j = 0; j < my_tiles && ok; ++j) {
                const uint32_t buf = (uint32_t)j & 1u, cph = ((uint32_t)j >> 1) & 1u;
                if (!(ok = mbar_wait_warp(acce_bar(buf), cph ^ 1u, 0x611))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * ACC_COLS;
                for (int st = 0; st < p.nsteps; ++st, ++it) {
                    if (!(ok = mbar_wait_warp(afull_bar(a), aph, 0x612))) break;
                    tc_fence_after();
                    if (leader) {
                        const uint32_t a_tmem = tmem_base + 2 * ACC_COLS + a * A_COLS;
#pragma unroll
                        for (int ks = 0; ks < KS; ++ks) {
                            const int kb = st * KS + ks;
                            if (kb < p.nkb) {
                                const uint64_t bdesc = smem_desc(base + kb * XB_BYTES);
#pragma unroll
                                for (int i = 0; i < 4; ++i)      // class i: its own accumulator, 32 positions = 8 columns
                                    umma_i8_ts(d_tmem + NTOK * i, a_tmem + 32u * ks + 8u * i, bdesc + 2u * i, IDESC, kb != 0);
                            }
                        }
                        umma_commit(done_bar(it));
                    }
                    if (++a == AS) { a = 0; aph ^= 1u; }
                }
                if (ok && leader) umma_commit(accf_bar(buf));
            }
        } else if (warp >= 8) {
            // ---------------- unpack warps
            const int qd = warp & 3;                     // TMEM lane quadrant
            const int group = (warp - 8) >> 2;
            const int row = qd * 32 + lane;
            const int total = my_tiles * p.nsteps;
            int s = group % p.ts;
            uint32_t a = group % AS, sph = 0;
            get_tmem();
            bool ok = tmem_ok;
            for (int it = group; it < total && ok; it += 2) {
                if (!(ok = mbar_wait_warp(raw_bar(s), sph, 0x621))) break;
                const uint8_t *pr = base_ptr + p.off_ring + (size_t)s * P_BYTES + row * PK_ROW;
                uint4 pv[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) pv[c] = *reinterpret_cast<const uint4 *>(pr + ((c ^ (row & 7)) << 4));
                if (it >= AS && !(ok = mbar_wait_warp(done_bar(it - AS), done_par(it - AS), 0x622))) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    const uint32_t wv[8] = {pv[2 * ks].x, pv[2 * ks].y, pv[2 * ks].z, pv[2 * ks].w,
                                            pv[2 * ks + 1].x, pv[2 * ks + 1].y, pv[2 * ks + 1].z, pv[2 * ks + 1].w};
                    uint32_t r[32];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
#pragma unroll
                        for (int g = 0; g < 8; ++g) r[8 * i + g] = wv[g] & (0x03030303u << (6 - 2 * i));
                    tmem_st32_issue(tmem_base + ((uint32_t)(qd * 32) << 16) + 2 * ACC_COLS + a * A_COLS + 32u * ks, r);
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(afull_bar(a));
                    mbar_arrive(pfree_bar(s));
                }
                if ((s += 2) >= p.ts) { s -= p.ts; sph ^= 1u; }
                a = (a + 2) % AS;
            }
        } else if (warp >= 4) {
            // ---------------- epilogue warps
            const int qd = warp & 3;
            get_tmem();
            bool ok = tmem_ok;
            for (int j = 0; j < my_tiles && ok; ++j) {
                const uint32_t buf = (uint32_t)j & 1u, cph = ((uint32_t)j >> 1) & 1u;
                const int64_t n = ((int64_t)blockIdx.x + (int64_t)j * gridDim.x) * BW + qd * 32 + lane;
                if (!(ok = mbar_wait_warp(accf_bar(buf), cph, 0x631))) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(qd * 32) << 16) + buf * ACC_COLS;
                uint32_t c01[32], c23[32];
                tmem_ld32(taddr, c01);
                tmem_ld32(taddr + 32, c23);
                tc_fence_before();
                mbar_arrive(acce_bar(buf));
                if (n < p.N) {
                    const float bias = p.bias ? p.bias[n] : 0.0f;
#pragma unroll
                    for (int tok = 0; tok < NTOK; ++tok) {
                        if (tok < p.M) {                                  // warp-uniform
                            const int accv = ((int)c01[tok] >> 6) + ((int)c01[16 + tok] >> 4) + ((int)c23[tok] >> 2) +
                                             (int)c23[16 + tok] - rowsum_s[tok];
                            const int64_t o = (int64_t)tok * p.N + n;
                            if (p.acc_out) p.acc_out[o] = accv;
                            float v = bitlinear_finalize(accv, scale_s[tok], p.weight_scale);
                            if (p.bias) v = __fadd_rn(v, bias);
                            if (p.residual) v = __fadd_rn(v, p.residual[o]);
                            store_out(p.y, p.y_dtype, o, v);
                        }
                    }
                }
            }
        }
    }
    // ---------------- teardown: every thread arrives here, on success and after an expired wait
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {                                                 // the allocating warp frees
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(*slot_ptr) : "memory");
    }
}

}  // namespace dec

// ---------------------------------------------------------------- host side
static int dec_smem_budget()
{
    static int v = 0;
    if (!v) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    }
    return v;
}

static bool dec_plan(dec::Params &p, int *smem_bytes, int *grid)
{
    using namespace dec;
    p.nkb = (int)((p.K + 127) / 128);
    p.nsteps = (int)((p.K + 128 * KS - 1) / (128 * KS));
    p.ntiles = (int)((p.N + BW - 1) / BW);
    const int xs = p.nkb * XB_BYTES;
    const int misc = 256, bar_bytes = 512;
    const int room = dec_smem_budget() - 1024 - xs - misc - bar_bytes;
    p.ts = room / P_BYTES;
    if (p.ts > MAX_TS) p.ts = MAX_TS;
    if (p.ts < 3) return false;
    p.off_ring = xs;
    p.off_misc = xs + p.ts * P_BYTES;
    p.off_bar = p.off_misc + misc;
    *smem_bytes = 1024 + p.off_bar + bar_bytes;
    *grid = p.ntiles < sm100::sm_count() ? p.ntiles : sm100::sm_count();
    return true;
}

template <typename XT>
static int launch_decode(dec::Params &p, cudaStream_t st)
{
    int smem = 0, grid = 0;
    if (!dec_plan(p, &smem, &grid))
        return fail(NSLQ_ERR_UNSUPPORTED, "ternary_decode_kernel: K=%lld does not fit shared memory", (long long)p.K);
    static std::atomic<size_t> reserved[kMaxDevices];
    if (reserve_smem(dec::ternary_decode_kernel<XT>, reserved, (size_t)smem) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "ternary_decode_kernel: cannot reserve %d bytes of shared memory: %s", smem,
                    cudaGetErrorString(cudaGetLastError()));
    CUtensorMap tmap_w;
    int rc = sm100::make_map_2d(&tmap_w, p.w, (uint64_t)(p.K / 4), (uint64_t)p.N, dec::PK_ROW, dec::BW, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    cudaError_t e = launch_kernel(dec::ternary_decode_kernel<XT>, dim3(grid), dim3(dec::THREADS), (size_t)smem, st, tmap_w, p);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "ternary_decode_kernel: %s", cudaGetErrorString(e));
    return check_launch("ternary_decode_kernel");
}

static bool dec_shape_ok(const void *w, int64_t M, int64_t N, int64_t K)
{
    if (!(M >= 1 && M <= dec::NTOK && (K % 64 == 0) && aligned16(w) && N < (1ll << 31) && K < (1ll << 24))) return false;
    dec::Params p{};
    p.N = N; p.K = K; p.M = (int)M;
    int smem = 0, grid = 0;
    return dec_plan(p, &smem, &grid);
}

// Already-quantised activations (consumption order), M <= 16.
bool ternary_decode_supported(const void *w, const void *q_perm, int64_t M, int64_t N, int64_t K)
{
    return aligned16(q_perm) && dec_shape_ok(w, M, N, K);
}

int ternary_decode_dispatch(const uint8_t *w, const int8_t *q_perm, const float *scale, const int32_t *rowsum, int M,
                            int64_t N, int64_t K, float weight_scale, void *y, int y_dtype, int32_t *acc_out,
                            const float *bias, const float *residual, cudaStream_t st)
{
    dec::Params p{};
    p.w = w; p.q = q_perm; p.scale = scale; p.rowsum = rowsum; p.y = y; p.acc_out = acc_out; p.bias = bias;
    p.residual = residual; p.N = N; p.K = K; p.M = M; p.y_dtype = y_dtype; p.weight_scale = weight_scale;
    return launch_decode<void>(p, st);
}

// Activations in their own dtype, quantised inside the kernel; M <= 2.
bool ternary_decode_fused_supported(const void *w, const void *x, int x_dtype, int64_t M, int64_t N, int64_t K)
{
    if (M > dec::FUSED_MAX_M || !aligned16(x)) return false;
    if (x_dtype != NSLQ_DTYPE_F32 && x_dtype != NSLQ_DTYPE_FP16 && x_dtype != NSLQ_DTYPE_BF16) return false;
    return dec_shape_ok(w, M, N, K);
}

int ternary_decode_fused_dispatch(const uint8_t *w, const void *x, int x_dtype, int M, int64_t N, int64_t K,
                                  float weight_scale, void *y, int y_dtype, int32_t *acc_out, const float *bias,
                                  const float *residual, cudaStream_t st)
{
    dec::Params p{};
    p.w = w; p.x = x; p.y = y; p.acc_out = acc_out; p.bias = bias; p.residual = residual;
    p.N = N; p.K = K; p.M = M; p.y_dtype = y_dtype; p.weight_scale = weight_scale;
    switch (x_dtype) {
    case NSLQ_DTYPE_F32: return launch_decode<float>(p, st);
    case NSLQ_DTYPE_FP16: return launch_decode<__half>(p, st);
    case NSLQ_DTYPE_BF16: return launch_decode<__nv_bfloat16>(p, st);
    default: return fail(NSLQ_ERR_ARG, "BitLinear: x_dtype %d not in {F32,FP16,BF16}", x_dtype);
    }
}

// The status word of this translation unit's kernels (see sm100::read_wait_status).
int ternary_decode_status(int *out) { return sm100::read_wait_status(out); }

}  // namespace nslq
