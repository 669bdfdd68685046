// Stage 3 for W4A16: prefill GEMM (M > 16 tokens) on the 5th-generation tensor cores (sm_100a),
// exact in the weights.
//
//   y[m,n] = sum_g scale[n,g] * ( sum_{k in g} q[n,k] * x[m,k]  -  zp[n,g] * sum_{k in g} x[m,k] )
//
// Same formulation as the decode kernel (w4a16_decode_sm100.cu), on the skeleton of the ternary
// GEMM (ternary_gemm_sm100.cu): the product is computed transposed, D[n, m], with the weights as
// the M-side operand in TENSOR memory.  The 4-bit codes go to the tensor core undequantised, as
// the 16-bit floats MAGIC + q (bf16 128 + q, fp16 1024 + q: exact), every block of 128 k gets a
// fresh fp32 accumulator, and the epilogue warps apply
//       y += scale[n,g] * (acc - (MAGIC + zp[n,g]) * xsum[m, block])
// in fp32 while the next blocks are being multiplied.  Nothing is rounded before the
// accumulation (an earlier form wrote bf16((q - zp) * scale) into shared memory and lost 1e-2 of
// the row rms there), zero points may be fractional (AWQ's float zeros), and the expanded
// weights never cross shared memory.
//
// Persistent, warp-specialised, one CTA per SM, tiles of 128 weight rows x 128 tokens, one
// pipeline step = one block of 128 k:
//   warp 0       TMA producer: per step the activation tile (two sub-tiles of 128 tokens x 64 k,
//                SWIZZLE_128B) and the packed weight tile (128 rows x 64 bytes, SWIZZLE_64B, so
//                that a thread per row reads its 64 bytes conflict-free), this CTA only.
//   warps 2-9    unpack, two groups of four warps on alternate steps.  A thread owns a weight row
//                (a TMEM lane): 16 words of 8 nibbles -> 64 registers of two 16-bit floats in k
//                order -> tcgen05.st.  The same thread owns a token of the tile and adds up its
//                128 activations of the block in fp32 (xsum) into a small shared-memory ring.
//   warp 1       MMA issuer (converged warp, elected lane): eight tcgen05.mma.kind::f16 (M=128,
//                N=128, K=16) per step into the step's accumulator buffer, one commit per step.
//   warps 10-17  epilogue, two warps per TMEM lane quadrant, each taking 64 of the tile's tokens:
//                per step tcgen05.ld of the accumulator, two FMAs per value into fp32 partial
//                outputs held in registers, stored once per tile.
//
// Every mbarrier wait is bounded; a wait that gives up raises a CTA-wide flag, every role
// leaves, outstanding copies and MMAs are waited for (bounded), and the common teardown frees
// the tensor memory.
#include <type_traits>

#include "sm100_common.cuh"

namespace nslq {
namespace w4gemm {

using namespace sm100;

constexpr int BW = 128;                  // weight rows per tile = MMA M = TMEM lanes
constexpr int BKK = 128;                 // k per pipeline step (one accumulator block)
constexpr int THREADS = 576;             // 18 warps: 0 TMA, 1 MMA, 2-9 unpack, 10-17 epilogue
constexpr int P_ROW = BKK / 2;           // packed bytes per weight row and step
constexpr int P_BYTES = BW * P_ROW;      // 8 KiB
constexpr int A_COLS = BKK / 2;          // TMEM columns of one operand stage (two 16-bit values per column)
constexpr int AS = 4;                    // operand stages: columns 256..511
constexpr int NB = 2;                    // accumulator buffers, at columns 0 and 128
constexpr int ND = 8;                    // ring of "step retired" barriers
constexpr int XR = 8;                    // ring of per-step token sums: the unpack warps run at most AS + NB steps ahead of the epilogue
constexpr int EG = 16;                   // tokens per tcgen05.ld of the epilogue
constexpr int BAR_BYTES = 512;
static_assert(AS < ND && XR >= AS + NB + 1, "ring depths");

// BT = tokens per tile = MMA N: 128, or 96 / 64 where that wastes fewer SM-rounds on the shape.
template <int BT> struct Cfg {
    static_assert(BT == 64 || BT == 96 || BT == 128, "token tile");
    static constexpr int X_SUB = BT * 128;            // one 128-byte-swizzled sub-tile: BT tokens x 64 k of 16-bit values
    static constexpr int X_BYTES = 2 * X_SUB;
    static constexpr int T_BYTES = X_BYTES + P_BYTES; // one copy stage, a multiple of 1024
    static constexpr int TS = (BT == 128) ? 5 : (BT == 96 ? 6 : 7);   // copy stages
    static constexpr int HALF_T = BT / 2;             // tokens per epilogue warp
    static constexpr int XSUM_BYTES = XR * BT * 4;
    static constexpr int SMEM = TS * T_BYTES + XSUM_BYTES + BAR_BYTES + 1024;
    static_assert(SMEM <= 232448, "over the 227 KiB a CTA may use");
    static_assert(TS < ND && T_BYTES % 1024 == 0 && HALF_T % EG == 0, "stage geometry");
};

struct Params {
    const float *scale_t;    // [G][N] (transposed table: a lane per row reads coalesced)
    const float *zc_t;       // [G][N] zero point in code units (may be fractional)
    void *y;                 // [M][N]
    int64_t M, N, K;
    int G, gs, y_dtype;
    int tiles_t, tiles_w, nkb;   // token tiles, weight-row tiles, blocks of 128 k
};

template <bool BF16, int BT> static __device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t accumulate)
{
    constexpr uint32_t fmt = BF16 ? 1u : 0u;
    constexpr uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BT >> 3) << 17) | ((uint32_t)(BW >> 4) << 24);
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// Eight nibbles of a word (k = 0..7 at bits 0, 4, ..., 28) -> four registers of two 16-bit floats
// MAGIC + q in k order (low half = even k).  x holds the even nibbles as bytes, y the odd ones; two
// byte permutes interleave them, one more per pair puts the exponent byte above each code.
template <uint32_t MAGIC_HI> static __device__ __forceinline__ void expand8(uint32_t w, uint32_t *r)
{
    const uint32_t x = w & 0x0F0F0F0Fu, y = (w >> 4) & 0x0F0F0F0Fu;
    const uint32_t p01 = __byte_perm(x, y, 0x5140);       // (x0, y0, x1, y1): k = 0, 1, 2, 3
    const uint32_t p23 = __byte_perm(x, y, 0x7362);       // (x2, y2, x3, y3): k = 4, 5, 6, 7
    r[0] = __byte_perm(p01, MAGIC_HI, 0x4140);            // (k0, hi, k1, hi)
    r[1] = __byte_perm(p01, MAGIC_HI, 0x4342);
    r[2] = __byte_perm(p23, MAGIC_HI, 0x4140);
    r[3] = __byte_perm(p23, MAGIC_HI, 0x4342);
}

template <typename T> struct OutStore;
template <> struct OutStore<float> {
    static __device__ __forceinline__ void put(void *y, int64_t o, float v) { reinterpret_cast<float *>(y)[o] = v; }
};
template <> struct OutStore<__nv_bfloat16> {
    static __device__ __forceinline__ void put(void *y, int64_t o, float v) { reinterpret_cast<__nv_bfloat16 *>(y)[o] = __float2bfloat16_rn(v); }
};
template <> struct OutStore<__half> {
    static __device__ __forceinline__ void put(void *y, int64_t o, float v) { reinterpret_cast<__half *>(y)[o] = __float2half_rn(v); }
};

// ---------------------------------------------------------------- kernel
// ZPI: the zero points are whole numbers (QuantizedTensor form).  The unpack warps then subtract
// (MAGIC + zp) from (MAGIC + q) with one packed 16-bit subtraction -- exact, both are integers below
// 2^8 (bf16) or 2^11 (fp16) -- so the tensor core multiplies q - zp itself: no token sums, one FMA per
// value in the epilogue.  Fractional zero points (AWQ's float zeros) keep the form with the sums.
template <typename XT, bool ZPI, int BT>
__global__ void __launch_bounds__(THREADS, 1)
w4a16_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, const Params p)
{
    using C = Cfg<BT>;
    constexpr int X_SUB = C::X_SUB, X_BYTES = C::X_BYTES, T_BYTES = C::T_BYTES, TS = C::TS, HALF_T = C::HALF_T, XSUM_BYTES = C::XSUM_BYTES;
    constexpr bool BF16 = std::is_same<XT, __nv_bfloat16>::value;
    constexpr uint32_t MAGIC_HI = BF16 ? 0x43434343u : 0x64646464u;
    constexpr float MAGIC = BF16 ? 128.0f : 1024.0f;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                  // 1024-byte aligned (swizzle atom)
    uint8_t *base_ptr = smem_raw + (base - raw);
    float *xsum = reinterpret_cast<float *>(base_ptr + TS * T_BYTES);              // [XR][BT]
    const uint32_t bars = base + TS * T_BYTES + XSUM_BYTES;
    // barrier map (8 bytes each): raw[t] (copy stage landed), pfree[t] (stage read by the four unpack warps),
    // afull[a] (codes stored in TMEM, token sums written), done[8] (MMAs of step i retired: one commit per
    // step frees the copy stage i mod TS and the operand stage i mod AS and hands the accumulator to the
    // epilogue), acce[2] (accumulator read out), drain (used only when a wait gave up); then the TMEM slot
    // and the CTA-wide abort flag.
    constexpr int NBAR = 2 * TS + AS + ND + NB + 1;
    static_assert(NBAR * 8 + 16 <= BAR_BYTES, "barrier area");
    auto raw_bar = [&](int t) { return bars + 8u * t; };
    auto pfree_bar = [&](int t) { return bars + 8u * (TS + t); };
    auto afull_bar = [&](int a) { return bars + 8u * (2 * TS + a); };
    auto done_bar = [&](uint32_t i) { return bars + 8u * (2 * TS + AS + (i & (ND - 1))); };
    auto done_par = [&](uint32_t i) { return (i / ND) & 1u; };
    auto acce_bar = [&](int b) { return bars + 8u * (2 * TS + AS + ND + b); };
    const uint32_t drain_bar = bars + 8u * (2 * TS + AS + ND + NB);
    const uint32_t slot = bars + 8u * NBAR;
    volatile uint32_t *slot_ptr = reinterpret_cast<volatile uint32_t *>(base_ptr + TS * T_BYTES + XSUM_BYTES + 8 * NBAR);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(base_ptr + TS * T_BYTES + XSUM_BYTES + 8 * NBAR + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ntiles = p.tiles_t * p.tiles_w;
    const int my_tiles = (int)blockIdx.x < ntiles ? (ntiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int t = 0; t < TS; ++t) { mbar_init(raw_bar(t), 1); mbar_init(pfree_bar(t), 4); }
        for (int a = 0; a < AS; ++a) mbar_init(afull_bar(a), 4);
        for (int i = 0; i < ND; ++i) mbar_init(done_bar(i), 1);
        for (int b = 0; b < NB; ++b) mbar_init(acce_bar(b), 256);
        mbar_init(drain_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(slot) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *slot_ptr;

    pdl_wait();                 // the activations come from the preceding kernel
    pdl_launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0, it = 0;
            bool ok = true;
            for (int j = 0; j < my_tiles && ok; ++j) {
                const int tile = (int)blockIdx.x + j * (int)gridDim.x;
                const int m0 = (tile % p.tiles_t) * BT, n0 = (tile / p.tiles_t) * BW;
                for (int kb = 0; kb < p.nkb; ++kb, ++it) {
                    if (it >= (uint32_t)TS) {          // the stage's previous user: step it - TS
                        if (!(ok = mbar_wait(done_bar(it - TS), done_par(it - TS), 0x1101, abort_flag))) break;
                        if (!(ok = mbar_wait(pfree_bar(s), ph ^ 1u, 0x1102, abort_flag))) break;
                    }
                    const uint32_t st = base + s * T_BYTES;
                    mbar_arrive_expect_tx(raw_bar(s), T_BYTES);
                    tma_load_2d(st, &tmap_x, kb * 256, m0, raw_bar(s));                  // inner coordinate in bytes: 128 k x 2
                    tma_load_2d(st + X_SUB, &tmap_x, kb * 256 + 128, m0, raw_bar(s));
                    tma_load_2d(st + X_BYTES, &tmap_w, kb * P_ROW, n0, raw_bar(s));
                    if (++s == TS) { s = 0; ph ^= 1u; }
                }
            }
            if (*abort_flag) {
                // copies this thread issued may still be on their way into shared memory: the CTA must not end under them
                const uint32_t first = it > (uint32_t)TS ? it - TS : 0u;
                for (uint32_t j = first; j < it; ++j) mbar_wait(raw_bar((int)(j % TS)), (j / TS) & 1u, 0x1103);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the whole warp runs the loop, one elected lane issues
        const bool leader = elect_one();
        uint32_t a = 0, aph = 0, it = 0;
        int s = 0;
        bool ok = true;
        for (int j = 0; j < my_tiles && ok; ++j) {
            for (int kb = 0; kb < p.nkb; ++kb, ++it) {
                const uint32_t sb = it % NB;
                if (!(ok = mbar_wait_warp(acce_bar(sb), ((it / NB) & 1u) ^ 1u, 0x1201, abort_flag))) break;   // accumulator of step it - NB read out
                if (!(ok = mbar_wait_warp(afull_bar(a), aph, 0x1202, abort_flag))) break;                    // codes stored (and the copy stage landed)
                tc_fence_after();
                if (leader) {
                    const uint32_t a_tmem = tmem_base + 256 + a * A_COLS;
                    const uint32_t d_tmem = tmem_base + sb * 128;
#pragma unroll
                    for (int k16 = 0; k16 < 8; ++k16) {        // 16 k = 32 bytes of a token row = 8 TMEM columns per MMA
                        const uint64_t bdesc = smem_desc(base + s * T_BYTES + (k16 >> 2) * X_SUB) + 2u * (k16 & 3);
                        umma_f16_ts<BF16, BT>(d_tmem, a_tmem + 8u * k16, bdesc, k16 != 0);
                    }
                    umma_commit(done_bar(it));
                }
                if (++s == TS) s = 0;
                if (++a == AS) { a = 0; aph ^= 1u; }
            }
        }
        if (__any_sync(0xffffffffu, *abort_flag != 0)) {
            // leaving early: every MMA issued so far must have retired before the tensor memory is freed
            if (leader) umma_commit(drain_bar);
            __syncwarp();
            mbar_wait_warp(drain_bar, 0, 0x1203);
        }
    } else if (warp < 10) {
        // ---------------- unpack warps: codes of this thread's weight row into its TMEM lane, and the sum of
        // this thread's token over the block
        const int q = warp & 3;                      // TMEM lane quadrant of this warp
        const int group = (warp - 2) >> 2;           // group 0 takes even steps, group 1 odd
        const int row = q * 32 + lane;               // weight row of the tile = token of the tile
        const int total = my_tiles * p.nkb;
        const int bpg = p.gs / BKK;
        int s = group % TS;
        uint32_t a = group % AS, sph = 0;
        bool ok = true;
        uint32_t zsub = 0;                           // two copies of MAGIC + zp of this row and group, as 16-bit floats
        float z_next = 0.0f;
        auto fetch_z = [&](int step) {               // MAGIC + zero point of this thread's row in the group of pipeline step `step`
            const int jt = step / p.nkb, kb = step - jt * p.nkb;
            const int tile = (int)blockIdx.x + jt * (int)gridDim.x;
            int64_t nrow = (int64_t)(tile / p.tiles_t) * BW + row;
            if (nrow >= p.N) nrow = p.N - 1;         // rows past N: any constants, their results are not stored
            return MAGIC + __ldg(p.zc_t + (int64_t)(kb / bpg) * p.N + nrow);
        };
        for (int it = group; it < total && ok; it += 2) {
            if (ZPI) {
                // this step's constant was fetched during the previous step of this group; fetch the next one now
                if (it == group) z_next = fetch_z(it);
                const float z = z_next;
                if (it + 2 < total) z_next = fetch_z(it + 2);
                uint32_t h;
                if constexpr (BF16) h = __bfloat16_as_ushort(__float2bfloat16_rn(z)); else h = __half_as_ushort(__float2half_rn(z));
                zsub = h | (h << 16);
            }
            if (!(ok = mbar_wait_warp(raw_bar(s), sph, 0x1301, abort_flag))) break;
            const uint8_t *stage = base_ptr + s * T_BYTES;
            // packed row: 64 bytes, SWIZZLE_64B (16-byte chunk c of row r sits at chunk c ^ ((r >> 1) & 3))
            const uint8_t *pr = stage + X_BYTES + row * P_ROW;
            uint4 pv[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) pv[c] = *reinterpret_cast<const uint4 *>(pr + ((c ^ ((row >> 1) & 3)) << 4));
            // token sum: the 2 x 128 bytes of this token in the two sub-tiles; every 16-byte chunk is read once, in an
            // order rotated by the lane so that a quarter-warp touches eight different bank groups (swizzle
            // positions do not matter for a sum over the whole row)
            float sum = 0.0f;
#pragma unroll
            for (int sub = 0; sub < ((ZPI || row >= BT) ? 0 : 2); ++sub) {
                const uint8_t *xr = stage + sub * X_SUB + row * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(xr + (((c + lane) & 7) << 4));
                    const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if constexpr (BF16) {
                            sum += __uint_as_float(ww[i] << 16) + __uint_as_float(ww[i] & 0xffff0000u);
                        } else {
                            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&ww[i]));
                            sum += f.x + f.y;
                        }
                    }
                }
            }
            if (it >= AS && !(ok = mbar_wait_warp(done_bar(it - AS), done_par(it - AS), 0x1302, abort_flag))) break;   // operand stage reusable
            tc_fence_after();
            if (!ZPI && row < BT) xsum[(it & (XR - 1)) * BT + row] = sum;
#pragma unroll
            for (int h = 0; h < 2; ++h) {            // 32 packed bytes = 64 k = 32 columns
                const uint32_t wv[8] = {pv[2 * h].x, pv[2 * h].y, pv[2 * h].z, pv[2 * h].w,
                                        pv[2 * h + 1].x, pv[2 * h + 1].y, pv[2 * h + 1].z, pv[2 * h + 1].w};
                uint32_t r[32];
#pragma unroll
                for (int jw = 0; jw < 8; ++jw) expand8<MAGIC_HI>(wv[jw], r + 4 * jw);
                if (ZPI) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        if constexpr (BF16) {
                            const __nv_bfloat162 d = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&r[c]), *reinterpret_cast<const __nv_bfloat162 *>(&zsub));
                            r[c] = *reinterpret_cast<const uint32_t *>(&d);
                        } else {
                            const __half2 d = __hsub2(*reinterpret_cast<const __half2 *>(&r[c]), *reinterpret_cast<const __half2 *>(&zsub));
                            r[c] = *reinterpret_cast<const uint32_t *>(&d);
                        }
                    }
                }
                tmem_st32_issue(tmem_base + ((uint32_t)(q * 32) << 16) + 256 + a * A_COLS + 32u * h, r);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(afull_bar(a));
                mbar_arrive(pfree_bar(s));
            }
            if ((s += 2) >= TS) { s -= TS; sph ^= 1u; }
            a = (a + 2) % AS;
        }
    } else {
        // ---------------- epilogue warps (TMEM -> registers, per-block scale and zero point, -> global at the end of a tile)
        const int q = warp & 3;                       // TMEM lane quadrant of this warp
        const int half = (warp - 10) >> 2;            // which 64 of the tile's tokens
        const int bpg = p.gs / BKK;                   // blocks of 128 k per quantisation group
        uint32_t it = 0;
        bool ok = true;
        for (int j = 0; j < my_tiles && ok; ++j) {
            const int tile = (int)blockIdx.x + j * (int)gridDim.x;
            const int64_t m0 = (int64_t)(tile % p.tiles_t) * BT + half * HALF_T, n0 = (int64_t)(tile / p.tiles_t) * BW;
            const int64_t n = n0 + q * 32 + lane;
            const bool n_ok = n < p.N;
            const int64_t nc = n_ok ? n : p.N - 1;    // rows past N read the last row's constants; their results are not stored
            float yacc[HALF_T];
#pragma unroll
            for (int t = 0; t < HALF_T; ++t) yacc[t] = 0.0f;
            // The group constants of a step are fetched one step ahead (a read from L2 costs about as much as a
            // whole step here, and nothing else in this warp could cover it).
            auto load_consts = [&](int kb, float &s_out, float &c_out) {
                const int g = (kb < p.nkb ? kb : p.nkb - 1) / bpg;
                s_out = __ldg(p.scale_t + (int64_t)g * p.N + nc);
                c_out = ZPI ? 0.0f : -(MAGIC + __ldg(p.zc_t + (int64_t)g * p.N + nc));
            };
            float sc, cm, sc_next, cm_next;
            load_consts(0, sc_next, cm_next);
            for (int kb = 0; kb < p.nkb && ok; ++kb, ++it) {
                const uint32_t sb = it % NB;
                sc = sc_next; cm = cm_next;
                load_consts(kb + 1, sc_next, cm_next);
                if (!(ok = mbar_wait_warp(done_bar(it), done_par(it), 0x1401, abort_flag))) break;
                tc_fence_after();
                const float4 *xs4 = reinterpret_cast<const float4 *>(xsum + (it & (XR - 1)) * BT + half * HALF_T);
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + sb * 128 + half * HALF_T;
#pragma unroll
                for (int gi = 0; gi < HALF_T / EG; ++gi) {
                    uint32_t r[EG];
                    tmem_ld16(taddr + gi * EG, r);
                    float xs[EG];
                    if (!ZPI) {
#pragma unroll
                        for (int e4 = 0; e4 < EG / 4; ++e4) {
                            const float4 v = xs4[gi * (EG / 4) + e4];
                            xs[4 * e4] = v.x; xs[4 * e4 + 1] = v.y; xs[4 * e4 + 2] = v.z; xs[4 * e4 + 3] = v.w;
                        }
                    }
                    if (gi == HALF_T / EG - 1) {      // last read of this step's accumulator and token sums: hand them back
                        tc_fence_before();
                        mbar_arrive(acce_bar(sb));
                    }
#pragma unroll
                    for (int e = 0; e < EG; ++e) {
                        if (ZPI) yacc[gi * EG + e] = fmaf(sc, __uint_as_float(r[e]), yacc[gi * EG + e]);
                        else yacc[gi * EG + e] = fmaf(sc, fmaf(cm, xs[e], __uint_as_float(r[e])), yacc[gi * EG + e]);
                    }
                }
            }
            if (ok && n_ok) {
#pragma unroll
                for (int t = 0; t < HALF_T; ++t) {
                    const int64_t m = m0 + t;
                    if (m < p.M) {                    // warp-uniform
                        const int64_t o = m * p.N + n;
                        if (p.y_dtype == NSLQ_DTYPE_F32) OutStore<float>::put(p.y, o, yacc[t]);
                        else if (p.y_dtype == NSLQ_DTYPE_BF16) OutStore<__nv_bfloat16>::put(p.y, o, yacc[t]);
                        else OutStore<__half>::put(p.y, o, yacc[t]);
                    }
                }
            }
            __syncwarp();                             // the next tile starts with a warp-wide tcgen05.ld
        }
    }
    // ---------------- teardown: every thread arrives here, on success and after a wait that gave up
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

}  // namespace w4gemm

// ---------------------------------------------------------------- host side
// 16-bit activations, whole blocks of 128 k (K % 128 == 0, groups a multiple of 128), 16-byte aligned
// pointers.  Zero points may be fractional, so both the QuantizedTensor and the AWQ form qualify.
bool w4a16_gemm_supported(const void *codes, const void *x, int x_dtype, int64_t M, int64_t N, int64_t K, int64_t gs)
{
    return (x_dtype == NSLQ_DTYPE_BF16 || x_dtype == NSLQ_DTYPE_FP16) && (K % 128 == 0) && gs > 0 && (gs % 128 == 0) &&
           aligned16(codes) && aligned16(x) && M > 0 && M < (1ll << 31) && N > 0 && N < (1ll << 31) && K < (1ll << 30);
}

template <typename XT, bool ZPI, int BT>
static int launch_w4_gemm(const uint8_t *codes, const void *x, w4gemm::Params &p, cudaStream_t st)
{
    using namespace w4gemm;
    using C = Cfg<BT>;
    static std::atomic<size_t> reserved[kMaxDevices];
    if (reserve_smem(w4a16_gemm_kernel<XT, ZPI, BT>, reserved, (size_t)C::SMEM) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "w4a16_gemm_kernel: cannot reserve %d bytes of shared memory: %s", C::SMEM,
                    cudaGetErrorString(cudaGetLastError()));
    CUtensorMap tmap_x, tmap_w;
    int rc = sm100::make_map_2d(&tmap_x, x, (uint64_t)p.K * 2, (uint64_t)p.M, 128, BT, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = sm100::make_map_2d(&tmap_w, codes, (uint64_t)(p.K / 2), (uint64_t)p.N, P_ROW, BW, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
    p.tiles_t = (int)((p.M + BT - 1) / BT);
    p.tiles_w = (int)((p.N + BW - 1) / BW);
    p.nkb = (int)(p.K / BKK);
    const int tiles = p.tiles_t * p.tiles_w;
    const int grid = tiles < sm100::sm_count() ? tiles : sm100::sm_count();
    cudaError_t e = launch_kernel(w4a16_gemm_kernel<XT, ZPI, BT>, dim3(grid), dim3(THREADS), (size_t)C::SMEM, st, tmap_x, tmap_w, p);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "w4a16_gemm_kernel: %s", cudaGetErrorString(e));
    return check_launch("w4a16_gemm_kernel");
}

// Token-tile width: the one that wastes fewer SM-rounds on the shape (ties go to the wider tile, which
// re-reads the packed weights less often).
template <typename XT, bool ZPI>
static int pick_w4_gemm(const uint8_t *codes, const void *x, w4gemm::Params &p, cudaStream_t st)
{
    const int sms = sm100::sm_count();
    auto cost = [&](int bt) {
        const int64_t tiles = ((p.M + bt - 1) / bt) * ((p.N + w4gemm::BW - 1) / w4gemm::BW);
        return (double)((tiles + sms - 1) / sms) * bt;
    };
    const double c128 = cost(128), c96 = cost(96), c64 = cost(64);
    if (c128 <= c96 && c128 <= c64) return launch_w4_gemm<XT, ZPI, 128>(codes, x, p, st);
    if (c96 <= c64) return launch_w4_gemm<XT, ZPI, 96>(codes, x, p, st);
    return launch_w4_gemm<XT, ZPI, 64>(codes, x, p, st);
}

// One launch takes at most this many token rows (the same precaution as the ternary GEMM takes:
// launches stay in the hundred-microsecond range).
constexpr int64_t W4_GEMM_MAX_ROWS = 4096;

// scale_t, zc_t: the handle's transposed [G][N] tables.
int w4a16_gemm_dispatch(const uint8_t *codes, const float *scale_t, const float *zc_t, int zp_integer, int64_t N, int64_t K, int G,
                        int gs, const void *x, int x_dtype, int64_t M, void *y, int y_dtype, cudaStream_t st)
{
    const int es = y_dtype == NSLQ_DTYPE_F32 ? 4 : 2;
    for (int64_t m0 = 0; m0 < M; m0 += W4_GEMM_MAX_ROWS) {
        const int64_t mc = (M - m0) < W4_GEMM_MAX_ROWS ? (M - m0) : W4_GEMM_MAX_ROWS;
        w4gemm::Params p{scale_t, zc_t, (char *)y + m0 * N * es, mc, N, K, G, gs, y_dtype, 0, 0, 0};
        const void *xm = (const char *)x + m0 * K * 2;
        int rc;
        if (x_dtype == NSLQ_DTYPE_BF16) rc = zp_integer ? pick_w4_gemm<__nv_bfloat16, true>(codes, xm, p, st) : pick_w4_gemm<__nv_bfloat16, false>(codes, xm, p, st);
        else rc = zp_integer ? pick_w4_gemm<__half, true>(codes, xm, p, st) : pick_w4_gemm<__half, false>(codes, xm, p, st);
        if (rc) return rc;
    }
    return NSLQ_OK;
}

// The status word of this translation unit's kernels (see sm100::read_wait_status).
int w4a16_gemm_status(int *out) { return sm100::read_wait_status(out); }

}  // namespace nslq
