// W4A16 decode (M <= 16 tokens) on the 5th-generation tensor cores: a weight stream.
//
//   y[m,n] = sum_g scale[n,g] * sum_{k in g} (q[n,k] - zp[n,g]) * x[m,k]
//
// Same skeleton as the BitLinear decode kernel (ternary_decode_sm100.cu): the packed weights are
// the 128-row M-side operand of tcgen05.mma, expanded by the unpack warps straight into TENSOR
// memory; the (at most 16) tokens are the N side and stay resident in shared memory.  Per byte
// of weights this costs about half the instructions of the mma.sync kernel, and the tokens are
// not re-read per row tile.
//
//   Codes are fed to the tensor core undequantised: ((w >> 4s) & 0x000F000F) | MAGIC2 is a pair of
//   16-bit floats MAGIC + q (bf16: 128 + q, fp16: 1024 + q; both exact) -- one shift and one
//   three-input logic op per two weights.  The pair is (k = s, k = s + 4) of an 8-k chunk, so the
//   tokens are stored in the matching order (position 2s + h of every 8 holds k = s + 4h).
//   Every 128 k get a fresh fp32 accumulator; the epilogue warps turn it into
//       y += scale[n,g] * (acc - (MAGIC + zp[n,g]) * xsum[m, 128-block])
//   while the next blocks are being multiplied, with xsum the fp32 sum of the block's activations
//   taken when the tokens are staged.  acc is ~MAGIC * |sum x| in magnitude, so its fp32 rounding
//   (2^-24 relative) is ~1e-5 of a typical block result: far inside the 1e-2 / 1e-3 bars.
//
// Persistent, warp-specialised, one CTA per SM, tiles of 128 weight rows:
//   warp 0      TMA producer: per step one cp.async.bulk.tensor copy (this CTA only) of 128 rows x
//               128 packed bytes (256 k), SWIZZLE_128B, ring of up to 8 stages.
//   warp 2      allocates tensor memory while the others already work.
//   all but 0,2 stage the tokens (permute, block sums); then warp 1 issues the MMAs (converged
//               warp, elected lane; 16 x tcgen05.mma.kind::f16 M=128 N=16 K=16 per step, one commit
//               per step) and warps 4-7 run the epilogue above (fp32 partial outputs in registers,
//               stored once per tile).
//   warps 8-15  unpack, two groups of four warps on alternate steps, a thread per weight row.
//
// Every mbarrier wait is bounded in time; on expiry the kernel records a status word and falls
// through to the common teardown, which frees its TMEM.
#include <type_traits>

#include "sm100_common.cuh"

namespace nslq {

namespace w4dec {

using namespace sm100;

constexpr int BW = 128;                  // weight rows per tile = MMA M = TMEM lanes
constexpr int NTOK = 16;                 // MMA N: token slots
constexpr int THREADS = 512;
constexpr int KS = 2;                    // 128-k blocks per pipeline step
constexpr int PK_ROW = KS * 64;          // packed bytes per row and step = one swizzle line
constexpr int P_BYTES = BW * PK_ROW;     // 16 KiB per stage
constexpr int A_COLS = KS * 64;          // TMEM columns per operand stage (two 16-bit values per column)
constexpr int AS = 3;                    // operand stages: columns 128..511
constexpr int NB = 4;                    // accumulator buffers (one per step in flight), 32 columns each
constexpr int ACC_COLS = KS * NTOK;
constexpr int MAX_TS = 8;
constexpr int ND = 16;                   // ring of "step retired" barriers, > MAX_TS
constexpr int XB_BYTES = NTOK * 128;     // token operand of one block of 64 k: 2 KiB
constexpr int SWARPS = 14;               // every warp but the producer (0) and the allocator (2) stages the tokens
constexpr int SW = SWARPS * 32;

struct Params {
    const uint8_t *codes;    // [N][K/2], low nibble = even k
    const float *scale;      // [G][N] (transposed table: a thread per row reads coalesced)
    const float *zc;         // [G][N] zero point in code units
    const void *x;           // [M][K] bf16 or fp16
    void *y;                 // [M][N]
    int64_t N, K;
    int M, G, gs, y_dtype;
    int ts, nkb, nsteps, ntiles, gmul;       // nkb = blocks of 128 k; gmul = ceil(65536 / (128-k blocks per group))
    int off_ring, off_xsum, off_tab, off_bar;
};

static __device__ __forceinline__ void cp_async4(uint32_t dst, const void *src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
static __device__ __forceinline__ void stage_sync() { asm volatile("bar.sync 1, %0;" ::"n"(SW) : "memory"); }

template <bool BF16> static __device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t accumulate)
{
    constexpr uint32_t fmt = BF16 ? 1u : 0u;
    constexpr uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(NTOK >> 3) << 17) | ((uint32_t)(BW >> 4) << 24);
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

template <typename XT>
__global__ void __launch_bounds__(THREADS, 1)
w4a16_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const Params p)
{
    constexpr bool BF16 = std::is_same<XT, __nv_bfloat16>::value;
    constexpr uint32_t MAGIC2 = BF16 ? 0x43004300u : 0x64006400u;
    constexpr float MAGIC = BF16 ? 128.0f : 1024.0f;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                  // 1024-byte aligned (swizzle atom)
    uint8_t *base_ptr = smem_raw + (base - raw);
    // [token operand: 2*nkb blocks x 2 KiB][ring: ts x 16 KiB][xsum: nkb x 16 fp32][tables: 2 x G x 128 fp32][barriers]
    const uint32_t ring = base + p.off_ring;
    float *xsum = reinterpret_cast<float *>(base_ptr + p.off_xsum);
    float *tab = reinterpret_cast<float *>(base_ptr + p.off_tab);       // [2][G][128]: scale, zero point of the tile's rows
    const uint32_t bars = base + p.off_bar;
    auto raw_bar = [&](int t) { return bars + 8u * t; };
    auto pfree_bar = [&](int t) { return bars + 8u * (MAX_TS + t); };
    auto afull_bar = [&](int a) { return bars + 8u * (2 * MAX_TS + a); };
    auto done_bar = [&](uint32_t i) { return bars + 8u * (2 * MAX_TS + AS + (i & (ND - 1))); };
    auto done_par = [&](uint32_t i) { return (i / ND) & 1u; };
    auto acce_bar = [&](int b) { return bars + 8u * (2 * MAX_TS + AS + ND + b); };
    const uint32_t tmem_bar = bars + 8u * (2 * MAX_TS + AS + ND + NB);
    constexpr int NBAR = 2 * MAX_TS + AS + ND + NB + 1;
    const uint32_t slot = bars + 8u * NBAR;
    volatile uint32_t *slot_ptr = reinterpret_cast<volatile uint32_t *>(base_ptr + p.off_bar + 8 * NBAR);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int my_tiles = (int)blockIdx.x < p.ntiles ? (p.ntiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (threadIdx.x == 0) {
        for (int t = 0; t < p.ts; ++t) { mbar_init(raw_bar(t), 1); mbar_init(pfree_bar(t), 4); }
        for (int a = 0; a < AS; ++a) mbar_init(afull_bar(a), 4);
        for (int i = 0; i < ND; ++i) mbar_init(done_bar(i), 1);
        for (int b = 0; b < NB; ++b) mbar_init(acce_bar(b), 128);
        mbar_init(tmem_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
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
        tmem_ok = mbar_wait_warp(tmem_bar, 0, 0x740);
        tc_fence_after();
        tmem_base = *slot_ptr;
    };

    if (warp == 0) {
        // ---------------- TMA producer (the weights do not depend on the preceding kernel)
        pdl_launch_dependents();
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0, it = 0;
            bool ok = true;
            for (int j = 0; j < my_tiles && ok; ++j) {
                const int n0 = ((int)blockIdx.x + j * (int)gridDim.x) * BW;
                for (int st = 0; st < p.nsteps; ++st, ++it) {
                    if (it >= (uint32_t)p.ts) {        // the stage's previous user: step it - ts
                        if (!(ok = mbar_wait(done_bar(it - p.ts), done_par(it - p.ts), 0x701))) break;
                        if (!(ok = mbar_wait(pfree_bar(s), ph ^ 1u, 0x702))) break;
                    }
                    mbar_arrive_expect_tx(raw_bar(s), P_BYTES);
                    tma_load_2d(ring + s * P_BYTES, &tmap_w, st * PK_ROW, n0, raw_bar(s));
                    if (++s == p.ts) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else {
        if (warp != 2) {
            // ---------------- the tokens into shared memory (all warps but 0 and 2; sixteen tokens
            // are 128 KiB to permute and sum, too much for a few warps): one 16-byte chunk of 8 k
            // per thread and step, 16 consecutive lanes = one 128-k block of one token
            pdl_wait();
            const int wq = warp == 1 ? 0 : warp - 2, tq = wq * 32 + lane;
            const int chunks_row = (int)(p.K >> 3), all = p.nkb * 16 * p.M;      // padded to whole 128-k blocks
            const uint4 *src = reinterpret_cast<const uint4 *>(p.x);
            constexpr int UL = 8;                                  // loads in flight per thread
            // (token, chunk in the padded row) of this thread's element, advanced by SW per element: one
            // division per thread instead of four per element (they made this stage ten microseconds
            // long at sixteen tokens).
            const int row_chunks = p.nkb * 16;
            int m_next = tq / row_chunks, cc_next = tq - m_next * row_chunks;
            const int adv_m = SW / row_chunks, adv_c = SW - adv_m * row_chunks;
            for (int e0 = 0; e0 < all; e0 += UL * SW) {
                uint4 vv[UL];
                int mm[UL], cq[UL];
#pragma unroll
                for (int u = 0; u < UL; ++u) {
                    const int e = e0 + u * SW + tq;
                    mm[u] = m_next; cq[u] = cc_next;
                    m_next += adv_m;
                    cc_next += adv_c;
                    if (cc_next >= row_chunks) { cc_next -= row_chunks; ++m_next; }
                    vv[u] = (e < all && cq[u] < chunks_row) ? __ldg(src + (int64_t)mm[u] * chunks_row + cq[u]) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int u = 0; u < UL; ++u) {
                    const int e = e0 + u * SW + tq;
                    const bool in = e < all;
                    const int m = in ? mm[u] : 0, cc = in ? cq[u] : 0;   // chunk index in the padded row
                    const uint4 v = vv[u];
                    // (e0..e7) -> positions (e0,e4,e1,e5,e2,e6,e3,e7)
                    uint4 o;
                    o.x = __byte_perm(v.x, v.z, 0x5410); o.y = __byte_perm(v.x, v.z, 0x7632);
                    o.z = __byte_perm(v.y, v.w, 0x5410); o.w = __byte_perm(v.y, v.w, 0x7632);
                    float sum = 0.0f;
                    const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if constexpr (BF16) {
                            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&ww[i]));
                            sum += f.x + f.y;
                        } else {
                            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&ww[i]));
                            sum += f.x + f.y;
                        }
                    }
#pragma unroll
                    for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);   // 16 lanes = one block
                    if (in) {
                        const int bb = cc >> 3, c = cc & 7;                // block of 64 k, chunk inside it
                        *reinterpret_cast<uint4 *>(base_ptr + (size_t)bb * XB_BYTES + (m >> 3) * 1024 + (m & 7) * 128 +
                                                   ((c ^ (m & 7)) << 4)) = o;
                        if ((lane & 15) == 0) xsum[(cc >> 4) * NTOK + m] = sum;
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
                for (int st = 0; st < p.nsteps; ++st, ++it) {
                    const uint32_t sb = it % NB;
                    if (!(ok = mbar_wait_warp(acce_bar(sb), ((it / NB) & 1u) ^ 1u, 0x711))) break;   // accumulators of step it - NB read out
                    if (!(ok = mbar_wait_warp(afull_bar(a), aph, 0x712))) break;
                    tc_fence_after();
                    if (leader) {
                        const uint32_t a_tmem = tmem_base + NB * ACC_COLS + a * A_COLS;
#pragma unroll
                        for (int ks = 0; ks < KS; ++ks) {
                            const int kb = st * KS + ks;
                            if (kb < p.nkb) {
                                const uint32_t d_tmem = tmem_base + sb * ACC_COLS + NTOK * ks;
#pragma unroll
                                for (int k16 = 0; k16 < 8; ++k16) {          // 16 k = 32 bytes = 8 columns per MMA
                                    const uint64_t bdesc = smem_desc(base + (2 * kb + (k16 >> 2)) * XB_BYTES) + 2u * (k16 & 3);
                                    umma_f16_ts<BF16>(d_tmem, a_tmem + 64u * ks + 8u * k16, bdesc, k16 != 0);
                                }
                            }
                        }
                        umma_commit(done_bar(it));
                    }
                    if (++a == AS) { a = 0; aph ^= 1u; }
                }
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
                if (!(ok = mbar_wait_warp(raw_bar(s), sph, 0x721))) break;
                const uint8_t *pr = base_ptr + p.off_ring + (size_t)s * P_BYTES + row * PK_ROW;
                uint4 pv[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) pv[c] = *reinterpret_cast<const uint4 *>(pr + ((c ^ (row & 7)) << 4));
                if (it >= AS && !(ok = mbar_wait_warp(done_bar(it - AS), done_par(it - AS), 0x722))) break;
                tc_fence_after();
#pragma unroll
                for (int h = 0; h < 4; ++h) {            // 32 packed bytes = 64 k = 32 columns
                    const uint32_t wv[8] = {pv[2 * h].x, pv[2 * h].y, pv[2 * h].z, pv[2 * h].w,
                                            pv[2 * h + 1].x, pv[2 * h + 1].y, pv[2 * h + 1].z, pv[2 * h + 1].w};
                    uint32_t r[32];
#pragma unroll
                    for (int jw = 0; jw < 8; ++jw)
#pragma unroll
                        for (int sft = 0; sft < 4; ++sft) r[4 * jw + sft] = ((wv[jw] >> (4 * sft)) & 0x000F000Fu) | MAGIC2;
                    tmem_st32_issue(tmem_base + ((uint32_t)(qd * 32) << 16) + NB * ACC_COLS + a * A_COLS + 32u * h, r);
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
            // ---------------- epilogue warps: one weight row per thread, 16 partial outputs in registers
            const int qd = warp & 3;
            get_tmem();
            bool ok = tmem_ok;
            uint32_t it = 0;
            for (int j = 0; j < my_tiles && ok; ++j) {
                const int64_t n = ((int64_t)blockIdx.x + (int64_t)j * gridDim.x) * BW + qd * 32 + lane;
                const bool n_ok = n < p.N;
                float yacc[NTOK];
#pragma unroll
                for (int t = 0; t < NTOK; ++t) yacc[t] = 0.0f;
                // The row's group constants (scale, zero point) go to shared memory once per tile with
                // 4-byte cp.async (coalesced: the tables are [G][N]); loads issued inside the step loop,
                // however far ahead, cost ~750 cycles a step here.  A thread reads back only what it
                // copied itself, so no barrier is needed.
                float *tab_s = tab + (qd * 32 + lane), *tab_z = tab_s + p.G * BW;
                if (n_ok) {
                    for (int g = 0; g < p.G; ++g) {
                        cp_async4(smem_u32(tab_s + g * BW), p.scale + (int64_t)g * p.N + n);
                        cp_async4(smem_u32(tab_z + g * BW), p.zc + (int64_t)g * p.N + n);
                    }
                }
                asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
                for (int st = 0; st < p.nsteps && ok; ++st, ++it) {
                    const uint32_t sb = it % NB;
                    // The step's group constants and token sums do not depend on the MMAs: they are read
                    // before the wait, so their latency hides behind it (this warp is alone on its
                    // scheduler for most of the tile and nothing else would cover it).
                    float sc[KS], cm[KS];
                    float4 xs[KS][NTOK / 4];
#pragma unroll
                    for (int ks = 0; ks < KS; ++ks) {
                        const int kb = st * KS + ks, kbc = min(kb, p.nkb - 1);
                        const int g = (int)(((uint32_t)kbc * (uint32_t)p.gmul) >> 16);   // kb / (128-k blocks per group), no divide
                        sc[ks] = kb < p.nkb ? tab_s[g * BW] : 0.0f;
                        cm[ks] = -(MAGIC + tab_z[g * BW]);
                        const float4 *xs4 = reinterpret_cast<const float4 *>(xsum + kbc * NTOK);
#pragma unroll
                        for (int t4 = 0; t4 < NTOK / 4; ++t4) xs[ks][t4] = xs4[t4];
                    }
                    if (!(ok = mbar_wait_warp(done_bar(it), done_par(it), 0x731))) break;
                    tc_fence_after();
                    uint32_t r[KS * NTOK];
                    tmem_ld32(tmem_base + ((uint32_t)(qd * 32) << 16) + sb * ACC_COLS, r);
                    tc_fence_before();
                    mbar_arrive(acce_bar(sb));
#pragma unroll
                    for (int t4 = 0; t4 < NTOK / 4; ++t4) {
                        if (4 * t4 >= p.M) continue;                         // warp-uniform: only the tokens that exist
#pragma unroll
                        for (int ks = 0; ks < KS; ++ks) {
                            if (st * KS + ks >= p.nkb) continue;             // warp-uniform: its accumulator was never written
                            const float xe[4] = {xs[ks][t4].x, xs[ks][t4].y, xs[ks][t4].z, xs[ks][t4].w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int t = 4 * t4 + e;
                                yacc[t] = fmaf(sc[ks], fmaf(cm[ks], xe[e], __uint_as_float(r[ks * NTOK + t])), yacc[t]);
                            }
                        }
                    }
                }
                if (ok && n_ok) {
#pragma unroll
                    for (int t = 0; t < NTOK; ++t)
                        if (t < p.M) store_out(p.y, p.y_dtype, (int64_t)t * p.N + n, yacc[t]);   // warp-uniform test
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

}  // namespace w4dec

// ---------------------------------------------------------------- host side
static int w4dec_smem_budget()
{
    static int v = 0;
    if (!v) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    }
    return v;
}

static bool w4dec_plan(w4dec::Params &p, int *smem_bytes, int *grid)
{
    using namespace w4dec;
    p.nkb = (int)((p.K + 127) / 128);
    p.nsteps = (p.nkb + KS - 1) / KS;
    p.ntiles = (int)((p.N + BW - 1) / BW);
    const int xs = 2 * p.nkb * XB_BYTES;
    const int xsum = (p.nkb * NTOK * 4 + 127) & ~127, bar_bytes = 512;
    const int tabs = 2 * p.G * BW * 4;
    const int room = w4dec_smem_budget() - 1024 - xs - xsum - tabs - bar_bytes;
    p.ts = room / P_BYTES;
    if (p.ts > MAX_TS) p.ts = MAX_TS;
    if (p.ts < 3) return false;
    p.off_ring = xs;
    p.off_xsum = xs + p.ts * P_BYTES;
    p.off_tab = p.off_xsum + xsum;
    p.off_bar = p.off_tab + tabs;
    *smem_bytes = 1024 + p.off_bar + bar_bytes;
    *grid = p.ntiles < sm100::sm_count() ? p.ntiles : sm100::sm_count();
    return true;
}

// bf16 or fp16 activations, M <= 16, groups of a multiple of 128 k, K % 64 == 0, 16-byte aligned
// pointers, tokens small enough to stay in shared memory (K up to ~5000).
bool w4a16_decode_supported(const void *codes, const void *x, int x_dtype, int64_t M, int64_t N, int64_t K, int64_t gs)
{
    if (!(x_dtype == NSLQ_DTYPE_BF16 || x_dtype == NSLQ_DTYPE_FP16)) return false;
    if (!(M >= 1 && M <= w4dec::NTOK && (K % 64 == 0) && (gs % 128 == 0) && aligned16(codes) && aligned16(x) &&
          N < (1ll << 31) && K < (1ll << 24)))
        return false;
    w4dec::Params p{};
    p.N = N; p.K = K; p.M = (int)M; p.gs = (int)gs; p.G = (int)((K + gs - 1) / gs);
    int smem = 0, grid = 0;
    return w4dec_plan(p, &smem, &grid);
}

template <typename XT>
static int launch_w4_decode(w4dec::Params &p, cudaStream_t st)
{
    int smem = 0, grid = 0;
    if (!w4dec_plan(p, &smem, &grid))
        return fail(NSLQ_ERR_UNSUPPORTED, "w4a16_decode_kernel: K=%lld does not fit shared memory", (long long)p.K);
    static std::atomic<size_t> reserved[kMaxDevices];
    if (reserve_smem(w4dec::w4a16_decode_kernel<XT>, reserved, (size_t)smem) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "w4a16_decode_kernel: cannot reserve %d bytes of shared memory: %s", smem,
                    cudaGetErrorString(cudaGetLastError()));
    CUtensorMap tmap_w;
    int rc = sm100::make_map_2d(&tmap_w, p.codes, (uint64_t)(p.K / 2), (uint64_t)p.N, w4dec::PK_ROW, w4dec::BW, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    cudaError_t e = launch_kernel(w4dec::w4a16_decode_kernel<XT>, dim3(grid), dim3(w4dec::THREADS), (size_t)smem, st, tmap_w, p);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "w4a16_decode_kernel: %s", cudaGetErrorString(e));
    return check_launch("w4a16_decode_kernel");
}

int w4a16_decode_dispatch(const uint8_t *codes, const float *scale, const float *zc, int64_t N, int64_t K, int G, int gs,
                          const void *x, int x_dtype, int M, void *y, int y_dtype, cudaStream_t st)
{
    w4dec::Params p{};
    p.codes = codes; p.scale = scale; p.zc = zc; p.x = x; p.y = y; p.N = N; p.K = K; p.M = M; p.G = G; p.gs = gs;
    p.y_dtype = y_dtype; p.gmul = (65536 + gs / 128 - 1) / (gs / 128);
    return x_dtype == NSLQ_DTYPE_BF16 ? launch_w4_decode<__nv_bfloat16>(p, st) : launch_w4_decode<__half>(p, st);
}

// The status word of this translation unit's kernels (see sm100::read_wait_status).
int w4a16_decode_status(int *out) { return sm100::read_wait_status(out); }

}  // namespace nslq
