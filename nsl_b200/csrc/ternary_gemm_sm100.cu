// Stage 3: BitLinear prefill GEMM on the 5th-generation tensor cores (sm_100a).
//
//   acc[m,n] = sum_k q[m,k] * W[n,k]        int8 x ternary, exact int32
//
// The product is computed transposed, D[n, m] = W[n, :] . q[m, :], so that the weight
// codes are the M-side operand and can live in TENSOR memory: the unpack warps write them
// with tcgen05.st and they never pass through shared memory as bytes.  Shared memory then
// carries only the int8 activations (written once by the copy engine, read once by the
// tensor core) and the still-packed 2-bit weights -- about 60 % of the bytes per MAC of
// a layout that expands the codes in shared memory, and shared-memory bandwidth is what
// bounds this kernel.  A side effect: an accumulator lane is an output feature, so 32
// lanes hold 32 consecutive n of one token and the epilogue stores whole 128-byte lines
// straight from registers, with no transposition patch.
//
// Persistent, warp-specialised kernel, one CTA per SM, tiles of 128 weight rows x BT tokens:
//
//   warp 0      TMA producer: per step, cp.async.bulk.tensor copies (2-D, this CTA only)
//               into a ring of copy stages: the int8 activation tile (BT tokens x 128 k
//               per k-block, SWIZZLE_128B) and the packed weight tile (128 rows x 32
//               bytes per k-block, swizzled so that a thread per row reads without bank
//               conflicts); out-of-range rows and the K tail are zero-filled.
//   warps 8-15  unpack, two groups of four warps (one warp per TMEM lane quadrant) taking
//               alternate k-blocks: each thread reads the 32 packed bytes of its weight
//               row, expands them with (w >> s) & 0x03030303 into 32 words of u8 codes
//               {0,1,2} and stores them into its lane of a ring of TMEM operand stages.
//               The activations are stored in the matching order (position 4i+j of
//               every 16 holds k = 4j+i), so nothing is permuted here.
//   warp 1      MMA issuer: the warp runs the loop in uniform control flow and one
//               elected lane issues tcgen05.mma.kind::i8 (M=128, N=BT, K=32; A = u8 codes
//               in TMEM, B = s8 activations in shared memory, D = s32 in TMEM) four times
//               per k-block and releases both stages with tcgen05.commit.  It waits only
//               for the codes: they are published after the copy stage was seen complete,
//               so the activation tile of the same copy stage has landed too.
//   warps 4-7,  epilogue, two warps per TMEM lane quadrant, each taking half of the
//   16-19       tile's tokens: tcgen05.ld the accumulator (double-buffered in TMEM, so
//               the next tile's MMAs run meanwhile), subtract the token's row sum
//               (code = trit + 1), apply ((scale/127)*acc)*weight_scale with separately
//               rounded steps and store.
//
// Every mbarrier wait is bounded in time; on expiry the kernel records a status
// word (read with nslq_device_status) and falls through to the common teardown,
// which frees its TMEM.  No spin is unbounded and no block-wide barrier sits inside a role.
#include "sm100_common.cuh"

namespace nslq {

namespace gemm {

using namespace sm100;

constexpr int BW = 128;                  // weight rows per tile = MMA M = TMEM lanes
constexpr int BK = 128;                  // bytes of int8 along K per k-block = one 128B swizzle row
constexpr int THREADS = 640;            // 20 warps: 0 TMA, 1 MMA, 4-7 and 16-19 epilogue, 8-15 unpack

template <int BT> struct Cfg {
    static_assert(BT == 64 || BT == 128 || BT == 192, "token tile");
    // k-blocks (128 k) per pipeline step.  One step costs the MMA warp one barrier round trip and
    // two commits whatever its size, and with one k-block per step that overhead, not the tensor
    // pipe, set the pace; the wide tile has TMEM columns for single k-block stages only.
    static constexpr int KS = (BT == 192) ? 1 : 2;
    static constexpr int X_SUB = BT * BK;                             // one 128-byte-swizzled activation sub-tile
    static constexpr int X_BYTES = KS * X_SUB;
    static constexpr int PK_ROW = KS * (BK / 4);                      // packed bytes per weight row and step
    static constexpr int P_BYTES = BW * PK_ROW;                       // packed 2-bit weight tile as it sits in global memory
    static constexpr int T_BYTES = X_BYTES + P_BYTES;                 // one copy stage, multiple of 1024
    static constexpr int TS = (BT == 128) ? 5 : 7;                      // copy stages in flight
    static constexpr int A_COLS = 32 * KS;                            // TMEM columns per operand stage
    static constexpr int AS = (512 - 2 * BT) / A_COLS;                // TMEM operand stages: 4
    static constexpr int HALF_T = BT / 2;                             // tokens per epilogue warp
    static constexpr int SCALE_BYTES = 8 * HALF_T * 8;                // per epilogue warp: scale/127 and row sum per token
    static constexpr int BAR_BYTES = 512;
    static constexpr int STAGE_BYTES = 2 * 16 * 128 * 4;              // per token half: 16 tokens x 128 features of output, up to 4 bytes each
    static constexpr int SMEM = TS * T_BYTES + SCALE_BYTES + BAR_BYTES + STAGE_BYTES + 1024;   // + alignment slack
    static_assert(SMEM <= 232448, "over the 227 KiB a CTA may use");
    static constexpr uint32_t IDESC = (2u << 4)        // D format: s32
                                      | (0u << 7)      // A format: unsigned 8-bit (codes)
                                      | (1u << 10)     // B format: signed 8-bit (activations)
                                      | ((uint32_t)(BT >> 3) << 17) | ((uint32_t)(BW >> 4) << 24);
    // TMEM columns (512 allocated).  BT = 64, 128: accumulators at 0 and BT, operand stages from 2 BT.
    // BT = 192: accumulators at 0 and 256 (kept on 256-column boundaries), operand stages in the
    // two 64-column gaps behind them.
    static __device__ __forceinline__ uint32_t acc_col(uint32_t buf) { return BT == 192 ? buf * 256u : buf * (uint32_t)BT; }
    static __device__ __forceinline__ uint32_t a_col(uint32_t a)
    {
        return BT == 192 ? 192u + 32u * (a & 1u) + 256u * (a >> 1) : 2u * BT + (uint32_t)A_COLS * a;
    }
};

struct Params {
    const uint8_t *w;        // [N][K/4]
    const float *scale;      // [M]
    const int32_t *rowsum;   // [M]
    void *y;                 // [M][N]
    int32_t *acc_out;        // [M][N] or null
    const float *bias;       // [N] or null
    const float *residual;   // [M][N] or null
    int64_t M, N, K;
    int y_dtype;
    float weight_scale;
    int tiles_t, tiles_w;    // token tiles, weight-row tiles
    int64_t ldy;             // elements between consecutive token rows of y (N when y is [M][N])
    int npeer;               // copies of y in other GPUs' memory that receive the same stores
    void *y_peer[NSLQ_MAX_RANKS - 1];
    int wide;                // y, its copies and ldy allow 16-byte stores
};

template <typename T> struct OutStore;
template <> struct OutStore<float> {
    static __device__ __forceinline__ float cvt(float v) { return v; }
    static __device__ __forceinline__ void put(void *y, int64_t o, float v) { reinterpret_cast<float *>(y)[o] = v; }
};
template <> struct OutStore<__nv_bfloat16> {
    static __device__ __forceinline__ __nv_bfloat16 cvt(float v) { return __float2bfloat16_rn(v); }
    static __device__ __forceinline__ void put(void *y, int64_t o, float v) { reinterpret_cast<__nv_bfloat16 *>(y)[o] = __float2bfloat16_rn(v); }
};
template <> struct OutStore<__half> {
    static __device__ __forceinline__ __half cvt(float v) { return __float2half_rn(v); }
    static __device__ __forceinline__ void put(void *y, int64_t o, float v) { reinterpret_cast<__half *>(y)[o] = __float2half_rn(v); }
};

// Barrier of the four epilogue warps that share a token half (ids 1 and 2; id 0 is __syncthreads).  Every one of
// the four executes the same sequence of these: they are reached only between the wait for a finished
// accumulator, which the four pass or give up together, and the end of that tile's groups, with no exit between.
static __device__ __forceinline__ void half_sync(int half)
{
    asm volatile("bar.sync %0, 128;" ::"r"(1 + half) : "memory");
}

// Sixteen tokens of one accumulator lane (output feature n): finalise and store.  Kept small and
// called from a rolled loop on purpose: the epilogue as straight-line code for a whole tile does
// not fit the instruction cache next to the other roles and then runs at the refill rate.
constexpr int EG = 16;                   // tokens per epilogue step
// `valid` (tokens of the group inside M) is warp-uniform.  The arithmetic is branch-free so the 16
// independent chains overlap; only the stores are guarded, by one test per group on the common path.
//
// Full tiles of a result that allows 16-byte stores go out through shared memory (`stage`, [16 tokens][128
// features] of the four warps of a token half): a lane owns one feature, so direct stores are 2 or 4 bytes per
// lane and 64 or 128 contiguous bytes per instruction -- over NVLink, into the other ranks' copies, such
// stores reached 340 GB/s where 16 bytes per lane in whole 256- or 512-byte rows reach 560.
template <typename T>
static __device__ __forceinline__ void store_group(const Params &p, const uint32_t (&r)[EG], const float *s127, const int *rs,
                                                   int64_t mt, int64_t n0, int q, int lane, int half, bool wide, T *stage, float bias)
{
    const int64_t n = n0 + q * 32 + lane;
    const bool n_ok = n < p.N;
    int acc[EG];
    float v[EG];
#pragma unroll
    for (int j4 = 0; j4 < EG / 4; ++j4) {
        const float4 sv = *reinterpret_cast<const float4 *>(s127 + 4 * j4);
        const int4 rv = *reinterpret_cast<const int4 *>(rs + 4 * j4);
        const float se[4] = {sv.x, sv.y, sv.z, sv.w};
        const int re[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int j = 4 * j4 + e;
            acc[j] = (int)r[j] - re[e];
            v[j] = __fmul_rn(__fmul_rn(se[e], __int2float_rn(acc[j])), p.weight_scale);
        }
    }
    if (p.bias) {
#pragma unroll
        for (int j = 0; j < EG; ++j) v[j] = __fadd_rn(v[j], bias);
    }
    const int64_t o = mt * p.N + n;
    const int64_t left = p.M - mt;
    if (wide) {                                        // uniform over the four warps of the half; the tile lies inside N
        if (p.acc_out || p.residual) {
#pragma unroll
            for (int j = 0; j < EG; ++j) {
                if (j < left) {
                    if (p.acc_out) p.acc_out[o + j * p.N] = acc[j];
                    if (p.residual) v[j] = __fadd_rn(v[j], p.residual[o + j * p.N]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < EG; ++j) stage[j * BW + q * 32 + lane] = OutStore<T>::cvt(v[j]);
        half_sync(half);
        constexpr int VR = BW * (int)sizeof(T) / 16;   // 16-byte vectors per row of the tile
        constexpr int RPI = 32 / VR;                   // rows per warp instruction
#pragma unroll
        for (int i = 0; i < 4 / RPI; ++i) {
            const int row = 4 * q + i * RPI + lane / VR, c = lane % VR;
            if (row < left) {
                const uint4 val = reinterpret_cast<const uint4 *>(stage)[row * VR + c];
                const int64_t off = ((mt + row) * p.ldy + n0) * (int64_t)sizeof(T) + 16 * c;
                *reinterpret_cast<uint4 *>(reinterpret_cast<char *>(p.y) + off) = val;
                // column-sharded run: the same rows go straight into every other rank's copy of the
                // gathered output (plain stores over NVLink; the all-gather rides in the epilogue)
                for (int pi = 0; pi < p.npeer; ++pi) *reinterpret_cast<uint4 *>(reinterpret_cast<char *>(p.y_peer[pi]) + off) = val;
            }
        }
        half_sync(half);                               // the stage is free for the next group
        return;
    }
    // no early return for lanes past N: the caller's next instruction is a warp-wide
    // tcgen05.ld, which every lane must reach together
    if (n_ok) {
    const int64_t oy = mt * p.ldy + n;
    if (left >= EG) {
        if (p.acc_out) {
#pragma unroll
            for (int j = 0; j < EG; ++j) p.acc_out[o + j * p.N] = acc[j];
        }
        if (p.residual) {
            float res[EG];
#pragma unroll
            for (int j = 0; j < EG; ++j) res[j] = p.residual[o + j * p.N];
#pragma unroll
            for (int j = 0; j < EG; ++j) v[j] = __fadd_rn(v[j], res[j]);
        }
#pragma unroll
        for (int j = 0; j < EG; ++j) OutStore<T>::put(p.y, oy + j * p.ldy, v[j]);
        for (int pi = 0; pi < p.npeer; ++pi) {
            void *yp = p.y_peer[pi];
#pragma unroll
            for (int j = 0; j < EG; ++j) OutStore<T>::put(yp, oy + j * p.ldy, v[j]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < EG; ++j) {
            if (j < left) {
                const int64_t oj = o + j * p.N;
                if (p.acc_out) p.acc_out[oj] = acc[j];
                float vj = v[j];
                if (p.residual) vj = __fadd_rn(vj, p.residual[oj]);
                OutStore<T>::put(p.y, oy + j * p.ldy, vj);
                for (int pi = 0; pi < p.npeer; ++pi) OutStore<T>::put(p.y_peer[pi], oy + j * p.ldy, vj);
            }
        }
    }
    }
}

// ---------------------------------------------------------------- kernel
template <int BT>
__global__ void __launch_bounds__(THREADS, 1)
ternary_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, const Params p)
{
    using C = Cfg<BT>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                  // 1024-byte aligned (swizzle atom)
    uint8_t *base_ptr = smem_raw + (base - raw);
    float *scale_ptr = reinterpret_cast<float *>(base_ptr + C::TS * C::T_BYTES);
    const uint32_t bars = base + C::TS * C::T_BYTES + C::SCALE_BYTES;
    // barrier map (8 bytes each): raw[t] (copy stage landed), pfree[t] (packed tile of the copy stage
    // read by the four unpack warps), afull[a] (codes stored in TMEM), done[8] (MMAs of step i retired,
    // i mod 8: ONE commit per step, which frees both the copy stage i mod TS and the operand stage
    // i mod AS -- a second commit per step cost the issuing thread ~190 cycles), acc_full[2],
    // acc_empty[2]; then the TMEM slot.  A waiter of done[] is at most TS steps behind the commit it
    // waits for and the ring has 8 > TS entries, so the phase it tests cannot have been overtaken.
    constexpr int ND = 8;
    static_assert(C::TS < ND && C::AS < ND, "done ring too short");
    constexpr int NBAR = 2 * C::TS + C::AS + ND + 5;
    static_assert(NBAR * 8 + 16 <= C::BAR_BYTES, "barrier area");
    auto raw_bar = [&](int t) { return bars + 8u * t; };
    auto pfree_bar = [&](int t) { return bars + 8u * (C::TS + t); };
    auto afull_bar = [&](int a) { return bars + 8u * (2 * C::TS + a); };
    auto done_bar = [&](uint32_t i) { return bars + 8u * (2 * C::TS + C::AS + (i & (ND - 1))); };
    auto accf_bar = [&](int b) { return bars + 8u * (2 * C::TS + C::AS + ND + b); };
    auto acce_bar = [&](int b) { return bars + 8u * (2 * C::TS + C::AS + ND + 2 + b); };
    const uint32_t drain_bar = bars + 8u * (2 * C::TS + C::AS + ND + 4);   // used only when a wait gave up
    // parity of the phase of done[i mod 8] that step i completes
    auto done_par = [&](uint32_t i) { return (i / ND) & 1u; };
    const uint32_t slot = bars + 8u * NBAR;
    volatile uint32_t *slot_ptr = reinterpret_cast<volatile uint32_t *>(base_ptr + C::TS * C::T_BYTES + C::SCALE_BYTES + 8 * NBAR);
    // CTA-wide "a wait gave up" flag: raised by the role whose wait expired, seen by every other wait
    volatile int *abort_flag = reinterpret_cast<volatile int *>(base_ptr + C::TS * C::T_BYTES + C::SCALE_BYTES + 8 * NBAR + 8);

    uint8_t *stage_ptr = base_ptr + C::TS * C::T_BYTES + C::SCALE_BYTES + C::BAR_BYTES;   // output staging of the epilogue

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (int)((p.K + BK * C::KS - 1) / (BK * C::KS));   // pipeline steps per tile
    const int ntiles = p.tiles_t * p.tiles_w;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int t = 0; t < C::TS; ++t) { mbar_init(raw_bar(t), 1); mbar_init(pfree_bar(t), 4); }
        for (int a = 0; a < C::AS; ++a) mbar_init(afull_bar(a), 4);
        for (int i = 0; i < ND; ++i) mbar_init(done_bar(i), 1);
        for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), 256); }
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

    pdl_wait();   // activations, scales and row sums come from the preceding kernel
    // The next kernel of the stream may be scheduled from here on: it takes the SMs this grid leaves idle
    // (fewer tiles than SMs, the last partial round) for its own prologue and waits for this grid's
    // completion before it touches memory.
    pdl_launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer (activation tile + packed weight tile)
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0, it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const int m0 = (tile % p.tiles_t) * BT, n0 = (tile / p.tiles_t) * BW;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    if (it >= (uint32_t)C::TS) {       // the stage's previous user: step it - TS
                        if (!(ok = mbar_wait(done_bar(it - C::TS), done_par(it - C::TS), 0x101, abort_flag))) break;
                        if (!(ok = mbar_wait(pfree_bar(s), ph ^ 1u, 0x102, abort_flag))) break;
                    }
                    const uint32_t st = base + s * C::T_BYTES;
                    mbar_arrive_expect_tx(raw_bar(s), C::T_BYTES);
#pragma unroll
                    for (int ks = 0; ks < C::KS; ++ks)
                        tma_load_2d(st + ks * C::X_SUB, &tmap_x, (kb * C::KS + ks) * BK, m0, raw_bar(s));
                    tma_load_2d(st + C::X_BYTES, &tmap_w, kb * C::PK_ROW, n0, raw_bar(s));
                    if (++s == C::TS) { s = 0; ph ^= 1u; }
                }
            }
            if (*abort_flag) {
                // A wait gave up somewhere in this CTA.  Copies this thread issued may still be on
                // their way into shared memory; the CTA must not end under them.  Wait (bounded, and
                // without looking at the flag) for the last TS stages it armed.
                const uint32_t first = it > (uint32_t)C::TS ? it - C::TS : 0u;
                for (uint32_t j = first; j < it; ++j)
                    mbar_wait(raw_bar((int)(j % C::TS)), (j / C::TS) & 1u, 0x103);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer.  The whole warp runs the loop in uniform control flow and one
        // elected lane issues: measured here, eight MMAs issue in ~120 cycles from a converged warp
        // and in ~450 from a lone diverged lane.
        const bool leader = elect_one();
        uint32_t a = 0, aph = 0, t = 0, it = 0;
        int s = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++t) {
            const uint32_t buf = t & 1u, cph = (t >> 1) & 1u;
            if (!(ok = mbar_wait_warp(acce_bar(buf), cph ^ 1u, 0x201, abort_flag))) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + C::acc_col(buf);
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                if (!(ok = mbar_wait_warp(afull_bar(a), aph, 0x203, abort_flag))) break;    // codes stored (and the copy stage landed)
                tc_fence_after();
                if (leader) {
                    const uint32_t a_tmem = tmem_base + C::a_col(a);
                    // MMAs of this step that hold any k < K (the last step of a tile may be part empty)
                    const int64_t k_left = p.K - (int64_t)kb * (BK * C::KS);
                    const int nmma = k_left >= BK * C::KS ? 4 * C::KS : (int)((k_left + 31) / 32);
#pragma unroll
                    for (int k4 = 0; k4 < 4 * C::KS; ++k4) {   // 32 bytes of K per MMA: 8 TMEM columns, descriptor start + 2 (16-byte units)
                        const uint64_t bdesc = smem_desc(base + s * C::T_BYTES + (k4 >> 2) * C::X_SUB);
                        if (k4 < nmma) umma_i8_ts(d_tmem, a_tmem + 8u * k4, bdesc + 2u * (k4 & 3), C::IDESC, (kb | k4) != 0);
                    }
                    umma_commit(done_bar(it));
                }
                if (++s == C::TS) s = 0;
                if (++a == C::AS) { a = 0; aph ^= 1u; }
            }
            if (ok && leader) umma_commit(accf_bar(buf));
        }
        if (__any_sync(0xffffffffu, *abort_flag != 0)) {
            // Leaving early: tensor memory is freed in the teardown, so every MMA issued so far must
            // have retired first.  One more commit tracks them all; wait for it (bounded).
            if (leader) umma_commit(drain_bar);
            __syncwarp();
            mbar_wait_warp(drain_bar, 0, 0x204);
        }
    } else if (warp >= 8 && warp < 16) {
        // ---------------- unpack warps (packed row -> u8 codes in this thread's TMEM lane)
        const int q = warp & 3;                      // TMEM lane quadrant of this warp
        const int group = (warp - 8) >> 2;           // group 0 takes even pipeline iterations, group 1 odd
        const int row = q * 32 + lane;
        bool ok = true;
        const int total_it = ((ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x) * nkb;
        int s = group % C::TS;                       // ring positions of iteration `it`, stepped by two
        uint32_t a = group % C::AS, sph = 0, aph = 0;
        for (int it = group; it < total_it && ok; it += 2) {
            if (!(ok = mbar_wait_warp(raw_bar(s), sph, 0x301, abort_flag))) break;                            // packed tile landed
            // The packed tile is copied with a 64-byte (KS = 2) or 32-byte (KS = 1) swizzle: 16-byte chunk c of row r
            // sits at chunk c ^ ((r >> 1) & 3) resp. c ^ ((r >> 2) & 1), which spreads the eight rows a quarter-warp
            // reads at once over all banks (unswizzled, rows 64 or 32 bytes apart collide four resp. two ways).
            const uint4 *pk = reinterpret_cast<const uint4 *>(base_ptr + s * C::T_BYTES + C::X_BYTES + row * C::PK_ROW);
            const int sw = C::KS == 2 ? ((row >> 1) & 3) : ((row >> 2) & 1);
            uint4 pv[2 * C::KS];
#pragma unroll
            for (int i = 0; i < 2 * C::KS; ++i) pv[i] = pk[i ^ sw];
            if (it >= C::AS && !(ok = mbar_wait_warp(done_bar(it - C::AS), done_par(it - C::AS), 0x302, abort_flag))) break;   // operand stage reusable
            tc_fence_after();
#pragma unroll
            for (int h = 0; h < C::KS; ++h) {                                                // one k-block: 32 bytes -> 32 columns
                const uint32_t wv[8] = {pv[2 * h].x, pv[2 * h].y, pv[2 * h].z, pv[2 * h].w,
                                        pv[2 * h + 1].x, pv[2 * h + 1].y, pv[2 * h + 1].z, pv[2 * h + 1].w};
                uint32_t r[32];
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    r[4 * g + 0] = (wv[g] >> 6) & 0x03030303u; r[4 * g + 1] = (wv[g] >> 4) & 0x03030303u;
                    r[4 * g + 2] = (wv[g] >> 2) & 0x03030303u; r[4 * g + 3] = wv[g] & 0x03030303u;
                }
                tmem_st32_issue(tmem_base + ((uint32_t)(q * 32) << 16) + C::a_col(a) + 32u * h, r);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(afull_bar(a));
                mbar_arrive(pfree_bar(s));
            }
            if ((s += 2) >= C::TS) { s -= C::TS; sph ^= 1u; }
            if ((a += 2) >= (uint32_t)C::AS) { a -= C::AS; aph ^= 1u; }
        }
    } else if (warp >= 4) {
        // ---------------- epilogue warps (TMEM -> registers -> global)
        const int q = warp & 3;                       // TMEM lane quadrant of this warp
        const int half = warp >> 4;                   // warps 4-7: first half of the tile's tokens, 16-19: second
        float *s127 = scale_ptr + (half * 4 + q) * 2 * C::HALF_T;         // this warp's per-token factors
        int *rs = reinterpret_cast<int *>(s127 + C::HALF_T);
        uint32_t t = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++t) {
            const uint32_t buf = t & 1u, cph = (t >> 1) & 1u;
            const int64_t m0 = (int64_t)(tile % p.tiles_t) * BT + half * C::HALF_T, n0 = (int64_t)(tile / p.tiles_t) * BW;
            const int64_t n = n0 + q * 32 + lane;
            const float bias = (p.bias && n < p.N) ? p.bias[n] : 0.0f;
            const bool wide = p.wide && n0 + BW <= p.N;
            uint8_t *stage = stage_ptr + half * (C::STAGE_BYTES / 2);
            __syncwarp();                             // the previous tile's reads of the factors are done
            for (int i = lane; i < C::HALF_T; i += 32) {
                const int64_t m = m0 + i;
                s127[i] = m < p.M ? __fdiv_rn(p.scale[m], 127.0f) : 0.0f;
                rs[i] = m < p.M ? p.rowsum[m] : 0;
            }
            __syncwarp();
            if (!(ok = mbar_wait_warp(accf_bar(buf), cph, 0x401, abort_flag))) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + C::acc_col(buf) + half * C::HALF_T;
#pragma unroll 1
            for (int g = 0; g < C::HALF_T / EG; ++g) {
                uint32_t r[EG];
                __syncwarp();                         // tcgen05.ld is warp-wide: re-form the warp after the guarded stores
                tmem_ld16(taddr + g * EG, r);
                if (g == C::HALF_T / EG - 1) {       // this thread's last read of the accumulator: hand it back
                    tc_fence_before();
                    mbar_arrive(acce_bar(buf));
                }
                const int64_t mt = m0 + g * EG;
                if (mt >= p.M) continue;             // warp-uniform
                if (p.y_dtype == NSLQ_DTYPE_F32)
                    store_group<float>(p, r, s127 + g * EG, rs + g * EG, mt, n0, q, lane, half, wide, reinterpret_cast<float *>(stage), bias);
                else if (p.y_dtype == NSLQ_DTYPE_BF16)
                    store_group<__nv_bfloat16>(p, r, s127 + g * EG, rs + g * EG, mt, n0, q, lane, half, wide, reinterpret_cast<__nv_bfloat16 *>(stage), bias);
                else
                    store_group<__half>(p, r, s127 + g * EG, rs + g * EG, mt, n0, q, lane, half, wide, reinterpret_cast<__half *>(stage), bias);
            }
        }
    }
    // ---------------- teardown: every thread arrives here, on success and after an expired wait
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

}  // namespace gemm

// ---------------------------------------------------------------- host side
// The tensor-core path needs whole 16-byte vectors for the copy engine: K % 64 == 0 (packed
// rows and TMA strides) and 16-byte aligned weight and activation pointers.
bool ternary_gemm_supported(const void *w, const void *q_perm, int64_t M, int64_t N, int64_t K)
{
    return (K % 64 == 0) && aligned16(w) && aligned16(q_perm) && M > 0 && M < (1ll << 31) && N < (1ll << 31) &&
           K < (1ll << 31);
}

template <int BT>
static int launch_gemm(const void *q_perm, gemm::Params &p, cudaStream_t st)
{
    using C = gemm::Cfg<BT>;
    static std::atomic<size_t> reserved[kMaxDevices];
    if (reserve_smem(gemm::ternary_gemm_kernel<BT>, reserved, (size_t)C::SMEM) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "ternary_gemm_kernel: cannot reserve %d bytes of shared memory: %s", C::SMEM,
                    cudaGetErrorString(cudaGetLastError()));
    CUtensorMap tmap_x, tmap_w;
    int rc = sm100::make_map_2d(&tmap_x, q_perm, (uint64_t)p.K, (uint64_t)p.M, gemm::BK, BT, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = sm100::make_map_2d(&tmap_w, p.w, (uint64_t)(p.K / 4), (uint64_t)p.N, C::PK_ROW, gemm::BW,
                            C::KS == 2 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    if (rc) return rc;
    p.tiles_t = (int)((p.M + BT - 1) / BT);
    p.tiles_w = (int)((p.N + gemm::BW - 1) / gemm::BW);
    const int tiles = p.tiles_t * p.tiles_w;
    const int grid = tiles < sm100::sm_count() ? tiles : sm100::sm_count();
    cudaError_t e = launch_kernel(gemm::ternary_gemm_kernel<BT>, dim3(grid), dim3(gemm::THREADS), (size_t)C::SMEM, st, tmap_x, tmap_w, p);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "ternary_gemm_kernel: %s", cudaGetErrorString(e));
    return check_launch("ternary_gemm_kernel");
}

static int gemm_one_launch(const uint8_t *w, const int8_t *q_perm, const float *scale, const int32_t *rowsum, int64_t M,
                           int64_t N, int64_t K, float weight_scale, void *y, int y_dtype, int32_t *acc_out,
                           const float *bias, const float *residual, const OutSpec *os, int64_t row_off, cudaStream_t st)
{
    gemm::Params p{w, scale, rowsum, y, acc_out, bias, residual, M, N, K, y_dtype, weight_scale, 0, 0, N, 0, {}, 0};
    const int es = y_dtype == NSLQ_DTYPE_F32 ? 4 : 2;
    if (os) {
        p.ldy = os->ldy;
        p.npeer = os->npeer;
        for (int i = 0; i < os->npeer; ++i) p.y_peer[i] = (char *)os->peer[i] + row_off * os->ldy * es;
    }
    // Whole rows of a tile as 16-byte vectors, for results that also go to other GPUs (a local-only result is
    // stored directly: measured, the staging costs the single-GPU prefill GEMM 6 us of 47).  Every row start of y
    // and of its copies must be 16-byte aligned.
    p.wide = p.npeer > 0 && aligned16(p.y) && (p.ldy * es) % 16 == 0;
    for (int i = 0; i < p.npeer; ++i) p.wide = p.wide && aligned16(p.y_peer[i]);
    // Token-tile width: the one that wastes fewer SM-rounds on this shape (ties go to the wider
    // tile, which moves fewer shared-memory bytes per MAC).
    const int sms = sm100::sm_count();
    auto rounds_cost = [&](int bt) {
        const int64_t tiles = ((M + bt - 1) / bt) * ((N + gemm::BW - 1) / gemm::BW);
        const int64_t rounds = (tiles + sms - 1) / sms;
        return (double)rounds * bt;
    };
    // Up to 64 rows: a 64-token tile halves the MMA work of every step (one tile per CTA, the launch is
    // a latency chain of prologue, K / 256 steps and epilogue).
    if (M <= 64) return launch_gemm<64>(q_perm, p, st);
    if (rounds_cost(192) <= rounds_cost(128)) return launch_gemm<192>(q_perm, p, st);
    return launch_gemm<128>(q_perm, p, st);
}

// One launch takes at most GEMM_MAX_ROWS token rows; longer batches run as several launches on the
// same stream.  Reason: at M = 32768 (118 tiles per CTA, about a millisecond per launch) roughly one
// launch in fifteen ended in cudaErrorLaunchFailure on this machine, also in isolation with identical
// inputs and with every wait bounded; reading the kernel has not shown a cause, and launches of
// 4096 rows (a hundred microseconds) have run by the thousand, inside the same 26-layer prefill that
// failed, without one.  The working guess is that a persistent kernel holding tensor memory does
// not survive being time-sliced against another tenant of the GPU; short launches sidestep it.
constexpr int64_t GEMM_MAX_ROWS = 4096;

int ternary_gemm_dispatch(const uint8_t *w, const int8_t *q_perm, const float *scale, const int32_t *rowsum, int64_t M,
                          int64_t N, int64_t K, float weight_scale, void *y, int y_dtype, int32_t *acc_out,
                          const float *bias, const float *residual, const OutSpec *os, cudaStream_t st)
{
    const int es = y_dtype == NSLQ_DTYPE_F32 ? 4 : 2;
    const int64_t ldy = os ? os->ldy : N;
    for (int64_t m0 = 0; m0 < M; m0 += GEMM_MAX_ROWS) {
        const int64_t mc = (M - m0) < GEMM_MAX_ROWS ? (M - m0) : GEMM_MAX_ROWS;
        int rc = gemm_one_launch(w, q_perm + m0 * K, scale + m0, rowsum + m0, mc, N, K, weight_scale,
                                 (char *)y + m0 * ldy * es, y_dtype, acc_out ? acc_out + m0 * N : nullptr, bias,
                                 residual ? residual + m0 * N : nullptr, os, m0, st);
        if (rc) return rc;
    }
    return NSLQ_OK;
}

// The status word of this translation unit's kernels (see sm100::read_wait_status).
int ternary_gemm_status(int *out) { return sm100::read_wait_status(out); }

}  // namespace nslq
