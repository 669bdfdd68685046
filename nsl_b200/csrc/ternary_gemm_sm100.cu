// Stage 3: BitLinear prefill GEMM on the 5th-generation tensor cores (sm_100a).
//
//   acc[m,n] = sum_k q[m,k] * W[n,k]        int8 x ternary, exact int32
//
// Persistent, warp-specialised kernel, one CTA per SM, 128 x BN output tiles:
//
//   warp 0      TMA producer: per k-block, two cp.async.bulk.tensor copies (2-D, no
//               multicast): the int8 activation tile (128 rows x 128 k,
//               SWIZZLE_128B) and the still-packed 2-bit weight tile (BN rows x 32
//               bytes) land in a deep ring of "copy" stages (22-24 KiB each);
//               out-of-range rows and the K tail are zero-filled by the copy engine.
//   warps 8-15  unpack (two groups of four warps taking alternate k-blocks, so one
//               group's latency hides behind the other's): read the packed tile
//               from shared memory, expand it in
//               registers with (w >> s) & 0x03030303 -- one 32-bit word of packed
//               bytes becomes one 16-byte group of u8 codes {0,1,2} -- and write it
//               into a second, shorter ring of "codes" stages in the K-major
//               128-byte-swizzled layout the tensor core reads, then publish it with
//               fence.proxy.async + mbarrier arrive.  Two rings because the copies'
//               latency (long) and the unpack-to-MMA latency (short) want different
//               depths, and the packed tile is a quarter the size of its codes.
//               The activations are stored in the matching order (position 4i+j of
//               every 16 holds k = 4j+i), so nothing is permuted here.
//   warp 1      MMA issuer: the warp runs the loop in uniform control flow and one
//               elected lane issues tcgen05.mma.kind::i8 (M=128, N=BN, K=32; A = s8
//               activations, B = u8 codes, D = s32 in TMEM) four times per k-block
//               and releases both stages with tcgen05.commit.  It waits only for the
//               codes: they are published after the copy stage was seen complete, so
//               the activation tile of the same copy stage has landed too.
//   warps 4-7,  epilogue, two warps per TMEM lane quadrant, each taking half of the
//   16-19       tile's columns: tcgen05.ld the accumulator (double-buffered in TMEM,
//               so the next tile's MMAs run meanwhile), subtract the token's row sum
//               (code = trit + 1), apply ((scale/127)*acc)*weight_scale with
//               separately rounded steps, transpose through a swizzled shared-memory
//               patch and store 128-byte row segments.
//
// Every mbarrier wait is bounded in time; on expiry the kernel records a status
// word (read with nslq_device_status) and falls through to the common teardown,
// which frees its TMEM.  No spin is unbounded.
#include "sm100_common.cuh"

namespace nslq {

namespace gemm {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 128;                  // bytes of int8 along K per stage = one 128B swizzle row
constexpr int THREADS = 640;            // 20 warps: 0 TMA, 1 MMA, 4-7 and 16-19 epilogue, 8-15 unpack
constexpr int A_BYTES = BM * BK;         // 16 KiB
constexpr int STAGE_PAD = 32;            // floats per staged row: one 128-byte line, 16-byte chunks XOR-swizzled by row
constexpr int STAGING_BYTES = 8 * 32 * STAGE_PAD * 4;   // one 32 x 32 patch per epilogue warp

template <int BN> struct Cfg {
    static constexpr int B_BYTES = BN * BK;          // unpacked u8 codes
    static constexpr int P_BYTES = BN * (BK / 4);    // packed 2-bit tile as it sits in global memory
    static constexpr int T_BYTES = A_BYTES + P_BYTES;                 // one copy stage, multiple of 1024
    static constexpr int TS = (BN == 256) ? 4 : 5;                    // copy stages in flight
    static constexpr int BS = 3;                                      // codes stages in flight
    static constexpr int RING_BYTES = TS * T_BYTES + BS * B_BYTES;
    static constexpr int SMEM = RING_BYTES + STAGING_BYTES + 256 + 1024;  // + barriers + alignment slack
    static_assert(SMEM <= 232448, "over the 227 KiB a CTA may use");
    static constexpr uint32_t IDESC = (2u << 4)        // D format: s32
                                      | (1u << 7)      // A format: signed 8-bit
                                      | (0u << 10)     // B format: unsigned 8-bit
                                      | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
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
    int tiles_m, tiles_n;
};

// ---------------------------------------------------------------- kernel
template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
ternary_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w, const Params p)
{
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                  // 1024-byte aligned (swizzle atom)
    uint8_t *base_ptr = smem_raw + (base - raw);
    const uint32_t codes = base + C::TS * C::T_BYTES;               // codes ring follows the copy ring
    uint8_t *codes_ptr = base_ptr + C::TS * C::T_BYTES;
    const uint32_t staging = base + C::RING_BYTES;
    float *staging_ptr = reinterpret_cast<float *>(base_ptr + C::RING_BYTES);
    const uint32_t bars = staging + STAGING_BYTES;
    // barrier map (8 bytes each): raw[t] (copy stage landed), tfree[t] (copy stage consumed: four
    // unpack warps + the MMAs' commit), bfull[b] (codes written), bfree[b] (MMAs of the codes stage
    // retired), acc_full[2], acc_empty[2]; then the TMEM slot
    constexpr int NBAR = 2 * C::TS + 2 * C::BS + 4;
    static_assert(NBAR * 8 + 8 <= 256, "barrier area");
    auto raw_bar = [&](int t) { return bars + 8u * t; };
    auto tfree_bar = [&](int t) { return bars + 8u * (C::TS + t); };
    auto bfull_bar = [&](int b) { return bars + 8u * (2 * C::TS + b); };
    auto bfree_bar = [&](int b) { return bars + 8u * (2 * C::TS + C::BS + b); };
    auto accf_bar = [&](int b) { return bars + 8u * (2 * C::TS + 2 * C::BS + b); };
    auto acce_bar = [&](int b) { return bars + 8u * (2 * C::TS + 2 * C::BS + 2 + b); };
    const uint32_t slot = bars + 8u * NBAR;
    volatile uint32_t *slot_ptr = reinterpret_cast<volatile uint32_t *>(base_ptr + C::RING_BYTES + STAGING_BYTES + 8 * NBAR);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (int)((p.K + BK - 1) / BK);
    const int ntiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int t = 0; t < C::TS; ++t) { mbar_init(raw_bar(t), 1); mbar_init(tfree_bar(t), 5); }
        for (int b = 0; b < C::BS; ++b) { mbar_init(bfull_bar(b), 4); mbar_init(bfree_bar(b), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), 256); }
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

    if (warp == 0) {
        // ---------------- TMA producer (activation tile + packed weight tile)
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const int m0 = (tile % p.tiles_m) * BM, n0 = (tile / p.tiles_m) * BN;
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!(ok = mbar_wait(tfree_bar(s), ph ^ 1u, 0x101))) break;
                    const uint32_t st = base + s * C::T_BYTES;
                    mbar_arrive_expect_tx(raw_bar(s), A_BYTES + C::P_BYTES);
                    tma_load_2d(st, &tmap_a, kb * BK, m0, raw_bar(s));
                    tma_load_2d(st + A_BYTES, &tmap_w, kb * (BK / 4), n0, raw_bar(s));
                    if (++s == C::TS) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (whole warp in the loop, one elected lane issues)
        const bool leader = elect_one();
        int s = 0, b = 0;
        uint32_t bph = 0, t = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++t) {
            const uint32_t buf = t & 1u, aph = (t >> 1) & 1u;
            if (!(ok = mbar_wait(acce_bar(buf), aph ^ 1u, 0x201))) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * 256u;
            for (int kb = 0; kb < nkb; ++kb) {
                if (!(ok = mbar_wait(bfull_bar(b), bph, 0x203))) break;    // codes unpacked (and the copy stage landed)
                tc_fence_after();
                if (leader) {
                    const uint64_t adesc = smem_desc(base + s * C::T_BYTES), bdesc = smem_desc(codes + b * C::B_BYTES);
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4)   // 32 bytes of K per MMA: descriptor start + 2 (16-byte units)
                        umma_i8(d_tmem, adesc + 2u * k4, bdesc + 2u * k4, C::IDESC, (kb | k4) != 0);
                    umma_commit(tfree_bar(s));
                    umma_commit(bfree_bar(b));
                }
                if (++s == C::TS) s = 0;
                if (++b == C::BS) { b = 0; bph ^= 1u; }
            }
            if (ok && leader) umma_commit(accf_bar(buf));
        }
    } else if (warp >= 8 && warp < 16) {
        // ---------------- unpack warps (packed tile -> u8 codes, swizzled K-major)
        constexpr int WPT = BN * 8 / 128;            // packed 32-bit words per thread per stage
        const int u = threadIdx.x & 127;
        const int group = (warp - 8) >> 2;           // group 0 takes even pipeline iterations, group 1 odd
        bool ok = true;
        const int total_it = ((ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x) * nkb;
        int s = group % C::TS, b = group % C::BS;            // ring positions of iteration `it`, stepped by two
        uint32_t sph = 0, bph = 0;
        for (int it = group; it < total_it && ok; it += 2) {
            if (!(ok = mbar_wait(raw_bar(s), sph, 0x301))) break;                            // packed tile landed
            const uint32_t *pk = reinterpret_cast<const uint32_t *>(base_ptr + s * C::T_BYTES + A_BYTES);
            // One 32-bit word (16 trits) per thread and step: 8 consecutive lanes fill the eight
            // 16-byte chunks of one 128-byte row, so every quarter-warp store is one full line.
            uint32_t cur[WPT];
#pragma unroll
            for (int i = 0; i < WPT; ++i) cur[i] = pk[i * 128 + u];
            if (!(ok = mbar_wait(bfree_bar(b), bph ^ 1u, 0x302))) break;                     // codes stage reusable
            uint8_t *bst = codes_ptr + b * C::B_BYTES;
#pragma unroll
            for (int i = 0; i < WPT; ++i) {
                const int wi = i * 128 + u, row = wi >> 3, c = wi & 7;
                const uint32_t w = cur[i];
                uint4 v;
                v.x = (w >> 6) & 0x03030303u; v.y = (w >> 4) & 0x03030303u;
                v.z = (w >> 2) & 0x03030303u; v.w = w & 0x03030303u;
                *reinterpret_cast<uint4 *>(bst + (row >> 3) * 1024 + (row & 7) * 128 + ((c ^ (row & 7)) << 4)) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bfull_bar(b));
                mbar_arrive(tfree_bar(s));
            }
            if ((s += 2) >= C::TS) { s -= C::TS; sph ^= 1u; }
            if ((b += 2) >= C::BS) { b -= C::BS; bph ^= 1u; }
        }
    } else if (warp >= 4) {
        // ---------------- epilogue warps (TMEM -> registers -> shared patch -> global)
        const int q = warp & 3;                       // TMEM lane quadrant of this warp
        const int half = warp >> 4;                   // warps 4-7: first half of the columns, 16-19: second
        constexpr int NC = BN / 32, C_HALF = NC / 2;
        const int c_begin = half * C_HALF, c_end = c_begin + C_HALF;
        float *patch = staging_ptr + (half * 4 + q) * 32 * STAGE_PAD;
        uint32_t t = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++t) {
            const uint32_t buf = t & 1u, aph = (t >> 1) & 1u;
            const int64_t m0 = (int64_t)(tile % p.tiles_m) * BM, n0 = (int64_t)(tile / p.tiles_m) * BN;
            const int64_t my_m = m0 + q * 32 + lane;
            const bool m_ok = my_m < p.M;
            const float s127 = m_ok ? __fdiv_rn(p.scale[my_m], 127.0f) : 0.0f;
            const int rsum = m_ok ? p.rowsum[my_m] : 0;
            if (!(ok = mbar_wait(accf_bar(buf), aph, 0x401))) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256u;
#pragma unroll 1
            for (int c = c_begin; c < c_end; ++c) {
                uint32_t r[32];
                tmem_ld32(taddr + c * 32, r);
                if (c == c_end - 1) {                // this thread's last read of the accumulator: hand it back
                    tc_fence_before();
                    mbar_arrive(acce_bar(buf));
                }
                if (n0 + c * 32 >= p.N) continue;    // warp-uniform
                const int64_t ncol = n0 + c * 32 + (lane & 7) * 4;
                if (p.acc_out) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        int4 v = make_int4((int)r[4 * j] - rsum, (int)r[4 * j + 1] - rsum, (int)r[4 * j + 2] - rsum, (int)r[4 * j + 3] - rsum);
                        *reinterpret_cast<int4 *>(patch + lane * STAGE_PAD + 4 * (j ^ (lane & 7))) = v;
                    }
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rl = 4 * i + (lane >> 3);
                        const int64_t m = m0 + q * 32 + rl;
                        const int4 v = *reinterpret_cast<const int4 *>(patch + rl * STAGE_PAD + 4 * ((lane & 7) ^ (rl & 7)));
                        if (m < p.M && ncol < p.N) *reinterpret_cast<int4 *>(p.acc_out + m * p.N + ncol) = v;
                    }
                    __syncwarp();
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float4 v;
                    v.x = __fmul_rn(__fmul_rn(s127, __int2float_rn((int)r[4 * j + 0] - rsum)), p.weight_scale);
                    v.y = __fmul_rn(__fmul_rn(s127, __int2float_rn((int)r[4 * j + 1] - rsum)), p.weight_scale);
                    v.z = __fmul_rn(__fmul_rn(s127, __int2float_rn((int)r[4 * j + 2] - rsum)), p.weight_scale);
                    v.w = __fmul_rn(__fmul_rn(s127, __int2float_rn((int)r[4 * j + 3] - rsum)), p.weight_scale);
                    *reinterpret_cast<float4 *>(patch + lane * STAGE_PAD + 4 * (j ^ (lane & 7))) = v;
                }
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int rl = 4 * i + (lane >> 3);
                    const int64_t m = m0 + q * 32 + rl;
                    float4 v = *reinterpret_cast<const float4 *>(patch + rl * STAGE_PAD + 4 * ((lane & 7) ^ (rl & 7)));
                    if (m < p.M && ncol < p.N) {
                        const int64_t o = m * p.N + ncol;
                        if (p.bias) {
                            const float4 b = *reinterpret_cast<const float4 *>(p.bias + ncol);
                            v.x = __fadd_rn(v.x, b.x); v.y = __fadd_rn(v.y, b.y); v.z = __fadd_rn(v.z, b.z); v.w = __fadd_rn(v.w, b.w);
                        }
                        if (p.residual) {
                            const float4 b = *reinterpret_cast<const float4 *>(p.residual + o);
                            v.x = __fadd_rn(v.x, b.x); v.y = __fadd_rn(v.y, b.y); v.z = __fadd_rn(v.z, b.z); v.w = __fadd_rn(v.w, b.w);
                        }
                        if (p.y_dtype == NSLQ_DTYPE_F32) {
                            *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.y) + o) = v;
                        } else if (p.y_dtype == NSLQ_DTYPE_BF16) {
                            __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                            uint2 pk = make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
                            *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(p.y) + o) = pk;
                        } else {
                            __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
                            uint2 pk = make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
                            *reinterpret_cast<uint2 *>(reinterpret_cast<__half *>(p.y) + o) = pk;
                        }
                    }
                }
                __syncwarp();
            }
        }
    }
    // ---------------- teardown: every thread arrives here, on success and after an expired wait
    pdl_launch_dependents();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

}  // namespace gemm

// ---------------------------------------------------------------- host side
// The tensor-core path needs whole 16-byte vectors everywhere: K % 64 == 0 (packed
// rows and TMA strides), N % 4 == 0 (vector stores) and aligned base pointers.
bool ternary_gemm_supported(const void *w, const void *q_perm, int64_t M, int64_t N, int64_t K)
{
    return (K % 64 == 0) && (N % 4 == 0) && aligned16(w) && aligned16(q_perm) && M > 0 && M < (1ll << 31) &&
           N < (1ll << 31) && K < (1ll << 31);
}

template <int BN>
static int launch_gemm(const void *q_perm, gemm::Params &p, cudaStream_t st)
{
    using C = gemm::Cfg<BN>;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemm::ternary_gemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess)
            return fail(NSLQ_ERR_CUDA, "ternary_gemm_kernel: cannot reserve %d bytes of shared memory: %s", C::SMEM,
                        cudaGetErrorString(cudaGetLastError()));
        attr_set = true;
    }
    CUtensorMap tmap_a, tmap_w;
    int rc = sm100::make_map_2d(&tmap_a, q_perm, (uint64_t)p.K, (uint64_t)p.M, gemm::BK, gemm::BM, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = sm100::make_map_2d(&tmap_w, p.w, (uint64_t)(p.K / 4), (uint64_t)p.N, gemm::BK / 4, BN, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    p.tiles_m = (int)((p.M + gemm::BM - 1) / gemm::BM);
    p.tiles_n = (int)((p.N + BN - 1) / BN);
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < sm100::sm_count() ? tiles : sm100::sm_count();
    gemm::ternary_gemm_kernel<BN><<<grid, gemm::THREADS, C::SMEM, st>>>(tmap_a, tmap_w, p);
    return check_launch("ternary_gemm_kernel");
}

int ternary_gemm_dispatch(const uint8_t *w, const int8_t *q_perm, const float *scale, const int32_t *rowsum, int64_t M,
                          int64_t N, int64_t K, float weight_scale, void *y, int y_dtype, int32_t *acc_out,
                          const float *bias, const float *residual, cudaStream_t st)
{
    if ((acc_out && !aligned16(acc_out)) || !aligned16(y) || (bias && !aligned16(bias)) || (residual && !aligned16(residual)))
        return fail(NSLQ_ERR_ARG, "BitLinear GEMM: y, acc_out, bias and residual must be 16-byte aligned");
    gemm::Params p{w, scale, rowsum, y, acc_out, bias, residual, M, N, K, y_dtype, weight_scale, 0, 0};
    // Tile width: the one that wastes fewer SM-rounds on this shape.
    const int sms = sm100::sm_count();
    auto rounds_cost = [&](int bn) {
        const int64_t tiles = ((M + gemm::BM - 1) / gemm::BM) * ((N + bn - 1) / bn);
        const int64_t rounds = (tiles + sms - 1) / sms;
        return (double)rounds * bn;
    };
    if (rounds_cost(192) < rounds_cost(256)) return launch_gemm<192>(q_perm, p, st);
    return launch_gemm<256>(q_perm, p, st);
}

// The status word of this translation unit's kernels (see sm100::read_wait_status).
int ternary_gemm_status(int *out) { return sm100::read_wait_status(out); }

}  // namespace nslq
