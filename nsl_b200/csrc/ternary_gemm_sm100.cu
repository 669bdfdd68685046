// Stage 3: BitLinear prefill GEMM on the 5th-generation tensor cores (sm_100a).
//
//   acc[m,n] = sum_k q[m,k] * W[n,k]        int8 x ternary, exact int32
//
// Persistent, warp-specialised kernel, one CTA per SM, 128 x BN output tiles:
//
//   warp 0      TMA producer: per stage, two cp.async.bulk.tensor copies (2-D, no
//               multicast): the int8 activation tile (128 rows x 128 k,
//               SWIZZLE_128B) and the still-packed 2-bit weight tile (BN rows x 32
//               bytes) land in a ring of shared-memory stages; out-of-range rows
//               and the K tail are zero-filled by the copy engine.
//   warps 8-15  unpack (two groups of four warps taking alternate stages, so one
//               group's latency hides behind the other's): read the packed tile
//               from shared memory, expand it in
//               registers with (w >> s) & 0x03030303 -- one 32-bit word of packed
//               bytes becomes one 16-byte group of u8 codes {0,1,2} -- and write it
//               into the same stage in the K-major 128-byte-swizzled layout the
//               tensor core reads, then publish it with fence.proxy.async +
//               mbarrier arrive.
//               The activations are stored in the matching order (position 4i+j of
//               every 16 holds k = 4j+i), so nothing is permuted here.
//   warp 1      MMA issuer: one thread issues tcgen05.mma.kind::i8 (M=128, N=BN,
//               K=32; A = s8 activations, B = u8 codes, D = s32 in TMEM) four times
//               per stage and releases the stage with tcgen05.commit.
//   warps 4-7   epilogue: tcgen05.ld the accumulator (double-buffered in TMEM, so
//               the next tile's MMAs run meanwhile), subtract the token's row sum
//               (code = trit + 1), apply ((scale/127)*acc)*weight_scale with
//               separately rounded steps, transpose through a padded shared-memory
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
constexpr int THREADS = 512;            // 16 warps: 0 TMA, 1 MMA, 4-7 epilogue, 8-15 unpack
constexpr int A_BYTES = BM * BK;         // 16 KiB
constexpr int STAGE_PAD = 36;            // floats per staged row (32 + 4: conflict-free 16-byte accesses)
constexpr int STAGING_BYTES = 4 * 32 * STAGE_PAD * 4;

template <int BN> struct Cfg {
    static constexpr int B_BYTES = BN * BK;          // unpacked u8 codes
    static constexpr int P_BYTES = BN * (BK / 4);    // packed 2-bit tile as it sits in global memory
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + P_BYTES;   // multiple of 1024
    static constexpr int STAGES = (BN == 256) ? 3 : 4;
    static constexpr int SMEM = STAGES * STAGE_BYTES + STAGING_BYTES + 256 + 1024;  // + barriers + alignment slack
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
    const uint32_t staging = base + C::STAGES * C::STAGE_BYTES;
    float *staging_ptr = reinterpret_cast<float *>(base_ptr + C::STAGES * C::STAGE_BYTES);
    const uint32_t bars = staging + STAGING_BYTES;
    // barrier map (8 bytes each): raw[s] (TMA bytes landed), full[s] (codes unpacked), empty[s]
    // (MMAs of the stage retired), acc_full[2], acc_empty[2]; then the TMEM slot
    auto raw_bar = [&](int s) { return bars + 8u * s; };
    auto full_bar = [&](int s) { return bars + 8u * (C::STAGES + s); };
    auto empty_bar = [&](int s) { return bars + 8u * (2 * C::STAGES + s); };
    auto accf_bar = [&](int b) { return bars + 8u * (3 * C::STAGES + b); };
    auto acce_bar = [&](int b) { return bars + 8u * (3 * C::STAGES + 2 + b); };
    const uint32_t slot = bars + 8u * (3 * C::STAGES + 4);
    volatile uint32_t *slot_ptr = reinterpret_cast<volatile uint32_t *>(base_ptr + C::STAGES * C::STAGE_BYTES + STAGING_BYTES + 8 * (3 * C::STAGES + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (int)((p.K + BK - 1) / BK);
    const int ntiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(raw_bar(s), 1); mbar_init(full_bar(s), 128); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), 128); }
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
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const int m0 = (tile % p.tiles_m) * BM, n0 = (tile / p.tiles_m) * BN;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % C::STAGES;
                    const uint32_t ph = (it / C::STAGES) & 1u;
                    if (!(ok = mbar_wait(empty_bar(s), ph ^ 1u, 0x101))) break;
                    const uint32_t st = base + s * C::STAGE_BYTES;
                    mbar_arrive_expect_tx(raw_bar(s), A_BYTES + C::P_BYTES);
                    tma_load_2d(st, &tmap_a, kb * BK, m0, raw_bar(s));
                    tma_load_2d(st + A_BYTES + C::B_BYTES, &tmap_w, kb * (BK / 4), n0, raw_bar(s));
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0) {
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++t) {
                const uint32_t buf = t & 1u, aph = (t >> 1) & 1u;
                if (!(ok = mbar_wait(acce_bar(buf), aph ^ 1u, 0x201))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * 256u;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % C::STAGES;
                    const uint32_t ph = (it / C::STAGES) & 1u;
                    if (!(ok = mbar_wait(raw_bar(s), ph, 0x202))) break;    // activation tile landed
                    if (!(ok = mbar_wait(full_bar(s), ph, 0x203))) break;   // weight codes unpacked
                    tc_fence_after();
                    const uint32_t a_addr = base + s * C::STAGE_BYTES;
                    const uint64_t adesc = smem_desc(a_addr), bdesc = smem_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4)   // 32 bytes of K per MMA: descriptor start + 2 (16-byte units)
                        umma_i8(d_tmem, adesc + 2u * k4, bdesc + 2u * k4, C::IDESC, (kb | k4) != 0);
                    umma_commit(empty_bar(s));
                }
                if (ok) umma_commit(accf_bar(buf));
            }
        }
    } else if (warp >= 8) {
        // ---------------- unpack warps (packed tile -> u8 codes, swizzled K-major)
        constexpr int PER = BN * 2 / 128;            // 16-byte pieces of the packed tile per thread per stage
        const int u = threadIdx.x & 127;
        const int group = (warp - 8) >> 2;           // group 0 takes even pipeline iterations, group 1 odd
        bool ok = true;
        const int total_it = ((ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x) * nkb;
        for (int it = group; it < total_it && ok; it += 2) {
            {
                const int s = it % C::STAGES;
                const uint32_t ph = (it / C::STAGES) & 1u;
                // raw[s] completes only after the producer saw empty[s], so the codes
                // buffer of this stage is free to overwrite once the packed tile is here.
                if (!(ok = mbar_wait(raw_bar(s), ph, 0x301))) break;
                uint8_t *bst = base_ptr + s * C::STAGE_BYTES + A_BYTES;
                const uint4 *pk = reinterpret_cast<const uint4 *>(bst + C::B_BYTES);
                uint4 cur[PER];
#pragma unroll
                for (int i = 0; i < PER; ++i) cur[i] = pk[i * 128 + u];
#pragma unroll
                for (int i = 0; i < PER; ++i) {
                    const int idx = i * 128 + u, row = idx >> 1, half = idx & 1;
                    const uint32_t ww[4] = {cur[i].x, cur[i].y, cur[i].z, cur[i].w};
                    uint8_t *rowp = bst + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t w = ww[j];
                        uint4 v;
                        v.x = (w >> 6) & 0x03030303u; v.y = (w >> 4) & 0x03030303u;
                        v.z = (w >> 2) & 0x03030303u; v.w = w & 0x03030303u;
                        const int c = half * 4 + j;
                        *reinterpret_cast<uint4 *>(rowp + ((c ^ (row & 7)) << 4)) = v;
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(full_bar(s));
            }
        }
    } else if (warp >= 4) {
        // ---------------- epilogue warps (TMEM -> registers -> shared patch -> global)
        const int q = warp & 3;                       // TMEM lane quadrant of this warp
        float *patch = staging_ptr + q * 32 * STAGE_PAD;
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
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(taddr + c * 32, r);
                if (c == BN / 32 - 1) {              // last read of this accumulator: hand it back
                    tc_fence_before();
                    mbar_arrive(acce_bar(buf));
                }
                if (n0 + c * 32 >= p.N) continue;    // warp-uniform
                const int64_t ncol = n0 + c * 32 + (lane & 7) * 4;
                if (p.acc_out) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        int4 v = make_int4((int)r[4 * j] - rsum, (int)r[4 * j + 1] - rsum, (int)r[4 * j + 2] - rsum, (int)r[4 * j + 3] - rsum);
                        *reinterpret_cast<int4 *>(patch + lane * STAGE_PAD + 4 * j) = v;
                    }
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rl = 4 * i + (lane >> 3);
                        const int64_t m = m0 + q * 32 + rl;
                        const int4 v = *reinterpret_cast<const int4 *>(patch + rl * STAGE_PAD + (lane & 7) * 4);
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
                    *reinterpret_cast<float4 *>(patch + lane * STAGE_PAD + 4 * j) = v;
                }
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int rl = 4 * i + (lane >> 3);
                    const int64_t m = m0 + q * 32 + rl;
                    float4 v = *reinterpret_cast<const float4 *>(patch + rl * STAGE_PAD + (lane & 7) * 4);
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
