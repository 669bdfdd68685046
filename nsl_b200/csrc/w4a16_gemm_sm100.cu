// Stage 3 for W4A16: prefill GEMM on the 5th-generation tensor cores (sm_100a).
//
//   y[m,n] = sum_k x[m,k] * (q[n,k] - zp[n,k/g]) * scale[n,k/g]      bf16 x bf16 -> fp32
//
// Same persistent, warp-specialised skeleton as the ternary GEMM (one CTA per SM,
// 128 x BN output tiles, TMEM double-buffered accumulators, every wait bounded):
//
//   warp 0      TMA producer: the bf16 activation tile (128 rows x 64 k, SWIZZLE_128B)
//               and the still-packed uint4 weight tile (BN rows x 32 bytes) per stage.
//   warps 8-15  dequantise: a 32-bit word holds 8 codes; ((w >> 4i) & 0x000F000F) |
//               0x43004300 is the bf16 pair (128+q[i], 128+q[i+4]); two byte-permutes
//               put the pairs back in k order, one bf16x2 subtract removes (128+zp)
//               exactly and one bf16x2 multiply applies the group scale, so each
//               weight is rounded once: bf16((q-zp)*scale).  The 16-byte groups are
//               written in the K-major 128-byte-swizzled layout the tensor core reads.
//   warp 1      MMA issuer: tcgen05.mma.kind::f16 (M=128, N=BN, K=16), four per stage.
//   warps 4-7   epilogue: tcgen05.ld, convert, transpose through a padded shared-memory
//               patch, 128-byte row-segment stores.
//
// Requires integer zero points (the QuantizedTensor / benchmark form); AWQ float zeros
// are served by the streaming kernel instead.  Scales are applied in bf16.
#include "sm100_common.cuh"

namespace nslq {
namespace w4gemm {

using namespace sm100;

constexpr int BM = 128;
constexpr int BKB = 128;                 // bytes of bf16 along K per stage (64 elements)
constexpr int BKE = 64;                  // elements of K per stage
constexpr int THREADS = 512;             // 16 warps: 0 TMA, 1 MMA, 4-7 epilogue, 8-15 dequantise
constexpr int A_BYTES = BM * BKB;
constexpr int STAGE_PAD = 36;
constexpr int STAGING_BYTES = 4 * 32 * STAGE_PAD * 4;

template <int BN> struct Cfg {
    static constexpr int B_BYTES = BN * BKB;         // dequantised bf16 tile
    static constexpr int P_BYTES = BN * (BKE / 2);   // packed codes: 32 bytes per row
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + P_BYTES;
    static constexpr int STAGES = (BN == 256) ? 3 : 4;
    static constexpr int SMEM = STAGES * STAGE_BYTES + STAGING_BYTES + 256 + 1024;
    static constexpr uint32_t IDESC = (1u << 4)        // D format: f32
                                      | (1u << 7)      // A format: bf16
                                      | (1u << 10)     // B format: bf16
                                      | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
};

struct Params {
    const float *scale;   // [N][G]
    const float *zc;      // [N][G] integer-valued
    void *y;              // [M][N]
    int64_t M, N, K;
    int G, gs, y_dtype;
    int tiles_m, tiles_n;
};

static __device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

static __device__ __forceinline__ uint32_t bf162_sub_mul(uint32_t v, uint32_t c, uint32_t s)
{
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162 *>(&v);
    const __nv_bfloat162 cc = *reinterpret_cast<const __nv_bfloat162 *>(&c);
    const __nv_bfloat162 ss = *reinterpret_cast<const __nv_bfloat162 *>(&s);
    a = __hmul2(__hsub2(a, cc), ss);      // (128+q) - (128+zp) is exact; one rounding in the multiply
    return *reinterpret_cast<uint32_t *>(&a);
}

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
w4a16_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w, const Params p)
{
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw);
    const uint32_t staging = base + C::STAGES * C::STAGE_BYTES;
    float *staging_ptr = reinterpret_cast<float *>(base_ptr + C::STAGES * C::STAGE_BYTES);
    const uint32_t bars = staging + STAGING_BYTES;
    auto raw_bar = [&](int s) { return bars + 8u * s; };
    auto full_bar = [&](int s) { return bars + 8u * (C::STAGES + s); };
    auto empty_bar = [&](int s) { return bars + 8u * (2 * C::STAGES + s); };
    auto accf_bar = [&](int b) { return bars + 8u * (3 * C::STAGES + b); };
    auto acce_bar = [&](int b) { return bars + 8u * (3 * C::STAGES + 2 + b); };
    const uint32_t slot = bars + 8u * (3 * C::STAGES + 4);
    volatile uint32_t *slot_ptr = reinterpret_cast<volatile uint32_t *>(base_ptr + C::STAGES * C::STAGE_BYTES + STAGING_BYTES + 8 * (3 * C::STAGES + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (int)((p.K + BKE - 1) / BKE);
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

    pdl_wait();

    if (warp == 0) {
        // ---------------- TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const int m0 = (tile % p.tiles_m) * BM, n0 = (tile / p.tiles_m) * BN;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % C::STAGES;
                    const uint32_t ph = (it / C::STAGES) & 1u;
                    if (!(ok = mbar_wait(empty_bar(s), ph ^ 1u, 0x1101))) break;
                    const uint32_t st = base + s * C::STAGE_BYTES;
                    mbar_arrive_expect_tx(raw_bar(s), A_BYTES + C::P_BYTES);
                    tma_load_2d(st, &tmap_a, kb * BKB, m0, raw_bar(s));                           // x in bytes along K
                    tma_load_2d(st + A_BYTES + C::B_BYTES, &tmap_w, kb * (BKE / 2), n0, raw_bar(s));
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the whole warp runs the loop, one elected lane issues (MMAs
        // issue several times faster from a converged warp than from a lone diverged lane).  It
        // waits only for the dequantised weights: they are published after the copy stage was
        // seen complete, so the activation tile of the same stage has landed too.
        const bool leader = elect_one();
        uint32_t it = 0, t = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++t) {
            const uint32_t buf = t & 1u, aph = (t >> 1) & 1u;
            if (!(ok = mbar_wait_warp(acce_bar(buf), aph ^ 1u, 0x1201))) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * 256u;
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = it % C::STAGES;
                const uint32_t ph = (it / C::STAGES) & 1u;
                if (!(ok = mbar_wait_warp(full_bar(s), ph, 0x1203))) break;
                tc_fence_after();
                if (leader) {
                    const uint32_t a_addr = base + s * C::STAGE_BYTES;
                    const uint64_t adesc = smem_desc(a_addr), bdesc = smem_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4)   // 16 bf16 = 32 bytes of K per MMA
                        umma_f16(d_tmem, adesc + 2u * k4, bdesc + 2u * k4, C::IDESC, (kb | k4) != 0);
                    umma_commit(empty_bar(s));
                }
            }
            if (ok && leader) umma_commit(accf_bar(buf));
        }
    } else if (warp >= 8) {
        // ---------------- dequantise warps (two groups on alternate stages)
        constexpr int PER = BN * 2 / 128;
        const int u = threadIdx.x & 127;
        const int group = (warp - 8) >> 2;
        bool ok = true;
        const int my_tiles = (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
        const int total_it = my_tiles * nkb;
        for (int it = group; it < total_it && ok; it += 2) {
            const int tile = (int)blockIdx.x + (it / nkb) * (int)gridDim.x, kb = it % nkb;
            const int64_t n0 = (int64_t)(tile / p.tiles_m) * BN;
            const int grp = (kb * BKE) / p.gs;
            // group constants of this thread's rows: issued before the wait so they overlap it
            float sc[PER], zz[PER];
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int64_t n = n0 + ((i * 128 + u) >> 1);
                const bool v = n < p.N;
                sc[i] = v ? __ldg(p.scale + n * p.G + grp) : 0.0f;
                zz[i] = v ? __ldg(p.zc + n * p.G + grp) : 0.0f;
            }
            const int s = it % C::STAGES;
            const uint32_t ph = (it / C::STAGES) & 1u;
            if (!(ok = mbar_wait_warp(raw_bar(s), ph, 0x1301))) break;
            uint8_t *bst = base_ptr + s * C::STAGE_BYTES + A_BYTES;
            const uint4 *pk = reinterpret_cast<const uint4 *>(bst + C::B_BYTES);
            uint4 cur[PER];
#pragma unroll
            for (int i = 0; i < PER; ++i) cur[i] = pk[i * 128 + u];
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int idx = i * 128 + u, row = idx >> 1, half = idx & 1;
                const __nv_bfloat162 s2 = __float2bfloat162_rn(sc[i]);
                const __nv_bfloat162 c2 = __float2bfloat162_rn(128.0f + zz[i]);
                const uint32_t su = *reinterpret_cast<const uint32_t *>(&s2), cu = *reinterpret_cast<const uint32_t *>(&c2);
                const uint32_t ww[4] = {cur[i].x, cur[i].y, cur[i].z, cur[i].w};
                uint8_t *rowp = bst + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t w = ww[j];
                    const uint32_t r0 = (w & 0x000F000Fu) | 0x43004300u;            // (q0, q4) + 128
                    const uint32_t r1 = ((w >> 4) & 0x000F000Fu) | 0x43004300u;     // (q1, q5)
                    const uint32_t r2 = ((w >> 8) & 0x000F000Fu) | 0x43004300u;     // (q2, q6)
                    const uint32_t r3 = ((w >> 12) & 0x000F000Fu) | 0x43004300u;    // (q3, q7)
                    uint4 v;
                    v.x = bf162_sub_mul(__byte_perm(r0, r1, 0x5410), cu, su);       // (q0, q1)
                    v.y = bf162_sub_mul(__byte_perm(r2, r3, 0x5410), cu, su);       // (q2, q3)
                    v.z = bf162_sub_mul(__byte_perm(r0, r1, 0x7632), cu, su);       // (q4, q5)
                    v.w = bf162_sub_mul(__byte_perm(r2, r3, 0x7632), cu, su);       // (q6, q7)
                    const int c = half * 4 + j;
                    *reinterpret_cast<uint4 *>(rowp + ((c ^ (row & 7)) << 4)) = v;
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(full_bar(s));
        }
    } else if (warp >= 4) {
        // ---------------- epilogue warps
        const int q = warp & 3;
        float *patch = staging_ptr + q * 32 * STAGE_PAD;
        uint32_t t = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++t) {
            const uint32_t buf = t & 1u, aph = (t >> 1) & 1u;
            const int64_t m0 = (int64_t)(tile % p.tiles_m) * BM, n0 = (int64_t)(tile / p.tiles_m) * BN;
            const bool interior = (m0 + BM <= p.M) && (n0 + BN <= p.N);   // no bounds tests inside the tile
            if (!(ok = mbar_wait_warp(accf_bar(buf), aph, 0x1401))) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256u;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(taddr + c * 32, r);
                if (c == BN / 32 - 1) {
                    tc_fence_before();
                    mbar_arrive(acce_bar(buf));
                }
                if (n0 + c * 32 >= p.N) continue;
                const int64_t ncol = n0 + c * 32 + (lane & 7) * 4;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    *reinterpret_cast<uint4 *>(patch + lane * STAGE_PAD + 4 * j) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int rl = 4 * i + (lane >> 3);
                    const int64_t m = m0 + q * 32 + rl;
                    const float4 v = *reinterpret_cast<const float4 *>(patch + rl * STAGE_PAD + (lane & 7) * 4);
                    if (interior || (m < p.M && ncol < p.N)) {
                        const int64_t o = m * p.N + ncol;
                        if (p.y_dtype == NSLQ_DTYPE_F32) {
                            *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.y) + o) = v;
                        } else if (p.y_dtype == NSLQ_DTYPE_BF16) {
                            __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                            *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(p.y) + o) =
                                make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
                        } else {
                            __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
                            *reinterpret_cast<uint2 *>(reinterpret_cast<__half *>(p.y) + o) =
                                make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
                        }
                    }
                }
                __syncwarp();
            }
        }
    }
    // ---------------- teardown (reached on success and after an expired wait alike)
    pdl_launch_dependents();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

}  // namespace w4gemm

// ---------------------------------------------------------------- host side
// bf16 activations, integer zero points, group size a multiple of 64 (a stage never straddles
// two groups), K % 64 == 0, N % 4 == 0 (vector stores), 16-byte aligned pointers.
bool w4a16_gemm_supported(const void *codes, const void *x, int x_dtype, int zp_integer, int64_t M, int64_t N,
                          int64_t K, int64_t gs)
{
    return x_dtype == NSLQ_DTYPE_BF16 && zp_integer && (K % 64 == 0) && (gs % 64 == 0) && (N % 4 == 0) &&
           aligned16(codes) && aligned16(x) && M > 0 && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 30);
}

template <int BN>
static int launch_w4_gemm(const uint8_t *codes, const void *x, w4gemm::Params &p, cudaStream_t st)
{
    using C = w4gemm::Cfg<BN>;
    static std::atomic<size_t> reserved[kMaxDevices];
    if (reserve_smem(w4gemm::w4a16_gemm_kernel<BN>, reserved, (size_t)C::SMEM) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "w4a16_gemm_kernel: cannot reserve %d bytes of shared memory: %s", C::SMEM,
                    cudaGetErrorString(cudaGetLastError()));
    CUtensorMap tmap_a, tmap_w;
    int rc = sm100::make_map_2d(&tmap_a, x, (uint64_t)p.K * 2, (uint64_t)p.M, w4gemm::BKB, w4gemm::BM, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = sm100::make_map_2d(&tmap_w, codes, (uint64_t)(p.K / 2), (uint64_t)p.N, w4gemm::BKE / 2, BN, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    p.tiles_m = (int)((p.M + w4gemm::BM - 1) / w4gemm::BM);
    p.tiles_n = (int)((p.N + BN - 1) / BN);
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < sm100::sm_count() ? tiles : sm100::sm_count();
    w4gemm::w4a16_gemm_kernel<BN><<<grid, w4gemm::THREADS, C::SMEM, st>>>(tmap_a, tmap_w, p);
    return check_launch("w4a16_gemm_kernel");
}

static int w4_gemm_one_launch(const uint8_t *codes, const float *scale, const float *zc, int64_t N, int64_t K, int G, int gs,
                              const void *x, int64_t M, void *y, int y_dtype, cudaStream_t st)
{
    w4gemm::Params p{scale, zc, y, M, N, K, G, gs, y_dtype, 0, 0};
    const int sms = sm100::sm_count();
    auto rounds_cost = [&](int bn) {
        const int64_t tiles = ((M + w4gemm::BM - 1) / w4gemm::BM) * ((N + bn - 1) / bn);
        return (double)((tiles + sms - 1) / sms) * bn;
    };
    if (rounds_cost(192) < rounds_cost(256)) return launch_w4_gemm<192>(codes, x, p, st);
    return launch_w4_gemm<256>(codes, x, p, st);
}

// Long batches run as several launches of at most W4_GEMM_MAX_ROWS token rows, like the ternary
// GEMM: persistent tensor-memory kernels that ran for about a millisecond ended, now and then, in
// cudaErrorLaunchFailure on this machine; launches of a few hundred microseconds never did.
constexpr int64_t W4_GEMM_MAX_ROWS = 4096;

int w4a16_gemm_dispatch(const uint8_t *codes, const float *scale, const float *zc, int64_t N, int64_t K, int G, int gs,
                        const void *x, int64_t M, void *y, int y_dtype, cudaStream_t st)
{
    if (!aligned16(y)) return fail(NSLQ_ERR_ARG, "W4A16 GEMM: y must be 16-byte aligned");
    const int es = y_dtype == NSLQ_DTYPE_F32 ? 4 : 2;
    for (int64_t m0 = 0; m0 < M; m0 += W4_GEMM_MAX_ROWS) {
        const int64_t mc = (M - m0) < W4_GEMM_MAX_ROWS ? (M - m0) : W4_GEMM_MAX_ROWS;
        int rc = w4_gemm_one_launch(codes, scale, zc, N, K, G, gs, (const char *)x + m0 * K * 2, mc,
                                    (char *)y + m0 * N * es, y_dtype, st);
        if (rc) return rc;
    }
    return NSLQ_OK;
}

int w4a16_gemm_status(int *out) { return sm100::read_wait_status(out); }

}  // namespace nslq
