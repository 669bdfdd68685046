// Shared pieces of the tcgen05 / TMA kernels (sm_100a): PTX wrappers, bounded mbarrier waits,
// descriptor helpers and the host-side tensor-map encoder.  Header-only; every translation unit
// that includes it gets its own wait-status word (device variables are not shared across
// translation units without relocatable device code).
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace nslq {
namespace sm100 {

// 0 = ok; else the site code of the first bounded wait that expired in this unit's kernels.
static __device__ int g_wait_status = 0;
constexpr unsigned long long WAIT_NS = 2000000000ull;   // 2 s per wait, then give up

// ---------------------------------------------------------------- PTX wrappers
static __device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

static __device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
static __device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
static __device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
static __device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: true when the phase completed, false once it has given up (status word set).
// It gives up only when BOTH two seconds of wall clock have passed AND the thread has polled
// MIN_POLLS times itself: %globaltimer keeps running while the context is switched out for
// another tenant of the GPU, the poll count does not, so a pre-empted kernel is not mistaken for
// a stuck one.  `abort` (optional, shared memory, zeroed by the kernel) is a CTA-wide flag: the
// role whose wait expires raises it and every other role's wait leaves at its next check, so
// the whole CTA reaches its teardown together instead of each role serving its own two seconds.
constexpr uint32_t MIN_POLLS = 1u << 20;
static __device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int site, volatile int *abort = nullptr)
{
    long long t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((spin & 63u) == 63u) {
            if (abort && *abort) return false;
            // signed difference: should %globaltimer ever step backwards between two reads, an
            // unsigned difference would read as an instant timeout
            const long long now = (long long)globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > (long long)WAIT_NS && spin >= MIN_POLLS) {
                atomicCAS(&g_wait_status, 0, site);
                if (abort) *abort = 1;
                return false;
            }
        }
    }
}
// True in exactly one lane of a converged warp; the compiler keeps the guarded code on the uniform path.
static __device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
// The same wait for a whole warp (every lane must call it).  Lanes poll on their own and can leave
// the loop in different iterations; the .sync.aligned tcgen05 instructions that follow a wait need
// the warp converged, so it is re-formed here and the outcome made uniform.  (A version of
// mbar_wait that slept between polls let the lanes drift apart and, without this, ended in rare
// launch failures in millisecond-long launches.)
static __device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, int site, volatile int *abort = nullptr)
{
    const bool ok = mbar_wait(bar, parity, site, abort);
    return __all_sync(0xffffffffu, ok) != 0;
}
static __device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *tmap, int x, int y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar) : "memory");
}
static __device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
static __device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
static __device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
static __device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

static __device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

static __device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// Writes 32 consecutive 32-bit columns of this thread's TMEM lane (the warp's lane quadrant);
// tmem_st_wait() returns once the thread's stores have been performed.
static __device__ __forceinline__ void tmem_st32_issue(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
static __device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Integer MMA with the A operand (M = 128 rows, one per TMEM lane, four 8-bit K elements per
// 32-bit column) in tensor memory and the B operand described in shared memory.
static __device__ __forceinline__ void umma_i8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// K-major, 128-byte swizzle: 8-row groups 1024 B apart (SBO), LBO unused (=1), version 1.
static __device__ __forceinline__ uint64_t smem_desc(uint32_t addr)
{
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}


// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_tiled()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

static inline int sm_count() { return sm_count_current(); }

static inline int make_map_2d(CUtensorMap *m, const void *ptr, uint64_t inner_bytes, uint64_t rows, uint32_t box_inner,
                       uint32_t box_rows, CUtensorMapSwizzle swz)
{
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return fail(NSLQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t gdim[2] = {inner_bytes, rows};
    const cuuint64_t gstride[1] = {inner_bytes};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), gdim, gstride, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(NSLQ_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for %llu x %llu bytes", (int)r,
                    (unsigned long long)rows, (unsigned long long)inner_bytes);
    return NSLQ_OK;
}


// Reads and clears this unit's wait-status word.
static inline int read_wait_status(int *out)
{
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_wait_status, sizeof(int)) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "nslq_device_status: %s", cudaGetErrorString(cudaGetLastError()));
    if (v != 0) cudaMemcpyToSymbol(g_wait_status, &zero, sizeof(int));
    *out = v;
    return NSLQ_OK;
}

}  // namespace sm100
}  // namespace nslq
