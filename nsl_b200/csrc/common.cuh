// Shared helpers of the sm_100a quantized-linear kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/nslq_b200.h"

// The object behind nslq_bitlinear_t: a borrowed packed weight and its shape.
struct nslq_bitlinear {
    const uint8_t *packed;   // [N][K/4], NSL's packed ternary layout
    int64_t N, K;
    float weight_scale;
};

namespace nslq {

// Where a linear's output goes when it is not a plain [M][N] array: the row stride of y
// (a column block of a wider [M][ldy] result) and, in a column-sharded run, the address of
// the same block in the other ranks' copies of that result, which receive the same stores.
struct OutSpec {
    int64_t ldy;
    int npeer;
    void *peer[NSLQ_MAX_RANKS - 1];
};

// Records the calling thread's last error text and returns `code`.
int fail(int code, const char *fmt, ...);
// Checks cudaGetLastError() after a launch.
int check_launch(const char *what);

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// One-time CUDA state is per device (a function attribute set on device 0 says nothing about
// device 1), so launchers keep it in tables indexed by the current device.
constexpr int kMaxDevices = 64;
static inline int device_index()
{
    int d = 0;
    cudaGetDevice(&d);
    return (d >= 0 && d < kMaxDevices) ? d : 0;
}
// Makes sure `kernel` may use `smem` bytes of dynamic shared memory on the current device.
// `table` is the launcher's own static table (zero-initialised); safe from several host threads.
template <typename K>
static inline cudaError_t reserve_smem(K kernel, std::atomic<size_t> (&table)[kMaxDevices], size_t smem)
{
    std::atomic<size_t> &slot = table[device_index()];
    if (smem <= 48 * 1024 || smem <= slot.load(std::memory_order_acquire)) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) {
        size_t seen = slot.load(std::memory_order_relaxed);
        while (seen < smem && !slot.compare_exchange_weak(seen, smem, std::memory_order_release)) {}
    }
    return e;
}
static inline int sm_count_current()
{
    static std::atomic<int> n[kMaxDevices];
    const int d = device_index();
    int v = n[d].load(std::memory_order_relaxed);
    if (!v) {
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, d);
        n[d].store(v, std::memory_order_relaxed);
    }
    return v;
}

template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float to_f32(float v) { return v; }
    static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <> struct Elem<__half> {
    static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};

// Stores an fp32 result as dtype tag `dt` (F32 / FP16 / BF16), round to nearest even.
static __device__ __forceinline__ void store_out(void *y, int dt, int64_t idx, float v)
{
    if (dt == NSLQ_DTYPE_F32) reinterpret_cast<float *>(y)[idx] = v;
    else if (dt == NSLQ_DTYPE_BF16) reinterpret_cast<__nv_bfloat16 *>(y)[idx] = __float2bfloat16_rn(v);
    else reinterpret_cast<__half *>(y)[idx] = __float2half_rn(v);
}

// BitLinear epilogue, each step separately rounded (no fused multiply-add):
//   ((scale / 127) * (float)acc) * weight_scale [+ bias] [+ residual]
static __device__ __forceinline__ float bitlinear_finalize(int acc, float act_scale, float weight_scale)
{
    float v = __fmul_rn(__fdiv_rn(act_scale, 127.0f), __int2float_rn(acc));
    return __fmul_rn(v, weight_scale);
}

// Programmatic dependent launch: both are no-ops for a kernel launched without
// the attribute.  wait = results of the preceding kernel in the stream are visible.
static __device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
static __device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Per-token absmax int8 quantisation of one value, the reference's arithmetic
// (crates/nsl-codegen/tests/bitnet_reference_impl.rs:58-70): v = x*inv (inv = 127/scale,
// IEEE divide), clamp to [-127,127], round half away from zero, saturating cast, NaN -> 0.
static __device__ __forceinline__ int quant_one(float x, float inv)
{
    const float s = __fmul_rn(x, inv);
    // Round half away from zero as trunc(s + copysign(0.5, s)).  The sum is exact or rounds inside
    // the same integer interval for every |s| >= 0.5 (s and s + 0.5 share a binade or the sum lands
    // on a representable value one ulp below the next integer); only below 0.5, where s has finer
    // ulps than the sum, can the addition round up to 1.0 -- those values round to 0 and are taken
    // out first.  One conversion instead of a trunc and a conversion: the quantisers are bound by
    // issued instructions, and conversions issue at a quarter of the ALU rate.
    const float h = __int_as_float((__float_as_int(s) & 0x80000000) | 0x3f000000);      // copysign(0.5, s)
    const int r = fabsf(s) < 0.5f ? 0 : __float2int_rz(__fadd_rn(s, h));               // saturating; NaN -> 0
    // The float clamp of the reference commutes with the rounding: clamping the rounded integer
    // gives the same value for every input, and the saturating conversion maps +-inf to the
    // int extremes (then +-127) and NaN to 0, exactly as `clamp(..).round() as i8` does.
    return max(-127, min(127, r));
}

// Four consecutive elements of a row as fp32 (vector load; row must be 16-byte aligned for
// fp32, 8-byte for the 16-bit types).
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float *row, int64_t v) {
        return reinterpret_cast<const float4 *>(row)[v];
    }
};
template <> struct Vec4<__half> {
    static __device__ __forceinline__ float4 load(const __half *row, int64_t v) {
        uint2 r = reinterpret_cast<const uint2 *>(row)[v];
        float2 a = __half22float2(*reinterpret_cast<__half2 *>(&r.x));
        float2 b = __half22float2(*reinterpret_cast<__half2 *>(&r.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16 *row, int64_t v) {
        uint2 r = reinterpret_cast<const uint2 *>(row)[v];
        float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&r.x));
        float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&r.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
};

// Four quantised values of lane j of a quad (k = 4j..4j+3 of a group of 16) -> the word this
// lane stores in the consumption order (position 4i+j holds k = 4j+i): lane i gets byte i of
// the four lanes' words, a 4x4 byte transpose across the quad.  `mask` names the
// participating lanes (whole quads).
static __device__ __forceinline__ uint32_t quad_transpose(uint32_t w, unsigned mask)
{
    const int lane = threadIdx.x & 31, qb = lane & ~3, i = lane & 3;
    const uint32_t w0 = __shfl_sync(mask, w, qb + 0), w1 = __shfl_sync(mask, w, qb + 1);
    const uint32_t w2 = __shfl_sync(mask, w, qb + 2), w3 = __shfl_sync(mask, w, qb + 3);
    const uint32_t lo = __byte_perm(w0, w1, 0x0040 + i * 0x0011);   // (w0.b[i], w1.b[i], -, -)
    const uint32_t hi = __byte_perm(w2, w3, 0x0040 + i * 0x0011);
    return __byte_perm(lo, hi, 0x5410);
}

static __device__ __forceinline__ uint32_t pack4_i8(int q0, int q1, int q2, int q3)
{
    return (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) |
           ((uint32_t)(q3 & 0xff) << 24);
}

// Launch with the programmatic-dependent-launch attribute (when enabled): the kernel may be
// scheduled while the preceding kernel of the stream drains; it must call pdl_wait() before
// it touches anything that kernel produced or still reads.
extern int g_use_pdl;
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                        cudaStream_t st, Args &&...args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// 128-bit streaming load of weights that are read exactly once.
static __device__ __forceinline__ uint4 ld_stream_u4(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

}  // namespace nslq
