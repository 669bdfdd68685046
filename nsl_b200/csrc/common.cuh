// Shared helpers of the sm_100a quantized-linear kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nslq_b200.h"

// The object behind nslq_bitlinear_t: a borrowed packed weight and its shape.
struct nslq_bitlinear {
    const uint8_t *packed;   // [N][K/4], NSL's packed ternary layout
    int64_t N, K;
    float weight_scale;
};

namespace nslq {

// Records the calling thread's last error text and returns `code`.
int fail(int code, const char *fmt, ...);
// Checks cudaGetLastError() after a launch.
int check_launch(const char *what);

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

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

// 128-bit streaming load of weights that are read exactly once.
static __device__ __forceinline__ uint4 ld_stream_u4(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

}  // namespace nslq
