// TEST AND BENCHMARK INFRASTRUCTURE -- never linked into nsl_b200/libnslq_b200.so and never on the product path.
//
// A CUDA C++ restatement of the STRUCTURE of the one GPU kernel NSL emits for a BitLinear forward pass
// (crates/nsl-codegen/src/bitnet/mod.rs:133-236 `synthesize_kernel`; phases absmean_quant.rs, packed_load.rs,
// ternary_gemm.rs:54-116, finalize.rs), so that the benchmark can put a GPU baseline of the reference's own
// design beside the library's kernels.  NSL emits PTX text at compile time; this file is written from the
// emitter's description of what a thread does, in this repository's own code:
//
//   grid (ceil(out_dim / block_n), rows), block_n threads (NSL's tests use block_n = 128);
//   1. the CTA reduces |x| over its activation row, quantises the WHOLE row to int8 into shared memory
//      (every CTA of a row repeats this: "each CTA redundantly recomputes the row absmax", mod.rs:124-128);
//   2. thread t owns output column blockIdx.x * block_n + t and walks k in steps of four: one global byte load of
//      packed weights (row-major [out_dim][hidden/4], so neighbouring threads read bytes hidden/4 apart: no
//      staging, no coalescing), four 2-bit codes -> trits, four shared-memory int8 loads, mul + add each;
//   3. y = (scale / 127) * acc, * weight_scale, + bias, + residual, store.
//
// The arithmetic is the reference's (crates/nsl-codegen/tests/bitnet_reference_impl.rs:46-98), so its outputs
// equal the CPU checker's bit for bit -- which tests/test_gpu_prior_art.py verifies before anyone times it.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace {

constexpr int BLOCK_N = 128;

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__global__ void __launch_bounds__(BLOCK_N) prior_art_bitlinear_kernel(const float *__restrict__ x, const uint8_t *__restrict__ w,
                                                                      float *__restrict__ y, int32_t *__restrict__ acc_out,
                                                                      int hidden, int out_dim, float weight_scale,
                                                                      const float *__restrict__ bias, const float *__restrict__ residual)
{
    extern __shared__ int8_t qact[];                          // [hidden]
    __shared__ float red[BLOCK_N / 32];
    __shared__ float scale_s;
    const int row = blockIdx.y;
    const float *xr = x + (int64_t)row * hidden;

    // 1. absmax of the row, then the whole row quantised into shared memory
    float mx = 0.0f;
    for (int k = threadIdx.x; k < hidden; k += BLOCK_N) mx = fmaxf(mx, fabsf(xr[k]));
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int i = 0; i < BLOCK_N / 32; ++i) s = fmaxf(s, red[i]);
        scale_s = s;
    }
    __syncthreads();
    const float scale = scale_s;
    const float inv = scale == 0.0f ? 0.0f : __fdiv_rn(127.0f, scale);
    for (int k = threadIdx.x; k < hidden; k += BLOCK_N) {
        int8_t q = 0;
        if (scale != 0.0f) {
            float v = __fmul_rn(xr[k], inv);
            v = v < -127.0f ? -127.0f : (v > 127.0f ? 127.0f : v);        // NaN passes through, as f32::clamp
            v = roundf(v);                                                 // half away from zero, as f32::round
            q = (v != v) ? 0 : (int8_t)v;                                  // `as i8`: NaN -> 0
        }
        qact[k] = q;
    }
    __syncthreads();

    // 2. one thread per output column, four trits per packed byte, scalar multiply-add
    const int col = blockIdx.x * BLOCK_N + threadIdx.x;
    if (col >= out_dim) return;                               // after the last barrier, as the emitter requires
    const uint8_t *wr = w + (int64_t)col * (hidden >> 2);
    int acc = 0;
    for (int k = 0; k < hidden; k += 4) {
        const uint32_t b = wr[k >> 2];
        acc += (int)qact[k + 0] * ((int)((b >> 6) & 3u) - 1);
        acc += (int)qact[k + 1] * ((int)((b >> 4) & 3u) - 1);
        acc += (int)qact[k + 2] * ((int)((b >> 2) & 3u) - 1);
        acc += (int)qact[k + 3] * ((int)(b & 3u) - 1);
    }

    // 3. finalize
    const int64_t o = (int64_t)row * out_dim + col;
    if (acc_out) acc_out[o] = acc;
    float v = __fmul_rn(__fmul_rn(__fdiv_rn(scale, 127.0f), (float)acc), weight_scale);
    if (bias) v = __fadd_rn(v, bias[col]);
    if (residual) v = __fadd_rn(v, residual[o]);
    y[o] = v;
}

// The reference's route for a weight-only-quantised linear (crates/nsl-runtime/src/quantize.rs:547-585
// nsl_qtensor_matmul_mixed): dequantise the whole weight to a dense tensor, every call, then a dense matmul (on the GPU its
// f32 tensor-core GEMM).  This kernel is the dequantisation, (q - zp) * scale in f64 rounded to f32 (dequantize_val, :258-266),
// for INT4 codes [N][K/2] (low nibble = even k) with per-group scale and zero point [N][K/group]; the dense matmul is the BLAS
// library's, called by the benchmark.  The reference dequantises on the CPU; doing it on the GPU flatters the baseline.
__global__ void __launch_bounds__(256) prior_art_w4_dequant_kernel(const uint8_t *__restrict__ codes, const float *__restrict__ scale,
                                                                   const uint8_t *__restrict__ zp, float *__restrict__ out, int64_t N,
                                                                   int64_t K, int64_t group)
{
    const int64_t G = (K + group - 1) / group;
    const int64_t total = N * (K >> 1);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / (K >> 1), kb = i % (K >> 1);
        const uint8_t b = codes[i];
        const int64_t g = (2 * kb) / group;
        const double sc = (double)scale[n * G + g];
        const double z = (double)zp[n * G + g];
        out[n * K + 2 * kb] = (float)(((double)(b & 15u) - z) * sc);
        out[n * K + 2 * kb + 1] = (float)(((double)(b >> 4) - z) * sc);
    }
}

}  // namespace

extern "C" int nslo_gpu_prior_art_w4_dequant(const uint8_t *codes, const float *scale, const uint8_t *zp, float *out, int64_t N, int64_t K,
                                             int64_t group, void *stream)
{
    if (!codes || !scale || !zp || !out || N <= 0 || K <= 0 || K % 2 != 0 || group <= 0 || group % 2 != 0) return -1;
    prior_art_w4_dequant_kernel<<<148 * 8, 256, 0, (cudaStream_t)stream>>>(codes, scale, zp, out, N, K, group);
    return (int)cudaGetLastError();
}

// x [rows][hidden] f32, w [out_dim][hidden/4] NSL's packed bytes, y [rows][out_dim] f32, all on the device.
// Returns 0, -1 for a bad argument, or the CUDA error code of the launch.
extern "C" int nslo_gpu_prior_art_bitlinear(const float *x, const uint8_t *w, float *y, int32_t *acc_out, int64_t rows,
                                            int64_t hidden, int64_t out_dim, float weight_scale, const float *bias,
                                            const float *residual, void *stream)
{
    if (!x || !w || !y || rows <= 0 || hidden <= 0 || out_dim <= 0 || hidden % 4 != 0 || rows > 65535 || hidden > 48 * 1024 ||
        out_dim * hidden > 0xffffffffLL)                      // the emitter's own refusals: SMEM budget, 32-bit trit index
        return -1;
    const dim3 grid((unsigned)((out_dim + BLOCK_N - 1) / BLOCK_N), (unsigned)rows);
    prior_art_bitlinear_kernel<<<grid, BLOCK_N, (size_t)hidden, (cudaStream_t)stream>>>(x, w, y, acc_out, (int)hidden, (int)out_dim,
                                                                                        weight_scale, bias, residual);
    return (int)cudaGetLastError();
}
