// extern "C" entry points of libnslq_b200: argument checks, handle objects,
// kernel selection.  No arithmetic happens on the host and there is no CPU path:
// every computing call ends in a kernel launch or an error status.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace nslq {

static thread_local char g_err[512] = "";
int g_use_pdl = 1;

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int check_launch(const char *what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return NSLQ_OK;
}

// kernels (other translation units)
int act_quant_dispatch(const void *, int, int64_t, int64_t, int8_t *, int8_t *, float *, int32_t *, cudaStream_t);
int rmsnorm_act_quant_dispatch(const void *, int, const float *, double, int64_t, int64_t, float *, int8_t *, int8_t *,
                               float *, int32_t *, cudaStream_t);
int swiglu_act_quant_dispatch(const void *, const void *, int, int64_t, int64_t, int64_t, int64_t, float *, int8_t *, int8_t *, float *,
                              int32_t *, cudaStream_t);
int decode_attention_dispatch(const void *, const void *, const void *, int64_t, int64_t, int64_t, void *, void *, const float *, const float *,
                              const int64_t *, int64_t, int64_t, int64_t, int64_t, int64_t, float, void *, cudaStream_t);
bool ternary_gemv_supported(const void *, const void *, int64_t);
bool ternary_gemv_bulk_takes_one_row(int64_t);
int ternary_gemv_dispatch(const uint8_t *, const int8_t *, const float *, const int32_t *, int, int64_t, int64_t,
                          float, void *, int, int32_t *, const float *, const float *, cudaStream_t);
int ternary_scalar_dispatch(const uint8_t *, const int8_t *, const float *, int64_t, int64_t, int64_t, float,
                            void *, int, int32_t *, const float *, const float *, cudaStream_t);
bool ternary_gemv_fused_supported(const void *, const void *, int64_t, int64_t);
bool ternary_gemv_src_supported(const void *, const void *, const void *, const float *, int64_t, int64_t);
int ternary_gemv_src_dispatch(const uint8_t *, const void *, const void *, const float *, double, int, int, int64_t, int64_t, float, void *,
                              int, int32_t *, const float *, const float *, cudaStream_t);
int ternary_gemv_multi_dispatch_q(int, const uint8_t *const *, const int64_t *, const float *, void *const *, const int8_t *, const float *,
                                  const int32_t *, int, int64_t, int, cudaStream_t);
int ternary_gemv_multi_dispatch(int, const uint8_t *const *, const int64_t *, const float *, const float *const *, void *const *, const void *,
                                const float *, double, int, int, int64_t, int, cudaStream_t);
int ternary_gemv_fused_dispatch(const uint8_t *, const void *, int, int, int64_t, int64_t, float, void *, int, int32_t *,
                                const float *, const float *, cudaStream_t);
bool ternary_decode_supported(const void *, const void *, int64_t, int64_t, int64_t);
int ternary_decode_dispatch(const uint8_t *, const int8_t *, const float *, const int32_t *, int, int64_t, int64_t,
                            float, void *, int, int32_t *, const float *, const float *, cudaStream_t);
bool ternary_decode_fused_supported(const void *, const void *, int, int64_t, int64_t, int64_t);
int ternary_decode_fused_dispatch(const uint8_t *, const void *, int, int, int64_t, int64_t, float, void *, int, int32_t *,
                                  const float *, const float *, cudaStream_t);
int ternary_decode_status(int *);
int ternary_gemv_status(int *);
int decode_attention_status(int *);
int decode_glue_status(int *);
bool ternary_gemm_supported(const void *, const void *, int64_t, int64_t, int64_t);
int ternary_gemm_dispatch(const uint8_t *, const int8_t *, const float *, const int32_t *, int64_t, int64_t,
                          int64_t, float, void *, int, int32_t *, const float *, const float *, const OutSpec *, cudaStream_t);
int ternary_gemm_status(int *);
int w4a16_gemm_status(int *);
bool w4a16_gemv_supported(const void *, const void *, int, int64_t, int64_t);
int w4a16_gemv_dispatch(const uint8_t *, const float *, const float *, int64_t, int64_t, int, int, const void *,
                        int, int, void *, int, cudaStream_t);
int w4a16_scalar_dispatch(const uint8_t *, const float *, const float *, int64_t, int64_t, int, int, const void *,
                          int, int64_t, void *, int, cudaStream_t);
bool w4a16_decode_supported(const void *, const void *, int, int64_t, int64_t, int64_t, int64_t);
int w4a16_decode_dispatch(const uint8_t *, const float *, const float *, int64_t, int64_t, int, int, const void *, int,
                          int, void *, int, cudaStream_t);   // tables transposed, [G][N]
int w4a16_decode_status(int *);
bool w4a16_gemm_supported(const void *, const void *, int, int64_t, int64_t, int64_t, int64_t);
int w4a16_gemm_dispatch(const uint8_t *, const float *, const float *, int, int64_t, int64_t, int, int, const void *, int, int64_t,
                        void *, int, cudaStream_t);   // tables transposed, [G][N]

int ternary_quantize_pack_dispatch(const void *, int, int64_t, uint8_t *, float *, cudaStream_t);
int int4_quantize_nk_dispatch(const void *, int, int64_t, int64_t, int64_t, uint8_t *, float *, uint8_t *, cudaStream_t);
int awq_quantize_kn_dispatch(const void *, int, int64_t, int64_t, int64_t, uint8_t *, double *, double *, cudaStream_t);
int qtensor_quantize_dispatch(const void *, int, const int64_t *, int, int, int, int, int64_t, uint8_t *, float *, uint8_t *, cudaStream_t);
int qtensor_dequantize_dispatch(const uint8_t *, const float *, const uint8_t *, const int64_t *, int, int, int, int, int64_t, void *, int, cudaStream_t);
int64_t qtensor_num_scales(const int64_t *, int, int, int, int64_t);

// Which decode kernel for M <= 16 tokens.  The tensor-memory kernel (ternary_decode_kernel) streams
// at 4-5 TB/s but has ~5 us of start-up (TMEM allocation, token staging, pipeline fill); the
// register-staged kernels (ternary_gemv*.cu) start in ~2 us and stream at 1-2 TB/s.  Measured
// crossovers on B200 (K = 3200): 13 MB of packed weights at M = 1, 10 MB at M = 4, 28 MB at M = 8,
// none at M = 16 (the tensor-memory kernel wins from the smallest size).  (One row in its own dtype never gets
// here: nslq_bitlinear_forward sends it to the bulk-copy kernel first; the rule still decides for pre-quantised rows.)
static inline bool decode_pays(int64_t M, int64_t N, int64_t K)
{
    const double mb = (double)N * (double)K / 4.0 / 1.0e6;
    if (M > 8) return true;
    if (M > 4) return mb >= 28.0;
    return mb >= 12.0;
}

// W4A16, M <= 16: the tensor-memory kernel (w4a16_decode_kernel) against the mma.sync kernel
// (w4a16_gemv_persistent_kernel).  Measured on [11008, 4096], group 128: 14.8 vs 13.1 us at M = 1,
// 15.1 vs 16.7 at M = 4, 16.9 vs 22.7 at M = 8, 19.2 vs 35 at M = 16 -- the new kernel's cost barely
// depends on M, the old one's grows with it.
static inline bool w4_decode_pays(int64_t M, int64_t, int64_t) { return M >= 4; }

static inline int out_elem_size(int dt)
{
    return dt == NSLQ_DTYPE_F32 ? 4 : (dt == NSLQ_DTYPE_FP16 || dt == NSLQ_DTYPE_BF16) ? 2 : 0;
}

static inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

}  // namespace nslq

using namespace nslq;

struct nslq_w4a16 {
    const uint8_t *codes;   // [N][K/2]
    uint8_t *codes_owned;   // non-null when the library made its own copy
    float *scale;           // [N][G] owned
    float *zc;              // [N][G] owned, zero point in code units
    float *scale_t, *zc_t;  // the same two tables transposed, [G][N]: coalesced for a thread per row
    int64_t N, K;
    int G, gs;
    int zp_integer;         // zero points are whole numbers (QuantizedTensor form), not AWQ float zeros
};

// ------------------------------------------------------------------ small table kernels
namespace nslq {

// [N][G] -> [G][N] for both tables (small, run once per weight)
__global__ void w4_transpose_kernel(const float *__restrict__ scale, const float *__restrict__ zc, int64_t N, int G,
                                    float *__restrict__ scale_t, float *__restrict__ zc_t)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;     // index into the [G][N] output
    if (i >= N * G) return;
    const int64_t g = i / N, n = i - g * N;
    scale_t[i] = scale[n * G + g];
    zc_t[i] = zc[n * G + g];
}

template <typename S>
__global__ void w4_tables_nk_kernel(const S *__restrict__ scales, const uint8_t *__restrict__ zp, int zp_packed,
                                    int64_t n, float *__restrict__ scale_out, float *__restrict__ zc_out)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    scale_out[i] = (float)scales[i];
    int z = zp_packed ? ((i & 1) ? (zp[i >> 1] >> 4) : (zp[i >> 1] & 15)) : zp[i];
    zc_out[i] = (float)z;
}

// AWQ [K,N] -> [N,K]: one thread per output byte (n, k/2).
__global__ void awq_repack_codes_kernel(const uint8_t *__restrict__ data, int64_t K, int64_t N,
                                        uint8_t *__restrict__ out)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t kb = K >> 1;
    if (i >= N * kb) return;
    const int64_t n = i / kb, k0 = (i % kb) * 2;
    const int64_t f0 = k0 * N + n, f1 = (k0 + 1) * N + n;
    const uint8_t q0 = (f0 & 1) ? (data[f0 >> 1] >> 4) : (data[f0 >> 1] & 15);
    const uint8_t q1 = (f1 & 1) ? (data[f1 >> 1] >> 4) : (data[f1 >> 1] & 15);
    out[i] = (uint8_t)(q0 | (q1 << 4));
}

// AWQ tables [G,N] f64 -> [N,G] f32; zero (group minimum) becomes a zero point in
// code units: q*s + z = (q - (-z/s)) * s.
__global__ void awq_tables_kernel(const double *__restrict__ scales, const double *__restrict__ zeros, int G,
                                  int64_t N, float *__restrict__ scale_out, float *__restrict__ zc_out)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N * G) return;
    const int64_t n = i / G;
    const int g = (int)(i % G);
    const double s = scales[(int64_t)g * N + n], z = zeros[(int64_t)g * N + n];
    scale_out[i] = (float)s;
    zc_out[i] = (float)(-z / s);
}

// QuantizedTensor [K,N] (index rules of crates/nsl-runtime/src/quantize.rs:366-417, :436-537) -> the
// [N][G] tables of the streaming kernels, for the granularities whose scale index does not depend on
// k inside a group of `gs` consecutive k: per tensor (one scale), per channel along axis 1 (scale[n]),
// per group along axis 0 (scale[k / group], shared by every n).
__global__ void qtensor_tables_kernel(const float *__restrict__ scale, const uint8_t *__restrict__ zp, int gran, int64_t N,
                                      int G, float *__restrict__ scale_out, float *__restrict__ zc_out)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N * G) return;
    const int64_t n = i / G;
    const int g = (int)(i % G);
    const int64_t si = gran == 0 ? 0 : (gran == 1 ? n : g);
    scale_out[i] = scale[si];
    zc_out[i] = (float)zp[si];
}

// Counts the bytes of a packed ternary weight that hold the reserved 2-bit code 0b11.
__global__ void __launch_bounds__(256) count_invalid_codes_kernel(const uint8_t *__restrict__ packed, int64_t nbytes,
                                                                  unsigned long long *__restrict__ count)
{
    unsigned long long bad = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nbytes; i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t b = packed[i];
        bad += ((b & (b >> 1)) & 0x55u) != 0;              // some field has both bits set
    }
    for (int o = 16; o > 0; o >>= 1) bad += __shfl_xor_sync(0xffffffffu, bad, o);
    if ((threadIdx.x & 31) == 0 && bad) atomicAdd(count, bad);
}

// fp32 activations for the 16-bit kernels without rounding them: x = hi + mid + lo, three bf16 parts
// (each remainder is exact in fp32 and is rounded again: 3 x 8 significant bits cover fp32's 24), stacked
// as rows [0, M) = hi, [M, 2M) = mid, [2M, 3M) = lo; the three parts of the result are added afterwards.
__global__ void split_f32_bf16_kernel(const float *__restrict__ x, int64_t n, __nv_bfloat16 *__restrict__ out)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = x[i];
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
    out[i] = hi;
    out[n + i] = mid;
    out[2 * n + i] = __float2bfloat16_rn(r1 - __bfloat162float(mid));
}

__global__ void add_parts_kernel(const float *__restrict__ yy, int64_t n, void *__restrict__ y, int y_dtype)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    store_out(y, y_dtype, i, (yy[2 * n + i] + yy[n + i]) + yy[i]);
}

}  // namespace nslq

// ------------------------------------------------------------------ extern "C"
extern "C" {

int nslq_version(void) { return 100; }

const char *nslq_last_error(void) { return g_err; }

void nslq_set_dependent_launch(int enable) { g_use_pdl = enable ? 1 : 0; }

int nslq_device_status(int *status)
{
    if (!status) return fail(NSLQ_ERR_ARG, "nslq_device_status: null output");
    // The words live in device memory: reading them waits for the work in front of the read (the
    // copies below run on the legacy default stream, which orders them behind every blocking stream).
    int a = 0, b = 0, c = 0, d = 0, e = 0;
    int rc = ternary_gemm_status(&a);
    if (rc) return rc;
    if ((rc = w4a16_gemm_status(&b))) return rc;
    if ((rc = ternary_decode_status(&c))) return rc;
    if ((rc = w4a16_decode_status(&d))) return rc;
    if ((rc = ternary_gemv_status(&e))) return rc;
    int f = 0;
    if ((rc = decode_attention_status(&f))) return rc;
    int g = 0;
    if ((rc = decode_glue_status(&g))) return rc;
    *status = a ? a : (b ? b : (c ? c : (d ? d : (e ? e : (f ? f : g)))));
    return NSLQ_OK;
}

int nslq_act_quant_i8(const void *x, int x_dtype, int64_t M, int64_t K, int8_t *q_plain, int8_t *q_perm,
                      float *scale, int32_t *rowsum, void *stream)
{
    return act_quant_dispatch(x, x_dtype, M, K, q_plain, q_perm, scale, rowsum, (cudaStream_t)stream);
}

int nslq_rmsnorm_act_quant_i8(const void *x, int x_dtype, const float *weight, double eps, int64_t M, int64_t K,
                              float *h_out, int8_t *q_plain, int8_t *q_perm, float *scale, int32_t *rowsum, void *stream)
{
    return rmsnorm_act_quant_dispatch(x, x_dtype, weight, eps, M, K, h_out, q_plain, q_perm, scale, rowsum, (cudaStream_t)stream);
}

int nslq_swiglu_act_quant_i8(const void *gate, const void *up, int dtype, int64_t M, int64_t K, int64_t gate_ld,
                             int64_t up_ld, float *h_out,
                             int8_t *q_plain, int8_t *q_perm, float *scale, int32_t *rowsum, void *stream)
{
    return swiglu_act_quant_dispatch(gate, up, dtype, M, K, gate_ld, up_ld, h_out, q_plain, q_perm, scale, rowsum, (cudaStream_t)stream);
}

int nslq_decode_attention(const void *q, const void *k_new, const void *v_new, int64_t q_batch_stride,
                          int64_t k_batch_stride, int64_t v_batch_stride, void *k_cache, void *v_cache,
                          const float *cos_table, const float *sin_table, const int64_t *pos, int64_t B, int64_t H,
                          int64_t Hkv, int64_t D, int64_t max_ctx, float sm_scale, void *out, void *stream)
{
    return decode_attention_dispatch(q, k_new, v_new, q_batch_stride, k_batch_stride, v_batch_stride, k_cache, v_cache, cos_table, sin_table, pos, B, H, Hkv, D, max_ctx,
                                     sm_scale, out, (cudaStream_t)stream);
}

int nslq_bitlinear_create(const uint8_t *packed, int64_t N, int64_t K, float weight_scale,
                          nslq_bitlinear_t **out)
{
    if (!packed || !out) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_create: null argument");
    if (N <= 0 || K <= 0) return fail(NSLQ_ERR_SHAPE, "nslq_bitlinear_create: N=%lld K=%lld", (long long)N, (long long)K);
    if (K % 4 != 0) return fail(NSLQ_ERR_SHAPE, "nslq_bitlinear_create: hidden_dim %lld is not a multiple of 4", (long long)K);
    nslq_bitlinear *h = (nslq_bitlinear *)malloc(sizeof(nslq_bitlinear));
    if (!h) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_create: out of host memory");
    h->packed = packed; h->N = N; h->K = K; h->weight_scale = weight_scale;
    *out = h;
    return NSLQ_OK;
}

void nslq_bitlinear_destroy(nslq_bitlinear_t *w) { free(w); }

int nslq_bitlinear_validate(const nslq_bitlinear_t *w, int64_t *invalid_bytes, void *stream)
{
    if (!w) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_validate: null handle");
    unsigned long long *d = nullptr, h = 0;
    if (cudaMalloc(&d, sizeof(h)) != cudaSuccess || cudaMemsetAsync(d, 0, sizeof(h), (cudaStream_t)stream) != cudaSuccess) {
        if (d) cudaFree(d);
        return fail(NSLQ_ERR_CUDA, "nslq_bitlinear_validate: %s", cudaGetErrorString(cudaGetLastError()));
    }
    const int64_t nb = w->N * (w->K / 4);
    const unsigned blocks = (unsigned)(nb / 256 / 8 + 1 < 1184 ? nb / 256 / 8 + 1 : 1184);
    count_invalid_codes_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(w->packed, nb, d);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpyAsync(&h, d, sizeof(h), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    cudaFree(d);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "nslq_bitlinear_validate: %s", cudaGetErrorString(e));
    if (invalid_bytes) *invalid_bytes = (int64_t)h;
    if (h) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_validate: %llu packed bytes hold the reserved 2-bit code 0b11 (not a trit)", h);
    return NSLQ_OK;
}

// workspace layout: [q_perm or q_plain: M*K, 256-aligned][scale: M f32, 256-aligned][rowsum: M i32]
int64_t nslq_bitlinear_workspace_bytes(int64_t M, int64_t K)
{
    if (M < 0 || K <= 0) return 0;
    return align_up(M * K, 256) + align_up(M * 4, 256) + align_up(M * 4, 256);
}

int nslq_bitlinear_forward_quantized(const nslq_bitlinear_t *w, const int8_t *q_perm, const float *scale,
                                     const int32_t *rowsum, int64_t M, void *y, int y_dtype, int32_t *acc_out,
                                     const float *bias, const float *residual, void *stream)
{
    if (!w || !q_perm || !scale || !rowsum || !y) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward_quantized: null argument");
    if (!out_elem_size(y_dtype)) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward_quantized: y_dtype %d not in {F32,FP16,BF16}", y_dtype);
    if (M < 0) return fail(NSLQ_ERR_SHAPE, "nslq_bitlinear_forward_quantized: M=%lld", (long long)M);
    if (M == 0) return NSLQ_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (M > 16 && ternary_gemm_supported(w->packed, q_perm, M, w->N, w->K))
        return ternary_gemm_dispatch(w->packed, q_perm, scale, rowsum, M, w->N, w->K, w->weight_scale, y, y_dtype,
                                     acc_out, bias, residual, nullptr, st);
    if (!ternary_gemv_supported(w->packed, q_perm, w->K))
        return fail(NSLQ_ERR_UNSUPPORTED, "nslq_bitlinear_forward_quantized: needs K %% 64 == 0 and 16-byte aligned buffers (K=%lld)",
                    (long long)w->K);
    const int es = out_elem_size(y_dtype);
    for (int64_t m0 = 0; m0 < M; m0 += 16) {
        const int mc = (int)((M - m0) < 16 ? (M - m0) : 16);
        if (decode_pays(mc, w->N, w->K) && ternary_decode_supported(w->packed, q_perm + m0 * w->K, mc, w->N, w->K)) {
            int rc = ternary_decode_dispatch(w->packed, q_perm + m0 * w->K, scale + m0, rowsum + m0, mc, w->N, w->K,
                                             w->weight_scale, (char *)y + m0 * w->N * es, y_dtype,
                                             acc_out ? acc_out + m0 * w->N : nullptr, bias,
                                             residual ? residual + m0 * w->N : nullptr, st);
            if (rc) return rc;
            continue;
        }
        int rc = ternary_gemv_dispatch(w->packed, q_perm + m0 * w->K, scale + m0, rowsum + m0, mc, w->N, w->K,
                                       w->weight_scale, (char *)y + m0 * w->N * es, y_dtype,
                                       acc_out ? acc_out + m0 * w->N : nullptr, bias,
                                       residual ? residual + m0 * w->N : nullptr, st);
        if (rc) return rc;
    }
    return NSLQ_OK;
}

int nslq_bitlinear_forward(const nslq_bitlinear_t *w, const void *x, int x_dtype, int64_t M, void *y, int y_dtype,
                           int32_t *acc_out, const float *bias, const float *residual, void *workspace,
                           int64_t workspace_bytes, void *stream)
{
    if (!w || !x || !y) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward: null argument");
    if (!out_elem_size(y_dtype)) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward: y_dtype %d not in {F32,FP16,BF16}", y_dtype);
    if (M < 0) return fail(NSLQ_ERR_SHAPE, "nslq_bitlinear_forward: M=%lld", (long long)M);
    if (M == 0) return NSLQ_OK;
    const int64_t need = nslq_bitlinear_workspace_bytes(M, w->K);
    if (!workspace || workspace_bytes < need)
        return fail(NSLQ_ERR_WORKSPACE, "nslq_bitlinear_forward: workspace %lld bytes, need %lld", (long long)workspace_bytes, (long long)need);
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward: workspace not 256-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    int8_t *q = (int8_t *)workspace;
    float *scale = (float *)((char *)workspace + align_up(M * w->K, 256));
    int32_t *rowsum = (int32_t *)((char *)scale + align_up(M * 4, 256));
    // One token row: the bulk-copy kernel at every size it takes.  Measured against the tensor-memory kernel in chains of
    // dependent calls: 5.5 against 7.1 us on 12.8 MB of packed weights, 9.3 against 9.2 us on 25.6 MB -- and 5.1
    // against 8.5 us there when four independent calls run side by side (0.76 against 0.46 of the HBM rate).
    const bool bulk_one = M == 1 && ternary_gemv_bulk_takes_one_row(w->K) && ternary_gemv_fused_supported(w->packed, x, M, w->K) &&
                          (x_dtype == NSLQ_DTYPE_F32 || aligned16(x));
    if (bulk_one)
        return ternary_gemv_fused_dispatch(w->packed, x, x_dtype, 1, w->N, w->K, w->weight_scale, y, y_dtype, acc_out, bias, residual, st);
    if (decode_pays(M, w->N, w->K) && ternary_decode_fused_supported(w->packed, x, x_dtype, M, w->N, w->K))
        return ternary_decode_fused_dispatch(w->packed, x, x_dtype, (int)M, w->N, w->K, w->weight_scale, y, y_dtype, acc_out,
                                             bias, residual, st);
    // One launch that also quantises the tokens pays for one of them: every CTA repeats the quantisation.  Measured in
    // chains over weights that come from HBM, one launch against quantiser + pre-quantised kernel: one row 3.9 against
    // 5.3 us ([8640, 3200]) and 5.4 against 6.7 ([3200, 8640]); two rows 6.0 against 5.6 and 9.4 against 7.2; four rows
    // ([3200, 3200]) 7.3 against 1.7 + 2.9.
    if (M == 1 && !decode_pays(M, w->N, w->K) && ternary_gemv_fused_supported(w->packed, x, M, w->K) &&
        (x_dtype == NSLQ_DTYPE_F32 || aligned16(x)))
        return ternary_gemv_fused_dispatch(w->packed, x, x_dtype, (int)M, w->N, w->K, w->weight_scale, y, y_dtype, acc_out,
                                           bias, residual, st);
    const bool fast = (w->K % 64 == 0) && aligned16(w->packed);
    if (fast) {
        int rc = act_quant_dispatch(x, x_dtype, M, w->K, nullptr, q, scale, rowsum, st);
        if (rc) return rc;
        return nslq_bitlinear_forward_quantized(w, q, scale, rowsum, M, y, y_dtype, acc_out, bias, residual, stream);
    }
    int rc = act_quant_dispatch(x, x_dtype, M, w->K, q, nullptr, scale, rowsum, st);
    if (rc) return rc;
    return ternary_scalar_dispatch(w->packed, q, scale, M, w->N, w->K, w->weight_scale, y, y_dtype, acc_out, bias,
                                   residual, st);
}

// The RMSNorm or the SiLU(gate) * up in front of a projection, formed inside the projection's own launch for
// one token; the same two launches as the separate entry points (bit-equal results) above that.  (Measured in the
// decoder at two tokens: 1.38 ms per step with the prologue inside every projection's CTAs, whose two rows are formed one
// after the other, against 1.17 ms with the separate launch.)
static int forward_src(const char *who, const nslq_bitlinear_t *w, const void *x, const void *x2, const float *norm_w, double eps,
                       int x_dtype, int64_t M, void *y, int y_dtype, int32_t *acc_out, const float *bias, const float *residual,
                       void *workspace, int64_t workspace_bytes, void *stream)
{
    if (!w || !x || !y) return fail(NSLQ_ERR_ARG, "%s: null argument", who);
    if (!out_elem_size(y_dtype)) return fail(NSLQ_ERR_ARG, "%s: y_dtype %d not in {F32,FP16,BF16}", who, y_dtype);
    if (M < 0) return fail(NSLQ_ERR_SHAPE, "%s: M=%lld", who, (long long)M);
    if (M == 0) return NSLQ_OK;
    if (w->K % 64 != 0 || !aligned16(w->packed))
        return fail(NSLQ_ERR_UNSUPPORTED, "%s: K=%lld must be a multiple of 64 and the weight 16-byte aligned", who, (long long)w->K);
    cudaStream_t st = (cudaStream_t)stream;
    if (M == 1 && ternary_gemv_src_supported(w->packed, x, x2, norm_w, M, w->K))
        return ternary_gemv_src_dispatch(w->packed, x, x2, norm_w, eps, x_dtype, (int)M, w->N, w->K, w->weight_scale, y, y_dtype,
                                         acc_out, bias, residual, st);
    const int64_t need = nslq_bitlinear_workspace_bytes(M, w->K);
    if (!workspace || workspace_bytes < need)
        return fail(NSLQ_ERR_WORKSPACE, "%s: workspace %lld bytes, need %lld", who, (long long)workspace_bytes, (long long)need);
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(NSLQ_ERR_ARG, "%s: workspace not 256-byte aligned", who);
    int8_t *q = (int8_t *)workspace;
    float *scale = (float *)((char *)workspace + align_up(M * w->K, 256));
    int32_t *rowsum = (int32_t *)((char *)scale + align_up(M * 4, 256));
    const int rc = norm_w ? rmsnorm_act_quant_dispatch(x, x_dtype, norm_w, eps, M, w->K, nullptr, nullptr, q, scale, rowsum, st)
                          : swiglu_act_quant_dispatch(x, x2, x_dtype, M, w->K, w->K, w->K, nullptr, nullptr, q, scale, rowsum, st);
    if (rc) return rc;
    return nslq_bitlinear_forward_quantized(w, q, scale, rowsum, M, y, y_dtype, acc_out, bias, residual, stream);
}

int nslq_bitlinear_forward_rmsnorm(const nslq_bitlinear_t *w, const void *x, int x_dtype, int64_t M, const float *norm_weight,
                                   double eps, void *y, int y_dtype, int32_t *acc_out, const float *bias, const float *residual,
                                   void *workspace, int64_t workspace_bytes, void *stream)
{
    if (!norm_weight) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward_rmsnorm: null norm weight");
    return forward_src("nslq_bitlinear_forward_rmsnorm", w, x, nullptr, norm_weight, eps, x_dtype, M, y, y_dtype, acc_out, bias,
                       residual, workspace, workspace_bytes, stream);
}

int nslq_bitlinear_forward_swiglu(const nslq_bitlinear_t *w, const void *gate, const void *up, int dtype, int64_t M, void *y,
                                  int y_dtype, int32_t *acc_out, const float *bias, const float *residual, void *workspace,
                                  int64_t workspace_bytes, void *stream)
{
    if (!up) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward_swiglu: null up");
    return forward_src("nslq_bitlinear_forward_swiglu", w, gate, up, nullptr, 0.0, dtype, M, y, y_dtype, acc_out, bias, residual,
                       workspace, workspace_bytes, stream);
}

int nslq_bitlinear_forward_multi(const nslq_bitlinear_t *const *layers, int n_layers, const void *x, int x_dtype, int64_t M,
                                 const float *norm_weight, double eps, void *const *ys, int y_dtype, void *workspace,
                                 int64_t workspace_bytes, void *stream)
{
    const char *who = "nslq_bitlinear_forward_multi";
    if (!layers || !x || !ys) return fail(NSLQ_ERR_ARG, "%s: null argument", who);
    if (n_layers < 1 || n_layers > 4) return fail(NSLQ_ERR_ARG, "%s: %d layers, 1 to 4 are taken", who, n_layers);
    if (!out_elem_size(y_dtype)) return fail(NSLQ_ERR_ARG, "%s: y_dtype %d not in {F32,FP16,BF16}", who, y_dtype);
    for (int i = 0; i < n_layers; ++i) {
        if (!layers[i] || !ys[i]) return fail(NSLQ_ERR_ARG, "%s: null layer or output %d", who, i);
        if (layers[i]->K != layers[0]->K)
            return fail(NSLQ_ERR_SHAPE, "%s: layer %d has K=%lld, layer 0 K=%lld", who, i, (long long)layers[i]->K, (long long)layers[0]->K);
    }
    if (M < 0) return fail(NSLQ_ERR_SHAPE, "%s: M=%lld", who, (long long)M);
    if (M == 0) return NSLQ_OK;
    const int64_t K = layers[0]->K;
    if (K % 64 != 0) return fail(NSLQ_ERR_UNSUPPORTED, "%s: K=%lld must be a multiple of 64", who, (long long)K);
    cudaStream_t st = (cudaStream_t)stream;
    bool one_launch = M == 1;
    for (int i = 0; one_launch && i < n_layers; ++i)
        one_launch = ternary_gemv_src_supported(layers[i]->packed, x, nullptr, norm_weight, M, K);
    if (one_launch) {
        const uint8_t *ws[4];
        int64_t Ns[4];
        float scales[4];
        const float *biases[4];
        for (int i = 0; i < n_layers; ++i) { ws[i] = layers[i]->packed; Ns[i] = layers[i]->N; scales[i] = layers[i]->weight_scale; biases[i] = nullptr; }
        return ternary_gemv_multi_dispatch(n_layers, ws, Ns, scales, biases, ys, x, norm_weight, eps, x_dtype, (int)M, K, y_dtype, st);
    }
    // the rows are normalised and quantised once and every layer multiplies the same int8 rows
    const int64_t need = nslq_bitlinear_workspace_bytes(M, K);
    if (!workspace || workspace_bytes < need)
        return fail(NSLQ_ERR_WORKSPACE, "%s: workspace %lld bytes, need %lld", who, (long long)workspace_bytes, (long long)need);
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(NSLQ_ERR_ARG, "%s: workspace not 256-byte aligned", who);
    int8_t *q = (int8_t *)workspace;
    float *scale = (float *)((char *)workspace + align_up(M * K, 256));
    int32_t *rowsum = (int32_t *)((char *)scale + align_up(M * 4, 256));
    int rc = norm_weight ? rmsnorm_act_quant_dispatch(x, x_dtype, norm_weight, eps, M, K, nullptr, nullptr, q, scale, rowsum, st)
                         : act_quant_dispatch(x, x_dtype, M, K, nullptr, q, scale, rowsum, st);
    if (rc) return rc;
    // a few rows of small matrices: the streaming kernel takes all layers as one launch
    bool one_gemv = M <= 16 && n_layers > 1;
    for (int i = 0; one_gemv && i < n_layers; ++i)
        one_gemv = !decode_pays(M, layers[i]->N, K) && ternary_gemv_supported(layers[i]->packed, q, K);
    if (one_gemv) {
        const uint8_t *ws[4];
        int64_t Ns[4];
        float scales[4];
        for (int i = 0; i < n_layers; ++i) { ws[i] = layers[i]->packed; Ns[i] = layers[i]->N; scales[i] = layers[i]->weight_scale; }
        return ternary_gemv_multi_dispatch_q(n_layers, ws, Ns, scales, ys, q, scale, rowsum, (int)M, K, y_dtype, st);
    }
    for (int i = 0; i < n_layers; ++i)
        if ((rc = nslq_bitlinear_forward_quantized(layers[i], q, scale, rowsum, M, ys[i], y_dtype, nullptr, nullptr, nullptr, stream))) return rc;
    return NSLQ_OK;
}

// ---------------------------------------------------------------- W4A16
static int w4_alloc_tables(nslq_w4a16 *h)
{
    const size_t n = (size_t)h->N * (size_t)h->G;
    if (cudaMalloc(&h->scale, n * 4) != cudaSuccess || cudaMalloc(&h->zc, n * 4) != cudaSuccess ||
        cudaMalloc(&h->scale_t, n * 4) != cudaSuccess || cudaMalloc(&h->zc_t, n * 4) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "W4A16 tables: cudaMalloc failed: %s", cudaGetErrorString(cudaGetLastError()));
    return NSLQ_OK;
}

static int w4_transpose_tables(nslq_w4a16 *h)
{
    const int64_t n = h->N * h->G;
    nslq::w4_transpose_kernel<<<(unsigned)((n + 255) / 256), 256>>>(h->scale, h->zc, h->N, h->G, h->scale_t, h->zc_t);
    return nslq::check_launch("w4_transpose_kernel");
}

static int w4_check_shape(const char *who, int64_t N, int64_t K, int64_t gs)
{
    if (N <= 0 || K <= 0 || gs <= 0) return fail(NSLQ_ERR_SHAPE, "%s: N=%lld K=%lld group=%lld", who, (long long)N, (long long)K, (long long)gs);
    if (K % 2 != 0) return fail(NSLQ_ERR_SHAPE, "%s: K=%lld must be even (two codes per byte)", who, (long long)K);
    return NSLQ_OK;
}

int nslq_w4a16_create_nk(const uint8_t *codes, const void *scales, int scale_dtype, const uint8_t *zero_points,
                         int zp_packed, int64_t N, int64_t K, int64_t group_size, nslq_w4a16_t **out)
{
    if (!codes || !scales || !zero_points || !out) return fail(NSLQ_ERR_ARG, "nslq_w4a16_create_nk: null argument");
    int rc = w4_check_shape("nslq_w4a16_create_nk", N, K, group_size);
    if (rc) return rc;
    nslq_w4a16 *h = (nslq_w4a16 *)calloc(1, sizeof(nslq_w4a16));
    if (!h) return fail(NSLQ_ERR_ARG, "nslq_w4a16_create_nk: out of host memory");
    h->codes = codes; h->N = N; h->K = K; h->gs = (int)group_size; h->G = (int)((K + group_size - 1) / group_size);
    h->zp_integer = 1;
    if ((rc = w4_alloc_tables(h))) { nslq_w4a16_destroy(h); return rc; }
    const int64_t n = N * h->G;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    switch (scale_dtype) {
    case NSLQ_DTYPE_F32: w4_tables_nk_kernel<float><<<blocks, 256>>>((const float *)scales, zero_points, zp_packed, n, h->scale, h->zc); break;
    case NSLQ_DTYPE_F64: w4_tables_nk_kernel<double><<<blocks, 256>>>((const double *)scales, zero_points, zp_packed, n, h->scale, h->zc); break;
    case NSLQ_DTYPE_BF16: w4_tables_nk_kernel<__nv_bfloat16><<<blocks, 256>>>((const __nv_bfloat16 *)scales, zero_points, zp_packed, n, h->scale, h->zc); break;
    case NSLQ_DTYPE_FP16: w4_tables_nk_kernel<__half><<<blocks, 256>>>((const __half *)scales, zero_points, zp_packed, n, h->scale, h->zc); break;
    default: nslq_w4a16_destroy(h); return fail(NSLQ_ERR_ARG, "nslq_w4a16_create_nk: scale_dtype %d", scale_dtype);
    }
    if ((rc = check_launch("w4_tables_nk_kernel"))) { nslq_w4a16_destroy(h); return rc; }
    if ((rc = w4_transpose_tables(h))) { nslq_w4a16_destroy(h); return rc; }
    if (cudaDeviceSynchronize() != cudaSuccess) { nslq_w4a16_destroy(h); return fail(NSLQ_ERR_CUDA, "nslq_w4a16_create_nk: %s", cudaGetErrorString(cudaGetLastError())); }
    *out = h;
    return NSLQ_OK;
}

int nslq_w4a16_create_awq_kn(const uint8_t *data, const double *scales, const double *zeros, int64_t K, int64_t N,
                             int64_t group_size, nslq_w4a16_t **out)
{
    if (!data || !scales || !zeros || !out) return fail(NSLQ_ERR_ARG, "nslq_w4a16_create_awq_kn: null argument");
    int rc = w4_check_shape("nslq_w4a16_create_awq_kn", N, K, group_size);
    if (rc) return rc;
    nslq_w4a16 *h = (nslq_w4a16 *)calloc(1, sizeof(nslq_w4a16));
    if (!h) return fail(NSLQ_ERR_ARG, "nslq_w4a16_create_awq_kn: out of host memory");
    h->N = N; h->K = K; h->gs = (int)group_size; h->G = (int)((K + group_size - 1) / group_size);
    if ((rc = w4_alloc_tables(h))) { nslq_w4a16_destroy(h); return rc; }
    if (cudaMalloc(&h->codes_owned, (size_t)(N * (K / 2))) != cudaSuccess) {
        nslq_w4a16_destroy(h);
        return fail(NSLQ_ERR_CUDA, "nslq_w4a16_create_awq_kn: cudaMalloc failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    h->codes = h->codes_owned;
    const int64_t nb = N * (K / 2);
    awq_repack_codes_kernel<<<(unsigned)((nb + 255) / 256), 256>>>(data, K, N, h->codes_owned);
    if ((rc = check_launch("awq_repack_codes_kernel"))) { nslq_w4a16_destroy(h); return rc; }
    awq_tables_kernel<<<(unsigned)((N * h->G + 255) / 256), 256>>>(scales, zeros, h->G, N, h->scale, h->zc);
    if ((rc = check_launch("awq_tables_kernel"))) { nslq_w4a16_destroy(h); return rc; }
    if ((rc = w4_transpose_tables(h))) { nslq_w4a16_destroy(h); return rc; }
    if (cudaDeviceSynchronize() != cudaSuccess) { nslq_w4a16_destroy(h); return fail(NSLQ_ERR_CUDA, "nslq_w4a16_create_awq_kn: %s", cudaGetErrorString(cudaGetLastError())); }
    *out = h;
    return NSLQ_OK;
}

int nslq_w4a16_create_qtensor_kn(const uint8_t *data, const float *scale, const uint8_t *zero_point, int64_t K, int64_t N,
                                 int granularity, int gran_axis, int64_t group_size, nslq_w4a16_t **out)
{
    if (!data || !scale || !zero_point || !out) return fail(NSLQ_ERR_ARG, "nslq_w4a16_create_qtensor_kn: null argument");
    // the forms whose scale index is constant over each run of `gs` consecutive k of a column
    int64_t gs = 0;
    if (granularity == 0 || (granularity == 1 && gran_axis == 1)) gs = (K % 128 == 0) ? 128 : K;
    else if (granularity == 2 && gran_axis == 0) gs = group_size;
    else return fail(NSLQ_ERR_UNSUPPORTED, "nslq_w4a16_create_qtensor_kn: granularity %d along axis %d has no per-(column, k-group) form", granularity, gran_axis);
    int rc = w4_check_shape("nslq_w4a16_create_qtensor_kn", N, K, gs);
    if (rc) return rc;
    if ((K * N) % 2 != 0) return fail(NSLQ_ERR_SHAPE, "nslq_w4a16_create_qtensor_kn: K*N must be even");
    nslq_w4a16 *h = (nslq_w4a16 *)calloc(1, sizeof(nslq_w4a16));
    if (!h) return fail(NSLQ_ERR_ARG, "nslq_w4a16_create_qtensor_kn: out of host memory");
    h->N = N; h->K = K; h->gs = (int)gs; h->G = (int)((K + gs - 1) / gs); h->zp_integer = 1;
    if ((rc = w4_alloc_tables(h))) { nslq_w4a16_destroy(h); return rc; }
    if (cudaMalloc(&h->codes_owned, (size_t)(N * (K / 2))) != cudaSuccess) {
        nslq_w4a16_destroy(h);
        return fail(NSLQ_ERR_CUDA, "nslq_w4a16_create_qtensor_kn: cudaMalloc failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    h->codes = h->codes_owned;
    const int64_t nb = N * (K / 2);
    awq_repack_codes_kernel<<<(unsigned)((nb + 255) / 256), 256>>>(data, K, N, h->codes_owned);   // same nibble index: row*N + col
    if ((rc = check_launch("awq_repack_codes_kernel"))) { nslq_w4a16_destroy(h); return rc; }
    qtensor_tables_kernel<<<(unsigned)((N * h->G + 255) / 256), 256>>>(scale, zero_point, granularity, N, h->G, h->scale, h->zc);
    if ((rc = check_launch("qtensor_tables_kernel"))) { nslq_w4a16_destroy(h); return rc; }
    if ((rc = w4_transpose_tables(h))) { nslq_w4a16_destroy(h); return rc; }
    if (cudaDeviceSynchronize() != cudaSuccess) { nslq_w4a16_destroy(h); return fail(NSLQ_ERR_CUDA, "nslq_w4a16_create_qtensor_kn: %s", cudaGetErrorString(cudaGetLastError())); }
    *out = h;
    return NSLQ_OK;
}

void nslq_w4a16_destroy(nslq_w4a16_t *w)
{
    if (!w) return;
    if (w->scale) cudaFree(w->scale);
    if (w->zc) cudaFree(w->zc);
    if (w->scale_t) cudaFree(w->scale_t);
    if (w->zc_t) cudaFree(w->zc_t);
    if (w->codes_owned) cudaFree(w->codes_owned);
    free(w);
}

int nslq_w4a16_forward(const nslq_w4a16_t *w, const void *x, int x_dtype, int64_t M, void *y, int y_dtype,
                       void *stream)
{
    if (!w || !x || !y) return fail(NSLQ_ERR_ARG, "nslq_w4a16_forward: null argument");
    const int es = out_elem_size(y_dtype);
    if (!es) return fail(NSLQ_ERR_ARG, "nslq_w4a16_forward: y_dtype %d not in {F32,FP16,BF16}", y_dtype);
    if (M < 0) return fail(NSLQ_ERR_SHAPE, "nslq_w4a16_forward: M=%lld", (long long)M);
    if (M == 0) return NSLQ_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (M > 16 && w4a16_gemm_supported(w->codes, x, x_dtype, M, w->N, w->K, w->gs))
        return w4a16_gemm_dispatch(w->codes, w->scale_t, w->zc_t, w->zp_integer, w->N, w->K, w->G, w->gs, x, x_dtype, M, y, y_dtype, st);
    if (w4a16_gemv_supported(w->codes, x, x_dtype, w->K, w->gs)) {
        for (int64_t m0 = 0; m0 < M; m0 += 16) {
            const int mc = (int)((M - m0) < 16 ? (M - m0) : 16);
            const void *xm = (const char *)x + m0 * w->K * 2;
            if (w4_decode_pays(mc, w->N, w->K) && w4a16_decode_supported(w->codes, xm, x_dtype, mc, w->N, w->K, w->gs)) {
                int rc = w4a16_decode_dispatch(w->codes, w->scale_t, w->zc_t, w->N, w->K, w->G, w->gs, xm, x_dtype, mc,
                                               (char *)y + m0 * w->N * es, y_dtype, st);
                if (rc) return rc;
                continue;
            }
            int rc = w4a16_gemv_dispatch(w->codes, w->scale, w->zc, w->N, w->K, w->G, w->gs,
                                         (const char *)x + m0 * w->K * 2, x_dtype, mc,
                                         (char *)y + m0 * w->N * es, y_dtype, st);
            if (rc) return rc;
        }
        return NSLQ_OK;
    }
    return w4a16_scalar_dispatch(w->codes, w->scale, w->zc, w->N, w->K, w->G, w->gs, x, x_dtype, M, y, y_dtype, st);
}

int64_t nslq_w4a16_f32x_scratch_bytes(const nslq_w4a16_t *w, int64_t M)
{
    if (!w || M <= 0) return 0;
    return align_up(3 * M * w->K * 2, 256) + align_up(3 * M * w->N * 4, 256);
}

int nslq_w4a16_forward_f32x(const nslq_w4a16_t *w, const float *x, int64_t M, void *y, int y_dtype, void *scratch,
                            int64_t scratch_bytes, void *stream)
{
    if (!w || !x || !y) return fail(NSLQ_ERR_ARG, "nslq_w4a16_forward_f32x: null argument");
    if (!out_elem_size(y_dtype)) return fail(NSLQ_ERR_ARG, "nslq_w4a16_forward_f32x: y_dtype %d not in {F32,FP16,BF16}", y_dtype);
    if (M < 0) return fail(NSLQ_ERR_SHAPE, "nslq_w4a16_forward_f32x: M=%lld", (long long)M);
    if (M == 0) return NSLQ_OK;
    const int64_t need = nslq_w4a16_f32x_scratch_bytes(w, M);
    if (!scratch || scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 255u))
        return fail(NSLQ_ERR_WORKSPACE, "nslq_w4a16_forward_f32x: scratch %lld bytes (256-byte aligned), need %lld", (long long)scratch_bytes, (long long)need);
    cudaStream_t st = (cudaStream_t)stream;
    __nv_bfloat16 *xs = (__nv_bfloat16 *)scratch;
    float *yy = (float *)((char *)scratch + align_up(3 * M * w->K * 2, 256));
    const int64_t nx = M * w->K, ny = M * w->N;
    split_f32_bf16_kernel<<<(unsigned)((nx + 255) / 256), 256, 0, st>>>(x, nx, xs);
    int rc = check_launch("split_f32_bf16_kernel");
    if (rc) return rc;
    if ((rc = nslq_w4a16_forward(w, xs, NSLQ_DTYPE_BF16, 3 * M, yy, NSLQ_DTYPE_F32, stream))) return rc;
    add_parts_kernel<<<(unsigned)((ny + 255) / 256), 256, 0, st>>>(yy, ny, y, y_dtype);
    return check_launch("add_parts_kernel");
}

int nslq_ternary_quantize_pack(const void *w, int w_dtype, int64_t numel, uint8_t *packed, float *scale, void *stream)
{
    if (!w || !packed || !scale) return fail(NSLQ_ERR_ARG, "nslq_ternary_quantize_pack: null argument");
    if (numel <= 0) return fail(NSLQ_ERR_SHAPE, "nslq_ternary_quantize_pack: numel=%lld", (long long)numel);
    if (numel % 4 != 0) return fail(NSLQ_ERR_SHAPE, "nslq_ternary_quantize_pack: numel %lld is not a multiple of 4", (long long)numel);
    return ternary_quantize_pack_dispatch(w, w_dtype, numel, packed, scale, (cudaStream_t)stream);
}

int nslq_int4_quantize_nk(const void *w, int w_dtype, int64_t N, int64_t K, int64_t group_size, uint8_t *codes,
                          float *scale, uint8_t *zero_point, void *stream)
{
    if (!w || !codes || !scale || !zero_point) return fail(NSLQ_ERR_ARG, "nslq_int4_quantize_nk: null argument");
    if (N <= 0 || K <= 0 || group_size <= 0) return fail(NSLQ_ERR_SHAPE, "nslq_int4_quantize_nk: N=%lld K=%lld group=%lld", (long long)N, (long long)K, (long long)group_size);
    if (K % 2 != 0 || group_size % 2 != 0) return fail(NSLQ_ERR_SHAPE, "nslq_int4_quantize_nk: K and group_size must be even (K=%lld group=%lld)", (long long)K, (long long)group_size);
    return int4_quantize_nk_dispatch(w, w_dtype, N, K, group_size, codes, scale, zero_point, (cudaStream_t)stream);
}

int nslq_awq_quantize_kn(const void *w, int w_dtype, int64_t K, int64_t N, int64_t group_size, uint8_t *data,
                         double *scales, double *zeros, void *stream)
{
    if (!w || !data || !scales || !zeros) return fail(NSLQ_ERR_ARG, "nslq_awq_quantize_kn: null argument");
    if (N <= 0 || K <= 0 || group_size <= 0) return fail(NSLQ_ERR_SHAPE, "nslq_awq_quantize_kn: K=%lld N=%lld group=%lld", (long long)K, (long long)N, (long long)group_size);
    if ((K * N) % 8 != 0) return fail(NSLQ_ERR_SHAPE, "nslq_awq_quantize_kn: K*N = %lld must be a multiple of 8", (long long)(K * N));
    return awq_quantize_kn_dispatch(w, w_dtype, K, N, group_size, data, scales, zeros, (cudaStream_t)stream);
}

int64_t nslq_qtensor_num_scales(const int64_t *shape, int ndim, int granularity, int axis, int64_t group_size)
{
    return qtensor_num_scales(shape, ndim, granularity, axis, group_size);
}

int nslq_qtensor_quantize(const void *src, int src_dtype, const int64_t *shape, int ndim, int dtype, int granularity, int axis,
                          int64_t group_size, uint8_t *data, float *scale, uint8_t *zero_point, void *stream)
{
    if (!src || !data || !scale || !zero_point) return fail(NSLQ_ERR_ARG, "nslq_qtensor_quantize: null argument");
    return qtensor_quantize_dispatch(src, src_dtype, shape, ndim, dtype, granularity, axis, group_size, data, scale, zero_point, (cudaStream_t)stream);
}

int nslq_qtensor_dequantize(const uint8_t *data, const float *scale, const uint8_t *zero_point, const int64_t *shape, int ndim, int dtype,
                            int granularity, int axis, int64_t group_size, void *out, int out_dtype, void *stream)
{
    if (!data || !scale || !zero_point || !out) return fail(NSLQ_ERR_ARG, "nslq_qtensor_dequantize: null argument");
    return qtensor_dequantize_dispatch(data, scale, zero_point, shape, ndim, dtype, granularity, axis, group_size, out, out_dtype, (cudaStream_t)stream);
}

int nslq_shard_rows(int64_t N, int world, int rank, int64_t *row0, int64_t *rows)
{
    if (!row0 || !rows) return fail(NSLQ_ERR_ARG, "nslq_shard_rows: null output");
    if (world <= 0 || rank < 0 || rank >= world) return fail(NSLQ_ERR_ARG, "nslq_shard_rows: rank %d of %d", rank, world);
    if (N % world != 0) return fail(NSLQ_ERR_SHAPE, "nslq_shard_rows: out_dim %lld is not divisible by world size %d", (long long)N, world);
    *rows = N / world;
    *row0 = *rows * rank;
    return NSLQ_OK;
}

}  // extern "C"
