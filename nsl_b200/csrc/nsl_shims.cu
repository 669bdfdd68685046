// Entry points with NSL's calling convention (i64 handles = pointers to NSL's #[repr(C)] structs)
// on top of the C ABI.  Host code only, plus one generic kernel for the QuantizedTensor layouts
// the streaming kernels do not take.
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <map>
#include <mutex>
#include <utility>
#include <vector>

#include "../../include/nsl_shims.h"
#include "common.cuh"

// The mirrors must have NSL's layout (field order of the Rust #[repr(C)] structs).
static_assert(offsetof(NslTensor, data) == 8 && offsetof(NslTensor, shape) == 16 && offsetof(NslTensor, strides) == 24, "NslTensor");
static_assert(offsetof(NslTensor, ndim) == 32 && offsetof(NslTensor, len) == 40 && offsetof(NslTensor, refcount) == 48, "NslTensor");
static_assert(offsetof(NslTensor, device) == 56 && offsetof(NslTensor, dtype) == 58 && offsetof(NslTensor, owns_data) == 60, "NslTensor");
static_assert(offsetof(NslTensor, data_owner) == 64 && offsetof(NslTensor, slab_managed) == 72 && offsetof(NslTensor, tape_id) == 80, "NslTensor");
static_assert(sizeof(NslTensor) == 88 && sizeof(NslQuantizedTensor) == 88 && sizeof(NslAwqPackedWeight) == 64, "struct sizes");

namespace nslq {

// y[m,n] = sum_k x[m,k] * (q[k,n] - zp[idx]) * scale[idx], QuantizedTensor [K,N] of any dtype and
// granularity (index rules of crates/nsl-runtime/src/quantize.rs:436-537), f64 accumulation.
template <typename T>
__global__ void __launch_bounds__(128)
qtensor_matmul_generic_kernel(const T *__restrict__ x, const uint8_t *__restrict__ data, const float *__restrict__ scale,
                              const uint8_t *__restrict__ zp, float *__restrict__ y, int64_t K, int64_t N, int int4,
                              int gran, int axis, int gs)
{
    const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t m = blockIdx.y;
    if (n >= N) return;
    const int64_t ngroups_k = (K + gs - 1) / gs, ngroups_n = (N + gs - 1) / gs;
    double acc = 0.0;
    for (int64_t k = 0; k < K; ++k) {
        const int64_t flat = k * N + n;
        const int q = int4 ? ((flat & 1) ? (data[flat >> 1] >> 4) : (data[flat >> 1] & 15)) : data[flat];
        int64_t si = 0;
        if (gran == 1) si = (axis == 0) ? k : n;
        else if (gran == 2) si = (axis == 0) ? (k / gs) : (k * ngroups_n + n / gs);   // axis 0: outer_size 1
        (void)ngroups_k;
        acc += (double)Elem<T>::to_f32(x[m * K + k]) * (((double)q - (double)zp[si]) * (double)scale[si]);
    }
    y[m * N + n] = (float)acc;
}

struct DeviceWeight {
    nslq_w4a16_t *w4 = nullptr;          // streaming form, when the layout allows it
    bool w4_tried = false;
    std::vector<void *> owned;            // device buffers this entry allocated
    uint8_t *qdata = nullptr; float *qscale = nullptr; uint8_t *qzp = nullptr;   // QuantizedTensor copy on the device
};

// Device copies are cached per (host object, device): the same weight may be used on several GPUs.
static std::mutex g_lock;
static std::map<std::pair<const void *, int>, DeviceWeight> g_cache;

// The stream the shims launch on: NSL launches on a per-thread compute stream
// (crates/nsl-runtime/src/cuda/mod.rs:1931-1940), so the setting is per host thread.  Default: the
// legacy default stream.
static thread_local cudaStream_t t_stream = nullptr;

// Grow-only device scratch of the calling thread, one per device (quantised activations, split fp32
// rows).  nsl_quant_reserve_cuda sizes it up front so that no forward call allocates.
struct Scratch { void *p = nullptr; size_t bytes = 0; };
static thread_local Scratch t_scratch[kMaxDevices];

static void *scratch_for(size_t bytes)
{
    Scratch &sc = t_scratch[device_index()];
    if (sc.bytes >= bytes) return sc.p;
    if (sc.p) cudaFree(sc.p);                      // synchronises the device: reserve up front to avoid it
    sc.p = nullptr; sc.bytes = 0;
    const size_t want = (bytes + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
    if (cudaMalloc(&sc.p, want) != cudaSuccess) { sc.p = nullptr; return nullptr; }
    sc.bytes = want;
    return sc.p;
}

// Makes the tensor's device current for the duration of a call and puts the caller's back.
struct DeviceScope {
    int prev = 0, dev = 0;
    bool ok = false;
    DeviceScope(const NslTensor *t, const char *who)
    {
        if (t->device == 0) { fprintf(stderr, "%s: tensor is on the CPU; this entry point is the CUDA arm\n", who); return; }
        dev = (int)t->device - 1;
        cudaGetDevice(&prev);
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) { fprintf(stderr, "%s: cannot select CUDA device %d\n", who, dev); return; }
        ok = true;
    }
    ~DeviceScope() { if (ok && prev != dev) cudaSetDevice(prev); }
};

static void *upload(DeviceWeight &d, const void *host, size_t bytes)
{
    void *p = nullptr;
    if (cudaMalloc(&p, bytes ? bytes : 1) != cudaSuccess) return nullptr;
    if (bytes && cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice) != cudaSuccess) { cudaFree(p); return nullptr; }
    d.owned.push_back(p);
    return p;
}

static void release(DeviceWeight &d)
{
    if (d.w4) nslq_w4a16_destroy(d.w4);
    for (void *p : d.owned) cudaFree(p);
    d = DeviceWeight();
}

// x [M,K] of any float dtype through the streaming W4A16 kernels (fp32 x: split into three bf16 parts).
static int w4_forward_any(const nslq_w4a16_t *h, const NslTensor *x, int64_t M, NslTensor *y)
{
    if (x->dtype == NSLQ_DTYPE_F32) {
        const int64_t need = nslq_w4a16_f32x_scratch_bytes(h, M);
        void *sc = scratch_for((size_t)need);
        if (!sc) return fail(NSLQ_ERR_CUDA, "cannot allocate %lld bytes of scratch", (long long)need);
        return nslq_w4a16_forward_f32x(h, (const float *)x->data, M, y->data, (int)y->dtype, sc, need, t_stream);
    }
    return nslq_w4a16_forward(h, x->data, (int)x->dtype, M, y->data, (int)y->dtype, t_stream);
}

__global__ void scale_columns_kernel(const float *__restrict__ w, const float *__restrict__ s, int64_t total, int64_t n,
                                     float *__restrict__ out)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = __fmul_rn(w[i], s[i % n]);
}

}  // namespace nslq

using namespace nslq;

extern "C" {

void nsl_quant_set_stream_cuda(int64_t stream) { t_stream = reinterpret_cast<cudaStream_t>(stream); }

int64_t nsl_quant_reserve_cuda(int64_t bytes)
{
    if (bytes <= 0) return 0;
    return scratch_for((size_t)bytes) ? bytes : 0;
}

int64_t nsl_awq_matmul_cuda(int64_t input, int64_t packed, int64_t /*group_size*/, int64_t out)
{
    if (input == 0 || packed == 0 || out == 0) { fprintf(stderr, "nsl_awq_matmul: null pointer\n"); return 0; }
    const NslTensor *x = reinterpret_cast<const NslTensor *>(input);
    NslTensor *y = reinterpret_cast<NslTensor *>(out);
    const NslAwqPackedWeight *pw = reinterpret_cast<const NslAwqPackedWeight *>(packed);
    DeviceScope scope(x, "nsl_awq_matmul");
    if (!scope.ok || y->device != x->device) { if (scope.ok) fprintf(stderr, "nsl_awq_matmul: input and out are on different devices\n"); return 0; }
    const int64_t M = x->shape[0];                       // the original reads shape[0] only (awq.rs:270)
    nslq_w4a16_t *h = nullptr;
    {
        std::lock_guard<std::mutex> hold(g_lock);
        DeviceWeight &d = g_cache[std::make_pair((const void *)pw, scope.dev)];
        if (!d.w4) {
            const size_t nb = (size_t)((pw->k * pw->n + 1) / 2), nt = (size_t)(pw->num_groups * pw->n) * sizeof(double);
            void *dd = upload(d, pw->data, nb), *ds = upload(d, pw->scales, nt), *dz = upload(d, pw->zeros, nt);
            if (!dd || !ds || !dz ||
                nslq_w4a16_create_awq_kn((const uint8_t *)dd, (const double *)ds, (const double *)dz, pw->k, pw->n,
                                         pw->group_size, &d.w4) != NSLQ_OK) {
                fprintf(stderr, "nsl_awq_matmul: cannot stage the weight on the device: %s\n", nslq_last_error());
                release(d);
                g_cache.erase(std::make_pair((const void *)pw, scope.dev));
                return 0;
            }
            for (void *p : d.owned) cudaFree(p);         // create_awq_kn made its own re-laid-out copy
            d.owned.clear();
        }
        h = d.w4;
    }
    if (w4_forward_any(h, x, M, y) != NSLQ_OK) {
        fprintf(stderr, "nsl_awq_matmul: %s\n", nslq_last_error());
        return 0;
    }
    return out;
}

int64_t nsl_gptq_matmul_cuda(int64_t input, int64_t packed, int64_t group_size, int64_t /*bits*/, int64_t out)
{
    return nsl_awq_matmul_cuda(input, packed, group_size, out);
}

int64_t nsl_qtensor_matmul_mixed_cuda(int64_t x_ptr, int64_t qw_ptr, int64_t out)
{
    const NslQuantizedTensor *qw = reinterpret_cast<const NslQuantizedTensor *>(qw_ptr);
    if (qw->ndim != 2) {
        fprintf(stderr, "nsl: nsl_qtensor_matmul_mixed: quantized weight must be 2D, got %lldD\n", (long long)qw->ndim);
        abort();
    }
    const NslTensor *x = reinterpret_cast<const NslTensor *>(x_ptr);
    NslTensor *y = reinterpret_cast<NslTensor *>(out);
    if (x->ndim <= 0) { fprintf(stderr, "nsl: nsl_qtensor_matmul_mixed: x must be at least 1D\n"); abort(); }
    const int64_t K = qw->shape[0], N = qw->shape[1], x_last = x->shape[x->ndim - 1];
    if (x_last != K) {
        fprintf(stderr, "nsl: nsl_qtensor_matmul_mixed: x last dim (%lld) != qw dim 0 (%lld)\n", (long long)x_last, (long long)K);
        abort();
    }
    if (qw->dtype != 0 && qw->dtype != 1) { fprintf(stderr, "nsl: unknown quantization dtype %lld\n", (long long)qw->dtype); abort(); }
    DeviceScope scope(x, "nsl_qtensor_matmul_mixed");
    if (!scope.ok || y->device != x->device) { if (scope.ok) fprintf(stderr, "nsl_qtensor_matmul_mixed: x and out are on different devices\n"); return 0; }
    const int64_t M = x->len / K;
    const int gs = qw->group_size > 0 ? (int)qw->group_size : 1;
    DeviceWeight *d = nullptr;
    nslq_w4a16_t *w4 = nullptr;
    {
        std::lock_guard<std::mutex> hold(g_lock);
        d = &g_cache[std::make_pair((const void *)qw, scope.dev)];
        if (!d->qdata) {
            const size_t total = (size_t)(K * N), nb = qw->dtype == 1 ? (total + 1) / 2 : total;
            d->qdata = (uint8_t *)upload(*d, qw->data, nb);
            d->qscale = (float *)upload(*d, qw->scale, (size_t)qw->num_scales * sizeof(float));
            d->qzp = (uint8_t *)upload(*d, qw->zero_point, (size_t)qw->num_scales);
            if (!d->qdata || !d->qscale || !d->qzp) {
                fprintf(stderr, "nsl_qtensor_matmul_mixed: cannot stage the weight on the device\n");
                release(*d);
                g_cache.erase(std::make_pair((const void *)qw, scope.dev));
                return 0;
            }
        }
        // INT4 weights whose scale does not change along k inside a group are re-laid out once into the
        // [N,K] streaming order and multiplied by the W4A16 kernels; everything else keeps the generic kernel.
        if (!d->w4_tried && qw->dtype == 1 && K % 64 == 0) {
            d->w4_tried = true;
            const bool per_group_k = qw->granularity == 2 && qw->gran_axis == 0 && gs % 128 == 0;
            if (qw->granularity == 0 || (qw->granularity == 1 && qw->gran_axis == 1) || per_group_k) {
                if (nslq_w4a16_create_qtensor_kn(d->qdata, d->qscale, d->qzp, K, N, (int)qw->granularity, (int)qw->gran_axis, gs, &d->w4) != NSLQ_OK)
                    d->w4 = nullptr;
            }
        }
        w4 = d->w4;
    }
    if (w4 && (x->dtype == NSLQ_DTYPE_F32 || x->dtype == NSLQ_DTYPE_BF16 || x->dtype == NSLQ_DTYPE_FP16)) {
        if (w4_forward_any(w4, x, M, y) != NSLQ_OK) {
            fprintf(stderr, "nsl_qtensor_matmul_mixed: %s\n", nslq_last_error());
            return 0;
        }
        return out;
    }
    if (M > 65535 || y->dtype != NSLQ_DTYPE_F32) {
        fprintf(stderr, "nsl_qtensor_matmul_mixed: out must be f32 and M <= 65535 on this path\n");
        return 0;
    }
    dim3 grid((unsigned)((N + 127) / 128), (unsigned)M);
#define NSLQ_LAUNCH_GENERIC(T) qtensor_matmul_generic_kernel<T><<<grid, 128, 0, t_stream>>>((const T *)x->data, d->qdata, d->qscale, d->qzp, \
        (float *)y->data, K, N, qw->dtype == 1, (int)qw->granularity, (int)qw->gran_axis, gs)
    switch (x->dtype) {
    case NSLQ_DTYPE_F32: NSLQ_LAUNCH_GENERIC(float); break;
    case NSLQ_DTYPE_FP16: NSLQ_LAUNCH_GENERIC(__half); break;
    case NSLQ_DTYPE_BF16: NSLQ_LAUNCH_GENERIC(__nv_bfloat16); break;
    default: fprintf(stderr, "nsl_qtensor_matmul_mixed: x dtype %d is not a GPU float type\n", (int)x->dtype); return 0;
    }
#undef NSLQ_LAUNCH_GENERIC
    if (cudaGetLastError() != cudaSuccess) { fprintf(stderr, "nsl_qtensor_matmul_mixed: launch failed\n"); return 0; }
    return out;
}

void nsl_quant_forget_cuda(int64_t weight)
{
    std::lock_guard<std::mutex> hold(g_lock);
    const void *key = reinterpret_cast<const void *>(weight);
    for (auto it = g_cache.lower_bound(std::make_pair(key, 0)); it != g_cache.end() && it->first.first == key;) {
        int prev = 0;
        cudaGetDevice(&prev);
        if (prev != it->first.second) cudaSetDevice(it->first.second);
        release(it->second);
        if (prev != it->first.second) cudaSetDevice(prev);
        it = g_cache.erase(it);
    }
}

int64_t nsl_awq_pre_scale_weight_cuda(int64_t weight_ptr, int64_t scales_ptr, int64_t scales_len, double alpha, int64_t out)
{
    if (weight_ptr == 0 || out == 0) { fprintf(stderr, "nsl_awq_pre_scale_weight: null weight tensor\n"); return 0; }
    const NslTensor *t = reinterpret_cast<const NslTensor *>(weight_ptr);
    NslTensor *y = reinterpret_cast<NslTensor *>(out);
    if (t->ndim < 2) { fprintf(stderr, "nsl_awq_pre_scale_weight: weight must be 2D (got %lldD)\n", (long long)t->ndim); return 0; }
    DeviceScope scope(t, "nsl_awq_pre_scale_weight");
    if (!scope.ok || y->device != t->device) return 0;
    if (t->dtype != NSLQ_DTYPE_F32 || y->dtype != NSLQ_DTYPE_F32) {
        fprintf(stderr, "nsl_awq_pre_scale_weight: the CUDA arm takes f32 tensors (GPU tensors are f32 in NSL)\n");
        return 0;
    }
    const int64_t n = t->shape[1], total = t->len;
    if (scales_ptr == 0 || scales_len != n) {            // no scaling: a plain copy, as the original does
        if (cudaMemcpyAsync(y->data, t->data, (size_t)total * 4, cudaMemcpyDeviceToDevice, t_stream) != cudaSuccess) return 0;
        return out;
    }
    // scales[col]^alpha in f32 on the host, with the same libm powf the original calls; the device multiplies
    const float *hs = reinterpret_cast<const float *>(scales_ptr);
    std::vector<float> s((size_t)n);
    const float a = (float)alpha;
    for (int64_t c = 0; c < n; ++c) s[(size_t)c] = powf(hs[c], a);
    float *ds = (float *)scratch_for((size_t)n * 4);
    if (!ds || cudaMemcpyAsync(ds, s.data(), (size_t)n * 4, cudaMemcpyHostToDevice, t_stream) != cudaSuccess ||
        cudaStreamSynchronize(t_stream) != cudaSuccess) {     // `s` is pageable host memory that dies with this call
        fprintf(stderr, "nsl_awq_pre_scale_weight: cannot stage the column factors\n");
        return 0;
    }
    scale_columns_kernel<<<(unsigned)((total + 255) / 256), 256, 0, t_stream>>>((const float *)t->data, ds, total, n, (float *)y->data);
    if (cudaGetLastError() != cudaSuccess) { fprintf(stderr, "nsl_awq_pre_scale_weight: launch failed\n"); return 0; }
    if (cudaStreamSynchronize(t_stream) != cudaSuccess) return 0;      // the scratch may be reused by the next call
    return out;
}

// ---------------------------------------------------------------- load-time quantisers
// The host objects (QuantizedTensor, AwqPackedWeight) keep their buffers in host memory, as the originals do; the
// tensor to quantise is on the device, the arithmetic runs there and the bytes come back.  Load-time calls: they
// allocate and synchronise.
int64_t nsl_qtensor_quantize_cuda(int64_t tensor_ptr, int64_t qt_ptr)
{
    if (tensor_ptr == 0 || qt_ptr == 0) { fprintf(stderr, "nsl_qtensor_quantize: null argument\n"); return 0; }
    const NslTensor *t = reinterpret_cast<const NslTensor *>(tensor_ptr);
    NslQuantizedTensor *q = reinterpret_cast<NslQuantizedTensor *>(qt_ptr);
    DeviceScope scope(t, "nsl_qtensor_quantize");
    if (!scope.ok) return 0;
    if (t->dtype != NSLQ_DTYPE_F32 && t->dtype != NSLQ_DTYPE_F64) { fprintf(stderr, "nsl_qtensor_quantize: f32 or f64 tensors only\n"); return 0; }
    if (q->ndim != t->ndim) { fprintf(stderr, "nsl_qtensor_quantize: the QuantizedTensor was allocated for another shape\n"); return 0; }
    int64_t total = 1;
    for (int64_t d = 0; d < t->ndim; ++d) {
        if (q->shape[d] != t->shape[d]) { fprintf(stderr, "nsl_qtensor_quantize: the QuantizedTensor was allocated for another shape\n"); return 0; }
        total *= t->shape[d];
    }
    const int64_t ns = nslq_qtensor_num_scales(t->shape, (int)t->ndim, (int)q->granularity, (int)q->gran_axis, q->group_size);
    if (ns < 0 || ns != q->num_scales) { fprintf(stderr, "nsl_qtensor_quantize: %s\n", ns < 0 ? nslq_last_error() : "num_scales does not match the granularity"); return 0; }
    const size_t data_bytes = (size_t)(q->dtype == 1 ? (total + 1) / 2 : total);
    const size_t off_scale = (data_bytes + 255) & ~(size_t)255, off_zp = off_scale + (((size_t)ns * 4 + 255) & ~(size_t)255);
    uint8_t *sc = (uint8_t *)scratch_for(off_zp + (size_t)ns);
    if (!sc) { fprintf(stderr, "nsl_qtensor_quantize: cannot allocate device scratch\n"); return 0; }
    if (nslq_qtensor_quantize(t->data, (int)t->dtype, t->shape, (int)t->ndim, (int)q->dtype, (int)q->granularity, (int)q->gran_axis,
                              q->group_size, sc, (float *)(sc + off_scale), sc + off_zp, t_stream) != NSLQ_OK) {
        fprintf(stderr, "nsl_qtensor_quantize: %s\n", nslq_last_error());
        return 0;
    }
    if (cudaMemcpy(q->data, sc, data_bytes, cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(q->scale, sc + off_scale, (size_t)ns * 4, cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(q->zero_point, sc + off_zp, (size_t)ns, cudaMemcpyDeviceToHost) != cudaSuccess) {
        fprintf(stderr, "nsl_qtensor_quantize: copy to the host failed\n");
        return 0;
    }
    return qt_ptr;
}

int64_t nsl_qtensor_dequantize_cuda(int64_t qt_ptr, int64_t out)
{
    if (qt_ptr == 0 || out == 0) { fprintf(stderr, "nsl_qtensor_dequantize: null argument\n"); return 0; }
    const NslQuantizedTensor *q = reinterpret_cast<const NslQuantizedTensor *>(qt_ptr);
    NslTensor *y = reinterpret_cast<NslTensor *>(out);
    DeviceScope scope(y, "nsl_qtensor_dequantize");
    if (!scope.ok) return 0;
    if (y->dtype != NSLQ_DTYPE_F32 && y->dtype != NSLQ_DTYPE_F64) { fprintf(stderr, "nsl_qtensor_dequantize: f32 or f64 output only\n"); return 0; }
    int64_t total = 1;
    for (int64_t d = 0; d < q->ndim; ++d) total *= q->shape[d];
    if (y->len != total) { fprintf(stderr, "nsl_qtensor_dequantize: output of %lld elements for a tensor of %lld\n", (long long)y->len, (long long)total); return 0; }
    const int64_t ns = q->num_scales;
    const size_t data_bytes = (size_t)(q->dtype == 1 ? (total + 1) / 2 : total);
    const size_t off_scale = (data_bytes + 255) & ~(size_t)255, off_zp = off_scale + (((size_t)ns * 4 + 255) & ~(size_t)255);
    uint8_t *sc = (uint8_t *)scratch_for(off_zp + (size_t)ns);
    if (!sc || cudaMemcpyAsync(sc, q->data, data_bytes, cudaMemcpyHostToDevice, t_stream) != cudaSuccess ||
        cudaMemcpyAsync(sc + off_scale, q->scale, (size_t)ns * 4, cudaMemcpyHostToDevice, t_stream) != cudaSuccess ||
        cudaMemcpyAsync(sc + off_zp, q->zero_point, (size_t)ns, cudaMemcpyHostToDevice, t_stream) != cudaSuccess) {
        fprintf(stderr, "nsl_qtensor_dequantize: cannot stage the quantized tensor on the device\n");
        return 0;
    }
    if (nslq_qtensor_dequantize(sc, (const float *)(sc + off_scale), sc + off_zp, q->shape, (int)q->ndim, (int)q->dtype, (int)q->granularity,
                                (int)q->gran_axis, q->group_size, y->data, (int)y->dtype, t_stream) != NSLQ_OK) {
        fprintf(stderr, "nsl_qtensor_dequantize: %s\n", nslq_last_error());
        return 0;
    }
    if (cudaStreamSynchronize(t_stream) != cudaSuccess) return 0;      // the scratch may be reused by the next call
    return out;
}

int64_t nsl_awq_quantize_cuda(int64_t weight_ptr, int64_t group_size, int64_t packed_out)
{
    if (weight_ptr == 0 || packed_out == 0) { fprintf(stderr, "nsl_awq_quantize: null argument\n"); return 0; }
    const NslTensor *t = reinterpret_cast<const NslTensor *>(weight_ptr);
    NslAwqPackedWeight *pw = reinterpret_cast<NslAwqPackedWeight *>(packed_out);
    if (t->ndim != 2) { fprintf(stderr, "nsl_awq_quantize: weight must be 2D (got %lldD)\n", (long long)t->ndim); return 0; }
    DeviceScope scope(t, "nsl_awq_quantize");
    if (!scope.ok) return 0;
    const int64_t K = t->shape[0], N = t->shape[1];
    if (group_size <= 0 || pw->k != K || pw->n != N || pw->group_size != group_size || pw->num_groups != (K + group_size - 1) / group_size) {
        fprintf(stderr, "nsl_awq_quantize: the AwqPackedWeight was allocated for another shape or group size\n");
        return 0;
    }
    if (t->dtype != NSLQ_DTYPE_F32 && t->dtype != NSLQ_DTYPE_F64) { fprintf(stderr, "nsl_awq_quantize: f32 or f64 weights only\n"); return 0; }
    const size_t data_bytes = (size_t)((K * N + 1) / 2), tab = (size_t)pw->num_groups * (size_t)N * 8;
    const size_t off_s = (data_bytes + 255) & ~(size_t)255, off_z = off_s + ((tab + 255) & ~(size_t)255);
    uint8_t *sc = (uint8_t *)scratch_for(off_z + tab);
    if (!sc) { fprintf(stderr, "nsl_awq_quantize: cannot allocate device scratch\n"); return 0; }
    if (nslq_awq_quantize_kn(t->data, (int)t->dtype, K, N, group_size, sc, (double *)(sc + off_s), (double *)(sc + off_z), t_stream) != NSLQ_OK) {
        fprintf(stderr, "nsl_awq_quantize: %s\n", nslq_last_error());
        return 0;
    }
    if (cudaStreamSynchronize(t_stream) != cudaSuccess || cudaMemcpy(pw->data, sc, data_bytes, cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(pw->scales, sc + off_s, tab, cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(pw->zeros, sc + off_z, tab, cudaMemcpyDeviceToHost) != cudaSuccess) {
        fprintf(stderr, "nsl_awq_quantize: copy to the host failed\n");
        return 0;
    }
    return packed_out;
}

// ---------------------------------------------------------------- BitLinear trio
struct NslBitlinearHandle {
    nslq_bitlinear_t *w;
    uint8_t *packed_dev;
    int64_t N, K;
    int device;
};

int64_t nsl_bitlinear_pack(int64_t packed_bytes, int64_t out_dim, int64_t hidden_dim, double weight_scale)
{
    if (packed_bytes == 0) { fprintf(stderr, "nsl_bitlinear_pack: null pointer\n"); return 0; }
    if (out_dim <= 0 || hidden_dim <= 0 || hidden_dim % 4 != 0) {
        fprintf(stderr, "nsl_bitlinear_pack: hidden_dim %lld must be a positive multiple of 4\n", (long long)hidden_dim);
        return 0;
    }
    // The reference's packed representation has no code 0b11 (try_unpack_byte, bitnet/pack.rs:60-67):
    // refuse such bytes here, on the host copy, before anything reaches the device.
    const uint8_t *src = reinterpret_cast<const uint8_t *>(packed_bytes);
    const size_t nb = (size_t)(out_dim * hidden_dim / 4);
    for (size_t i = 0; i < nb; ++i) {
        const unsigned b = src[i];
        if (((b & (b >> 1)) & 0x55u) != 0) {
            fprintf(stderr, "nsl_bitlinear_pack: byte %zu (0x%02X) holds the reserved 2-bit code 0b11\n", i, b);
            return 0;
        }
    }
    NslBitlinearHandle *h = new NslBitlinearHandle();
    cudaGetDevice(&h->device);
    if (cudaMalloc((void **)&h->packed_dev, nb) != cudaSuccess ||
        cudaMemcpy(h->packed_dev, src, nb, cudaMemcpyHostToDevice) != cudaSuccess ||
        nslq_bitlinear_create(h->packed_dev, out_dim, hidden_dim, (float)weight_scale, &h->w) != NSLQ_OK) {
        fprintf(stderr, "nsl_bitlinear_pack: cannot stage the weight on the device\n");
        if (h->packed_dev) cudaFree(h->packed_dev);
        delete h;
        return 0;
    }
    h->N = out_dim; h->K = hidden_dim;
    return reinterpret_cast<int64_t>(h);
}

int64_t nsl_bitlinear_forward(int64_t handle, int64_t x_ptr, int64_t out)
{
    if (handle == 0 || x_ptr == 0 || out == 0) { fprintf(stderr, "nsl_bitlinear_forward: null pointer\n"); return 0; }
    NslBitlinearHandle *h = reinterpret_cast<NslBitlinearHandle *>(handle);
    const NslTensor *x = reinterpret_cast<const NslTensor *>(x_ptr);
    NslTensor *y = reinterpret_cast<NslTensor *>(out);
    DeviceScope scope(x, "nsl_bitlinear_forward");
    if (!scope.ok || y->device != x->device) return 0;
    if (scope.dev != h->device) {
        fprintf(stderr, "nsl_bitlinear_forward: the weight was packed on CUDA device %d, x is on device %d\n", h->device, scope.dev);
        return 0;
    }
    if (x->ndim < 1 || x->shape[x->ndim - 1] != h->K) {
        fprintf(stderr, "nsl: nsl_bitlinear_forward: x last dim != hidden_dim (%lld)\n", (long long)h->K);
        abort();
    }
    const int64_t M = x->len / h->K;
    const int64_t need = nslq_bitlinear_workspace_bytes(M, h->K);
    int rc;
    if (need <= nslq_noalloc_scratch_bytes()) {
        // decode-sized calls use the area inside the library image: nothing is allocated, ever
        rc = nslq_bitlinear_forward_noalloc(h->w, x->data, (int)x->dtype, M, y->data, (int)y->dtype, t_stream);
    } else {
        // larger batches use the calling thread's scratch; nsl_quant_reserve_cuda sizes it up front,
        // otherwise it grows here (an allocation, hence a device synchronisation, on that call only)
        void *ws = scratch_for((size_t)need);
        if (!ws) { fprintf(stderr, "nsl_bitlinear_forward: cannot allocate %lld bytes of scratch\n", (long long)need); return 0; }
        rc = nslq_bitlinear_forward(h->w, x->data, (int)x->dtype, M, y->data, (int)y->dtype, nullptr, nullptr, nullptr, ws, need, t_stream);
    }
    if (rc != NSLQ_OK) {
        fprintf(stderr, "nsl_bitlinear_forward: %s\n", nslq_last_error());
        return 0;
    }
    return out;
}

void nsl_bitlinear_free(int64_t handle)
{
    if (handle == 0) return;
    NslBitlinearHandle *h = reinterpret_cast<NslBitlinearHandle *>(handle);
    int prev = 0;
    cudaGetDevice(&prev);
    if (prev != h->device) cudaSetDevice(h->device);
    nslq_bitlinear_destroy(h->w);
    if (h->packed_dev) cudaFree(h->packed_dev);
    if (prev != h->device) cudaSetDevice(prev);
    delete h;
}

}  // extern "C"
