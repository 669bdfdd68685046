// Entry points with NSL's calling convention (i64 handles = pointers to NSL's #[repr(C)] structs)
// on top of the C ABI.  Host code only, plus one generic kernel for the QuantizedTensor layouts
// the streaming kernels do not take.
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <unordered_map>
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
    nslq_bitlinear_t *bl = nullptr;
    std::vector<void *> owned;            // device buffers this entry allocated
    uint8_t *qdata = nullptr; float *qscale = nullptr; uint8_t *qzp = nullptr;   // generic QuantizedTensor copy
};

static std::mutex g_lock;
static std::unordered_map<const void *, DeviceWeight> g_cache;

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
    if (d.bl) nslq_bitlinear_destroy(d.bl);
    for (void *p : d.owned) cudaFree(p);
    d = DeviceWeight();
}

static bool tensor_on_gpu(const NslTensor *t, const char *who)
{
    if (t->device == 0) {
        fprintf(stderr, "%s: tensor is on the CPU; this entry point is the CUDA arm\n", who);
        return false;
    }
    cudaSetDevice((int)t->device - 1);
    return true;
}

}  // namespace nslq

using namespace nslq;

extern "C" {

int64_t nsl_awq_matmul_cuda(int64_t input, int64_t packed, int64_t /*group_size*/, int64_t out)
{
    if (input == 0 || packed == 0 || out == 0) { fprintf(stderr, "nsl_awq_matmul: null pointer\n"); return 0; }
    const NslTensor *x = reinterpret_cast<const NslTensor *>(input);
    NslTensor *y = reinterpret_cast<NslTensor *>(out);
    const NslAwqPackedWeight *pw = reinterpret_cast<const NslAwqPackedWeight *>(packed);
    if (!tensor_on_gpu(x, "nsl_awq_matmul") || !tensor_on_gpu(y, "nsl_awq_matmul")) return 0;
    const int64_t M = x->shape[0];                       // the original reads shape[0] only (awq.rs:270)
    nslq_w4a16_t *h = nullptr;
    {
        std::lock_guard<std::mutex> hold(g_lock);
        DeviceWeight &d = g_cache[pw];
        if (!d.w4) {
            const size_t nb = (size_t)((pw->k * pw->n + 1) / 2), nt = (size_t)(pw->num_groups * pw->n) * sizeof(double);
            void *dd = upload(d, pw->data, nb), *ds = upload(d, pw->scales, nt), *dz = upload(d, pw->zeros, nt);
            if (!dd || !ds || !dz ||
                nslq_w4a16_create_awq_kn((const uint8_t *)dd, (const double *)ds, (const double *)dz, pw->k, pw->n,
                                         pw->group_size, &d.w4) != NSLQ_OK) {
                fprintf(stderr, "nsl_awq_matmul: cannot stage the weight on the device: %s\n", nslq_last_error());
                release(d);
                g_cache.erase(pw);
                return 0;
            }
            for (void *p : d.owned) cudaFree(p);         // create_awq_kn made its own re-laid-out copy
            d.owned.clear();
        }
        h = d.w4;
    }
    if (nslq_w4a16_forward(h, x->data, (int)x->dtype, M, y->data, (int)y->dtype, nullptr) != NSLQ_OK) {
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
    if (!tensor_on_gpu(x, "nsl_qtensor_matmul_mixed") || !tensor_on_gpu(y, "nsl_qtensor_matmul_mixed")) return 0;
    const int64_t M = x->len / K;
    DeviceWeight *d = nullptr;
    {
        std::lock_guard<std::mutex> hold(g_lock);
        d = &g_cache[qw];
        if (!d->qdata) {
            const size_t total = (size_t)(K * N), nb = qw->dtype == 1 ? (total + 1) / 2 : total;
            d->qdata = (uint8_t *)upload(*d, qw->data, nb);
            d->qscale = (float *)upload(*d, qw->scale, (size_t)qw->num_scales * sizeof(float));
            d->qzp = (uint8_t *)upload(*d, qw->zero_point, (size_t)qw->num_scales);
            if (!d->qdata || !d->qscale || !d->qzp) {
                fprintf(stderr, "nsl_qtensor_matmul_mixed: cannot stage the weight on the device\n");
                release(*d);
                g_cache.erase(qw);
                return 0;
            }
        }
    }
    if (M > 65535 || y->dtype != NSLQ_DTYPE_F32) {
        fprintf(stderr, "nsl_qtensor_matmul_mixed: out must be f32 and M <= 65535 on this path\n");
        return 0;
    }
    dim3 grid((unsigned)((N + 127) / 128), (unsigned)M);
    const int gs = qw->group_size > 0 ? (int)qw->group_size : 1;
#define NSLQ_LAUNCH_GENERIC(T) qtensor_matmul_generic_kernel<T><<<grid, 128>>>((const T *)x->data, d->qdata, d->qscale, d->qzp, \
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
    auto it = g_cache.find(reinterpret_cast<const void *>(weight));
    if (it == g_cache.end()) return;
    release(it->second);
    g_cache.erase(it);
}

// ---------------------------------------------------------------- BitLinear trio
struct NslBitlinearHandle {
    nslq_bitlinear_t *w;
    uint8_t *packed_dev;
    void *workspace;
    int64_t workspace_bytes, N, K;
};

int64_t nsl_bitlinear_pack(int64_t packed_bytes, int64_t out_dim, int64_t hidden_dim, double weight_scale)
{
    if (packed_bytes == 0) { fprintf(stderr, "nsl_bitlinear_pack: null pointer\n"); return 0; }
    if (out_dim <= 0 || hidden_dim <= 0 || hidden_dim % 4 != 0) {
        fprintf(stderr, "nsl_bitlinear_pack: hidden_dim %lld must be a positive multiple of 4\n", (long long)hidden_dim);
        return 0;
    }
    NslBitlinearHandle *h = new NslBitlinearHandle();
    const size_t nb = (size_t)(out_dim * hidden_dim / 4);
    if (cudaMalloc((void **)&h->packed_dev, nb) != cudaSuccess ||
        cudaMemcpy(h->packed_dev, reinterpret_cast<const void *>(packed_bytes), nb, cudaMemcpyHostToDevice) != cudaSuccess ||
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
    if (!tensor_on_gpu(x, "nsl_bitlinear_forward") || !tensor_on_gpu(y, "nsl_bitlinear_forward")) return 0;
    if (x->ndim < 1 || x->shape[x->ndim - 1] != h->K) {
        fprintf(stderr, "nsl: nsl_bitlinear_forward: x last dim != hidden_dim (%lld)\n", (long long)h->K);
        abort();
    }
    const int64_t M = x->len / h->K;
    const int64_t need = nslq_bitlinear_workspace_bytes(M, h->K);
    if (need > h->workspace_bytes) {                     // grows monotonically; a runtime with its own allocator passes
        if (h->workspace) cudaFree(h->workspace);        // a workspace through nslq_bitlinear_forward instead
        if (cudaMalloc(&h->workspace, (size_t)need) != cudaSuccess) { h->workspace = nullptr; h->workspace_bytes = 0; return 0; }
        h->workspace_bytes = need;
    }
    if (nslq_bitlinear_forward(h->w, x->data, (int)x->dtype, M, y->data, (int)y->dtype, nullptr, nullptr, nullptr,
                               h->workspace, h->workspace_bytes, nullptr) != NSLQ_OK) {
        fprintf(stderr, "nsl_bitlinear_forward: %s\n", nslq_last_error());
        return 0;
    }
    return out;
}

void nsl_bitlinear_free(int64_t handle)
{
    if (handle == 0) return;
    NslBitlinearHandle *h = reinterpret_cast<NslBitlinearHandle *>(handle);
    nslq_bitlinear_destroy(h->w);
    if (h->packed_dev) cudaFree(h->packed_dev);
    if (h->workspace) cudaFree(h->workspace);
    delete h;
}

}  // extern "C"
