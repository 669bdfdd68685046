// BitLinear forward for callers that must not allocate device memory.
//
// nslq_bitlinear_forward needs a scratch buffer (quantised activations, scales,
// row sums) and expects the caller to bring one.  Some hosts cannot: NSL's runtime
// hands out all device memory through its own caching allocator and frees it on
// its own schedule, so a foreign library has no buffer it may keep; a latency-bound
// decode loop cannot afford cudaMalloc's device-wide synchronisation; a plug-in
// loaded late may find the device already fully reserved.  For them this file
// keeps one fixed scratch area in the library's own device image and runs the very
// same kernels on it.  Nothing here calls cudaMalloc, cudaFree or any routine that
// allocates.
#include <mutex>

#include "common.cuh"

// The scratch itself: part of the loaded module, so every GPU that loads the
// library holds these bytes from load until the process exits.
#define NSLQ_NOALLOC_SCRATCH_BYTES (512 * 1024)
static __device__ __align__(256) unsigned char g_noalloc_scratch[NSLQ_NOALLOC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_setup_lock;
void *g_scratch_addr[kMaxDevices] = {nullptr};

// In host code `g_noalloc_scratch` is only a handle for the symbol, not an address
// a kernel could use; the device address has to be asked for, once per device,
// while that device is current.
int scratch_for_current_device(void **out)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return nslq::fail(NSLQ_ERR_CUDA, "nslq_bitlinear_forward_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices)
        return nslq::fail(NSLQ_ERR_UNSUPPORTED, "nslq_bitlinear_forward_noalloc: device index %d is beyond the %d this entry point tracks", dev, kMaxDevices);
    std::lock_guard<std::mutex> hold(g_setup_lock);
    if (!g_scratch_addr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return nslq::fail(NSLQ_ERR_CUDA, "nslq_bitlinear_forward_noalloc: cudaGetSymbolAddress on device %d: %s", dev, cudaGetErrorString(e));
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return NSLQ_OK;
}

}  // namespace

extern "C" {

int64_t nslq_noalloc_scratch_bytes(void) { return NSLQ_NOALLOC_SCRATCH_BYTES; }

int nslq_bitlinear_forward_noalloc(const nslq_bitlinear_t *w, const void *x, int x_dtype, int64_t M, void *y,
                                   int y_dtype, void *stream)
{
    if (!w || !x || !y) return nslq::fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward_noalloc: null argument");
    if (M < 0) return nslq::fail(NSLQ_ERR_SHAPE, "nslq_bitlinear_forward_noalloc: M=%lld", (long long)M);
    const int64_t need = nslq_bitlinear_workspace_bytes(M, w->K);
    if (need > NSLQ_NOALLOC_SCRATCH_BYTES)
        return nslq::fail(NSLQ_ERR_WORKSPACE,
                          "nslq_bitlinear_forward_noalloc: M=%lld tokens of width K=%lld need %lld bytes of scratch, the built-in "
                          "area holds %d; use nslq_bitlinear_forward with a workspace of your own for this size",
                          (long long)M, (long long)w->K, (long long)need, NSLQ_NOALLOC_SCRATCH_BYTES);
    void *scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    // Every byte the kernels read from the scratch is written earlier in the same call
    // (activation quantisation fills codes, scales and row sums), so nothing has to be
    // cleared even though the area still holds the previous call's contents.
    return nslq_bitlinear_forward(w, x, x_dtype, M, y, y_dtype, nullptr, nullptr, nullptr, scratch,
                                  NSLQ_NOALLOC_SCRATCH_BYTES, stream);
}

}  // extern "C"
