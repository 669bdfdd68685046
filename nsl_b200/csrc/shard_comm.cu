// Column-parallel sharding across the GPUs of one node: the communicator object behind
// nslq_comm_t, the NCCL all-gather of output shards, and the peer-memory path (buffers every
// rank can store into, a flag barrier, an all-gather by peer stores).
//
// NCCL is reached through dlopen/dlsym, so the library loads on a machine without it and a
// process that already carries a NCCL (PyTorch's) keeps using that one.  The contract follows
// NSL's NCCL backend (crates/nsl-runtime/src/tensor_parallel/collective.rs:854-1130): rank 0
// mints a unique id, the host distributes it, every rank joins under a watchdog deadline
// (NSL_NCCL_TIMEOUT_SECS, default 300), collectives are issued on the caller's stream and
// completion can be awaited with a deadline instead of an unbounded synchronise.
//
// Peer memory: cudaMalloc + CUDA IPC handles exchanged over the communicator.  Only plain
// loads/stores ever touch a peer's memory here (no bulk-tensor copies, no multicast objects).
#include <dlfcn.h>
#include <nccl.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include "common.cuh"
#include "shard_comm.cuh"

namespace nslq {

// ------------------------------------------------------------------ NCCL through dlsym
struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId *);
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*CommAbort)(ncclComm_t);
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *);
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    const char *(*GetErrorString)(ncclResult_t);
    bool ok;
};

static const NcclApi *nccl_api()
{
    static NcclApi api = {};
    static std::once_flag once;
    std::call_once(once, [] {
        // a NCCL already in the process (e.g. the one PyTorch ships) wins over the system's
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
#define NSLQ_SYM(field, name) *(void **)(&api.field) = dlsym(h, name)
        NSLQ_SYM(GetUniqueId, "ncclGetUniqueId");
        NSLQ_SYM(CommInitRank, "ncclCommInitRank");
        NSLQ_SYM(CommDestroy, "ncclCommDestroy");
        NSLQ_SYM(CommAbort, "ncclCommAbort");
        NSLQ_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
        NSLQ_SYM(AllGather, "ncclAllGather");
        NSLQ_SYM(GetErrorString, "ncclGetErrorString");
#undef NSLQ_SYM
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.CommAbort && api.CommGetAsyncError &&
                 api.AllGather && api.GetErrorString;
    });
    return api.ok ? &api : nullptr;
}

static long timeout_secs()
{
    const char *e = getenv("NSL_NCCL_TIMEOUT_SECS");
    if (e) {
        char *end = nullptr;
        long v = strtol(e, &end, 10);
        if (end != e && v > 0) return v;
    }
    return 300;
}

// ------------------------------------------------------------------ device side
// Status word of the peer-memory kernels of one communicator (0 = ok).
//   0x501  a barrier wait ran out: some peer never signalled this epoch
constexpr unsigned long long PEER_WAIT_NS = 2000000000ull;

static __device__ __forceinline__ unsigned long long gtimer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// One CTA, one thread per rank.  Thread r publishes this rank's new epoch in rank r's flag
// row and then waits until rank r's epoch has arrived here.  Everything that happened before
// this kernel in the stream (the stores of the preceding kernels into peers' memory) is
// ordered before the release store; everything after it in the stream sees what the peers
// wrote before their own signal.  The wait is bounded: when it runs out the kernel records
// 0x501 and returns, and the context stays usable.
__global__ void peer_barrier_kernel(PeerBarrierArgs a)
{
    __shared__ uint32_t epoch_s;
    if (threadIdx.x == 0) {
        const uint32_t e = *a.epoch + 1u;
        *a.epoch = e;
        epoch_s = e;
    }
    __syncthreads();
    const uint32_t epoch = epoch_s;
    const int r = threadIdx.x;
    if (r >= a.world) return;
    __threadfence_system();
    uint32_t *remote = a.flags[r] + a.rank;                 // my slot in rank r's row
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const uint32_t *mine = a.flags[a.rank] + r;             // rank r's slot in my row
    long long t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if ((int32_t)(v - epoch) >= 0) break;
        if ((spin & 255u) == 255u) {
            const long long now = (long long)gtimer();
            if (t0 == 0) t0 = now;
            else if (now - t0 > (long long)PEER_WAIT_NS) { atomicCAS(a.status, 0, 0x501); break; }
        }
    }
}

// All-gather by peer stores: this rank's [M, n_local] block goes to columns
// [col0, col0 + n_local) of the [M, ld] result in every rank's copy (its own included).
// 16-byte vectors; rows and blocks are 16-byte aligned by the host-side checks.
__global__ void __launch_bounds__(256)
peer_push_cols_kernel(const uint4 *__restrict__ src, PeerPtrs dst, int world, int64_t M, int64_t row_vecs,
                      int64_t ld_vecs, int64_t col0_vecs)
{
    pdl_wait();
    const int64_t total = M * row_vecs;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / row_vecs, c = i - m * row_vecs;
        const uint4 v = src[i];
        const int64_t o = m * ld_vecs + col0_vecs + c;
        for (int r = 0; r < world; ++r) reinterpret_cast<uint4 *>(dst.p[r])[o] = v;
    }
}

// [G][M][n] -> [M][G*n] (the layout NCCL's all-gather leaves -> row-major result)
__global__ void __launch_bounds__(256)
assemble_cols_kernel(const uint8_t *__restrict__ gathered, uint8_t *__restrict__ out, int world, int64_t M,
                     int64_t row_bytes)
{
    const int64_t total = (int64_t)world * M * row_bytes;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t g = i / (M * row_bytes), rem = i - g * (M * row_bytes);
        const int64_t m = rem / row_bytes, b = rem - m * row_bytes;
        out[(m * world + g) * row_bytes + b] = gathered[i];
    }
}

// other translation units
int act_quant_dispatch(const void *, int, int64_t, int64_t, int8_t *, int8_t *, float *, int32_t *, cudaStream_t);
bool ternary_gemm_supported(const void *, const void *, int64_t, int64_t, int64_t);
int ternary_gemm_dispatch(const uint8_t *, const int8_t *, const float *, const int32_t *, int64_t, int64_t,
                          int64_t, float, void *, int, int32_t *, const float *, const float *, const OutSpec *, cudaStream_t);

static inline int64_t align256(int64_t v) { return (v + 255) / 256 * 256; }

static int elem_size(int dt)
{
    switch (dt) {
    case NSLQ_DTYPE_F64: return 8;
    case NSLQ_DTYPE_F32: case NSLQ_DTYPE_I32: return 4;
    case NSLQ_DTYPE_FP16: case NSLQ_DTYPE_BF16: return 2;
    case NSLQ_DTYPE_INT8: return 1;
    default: return 0;
    }
}

// The peers' addresses of a pointer inside one of the communicator's shared buffers.
int comm_peer_ptrs(const nslq_comm *c, const void *local, int64_t bytes, PeerPtrs *out)
{
    const char *p = (const char *)local;
    for (const SymmBuf &b : c->bufs) {
        const char *base = (const char *)b.base[c->rank];
        if (p >= base && p + bytes <= base + b.bytes) {
            for (int r = 0; r < c->world; ++r) out->p[r] = (char *)b.base[r] + (p - base);
            return NSLQ_OK;
        }
    }
    return fail(NSLQ_ERR_ARG, "pointer %p (+%lld bytes) is not inside a buffer of nslq_symm_alloc on this communicator",
                local, (long long)bytes);
}

static int comm_check(const nslq_comm *c, const char *who)
{
    if (!c) return fail(NSLQ_ERR_ARG, "%s: null communicator", who);
    if (c->aborted) return fail(NSLQ_ERR_COMM, "%s: the communicator was aborted after an earlier failure", who);
    return NSLQ_OK;
}

static int nccl_fail(nslq_comm *c, const char *what, ncclResult_t rc)
{
    const NcclApi *n = nccl_api();
    fail(NSLQ_ERR_COMM, "%s failed on rank %d: %s", what, c->rank, n ? n->GetErrorString(rc) : "NCCL not loaded");
    if (n && c->comm && !c->aborted) { n->CommAbort((ncclComm_t)c->comm); c->aborted = true; }
    return NSLQ_ERR_COMM;
}

}  // namespace nslq

using namespace nslq;

extern "C" {

int nslq_shard_unique_id(void *id_out)
{
    if (!id_out) return fail(NSLQ_ERR_ARG, "nslq_shard_unique_id: null output");
    const NcclApi *n = nccl_api();
    if (!n) return fail(NSLQ_ERR_COMM, "nslq_shard_unique_id: libnccl.so.2 cannot be loaded: %s", dlerror());
    static_assert(sizeof(ncclUniqueId) == NSLQ_UNIQUE_ID_BYTES, "unique id size");
    ncclUniqueId id;
    ncclResult_t rc = n->GetUniqueId(&id);
    if (rc != ncclSuccess) return fail(NSLQ_ERR_COMM, "ncclGetUniqueId: %s", n->GetErrorString(rc));
    memcpy(id_out, &id, sizeof(id));
    return NSLQ_OK;
}

int nslq_shard_init(const void *unique_id, int rank, int world, nslq_comm_t **out)
{
    if (!out) return fail(NSLQ_ERR_ARG, "nslq_shard_init: null output");
    *out = nullptr;
    if (world <= 0 || world > NSLQ_MAX_RANKS || rank < 0 || rank >= world)
        return fail(NSLQ_ERR_ARG, "nslq_shard_init: rank %d of %d (at most %d ranks)", rank, world, NSLQ_MAX_RANKS);
    if (world > 1 && !unique_id) return fail(NSLQ_ERR_ARG, "nslq_shard_init: null unique id");
    nslq_comm *c = new nslq_comm();
    c->rank = rank; c->world = world;
    if (cudaGetDevice(&c->device) != cudaSuccess) {
        delete c;
        return fail(NSLQ_ERR_CUDA, "nslq_shard_init: cudaGetDevice: %s", cudaGetErrorString(cudaGetLastError()));
    }
    if (world > 1) {
        const NcclApi *n = nccl_api();
        if (!n) { delete c; return fail(NSLQ_ERR_COMM, "nslq_shard_init: libnccl.so.2 cannot be loaded"); }
        ncclUniqueId id;
        memcpy(&id, unique_id, sizeof(id));
        // ncclCommInitRank blocks until the whole clique has arrived.  A peer that died after the
        // id was handed out would leave this rank waiting for ever, so a watchdog ends the process
        // at the deadline, loudly, as NSL's backend does (collective.rs:906-934).
        std::atomic<bool> done(false);
        const long secs = timeout_secs();
        std::thread watchdog([&done, secs, rank] {
            const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(secs);
            while (!done.load(std::memory_order_acquire)) {
                if (std::chrono::steady_clock::now() >= deadline) {
                    fprintf(stderr, "nslq: ncclCommInitRank timed out after %lds on rank %d -- a peer rank likely died before "
                                    "joining. Aborting (NSL_NCCL_TIMEOUT_SECS tunes the deadline).\n", secs, rank);
                    abort();
                }
                std::this_thread::sleep_for(std::chrono::milliseconds(50));
            }
        });
        ncclComm_t comm = nullptr;
        ncclResult_t rc = n->CommInitRank(&comm, world, id, rank);
        done.store(true, std::memory_order_release);
        watchdog.join();
        if (rc != ncclSuccess) {
            delete c;
            return fail(NSLQ_ERR_COMM, "ncclCommInitRank(rank %d of %d): %s", rank, world, n->GetErrorString(rc));
        }
        c->comm = comm;
    }
    // barrier state: one row of `world` epoch slots per rank, in memory every rank can store into
    void *state = nullptr;
    if (cudaMalloc(&state, 256) != cudaSuccess || cudaMemset(state, 0, 256) != cudaSuccess) {
        nslq_shard_destroy(c);
        return fail(NSLQ_ERR_CUDA, "nslq_shard_init: device state: %s", cudaGetErrorString(cudaGetLastError()));
    }
    c->state = (uint32_t *)state;                 // [0] epoch, [1] status
    *out = c;
    void *flags = nullptr;
    int rc = nslq_symm_alloc(c, 256, &flags);
    if (rc) { *out = nullptr; nslq_shard_destroy(c); return rc; }
    c->flag_buf = 0;
    return NSLQ_OK;
}

void nslq_shard_destroy(nslq_comm_t *c)
{
    if (!c) return;
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    for (SymmBuf &b : c->bufs) {
        for (int r = 0; r < c->world; ++r)
            if (r != c->rank && b.base[r]) cudaIpcCloseMemHandle(b.base[r]);
        if (b.base[c->rank]) cudaFree(b.base[c->rank]);
    }
    if (c->state) cudaFree(c->state);
    const NcclApi *n = nccl_api();
    // an aborted communicator must not be destroyed as well (collective.rs:861-865)
    if (n && c->comm && !c->aborted) n->CommDestroy((ncclComm_t)c->comm);
    delete c;
}

int nslq_shard_info(const nslq_comm_t *c, int *rank, int *world)
{
    if (!c) return fail(NSLQ_ERR_ARG, "nslq_shard_info: null communicator");
    if (rank) *rank = c->rank;
    if (world) *world = c->world;
    return NSLQ_OK;
}

int nslq_allgather_cols(nslq_comm_t *c, const void *y_local, int dtype, int64_t M, int64_t N_local, void *gathered,
                        void *y_full, void *stream)
{
    int rc = comm_check(c, "nslq_allgather_cols");
    if (rc) return rc;
    const int es = elem_size(dtype);
    if (!es) return fail(NSLQ_ERR_ARG, "nslq_allgather_cols: dtype tag %d", dtype);
    if (!y_local || !gathered) return fail(NSLQ_ERR_ARG, "nslq_allgather_cols: null buffer");
    if (M < 0 || N_local <= 0) return fail(NSLQ_ERR_SHAPE, "nslq_allgather_cols: M=%lld N_local=%lld", (long long)M, (long long)N_local);
    if (M == 0) return NSLQ_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t bytes = (size_t)M * (size_t)N_local * es;
    if (c->world == 1) {
        if (gathered != y_local && cudaMemcpyAsync(gathered, y_local, bytes, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
            return fail(NSLQ_ERR_CUDA, "nslq_allgather_cols: %s", cudaGetErrorString(cudaGetLastError()));
    } else {
        const NcclApi *n = nccl_api();
        ncclResult_t nrc = n->AllGather(y_local, gathered, bytes, ncclInt8, (ncclComm_t)c->comm, st);
        if (nrc != ncclSuccess) return nccl_fail(c, "ncclAllGather", nrc);
    }
    if (y_full && (M > 1 || y_full != gathered)) {
        if (M == 1) {            // [G][1][n] already is [1][G*n]
            if (cudaMemcpyAsync(y_full, gathered, bytes * c->world, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
                return fail(NSLQ_ERR_CUDA, "nslq_allgather_cols: %s", cudaGetErrorString(cudaGetLastError()));
            return NSLQ_OK;
        }
        if (y_full == gathered) return fail(NSLQ_ERR_ARG, "nslq_allgather_cols: y_full must not alias gathered for M > 1");
        const int64_t total = (int64_t)bytes * c->world;
        const unsigned blocks = (unsigned)(total / 256 + 1 < 2048 ? total / 256 + 1 : 2048);
        assemble_cols_kernel<<<blocks, 256, 0, st>>>((const uint8_t *)gathered, (uint8_t *)y_full, c->world, M, N_local * es);
        return check_launch("assemble_cols_kernel");
    }
    return NSLQ_OK;
}

int nslq_shard_wait(nslq_comm_t *c, void *stream, int64_t timeout_ms)
{
    if (!c) return fail(NSLQ_ERR_ARG, "nslq_shard_wait: null communicator");
    const NcclApi *n = c->world > 1 ? nccl_api() : nullptr;
    const auto deadline = std::chrono::steady_clock::now() +
                          std::chrono::milliseconds(timeout_ms > 0 ? timeout_ms : timeout_secs() * 1000);
    for (;;) {
        cudaError_t e = cudaStreamQuery((cudaStream_t)stream);
        if (e == cudaSuccess) break;
        if (e != cudaErrorNotReady) return fail(NSLQ_ERR_CUDA, "nslq_shard_wait: %s", cudaGetErrorString(e));
        if (n && c->comm && !c->aborted) {
            ncclResult_t aerr = ncclSuccess;
            n->CommGetAsyncError((ncclComm_t)c->comm, &aerr);
            if (aerr != ncclSuccess && aerr != ncclInProgress) return nccl_fail(c, "collective (asynchronous error)", aerr);
        }
        if (std::chrono::steady_clock::now() >= deadline) {
            // a peer likely died mid-collective: give up on the communicator, tell the caller
            if (n && c->comm && !c->aborted) { n->CommAbort((ncclComm_t)c->comm); c->aborted = true; }
            return fail(NSLQ_ERR_TIMEOUT, "nslq_shard_wait: rank %d still waiting at the deadline; communicator aborted", c->rank);
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    if (n && c->comm && !c->aborted) {
        ncclResult_t aerr = ncclSuccess;
        n->CommGetAsyncError((ncclComm_t)c->comm, &aerr);
        if (aerr != ncclSuccess) return nccl_fail(c, "collective (asynchronous error)", aerr);
    }
    return NSLQ_OK;
}

// ------------------------------------------------------------------ peer memory
int nslq_symm_alloc(nslq_comm_t *c, int64_t bytes, void **local_ptr)
{
    int rc = comm_check(c, "nslq_symm_alloc");
    if (rc) return rc;
    if (!local_ptr || bytes <= 0) return fail(NSLQ_ERR_ARG, "nslq_symm_alloc: bytes=%lld", (long long)bytes);
    SymmBuf b = {};
    b.bytes = (bytes + 255) / 256 * 256;
    void *mine = nullptr;
    if (cudaMalloc(&mine, (size_t)b.bytes) != cudaSuccess || cudaMemset(mine, 0, (size_t)b.bytes) != cudaSuccess) {
        if (mine) cudaFree(mine);
        return fail(NSLQ_ERR_CUDA, "nslq_symm_alloc: %lld bytes: %s", (long long)b.bytes, cudaGetErrorString(cudaGetLastError()));
    }
    b.base[c->rank] = mine;
    if (c->world > 1) {
        const NcclApi *n = nccl_api();
        cudaIpcMemHandle_t h;
        cudaIpcMemHandle_t *all = nullptr;
        std::vector<cudaIpcMemHandle_t> host(c->world);
        bool ok = cudaIpcGetMemHandle(&h, mine) == cudaSuccess &&
                  cudaMalloc((void **)&all, sizeof(h) * c->world) == cudaSuccess &&
                  cudaMemcpy(all + c->rank, &h, sizeof(h), cudaMemcpyHostToDevice) == cudaSuccess;
        if (!ok) {
            if (all) cudaFree(all);
            cudaFree(mine);
            return fail(NSLQ_ERR_CUDA, "nslq_symm_alloc: IPC handle: %s", cudaGetErrorString(cudaGetLastError()));
        }
        ncclResult_t nrc = n->AllGather(all + c->rank, all, sizeof(h), ncclInt8, (ncclComm_t)c->comm, nullptr);
        if (nrc != ncclSuccess) { cudaFree(all); cudaFree(mine); return nccl_fail(c, "ncclAllGather (IPC handles)", nrc); }
        rc = nslq_shard_wait(c, nullptr, 0);
        if (rc) { cudaFree(all); cudaFree(mine); return rc; }
        cudaMemcpy(host.data(), all, sizeof(h) * c->world, cudaMemcpyDeviceToHost);
        cudaFree(all);
        for (int r = 0; r < c->world; ++r) {
            if (r == c->rank) continue;
            cudaError_t e = cudaIpcOpenMemHandle(&b.base[r], host[r], cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
                for (int q = 0; q < r; ++q)
                    if (q != c->rank && b.base[q]) cudaIpcCloseMemHandle(b.base[q]);
                cudaFree(mine);
                return fail(NSLQ_ERR_CUDA, "nslq_symm_alloc: cannot map rank %d's buffer on rank %d: %s", r, c->rank, cudaGetErrorString(e));
            }
        }
    }
    c->bufs.push_back(b);
    *local_ptr = mine;
    return NSLQ_OK;
}

int nslq_peer_barrier(nslq_comm_t *c, void *stream)
{
    int rc = comm_check(c, "nslq_peer_barrier");
    if (rc) return rc;
    if (c->world == 1) return NSLQ_OK;
    PeerBarrierArgs a = {};
    const SymmBuf &fb = c->bufs[c->flag_buf];
    for (int r = 0; r < c->world; ++r) a.flags[r] = (uint32_t *)fb.base[r];
    a.epoch = c->state; a.status = (int *)(c->state + 1);
    a.rank = c->rank; a.world = c->world;
    // launched without the dependent-launch attribute: it must not start before the kernels in
    // front of it have completed, since completing them is what it announces
    peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(a);
    return check_launch("peer_barrier_kernel");
}

int nslq_peer_allgather_cols(nslq_comm_t *c, const void *y_local, int dtype, int64_t M, int64_t N_local, void *y_full,
                             void *stream)
{
    int rc = comm_check(c, "nslq_peer_allgather_cols");
    if (rc) return rc;
    const int es = elem_size(dtype);
    if (!es) return fail(NSLQ_ERR_ARG, "nslq_peer_allgather_cols: dtype tag %d", dtype);
    if (!y_local || !y_full) return fail(NSLQ_ERR_ARG, "nslq_peer_allgather_cols: null buffer");
    if (M <= 0 || N_local <= 0) return M == 0 ? NSLQ_OK : fail(NSLQ_ERR_SHAPE, "nslq_peer_allgather_cols: M=%lld N_local=%lld", (long long)M, (long long)N_local);
    const int64_t row_bytes = N_local * es;
    if (row_bytes % 16 != 0 || !aligned16(y_local) || !aligned16(y_full))
        return fail(NSLQ_ERR_UNSUPPORTED, "nslq_peer_allgather_cols: shard rows of %lld bytes: rows and buffers must be multiples of 16 bytes", (long long)row_bytes);
    PeerPtrs dst = {};
    if ((rc = comm_peer_ptrs(c, y_full, M * row_bytes * c->world, &dst))) return rc;
    const int64_t vecs = M * (row_bytes / 16);
    const unsigned blocks = (unsigned)(vecs / 256 + 1 < 1184 ? vecs / 256 + 1 : 1184);
    cudaError_t e = launch_kernel(peer_push_cols_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream,
                                  (const uint4 *)y_local, dst, c->world, M, row_bytes / 16, row_bytes / 16 * c->world,
                                  row_bytes / 16 * c->rank);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "peer_push_cols_kernel: %s", cudaGetErrorString(e));
    return check_launch("peer_push_cols_kernel");
}

int nslq_symm_free(nslq_comm_t *c, void *local_ptr)
{
    if (!c || !local_ptr) return fail(NSLQ_ERR_ARG, "nslq_symm_free: null argument");
    for (size_t i = 0; i < c->bufs.size(); ++i) {
        SymmBuf &b = c->bufs[i];
        if (b.base[c->rank] != local_ptr) continue;
        if ((int)i == c->flag_buf) return fail(NSLQ_ERR_ARG, "nslq_symm_free: that is the communicator's own flag buffer");
        cudaDeviceSynchronize();
        for (int r = 0; r < c->world; ++r)
            if (r != c->rank && b.base[r]) cudaIpcCloseMemHandle(b.base[r]);
        cudaFree(b.base[c->rank]);
        b = SymmBuf();                      // slot stays (indices of the others do not move)
        return NSLQ_OK;
    }
    return fail(NSLQ_ERR_ARG, "nslq_symm_free: %p is not a buffer of nslq_symm_alloc on this communicator", local_ptr);
}

int64_t nslq_bitlinear_gathered_workspace_bytes(int64_t M, int64_t K, int64_t N_local)
{
    if (M < 0 || K <= 0 || N_local <= 0) return 0;
    // quantised activations, then (M <= 16 only) this rank's [M, N_local] block before it is pushed
    return nslq_bitlinear_workspace_bytes(M, K) + (M <= 16 ? align256(M * N_local * 4) : 0);
}

int nslq_bitlinear_forward_quantized_cols(const nslq_bitlinear_t *w, const int8_t *q_perm, const float *scale,
                                          const int32_t *rowsum, int64_t M, void *const *y_copies, int n_copies,
                                          int64_t ldy, int64_t col0, int y_dtype, const float *bias, void *y_scratch,
                                          int64_t y_scratch_bytes, void *stream)
{
    if (!w || !q_perm || !scale || !rowsum || !y_copies) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward_quantized_cols: null argument");
    if (n_copies < 1 || n_copies > NSLQ_MAX_RANKS) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward_quantized_cols: %d copies (1..%d)", n_copies, NSLQ_MAX_RANKS);
    for (int i = 0; i < n_copies; ++i)
        if (!y_copies[i]) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward_quantized_cols: copy %d is null", i);
    const int es = y_dtype == NSLQ_DTYPE_F32 ? 4 : (y_dtype == NSLQ_DTYPE_BF16 || y_dtype == NSLQ_DTYPE_FP16) ? 2 : 0;
    if (!es) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward_quantized_cols: y_dtype %d not in {F32,FP16,BF16}", y_dtype);
    if (M < 0 || col0 < 0 || ldy < col0 + w->N)
        return fail(NSLQ_ERR_SHAPE, "nslq_bitlinear_forward_quantized_cols: M=%lld, columns [%lld, %lld) of rows of %lld", (long long)M,
                    (long long)col0, (long long)(col0 + w->N), (long long)ldy);
    if (M == 0) return NSLQ_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (M > 16 && ternary_gemm_supported(w->packed, q_perm, M, w->N, w->K)) {
        // the GEMM's epilogue stores each finished tile into every copy
        OutSpec os = {};
        os.ldy = ldy;
        for (int i = 1; i < n_copies; ++i) os.peer[os.npeer++] = (char *)y_copies[i] + col0 * es;
        return ternary_gemm_dispatch(w->packed, q_perm, scale, rowsum, M, w->N, w->K, w->weight_scale,
                                     (char *)y_copies[0] + col0 * es, y_dtype, nullptr, bias, nullptr, &os, st);
    }
    // decode-sized calls: compute the block once, then one kernel stores it into every copy
    const int64_t need = align256(M * w->N * es);
    if (!y_scratch || y_scratch_bytes < need)
        return fail(NSLQ_ERR_WORKSPACE, "nslq_bitlinear_forward_quantized_cols: scratch for the block: %lld bytes, need %lld",
                    (long long)y_scratch_bytes, (long long)need);
    const int64_t row_bytes = w->N * es;
    if (row_bytes % 16 != 0 || (ldy * es) % 16 != 0 || (col0 * es) % 16 != 0 || !aligned16(y_scratch))
        return fail(NSLQ_ERR_UNSUPPORTED, "nslq_bitlinear_forward_quantized_cols: block rows, row stride and column offset must be multiples of 16 bytes");
    int rc = nslq_bitlinear_forward_quantized(w, q_perm, scale, rowsum, M, y_scratch, y_dtype, nullptr, bias, nullptr, stream);
    if (rc) return rc;
    PeerPtrs dst = {};
    for (int i = 0; i < n_copies; ++i) {
        if (!aligned16(y_copies[i])) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward_quantized_cols: copy %d is not 16-byte aligned", i);
        dst.p[i] = y_copies[i];
    }
    const int64_t vecs = M * (row_bytes / 16);
    const unsigned blocks = (unsigned)(vecs / 256 + 1 < 1184 ? vecs / 256 + 1 : 1184);
    cudaError_t e = launch_kernel(peer_push_cols_kernel, dim3(blocks), dim3(256), 0, st, (const uint4 *)y_scratch, dst,
                                  n_copies, M, row_bytes / 16, ldy * es / 16, col0 * es / 16);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "peer_push_cols_kernel: %s", cudaGetErrorString(e));
    return check_launch("peer_push_cols_kernel");
}

int nslq_bitlinear_forward_quantized_gathered(nslq_comm_t *c, const nslq_bitlinear_t *w, const int8_t *q_perm,
                                              const float *scale, const int32_t *rowsum, int64_t M, void *y_full,
                                              int y_dtype, const float *bias, void *y_scratch, int64_t y_scratch_bytes,
                                              void *stream)
{
    int rc = comm_check(c, "nslq_bitlinear_forward_gathered");
    if (rc) return rc;
    if (!w || !y_full) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward_gathered: null argument");
    const int es = y_dtype == NSLQ_DTYPE_F32 ? 4 : 2;
    const int64_t n_total = w->N * c->world;
    PeerPtrs pp = {};
    if ((rc = comm_peer_ptrs(c, y_full, (M > 0 ? M : 0) * n_total * es, &pp))) return rc;
    void *copies[NSLQ_MAX_RANKS];
    copies[0] = y_full;                                   // this rank's own copy first
    int n = 1;
    for (int r = 0; r < c->world; ++r)
        if (r != c->rank) copies[n++] = pp.p[r];
    return nslq_bitlinear_forward_quantized_cols(w, q_perm, scale, rowsum, M, copies, n, n_total, w->N * c->rank, y_dtype,
                                                 bias, y_scratch, y_scratch_bytes, stream);
}

int nslq_bitlinear_forward_cols(const nslq_bitlinear_t *w, const void *x, int x_dtype, int64_t M, void *const *y_copies,
                                int n_copies, int64_t ldy, int64_t col0, int y_dtype, const float *bias, void *workspace,
                                int64_t workspace_bytes, void *stream)
{
    if (!w || !x || !y_copies) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward_cols: null argument");
    if (M < 0) return fail(NSLQ_ERR_SHAPE, "nslq_bitlinear_forward_cols: M=%lld", (long long)M);
    if (M == 0) return NSLQ_OK;
    if (w->K % 64 != 0 || !aligned16(w->packed))
        return fail(NSLQ_ERR_UNSUPPORTED, "nslq_bitlinear_forward_cols: needs K %% 64 == 0 and a 16-byte aligned weight (K=%lld)", (long long)w->K);
    const int64_t need = nslq_bitlinear_gathered_workspace_bytes(M, w->K, w->N);
    if (!workspace || workspace_bytes < need)
        return fail(NSLQ_ERR_WORKSPACE, "nslq_bitlinear_forward_cols: workspace %lld bytes, need %lld", (long long)workspace_bytes, (long long)need);
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward_cols: workspace not 256-byte aligned");
    int8_t *q = (int8_t *)workspace;
    float *scale = (float *)((char *)workspace + align256(M * w->K));
    int32_t *rowsum = (int32_t *)((char *)scale + align256(M * 4));
    void *y_scratch = (char *)rowsum + align256(M * 4);
    int rc = act_quant_dispatch(x, x_dtype, M, w->K, nullptr, q, scale, rowsum, (cudaStream_t)stream);
    if (rc) return rc;
    return nslq_bitlinear_forward_quantized_cols(w, q, scale, rowsum, M, y_copies, n_copies, ldy, col0, y_dtype, bias, y_scratch,
                                                 workspace_bytes - nslq_bitlinear_workspace_bytes(M, w->K), stream);
}

int nslq_bitlinear_forward_gathered(nslq_comm_t *c, const nslq_bitlinear_t *w, const void *x, int x_dtype, int64_t M,
                                    void *y_full, int y_dtype, const float *bias, void *workspace, int64_t workspace_bytes,
                                    void *stream)
{
    int rc = comm_check(c, "nslq_bitlinear_forward_gathered");
    if (rc) return rc;
    if (!w || !y_full) return fail(NSLQ_ERR_ARG, "nslq_bitlinear_forward_gathered: null argument");
    const int es = y_dtype == NSLQ_DTYPE_F32 ? 4 : 2;
    const int64_t n_total = w->N * c->world;
    PeerPtrs pp = {};
    if ((rc = comm_peer_ptrs(c, y_full, (M > 0 ? M : 0) * n_total * es, &pp))) return rc;
    void *copies[NSLQ_MAX_RANKS];
    copies[0] = y_full;                                   // this rank's own copy first
    int n = 1;
    for (int r = 0; r < c->world; ++r)
        if (r != c->rank) copies[n++] = pp.p[r];
    return nslq_bitlinear_forward_cols(w, x, x_dtype, M, copies, n, n_total, w->N * c->rank, y_dtype, bias, workspace,
                                       workspace_bytes, stream);
}

int nslq_peer_push_cols_async(nslq_comm_t *c, void *y_full, int dtype, int64_t M, int64_t N_local, void *stream)
{
    int rc = comm_check(c, "nslq_peer_push_cols_async");
    if (rc) return rc;
    const int es = elem_size(dtype);
    if (!es) return fail(NSLQ_ERR_ARG, "nslq_peer_push_cols_async: dtype tag %d", dtype);
    if (!y_full) return fail(NSLQ_ERR_ARG, "nslq_peer_push_cols_async: null buffer");
    if (M <= 0 || N_local <= 0) return M == 0 ? NSLQ_OK : fail(NSLQ_ERR_SHAPE, "nslq_peer_push_cols_async: M=%lld N_local=%lld", (long long)M, (long long)N_local);
    const size_t row = (size_t)N_local * es, pitch = row * c->world, off = row * c->rank;
    PeerPtrs dst = {};
    if ((rc = comm_peer_ptrs(c, y_full, (int64_t)(M * pitch), &dst))) return rc;
    // one strided copy per peer, by the copy engines: no SM is involved, so the transfer runs under
    // whatever kernels follow on other streams
    for (int i = 1; i < c->world; ++i) {
        const int r = (c->rank + i) % c->world;              // staggered, so the ranks do not all write to the same peer first
        cudaError_t e = cudaMemcpy2DAsync((char *)dst.p[r] + off, pitch, (const char *)y_full + off, pitch, row, (size_t)M,
                                          cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
        if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "nslq_peer_push_cols_async: copy to rank %d: %s", r, cudaGetErrorString(e));
    }
    return NSLQ_OK;
}

int nslq_shard_status(nslq_comm_t *c, int *status)
{
    if (!c || !status) return fail(NSLQ_ERR_ARG, "nslq_shard_status: null argument");
    int v = 0;
    if (cudaMemcpy(&v, c->state + 1, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
        return fail(NSLQ_ERR_CUDA, "nslq_shard_status: %s", cudaGetErrorString(cudaGetLastError()));
    if (v) cudaMemset(c->state + 1, 0, sizeof(int));
    *status = v;
    return NSLQ_OK;
}

}  // extern "C"
