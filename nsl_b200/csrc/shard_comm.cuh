// The object behind nslq_comm_t and the small argument structs of the peer-memory kernels.
#pragma once
#include <stdint.h>

#include <vector>

#include "../../include/nslq_b200.h"

namespace nslq {

// One buffer of nslq_symm_alloc: the same allocation as seen from this process, per rank
// (base[rank] is the rank's own cudaMalloc, the others are CUDA IPC mappings of the peers').
struct SymmBuf {
    void *base[NSLQ_MAX_RANKS];
    int64_t bytes;
};

struct PeerPtrs {
    void *p[NSLQ_MAX_RANKS];
};

struct PeerBarrierArgs {
    uint32_t *flags[NSLQ_MAX_RANKS];   // flags[r]: rank r's row of `world` epoch slots
    uint32_t *epoch;                   // this rank's barrier count (device memory)
    int *status;
    int rank, world;
};

}  // namespace nslq

struct nslq_comm {
    int rank = 0, world = 1, device = 0;
    void *comm = nullptr;              // ncclComm_t, null when world == 1
    bool aborted = false;
    uint32_t *state = nullptr;         // device: [0] barrier epoch, [1] status word
    int flag_buf = 0;                  // index in bufs of the barrier's flag rows
    std::vector<nslq::SymmBuf> bufs;
};

namespace nslq {
// Fills out->p[r] with rank r's address of `local` (which must lie inside a shared buffer).
int comm_peer_ptrs(const nslq_comm *c, const void *local, int64_t bytes, PeerPtrs *out);
}  // namespace nslq
