// Transport of generator sharding (see shard_plane.cu): an NCCL communicator bound at run time and, on top
// of it, peer-mapped buffers for the fused "sum over ranks + classify" kernel of the ReLU step.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

namespace nnvb {

constexpr int MAX_SHARD_RANKS = 16;
// doubles in front of the two sum slots of a peer buffer; the first `world` of them are the ranks' flags
// (unsigned 64-bit epochs)
constexpr int64_t PEER_HEADER = 32;
// polls of a peer flag before the classify kernel gives up (about two seconds with the back-off used)
constexpr long long PEER_WAIT_POLLS = 4000000;

int nccl_unique_id(void* out128);

struct ShardPlane {
    int rank = 0, world = 1;
    void* comm = nullptr;               // ncclComm_t
    // peer memory
    bool want_p2p = false;              // asked for at set-up; cleared for good when a mapping fails on any rank
    bool p2p_ok = false;
    double* own = nullptr;              // this rank's buffer
    std::vector<double*> peer;          // [world] every rank's buffer as mapped here (peer[rank] == own)
    double** d_peer_tab = nullptr;      // device copy of `peer`
    int* d_status = nullptr;            // [0] != 0: a wait ran out ([1] = rank waited for, [2] = epoch)
    int64_t cap_doubles = 0;            // doubles per slot
    unsigned long long epoch = 0;       // calls so far; slot of a call = epoch & 1

    int init(int rank, int world, const void* id128);
    int allreduce(double* buf, int64_t count, cudaStream_t st);
    // collective: every rank calls it with the same size at the same point of its call sequence
    int ensure_peer(int64_t slot_doubles, cudaStream_t st);
    // where the reduce kernel of the next call writes this rank's sums
    double* next_slot() const { return own + PEER_HEADER + ((epoch + 1) & 1) * cap_doubles; }
    // offset (doubles) of the current call's slot in every rank's buffer
    int64_t slot_offset() const { return PEER_HEADER + (epoch & 1) * cap_doubles; }
    // after the sums of a call are written: advance the epoch and raise the flags at the peers
    int publish(cudaStream_t st, int64_t* launches);
    void release();
};

}  // namespace nnvb
