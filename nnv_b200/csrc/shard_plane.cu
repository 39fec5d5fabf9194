// Data plane of generator sharding inside the library: the sum over ranks of the partial bound sums.
//
// Two transports, both set up by nnvb_set_shard_nccl:
//  * NCCL, bound at run time (dlopen of libnccl.so.2, so that the library neither links against NCCL
//    nor clashes with the copy a host process may already have loaded): ncclAllReduce(ncclDouble,
//    ncclSum) on the engine's stream.  It serves every small reduction (halfspace margins, witness rows)
//    and is the fallback for the bound sums.
//  * peer memory: every rank keeps its [nq][2][N] partial sums in a buffer the other ranks have mapped
//    (CUDA IPC over NVLink).  After writing its sums a rank raises a flag in every peer's buffer; the
//    classify kernel of a rank waits (bounded) for the flags of all peers and then adds the ranks' sums in
//    rank order with plain loads from peer memory while it classifies: one pass, no separate reduction
//    kernel, and the same additions in the same order on every rank.  No multicast of any kind is used.
#include "common.cuh"
#include "shard_plane.cuh"

#include <dlfcn.h>
#include <nccl.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

namespace nnvb {

namespace {

struct NcclApi {
    void* lib = nullptr;
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRank) CommInitRank = nullptr;
    decltype(&ncclAllReduce) AllReduce = nullptr;
    decltype(&ncclAllGather) AllGather = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
    bool ok = false;
};

NcclApi g_nccl;
std::mutex g_nccl_mutex;

int nccl_load() {
    std::lock_guard<std::mutex> lock(g_nccl_mutex);
    if (g_nccl.ok) return NNVB_OK;
    // a copy the process already holds (a host framework's) is found by its soname first
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
        set_error("generator sharding needs NCCL: libnccl.so.2 could not be loaded (%s)", dlerror());
        return NNVB_E_UNSUPPORTED;
    }
    g_nccl.lib = h;
#define NNVB_SYM(name)                                                              \
    g_nccl.name = reinterpret_cast<decltype(g_nccl.name)>(dlsym(h, "nccl" #name));  \
    if (!g_nccl.name) {                                                             \
        set_error("libnccl.so.2 lacks nccl" #name);                                 \
        return NNVB_E_UNSUPPORTED;                                                  \
    }
    NNVB_SYM(GetUniqueId)
    NNVB_SYM(CommInitRank)
    NNVB_SYM(AllReduce)
    NNVB_SYM(AllGather)
    NNVB_SYM(CommDestroy)
    NNVB_SYM(GetErrorString)
#undef NNVB_SYM
    g_nccl.ok = true;
    return NNVB_OK;
}

#define NNVB_NCCL(call)                                                                        \
    do {                                                                                       \
        ncclResult_t r_ = (call);                                                              \
        if (r_ != ncclSuccess) {                                                               \
            set_error("%s failed: %s", #call, g_nccl.GetErrorString(r_));                      \
            return NNVB_E_CUDA;                                                                \
        }                                                                                      \
    } while (0)

}  // namespace

int nccl_unique_id(void* out128) {
    NNVB_TRY(nccl_load());
    static_assert(sizeof(ncclUniqueId) == NNVB_NCCL_ID_BYTES, "NCCL unique id size");
    ncclUniqueId id;
    NNVB_NCCL(g_nccl.GetUniqueId(&id));
    memcpy(out128, &id, sizeof(id));
    return NNVB_OK;
}

int ShardPlane::init(int rank_, int world_, const void* id128) {
    NNVB_TRY(nccl_load());
    rank = rank_;
    world = world_;
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclComm_t c = nullptr;
    NNVB_NCCL(g_nccl.CommInitRank(&c, world, id, rank));
    comm = c;
    return NNVB_OK;
}

int ShardPlane::allreduce(double* buf, int64_t count, cudaStream_t st) {
    if (!comm) {
        set_error("the NCCL communicator of this context is not set up");
        return NNVB_E_STATE;
    }
    NNVB_NCCL(g_nccl.AllReduce(buf, buf, size_t(count), ncclDouble, ncclSum, static_cast<ncclComm_t>(comm), st));
    return NNVB_OK;
}

void ShardPlane::release() {
    for (int r = 0; r < (int)peer.size(); ++r)
        if (peer[r] && r != rank) cudaIpcCloseMemHandle(peer[r]);
    peer.clear();
    if (own) cudaFree(own);
    own = nullptr;
    cap_doubles = 0;
    if (d_peer_tab) cudaFree(d_peer_tab);
    d_peer_tab = nullptr;
    if (d_status) cudaFree(d_status);
    d_status = nullptr;
    if (comm && g_nccl.ok) g_nccl.CommDestroy(static_cast<ncclComm_t>(comm));
    comm = nullptr;
    p2p_ok = false;
}

// Peer buffer of a rank: [PEER_HEADER doubles: flags[world] as uint64 | slot 0 | slot 1], each slot
// `slot_doubles` long.  (Re)allocated collectively: every rank calls this with the same size at the same point.
int ShardPlane::ensure_peer(int64_t slot_doubles, cudaStream_t st) {
    if (!want_p2p || world <= 1) return NNVB_OK;
    if (p2p_ok && slot_doubles <= cap_doubles) return NNVB_OK;
    NNVB_CUDA(cudaStreamSynchronize(st));
    // a failure on any rank must switch every rank to the NCCL path: the outcome is agreed on at the end
    int fail = 0;
    for (int r = 0; r < (int)peer.size(); ++r)
        if (peer[r] && r != rank) cudaIpcCloseMemHandle(peer[r]);
    peer.assign(world, nullptr);
    if (own) cudaFree(own);
    own = nullptr;
    p2p_ok = false;
    epoch = 0;
    const int64_t want = slot_doubles + slot_doubles / 4;
    const size_t bytes = sizeof(double) * size_t(PEER_HEADER + 2 * want);
    cudaIpcMemHandle_t mine;
    memset(&mine, 0, sizeof(mine));
    if (cudaMalloc(reinterpret_cast<void**>(&own), bytes) != cudaSuccess) { own = nullptr; fail = 1; cudaGetLastError(); }
    if (!fail && cudaMemset(own, 0, sizeof(double) * PEER_HEADER) != cudaSuccess) { fail = 1; cudaGetLastError(); }
    if (!fail && cudaIpcGetMemHandle(&mine, own) != cudaSuccess) { fail = 1; cudaGetLastError(); }
    // exchange the handles (and the failure flags) through NCCL
    const size_t rec = sizeof(cudaIpcMemHandle_t) + 8;
    std::vector<char> h_send(rec, 0), h_all(rec * world, 0);
    memcpy(h_send.data(), &mine, sizeof(mine));
    h_send[sizeof(mine)] = char(fail);
    char *d_send = nullptr, *d_all = nullptr;
    NNVB_CUDA(cudaMalloc(reinterpret_cast<void**>(&d_send), rec));
    NNVB_CUDA(cudaMalloc(reinterpret_cast<void**>(&d_all), rec * world));
    NNVB_CUDA(cudaMemcpyAsync(d_send, h_send.data(), rec, cudaMemcpyHostToDevice, st));
    NNVB_NCCL(g_nccl.AllGather(d_send, d_all, rec, ncclChar, static_cast<ncclComm_t>(comm), st));
    NNVB_CUDA(cudaMemcpyAsync(h_all.data(), d_all, rec * world, cudaMemcpyDeviceToHost, st));
    NNVB_CUDA(cudaStreamSynchronize(st));
    for (int r = 0; r < world; ++r) fail |= h_all[rec * r + sizeof(cudaIpcMemHandle_t)];
    if (!fail) {
        for (int r = 0; r < world && !fail; ++r) {
            if (r == rank) { peer[r] = own; continue; }
            cudaIpcMemHandle_t h;
            memcpy(&h, h_all.data() + rec * r, sizeof(h));
            void* p = nullptr;
            if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { fail = 1; cudaGetLastError(); }
            else peer[r] = static_cast<double*>(p);
        }
    }
    // second agreement: did every rank map every peer?
    h_send[0] = char(fail);
    NNVB_CUDA(cudaMemcpyAsync(d_send, h_send.data(), 8, cudaMemcpyHostToDevice, st));
    NNVB_NCCL(g_nccl.AllGather(d_send, d_all, 8, ncclChar, static_cast<ncclComm_t>(comm), st));
    NNVB_CUDA(cudaMemcpyAsync(h_all.data(), d_all, 8 * size_t(world), cudaMemcpyDeviceToHost, st));
    NNVB_CUDA(cudaStreamSynchronize(st));
    for (int r = 0; r < world; ++r) fail |= h_all[8 * r];
    cudaFree(d_send);
    cudaFree(d_all);
    if (fail) {
        // every rank drops to the NCCL all-reduce
        for (int r = 0; r < world; ++r)
            if (peer[r] && r != rank) cudaIpcCloseMemHandle(peer[r]);
        peer.assign(world, nullptr);
        if (own) cudaFree(own);
        own = nullptr;
        want_p2p = false;
        return NNVB_OK;
    }
    if (!d_peer_tab) NNVB_CUDA(cudaMalloc(reinterpret_cast<void**>(&d_peer_tab), sizeof(double*) * MAX_SHARD_RANKS));
    if (!d_status) {
        NNVB_CUDA(cudaMalloc(reinterpret_cast<void**>(&d_status), sizeof(int) * 4));
        NNVB_CUDA(cudaMemset(d_status, 0, sizeof(int) * 4));
    }
    NNVB_CUDA(cudaMemcpy(d_peer_tab, peer.data(), sizeof(double*) * world, cudaMemcpyHostToDevice));
    cap_doubles = want;
    p2p_ok = true;
    return NNVB_OK;
}

namespace {

// Raise this rank's flag in every peer's buffer: its sums of call `epoch` are complete.
__global__ void shard_publish_kernel(double* const* __restrict__ peer_tab, int rank, int world, unsigned long long epoch) {
    const int r = threadIdx.x;
    if (r >= world) return;
    __threadfence_system();          // the sums written by the preceding kernel are visible before the flag
    volatile unsigned long long* flags = reinterpret_cast<volatile unsigned long long*>(peer_tab[r]);
    flags[rank] = epoch;
}

}  // namespace

int ShardPlane::publish(cudaStream_t st, int64_t* launches) {
    ++epoch;
    shard_publish_kernel<<<1, 32, 0, st>>>(d_peer_tab, rank, world, epoch);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

}  // namespace nnvb
