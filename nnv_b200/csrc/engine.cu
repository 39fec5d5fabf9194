// Host side of libnnvb200.so: contexts, networks, batches of star sets and the
// layer loop of NN.reach (NN.m:1529-1551), all behind the C ABI of
// include/nnvb200.h.  The arithmetic lives in the kernel files; this file
// owns device memory, the per-query column bookkeeping and the order of
// launches on the context's stream.
#include "common.cuh"
#include "shard_plane.cuh"

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

namespace nnvb {

static thread_local char g_err[1024] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

// Device buffer that grows geometrically and is reused across calls, so that a
// steady-state reach performs no allocation.
struct DevBuf {
    void* p = nullptr;
    size_t cap = 0;
    int ensure(size_t bytes, cudaStream_t st, bool keep = false) {
        if (bytes <= cap) return NNVB_OK;
        size_t want = std::max(bytes, cap + cap / 2);
        want = (want + 255) / 256 * 256;
        void* np = nullptr;
        NNVB_CUDA(cudaStreamSynchronize(st));
        cudaError_t e = cudaMalloc(&np, want);
        if (e != cudaSuccess) {
            set_error("device allocation of %zu bytes failed: %s", want, cudaGetErrorString(e));
            cudaGetLastError();
            return NNVB_E_CAPACITY;
        }
        if (keep && p && cap) NNVB_CUDA(cudaMemcpy(np, p, cap, cudaMemcpyDeviceToDevice));
        if (p) NNVB_CUDA(cudaFree(p));
        p = np;
        cap = want;
        return NNVB_OK;
    }
    void release() {
        if (p) cudaFree(p);
        p = nullptr;
        cap = 0;
    }
    template <typename T>
    T* as() const { return static_cast<T*>(p); }
};

struct PinnedBuf {
    void* p = nullptr;
    size_t cap = 0;
    int ensure(size_t bytes, bool keep = false) {
        if (bytes <= cap) return NNVB_OK;
        size_t want = std::max(bytes, cap + cap / 2);
        void* np = nullptr;
        NNVB_CUDA(cudaMallocHost(&np, want));
        if (keep && p && cap) memcpy(np, p, cap);
        if (p) cudaFreeHost(p);
        p = np;
        cap = want;
        return NNVB_OK;
    }
    void release() {
        if (p) cudaFreeHost(p);
        p = nullptr;
        cap = 0;
    }
    template <typename T>
    T* as() const { return static_cast<T*>(p); }
};

}  // namespace nnvb

using namespace nnvb;

struct ReluLayerRecord {
    int64_t N = 0;
    int64_t K = 0;                       // new columns over the batch
    int64_t n_dead = 0;
    int64_t cols_after = 0;
    std::vector<int64_t> new_off;        // [nq+1] host copy of the per-query scan
    std::vector<int64_t> P_in;           // [nq] predicates entering the layer
    DevBuf idx, q, c, l, u;              // per new column
    DevBuf G, G_off;                     // crossing rows (keep_constraints)
    std::vector<int64_t> h_G_off;
    DevBuf lb, ub, rank, P_in_dev;       // [nq][N] bounds and crossing ranks, [nq] P_in (keep_layer_bounds)
    DevBuf new_off_dev;                  // [nq+1] device copy of new_off (keep_constraints)
    bool has_G = false, has_bounds = false;
    void release() {
        idx.release(); q.release(); c.release(); l.release(); u.release();
        G.release(); G_off.release(); lb.release(); ub.release(); rank.release(); P_in_dev.release();
        new_off_dev.release();
    }
};

// Working memory of a reach.  It belongs to the context: every batch of the
// context reuses it, so a steady-state reach allocates nothing, and the results
// of a batch stay readable until another batch of the same context is reached.
struct WorkBufs {
    DevBuf col_q, pl, pu, col_pos, box;      // box: int4 {h0, w0, wh, ww} window of each column
    DevBuf qcol_off[2], qcol_idx[2];
    DevBuf chunk_beg, chunk_end, q_chunk_off, partial, sums;
    DevBuf state_cf;                     // the row states in channel-fastest order (readers of compact storage)
    DevBuf lb, ub, state, rank, blk_cross, q_cross, q_dead, q_new_off, gen_off;
    DevBuf tmp;                          // gathers for downloads
    DevBuf fcg;                          // column grouping of the window-gathered FC
    DevBuf winsort;                      // origin bins and sorted columns of the windowed bound reduction
    DevBuf hot_idx, hot_scale;           // neuron and scale of one-hot columns carried through a pooling layer
    DevBuf pack2[2];                     // compact (window-only, channel-fastest) storage of the windowed cohorts: a layer
                                         // reads one buffer and writes the other
    DevBuf hs_G, hs_g, hs_q, hs_margin, hs_r, hs_roff, hs_val, hs_scale, hs_bound, wit[2];   // halfspace tests
    std::vector<std::unique_ptr<ReluLayerRecord>> relu;
    void release() {
        DevBuf* bufs[] = {&col_q, &pl, &pu, &col_pos, &box, &qcol_off[0], &qcol_off[1], &qcol_idx[0], &qcol_idx[1],
                          &chunk_beg, &chunk_end, &q_chunk_off, &partial, &sums, &lb, &ub, &state, &state_cf, &rank, &blk_cross,
                          &q_cross, &q_dead, &q_new_off, &gen_off, &tmp, &fcg, &winsort, &hot_idx, &hot_scale, &pack2[0], &pack2[1], &hs_G, &hs_g, &hs_q, &hs_margin, &hs_r,
                          &hs_roff, &hs_val, &hs_scale, &hs_bound, &wit[0], &wit[1]};
        for (DevBuf* d : bufs) d->release();
        for (auto& r : relu) r->release();
        relu.clear();
    }
};

struct nnvb_ctx {
    int device = 0;
    int sm_count = 1;       // multiprocessors of the device: grids are sized in multiples of it
    cudaStream_t stream = nullptr;
    char* arena = nullptr;
    size_t arena_bytes = 0;
    int64_t launches = 0;
    PinnedBuf scratch;      // small host->device traffic of the layer loop
    // staging and input buffers of destroyed batches, handed to the next batches: a caller that builds a
    // batch per call (the usual way through the host API) then allocates nothing in the steady state
    std::vector<PinnedBuf> spare_pinned;
    std::vector<DevBuf> spare_dev;
    size_t scratch_off = 0; // bytes of `scratch` handed out since the last stream sync
    WorkBufs work;
    // generator sharding over ranks (world == 1: off)
    int rank = 0, world = 1;
    nnvb_allreduce_fn ar_fn = nullptr;
    void* ar_user = nullptr;
    ShardPlane plane;       // NCCL communicator and peer-mapped sum buffers owned by the library (nnvb_set_shard_nccl)
    DevBuf shard_flag;      // one double: "some rank cannot go on", summed over the ranks
    const void* result_owner = nullptr;   // the batch whose results the work buffers and the arena hold
    // per-kernel-family device timing (off by default)
    bool prof_on = false;
    struct ProfRec { int fam; cudaEvent_t a, b; double work; };
    std::vector<ProfRec> prof_recs;
    std::vector<cudaEvent_t> prof_pool;
    double prof_ms[NNVB_PROF_FAMILIES] = {0};
    double prof_work[NNVB_PROF_FAMILIES] = {0};
    int64_t prof_launches[NNVB_PROF_FAMILIES] = {0};
    double* vbuf(int i) const { return reinterpret_cast<double*>(arena + (arena_bytes / 2 / 256 * 256) * i); }
    size_t vbuf_bytes() const { return arena_bytes / 2 / 256 * 256; }
};

struct Layer {
    int type = 0;
    int64_t H = 0, W = 0, C = 0;       // input shape
    int64_t Ho = 0, Wo = 0, Co = 0;    // output shape
    ConvGeom cg{};
    ConvWeights cw{};
    PoolGeom pg{};
    // fc
    double* fc_wt = nullptr;
    int fc_ldw = 0;
    double* bias = nullptr;
    // bn
    double* bn_mean = nullptr;
    double* bn_den = nullptr;
    double* bn_rden = nullptr;
    double* bn_scale = nullptr;
    double* bn_offset = nullptr;
    bool fused_into_prev = false;      // bn applied in the previous conv's epilogue
    int fused_bn = -1;                 // conv: index of the bn layer it applies
};

struct nnvb_net {
    nnvb_ctx* ctx = nullptr;
    std::vector<Layer> layers;
    std::vector<void*> owned;          // device allocations
    int64_t in_shape[3] = {0, 0, 0};
    int64_t out_shape[3] = {0, 0, 0};
    int n_relu = 0;
};

struct nnvb_batch {
    nnvb_net* net = nullptr;
    int nq = 0;
    int kind = 0;                        // 0 unset, 1 bounds form, 2 star form
    int64_t N0 = 0, ld0 = 0;
    // host staging
    PinnedBuf h_in;                      // bounds: [nq][2][N0]; star: V [ld0 x ncols0]
    std::vector<int64_t> P0;             // generators per query (over all ranks)
    std::vector<int64_t> P0_loc;         // ... held by this rank (== P0 when the generators are not sharded)
    std::vector<int64_t> h_Pglob;        // predicates per query over all ranks, after the layers run so far
    DevBuf d_in_pos;                     // star form: predicate position of each uploaded generator column
    std::vector<char> is_set;
    std::vector<std::vector<double>> h_pl, h_pu, h_C, h_d;   // star form / constraints
    std::vector<int64_t> m0;
    std::vector<char> box_implies_C;     // every row of the input constraints holds on the whole predicate box
    std::vector<std::vector<double>> h_V;                    // star form staging per query
    // device inputs
    DevBuf d_in;                         // bounds or V
    DevBuf d_in_meta;                    // star form: pl, pu
    bool uploaded = false;
    // working state: the buffers live in the context (one reach at a time per context)
    WorkBufs* wk = nullptr;
    int list_cur = 0;
    // Column cohorts: runs of columns born together (centres, input generators, the columns of each
    // ReLU layer).  A windowed cohort's columns are exactly zero outside a wh x ww window whose origin
    // is kept per column (WorkBufs::box); the layer kernels then compute only the part that can be non-zero.
    // clean: the memory outside the columns' windows is known to hold zeros (false after a windowed launch
    // that wrote the windows only; readers then go by the windows, see ensure_clean)
    // qn: columns per query (they are stored query by query; empty for the centres)
    struct Cohort {
        int64_t col0, col1;
        bool dense;
        int wh, ww;
        bool clean = true;
        std::vector<int64_t> qn;
        // window-only copy of the columns in wk->pack, written by the convolution in front of a ReLU layer
        // (offset in doubles, -1: none) for the bound reduction; stale once any layer has run
        int64_t pack_off = -1, pack_stride = 0;
        int pack_buf = 0;                // which of wk->pack2 holds it
        // the full-length columns hold the data too (false: the cohort exists in compact form only; a reader
        // that wants columns has them written first, see ensure_full)
        bool full_valid = true;
    };
    std::vector<Cohort> cohorts;
    // work a ReLU step left to the layer that follows it (see relu_step)
    int64_t pend_mask_ncols = 0;         // > 0: rows with state != 0 of columns [0, n) read as zero
    int64_t pend_mask_N = 0;
    bool pend_mask_cf = false;           // wk->state_cf holds the same states in channel-fastest order
    int64_t pend_onehot = 0;             // > 0: the last n columns are implicit unit vectors
    ReluLayerRecord* pend_rec = nullptr; // ... of the neurons listed in this record,
    bool pend_scaled = false;            // ... or (after a pooling layer) of wk->hot_idx, times wk->hot_scale
    std::vector<int64_t> h_qcol_off;     // [nq+1]
    int64_t ncols = 0;
    int64_t N = 0, ld = 0;
    int64_t shape[3] = {0, 0, 0};
    double* V = nullptr;                 // current generator matrix (device)
    bool reached = false;
    nnvb_opts opts{};
    // final output ranges cache
    bool have_out_ranges = false;
    // LP-tightened bounds (nnvb_batch_set_bounds_hook): the hook runs inside relu_step, between the
    // classification by estimated ranges and the relaxation
    nnvb_bounds_fn bounds_fn = nullptr;
    void* bounds_user = nullptr;
    int hook_layer = -1;                 // >= 0: the hook of this ReLU layer is running
    bool hook_tightened = false;
    ReluWork hook_w{};                   // the layer's working set while the hook runs
};

namespace {

// number of indices r in [0, n) with r % world == rank
inline int64_t shard_count(int64_t n, int rank, int world) { return n > rank ? (n - rank + world - 1) / world : 0; }

// Scoped device timer for one kernel family: records an event pair on the stream
// around the launches issued while it lives.  No-op unless profiling is enabled.
struct ProfScope {
    nnvb_ctx* ctx;
    int fam;
    double work;
    int64_t l0;
    cudaEvent_t a = nullptr, b = nullptr;
    ProfScope(nnvb_ctx* c, int f, double w) : ctx(c), fam(f), work(w), l0(c->launches) {
        if (!ctx->prof_on) return;
        auto get = [&]() {
            cudaEvent_t e = nullptr;
            if (!ctx->prof_pool.empty()) { e = ctx->prof_pool.back(); ctx->prof_pool.pop_back(); }
            else cudaEventCreate(&e);
            return e;
        };
        a = get(); b = get();
        cudaEventRecord(a, ctx->stream);
    }
    // nothing was launched after all: the scope records no work
    void cancel() {
        if (!a) return;
        ctx->prof_pool.push_back(a);
        ctx->prof_pool.push_back(b);
        a = b = nullptr;
    }
    ~ProfScope() {
        if (!a) return;
        cudaEventRecord(b, ctx->stream);
        ctx->prof_recs.push_back({fam, a, b, work});
        ctx->prof_launches[fam] += ctx->launches - l0;
    }
};

void prof_drain(nnvb_ctx* ctx) {
    for (auto& r : ctx->prof_recs) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
            ctx->prof_ms[r.fam] += ms;
            ctx->prof_work[r.fam] += r.work;
        }
        ctx->prof_pool.push_back(r.a);
        ctx->prof_pool.push_back(r.b);
    }
    ctx->prof_recs.clear();
}

template <typename T>
int upload_vec(nnvb_net* net, const std::vector<T>& v, T** out) {
    void* d = nullptr;
    size_t bytes = std::max<size_t>(v.size() * sizeof(T), 16);
    NNVB_CUDA(cudaMalloc(&d, bytes));
    net->owned.push_back(d);
    if (!v.empty()) NNVB_CUDA(cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
    *out = static_cast<T*>(d);
    return NNVB_OK;
}

int capacity_error(const char* what, size_t need, size_t have) {
    set_error("%s needs %zu bytes, generator buffer holds %zu", what, need, have);
    return NNVB_E_CAPACITY;
}

int sync(nnvb_ctx* ctx) {
    NNVB_CUDA(cudaStreamSynchronize(ctx->stream));
    ctx->scratch_off = 0;   // every staged upload has landed
    if (!ctx->prof_recs.empty()) prof_drain(ctx);
    return NNVB_OK;
}

// Async H2D of a small host array through the context's pinned scratch.  Space
// is handed out linearly and only recycled after a stream sync, so uploads that
// are still in flight are never overwritten.
int h2d_small(nnvb_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (bytes == 0) return NNVB_OK;
    size_t o = (ctx->scratch_off + 63) / 64 * 64;
    if (o + bytes > ctx->scratch.cap) {
        NNVB_TRY(sync(ctx));
        NNVB_TRY(ctx->scratch.ensure(std::max<size_t>(2 * bytes, 1 << 22)));
        o = 0;
    }
    memcpy(static_cast<char*>(ctx->scratch.p) + o, src, bytes);
    NNVB_CUDA(cudaMemcpyAsync(dst, static_cast<char*>(ctx->scratch.p) + o, bytes, cudaMemcpyHostToDevice,
                              ctx->stream));
    ctx->scratch_off = o + bytes;
    return NNVB_OK;
}

int assemble_constraints(nnvb_batch* b, int q, int n_layers, int64_t* m_out, double* Cmat, double* d);
int forward_points(nnvb_net* net, WorkBufs* wk, nnvb_batch* b, int n, const int32_t* d_pair_q, double** X, int64_t* ldx,
                   const double* d_r, const int64_t* d_roff, double* d_alpha);

// Copy the centre (center_col >= 0) and the P_loc listed columns into out[N x (P+1)], each generator
// at its position in the query's predicate order (out is zero filled beforehand).
__global__ void gather_cols_kernel(int64_t N, int64_t ld, const double* __restrict__ V, int center_col,
                                   const int32_t* __restrict__ list, const int64_t* __restrict__ col_pos,
                                   int64_t P_loc, double* __restrict__ out) {
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= N) return;
    for (int64_t t = blockIdx.y; t <= P_loc; t += gridDim.y) {
        if (t == 0) {
            if (center_col >= 0) out[i] = V[int64_t(center_col) * ld + i];
        } else {
            const int64_t col = list[t - 1];
            out[(1 + col_pos[col]) * N + i] = V[col * ld + i];
        }
    }
}

__global__ void gather_vec_kernel(int64_t P_loc, int64_t P, const int32_t* __restrict__ list,
                                  const int64_t* __restrict__ col_pos, const double* __restrict__ a,
                                  const double* __restrict__ b, double* __restrict__ out) {
    const int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= P_loc) return;
    const int64_t pos = col_pos[list[t]];
    out[pos] = a[list[t]];
    out[P + pos] = b[list[t]];
}

}  // namespace

// ===========================================================================
// C ABI

extern "C" {

const char* nnvb_last_error(void) { return g_err; }

const char* nnvb_strerror(int status) {
    switch (status) {
        case NNVB_OK: return "ok";
        case NNVB_E_ARG: return "invalid argument";
        case NNVB_E_CUDA: return "CUDA runtime error";
        case NNVB_E_CAPACITY: return "set outgrew the device arena";
        case NNVB_E_STATE: return "call order violated";
        case NNVB_E_UNSUPPORTED: return "unsupported layer or option";
        default: return "unknown status";
    }
}

int nnvb_abi_version(void) { return 2; }

int nnvb_init(int device, size_t arena_bytes, nnvb_ctx** out) {
    NNVB_REQUIRE(out != nullptr, "nnvb_init: out is NULL");
    *out = nullptr;
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0) {
        set_error("no CUDA device available (%s); this engine has no CPU path",
                  e != cudaSuccess ? cudaGetErrorString(e) : "device count 0");
        cudaGetLastError();
        return NNVB_E_CUDA;
    }
    NNVB_REQUIRE(device >= 0 && device < ndev, "nnvb_init: device %d out of range (%d devices)", device, ndev);
    NNVB_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    NNVB_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        set_error("device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
        return NNVB_E_UNSUPPORTED;
    }
    auto ctx = new nnvb_ctx();
    ctx->device = device;
    ctx->sm_count = std::max(1, prop.multiProcessorCount);
    NNVB_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
    if (arena_bytes == 0) {
        size_t free_b = 0, total_b = 0;
        NNVB_CUDA(cudaMemGetInfo(&free_b, &total_b));
        arena_bytes = free_b / 2;
    }
    arena_bytes = arena_bytes / 512 * 512;
    e = cudaMalloc(reinterpret_cast<void**>(&ctx->arena), arena_bytes);
    if (e != cudaSuccess) {
        set_error("arena allocation of %zu bytes failed: %s", arena_bytes, cudaGetErrorString(e));
        cudaGetLastError();
        cudaStreamDestroy(ctx->stream);
        delete ctx;
        return NNVB_E_CAPACITY;
    }
    ctx->arena_bytes = arena_bytes;
    int s = ctx->scratch.ensure(1 << 22);
    if (s != NNVB_OK) return s;
    *out = ctx;
    return NNVB_OK;
}

int nnvb_destroy(nnvb_ctx* ctx) {
    if (!ctx) return NNVB_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    ctx->scratch.release();
    ctx->work.release();
    ctx->plane.release();
    ctx->shard_flag.release();
    prof_drain(ctx);
    for (cudaEvent_t e : ctx->prof_pool) cudaEventDestroy(e);
    for (auto& x : ctx->spare_pinned) x.release();
    for (auto& x : ctx->spare_dev) x.release();
    if (ctx->arena) cudaFree(ctx->arena);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return NNVB_OK;
}

int nnvb_profile_enable(nnvb_ctx* ctx, int on) {
    NNVB_REQUIRE(ctx, "nnvb_profile_enable: NULL context");
    NNVB_CUDA(cudaSetDevice(ctx->device));
    NNVB_TRY(sync(ctx));
    ctx->prof_on = on != 0;
    for (int f = 0; f < NNVB_PROF_FAMILIES; ++f) { ctx->prof_ms[f] = 0; ctx->prof_work[f] = 0; ctx->prof_launches[f] = 0; }
    return NNVB_OK;
}

int nnvb_profile_read(nnvb_ctx* ctx, int family, double* ms, int64_t* launches, double* work) {
    NNVB_REQUIRE(ctx && family >= 0 && family < NNVB_PROF_FAMILIES, "nnvb_profile_read: bad argument");
    NNVB_CUDA(cudaSetDevice(ctx->device));
    NNVB_TRY(sync(ctx));
    if (ms) *ms = ctx->prof_ms[family];
    if (launches) *launches = ctx->prof_launches[family];
    if (work) *work = ctx->prof_work[family];
    return NNVB_OK;
}

int nnvb_set_shard(nnvb_ctx* ctx, int rank, int world, nnvb_allreduce_fn fn, void* user) {
    NNVB_REQUIRE(ctx, "nnvb_set_shard: NULL context");
    NNVB_REQUIRE(world >= 1 && rank >= 0 && rank < world, "nnvb_set_shard: rank %d of %d", rank, world);
    NNVB_REQUIRE(world == 1 || fn != nullptr, "nnvb_set_shard: an all-reduce hook is required when world > 1");
    ctx->plane.release();
    ctx->rank = rank;
    ctx->world = world;
    ctx->ar_fn = fn;
    ctx->ar_user = user;
    ctx->result_owner = nullptr;
    return NNVB_OK;
}

int nnvb_nccl_unique_id(void* id_out) {
    NNVB_REQUIRE(id_out, "nnvb_nccl_unique_id: NULL output");
    return nccl_unique_id(id_out);
}

int nnvb_set_shard_nccl(nnvb_ctx* ctx, int rank, int world, const void* nccl_id, int peer_memory) {
    NNVB_REQUIRE(ctx, "nnvb_set_shard_nccl: NULL context");
    NNVB_REQUIRE(world >= 1 && world <= MAX_SHARD_RANKS && rank >= 0 && rank < world,
                 "nnvb_set_shard_nccl: rank %d of %d (at most %d ranks)", rank, world, MAX_SHARD_RANKS);
    NNVB_REQUIRE(world == 1 || nccl_id != nullptr, "nnvb_set_shard_nccl: the communicator id is required when world > 1");
    NNVB_CUDA(cudaSetDevice(ctx->device));
    NNVB_TRY(sync(ctx));
    ctx->plane.release();
    ctx->rank = rank;
    ctx->world = world;
    ctx->ar_fn = nullptr;
    ctx->ar_user = nullptr;
    ctx->result_owner = nullptr;
    if (world > 1) {
        NNVB_TRY(ctx->plane.init(rank, world, nccl_id));
        ctx->plane.want_p2p = peer_memory != 0;
    }
    return NNVB_OK;
}

void* nnvb_stream(nnvb_ctx* ctx) { return ctx ? static_cast<void*>(ctx->stream) : nullptr; }
int64_t nnvb_launch_count(nnvb_ctx* ctx) { return ctx ? ctx->launches : 0; }

// ---------------------------------------------------------------------------
// network

int nnvb_net_create(nnvb_ctx* ctx, const nnvb_layer_desc* layers, int n_layers, int64_t in_h, int64_t in_w,
                    int64_t in_c, nnvb_net** out) {
    NNVB_REQUIRE(ctx && out && (layers || n_layers == 0), "nnvb_net_create: NULL argument");
    NNVB_REQUIRE(in_h > 0 && in_w > 0 && in_c > 0, "nnvb_net_create: bad input shape");
    *out = nullptr;
    NNVB_CUDA(cudaSetDevice(ctx->device));
    std::unique_ptr<nnvb_net> net(new nnvb_net());
    net->ctx = ctx;
    net->in_shape[0] = in_h; net->in_shape[1] = in_w; net->in_shape[2] = in_c;
    int64_t H = in_h, W = in_w, C = in_c;
    auto fail = [&](int s) {
        for (void* p : net->owned) cudaFree(p);
        return s;
    };
    for (int li = 0; li < n_layers; ++li) {
        const nnvb_layer_desc& d = layers[li];
        Layer L;
        L.type = d.type;
        L.H = H; L.W = W; L.C = C;
        switch (d.type) {
            case NNVB_LAYER_CONV2D: {
                if (!(d.W && d.b && d.kh > 0 && d.kw > 0 && d.cin > 0 && d.cout > 0 && d.stride[0] > 0 &&
                      d.stride[1] > 0 && d.dilation[0] > 0 && d.dilation[1] > 0)) {
                    set_error("layer %d (conv2d): bad parameters", li);
                    return fail(NNVB_E_ARG);
                }
                if (d.cin != C) {
                    // Conv2DLayer.m:571-573
                    set_error("layer %d: input set contains %lld channels while the convolutional layer has %d channels",
                              li, (long long)C, d.cin);
                    return fail(NNVB_E_ARG);
                }
                ConvGeom& g = L.cg;
                g.H = (int)H; g.W = (int)W; g.Cin = (int)C;
                g.kh = d.kh; g.kw = d.kw; g.Cout = d.cout;
                g.pad_t = d.pad[0]; g.pad_l = d.pad[2];
                g.sh = d.stride[0]; g.sw = d.stride[1];
                g.dh = d.dilation[0]; g.dw = d.dilation[1];
                const int64_t hp = H + d.pad[0] + d.pad[1], wp = W + d.pad[2] + d.pad[3];
                const int64_t ho = (hp - int64_t(d.kh - 1) * g.dh - 1);
                const int64_t wo = (wp - int64_t(d.kw - 1) * g.dw - 1);
                if (ho < 0 || wo < 0) {
                    set_error("layer %d (conv2d): filter larger than padded input", li);
                    return fail(NNVB_E_ARG);
                }
                g.Ho = int(ho / g.sh + 1);
                g.Wo = int(wo / g.sw + 1);
                L.Ho = g.Ho; L.Wo = g.Wo; L.Co = g.Cout;
                int bn_tile, cs, n_tiles, n_chunks;
                const size_t nd = conv_weights_doubles(g, &bn_tile, &cs, &n_tiles, &n_chunks);
                std::vector<double> arranged(nd);
                conv_arrange_weights(g, d.W, arranged.data(), bn_tile, cs, n_tiles, n_chunks);
                int s = upload_vec(net.get(), arranged, &L.cw.w);
                if (s) return fail(s);
                std::vector<double> bias(d.b, d.b + d.cout);
                s = upload_vec(net.get(), bias, &L.cw.bias);
                if (s) return fail(s);
                L.cw.bn_tile = bn_tile; L.cw.cs = cs; L.cw.n_tiles = n_tiles; L.cw.n_chunks = n_chunks;
                if (g.sh == 1 && g.sw == 1 && g.dh == 1 && g.dw == 1) {
                    // footprints of unit vectors: the filter flipped in both directions, per input channel
                    std::vector<double> foot(size_t(d.cin) * d.kw * d.kh * d.cout);
                    for (int ci = 0; ci < d.cin; ++ci)
                        for (int owl = 0; owl < d.kw; ++owl)
                            for (int ohl = 0; ohl < d.kh; ++ohl)
                                for (int co = 0; co < d.cout; ++co)
                                    foot[((size_t(ci) * d.kw + owl) * d.kh + ohl) * d.cout + co] =
                                        d.W[size_t(d.kh - 1 - ohl) + size_t(d.kh) * ((d.kw - 1 - owl) + size_t(d.kw) * (ci + size_t(d.cin) * co))];
                    s = upload_vec(net.get(), foot, &L.cw.foot);
                    if (s) return fail(s);
                }
                break;
            }
            case NNVB_LAYER_FC: {
                const int64_t In = H * W * C;
                if (!(d.W && d.b && d.cout > 0)) {
                    set_error("layer %d (fc): bad parameters", li);
                    return fail(NNVB_E_ARG);
                }
                if (d.cin != In) {
                    // FullyConnectedLayer.m:307-309
                    set_error("layer %d: inconsistency between the size of the input image (%lld) and the InputSize of the layer (%d)",
                              li, (long long)In, d.cin);
                    return fail(NNVB_E_ARG);
                }
                const int Out = d.cout;
                const int ldw = (int)round_up(Out, 8);
                const int64_t In_pad = round_up(In, 16);
                // one more row than the padded input size: a row of zeros for the gathered FC, whose bulk copies
                // cannot zero-fill the weight rows of positions off the image
                std::vector<double> wt(size_t(In_pad + 1) * ldw, 0.0);
                for (int64_t k = 0; k < In; ++k)
                    for (int o = 0; o < Out; ++o) wt[size_t(k) * ldw + o] = d.W[size_t(o) + size_t(Out) * k];
                int s = upload_vec(net.get(), wt, &L.fc_wt);
                if (s) return fail(s);
                std::vector<double> bias(d.b, d.b + Out);
                s = upload_vec(net.get(), bias, &L.bias);
                if (s) return fail(s);
                L.fc_ldw = ldw;
                L.Ho = 1; L.Wo = 1; L.Co = Out;
                break;
            }
            case NNVB_LAYER_BN: {
                if (!(d.bn_mean && d.bn_var && d.bn_scale && d.bn_offset)) {
                    set_error("layer %d (bn): missing parameters", li);
                    return fail(NNVB_E_ARG);
                }
                // parameters per channel; a 1x1xN set takes N parameters (BatchNormalizationLayer.m:289-302)
                const int64_t nch = C;
                if (d.cout != 0 && d.cout != nch) {
                    set_error("layer %d (bn): %d channels of parameters for a set with %lld channels", li, d.cout,
                              (long long)nch);
                    return fail(NNVB_E_ARG);
                }
                std::vector<double> mean(d.bn_mean, d.bn_mean + nch), den(nch), scale(d.bn_scale, d.bn_scale + nch),
                    offset(d.bn_offset, d.bn_offset + nch);
                for (int64_t c = 0; c < nch; ++c) den[c] = std::sqrt(d.bn_var[c] + d.bn_eps);
                int s = upload_vec(net.get(), mean, &L.bn_mean);
                if (!s) s = upload_vec(net.get(), den, &L.bn_den);
                std::vector<double> rden(nch);
                for (int64_t c = 0; c < nch; ++c) rden[c] = 1.0 / den[c];
                if (!s) s = upload_vec(net.get(), rden, &L.bn_rden);
                if (!s) s = upload_vec(net.get(), scale, &L.bn_scale);
                if (!s) s = upload_vec(net.get(), offset, &L.bn_offset);
                if (s) return fail(s);
                L.Ho = H; L.Wo = W; L.Co = C;
                if (!net->layers.empty() && net->layers.back().type == NNVB_LAYER_CONV2D &&
                    net->layers.back().fused_bn < 0) {
                    L.fused_into_prev = true;
                    net->layers.back().fused_bn = li;
                }
                break;
            }
            case NNVB_LAYER_AVGPOOL2D: {
                if (!(d.pool[0] > 0 && d.pool[1] > 0 && d.stride[0] > 0 && d.stride[1] > 0)) {
                    set_error("layer %d (avgpool): bad parameters", li);
                    return fail(NNVB_E_ARG);
                }
                PoolGeom& g = L.pg;
                g.H = (int)H; g.W = (int)W; g.C = (int)C;
                g.ph = d.pool[0]; g.pw = d.pool[1];
                g.sh = d.stride[0]; g.sw = d.stride[1];
                g.pad_t = d.pad[0]; g.pad_l = d.pad[2];
                if (d.avgpool_divisor != NNVB_POOL_DIV_WINDOW && d.avgpool_divisor != NNVB_POOL_DIV_INSIDE) {
                    set_error("layer %d (avgpool): unknown divisor rule %d", li, d.avgpool_divisor);
                    return fail(NNVB_E_ARG);
                }
                g.clip = d.avgpool_divisor == NNVB_POOL_DIV_INSIDE ? 1 : 0;
                // a window that lies in the padding altogether has no entry to average
                if (d.pad[0] >= g.ph || d.pad[1] >= g.ph || d.pad[2] >= g.pw || d.pad[3] >= g.pw) {
                    set_error("layer %d (avgpool): padding must be smaller than the pooling window", li);
                    return fail(NNVB_E_ARG);
                }
                const int64_t hp = H + d.pad[0] + d.pad[1], wp = W + d.pad[2] + d.pad[3];
                if (hp < g.ph || wp < g.pw) {
                    set_error("layer %d (avgpool): window larger than padded input", li);
                    return fail(NNVB_E_ARG);
                }
                g.Ho = int((hp - g.ph) / g.sh + 1);
                g.Wo = int((wp - g.pw) / g.sw + 1);
                L.Ho = g.Ho; L.Wo = g.Wo; L.Co = C;
                break;
            }
            case NNVB_LAYER_RELU:
                L.Ho = H; L.Wo = W; L.Co = C;
                net->n_relu += 1;
                break;
            default:
                set_error("layer %d: type %d is outside the approx-star path of this engine", li, d.type);
                return fail(NNVB_E_UNSUPPORTED);
        }
        H = L.Ho; W = L.Wo; C = L.Co;
        net->layers.push_back(L);
    }
    net->out_shape[0] = H; net->out_shape[1] = W; net->out_shape[2] = C;
    *out = net.release();
    return NNVB_OK;
}

int nnvb_net_destroy(nnvb_net* net) {
    if (!net) return NNVB_OK;
    cudaSetDevice(net->ctx->device);
    cudaStreamSynchronize(net->ctx->stream);
    for (void* p : net->owned) cudaFree(p);
    delete net;
    return NNVB_OK;
}

int nnvb_net_evaluate(nnvb_net* net, int64_t n_points, const double* X, double* Y) {
    NNVB_REQUIRE(net && X && Y, "nnvb_net_evaluate: NULL argument");
    NNVB_REQUIRE(n_points >= 1, "nnvb_net_evaluate: need at least one input");
    nnvb_ctx* ctx = net->ctx;
    NNVB_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t st = ctx->stream;
    const int64_t N0 = net->in_shape[0] * net->in_shape[1] * net->in_shape[2], ld0 = lead_dim(N0);
    const int64_t Nout = net->out_shape[0] * net->out_shape[1] * net->out_shape[2];
    int64_t max_ld = ld0;
    for (const Layer& L : net->layers) max_ld = std::max(max_ld, lead_dim(L.Ho * L.Wo * L.Co));
    // slices of the inputs that bound the two working buffers to about 2 GiB each
    const int64_t cap = std::max<int64_t>(1, std::min<int64_t>((int64_t(1) << 31) / (max_ld * 8), 1 << 20));
    WorkBufs* wk = &ctx->work;
    for (int64_t p0 = 0; p0 < n_points; p0 += cap) {
        const int n = int(std::min(cap, n_points - p0));
        NNVB_TRY(wk->wit[0].ensure(sizeof(double) * max_ld * n, st));
        NNVB_TRY(wk->wit[1].ensure(sizeof(double) * max_ld * n, st));
        NNVB_CUDA(cudaMemcpy2DAsync(wk->wit[0].p, sizeof(double) * ld0, X + p0 * N0, sizeof(double) * N0,
                                    sizeof(double) * N0, size_t(n), cudaMemcpyHostToDevice, st));
        double* out = nullptr;
        int64_t ldx = 0;
        NNVB_TRY(forward_points(net, wk, nullptr, n, nullptr, &out, &ldx, nullptr, nullptr, nullptr));
        NNVB_CUDA(cudaMemcpy2DAsync(Y + p0 * Nout, sizeof(double) * Nout, out, sizeof(double) * ldx,
                                    sizeof(double) * Nout, size_t(n), cudaMemcpyDeviceToHost, st));
        NNVB_TRY(sync(ctx));
    }
    return NNVB_OK;
}

int nnvb_net_out_shape(const nnvb_net* net, int64_t shape[3]) {
    NNVB_REQUIRE(net && shape, "nnvb_net_out_shape: NULL argument");
    for (int i = 0; i < 3; ++i) shape[i] = net->out_shape[i];
    return NNVB_OK;
}

// ---------------------------------------------------------------------------
// batches

int nnvb_batch_create(nnvb_net* net, int n_queries, nnvb_batch** out) {
    NNVB_REQUIRE(net && out, "nnvb_batch_create: NULL argument");
    NNVB_REQUIRE(n_queries > 0, "nnvb_batch_create: need at least one query");
    auto b = new nnvb_batch();
    b->net = net;
    b->nq = n_queries;
    b->N0 = net->in_shape[0] * net->in_shape[1] * net->in_shape[2];
    b->ld0 = lead_dim(b->N0);
    b->P0.assign(n_queries, 0);
    b->P0_loc.assign(n_queries, 0);
    b->h_Pglob.assign(n_queries, 0);
    b->is_set.assign(n_queries, 0);
    b->h_pl.resize(n_queries); b->h_pu.resize(n_queries);
    b->h_C.resize(n_queries); b->h_d.resize(n_queries);
    b->h_V.resize(n_queries);
    b->m0.assign(n_queries, 0);
    b->box_implies_C.assign(n_queries, 1);
    b->wk = &net->ctx->work;
    nnvb_ctx* ctx = net->ctx;
    if (!ctx->spare_pinned.empty()) { b->h_in = ctx->spare_pinned.back(); ctx->spare_pinned.pop_back(); }
    for (DevBuf* d : {&b->d_in, &b->d_in_meta, &b->d_in_pos}) {
        if (ctx->spare_dev.empty()) break;
        *d = ctx->spare_dev.back();            // largest first: d_in is the big one
        ctx->spare_dev.pop_back();
    }
    *out = b;
    return NNVB_OK;
}

int nnvb_batch_destroy(nnvb_batch* b) {
    if (!b) return NNVB_OK;
    nnvb_ctx* ctx = b->net->ctx;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    // keep the buffers of up to four batches for the next ones (ascending by size, so that the largest is taken first)
    if (b->h_in.p && ctx->spare_pinned.size() < 4) ctx->spare_pinned.push_back(b->h_in);
    else b->h_in.release();
    for (DevBuf* d : {&b->d_in_pos, &b->d_in_meta, &b->d_in}) {
        if (d->p && ctx->spare_dev.size() < 12) ctx->spare_dev.push_back(*d);
        else d->release();
    }
    std::sort(ctx->spare_dev.begin(), ctx->spare_dev.end(), [](const DevBuf& x, const DevBuf& y) { return x.cap < y.cap; });
    if (ctx->result_owner == b) ctx->result_owner = nullptr;
    delete b;
    return NNVB_OK;
}

int nnvb_batch_set_bounds(nnvb_batch* b, int q, const double* lb, const double* ub) {
    NNVB_REQUIRE(b && lb && ub, "nnvb_batch_set_bounds: NULL argument");
    NNVB_REQUIRE(q >= 0 && q < b->nq, "nnvb_batch_set_bounds: query %d out of range", q);
    NNVB_REQUIRE(b->kind == 0 || b->kind == 1, "nnvb_batch_set_bounds: batch already holds star-form queries");
    b->kind = 1;
    const int64_t N = b->N0;
    NNVB_TRY(b->h_in.ensure(size_t(b->nq) * 2 * N * sizeof(double), true));
    double* dst = b->h_in.as<double>() + size_t(q) * 2 * N;
    memcpy(dst, lb, N * sizeof(double));
    memcpy(dst + N, ub, N * sizeof(double));
    int64_t P = 0;
    for (int64_t i = 0; i < N; ++i) {
        if (!(lb[i] <= ub[i])) {
            set_error("nnvb_batch_set_bounds: lb > ub (or NaN) at entry %lld", (long long)i);
            return NNVB_E_ARG;
        }
        P += (0.5 * (ub[i] - lb[i]) != 0.0 || N == 1) ? 1 : 0;
    }
    b->P0[q] = P;
    b->m0[q] = 1;                       // Star(lb,ub): C = zeros(1,P), d = 0 (Star.m:229-230)
    b->h_C[q].assign(size_t(P), 0.0);
    b->h_d[q].assign(1, 0.0);
    b->is_set[q] = 1;
    b->uploaded = false;
    b->reached = false;
    return NNVB_OK;
}

int nnvb_batch_set_star(nnvb_batch* b, int q, int64_t P, const double* V, const double* pl, const double* pu,
                        int64_t m, const double* Cmat, const double* d) {
    NNVB_REQUIRE(b && V, "nnvb_batch_set_star: NULL argument");
    NNVB_REQUIRE(q >= 0 && q < b->nq, "nnvb_batch_set_star: query %d out of range", q);
    NNVB_REQUIRE(P >= 0 && m >= 0, "nnvb_batch_set_star: negative size");
    NNVB_REQUIRE(P == 0 || (pl && pu), "nnvb_batch_set_star: predicate bounds missing");
    NNVB_REQUIRE(m == 0 || (Cmat && d), "nnvb_batch_set_star: constraint arrays missing");
    NNVB_REQUIRE(b->kind == 0 || b->kind == 2, "nnvb_batch_set_star: batch already holds bounds-form queries");
    b->kind = 2;
    const int64_t N = b->N0;
    b->h_V[q].assign(V, V + size_t(N) * (P + 1));
    b->h_pl[q].assign(pl, pl + P);
    b->h_pu[q].assign(pu, pu + P);
    for (int64_t j = 0; j < P; ++j) {
        if (!(pl[j] <= pu[j])) {
            set_error("nnvb_batch_set_star: pred_lb > pred_ub (or NaN) at predicate %lld", (long long)j);
            return NNVB_E_ARG;
        }
    }
    b->h_C[q].assign(Cmat, Cmat + size_t(m) * P);
    b->h_d[q].assign(d, d + m);
    // a witness at a corner of the predicate box is a point of the set only if the
    // set's own constraints hold on the whole box
    bool implied = true;
    for (int64_t r = 0; r < m && implied; ++r) {
        double mx = 0.0;
        for (int64_t j = 0; j < P; ++j) {
            const double c = Cmat[size_t(j) * m + r];
            mx += std::max(c * pl[j], c * pu[j]);
        }
        implied = mx <= d[r] + 1e-12 * (1.0 + std::fabs(d[r]));
    }
    b->box_implies_C[q] = implied ? 1 : 0;
    b->P0[q] = P;
    b->m0[q] = m;
    b->is_set[q] = 1;
    b->uploaded = false;
    b->reached = false;
    return NNVB_OK;
}

// Queries q0 .. q0+n-1 in one call (the per-set entry points cost a foreign-function call each, which bounds the
// end-to-end rate of batches of thousands of tiny sets).
int nnvb_batch_set_bounds_many(nnvb_batch* b, int q0, int n, const double* lb, const double* ub, int64_t stride) {
    NNVB_REQUIRE(b && lb && ub, "nnvb_batch_set_bounds_many: NULL argument");
    NNVB_REQUIRE(n >= 0 && q0 >= 0 && q0 + n <= b->nq, "nnvb_batch_set_bounds_many: queries %d..%d out of range", q0,
                 q0 + n - 1);
    NNVB_REQUIRE(stride >= b->N0, "nnvb_batch_set_bounds_many: stride %lld below the image size", (long long)stride);
    for (int k = 0; k < n; ++k) NNVB_TRY(nnvb_batch_set_bounds(b, q0 + k, lb + size_t(k) * stride, ub + size_t(k) * stride));
    return NNVB_OK;
}

int nnvb_batch_set_stars(nnvb_batch* b, int q0, int n, int64_t P, int64_t m, const double* V, const double* pl,
                         const double* pu, const double* Cmat, const double* d) {
    NNVB_REQUIRE(b && V, "nnvb_batch_set_stars: NULL argument");
    NNVB_REQUIRE(n >= 0 && q0 >= 0 && q0 + n <= b->nq, "nnvb_batch_set_stars: queries %d..%d out of range", q0,
                 q0 + n - 1);
    NNVB_REQUIRE(P >= 0 && m >= 0, "nnvb_batch_set_stars: negative size");
    const size_t vs = size_t(b->N0) * size_t(P + 1);
    for (int k = 0; k < n; ++k)
        NNVB_TRY(nnvb_batch_set_star(b, q0 + k, P, V + size_t(k) * vs, pl ? pl + size_t(k) * P : nullptr,
                                     pu ? pu + size_t(k) * P : nullptr, m, Cmat ? Cmat + size_t(k) * m * P : nullptr,
                                     d ? d + size_t(k) * m : nullptr));
    return NNVB_OK;
}

int nnvb_batch_upload(nnvb_batch* b) {
    NNVB_REQUIRE(b, "nnvb_batch_upload: NULL argument");
    nnvb_ctx* ctx = b->net->ctx;
    NNVB_CUDA(cudaSetDevice(ctx->device));
    for (int q = 0; q < b->nq; ++q) {
        if (!b->is_set[q]) {
            set_error("nnvb_batch_upload: query %d was never set", q);
            return NNVB_E_STATE;
        }
    }
    const int64_t N = b->N0;
    if (b->kind == 1) {
        const size_t bytes = size_t(b->nq) * 2 * N * sizeof(double);
        NNVB_TRY(b->d_in.ensure(bytes, ctx->stream));
        NNVB_CUDA(cudaMemcpyAsync(b->d_in.p, b->h_in.p, bytes, cudaMemcpyHostToDevice, ctx->stream));
        for (int q = 0; q < b->nq; ++q) b->P0_loc[q] = shard_count(b->P0[q], ctx->rank, ctx->world);
    } else {
        // arrange the batch as one matrix: centres first, then each query's generators
        // (with sharded generators: only the columns j with j % world == rank)
        const int rank = ctx->rank, world = ctx->world;
        int64_t ncols = b->nq;
        for (int q = 0; q < b->nq; ++q) {
            b->P0_loc[q] = shard_count(b->P0[q], rank, world);
            ncols += b->P0_loc[q];
        }
        const size_t vbytes = size_t(b->ld0) * ncols * sizeof(double);
        const size_t mbytes = size_t(ncols) * 2 * sizeof(double);
        const size_t pbytes = size_t(ncols) * sizeof(int64_t);
        NNVB_TRY(b->h_in.ensure(vbytes + mbytes + pbytes));
        double* hv = b->h_in.as<double>();
        double* hm = hv + size_t(b->ld0) * ncols;
        int64_t* hp = reinterpret_cast<int64_t*>(hm + 2 * ncols);
        int64_t col = b->nq;
        for (int q = 0; q < b->nq; ++q) {
            const double* src = b->h_V[q].data();
            memcpy(hv + size_t(q) * b->ld0, src, N * sizeof(double));
            hm[q] = 0.0; hm[ncols + q] = 0.0; hp[q] = 0;
            for (int64_t j = rank; j < b->P0[q]; j += world, ++col) {
                memcpy(hv + size_t(col) * b->ld0, src + size_t(N) * (j + 1), N * sizeof(double));
                hm[col] = b->h_pl[q][j];
                hm[ncols + col] = b->h_pu[q][j];
                hp[col] = j;
            }
        }
        NNVB_TRY(b->d_in.ensure(vbytes, ctx->stream));
        NNVB_TRY(b->d_in_meta.ensure(mbytes, ctx->stream));
        NNVB_TRY(b->d_in_pos.ensure(pbytes, ctx->stream));
        NNVB_CUDA(cudaMemcpyAsync(b->d_in.p, hv, vbytes, cudaMemcpyHostToDevice, ctx->stream));
        NNVB_CUDA(cudaMemcpyAsync(b->d_in_meta.p, hm, mbytes, cudaMemcpyHostToDevice, ctx->stream));
        NNVB_CUDA(cudaMemcpyAsync(b->d_in_pos.p, hp, pbytes, cudaMemcpyHostToDevice, ctx->stream));
    }
    b->uploaded = true;
    b->reached = false;
    return NNVB_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// the layer loop

namespace {

// Sum a device buffer over the ranks of a generator-sharded run (identity when unsharded).
int allreduce(nnvb_ctx* ctx, double* buf, int64_t count) {
    if (ctx->world <= 1 || count <= 0) return NNVB_OK;
    ProfScope ps(ctx, NNVB_PROF_ALLREDUCE, 8.0 * double(count));
    ctx->launches += 1;              // the collective's kernel
    if (ctx->plane.comm) return ctx->plane.allreduce(buf, count, ctx->stream);
    if (!ctx->ar_fn) {
        set_error("generator sharding is on but no all-reduce hook is installed");
        return NNVB_E_STATE;
    }
    const int rc = ctx->ar_fn(ctx->ar_user, buf, count, static_cast<void*>(ctx->stream));
    if (rc != 0) {
        set_error("the all-reduce hook failed with code %d", rc);
        return NNVB_E_CUDA;
    }
    return NNVB_OK;
}

// Sharded runs: a decision to stop must be the same on every rank, or the ranks that go on would wait in the
// next collective for the one that left.  Each rank contributes "I cannot go on" (0/1); the sum comes back.
int shard_agree(nnvb_ctx* ctx, bool local_fail, bool* any_fail) {
    *any_fail = local_fail;
    if (ctx->world <= 1) return NNVB_OK;
    NNVB_TRY(ctx->shard_flag.ensure(sizeof(double), ctx->stream));
    const double mine = local_fail ? 1.0 : 0.0;
    double all = 0.0;
    NNVB_TRY(h2d_small(ctx, ctx->shard_flag.p, &mine, sizeof(double)));
    NNVB_TRY(allreduce(ctx, ctx->shard_flag.as<double>(), 1));
    NNVB_CUDA(cudaMemcpyAsync(&all, ctx->shard_flag.p, sizeof(double), cudaMemcpyDeviceToHost, ctx->stream));
    NNVB_TRY(sync(ctx));
    *any_fail = all > 0.0;
    return NNVB_OK;
}

// Largest generator buffer (bytes) the layers [from, next ReLU layer] need for `ncols` columns of this rank.
size_t segment_need(const nnvb_batch* b, size_t from, int64_t ncols, int64_t ld_now) {
    size_t need = size_t(ld_now) * ncols * sizeof(double);
    const auto& layers = b->net->layers;
    for (size_t li = from; li < layers.size(); ++li) {
        const Layer& L = layers[li];
        if (L.type == NNVB_LAYER_RELU) break;
        need = std::max(need, size_t(lead_dim(L.Ho * L.Wo * L.Co)) * ncols * sizeof(double));
    }
    return need;
}

int ensure_col_meta(nnvb_batch* b, int64_t cols) {
    cudaStream_t st = b->net->ctx->stream;
    NNVB_TRY(b->wk->col_q.ensure(size_t(cols) * sizeof(int32_t), st, true));
    NNVB_TRY(b->wk->pl.ensure(size_t(cols) * sizeof(double), st, true));
    NNVB_TRY(b->wk->pu.ensure(size_t(cols) * sizeof(double), st, true));
    NNVB_TRY(b->wk->col_pos.ensure(size_t(cols) * sizeof(int64_t), st, true));
    NNVB_TRY(b->wk->box.ensure(size_t(cols) * sizeof(int4), st, true));
    for (int i = 0; i < 2; ++i) {
        NNVB_TRY(b->wk->qcol_idx[i].ensure(size_t(cols) * sizeof(int32_t), st, true));
        NNVB_TRY(b->wk->qcol_off[i].ensure(size_t(b->nq + 1) * sizeof(int64_t), st, true));
    }
    return NNVB_OK;
}

// windowed launches skip the zero fill of their output columns unless the caller wants the constraint rows
bool lazy_fill(const nnvb_batch* b) {
    static const bool always_fill = getenv("NNVB_ZERO_FILL") != nullptr;
    return !always_fill && !b->opts.keep_constraints;
}

int init_sets(nnvb_batch* b) {
    nnvb_ctx* ctx = b->net->ctx;
    cudaStream_t st = ctx->stream;
    const int nq = b->nq;
    const int64_t N = b->N0, ld = b->ld0;
    int64_t ncols = nq;
    b->h_qcol_off.assign(nq + 1, 0);
    std::vector<int64_t> gen_off(nq + 1);
    for (int q = 0; q < nq; ++q) {
        gen_off[q] = ncols;
        b->h_qcol_off[q] = ncols - nq;
        ncols += b->P0_loc[q];
        b->h_Pglob[q] = b->P0[q];
    }
    gen_off[nq] = ncols;
    b->h_qcol_off[nq] = ncols - nq;
    NNVB_REQUIRE(ncols < (int64_t(1) << 31), "batch has too many generator columns (%lld)", (long long)ncols);
    NNVB_TRY(ensure_col_meta(b, ncols));
    b->list_cur = 0;
    NNVB_TRY(h2d_small(ctx, b->wk->qcol_off[0].p, b->h_qcol_off.data(), sizeof(int64_t) * (nq + 1)));
    bool implicit = false;               // the generator columns are not stored: the first layer writes their images
    if (b->kind == 1) {
        // a generator of ImageStar(lb,ub) is a half width times a unit vector: when the first layer writes the
        // images of such columns itself, they start out as (entry, half width) pairs and are never stored
        static const bool eager = getenv("NNVB_EAGER_RELU") != nullptr;
        const int t0 = b->net->layers.empty() ? 0 : b->net->layers[0].type;
        implicit = !eager && lazy_fill(b) && ncols > nq && N < (int64_t(1) << 31) &&
                   (t0 == NNVB_LAYER_CONV2D || t0 == NNVB_LAYER_FC || t0 == NNVB_LAYER_AVGPOOL2D);
        const size_t need = size_t(ld) * ((implicit && ctx->world == 1) ? nq : ncols) * sizeof(double);
        {
            bool stop = need > ctx->vbuf_bytes();      // agreed on by all ranks of a sharded run
            const bool mine = stop;
            NNVB_TRY(shard_agree(ctx, stop, &stop));
            if (stop) {
                if (mine) return capacity_error("input set", need, ctx->vbuf_bytes());
                set_error("another rank's share of the set outgrew its arena");
                return NNVB_E_CAPACITY;
            }
        }
        NNVB_TRY(b->wk->gen_off.ensure(sizeof(int64_t) * (nq + 1), st));
        NNVB_TRY(h2d_small(ctx, b->wk->gen_off.p, gen_off.data(), sizeof(int64_t) * (nq + 1)));
        double* V = ctx->vbuf(0);
        if (implicit) {
            NNVB_TRY(b->wk->hot_idx.ensure(sizeof(int32_t) * (ncols - nq), st));
            NNVB_TRY(b->wk->hot_scale.ensure(sizeof(double) * (ncols - nq), st));
        }
        NNVB_CUDA(cudaMemsetAsync(V, 0, size_t(ld) * (implicit ? nq : ncols) * sizeof(double), st));
        NNVB_TRY(launch_build_from_bounds(st, nq, N, ld, b->d_in.as<double>(), b->wk->gen_off.as<int64_t>(), ctx->rank,
                                          ctx->world, V,
                                          b->wk->col_q.as<int32_t>(), b->wk->pl.as<double>(), b->wk->pu.as<double>(),
                                          b->wk->qcol_idx[0].as<int32_t>(), b->wk->col_pos.as<int64_t>(),
                                          int(b->net->in_shape[0]), int(b->net->in_shape[1]),
                                          b->wk->box.as<int4>(), implicit ? b->wk->hot_idx.as<int32_t>() : nullptr,
                                          implicit ? b->wk->hot_scale.as<double>() : nullptr, &ctx->launches));
        b->V = V;
    } else {
        // metadata is a pure function of the staged queries
        std::vector<int32_t> col_q(ncols), list(ncols - nq);
        int64_t col = nq;
        for (int q = 0; q < nq; ++q) {
            col_q[q] = q;
            for (int64_t t = 0; t < b->P0_loc[q]; ++t, ++col) {
                col_q[col] = q;
                list[col - nq] = int32_t(col);
            }
        }
        NNVB_TRY(h2d_small(ctx, b->wk->col_q.p, col_q.data(), sizeof(int32_t) * ncols));
        NNVB_CUDA(cudaMemcpyAsync(b->wk->col_pos.p, b->d_in_pos.p, sizeof(int64_t) * ncols, cudaMemcpyDeviceToDevice, st));
        NNVB_TRY(h2d_small(ctx, b->wk->qcol_idx[0].p, list.data(), sizeof(int32_t) * (ncols - nq)));
        NNVB_CUDA(cudaMemcpyAsync(b->wk->pl.p, b->d_in_meta.p, sizeof(double) * ncols, cudaMemcpyDeviceToDevice, st));
        NNVB_CUDA(cudaMemcpyAsync(b->wk->pu.p, b->d_in_meta.as<double>() + ncols, sizeof(double) * ncols,
                                  cudaMemcpyDeviceToDevice, st));
        NNVB_TRY(launch_fill_dense_windows(st, ncols, b->wk->box.as<int4>(), &ctx->launches));
        b->V = b->d_in.as<double>();      // read-only; in-place layers copy it first
    }
    b->ncols = ncols;
    b->N = N;
    b->ld = ld;
    b->pend_onehot = implicit ? ncols - nq : 0;
    b->pend_scaled = implicit;
    for (int i = 0; i < 3; ++i) b->shape[i] = b->net->in_shape[i];
    // centres are dense; box generators touch one pixel each; general generators are taken as dense
    static const bool no_windows = getenv("NNVB_NO_WINDOWS") != nullptr;
    b->cohorts.clear();
    const int BIG = 1 << 20;      // window size of columns that are dense from the start
    b->cohorts.push_back({0, nq, true, BIG, BIG, true, {}});
    if (ncols > nq) {
        const bool dense0 = b->kind != 1;
        b->cohorts.push_back({nq, ncols, dense0 || no_windows, dense0 ? BIG : 1, dense0 ? BIG : 1, true,
                              std::vector<int64_t>(b->P0_loc.begin(), b->P0_loc.end())});
    }
    return NNVB_OK;
}

// the buffer the next out-of-place layer writes to
double* other_vbuf(nnvb_batch* b) {
    nnvb_ctx* ctx = b->net->ctx;
    return b->V == ctx->vbuf(0) ? ctx->vbuf(1) : ctx->vbuf(0);
}

// Leading columns whose full-length storage is in use: cohorts kept in compact form only, and unit-vector columns
// no layer has written yet, occupy none (a sharded run counts every column: its ranks agree on one figure).
int64_t full_extent(const nnvb_batch* b) {
    if (b->net->ctx->world > 1) return b->ncols;
    int64_t ext = b->nq;
    const int64_t first_hot = b->ncols - b->pend_onehot;
    for (const auto& co : b->cohorts)
        if (co.full_valid && co.col0 < first_hot) ext = std::max(ext, std::min(co.col1, first_hot));
    return ext;
}

int make_writable(nnvb_batch* b, int64_t extra_cols) {
    nnvb_ctx* ctx = b->net->ctx;
    const size_t need = size_t(b->ld) * (full_extent(b) + extra_cols) * sizeof(double);
    if (need > ctx->vbuf_bytes()) return capacity_error("generator matrix", need, ctx->vbuf_bytes());
    if (b->V != ctx->vbuf(0) && b->V != ctx->vbuf(1)) {
        double* dst = ctx->vbuf(0);
        NNVB_CUDA(cudaMemcpyAsync(dst, b->V, size_t(b->ld) * b->ncols * sizeof(double), cudaMemcpyDeviceToDevice,
                                  ctx->stream));
        b->V = dst;
    }
    return NNVB_OK;
}

// lazy_mask: do not clear the dead/crossing rows in memory; the next layer reads them as zero.
// lazy_onehot: do not materialise the appended unit-vector columns; the next layer writes their images.
// Windowed launches write the columns' windows only.  A reader that does not go by the windows first has
// the rest of those columns cleared.
// A cohort kept in compact form only gets its full-length columns written (windows only when the run fills
// lazily: the memory outside the windows then stays stale, as after any windowed launch).
int ensure_full(nnvb_batch* b, nnvb_batch::Cohort& co) {
    if (co.full_valid) return NNVB_OK;
    nnvb_ctx* ctx = b->net->ctx;
    if (co.pack_off < 0) {
        set_error("internal: a cohort has neither compact nor full-length storage");
        return NNVB_E_STATE;
    }
    NNVB_TRY(make_writable(b, 0));
    {
        const size_t need = size_t(b->ld) * co.col1 * sizeof(double);
        if (need > ctx->vbuf_bytes()) return capacity_error("columns of a cohort kept in compact form", need, ctx->vbuf_bytes());
    }
    const bool clear = !lazy_fill(b);
    ProfScope ps(ctx, NNVB_PROF_RELAX, 16.0 * double(co.pack_stride) * double(co.col1 - co.col0));
    NNVB_TRY(launch_expand_compact(ctx->stream, int(b->shape[0]), int(b->shape[1]), int(b->shape[2]), b->wk->box.as<int4>(),
                                   co.col0, co.col1 - co.col0, co.wh, co.ww,
                                   b->wk->pack2[co.pack_buf].as<double>() + co.pack_off, co.pack_stride, b->V, b->ld, clear,
                                   &ctx->launches));
    co.full_valid = true;
    co.clean = clear;
    return NNVB_OK;
}

int ensure_clean(nnvb_batch* b, nnvb_batch::Cohort& co) {
    NNVB_TRY(ensure_full(b, co));
    if (co.clean) return NNVB_OK;
    nnvb_ctx* ctx = b->net->ctx;
    NNVB_TRY(launch_zero_outside_windows(ctx->stream, int(b->shape[0]), int(b->shape[1]), int(b->shape[2]),
                                         b->wk->box.as<int4>(), co.col0, co.col1 - co.col0, b->V, b->ld, &ctx->launches));
    co.clean = true;
    return NNVB_OK;
}

int relu_step_finish(nnvb_batch* b, ReluLayerRecord* rec, bool lazy_mask, bool lazy_onehot, size_t next_layer, ReluWork& w,
                     const std::vector<int64_t>& dead);

int relu_step(nnvb_batch* b, ReluLayerRecord* rec, bool lazy_mask, bool lazy_onehot, size_t next_layer, int relu_index) {
    nnvb_ctx* ctx = b->net->ctx;
    cudaStream_t st = ctx->stream;
    const int nq = b->nq;
    const int64_t N = b->N, ld = b->ld;
    NNVB_TRY(make_writable(b, 0));

    // Cohorts reduced through their windows: narrow windows on a wide set (see range_windows_kernel).
    static const bool no_skip = getenv("NNVB_NO_RANGE_SKIP") != nullptr;
    const int64_t img_h = b->shape[0], img_w = b->shape[1], img_c = b->shape[2];
    WinCohorts wc{};
    std::vector<char> is_win(b->cohorts.size(), 0);
    std::vector<int32_t> win_seg;
    {
        int64_t bin_base = 0;
        for (size_t k = 0; k < b->cohorts.size(); ++k) {
            auto& co = b->cohorts[k];
            const bool ok = !no_skip && !co.qn.empty() && N >= 256 && img_h * img_w * img_c == N && img_c <= 1024 &&
                            co.wh <= MAX_WIN_EXTENT && co.ww <= MAX_WIN_EXTENT &&
                            2 * int64_t(co.wh) * co.ww <= img_h * img_w && wc.n < MAX_WIN_COHORTS &&
                            !b->opts.keep_constraints && co.col1 > co.col0;
            if (!ok) continue;
            is_win[k] = 1;
            WinCohort& d = wc.c[wc.n++];
            d.col0 = co.col0; d.n = co.col1 - co.col0;
            d.wh = co.wh; d.ww = co.ww;
            d.KH = int(img_h) + co.wh - 1; d.KW = int(img_w) + co.ww - 1;
            d.bin_base = bin_base;
            d.pack_off = co.pack_off;
            d.pack_stride = co.pack_stride;
            bin_base += int64_t(nq) * (int64_t(d.KH) * d.KW + 1);
            int64_t c = co.col0;
            for (int q = 0; q < nq; ++q) { win_seg.push_back(int32_t(c)); c += co.qn[q]; }
        }
    }
    const int win_slices = wc.n > 0 ? range_windows_slices(int(img_h), int(img_w), int(img_c), nq, ctx->sm_count) : 0;
    // every other cohort is read as whole columns
    for (size_t k = 0; k < b->cohorts.size(); ++k)
        if (!is_win[k]) NNVB_TRY(ensure_clean(b, b->cohorts[k]));

    // chunk list: split the rest of every query's column list so that the grid fills the GPU; the windowed
    // cohorts of a query fill a few more chunks, its last
    const int64_t row_blocks = N >= 2048 ? ceil_div(ceil_div(N, 2), 256) : ceil_div(N, 32);
    int64_t total_P = 0, max_P = 0;
    for (int q = 0; q < nq; ++q) {
        int64_t pq = 0;
        for (size_t k = 0; k < b->cohorts.size(); ++k)
            if (!is_win[k] && !b->cohorts[k].qn.empty()) pq += b->cohorts[k].qn[q];
        total_P += pq;
        max_P = std::max(max_P, pq);
    }
    const int64_t want_chunks = std::max<int64_t>(1, ceil_div(int64_t(ctx->sm_count) * 16, row_blocks));
    int64_t CH = std::max<int64_t>(32, ceil_div(total_P, want_chunks));
    CH = std::min<int64_t>(CH, 1024);
    // the classify kernel adds a query's chunk partials one after the other: at most 96 chunks per query
    CH = std::max(CH, ceil_div(max_P, int64_t(96)));
    std::vector<int64_t> cbeg, cend;
    std::vector<int32_t> qoff(nq + 1);
    for (int q = 0; q < nq; ++q) {
        qoff[q] = (int32_t)cbeg.size();
        int64_t pos = b->h_qcol_off[q];          // the list of a query holds its cohorts one after the other
        for (size_t k = 0; k < b->cohorts.size(); ++k) {
            if (b->cohorts[k].qn.empty()) continue;
            const int64_t pend = pos + b->cohorts[k].qn[q];
            if (!is_win[k])
                for (int64_t p0 = pos; p0 < pend; p0 += CH) {
                    cbeg.push_back(p0);
                    cend.push_back(std::min(p0 + CH, pend));
                }
            pos = pend;
        }
        if (pos != b->h_qcol_off[q + 1]) {
            set_error("internal: cohort sizes of query %d do not add up to its column list", q);
            return NNVB_E_STATE;
        }
        for (int sl = 0; sl < win_slices; ++sl) { cbeg.push_back(0); cend.push_back(0); }
    }
    qoff[nq] = (int32_t)cbeg.size();
    const int n_chunks = (int)cbeg.size();
    NNVB_TRY(b->wk->chunk_beg.ensure(sizeof(int64_t) * std::max(n_chunks, 1), st));
    NNVB_TRY(b->wk->chunk_end.ensure(sizeof(int64_t) * std::max(n_chunks, 1), st));
    NNVB_TRY(b->wk->q_chunk_off.ensure(sizeof(int32_t) * (nq + 1), st));
    NNVB_TRY(b->wk->partial.ensure(sizeof(double) * 2 * N * std::max(n_chunks, 1), st));
    NNVB_TRY(h2d_small(ctx, b->wk->chunk_beg.p, cbeg.data(), sizeof(int64_t) * n_chunks));
    NNVB_TRY(h2d_small(ctx, b->wk->chunk_end.p, cend.data(), sizeof(int64_t) * n_chunks));
    NNVB_TRY(h2d_small(ctx, b->wk->q_chunk_off.p, qoff.data(), sizeof(int32_t) * (nq + 1)));

    const int nblk = relu_blocks_per_query(N);
    DevBuf& lbbuf = b->opts.keep_layer_bounds ? rec->lb : b->wk->lb;
    DevBuf& ubbuf = b->opts.keep_layer_bounds ? rec->ub : b->wk->ub;
    NNVB_TRY(lbbuf.ensure(sizeof(double) * nq * N, st));
    NNVB_TRY(ubbuf.ensure(sizeof(double) * nq * N, st));
    rec->has_bounds = b->opts.keep_layer_bounds != 0;
    NNVB_TRY(b->wk->state.ensure(size_t(nq) * N, st));
    DevBuf& rankbuf = b->opts.keep_layer_bounds ? rec->rank : b->wk->rank;
    NNVB_TRY(rankbuf.ensure(sizeof(int32_t) * nq * N, st));
    NNVB_TRY(b->wk->blk_cross.ensure(sizeof(int32_t) * nq * nblk, st));
    NNVB_TRY(b->wk->q_cross.ensure(sizeof(int64_t) * nq, st));
    NNVB_TRY(b->wk->q_dead.ensure(sizeof(int64_t) * nq, st));
    NNVB_TRY(b->wk->q_new_off.ensure(sizeof(int64_t) * (nq + 1), st));

    ReluWork w{};
    w.nq = nq; w.N = N; w.ld = ld; w.V = b->V;
    w.qcol_off = b->wk->qcol_off[b->list_cur].as<int64_t>();
    w.qcol_idx = b->wk->qcol_idx[b->list_cur].as<int32_t>();
    w.pl = b->wk->pl.as<double>(); w.pu = b->wk->pu.as<double>();
    w.box = b->wk->box.as<int4>();
    w.col_q = b->wk->col_q.as<int32_t>();
    w.img_h = int(img_h); w.img_w = int(img_w); w.img_c = int(img_c);
    w.win = wc;
    w.win_slices = win_slices;
    if (wc.n > 0) {
        const size_t ints = range_windows_scratch_ints(wc, nq, b->ncols);
        NNVB_TRY(b->wk->winsort.ensure(sizeof(int32_t) * (ints + win_seg.size()), st));
        w.win_scratch = b->wk->winsort.as<int32_t>();
        int32_t* seg_dev = w.win_scratch + ints;
        NNVB_TRY(h2d_small(ctx, seg_dev, win_seg.data(), sizeof(int32_t) * win_seg.size()));
        w.win_seg = seg_dev;
        // the compact copies are read when every windowed cohort has one (they then sit in one buffer: the
        // layer in front wrote them all); else the cohorts are read from their full-length columns
        bool all_packed = true;
        int buf = -1;
        for (size_t k = 0; k < b->cohorts.size(); ++k) {
            if (!is_win[k]) continue;
            const auto& co = b->cohorts[k];
            all_packed = all_packed && co.pack_off >= 0 && (buf < 0 || buf == co.pack_buf);
            if (co.pack_off >= 0) buf = co.pack_buf;
        }
        w.win_pack = all_packed && buf >= 0 ? b->wk->pack2[buf].as<double>() : nullptr;
        if (w.win_pack == nullptr)
            for (size_t k = 0; k < b->cohorts.size(); ++k)
                if (is_win[k]) NNVB_TRY(ensure_full(b, b->cohorts[k]));
    }
    w.n_chunks = n_chunks;
    w.chunk_beg = b->wk->chunk_beg.as<int64_t>(); w.chunk_end = b->wk->chunk_end.as<int64_t>();
    w.q_chunk_off = b->wk->q_chunk_off.as<int32_t>();
    w.partial = b->wk->partial.as<double>();
    w.lb = lbbuf.as<double>(); w.ub = ubbuf.as<double>();
    w.state = b->wk->state.as<uint8_t>(); w.rank = rankbuf.as<int32_t>();
    w.blk_cross = b->wk->blk_cross.as<int32_t>();
    w.q_cross = b->wk->q_cross.as<int64_t>(); w.q_dead = b->wk->q_dead.as<int64_t>();
    w.q_new_off = b->wk->q_new_off.as<int64_t>();

    bool used_peers = false;
    {
        // Star.estimateRanges: V read once, predicate bounds, lb/ub written
        // bytes: the columns' windows (all of a dense column) read once, predicate bounds, lb/ub written
        double v_bytes = 0.0;
        for (auto& co : b->cohorts) {
            const size_t k = size_t(&co - b->cohorts.data());
            const double px = is_win[k] ? double(co.wh) * co.ww : double(img_h * img_w);
            v_bytes += 8.0 * px * double(img_c) * double(co.col1 - co.col0);
        }
        ProfScope ps(ctx, NNVB_PROF_RANGES, v_bytes + 16.0 * double(b->ncols - nq) + 16.0 * double(N) * nq);
        NNVB_TRY(launch_estimate_ranges(st, w, &ctx->launches));
        if (ctx->world > 1) {
            // sharded generators: every rank holds part of each sum; add them over the ranks, then
            // all ranks classify the same numbers
            ShardPlane& pl = ctx->plane;
            if (pl.p2p_ok && int64_t(2) * N * nq <= pl.cap_doubles) {
                // peer memory: the sums go to this rank's mapped buffer, the flag tells the peers, and the
                // classification adds all ranks' sums itself (no reduction kernel in between)
                ProfScope pa(ctx, NNVB_PROF_ALLREDUCE, 8.0 * 2.0 * double(N) * nq);
                NNVB_TRY(launch_reduce_chunks(st, w, pl.next_slot(), &ctx->launches));
                NNVB_TRY(pl.publish(st, &ctx->launches));
                PeerSums psums{pl.d_peer_tab, pl.slot_offset(), pl.rank, pl.world, pl.epoch, pl.d_status, PEER_WAIT_POLLS};
                NNVB_TRY(launch_classify_scan(st, w, nullptr, &ctx->launches, &psums));
                used_peers = true;
            } else {
                NNVB_TRY(b->wk->sums.ensure(sizeof(double) * 2 * N * nq, st));
                NNVB_TRY(launch_reduce_chunks(st, w, b->wk->sums.as<double>(), &ctx->launches));
                NNVB_TRY(allreduce(ctx, b->wk->sums.as<double>(), int64_t(2) * N * nq));
                NNVB_TRY(launch_classify_scan(st, w, b->wk->sums.as<double>(), &ctx->launches));
            }
        } else {
            NNVB_TRY(launch_classify_scan(st, w, nullptr, &ctx->launches));
        }
    }

    // the crossing counts decide every size from here on: one host round trip per ReLU layer
    rec->new_off.resize(nq + 1);
    std::vector<int64_t> dead(nq);
    NNVB_CUDA(cudaMemcpyAsync(rec->new_off.data(), w.q_new_off, sizeof(int64_t) * (nq + 1), cudaMemcpyDeviceToHost, st));
    NNVB_CUDA(cudaMemcpyAsync(dead.data(), w.q_dead, sizeof(int64_t) * nq, cudaMemcpyDeviceToHost, st));
    int peer_status[4] = {0, 0, 0, 0};
    if (used_peers)
        NNVB_CUDA(cudaMemcpyAsync(peer_status, ctx->plane.d_status, sizeof(peer_status), cudaMemcpyDeviceToHost, st));
    NNVB_TRY(sync(ctx));
    if (peer_status[0] != 0) {
        // a peer never raised its flag (it failed or left): this reach is void, the context stays usable
        cudaMemsetAsync(ctx->plane.d_status, 0, sizeof(peer_status), st);
        set_error("generator sharding: rank %d did not deliver its bound sums for call %d within the wait limit",
                  peer_status[1], peer_status[2]);
        return NNVB_E_STATE;
    }
    const int64_t K = rec->new_off[nq];
    {
        // NNVB_TRACE: one line per ReLU layer on stderr (sizes as they are found, also when a later layer fails)
        static const bool trace = getenv("NNVB_TRACE") != nullptr;
        if (trace) {
            int64_t nd = 0;
            for (int q = 0; q < nq; ++q) nd += dead[q];
            fprintf(stderr, "[nnvb rank %d] relu: N=%lld columns(local)=%lld crossing=%lld dead=%lld buffer=%.2f GB\n",
                    ctx->rank, (long long)N, (long long)b->ncols, (long long)K, (long long)nd,
                    double(ld) * double(b->ncols) * 8e-9);
        }
    }
    if (b->bounds_fn != nullptr && K > 0) {
        // The neurons the estimates call crossing are listed (index, centre, estimated bounds) so that the hook
        // can read them and their rows, solve its LPs and hand the tightened bounds back; then the layer is
        // classified again from the bound arrays.
        if (ctx->world > 1) {
            set_error("LP-tightened bounds are not available with sharded generators");
            return NNVB_E_UNSUPPORTED;
        }
        const size_t k0 = size_t(K);
        NNVB_TRY(rec->idx.ensure(sizeof(int32_t) * k0, st));
        NNVB_TRY(rec->q.ensure(sizeof(int32_t) * k0, st));
        NNVB_TRY(rec->c.ensure(sizeof(double) * k0, st));
        NNVB_TRY(rec->l.ensure(sizeof(double) * k0, st));
        NNVB_TRY(rec->u.ensure(sizeof(double) * k0, st));
        ReluRecord r0{};
        r0.idx = rec->idx.as<int32_t>(); r0.q = rec->q.as<int32_t>();
        r0.c = rec->c.as<double>(); r0.l = rec->l.as<double>(); r0.u = rec->u.as<double>();
        NNVB_TRY(launch_rank_cross(st, w, r0, &ctx->launches));
        rec->N = N;
        rec->K = K;
        rec->P_in.resize(nq);
        for (int q = 0; q < nq; ++q) rec->P_in[q] = b->h_Pglob[q];
        b->hook_layer = relu_index;
        b->hook_tightened = false;
        b->hook_w = w;
        const int rc = b->bounds_fn(b->bounds_user, b, relu_index);
        b->hook_layer = -1;
        if (rc != 0) {
            set_error("the bounds hook failed with code %d at ReLU layer %d", rc, relu_index);
            return NNVB_E_STATE;
        }
        if (b->hook_tightened) {
            NNVB_TRY(launch_reclassify_scan(st, w, &ctx->launches));
            NNVB_CUDA(cudaMemcpyAsync(rec->new_off.data(), w.q_new_off, sizeof(int64_t) * (nq + 1), cudaMemcpyDeviceToHost, st));
            NNVB_CUDA(cudaMemcpyAsync(dead.data(), w.q_dead, sizeof(int64_t) * nq, cudaMemcpyDeviceToHost, st));
            NNVB_TRY(sync(ctx));
        }
    }
    return relu_step_finish(b, rec, lazy_mask, lazy_onehot, next_layer, w, dead);
}

// Second half of the ReLU step: the relaxation from the (possibly tightened) classification.
int relu_step_finish(nnvb_batch* b, ReluLayerRecord* rec, bool lazy_mask, bool lazy_onehot, size_t next_layer, ReluWork& w,
                     const std::vector<int64_t>& dead) {
    nnvb_ctx* ctx = b->net->ctx;
    cudaStream_t st = ctx->stream;
    const int nq = b->nq;
    const int64_t N = b->N, ld = b->ld;
    const int64_t K = rec->new_off[nq];
    rec->N = N;
    rec->K = K;
    rec->n_dead = 0;
    for (int q = 0; q < nq; ++q) rec->n_dead += dead[q];
    rec->P_in.resize(nq);
    for (int q = 0; q < nq; ++q) rec->P_in[q] = b->h_Pglob[q];     // predicates entering the layer, over all ranks
    const int rank = ctx->rank, world = ctx->world;
    if (world > 1 && b->opts.keep_constraints) {
        set_error("constraint records are not available with sharded generators");
        return NNVB_E_UNSUPPORTED;
    }
    const int64_t K_loc = shard_count(K, rank, world);
    if (b->opts.keep_layer_bounds || b->opts.keep_constraints || world > 1) {
        NNVB_TRY(rec->P_in_dev.ensure(sizeof(int64_t) * nq, st));
        NNVB_TRY(h2d_small(ctx, rec->P_in_dev.p, rec->P_in.data(), sizeof(int64_t) * nq));
    }

    const int64_t ncols_old = b->ncols;
    NNVB_REQUIRE(ncols_old + K_loc < (int64_t(1) << 31), "batch has too many generator columns");
    {
        // this layer's output and, with sharded generators, every layer up to the next ReLU step: the ranks hold
        // different column counts, so the go / no-go is agreed on before anybody enters the next collective
        // (new columns that stay implicit until the next layer, and cohorts kept in compact form, take no columns)
        size_t need = size_t(ld) * ((lazy_onehot && world == 1) ? full_extent(b) : ncols_old + K_loc) * sizeof(double);
        if (world > 1) need = std::max(need, segment_need(b, next_layer, ncols_old + K_loc, ld));
        bool stop = need > ctx->vbuf_bytes();
        const bool mine = stop;
        NNVB_TRY(shard_agree(ctx, stop, &stop));
        if (stop) {
            if (mine) return capacity_error("ReLU layer output", need, ctx->vbuf_bytes());
            set_error("another rank's share of the set outgrew its arena");
            return NNVB_E_CAPACITY;
        }
    }
    NNVB_TRY(ensure_col_meta(b, ncols_old + K_loc));
    // pointers may have moved
    w.qcol_off = b->wk->qcol_off[b->list_cur].as<int64_t>();
    w.qcol_idx = b->wk->qcol_idx[b->list_cur].as<int32_t>();
    w.pl = b->wk->pl.as<double>(); w.pu = b->wk->pu.as<double>();

    const size_t kk = size_t(std::max<int64_t>(K, 1));
    NNVB_TRY(rec->idx.ensure(sizeof(int32_t) * kk, st));
    NNVB_TRY(rec->q.ensure(sizeof(int32_t) * kk, st));
    NNVB_TRY(rec->c.ensure(sizeof(double) * kk, st));
    NNVB_TRY(rec->l.ensure(sizeof(double) * kk, st));
    NNVB_TRY(rec->u.ensure(sizeof(double) * kk, st));
    ReluRecord r{};
    r.idx = rec->idx.as<int32_t>(); r.q = rec->q.as<int32_t>();
    r.c = rec->c.as<double>(); r.l = rec->l.as<double>(); r.u = rec->u.as<double>();
    rec->has_G = false;
    if (b->opts.keep_constraints) {
        rec->h_G_off.assign(nq + 1, 0);
        for (int q = 0; q < nq; ++q)
            rec->h_G_off[q + 1] = rec->h_G_off[q] + (rec->new_off[q + 1] - rec->new_off[q]) * rec->P_in[q];
        NNVB_TRY(rec->G.ensure(sizeof(double) * std::max<int64_t>(rec->h_G_off[nq], 1), st));
        NNVB_TRY(rec->G_off.ensure(sizeof(int64_t) * (nq + 1), st));
        NNVB_TRY(h2d_small(ctx, rec->G_off.p, rec->h_G_off.data(), sizeof(int64_t) * (nq + 1)));
        r.G = rec->G.as<double>();
        r.G_off = rec->G_off.as<int64_t>();
        // the back-substitution bound of the verdict walks the records on the device
        NNVB_TRY(rec->new_off_dev.ensure(sizeof(int64_t) * (nq + 1), st));
        NNVB_CUDA(cudaMemcpyAsync(rec->new_off_dev.p, w.q_new_off, sizeof(int64_t) * (nq + 1), cudaMemcpyDeviceToDevice, st));
        rec->has_G = true;
    }
    // relaxation: lb/ub read, dead and crossing rows cleared in every column of their query,
    // one-hot columns and their predicate bounds written
    const int nxt = 1 - b->list_cur;
    double relax_bytes = 16.0 * double(N) * nq + 8.0 * double(N) * double(K_loc) + 16.0 * double(K_loc);
    for (int q = 0; q < nq; ++q)
        relax_bytes += 8.0 * double(dead[q] + rec->new_off[q + 1] - rec->new_off[q]) *
                       double(b->h_qcol_off[q + 1] - b->h_qcol_off[q] + 1);
    {
        ProfScope ps(ctx, NNVB_PROF_RELAX, relax_bytes);
        if (K > 0) NNVB_TRY(launch_rank_cross(st, w, r, &ctx->launches));
        if (b->opts.keep_constraints) lazy_mask = false;     // the row-clearing kernel also saves the crossing rows
        if ((K > 0 || rec->n_dead > 0) && !lazy_mask) {
            // rows are cleared in the full-length columns: cohorts kept in compact form are written out first,
            // and their compact copies no longer describe the tensor
            for (auto& co : b->cohorts) {
                if (co.col0 >= ncols_old) continue;
                NNVB_TRY(ensure_full(b, co));
                co.pack_off = -1;
            }
        }
        if ((K > 0 || rec->n_dead > 0) && !lazy_mask)
            NNVB_TRY(launch_relu_zero_rows(st, w, ncols_old, b->wk->col_q.as<int32_t>(), r, b->wk->col_pos.as<int64_t>(),
                                           &ctx->launches));
        NNVB_TRY(launch_relu_append(st, w, ncols_old, K_loc, rank, world, !lazy_onehot,
                                    world > 1 ? rec->P_in_dev.as<int64_t>() : nullptr, r, b->wk->col_q.as<int32_t>(),
                                    b->wk->pl.as<double>(), b->wk->pu.as<double>(), b->wk->col_pos.as<int64_t>(),
                                    int(b->shape[0]), int(b->shape[1]), b->wk->box.as<int4>(),
                                    b->wk->qcol_off[nxt].as<int64_t>(),
                                    b->wk->qcol_idx[nxt].as<int32_t>(), &ctx->launches));
    }
    b->list_cur = nxt;
    // local lists grow by the new columns this rank holds: those numbered c = rank (mod world)
    for (int q = 0; q <= nq; ++q) b->h_qcol_off[q] += shard_count(rec->new_off[q], rank, world);
    for (int q = 0; q < nq; ++q) b->h_Pglob[q] += rec->new_off[q + 1] - rec->new_off[q];
    b->ncols = ncols_old + K_loc;
    rec->cols_after = b->ncols;
    b->pend_mask_ncols = (lazy_mask && (K > 0 || rec->n_dead > 0)) ? ncols_old : 0;
    b->pend_mask_N = N;
    b->pend_mask_cf = false;
    if (b->pend_mask_ncols > 0 && b->shape[2] > 1 && b->shape[0] * b->shape[1] * b->shape[2] == N) {
        // readers of compact storage have neighbouring channels on neighbouring lanes: give them the states in that order
        bool any_compact = false;
        for (auto& co : b->cohorts) any_compact = any_compact || co.pack_off >= 0;
        if (any_compact && b->wk->state_cf.ensure(size_t(nq) * N, st) == NNVB_OK) {
            ProfScope ps(ctx, NNVB_PROF_RELAX, 2.0 * double(N) * nq);
            NNVB_TRY(launch_state_channel_fastest(st, nq, int(b->shape[0]), int(b->shape[1]), int(b->shape[2]),
                                                  b->wk->state.as<uint8_t>(), b->wk->state_cf.as<uint8_t>(), &ctx->launches));
            b->pend_mask_cf = true;
        }
    }
    b->pend_onehot = lazy_onehot ? K_loc : 0;
    b->pend_rec = rec;
    static const bool no_windows = getenv("NNVB_NO_WINDOWS") != nullptr;
    if (K_loc > 0) {
        std::vector<int64_t> qn(nq);
        for (int q = 0; q < nq; ++q)
            qn[q] = shard_count(rec->new_off[q + 1], rank, world) - shard_count(rec->new_off[q], rank, world);
        b->cohorts.push_back({ncols_old, ncols_old + K_loc, no_windows, 1, 1, true, std::move(qn)});
    }
    return NNVB_OK;
}

// Whether the consumers of layer li's output can all read compact storage: past the layer's fused BN and an
// optional ReLU layer (which reads compact copies and leaves its row clearing to a mask when a convolution or
// pooling layer follows), the next layer must be a convolution the windowed kernel covers, a pooling layer, or
// a fully connected layer right behind (no ReLU in between: its rows would have to be cleared in memory).
bool next_reads_compact(const nnvb_net* net, size_t li) {
    const auto& Ls = net->layers;
    size_t nx = li + 1;
    if (Ls[li].type == NNVB_LAYER_CONV2D && Ls[li].fused_bn >= 0) nx = size_t(Ls[li].fused_bn) + 1;
    bool relu = false;
    if (nx < Ls.size() && Ls[nx].type == NNVB_LAYER_RELU) { relu = true; ++nx; }
    if (nx >= Ls.size()) return false;
    const Layer& N = Ls[nx];
    if (N.type == NNVB_LAYER_CONV2D)
        return N.cg.sh == 1 && N.cg.sw == 1 && N.cg.dh == 1 && N.cg.dw == 1 && N.cg.kh == 3 && N.cg.kw <= 7 &&
               (N.cw.bn_tile == 32 || N.cw.bn_tile == 64);
    if (N.type == NNVB_LAYER_AVGPOOL2D) return true;
    if (N.type == NNVB_LAYER_FC) return !relu;
    return false;
}

int run_layers(nnvb_batch* b) {
    nnvb_net* net = b->net;
    nnvb_ctx* ctx = net->ctx;
    cudaStream_t st = ctx->stream;
    int relu_i = 0;
    if (ctx->world > 1) {
        // the first segment's capacity, agreed on by all ranks (later ones are agreed on in relu_step)
        const size_t need = segment_need(b, 0, b->ncols, b->ld);
        bool stop = need > ctx->vbuf_bytes();
        const bool mine = stop;
        NNVB_TRY(shard_agree(ctx, stop, &stop));
        if (stop) {
            if (mine) return capacity_error("layer output", need, ctx->vbuf_bytes());
            set_error("another rank's share of the set outgrew its arena");
            return NNVB_E_CAPACITY;
        }
        // peer-mapped sum buffers sized for the largest ReLU layer of this network (same on every rank)
        int64_t slot = 0, Ncur = b->N;
        for (const Layer& L : net->layers) {
            if (L.type == NNVB_LAYER_RELU) slot = std::max(slot, int64_t(2) * Ncur * b->nq);
            Ncur = L.Ho * L.Wo * L.Co;
        }
        if (ctx->plane.comm && slot > 0) NNVB_TRY(ctx->plane.ensure_peer(slot, st));
    }
    for (size_t li = 0; li < net->layers.size(); ++li) {
        const Layer& L = net->layers[li];
        const int64_t Nout = L.Ho * L.Wo * L.Co;
        const int64_t ld_out = lead_dim(Nout);
        if (L.type == NNVB_LAYER_CONV2D || L.type == NNVB_LAYER_FC || L.type == NNVB_LAYER_AVGPOOL2D) {
            const size_t need = size_t(ld_out) * b->ncols * sizeof(double);
            if (ctx->world > 1 && need > ctx->vbuf_bytes()) return capacity_error("layer output", need, ctx->vbuf_bytes());
            // full-length output columns [.., col1) must fit the buffer; cohorts that leave the layer in compact
            // form do not touch theirs, so the test is made per launch
            auto fits = [&](int64_t col1) -> int {
                const size_t nd = size_t(ld_out) * col1 * sizeof(double);
                return nd > ctx->vbuf_bytes() ? capacity_error("layer output", nd, ctx->vbuf_bytes()) : NNVB_OK;
            };
            double* out = other_vbuf(b);
            const bool lazy = lazy_fill(b);
            // Compact storage: a layer reads the cohorts' compact copies from one of the two buffers and writes
            // the other.  The cohorts keep their input state until the layer is through; the output state is
            // collected here and committed at the end.
            static const bool pack_on = getenv("NNVB_NO_PACK") == nullptr;
            static const bool compact_env = getenv("NNVB_NO_COMPACT") == nullptr;
            const bool compact_on = pack_on && compact_env && lazy;
            int in_buf = -1;
            for (auto& co : b->cohorts)
                if (co.pack_off >= 0) in_buf = co.pack_buf;
            const int out_buf = in_buf >= 0 ? 1 - in_buf : 0;
            const size_t n_co = b->cohorts.size();
            std::vector<int64_t> out_off(n_co, -1), out_stride(n_co, 0);
            std::vector<char> out_full(n_co, 1);
            auto comp_in = [&](const nnvb_batch::Cohort& co) -> const double* {
                return co.pack_off >= 0 ? b->wk->pack2[co.pack_buf].as<double>() + co.pack_off : nullptr;
            };
            // test aid: fill the output buffer with NaN patterns first, so that a reader that strays outside
            // the windows it was given shows up in the results instead of depending on what the memory held
            static const bool poison = getenv("NNVB_POISON") != nullptr;
            if (poison) NNVB_CUDA(cudaMemsetAsync(out, 0xFF, std::min(need, ctx->vbuf_bytes()), st));
            // columns the layer contracts densely, and the unit-vector columns whose images it writes directly
            const int64_t n_dense = b->ncols - b->pend_onehot;
            const int64_t n_hot = b->pend_onehot;
            HotCols hot{nullptr, 0, 1, nullptr};
            if (n_hot > 0 && b->pend_scaled)
                hot = HotCols{b->wk->hot_idx.as<int32_t>(), 0, 1, b->wk->hot_scale.as<double>()};
            else if (n_hot > 0)
                hot = HotCols{b->pend_rec->idx.as<int32_t>(), ctx->rank, ctx->world, nullptr};
            bool keep_hot = false;          // the one-hot columns stay unwritten past this layer
            RowMask mask{nullptr, nullptr, 0, 0};
            if (b->pend_mask_ncols > 0)
                mask = RowMask{b->wk->state.as<uint8_t>(), b->wk->col_q.as<int32_t>(), b->pend_mask_ncols, b->pend_mask_N,
                               b->pend_mask_cf ? b->wk->state_cf.as<uint8_t>() : nullptr};
            if (L.type == NNVB_LAYER_CONV2D) {
                ChanAffine bn{nullptr, nullptr, nullptr, nullptr, nullptr};
                if (L.fused_bn >= 0) {
                    const Layer& B = net->layers[L.fused_bn];
                    bn = ChanAffine{B.bn_mean, B.bn_den, B.bn_rden, B.bn_scale, B.bn_offset};
                }
                // one launch per cohort: dense cohorts are tiled over the whole image, windowed cohorts
                // compute one small output patch per column (the rest of their output stays zero)
                const double per_pos = 2.0 * L.cg.Cout * L.cg.kh * L.cg.kw * L.cg.Cin;
                // The windowed launches write their columns in compact form (window only, channel fastest) when a
                // ReLU layer follows (its bound reduction reads that form) or when every consumer reads it; in the
                // second case they write nothing else: the full-length columns of those cohorts stay untouched.
                double* pack_base = nullptr;
                int64_t pack_next = 0;
                const size_t nx = L.fused_bn >= 0 ? size_t(L.fused_bn) + 1 : li + 1;
                const bool relu_next = nx < net->layers.size() && net->layers[nx].type == NNVB_LAYER_RELU;
                const bool only = compact_on && L.cg.Cout % 2 == 0 && next_reads_compact(net, li);
                if (pack_on && (relu_next || only) && !b->opts.keep_constraints && L.cg.Cout % 2 == 0) {
                    int64_t tot = 0;
                    for (auto& co : b->cohorts) {
                        if (co.dense || co.col1 <= co.col0) continue;
                        const int64_t wh = (co.wh - 1 + (L.cg.kh - 1) * L.cg.dh) / L.cg.sh + 1;
                        const int64_t ww = (co.ww - 1 + (L.cg.kw - 1) * L.cg.dw) / L.cg.sw + 1;
                        if (wh * ww <= 128) tot += (co.col1 - co.col0) * wh * ww * L.cg.Cout;
                    }
                    // an optimisation only: a copy that would take more than an eighth of the arena, or that
                    // cannot be allocated, is left out and everything goes through the full-length columns
                    if (tot > 0 && sizeof(double) * size_t(tot) <= ctx->arena_bytes / 8 &&
                        b->wk->pack2[out_buf].ensure(sizeof(double) * tot, st) == NNVB_OK)
                        pack_base = b->wk->pack2[out_buf].as<double>();
                }
                const bool write_full = !(only && pack_base != nullptr);
                for (size_t k = 0; k < n_co; ++k) {
                    auto& co = b->cohorts[k];
                    const int64_t c1 = std::min(co.col1, n_dense);
                    if (c1 <= co.col0) continue;
                    const int wh = (co.wh - 1 + (L.cg.kh - 1) * L.cg.dh) / L.cg.sh + 1;
                    const int ww = (co.ww - 1 + (L.cg.kw - 1) * L.cg.dw) / L.cg.sw + 1;
                    const bool windowed = !co.dense && wh * ww <= 128 && 2 * wh * ww <= L.cg.Ho * L.cg.Wo;
                    if (windowed) {
                        if (!lazy) {
                            NNVB_TRY(fits(c1));
                            NNVB_CUDA(cudaMemsetAsync(out + co.col0 * ld_out, 0, sizeof(double) * ld_out * (c1 - co.col0), st));
                        }
                        ColWindows win{b->wk->box.as<int4>(), wh, ww};
                        // generator columns: the kernel that skips the taps falling outside the input window
                        // (its products: kh*kw per input position), else the patch-tiled kernel (per output position)
                        static const bool no_conv_win = getenv("NNVB_NO_CONV_WIN") != nullptr;
                        bool done = false;
                        if (!no_conv_win && co.col0 >= b->nq) {
                            ProfScope ps(ctx, NNVB_PROF_CONV, per_pos * co.wh * co.ww * double(c1 - co.col0));
                            double* pk = (pack_base && c1 == co.col1) ? pack_base + pack_next : nullptr;
                            if (pk == nullptr || write_full) NNVB_TRY(fits(c1));
                            NNVB_TRY(launch_conv_win(st, L.cg, L.cw, bn, mask, win, co.wh, co.ww, co.col0, b->V, b->ld,
                                                     (pk != nullptr && !write_full) ? nullptr : out, ld_out, c1 - co.col0, pk,
                                                     &done, &ctx->launches, comp_in(co), co.pack_stride));
                            if (!done && comp_in(co) != nullptr) {
                                // the compact-input form does not cover this geometry: from full-length columns
                                NNVB_TRY(ensure_full(b, co));
                                NNVB_TRY(launch_conv_win(st, L.cg, L.cw, bn, mask, win, co.wh, co.ww, co.col0, b->V, b->ld,
                                                         (pk != nullptr && !write_full) ? nullptr : out, ld_out, c1 - co.col0,
                                                         pk, &done, &ctx->launches));
                            }
                            if (!done) ps.cancel();
                            if (done && pk != nullptr) {
                                out_off[k] = pack_next;
                                out_stride[k] = int64_t(wh) * ww * L.cg.Cout;
                                out_full[k] = write_full ? 1 : 0;
                                pack_next += (c1 - co.col0) * out_stride[k];
                            }
                        }
                        if (!done) {
                            NNVB_TRY(ensure_full(b, co));
                            NNVB_TRY(fits(c1));
                            ProfScope ps(ctx, NNVB_PROF_CONV, per_pos * wh * ww * double(c1 - co.col0));
                            NNVB_TRY(launch_conv_f64(st, L.cg, L.cw, bn, mask, win, co.col0, b->V, b->ld, out, ld_out,
                                                     c1 - co.col0, b->nq, &ctx->launches));
                        }
                        co.clean = !lazy;
                    } else {
                        NNVB_TRY(ensure_full(b, co));
                        NNVB_TRY(fits(c1));
                        ProfScope ps(ctx, NNVB_PROF_CONV, per_pos * L.cg.Ho * L.cg.Wo * double(c1 - co.col0));
                        ColWindows win{b->wk->box.as<int4>(), 0, 0};     // whole images; the windows mask the reads
                        NNVB_TRY(launch_conv_f64(st, L.cg, L.cw, bn, mask, win, co.col0, b->V, b->ld, out, ld_out,
                                                 c1 - co.col0, b->nq, &ctx->launches));
                        co.clean = true;
                    }
                }
                ProfScope ps(ctx, NNVB_PROF_ONEHOT, 8.0 * double(lazy ? L.cg.kh * L.cg.kw * L.cg.Cout : Nout) * double(n_hot));
                // the unit-vector columns are one cohort (the last): its compact images follow the others
                const int64_t hot_stride = int64_t((L.cg.kh - 1) * L.cg.dh / L.cg.sh + 1) *
                                           ((L.cg.kw - 1) * L.cg.dw / L.cg.sw + 1) * L.cg.Cout;
                const bool pack_hot = pack_base != nullptr && n_hot > 0 && !b->cohorts.empty() &&
                                      b->cohorts.back().col0 == n_dense && b->cohorts.back().col1 == b->ncols &&
                                      !b->cohorts.back().dense;
                if (n_hot > 0 && !(pack_hot && !write_full)) NNVB_TRY(fits(b->ncols));
                NNVB_TRY(launch_conv_onehot(st, L.cg, L.cw, bn, hot, n_hot,
                                            (pack_hot && !write_full) ? nullptr : out + n_dense * ld_out, ld_out, !lazy,
                                            pack_hot ? pack_base + pack_next : nullptr, &ctx->launches));
                if (pack_hot) {
                    out_off[n_co - 1] = pack_next;
                    out_stride[n_co - 1] = hot_stride;
                    out_full[n_co - 1] = write_full ? 1 : 0;
                    pack_next += n_hot * hot_stride;
                }
                for (auto& co : b->cohorts)
                    if (co.col0 >= n_dense) co.clean = !lazy;
            } else if (L.type == NNVB_LAYER_FC) {
                // one launch per cohort: windowed cohorts contract only the weight rows of their windows
                static const bool no_fcg = getenv("NNVB_NO_FC_GATHER") != nullptr;
                const int In = int(L.H * L.W * L.C);
                NNVB_TRY(fits(b->ncols));
                // Cohorts that take the dense kernel and lie next to each other go in one launch: every launch
                // streams the whole weight matrix, so a launch per small cohort would re-read it per cohort.
                int64_t run0 = -1, run1 = -1;
                auto flush_dense = [&]() -> int {
                    if (run0 < 0) return NNVB_OK;
                    const int64_t n = run1 - run0;
                    ProfScope ps(ctx, NNVB_PROF_FC, 2.0 * double(L.Co) * double(In) * double(n));
                    NNVB_TRY(launch_fc_f64(st, In, int(L.Co), L.fc_wt, L.fc_ldw, L.bias, b->V + run0 * b->ld, b->ld,
                                           out + run0 * ld_out, ld_out, n, std::max<int64_t>(0, b->nq - run0),
                                           &ctx->launches));
                    run0 = run1 = -1;
                    return NNVB_OK;
                };
                for (auto& co : b->cohorts) {
                    const int64_t c1 = std::min(co.col1, n_dense);
                    if (c1 <= co.col0) continue;
                    const int64_t n = c1 - co.col0;
                    const bool gather = !no_fcg && !co.dense && 2 * co.wh * co.ww <= L.H * L.W &&
                                        fc_gather_fits(int(L.C), co.wh, co.ww);
                    if (gather) {
                        NNVB_TRY(flush_dense());
                        NNVB_TRY(b->wk->fcg.ensure(sizeof(int32_t) * fc_gather_scratch_ints(n, int(L.H), int(L.W), co.wh, co.ww), st));
                        ProfScope ps(ctx, NNVB_PROF_FC, 2.0 * double(L.Co) * double(L.C) * co.wh * co.ww * double(n));
                        // a cohort in compact form is contracted from there (when the launch covers all of it)
                        const double* cin = c1 == co.col1 ? comp_in(co) : nullptr;
                        if (cin == nullptr) NNVB_TRY(ensure_full(b, co));
                        NNVB_TRY(launch_fc_gather(st, int(L.H), int(L.W), int(L.C), co.wh, co.ww, int(L.Co), L.fc_wt, L.fc_ldw,
                                                  b->wk->box.as<int4>(), co.col0, n, b->V, b->ld, out, ld_out,
                                                  b->wk->fcg.as<int32_t>(), &ctx->launches, cin, co.pack_stride));
                    } else if (co.col1 <= b->nq && n <= 32 && In >= 1024) {
                        NNVB_TRY(flush_dense());
                        NNVB_TRY(ensure_full(b, co));
                        // a few centre columns: slice the contraction over the grid instead of two fat tiles
                        ProfScope ps(ctx, NNVB_PROF_FC, 2.0 * double(L.Co) * double(In) * double(n));
                        NNVB_TRY(b->wk->tmp.ensure(sizeof(double) * fc_skinny_scratch_doubles(In, int(L.Co), int(n)), st));
                        NNVB_TRY(launch_fc_skinny(st, In, int(L.Co), L.fc_wt, L.fc_ldw, L.bias, b->V + co.col0 * b->ld, b->ld,
                                                  out + co.col0 * ld_out, ld_out, int(n), b->wk->tmp.as<double>(),
                                                  &ctx->launches));
                    } else {
                        NNVB_TRY(ensure_clean(b, co));
                        if (run0 >= 0 && run1 != co.col0) NNVB_TRY(flush_dense());
                        if (run0 < 0) run0 = co.col0;
                        run1 = c1;
                    }
                }
                NNVB_TRY(flush_dense());
                ProfScope ps(ctx, NNVB_PROF_ONEHOT, 8.0 * double(Nout) * double(n_hot));
                NNVB_TRY(launch_fc_onehot(st, int(L.Co), L.fc_wt, L.fc_ldw, hot, n_hot, out + n_dense * ld_out, ld_out,
                                          &ctx->launches));
            } else {
                // cohorts in compact form stay in compact form when every consumer of this layer's output reads it
                const bool only = compact_on && !b->opts.keep_constraints && next_reads_compact(net, li);
                double* pack_base = nullptr;
                int64_t pack_next = 0;
                if (only) {
                    int64_t tot = 0;
                    for (auto& co : b->cohorts) {
                        if (co.dense || co.pack_off < 0 || co.col1 > n_dense) continue;
                        const int64_t wh = (co.wh - 1 + L.pg.ph - 1) / L.pg.sh + 1, ww = (co.ww - 1 + L.pg.pw - 1) / L.pg.sw + 1;
                        if (wh * ww <= 128) tot += (co.col1 - co.col0) * wh * ww * L.pg.C;
                    }
                    if (tot > 0 && sizeof(double) * size_t(tot) <= ctx->arena_bytes / 8 &&
                        b->wk->pack2[out_buf].ensure(sizeof(double) * tot, st) == NNVB_OK)
                        pack_base = b->wk->pack2[out_buf].as<double>();
                }
                for (size_t k = 0; k < n_co; ++k) {
                    auto& co = b->cohorts[k];
                    const int64_t c1 = std::min(co.col1, n_dense);
                    if (c1 <= co.col0) continue;
                    const int wh = (co.wh - 1 + L.pg.ph - 1) / L.pg.sh + 1;
                    const int ww = (co.ww - 1 + L.pg.pw - 1) / L.pg.sw + 1;
                    const bool windowed = !co.dense && wh * ww <= 128 && 2 * wh * ww <= L.pg.Ho * L.pg.Wo;
                    if (windowed && pack_base != nullptr && co.pack_off >= 0 && c1 == co.col1) {
                        ProfScope ps(ctx, NNVB_PROF_AVGPOOL,
                                     8.0 * (double(co.wh) * co.ww * L.pg.C + double(wh) * ww * L.pg.C) * double(c1 - co.col0));
                        out_off[k] = pack_next;
                        out_stride[k] = int64_t(wh) * ww * L.pg.C;
                        out_full[k] = 0;
                        NNVB_TRY(launch_avgpool_compact(st, L.pg, mask, b->wk->box.as<int4>(), co.col0, c1 - co.col0, co.wh, co.ww,
                                                        wh, ww, comp_in(co), co.pack_stride, pack_base + pack_next, out_stride[k],
                                                        &ctx->launches));
                        pack_next += (c1 - co.col0) * out_stride[k];
                        co.clean = false;
                    } else if (windowed) {
                        NNVB_TRY(ensure_full(b, co));
                        NNVB_TRY(fits(c1));
                        if (!lazy) NNVB_CUDA(cudaMemsetAsync(out + co.col0 * ld_out, 0, sizeof(double) * ld_out * (c1 - co.col0), st));
                        // bytes: the input windows read, the output windows (with a zero fill: columns) written
                        ProfScope ps(ctx, NNVB_PROF_AVGPOOL,
                                     8.0 * (double(co.wh) * co.ww * L.pg.C + (lazy ? double(wh) * ww * L.pg.C : double(Nout))) *
                                         double(c1 - co.col0));
                        ColWindows win{b->wk->box.as<int4>(), wh, ww};
                        NNVB_TRY(launch_avgpool_windowed(st, L.pg, mask, win, co.col0, b->V, b->ld, out, ld_out,
                                                         c1 - co.col0, &ctx->launches));
                        co.clean = !lazy;
                    } else {
                        NNVB_TRY(ensure_full(b, co));
                        NNVB_TRY(fits(c1));
                        ProfScope ps(ctx, NNVB_PROF_AVGPOOL, 8.0 * double(b->N + Nout) * double(c1 - co.col0));
                        // the kernel numbers columns from 0: shift the mask to the cohort's first column
                        RowMask m2 = mask;
                        if (m2.state != nullptr) {
                            m2.col_q += co.col0;
                            m2.ncols = std::max<int64_t>(0, mask.ncols - co.col0);
                        }
                        NNVB_TRY(launch_avgpool_f64(st, L.pg, m2, b->wk->box.as<int4>() + co.col0, b->V + co.col0 * b->ld, b->ld,
                                                    out + co.col0 * ld_out, ld_out, c1 - co.col0, &ctx->launches));
                        co.clean = true;
                    }
                }
                // pooling windows that tile the image send a one-hot column to a scaled one-hot column: when the
                // next layer writes the images of such columns itself, only their neurons and scales change here
                static const bool no_hot_pool = getenv("NNVB_NO_HOT_POOL") != nullptr;
                const int nt = li + 1 < net->layers.size() ? net->layers[li + 1].type : 0;
                keep_hot = n_hot > 0 && lazy && !no_hot_pool && pool_keeps_onehot(L.pg) &&
                           (nt == NNVB_LAYER_CONV2D || nt == NNVB_LAYER_FC || nt == NNVB_LAYER_AVGPOOL2D);
                if (keep_hot) {
                    ProfScope ps(ctx, NNVB_PROF_ONEHOT, 24.0 * double(n_hot));
                    NNVB_TRY(b->wk->hot_idx.ensure(sizeof(int32_t) * n_hot, st));
                    NNVB_TRY(b->wk->hot_scale.ensure(sizeof(double) * n_hot, st));
                    NNVB_TRY(launch_pool_onehot_track(st, L.pg, hot, n_hot, b->wk->hot_idx.as<int32_t>(),
                                                      b->wk->hot_scale.as<double>(), &ctx->launches));
                    b->pend_scaled = true;
                } else {
                    ProfScope ps(ctx, NNVB_PROF_ONEHOT, 8.0 * double(lazy ? L.pg.C : Nout) * double(n_hot));
                    if (n_hot > 0) NNVB_TRY(fits(b->ncols));
                    NNVB_TRY(launch_avgpool_onehot(st, L.pg, hot, n_hot, out + n_dense * ld_out, ld_out, !lazy,
                                                   &ctx->launches));
                    for (auto& co : b->cohorts)
                        if (co.col0 >= n_dense) co.clean = !lazy;
                }
            }
            // windows of the output tensor
            if (L.type == NNVB_LAYER_FC) {
                for (auto& co : b->cohorts) { co.dense = true; co.clean = true; co.wh = co.ww = 1 << 20; }
                NNVB_TRY(launch_fill_dense_windows(st, b->ncols, b->wk->box.as<int4>(), &ctx->launches));
            } else {
                const bool cv = L.type == NNVB_LAYER_CONV2D;
                const int eh = cv ? (L.cg.kh - 1) * L.cg.dh : L.pg.ph - 1, ew = cv ? (L.cg.kw - 1) * L.cg.dw : L.pg.pw - 1;
                const int sh = cv ? L.cg.sh : L.pg.sh, sw = cv ? L.cg.sw : L.pg.sw;
                const int pt = cv ? L.cg.pad_t : L.pg.pad_t, pl_ = cv ? L.cg.pad_l : L.pg.pad_l;
                bool any = false;
                for (auto& co : b->cohorts) {
                    // sizes are tracked for dense cohorts too: they still steer the bound reduction
                    co.wh = std::min((co.wh - 1 + eh) / sh + 1, 1 << 20);
                    co.ww = std::min((co.ww - 1 + ew) / sw + 1, 1 << 20);
                    if (co.dense) continue;
                    if (int64_t(co.wh) * co.ww > 128 || 2 * int64_t(co.wh) * co.ww > L.Ho * L.Wo) co.dense = true;
                    else any = true;
                }
                (void)any;      // the boxes also steer the bound reduction, so they are kept for every column
                NNVB_TRY(launch_update_windows(st, b->ncols, b->wk->box.as<int4>(), pt, pl_, eh, ew, sh, sw,
                                               &ctx->launches));
            }
            b->pend_mask_ncols = 0;
            if (!keep_hot) {
                b->pend_onehot = 0;
                b->pend_scaled = false;
            }
            // the cohorts' storage after the layer
            for (size_t k = 0; k < n_co; ++k) {
                auto& co = b->cohorts[k];
                co.pack_off = out_off[k];
                co.pack_stride = out_stride[k];
                co.pack_buf = out_buf;
                co.full_valid = out_full[k] != 0 || out_off[k] < 0;
            }
            b->V = out;
            b->N = Nout;
            b->ld = ld_out;
        } else if (L.type == NNVB_LAYER_BN) {
            if (!L.fused_into_prev) {
                NNVB_TRY(make_writable(b, 0));
                for (auto& co : b->cohorts) {
                    NNVB_TRY(ensure_full(b, co));
                    co.pack_off = -1;
                }
                ChanAffine bn{L.bn_mean, L.bn_den, L.bn_rden, L.bn_scale, L.bn_offset};
                ProfScope ps(ctx, NNVB_PROF_BN, 16.0 * double(b->N) * double(b->ncols));
                NNVB_TRY(launch_bn_f64(st, bn, L.H * L.W, b->N, b->V, b->ld, b->ncols, b->nq, &ctx->launches));
            }
        } else if (L.type == NNVB_LAYER_RELU) {
            // what follows decides how much of the step can be left to it: a convolution or pooling layer
            // masks the cleared rows while loading and writes the images of the new unit-vector columns;
            // a fully connected layer does the latter only
            static const bool eager = getenv("NNVB_EAGER_RELU") != nullptr;
            int nt = li + 1 < net->layers.size() ? net->layers[li + 1].type : 0;
            static const bool eager_mask = getenv("NNVB_EAGER_MASK") != nullptr;
            const bool lazy_mask = !eager && !eager_mask && (nt == NNVB_LAYER_CONV2D || nt == NNVB_LAYER_AVGPOOL2D) &&
                                   int64_t(b->nq) * b->N < (int64_t(1) << 31);     // the mask offsets are 32-bit
            const bool lazy_onehot = !eager && (nt == NNVB_LAYER_CONV2D || nt == NNVB_LAYER_AVGPOOL2D || nt == NNVB_LAYER_FC);
            NNVB_TRY(relu_step(b, b->wk->relu[relu_i].get(), lazy_mask, lazy_onehot, li + 1, relu_i));
            ++relu_i;
        }
        b->shape[0] = L.Ho; b->shape[1] = L.Wo; b->shape[2] = L.Co;
    }
    // the readers of the final set (downloads, output ranges, halfspace rows) take whole columns
    for (auto& co : b->cohorts) NNVB_TRY(ensure_clean(b, co));
    return NNVB_OK;
}

int check_reached(const nnvb_batch* b, int q) {
    if (!b) { set_error("NULL batch"); return NNVB_E_ARG; }
    if (b->hook_layer >= 0) {            // inside the bounds hook: the layers run so far can be read
        if (q < 0 || q >= b->nq) { set_error("query %d out of range", q); return NNVB_E_ARG; }
        return NNVB_OK;
    }
    if (!b->reached) { set_error("results requested before nnvb_batch_reach succeeded"); return NNVB_E_STATE; }
    if (b->net->ctx->result_owner != b) {
        set_error("the results of this batch were overwritten by a later reach on the same context");
        return NNVB_E_STATE;
    }
    if (q < 0 || q >= b->nq) { set_error("query %d out of range", q); return NNVB_E_ARG; }
    return NNVB_OK;
}

// Star.estimateRanges of the current set into b->wk->lb / b->wk->ub (no classification side effects kept)
int output_ranges(nnvb_batch* b) {
    if (b->have_out_ranges) return NNVB_OK;
    nnvb_ctx* ctx = b->net->ctx;
    cudaStream_t st = ctx->stream;
    const int nq = b->nq;
    const int64_t N = b->N;
    std::vector<int64_t> cbeg(nq), cend(nq);
    std::vector<int32_t> qoff(nq + 1);
    for (int q = 0; q < nq; ++q) { cbeg[q] = b->h_qcol_off[q]; cend[q] = b->h_qcol_off[q + 1]; qoff[q] = q; }
    qoff[nq] = nq;
    NNVB_TRY(b->wk->chunk_beg.ensure(sizeof(int64_t) * nq, st));
    NNVB_TRY(b->wk->chunk_end.ensure(sizeof(int64_t) * nq, st));
    NNVB_TRY(b->wk->q_chunk_off.ensure(sizeof(int32_t) * (nq + 1), st));
    NNVB_TRY(b->wk->partial.ensure(sizeof(double) * 2 * N * nq, st));
    NNVB_TRY(h2d_small(ctx, b->wk->chunk_beg.p, cbeg.data(), sizeof(int64_t) * nq));
    NNVB_TRY(h2d_small(ctx, b->wk->chunk_end.p, cend.data(), sizeof(int64_t) * nq));
    NNVB_TRY(h2d_small(ctx, b->wk->q_chunk_off.p, qoff.data(), sizeof(int32_t) * (nq + 1)));
    const int nblk = relu_blocks_per_query(N);
    NNVB_TRY(b->wk->lb.ensure(sizeof(double) * nq * N, st));
    NNVB_TRY(b->wk->ub.ensure(sizeof(double) * nq * N, st));
    NNVB_TRY(b->wk->state.ensure(size_t(nq) * N, st));
    NNVB_TRY(b->wk->blk_cross.ensure(sizeof(int32_t) * nq * nblk, st));
    NNVB_TRY(b->wk->q_cross.ensure(sizeof(int64_t) * nq, st));
    NNVB_TRY(b->wk->q_dead.ensure(sizeof(int64_t) * nq, st));
    NNVB_TRY(b->wk->q_new_off.ensure(sizeof(int64_t) * (nq + 1), st));
    ReluWork w{};
    w.nq = nq; w.N = N; w.ld = b->ld; w.V = b->V;
    w.qcol_off = b->wk->qcol_off[b->list_cur].as<int64_t>();
    w.qcol_idx = b->wk->qcol_idx[b->list_cur].as<int32_t>();
    w.pl = b->wk->pl.as<double>(); w.pu = b->wk->pu.as<double>();
    w.n_chunks = nq;
    w.chunk_beg = b->wk->chunk_beg.as<int64_t>(); w.chunk_end = b->wk->chunk_end.as<int64_t>();
    w.q_chunk_off = b->wk->q_chunk_off.as<int32_t>();
    w.partial = b->wk->partial.as<double>();
    w.lb = b->wk->lb.as<double>(); w.ub = b->wk->ub.as<double>();
    w.state = b->wk->state.as<uint8_t>();
    w.blk_cross = b->wk->blk_cross.as<int32_t>();
    w.q_cross = b->wk->q_cross.as<int64_t>(); w.q_dead = b->wk->q_dead.as<int64_t>();
    w.q_new_off = b->wk->q_new_off.as<int64_t>();
    NNVB_TRY(launch_estimate_ranges(st, w, &ctx->launches));
    if (ctx->world > 1) {
        NNVB_TRY(b->wk->sums.ensure(sizeof(double) * 2 * N * nq, st));
        NNVB_TRY(launch_reduce_chunks(st, w, b->wk->sums.as<double>(), &ctx->launches));
        NNVB_TRY(allreduce(ctx, b->wk->sums.as<double>(), int64_t(2) * N * nq));
        NNVB_TRY(launch_classify_scan(st, w, b->wk->sums.as<double>(), &ctx->launches));
    } else {
        NNVB_TRY(launch_classify_scan(st, w, nullptr, &ctx->launches));
    }
    b->have_out_ranges = true;
    return NNVB_OK;
}

// Run the layers over n points X [ld x n] held in wk.wit[0] (wk.wit[1] is the other buffer).  With a batch
// (witness pass, one point per halfspace pair) the ReLU layers apply the relaxed ReLU of the pair's query;
// without one (b == nullptr) they apply max(x, 0): NN.evaluate on n inputs at once.
int forward_points(nnvb_net* net, WorkBufs* wk, nnvb_batch* b, int n, const int32_t* d_pair_q, double** X, int64_t* ldx,
                   const double* d_r, const int64_t* d_roff, double* d_alpha) {
    nnvb_ctx* ctx = net->ctx;
    cudaStream_t st = ctx->stream;
    double* cur = wk->wit[0].as<double>();
    double* oth = wk->wit[1].as<double>();
    int64_t N = net->in_shape[0] * net->in_shape[1] * net->in_shape[2], ld = lead_dim(N);
    int relu_i = 0;
    for (size_t li = 0; li < net->layers.size(); ++li) {
        const Layer& L = net->layers[li];
        const int64_t Nout = L.Ho * L.Wo * L.Co;
        const int64_t ld_out = lead_dim(Nout);
        if (L.type == NNVB_LAYER_CONV2D) {
            ChanAffine bn{nullptr, nullptr, nullptr, nullptr, nullptr};
            if (L.fused_bn >= 0) {
                const Layer& B = net->layers[L.fused_bn];
                bn = ChanAffine{B.bn_mean, B.bn_den, B.bn_rden, B.bn_scale, B.bn_offset};
            }
            NNVB_TRY(launch_conv_f64(st, L.cg, L.cw, bn, RowMask{nullptr, nullptr, 0, 0}, ColWindows{nullptr, 0, 0}, 0, cur, ld, oth, ld_out, n, n, &ctx->launches));
            std::swap(cur, oth); N = Nout; ld = ld_out;
        } else if (L.type == NNVB_LAYER_FC) {
            if (n <= 512) {      // too few columns to fill the GPU with 128-column tiles: slice the contraction instead
                const int In = int(L.H * L.W * L.C);
                NNVB_TRY(wk->tmp.ensure(sizeof(double) * fc_skinny_scratch_doubles(In, int(L.Co), n), st));
                NNVB_TRY(launch_fc_skinny(st, In, int(L.Co), L.fc_wt, L.fc_ldw, L.bias, cur, ld, oth, ld_out, n,
                                          wk->tmp.as<double>(), &ctx->launches));
            } else
                NNVB_TRY(launch_fc_f64(st, int(L.H * L.W * L.C), int(L.Co), L.fc_wt, L.fc_ldw, L.bias, cur, ld, oth, ld_out,
                                       n, n, &ctx->launches));
            std::swap(cur, oth); N = Nout; ld = ld_out;
        } else if (L.type == NNVB_LAYER_AVGPOOL2D) {
            NNVB_TRY(launch_avgpool_f64(st, L.pg, RowMask{nullptr, nullptr, 0, 0}, nullptr, cur, ld, oth, ld_out, n, &ctx->launches));
            std::swap(cur, oth); N = Nout; ld = ld_out;
        } else if (L.type == NNVB_LAYER_BN) {
            if (!L.fused_into_prev) {
                ChanAffine bn{L.bn_mean, L.bn_den, L.bn_rden, L.bn_scale, L.bn_offset};
                NNVB_TRY(launch_bn_f64(st, bn, L.H * L.W, N, cur, ld, n, n, &ctx->launches));
            }
        } else if (L.type == NNVB_LAYER_RELU) {
            if (b != nullptr) {
                ReluLayerRecord& r = *wk->relu[relu_i++];
                NNVB_TRY(launch_witness_relu(st, n, d_pair_q, N, ld, cur, r.lb.as<double>(), r.ub.as<double>(),
                                             r.rank.as<int32_t>(), r.P_in_dev.as<int64_t>(), d_r, d_roff, d_alpha,
                                             &ctx->launches));
            } else {
                NNVB_TRY(launch_relu_points(st, n, N, ld, cur, &ctx->launches));
            }
        }
    }
    *X = cur;
    *ldx = ld;
    return NNVB_OK;
}

int witness_forward(nnvb_batch* b, int n, const int32_t* d_pair_q, double** X, int64_t* ldx, const double* d_r,
                    const int64_t* d_roff, double* d_alpha = nullptr) {
    return forward_points(b->net, b->wk, b, n, d_pair_q, X, ldx, d_r, d_roff, d_alpha);
}

// Relative guard on "this lower bound is positive": a bound b with term magnitudes M proves emptiness only
// when b > EMPTY_GUARD * (1 + M).
constexpr double EMPTY_GUARD = 1e-6;

// Test halfspace rows against the reached sets: pair p = (query pair_q[p], row G[p], offset g[p]).
// status: EMPTY when the box minimum of the row is positive; NONEMPTY when the greedy witness
// point lies inside the halfspace (needs the layer bounds kept during reach); else UNDECIDED.
// one_witness_per_query: the caller only needs to know whether SOME row of a query is non-empty (the robustness
// verdict: one reachable halfspace makes the query "unknown"), so the witness / back-substitution pass first runs
// on each query's most promising row (smallest box minimum) and only the queries it leaves open get their other
// rows tested.  Verdicts are the same; rows of a query that is already decided stay UNDECIDED.
int test_pairs(nnvb_batch* b, const std::vector<int32_t>& pair_q, const std::vector<double>& G,
               const std::vector<double>& g, std::vector<double>& margin, std::vector<int>& status,
               bool one_witness_per_query = false) {
    nnvb_ctx* ctx = b->net->ctx;
    cudaStream_t st = ctx->stream;
    const int n = (int)pair_q.size();
    const int64_t Nout = b->N;
    margin.assign(n, 0.0);
    status.assign(n, NNVB_UNDECIDED);
    if (n == 0) return NNVB_OK;
    ProfScope ps(ctx, NNVB_PROF_VERIFY, 0.0);
    NNVB_TRY(b->wk->hs_G.ensure(sizeof(double) * n * Nout, st));
    NNVB_TRY(b->wk->hs_g.ensure(sizeof(double) * n, st));
    NNVB_TRY(b->wk->hs_q.ensure(sizeof(int32_t) * n, st));
    NNVB_TRY(b->wk->hs_margin.ensure(sizeof(double) * n * (2 + 2 * HS_SPLIT), st));
    NNVB_CUDA(cudaMemcpyAsync(b->wk->hs_G.p, G.data(), sizeof(double) * n * Nout, cudaMemcpyHostToDevice, st));
    NNVB_CUDA(cudaMemcpyAsync(b->wk->hs_g.p, g.data(), sizeof(double) * n, cudaMemcpyHostToDevice, st));
    NNVB_CUDA(cudaMemcpyAsync(b->wk->hs_q.p, pair_q.data(), sizeof(int32_t) * n, cudaMemcpyHostToDevice, st));
    const int64_t* qoff = b->wk->qcol_off[b->list_cur].as<int64_t>();
    const int32_t* qidx = b->wk->qcol_idx[b->list_cur].as<int32_t>();
    const int add_center = ctx->rank == 0 ? 1 : 0;      // with sharded generators the centre term is added once
    NNVB_TRY(launch_halfspace_pairs(st, n, b->wk->hs_q.as<int32_t>(), Nout, b->ld, b->V, qoff, qidx, b->wk->pl.as<double>(),
                                    b->wk->pu.as<double>(), b->wk->hs_G.as<double>(), b->wk->hs_g.as<double>(),
                                    b->wk->hs_margin.as<double>(), nullptr, nullptr, b->wk->col_pos.as<int64_t>(),
                                    add_center, b->wk->hs_margin.as<double>() + 2 * n, &ctx->launches));
    NNVB_TRY(allreduce(ctx, b->wk->hs_margin.as<double>(), 2 * int64_t(n)));
    std::vector<double> mm(2 * size_t(n));
    NNVB_CUDA(cudaMemcpyAsync(mm.data(), b->wk->hs_margin.p, sizeof(double) * 2 * n, cudaMemcpyDeviceToHost, st));
    NNVB_TRY(sync(ctx));
    std::copy(mm.begin(), mm.begin() + n, margin.begin());
    std::vector<int> open;
    for (int p = 0; p < n; ++p) {
        // The minimum is a sum of 1e4..1e5 rounded terms in an order of its own; "positive" has to hold beyond
        // what that rounding can move, and beyond the feasibility tolerance of the LP that decides the same
        // question in Star.isEmptySet: the same relative guard as the witness test below.  Rows closer to zero
        // stay undecided and go to the LP.
        if (margin[p] > EMPTY_GUARD * (1.0 + mm[n + p])) status[p] = NNVB_VERDICT_EMPTY;
        else if (b->box_implies_C[pair_q[p]]) open.push_back(p);
    }
    // the witness pass needs the bounds of every ReLU layer, the back-substitution bound its crossing rows
    bool have_bounds = true, have_G = ctx->world == 1 && b->net->n_relu <= MAX_BACKSUB_LAYERS;
    for (int i = 0; i < b->net->n_relu; ++i) {
        have_bounds = have_bounds && b->wk->relu[i]->has_bounds;
        have_G = have_G && b->wk->relu[i]->has_G;
    }
    if (open.empty() || (!have_bounds && !have_G)) return NNVB_OK;
    BacksubLayers bs{};
    if (have_G) {
        bs.n = b->net->n_relu;
        for (int i = 0; i < bs.n; ++i) {
            ReluLayerRecord* rc = b->wk->relu[i].get();
            bs.L[i] = BacksubLayer{rc->G.as<double>(), rc->G_off.as<int64_t>(), rc->c.as<double>(), rc->l.as<double>(),
                                   rc->u.as<double>(), rc->new_off_dev.as<int64_t>(), rc->P_in_dev.as<int64_t>()};
        }
    }

    // witness points for the open pairs, in chunks that bound the scratch memory
    int64_t max_ld = b->ld0;
    for (const Layer& L : b->net->layers) max_ld = std::max(max_ld, lead_dim(L.Ho * L.Wo * L.Co));
    const int64_t chunk_cap = std::max<int64_t>(1, (int64_t(1) << 31) / (max_ld * 8));
    auto run = [&](const std::vector<int>& open) -> int {
    for (size_t c0 = 0; c0 < open.size(); c0 += chunk_cap) {
        const int m = (int)std::min<size_t>(chunk_cap, open.size() - c0);
        std::vector<int32_t> pq(m);
        std::vector<double> Gc(size_t(m) * Nout), gc(m);
        std::vector<int64_t> roff(m + 1, 0);
        for (int i = 0; i < m; ++i) {
            const int p = open[c0 + i];
            pq[i] = pair_q[p];
            gc[i] = g[p];
            std::copy(G.begin() + size_t(p) * Nout, G.begin() + size_t(p + 1) * Nout, Gc.begin() + size_t(i) * Nout);
            roff[i + 1] = roff[i] + b->h_Pglob[pq[i]];
        }
        NNVB_TRY(b->wk->hs_r.ensure(sizeof(double) * std::max<int64_t>(roff[m], 1), st));
        NNVB_TRY(b->wk->hs_roff.ensure(sizeof(int64_t) * (m + 1), st));
        NNVB_TRY(b->wk->hs_val.ensure(sizeof(double) * m, st));
        NNVB_TRY(b->wk->hs_scale.ensure(sizeof(double) * m, st));
        NNVB_TRY(b->wk->wit[0].ensure(sizeof(double) * max_ld * m, st));
        NNVB_TRY(b->wk->wit[1].ensure(sizeof(double) * max_ld * m, st));
        NNVB_CUDA(cudaMemcpyAsync(b->wk->hs_G.p, Gc.data(), sizeof(double) * m * Nout, cudaMemcpyHostToDevice, st));
        NNVB_CUDA(cudaMemcpyAsync(b->wk->hs_g.p, gc.data(), sizeof(double) * m, cudaMemcpyHostToDevice, st));
        NNVB_CUDA(cudaMemcpyAsync(b->wk->hs_q.p, pq.data(), sizeof(int32_t) * m, cudaMemcpyHostToDevice, st));
        NNVB_CUDA(cudaMemcpyAsync(b->wk->hs_roff.p, roff.data(), sizeof(int64_t) * (m + 1), cudaMemcpyHostToDevice, st));
        if (ctx->world > 1) NNVB_CUDA(cudaMemsetAsync(b->wk->hs_r.p, 0, sizeof(double) * roff[m], st));
        NNVB_TRY(launch_halfspace_pairs(st, m, b->wk->hs_q.as<int32_t>(), Nout, b->ld, b->V, qoff, qidx, b->wk->pl.as<double>(),
                                        b->wk->pu.as<double>(), b->wk->hs_G.as<double>(), b->wk->hs_g.as<double>(), nullptr,
                                        b->wk->hs_r.as<double>(), b->wk->hs_roff.as<int64_t>(),
                                        b->wk->col_pos.as<int64_t>(), add_center, nullptr, &ctx->launches));
        // every rank needs the coefficients of all predicates: each one wrote its own columns' entries
        NNVB_TRY(allreduce(ctx, b->wk->hs_r.as<double>(), roff[m]));
        if (have_bounds) {
            if (b->kind == 1) {
                NNVB_TRY(launch_witness_x0_bounds(st, m, b->wk->hs_q.as<int32_t>(), b->N0, b->ld0, b->d_in.as<double>(),
                                                  b->wk->hs_r.as<double>(), b->wk->hs_roff.as<int64_t>(), b->wk->wit[0].as<double>(),
                                                  &ctx->launches));
            } else {
                int64_t ncols0 = b->nq;
                std::vector<int64_t> gen0(b->nq + 1);
                for (int q = 0; q < b->nq; ++q) { gen0[q] = ncols0; ncols0 += b->P0_loc[q]; }
                gen0[b->nq] = ncols0;
                NNVB_TRY(b->wk->gen_off.ensure(sizeof(int64_t) * (b->nq + 1), st));
                NNVB_CUDA(cudaMemcpyAsync(b->wk->gen_off.p, gen0.data(), sizeof(int64_t) * (b->nq + 1), cudaMemcpyHostToDevice, st));
                // x0 = c + sum_j alpha_j G0_j: local generators here, summed over the ranks, centre added by rank 0
                NNVB_TRY(launch_witness_x0_star(st, m, b->wk->hs_q.as<int32_t>(), b->N0, b->ld0, b->ld0, b->d_in.as<double>(),
                                                b->wk->gen_off.as<int64_t>(), b->d_in_meta.as<double>(),
                                                b->d_in_meta.as<double>() + ncols0, b->wk->hs_r.as<double>(),
                                                b->wk->hs_roff.as<int64_t>(), b->d_in_pos.as<int64_t>(), add_center,
                                                b->wk->wit[0].as<double>(), &ctx->launches));
                NNVB_TRY(allreduce(ctx, b->wk->wit[0].as<double>(), b->ld0 * int64_t(m)));
            }
            double* X = nullptr;
            int64_t ldx = 0;
            NNVB_TRY(witness_forward(b, m, b->wk->hs_q.as<int32_t>(), &X, &ldx, b->wk->hs_r.as<double>(), b->wk->hs_roff.as<int64_t>()));
            NNVB_TRY(launch_witness_value(st, m, Nout, ldx, X, b->wk->hs_G.as<double>(), b->wk->hs_g.as<double>(),
                                          b->wk->hs_val.as<double>(), b->wk->hs_scale.as<double>(), &ctx->launches));
        }
        if (have_G) {
            // after the witness pass: the bound overwrites the rows
            NNVB_TRY(b->wk->hs_bound.ensure(sizeof(double) * 2 * m, st));
            NNVB_TRY(launch_backsub(st, bs, m, b->wk->hs_q.as<int32_t>(), Nout, b->ld, b->V, b->wk->hs_G.as<double>(),
                                    b->wk->hs_g.as<double>(), b->wk->hs_r.as<double>(), b->wk->hs_roff.as<int64_t>(), qoff, qidx,
                                    b->wk->pl.as<double>(), b->wk->pu.as<double>(), b->wk->hs_bound.as<double>(),
                                    &ctx->launches));
        }
        std::vector<double> val(m, 0.0), scale(m, 0.0), bound(2 * size_t(m), 0.0);
        if (have_bounds) {
            NNVB_CUDA(cudaMemcpyAsync(val.data(), b->wk->hs_val.p, sizeof(double) * m, cudaMemcpyDeviceToHost, st));
            NNVB_CUDA(cudaMemcpyAsync(scale.data(), b->wk->hs_scale.p, sizeof(double) * m, cudaMemcpyDeviceToHost, st));
        }
        if (have_G)
            NNVB_CUDA(cudaMemcpyAsync(bound.data(), b->wk->hs_bound.p, sizeof(double) * 2 * m, cudaMemcpyDeviceToHost, st));
        NNVB_TRY(sync(ctx));
        for (int i = 0; i < m; ++i) {
            const int pp = open[c0 + i];
            // a lower bound over the whole set that is positive beyond rounding: empty, with the bound as the margin
            if (have_G && bound[i] > EMPTY_GUARD * (1.0 + bound[m + i])) { status[pp] = NNVB_VERDICT_EMPTY; margin[pp] = bound[i]; }
            // accept only points clearly inside the halfspace: well beyond the feasibility
            // tolerance of an LP solver deciding the same question
            else if (have_bounds && val[i] < -1e-6 * (1.0 + scale[i])) status[pp] = NNVB_VERDICT_NONEMPTY;
        }
    }
    return NNVB_OK;
    };
    if (!one_witness_per_query) return run(open);
    std::vector<int> best(b->nq, -1), first, rest;
    for (int p : open) {
        int& bp = best[pair_q[p]];
        if (bp < 0 || margin[p] < margin[bp]) bp = p;
    }
    for (int q = 0; q < b->nq; ++q)
        if (best[q] >= 0) first.push_back(best[q]);
    NNVB_TRY(run(first));
    for (int p : open)
        if (p != best[pair_q[p]] && status[best[pair_q[p]]] != NNVB_VERDICT_NONEMPTY) rest.push_back(p);
    return run(rest);
}

}  // namespace

extern "C" {

int nnvb_batch_reach(nnvb_batch* b, const nnvb_opts* opts) {
    NNVB_REQUIRE(b, "nnvb_batch_reach: NULL argument");
    if (!b->uploaded) {
        set_error("nnvb_batch_reach: call nnvb_batch_upload first");
        return NNVB_E_STATE;
    }
    nnvb_ctx* ctx = b->net->ctx;
    NNVB_CUDA(cudaSetDevice(ctx->device));
    b->opts = opts ? *opts : nnvb_opts{};
    b->reached = false;
    b->have_out_ranges = false;
    ctx->result_owner = b;
    while ((int)b->wk->relu.size() < b->net->n_relu) b->wk->relu.emplace_back(new ReluLayerRecord());
    b->pend_mask_ncols = 0;
    b->pend_onehot = 0;
    b->pend_scaled = false;
    NNVB_TRY(init_sets(b));
    NNVB_TRY(run_layers(b));
    {
        // the warp-specialised convolution bounds its waits on shared-memory barriers; one that ran out left wrong
        // numbers behind and must not pass for a result
        int timeouts = 0;
        NNVB_TRY(conv_win_wait_timeouts(ctx->stream, &timeouts));
        if (timeouts != 0) {
            set_error("nnvb_batch_reach: a bounded wait inside conv_win_ws_kernel ran out; the results are not valid");
            return NNVB_E_CUDA;
        }
    }
    b->reached = true;
    return NNVB_OK;
}

int nnvb_batch_out_dims(const nnvb_batch* b, int q, int64_t* P, int64_t* m) {
    NNVB_TRY(check_reached(b, q));
    const int64_t Pq = b->h_Pglob[q];      // over all ranks when the generators are sharded
    if (P) *P = Pq;
    if (m) {
        int64_t mm = b->m0[q];
        // inside the bounds hook: the layers that have run so far
        const int n_done = b->hook_layer >= 0 ? b->hook_layer : b->net->n_relu;
        for (int i = 0; i < n_done; ++i) {
            const ReluLayerRecord& r = *b->wk->relu[i];
            if (r.new_off.size() > size_t(q) + 1) mm += 3 * (r.new_off[q + 1] - r.new_off[q]);
        }
        *m = mm;
    }
    return NNVB_OK;
}

int nnvb_batch_get_V(nnvb_batch* b, int q, double* V) {
    NNVB_TRY(check_reached(b, q));
    NNVB_REQUIRE(V, "nnvb_batch_get_V: NULL output");
    nnvb_ctx* ctx = b->net->ctx;
    NNVB_CUDA(cudaSetDevice(ctx->device));
    const int64_t P = b->h_Pglob[q];
    const int64_t P_loc = b->h_qcol_off[q + 1] - b->h_qcol_off[q];
    const size_t bytes = size_t(b->N) * (P + 1) * sizeof(double);
    NNVB_TRY(b->wk->tmp.ensure(bytes, ctx->stream));
    if (ctx->world > 1) NNVB_CUDA(cudaMemsetAsync(b->wk->tmp.p, 0, bytes, ctx->stream));
    dim3 grid((unsigned)ceil_div(b->N, 256), (unsigned)std::min<int64_t>(P_loc + 1, 32768));
    gather_cols_kernel<<<grid, 256, 0, ctx->stream>>>(b->N, b->ld, b->V, ctx->rank == 0 ? q : -1,
                                                      b->wk->qcol_idx[b->list_cur].as<int32_t>() + b->h_qcol_off[q],
                                                      b->wk->col_pos.as<int64_t>(), P_loc, b->wk->tmp.as<double>());
    NNVB_CUDA(cudaGetLastError());
    ctx->launches += 1;
    NNVB_CUDA(cudaMemcpyAsync(V, b->wk->tmp.p, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return sync(ctx);
}

int nnvb_batch_get_pred_bounds(nnvb_batch* b, int q, double* pl, double* pu) {
    NNVB_TRY(check_reached(b, q));
    nnvb_ctx* ctx = b->net->ctx;
    NNVB_CUDA(cudaSetDevice(ctx->device));
    const int64_t P = b->h_Pglob[q];
    const int64_t P_loc = b->h_qcol_off[q + 1] - b->h_qcol_off[q];
    if (P == 0) return NNVB_OK;
    NNVB_REQUIRE(pl && pu, "nnvb_batch_get_pred_bounds: NULL output");
    NNVB_TRY(b->wk->tmp.ensure(sizeof(double) * 2 * P, ctx->stream));
    if (ctx->world > 1) NNVB_CUDA(cudaMemsetAsync(b->wk->tmp.p, 0, sizeof(double) * 2 * P, ctx->stream));
    if (P_loc > 0) {
        gather_vec_kernel<<<(unsigned)ceil_div(P_loc, 256), 256, 0, ctx->stream>>>(
            P_loc, P, b->wk->qcol_idx[b->list_cur].as<int32_t>() + b->h_qcol_off[q], b->wk->col_pos.as<int64_t>(),
            b->wk->pl.as<double>(), b->wk->pu.as<double>(), b->wk->tmp.as<double>());
        NNVB_CUDA(cudaGetLastError());
        ctx->launches += 1;
    }
    NNVB_CUDA(cudaMemcpyAsync(pl, b->wk->tmp.p, sizeof(double) * P, cudaMemcpyDeviceToHost, ctx->stream));
    NNVB_CUDA(cudaMemcpyAsync(pu, b->wk->tmp.as<double>() + P, sizeof(double) * P, cudaMemcpyDeviceToHost, ctx->stream));
    return sync(ctx);
}

int nnvb_batch_get_ranges(nnvb_batch* b, int q, double* lb, double* ub) {
    NNVB_TRY(check_reached(b, q));
    NNVB_REQUIRE(lb && ub, "nnvb_batch_get_ranges: NULL output");
    nnvb_ctx* ctx = b->net->ctx;
    NNVB_CUDA(cudaSetDevice(ctx->device));
    NNVB_TRY(output_ranges(b));
    NNVB_CUDA(cudaMemcpyAsync(lb, b->wk->lb.as<double>() + size_t(q) * b->N, sizeof(double) * b->N,
                              cudaMemcpyDeviceToHost, ctx->stream));
    NNVB_CUDA(cudaMemcpyAsync(ub, b->wk->ub.as<double>() + size_t(q) * b->N, sizeof(double) * b->N,
                              cudaMemcpyDeviceToHost, ctx->stream));
    return sync(ctx);
}

int nnvb_batch_relu_layers(const nnvb_batch* b, int* n) {
    NNVB_REQUIRE(b && n, "nnvb_batch_relu_layers: NULL argument");
    *n = b->net->n_relu;
    return NNVB_OK;
}

int nnvb_batch_relu_stats(const nnvb_batch* b, int relu_layer, nnvb_relu_stats* stt) {
    NNVB_TRY(check_reached(b, 0));
    NNVB_REQUIRE(stt && relu_layer >= 0 && relu_layer < b->net->n_relu, "nnvb_batch_relu_stats: bad argument");
    const ReluLayerRecord& r = *b->wk->relu[relu_layer];
    stt->n_neurons = r.N;
    stt->n_cross = r.K;
    stt->n_dead = r.n_dead;
    stt->cols_after = r.cols_after;
    return NNVB_OK;
}

int nnvb_batch_get_crossing(nnvb_batch* b, int q, int relu_layer, int64_t* k, int64_t* idx, double* lb, double* ub) {
    NNVB_TRY(check_reached(b, q));
    NNVB_REQUIRE(relu_layer >= 0 && relu_layer < b->net->n_relu, "nnvb_batch_get_crossing: bad layer");
    nnvb_ctx* ctx = b->net->ctx;
    NNVB_CUDA(cudaSetDevice(ctx->device));
    ReluLayerRecord& r = *b->wk->relu[relu_layer];
    const int64_t c0 = r.new_off[q], kq = r.new_off[q + 1] - c0;
    if (k) *k = kq;
    if (kq == 0 || (!idx && !lb && !ub)) return NNVB_OK;
    std::vector<int32_t> h_idx(kq);
    NNVB_CUDA(cudaMemcpyAsync(h_idx.data(), r.idx.as<int32_t>() + c0, sizeof(int32_t) * kq, cudaMemcpyDeviceToHost,
                              ctx->stream));
    if (lb) NNVB_CUDA(cudaMemcpyAsync(lb, r.l.as<double>() + c0, sizeof(double) * kq, cudaMemcpyDeviceToHost, ctx->stream));
    if (ub) NNVB_CUDA(cudaMemcpyAsync(ub, r.u.as<double>() + c0, sizeof(double) * kq, cudaMemcpyDeviceToHost, ctx->stream));
    NNVB_TRY(sync(ctx));
    if (idx) for (int64_t t = 0; t < kq; ++t) idx[t] = h_idx[t];
    return NNVB_OK;
}

int nnvb_batch_get_layer_ranges(nnvb_batch* b, int q, int relu_layer, double* lb, double* ub) {
    NNVB_TRY(check_reached(b, q));
    NNVB_REQUIRE(relu_layer >= 0 && relu_layer < b->net->n_relu && lb && ub, "nnvb_batch_get_layer_ranges: bad argument");
    ReluLayerRecord& r = *b->wk->relu[relu_layer];
    if (!r.has_bounds) {
        set_error("layer bounds were not kept: set opts.keep_layer_bounds");
        return NNVB_E_STATE;
    }
    nnvb_ctx* ctx = b->net->ctx;
    NNVB_CUDA(cudaSetDevice(ctx->device));
    NNVB_CUDA(cudaMemcpyAsync(lb, r.lb.as<double>() + size_t(q) * r.N, sizeof(double) * r.N, cudaMemcpyDeviceToHost, ctx->stream));
    NNVB_CUDA(cudaMemcpyAsync(ub, r.ub.as<double>() + size_t(q) * r.N, sizeof(double) * r.N, cudaMemcpyDeviceToHost, ctx->stream));
    return sync(ctx);
}

int nnvb_batch_get_constraints(nnvb_batch* b, int q, double* Cmat, double* d) {
    NNVB_TRY(check_reached(b, q));
    NNVB_REQUIRE(Cmat && d, "nnvb_batch_get_constraints: NULL output");
    return assemble_constraints(b, q, b->net->n_relu, nullptr, Cmat, d);
}

int nnvb_batch_get_constraints_before(nnvb_batch* b, int q, int relu_layer, int64_t* m, double* Cmat, double* d) {
    NNVB_TRY(check_reached(b, q));
    NNVB_REQUIRE(relu_layer >= 0 && relu_layer <= b->net->n_relu && m, "nnvb_batch_get_constraints_before: bad argument");
    NNVB_REQUIRE(b->hook_layer < 0 || relu_layer <= b->hook_layer, "nnvb_batch_get_constraints_before: layer %d has not run yet", relu_layer);
    return assemble_constraints(b, q, relu_layer, m, Cmat, d);
}

int nnvb_batch_set_bounds_hook(nnvb_batch* b, nnvb_bounds_fn fn, void* user) {
    NNVB_REQUIRE(b, "nnvb_batch_set_bounds_hook: NULL batch");
    b->bounds_fn = fn;
    b->bounds_user = user;
    return NNVB_OK;
}

int nnvb_batch_get_crossing_rows(nnvb_batch* b, int q, int relu_layer, double* G, double* c) {
    NNVB_REQUIRE(b && b->hook_layer >= 0 && relu_layer == b->hook_layer,
                 "nnvb_batch_get_crossing_rows: only valid inside the bounds hook, for its layer");
    NNVB_REQUIRE(q >= 0 && q < b->nq && G && c, "nnvb_batch_get_crossing_rows: bad argument");
    nnvb_ctx* ctx = b->net->ctx;
    NNVB_CUDA(cudaSetDevice(ctx->device));
    ReluLayerRecord& r = *b->wk->relu[relu_layer];
    const int64_t c0 = r.new_off[q], k = r.new_off[q + 1] - c0, P = b->h_qcol_off[q + 1] - b->h_qcol_off[q];
    if (k == 0) return NNVB_OK;
    NNVB_TRY(b->wk->tmp.ensure(sizeof(double) * std::max<int64_t>(k * P, 1), ctx->stream));
    NNVB_TRY(launch_gather_rows(ctx->stream, k, P, r.idx.as<int32_t>() + c0,
                                b->wk->qcol_idx[b->list_cur].as<int32_t>() + b->h_qcol_off[q],
                                b->wk->col_pos.as<int64_t>(), b->V, b->ld, b->wk->tmp.as<double>(), &ctx->launches));
    if (P > 0) NNVB_CUDA(cudaMemcpyAsync(G, b->wk->tmp.p, sizeof(double) * k * P, cudaMemcpyDeviceToHost, ctx->stream));
    NNVB_CUDA(cudaMemcpyAsync(c, r.c.as<double>() + c0, sizeof(double) * k, cudaMemcpyDeviceToHost, ctx->stream));
    return sync(ctx);
}

int nnvb_batch_tighten_crossing(nnvb_batch* b, int q, int relu_layer, const double* xmin, const double* xmax) {
    NNVB_REQUIRE(b && b->hook_layer >= 0 && relu_layer == b->hook_layer,
                 "nnvb_batch_tighten_crossing: only valid inside the bounds hook, for its layer");
    NNVB_REQUIRE(q >= 0 && q < b->nq && xmin && xmax, "nnvb_batch_tighten_crossing: bad argument");
    nnvb_ctx* ctx = b->net->ctx;
    NNVB_CUDA(cudaSetDevice(ctx->device));
    ReluLayerRecord& r = *b->wk->relu[relu_layer];
    const int64_t c0 = r.new_off[q], k = r.new_off[q + 1] - c0;
    if (k == 0) return NNVB_OK;
    for (int64_t t = 0; t < k; ++t)
        NNVB_REQUIRE(xmin[t] <= xmax[t], "nnvb_batch_tighten_crossing: xmin > xmax (or NaN) at neuron %lld", (long long)t);
    NNVB_TRY(b->wk->tmp.ensure(sizeof(double) * 2 * k, ctx->stream));
    NNVB_TRY(h2d_small(ctx, b->wk->tmp.p, xmin, sizeof(double) * k));
    NNVB_TRY(h2d_small(ctx, b->wk->tmp.as<double>() + k, xmax, sizeof(double) * k));
    const ReluWork& w = b->hook_w;
    NNVB_TRY(launch_tighten_bounds(ctx->stream, k, w.N, r.idx.as<int32_t>() + c0, b->wk->tmp.as<double>(),
                                   b->wk->tmp.as<double>() + k, w.lb + int64_t(q) * w.N, w.ub + int64_t(q) * w.N,
                                   &ctx->launches));
    b->hook_tightened = true;
    return sync(ctx);        // tmp is reused by the next call
}

}  // extern "C"

namespace {

// Dense constraint system of query q after its first n_layers ReLU layers: rows of the input set, then per
// layer the three row blocks of PosLin.m:711-735.  *m_out (nullable) receives the row count; Cmat / d nullable.
int assemble_constraints(nnvb_batch* b, int q, int n_layers, int64_t* m_out, double* Cmat, double* d) {
    nnvb_ctx* ctx = b->net->ctx;
    if (ctx->world > 1) {
        set_error("constraint records are not available with sharded generators");
        return NNVB_E_UNSUPPORTED;
    }
    NNVB_CUDA(cudaSetDevice(ctx->device));
    int64_t m = b->m0[q], P = b->P0[q];
    for (int ri = 0; ri < n_layers; ++ri) {
        const ReluLayerRecord& r = *b->wk->relu[ri];
        const int64_t k = r.new_off[q + 1] - r.new_off[q];
        m += 3 * k;
        P += k;
    }
    if (m_out) *m_out = m;
    if (!Cmat || !d) return NNVB_OK;
    std::fill(Cmat, Cmat + size_t(m) * P, 0.0);
    // rows of the input set: [C0 0]
    const int64_t m0 = b->m0[q], P0 = b->P0[q];
    for (int64_t j = 0; j < P0; ++j)
        for (int64_t r = 0; r < m0; ++r) Cmat[size_t(j) * m + r] = b->h_C[q][size_t(j) * m0 + r];
    for (int64_t r = 0; r < m0; ++r) d[r] = b->h_d[q][r];
    int64_t row = m0;
    for (int ri = 0; ri < n_layers; ++ri) {
        ReluLayerRecord& r = *b->wk->relu[ri];
        const int64_t c0 = r.new_off[q], k = r.new_off[q + 1] - c0, Pin = r.P_in[q];
        if (k == 0) continue;
        if (!r.has_G) {
            set_error("constraint rows were not kept: set opts.keep_constraints");
            return NNVB_E_STATE;
        }
        std::vector<double> G(size_t(k) * Pin), c(k), l(k), u(k);
        if (Pin > 0)
            NNVB_CUDA(cudaMemcpyAsync(G.data(), r.G.as<double>() + r.h_G_off[q], sizeof(double) * k * Pin,
                                      cudaMemcpyDeviceToHost, ctx->stream));
        NNVB_CUDA(cudaMemcpyAsync(c.data(), r.c.as<double>() + c0, sizeof(double) * k, cudaMemcpyDeviceToHost, ctx->stream));
        NNVB_CUDA(cudaMemcpyAsync(l.data(), r.l.as<double>() + c0, sizeof(double) * k, cudaMemcpyDeviceToHost, ctx->stream));
        NNVB_CUDA(cudaMemcpyAsync(u.data(), r.u.as<double>() + c0, sizeof(double) * k, cudaMemcpyDeviceToHost, ctx->stream));
        NNVB_TRY(sync(ctx));
        // PosLin.m:711-735: C1 = [0 -I], d1 = 0; C2 = [G -I], d2 = -c; C3 = [-a.*G I], d3 = a.*c - a.*l
        for (int64_t t = 0; t < k; ++t) {
            const double a = u[t] / (u[t] - l[t]);
            const double bb = a * l[t];
            const int64_t newcol = Pin + t;
            Cmat[size_t(newcol) * m + row + t] = -1.0;
            Cmat[size_t(newcol) * m + row + k + t] = -1.0;
            Cmat[size_t(newcol) * m + row + 2 * k + t] = 1.0;
            d[row + t] = 0.0;
            d[row + k + t] = -c[t];
            d[row + 2 * k + t] = a * c[t] - bb;
            for (int64_t j = 0; j < Pin; ++j) {
                const double gv = G[size_t(j) * k + t];
                Cmat[size_t(j) * m + row + k + t] = gv;
                Cmat[size_t(j) * m + row + 2 * k + t] = -a * gv;
            }
        }
        row += 3 * k;
    }
    return NNVB_OK;
}

}  // namespace

extern "C" {

int nnvb_batch_halfspace_margins(nnvb_batch* b, int q, const double* G, const double* g, int nh, double* margin_lo,
                                 int* status) {
    NNVB_TRY(check_reached(b, q));
    NNVB_REQUIRE(G && g && nh > 0 && margin_lo, "nnvb_batch_halfspace_margins: bad argument");
    NNVB_CUDA(cudaSetDevice(b->net->ctx->device));
    const int64_t Nout = b->N;
    // row-major [nh][Nout] copy of the column-major G
    std::vector<double> Gr(size_t(nh) * Nout), gv(g, g + nh), margin;
    for (int h = 0; h < nh; ++h)
        for (int64_t o = 0; o < Nout; ++o) Gr[size_t(h) * Nout + o] = G[size_t(h) + size_t(nh) * o];
    std::vector<int32_t> pq(nh, q);
    std::vector<int> st;
    NNVB_TRY(test_pairs(b, pq, Gr, gv, margin, st));
    for (int h = 0; h < nh; ++h) {
        margin_lo[h] = margin[h];
        if (status) status[h] = st[h];
    }
    return NNVB_OK;
}

int nnvb_batch_halfspace_witness(nnvb_batch* b, int q, const double* G, double g, double* alpha, double* x_out,
                                 double* value) {
    NNVB_TRY(check_reached(b, q));
    NNVB_REQUIRE(G && alpha, "nnvb_batch_halfspace_witness: NULL argument");
    nnvb_ctx* ctx = b->net->ctx;
    if (ctx->world > 1) {
        set_error("witness points are not handed out with sharded generators");
        return NNVB_E_UNSUPPORTED;
    }
    for (int i = 0; i < b->net->n_relu; ++i)
        if (!b->wk->relu[i]->has_bounds) {
            set_error("layer bounds were not kept: set opts.keep_layer_bounds");
            return NNVB_E_STATE;
        }
    NNVB_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t st = ctx->stream;
    const int64_t Nout = b->N, P = b->h_Pglob[q];
    int64_t max_ld = b->ld0;
    for (const Layer& L : b->net->layers) max_ld = std::max(max_ld, lead_dim(L.Ho * L.Wo * L.Co));
    const int32_t pq = q;
    const int64_t roff[2] = {0, P};
    NNVB_TRY(b->wk->hs_G.ensure(sizeof(double) * Nout, st));
    NNVB_TRY(b->wk->hs_g.ensure(sizeof(double), st));
    NNVB_TRY(b->wk->hs_q.ensure(sizeof(int32_t), st));
    NNVB_TRY(b->wk->hs_r.ensure(sizeof(double) * 2 * std::max<int64_t>(P, 1), st));      // coefficients, then alpha
    NNVB_TRY(b->wk->hs_roff.ensure(sizeof(int64_t) * 2, st));
    NNVB_TRY(b->wk->hs_val.ensure(sizeof(double), st));
    NNVB_TRY(b->wk->hs_scale.ensure(sizeof(double), st));
    NNVB_TRY(b->wk->wit[0].ensure(sizeof(double) * max_ld, st));
    NNVB_TRY(b->wk->wit[1].ensure(sizeof(double) * max_ld, st));
    NNVB_TRY(h2d_small(ctx, b->wk->hs_G.p, G, sizeof(double) * Nout));
    NNVB_TRY(h2d_small(ctx, b->wk->hs_g.p, &g, sizeof(double)));
    NNVB_TRY(h2d_small(ctx, b->wk->hs_q.p, &pq, sizeof(int32_t)));
    NNVB_TRY(h2d_small(ctx, b->wk->hs_roff.p, roff, sizeof(roff)));
    double* d_r = b->wk->hs_r.as<double>();
    double* d_alpha = d_r + std::max<int64_t>(P, 1);
    NNVB_CUDA(cudaMemsetAsync(d_alpha, 0, sizeof(double) * P, st));
    const int64_t* qoff = b->wk->qcol_off[b->list_cur].as<int64_t>();
    const int32_t* qidx = b->wk->qcol_idx[b->list_cur].as<int32_t>();
    NNVB_TRY(launch_halfspace_pairs(st, 1, b->wk->hs_q.as<int32_t>(), Nout, b->ld, b->V, qoff, qidx, b->wk->pl.as<double>(),
                                    b->wk->pu.as<double>(), b->wk->hs_G.as<double>(), b->wk->hs_g.as<double>(), nullptr, d_r,
                                    b->wk->hs_roff.as<int64_t>(), b->wk->col_pos.as<int64_t>(), 1, nullptr, &ctx->launches));
    if (b->kind == 1) {
        NNVB_TRY(launch_witness_x0_bounds(st, 1, b->wk->hs_q.as<int32_t>(), b->N0, b->ld0, b->d_in.as<double>(), d_r,
                                          b->wk->hs_roff.as<int64_t>(), b->wk->wit[0].as<double>(), &ctx->launches));
    } else {
        int64_t ncols0 = b->nq;
        std::vector<int64_t> gen0(b->nq + 1);
        for (int k = 0; k < b->nq; ++k) { gen0[k] = ncols0; ncols0 += b->P0_loc[k]; }
        gen0[b->nq] = ncols0;
        NNVB_TRY(b->wk->gen_off.ensure(sizeof(int64_t) * (b->nq + 1), st));
        NNVB_TRY(h2d_small(ctx, b->wk->gen_off.p, gen0.data(), sizeof(int64_t) * (b->nq + 1)));
        NNVB_TRY(launch_witness_x0_star(st, 1, b->wk->hs_q.as<int32_t>(), b->N0, b->ld0, b->ld0, b->d_in.as<double>(),
                                        b->wk->gen_off.as<int64_t>(), b->d_in_meta.as<double>(),
                                        b->d_in_meta.as<double>() + ncols0, d_r, b->wk->hs_roff.as<int64_t>(),
                                        b->d_in_pos.as<int64_t>(), 1, b->wk->wit[0].as<double>(), &ctx->launches));
    }
    double* X = nullptr;
    int64_t ldx = 0;
    NNVB_TRY(witness_forward(b, 1, b->wk->hs_q.as<int32_t>(), &X, &ldx, d_r, b->wk->hs_roff.as<int64_t>(), d_alpha));
    NNVB_TRY(launch_witness_value(st, 1, Nout, ldx, X, b->wk->hs_G.as<double>(), b->wk->hs_g.as<double>(),
                                  b->wk->hs_val.as<double>(), b->wk->hs_scale.as<double>(), &ctx->launches));
    std::vector<double> r(size_t(std::max<int64_t>(P, 1)));
    if (P > 0) {
        NNVB_CUDA(cudaMemcpyAsync(r.data(), d_r, sizeof(double) * P, cudaMemcpyDeviceToHost, st));
        NNVB_CUDA(cudaMemcpyAsync(alpha, d_alpha, sizeof(double) * P, cudaMemcpyDeviceToHost, st));
    }
    if (x_out) NNVB_CUDA(cudaMemcpyAsync(x_out, X, sizeof(double) * Nout, cudaMemcpyDeviceToHost, st));
    if (value) NNVB_CUDA(cudaMemcpyAsync(value, b->wk->hs_val.p, sizeof(double), cudaMemcpyDeviceToHost, st));
    NNVB_TRY(sync(ctx));
    // the input predicates sit at the end of their range that lowers the row (the x0 kernels' rule)
    const int64_t P0 = b->P0[q];
    for (int64_t j = 0; j < P0; ++j) {
        if (b->kind == 1) alpha[j] = r[j] > 0.0 ? -1.0 : 1.0;
        else alpha[j] = r[j] > 0.0 ? b->h_pl[q][j] : b->h_pu[q][j];
    }
    return NNVB_OK;
}

int nnvb_batch_verify_robust(nnvb_batch* b, const int32_t* target, int kind, int* verdict, int* status,
                             double* margin_lo) {
    NNVB_TRY(check_reached(b, 0));
    NNVB_REQUIRE(target && verdict, "nnvb_batch_verify_robust: NULL argument");
    NNVB_REQUIRE(kind == 0 || kind == 1, "nnvb_batch_verify_robust: kind must be 0 ('max') or 1 ('min')");
    NNVB_CUDA(cudaSetDevice(b->net->ctx->device));
    const int nq = b->nq;
    const int64_t Nout = b->N;
    NNVB_REQUIRE(Nout >= 2, "nnvb_batch_verify_robust: output size must be >= 2");
    const int nh = int(Nout - 1);
    // NN.robustness_set (NN.m:1352-1367): rows over i != target; 'max': e_t - e_i, 'min': e_i - e_t
    std::vector<double> G(size_t(nq) * nh * Nout, 0.0), g(size_t(nq) * nh, 0.0), margin;
    std::vector<int32_t> pq(size_t(nq) * nh);
    for (int q = 0; q < nq; ++q) {
        const int t = target[q];
        NNVB_REQUIRE(t >= 0 && t < Nout, "target idx must be less than the output size of the NN (query %d: %d)", q, t);
        int h = 0;
        for (int i = 0; i < Nout; ++i) {
            if (i == t) continue;
            double* row = G.data() + (size_t(q) * nh + h) * Nout;
            if (kind == 0) { row[i] = -1.0; row[t] = 1.0; }
            else { row[i] = 1.0; row[t] = -1.0; }
            pq[size_t(q) * nh + h] = q;
            ++h;
        }
    }
    std::vector<int> st;
    NNVB_TRY(test_pairs(b, pq, G, g, margin, st, true));
    for (int q = 0; q < nq; ++q) {
        bool all_empty = true, any_nonempty = false;
        for (int h = 0; h < nh; ++h) {
            const int s = st[size_t(q) * nh + h];
            all_empty = all_empty && s == NNVB_VERDICT_EMPTY;
            any_nonempty = any_nonempty || s == NNVB_VERDICT_NONEMPTY;
            if (status) status[size_t(q) * nh + h] = s;
            if (margin_lo) margin_lo[size_t(q) * nh + h] = margin[size_t(q) * nh + h];
        }
        verdict[q] = any_nonempty ? NNVB_VERDICT_NONEMPTY : (all_empty ? NNVB_VERDICT_EMPTY : NNVB_UNDECIDED);
    }
    return NNVB_OK;
}

// ---------------------------------------------------------------------------
// single-layer entry points, built on the batch machinery

int nnvb_layer_apply(nnvb_ctx* ctx, const nnvb_layer_desc* layer, int64_t H, int64_t W, int64_t C, int64_t ncols,
                     const double* V_in, double* V_out, int64_t out_shape[3]) {
    NNVB_REQUIRE(ctx && layer && V_in && V_out, "nnvb_layer_apply: NULL argument");
    NNVB_REQUIRE(ncols >= 1, "nnvb_layer_apply: a set has at least its centre column");
    NNVB_REQUIRE(layer->type != NNVB_LAYER_RELU, "nnvb_layer_apply: use a one-layer network for ReLU (it changes the predicate count)");
    nnvb_net* net = nullptr;
    NNVB_TRY(nnvb_net_create(ctx, layer, 1, H, W, C, &net));
    nnvb_batch* b = nullptr;
    int s = nnvb_batch_create(net, 1, &b);
    const int64_t P = ncols - 1;
    std::vector<double> pl(size_t(P), -1.0), pu(size_t(P), 1.0);
    if (!s) s = nnvb_batch_set_star(b, 0, P, V_in, pl.data(), pu.data(), 0, nullptr, nullptr);
    if (!s) s = nnvb_batch_upload(b);
    if (!s) s = nnvb_batch_reach(b, nullptr);
    if (!s) s = nnvb_batch_get_V(b, 0, V_out);
    if (!s && out_shape) s = nnvb_net_out_shape(net, out_shape);
    nnvb_batch_destroy(b);
    nnvb_net_destroy(net);
    return s;
}

int nnvb_estimate_ranges(nnvb_ctx* ctx, int64_t N, int64_t P, const double* V, const double* pl, const double* pu,
                         double* lb, double* ub) {
    NNVB_REQUIRE(ctx && V && lb && ub, "nnvb_estimate_ranges: NULL argument");
    nnvb_net* net = nullptr;
    NNVB_TRY(nnvb_net_create(ctx, nullptr, 0, N, 1, 1, &net));
    nnvb_batch* b = nullptr;
    int s = nnvb_batch_create(net, 1, &b);
    std::vector<double> dl, du;
    if (P > 0 && (!pl || !pu)) {       // Star.m:1091-1096: empty predicate bounds default to [-1, 1]
        dl.assign(size_t(P), -1.0);
        du.assign(size_t(P), 1.0);
        pl = dl.data();
        pu = du.data();
    }
    if (!s) s = nnvb_batch_set_star(b, 0, P, V, pl, pu, 0, nullptr, nullptr);
    if (!s) s = nnvb_batch_upload(b);
    if (!s) s = nnvb_batch_reach(b, nullptr);
    if (!s) s = nnvb_batch_get_ranges(b, 0, lb, ub);
    nnvb_batch_destroy(b);
    nnvb_net_destroy(net);
    return s;
}

}  // extern "C"
