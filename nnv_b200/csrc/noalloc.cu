// Star.estimateRanges for callers that must not allocate device memory.
//
// Some hosts of this library own all device memory themselves and only lend
// pointers: a MATLAB session whose gpuArray pool has claimed the GPU, or a
// long-running service with a fixed, pre-sized arena.  For them a cudaMalloc
// inside the library either fails or fragments the pool they manage, so this
// one entry point runs the bound reduction with nothing but the caller's
// buffers and a fixed scratch array that is part of the loaded module.
//
// The scratch is the file-scope array below: NNVB_NOALLOC_SCRATCH_DOUBLES
// doubles (4 MiB).  Every GPU that loads the library carries one copy until the
// process exits.  All calls on a device share it, so two calls that overlap on
// the GPU (different streams, or different host threads) race on it; run them
// one after the other.  Nothing in it has to be zero: the first kernel of a
// call writes every word the second kernel of that call reads.
#include <cuda_runtime.h>

#include <mutex>

#include "common.cuh"

namespace {

constexpr int64_t SCRATCH_DOUBLES = NNVB_NOALLOC_SCRATCH_DOUBLES;
constexpr int MAX_DEVICES = 64;

static __device__ __align__(256) double g_scratch[SCRATCH_DOUBLES];

// Device address of g_scratch per device.  In host code the symbol g_scratch is
// only a handle; its device address comes from cudaGetSymbolAddress with that
// device current.
double* g_scratch_addr[MAX_DEVICES] = {nullptr};
int g_sm_count[MAX_DEVICES] = {0};
std::mutex g_setup_mutex;

// partial[chunk][0][i] += max(v,0)*pl + min(v,0)*pu over the chunk's columns, [1] likewise with pu/pl.
__global__ void __launch_bounds__(256)
noalloc_partial_kernel(int64_t N, int64_t P, int64_t ld, const double* __restrict__ V,
                       const double* __restrict__ pl, const double* __restrict__ pu, int64_t cols_per_chunk,
                       double* __restrict__ partial) {
    const int64_t i = int64_t(blockIdx.y) * blockDim.x + threadIdx.x;
    if (i >= N) return;
    const int64_t chunk = blockIdx.x;
    const int64_t j0 = chunk * cols_per_chunk;
    const int64_t j1 = j0 + cols_per_chunk < P ? j0 + cols_per_chunk : P;
    double lo = 0.0, hi = 0.0;
    for (int64_t j = j0; j < j1; ++j) {
        const double x = V[(j + 1) * ld + i];          // column 0 is the centre
        const double a = pl[j], b = pu[j];
        const double p = fmax(x, 0.0), n = fmin(x, 0.0);
        lo = fma(p, a, lo); lo = fma(n, b, lo);
        hi = fma(p, b, hi); hi = fma(n, a, hi);
    }
    partial[chunk * 2 * N + i] = lo;
    partial[chunk * 2 * N + N + i] = hi;
}

__global__ void __launch_bounds__(256)
noalloc_finalize_kernel(int64_t N, int64_t ld, const double* __restrict__ V, int64_t n_chunks,
                        const double* __restrict__ partial, double* __restrict__ lb, double* __restrict__ ub) {
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= N) return;
    double lo = 0.0, hi = 0.0;
    for (int64_t c = 0; c < n_chunks; ++c) {
        lo += partial[c * 2 * N + i];
        hi += partial[c * 2 * N + N + i];
    }
    const double c0 = V[i];
    lb[i] = c0 + lo;
    ub[i] = c0 + hi;
}

}  // namespace

extern "C" int nnvb_estimate_ranges_noalloc(void* stream, int64_t N, int64_t P, const double* V_dev, int64_t ld,
                                            const double* pl_dev, const double* pu_dev, double* lb_dev,
                                            double* ub_dev) {
    NNVB_REQUIRE(N > 0 && P >= 0 && ld >= N, "nnvb_estimate_ranges_noalloc: bad sizes (N=%lld, P=%lld, ld=%lld)",
                 (long long)N, (long long)P, (long long)ld);
    NNVB_REQUIRE(V_dev && lb_dev && ub_dev && (P == 0 || (pl_dev && pu_dev)), "nnvb_estimate_ranges_noalloc: NULL pointer");
    if (2 * N > SCRATCH_DOUBLES) {
        nnvb::set_error("nnvb_estimate_ranges_noalloc: N = %lld exceeds the fixed scratch (at most %lld rows); "
                        "use nnvb_estimate_ranges or the batch API for larger sets",
                        (long long)N, (long long)(SCRATCH_DOUBLES / 2));
        return NNVB_E_CAPACITY;
    }
    int dev = -1;
    NNVB_CUDA(cudaGetDevice(&dev));
    NNVB_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "nnvb_estimate_ranges_noalloc: device index %d not supported", dev);
    double* scratch = nullptr;
    int sms = 0;
    {
        // first call on this device: look the scratch address (and the SM count) up once.  The address is
        // cached for the life of the process; it does not survive a cudaDeviceReset of that device.
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (g_scratch_addr[dev] == nullptr) {
            void* p = nullptr;
            NNVB_CUDA(cudaGetSymbolAddress(&p, g_scratch));
            NNVB_CUDA(cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev));
            g_scratch_addr[dev] = static_cast<double*>(p);
        }
        scratch = g_scratch_addr[dev];
        sms = g_sm_count[dev] > 0 ? g_sm_count[dev] : 1;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // as many column chunks as the scratch holds, at least 64 columns each, at most what fills the GPU
    int64_t max_chunks = SCRATCH_DOUBLES / (2 * N);
    int64_t want = (P + 63) / 64;
    const int64_t row_blocks = (N + 255) / 256;
    const int64_t fill = (int64_t(sms) * 8 + row_blocks - 1) / row_blocks;
    if (want > fill) want = fill;
    if (want > max_chunks) want = max_chunks;
    if (want > 65535) want = 65535;
    if (want < 1) want = 1;
    const int64_t cols_per_chunk = P > 0 ? (P + want - 1) / want : 1;
    const int64_t n_chunks = P > 0 ? (P + cols_per_chunk - 1) / cols_per_chunk : 0;
    if (n_chunks > 0) {
        dim3 grid((unsigned)n_chunks, (unsigned)row_blocks);
        noalloc_partial_kernel<<<grid, 256, 0, st>>>(N, P, ld, V_dev, pl_dev, pu_dev, cols_per_chunk, scratch);
        NNVB_CUDA(cudaGetLastError());
    }
    noalloc_finalize_kernel<<<(unsigned)row_blocks, 256, 0, st>>>(N, ld, V_dev, n_chunks, scratch, lb_dev, ub_dev);
    NNVB_CUDA(cudaGetLastError());
    return NNVB_OK;
}
