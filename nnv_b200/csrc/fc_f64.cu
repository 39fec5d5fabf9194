// FullyConnected layer over every generator column at once:
//   Vout[Out x ncols] = W[Out x In] * Vin[In x ncols],  bias on the centre columns
// (FullyConnectedLayer.reach_star_single_input, FullyConnectedLayer.m:305-317;
//  Star.affineMap, Star.m:329-330).
//
// Dense FP64 contraction on the DMMA tensor path.  The GEMM is computed
// transposed so that both operands are read along their contiguous axis:
//   D[m = column j][n = output o] = sum_k Vin[k + j*ld_in] * Wt[k*ldw + o]
// A tiles (columns of V, k contiguous) and B tiles (rows of Wt, o contiguous)
// are staged through a 3-deep cp.async ring; shared-memory row strides are
// chosen = 4 (mod 8) doubles so the per-lane fragment reads hit 16 distinct
// 8-byte banks per half warp.
#include "common.cuh"
#include "mma_f64.cuh"

namespace nnvb {

namespace {

constexpr int FC_BK = 16;
constexpr int FC_STAGES = 3;
constexpr int FC_AST = FC_BK + 4;   // A row stride in shared memory (doubles)

template <int WM_TILES, int WN_TILES, int WARPS_M, int WARPS_N>
struct FcCfg {
    static constexpr int BM = WARPS_M * WM_TILES * 16;
    static constexpr int BN = WARPS_N * WN_TILES * 8;
    static constexpr int BST = BN + 4;
    static constexpr int THREADS = WARPS_M * WARPS_N * 32;
    static constexpr int A_STAGE = BM * FC_AST;
    static constexpr int B_STAGE = FC_BK * BST;
    static constexpr size_t SMEM = size_t(FC_STAGES) * (A_STAGE + B_STAGE) * sizeof(double);
};

template <int WM_TILES, int WN_TILES, int WARPS_M, int WARPS_N>
__global__ void __launch_bounds__(WARPS_M* WARPS_N * 32, 1)
fc_f64_kernel(int In, int In_pad, int Out, const double* __restrict__ Wt, int ldw,
              const double* __restrict__ bias, const double* __restrict__ Vin, int64_t ld_in,
              double* __restrict__ Vout, int64_t ld_out, int64_t ncols, int64_t n_center) {
    using Cfg = FcCfg<WM_TILES, WN_TILES, WARPS_M, WARPS_N>;
    extern __shared__ __align__(16) double smem[];
    double* As = smem;
    double* Bs = smem + FC_STAGES * Cfg::A_STAGE;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int wm = warp % WARPS_M;
    const int wn = warp / WARPS_M;
    const int g = lane >> 2;
    const int t = lane & 3;

    const int64_t j0 = int64_t(blockIdx.x) * Cfg::BM;
    const int n0 = blockIdx.y * Cfg::BN;
    const int KT = In_pad / FC_BK;

    auto load_stage = [&](int stage, int kt) {
        const int k0 = kt * FC_BK;
        double* a = As + stage * Cfg::A_STAGE;
        double* b = Bs + stage * Cfg::B_STAGE;
        // A: BM rows (columns of V) x 8 chunks of 2 doubles
        for (int c = tid; c < Cfg::BM * (FC_BK / 2); c += Cfg::THREADS) {
            const int row = c / (FC_BK / 2);
            const int kc = c % (FC_BK / 2);
            const int k = k0 + 2 * kc;
            const int64_t j = j0 + row;
            int bytes = 0;
            const double* src = Vin;
            if (j < ncols && k < In) {
                bytes = (In - k >= 2) ? 16 : 8;
                src = Vin + j * ld_in + k;
            }
            cp_async16(a + row * FC_AST + 2 * kc, src, bytes);
        }
        // B: BK rows of Wt x BN/2 chunks
        for (int c = tid; c < FC_BK * (Cfg::BN / 2); c += Cfg::THREADS) {
            const int kr = c / (Cfg::BN / 2);
            const int nc = c % (Cfg::BN / 2);
            const int n = n0 + 2 * nc;
            int bytes = 0;
            const double* src = Wt;
            if (n < ldw) {
                bytes = 16;
                src = Wt + int64_t(k0 + kr) * ldw + n;
            }
            cp_async16(b + kr * Cfg::BST + 2 * nc, src, bytes);
        }
    };

    double acc[WM_TILES][WN_TILES][4];
#pragma unroll
    for (int mi = 0; mi < WM_TILES; ++mi)
#pragma unroll
        for (int ni = 0; ni < WN_TILES; ++ni)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[mi][ni][r] = 0.0;

#pragma unroll
    for (int s = 0; s < FC_STAGES - 1; ++s) {
        if (s < KT) load_stage(s, s);
        cp_async_commit();
    }

    for (int kt = 0; kt < KT; ++kt) {
        cp_async_wait<FC_STAGES - 2>();
        __syncthreads();
        {
            const int nk = kt + FC_STAGES - 1;
            if (nk < KT) load_stage(nk % FC_STAGES, nk);
            cp_async_commit();
        }
        const double* a = As + (kt % FC_STAGES) * Cfg::A_STAGE + (wm * WM_TILES * 16 + g) * FC_AST + t;
        const double* b = Bs + (kt % FC_STAGES) * Cfg::B_STAGE + t * Cfg::BST + wn * WN_TILES * 8 + g;
#pragma unroll
        for (int kk = 0; kk < FC_BK; kk += 8) {
            double af[WM_TILES][4];
            double bf[WN_TILES][2];
#pragma unroll
            for (int mi = 0; mi < WM_TILES; ++mi) {
                const double* p = a + mi * 16 * FC_AST + kk;
                af[mi][0] = p[0];
                af[mi][1] = p[8 * FC_AST];
                af[mi][2] = p[4];
                af[mi][3] = p[8 * FC_AST + 4];
            }
#pragma unroll
            for (int ni = 0; ni < WN_TILES; ++ni) {
                const double* p = b + kk * Cfg::BST + ni * 8;
                bf[ni][0] = p[0];
                bf[ni][1] = p[4 * Cfg::BST];
            }
#pragma unroll
            for (int mi = 0; mi < WM_TILES; ++mi)
#pragma unroll
                for (int ni = 0; ni < WN_TILES; ++ni) dmma_16x8x8(acc[mi][ni], af[mi], bf[ni]);
        }
    }
    cp_async_wait<0>();

    // epilogue: bias on centre columns, store two adjacent outputs per lane
#pragma unroll
    for (int mi = 0; mi < WM_TILES; ++mi) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int64_t j = j0 + wm * WM_TILES * 16 + mi * 16 + g + half * 8;
            if (j >= ncols) continue;
            const bool is_center = j < n_center;
            double* dst = Vout + j * ld_out;
#pragma unroll
            for (int ni = 0; ni < WN_TILES; ++ni) {
                const int o = n0 + wn * WN_TILES * 8 + ni * 8 + 2 * t;
                if (o >= Out) continue;
                double v0 = acc[mi][ni][half * 2 + 0];
                double v1 = acc[mi][ni][half * 2 + 1];
                if (is_center) {
                    v0 += bias[o];
                    if (o + 1 < Out) v1 += bias[o + 1];
                }
                if (o + 1 < Out) {
                    *reinterpret_cast<double2*>(dst + o) = make_double2(v0, v1);
                } else {
                    dst[o] = v0;
                }
            }
        }
    }
}

template <int WM_TILES, int WN_TILES, int WARPS_M, int WARPS_N>
int launch_cfg(cudaStream_t st, int In, int Out, const double* Wt, int ldw, const double* bias,
               const double* Vin, int64_t ld_in, double* Vout, int64_t ld_out, int64_t ncols,
               int64_t n_center) {
    using Cfg = FcCfg<WM_TILES, WN_TILES, WARPS_M, WARPS_N>;
    auto kern = fc_f64_kernel<WM_TILES, WN_TILES, WARPS_M, WARPS_N>;
    static bool attr_set = false;
    if (!attr_set) {
        NNVB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM));
        attr_set = true;
    }
    dim3 grid((unsigned)ceil_div(ncols, Cfg::BM), (unsigned)ceil_div(Out, Cfg::BN));
    const int In_pad = (int)round_up(In, FC_BK);
    kern<<<grid, Cfg::THREADS, Cfg::SMEM, st>>>(In, In_pad, Out, Wt, ldw, bias, Vin, ld_in, Vout,
                                                ld_out, ncols, n_center);
    NNVB_CUDA(cudaGetLastError());
    return NNVB_OK;
}

}  // namespace

int launch_fc_f64(cudaStream_t st, int In, int Out, const double* Wt, int ldw, const double* bias,
                  const double* Vin, int64_t ld_in, double* Vout, int64_t ld_out, int64_t ncols,
                  int64_t n_center, int64_t* launches) {
    if (ncols <= 0) return NNVB_OK;
    int s;
    if (Out <= 16)
        s = launch_cfg<1, 2, 8, 1>(st, In, Out, Wt, ldw, bias, Vin, ld_in, Vout, ld_out, ncols, n_center);
    else if (Out <= 64)
        s = launch_cfg<2, 4, 4, 2>(st, In, Out, Wt, ldw, bias, Vin, ld_in, Vout, ld_out, ncols, n_center);
    else
        s = launch_cfg<2, 8, 4, 2>(st, In, Out, Wt, ldw, bias, Vin, ld_in, Vout, ld_out, ncols, n_center);
    if (s == NNVB_OK && launches) *launches += 1;
    return s;
}

namespace {
// FullyConnected image of one-hot columns: W * e_i = W(:, i), i.e. row i of the transposed weight copy.
__global__ void fc_onehot_kernel(int Out, const double* __restrict__ Wt, int ldw, const int32_t* __restrict__ rec_idx,
                                 int64_t c_first, int64_t c_step, double* __restrict__ Vout, int64_t ld_out) {
    const int64_t t = blockIdx.x;
    const double* src = Wt + int64_t(rec_idx[c_first + t * c_step]) * ldw;
    double* dst = Vout + t * ld_out;
    for (int o = threadIdx.x; o < Out; o += blockDim.x) dst[o] = src[o];
}
}  // namespace

int launch_fc_onehot(cudaStream_t st, int Out, const double* Wt, int ldw, const int32_t* rec_idx, int64_t c_first,
                     int64_t c_step, int64_t K_loc, double* Vout, int64_t ld_out, int64_t* launches) {
    if (K_loc <= 0) return NNVB_OK;
    fc_onehot_kernel<<<(unsigned)K_loc, 128, 0, st>>>(Out, Wt, ldw, rec_idx, c_first, c_step, Vout, ld_out);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

}  // namespace nnvb
