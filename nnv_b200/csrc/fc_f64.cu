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
constexpr int FCG_STAGES = 2;     // gathered FC: two stages, so that two blocks fit on an SM
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
// FullyConnected on a handful of columns (the witness points of the halfspace test): the tensor-core
// tiles would be almost empty and the K loop of a single tile is latency bound.  Here block (x, y) owns
// 32 outputs and a slice of 256 input rows: the slice of up to 8 columns is staged in shared memory,
// each lane keeps one output, the 8 warps split the slice and are combined in warp order, and the
// slice sums go to partial[slice][column][output]; a second kernel adds the slices in order plus the
// bias (every column is a point).
constexpr int SK_ROWS = 256;
__global__ void __launch_bounds__(256)
fc_skinny_kernel(int In, int Out, const double* __restrict__ Wt, int ldw, const double* __restrict__ Vin,
                 int64_t ld_in, int ncols, double* __restrict__ partial) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int o = blockIdx.x * 32 + lane;
    const int k0 = blockIdx.y * SK_ROWS;
    __shared__ double vs[8][SK_ROWS];
    __shared__ double red[8][8][33];
    for (int c0 = 0; c0 < ncols; c0 += 8) {
        const int nc = min(8, ncols - c0);
        for (int e = threadIdx.x; e < 8 * SK_ROWS; e += 256) {
            const int c = e / SK_ROWS, k = e % SK_ROWS;
            vs[c][k] = (c < nc && k0 + k < In) ? Vin[int64_t(c0 + c) * ld_in + k0 + k] : 0.0;
        }
        __syncthreads();
        double acc[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] = 0.0;
        for (int kk = warp * 32; kk < warp * 32 + 32; ++kk) {
            const double wv = (o < Out && k0 + kk < In) ? Wt[int64_t(k0 + kk) * ldw + o] : 0.0;
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[c] = fma(wv, vs[c][kk], acc[c]);
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) red[warp][c][lane] = acc[c];
        __syncthreads();
        for (int c = warp; c < nc; c += 8) {
            double v = 0.0;
#pragma unroll
            for (int w = 0; w < 8; ++w) v += red[w][c][lane];
            if (o < Out) partial[(int64_t(blockIdx.y) * ncols + c0 + c) * Out + o] = v;
        }
        __syncthreads();
    }
}

__global__ void fc_skinny_reduce_kernel(int Out, int ncols, int n_slices, const double* __restrict__ partial,
                                        const double* __restrict__ bias, double* __restrict__ Vout, int64_t ld_out) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= ncols * Out) return;
    const int c = e / Out, o = e % Out;
    double v = 0.0;
    for (int s = 0; s < n_slices; ++s) v += partial[(int64_t(s) * ncols + c) * Out + o];
    Vout[int64_t(c) * ld_out + o] = v + bias[o];
}

// FullyConnected image of one-hot columns: W * e_i = W(:, i), i.e. row i of the transposed weight copy,
// times the column's scale where it has one (the single product of the dense contraction).
__global__ void fc_onehot_kernel(int Out, const double* __restrict__ Wt, int ldw, HotCols hot,
                                 double* __restrict__ Vout, int64_t ld_out) {
    const int64_t t = blockIdx.x;
    const double* src = Wt + int64_t(hot.idx[hot.first + t * hot.step]) * ldw;
    double* dst = Vout + t * ld_out;
    if (hot.scale != nullptr) {
        const double sc = hot.scale[t];
        for (int o = threadIdx.x; o < Out; o += blockDim.x) dst[o] = src[o] * sc;
    } else {
        for (int o = threadIdx.x; o < Out; o += blockDim.x) dst[o] = src[o];
    }
}
}  // namespace

namespace {

// ---------------------------------------------------------------------------------------------------
// FullyConnected on windowed columns.  A column that is zero outside an wh x ww window of the H x W x C
// input only needs the C*wh*ww weight rows of that window:  out = sum_{rows in window} W(:, row) * v(row).
// Columns are grouped by window origin (counting sort on the device), every tile of 32 columns shares
// one origin and therefore one list of rows, and the contraction runs over that list only — the same
// DMMA tiles as the dense kernel with gathered operands.  Values equal the dense product (the skipped
// terms are products with zero), up to the order of the remaining additions.

// key of a window origin; h0 in [-(wh-1), H-1], w0 in [-(ww-1), W-1].  A window that does not meet the image
// belongs to an all-zero column (whatever its memory holds): such columns share the last bin, whose tiles
// contract nothing and write zeros.
__device__ __forceinline__ int fcg_key(int4 bx, int wh, int ww, int KH, int nbins) {
    const int bh = bx.x + wh - 1, bw = bx.y + ww - 1;
    const int KW = (nbins - 1) / KH;
    if (bh < 0 || bh >= KH || bw < 0 || bw >= KW) return nbins - 1;
    return bh + KH * bw;
}

__global__ void fcg_hist_kernel(int64_t col0, int64_t n, const int4* __restrict__ box, int wh, int ww, int KH,
                                int nbins, int32_t* __restrict__ hist) {
    const int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t < n) atomicAdd(hist + fcg_key(box[col0 + t], wh, ww, KH, nbins), 1);
}

// bin offsets and the tile table (a tile = up to tile_cols columns of one bin)
__global__ void __launch_bounds__(1024)
fcg_tiles_kernel(int nbins, int tile_cols, const int32_t* __restrict__ hist, int32_t* __restrict__ bin_start,
                 int32_t* __restrict__ cursor, int32_t* __restrict__ tile_key,
                 int32_t* __restrict__ tile_start, int32_t* __restrict__ tile_count,
                 int32_t* __restrict__ n_tiles) {
    // one block: exclusive scans of the bins' column counts and tile counts (1024 bins per round, carried on)
    __shared__ int wsum_c[32], wsum_t[32];
    __shared__ int carry_c, carry_t;
    if (threadIdx.x == 0) { carry_c = 0; carry_t = 0; }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int base = 0; base < nbins; base += 1024) {
        const int b = base + threadIdx.x;
        const int cnt = b < nbins ? hist[b] : 0;
        const int nt = (cnt + tile_cols - 1) / tile_cols;
        int ic = cnt, it = nt;
        for (int o = 1; o < 32; o <<= 1) {
            const int xc = __shfl_up_sync(0xffffffffu, ic, o), xt = __shfl_up_sync(0xffffffffu, it, o);
            if (lane >= o) { ic += xc; it += xt; }
        }
        if (lane == 31) { wsum_c[warp] = ic; wsum_t[warp] = it; }
        __syncthreads();
        int off = carry_c, t0 = carry_t;
        for (int w = 0; w < warp; ++w) { off += wsum_c[w]; t0 += wsum_t[w]; }
        off += ic - cnt;
        t0 += it - nt;
        if (b < nbins) {
            bin_start[b] = off;
            cursor[b] = 0;
            for (int k = 0; k < nt; ++k) {
                tile_key[t0 + k] = b;
                tile_start[t0 + k] = off + k * tile_cols;
                tile_count[t0 + k] = min(tile_cols, cnt - k * tile_cols);
            }
        }
        __syncthreads();
        if (threadIdx.x == 1023) { carry_c = off + cnt; carry_t = t0 + nt; }
        __syncthreads();
    }
    if (threadIdx.x == 0) *n_tiles = carry_t;
}

__global__ void fcg_scatter_kernel(int64_t col0, int64_t n, const int4* __restrict__ box, int wh, int ww, int KH,
                                   int nbins, const int32_t* __restrict__ bin_start, int32_t* __restrict__ cursor,
                                   int32_t* __restrict__ perm) {
    const int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= n) return;
    const int key = fcg_key(box[col0 + t], wh, ww, KH, nbins);
    perm[bin_start[key] + atomicAdd(cursor + key, 1)] = int32_t(col0 + t);
}

// Tiles of 32 columns x 256 outputs: columns sharing a window origin come in small groups (tens), so a
// short M tile keeps the tiles full; the weight rows of a tile are then re-read from L2 once per 32 columns.
constexpr int FCG_WM = 2, FCG_WN = 4, FCG_WARPS_M = 1, FCG_WARPS_N = 8;
constexpr int FCG_BM = FCG_WARPS_M * FCG_WM * 16;
constexpr size_t FCG_SMEM = size_t(FCG_STAGES) * (FcCfg<FCG_WM, FCG_WN, FCG_WARPS_M, FCG_WARPS_N>::A_STAGE +
                                                  FcCfg<FCG_WM, FCG_WN, FCG_WARPS_M, FCG_WARPS_N>::B_STAGE) * sizeof(double);

__global__ void __launch_bounds__(FCG_WARPS_M * FCG_WARPS_N * 32, FCG_WARPS_M * FCG_WARPS_N <= 8 ? 2 : 1)
fc_gather_kernel(int H, int W, int C, int wh, int ww, int KH, int Kt, int Kt_pad, int Out,
                 const double* __restrict__ Wt, int ldw, const double* __restrict__ Vin, int64_t ld_in,
                 double* __restrict__ Vout, int64_t ld_out, const int32_t* __restrict__ tile_key,
                 const int32_t* __restrict__ tile_start, const int32_t* __restrict__ tile_count,
                 const int32_t* __restrict__ n_tiles, const int32_t* __restrict__ perm,
                 const double* __restrict__ comp, int64_t comp_stride, int64_t comp_col0, int zero_row) {
    // zero_row: a row of Wt that holds zeros (stands in for the weight rows of positions off the image).
    // comp (nullable): the columns in compact form (window only, channel fastest; column j at
    // comp + (j - comp_col0)*comp_stride).  The contraction index then runs in that storage order,
    // k = (wl*wh + hl)*C + c, so that a column's operand row is one contiguous run.
    using Cfg = FcCfg<FCG_WM, FCG_WN, FCG_WARPS_M, FCG_WARPS_N>;
    if (int(blockIdx.x) >= *n_tiles) return;
    extern __shared__ __align__(16) double smem[];
    double* As = smem;
    double* Bs = smem + FCG_STAGES * Cfg::A_STAGE;
    int* rows_s = reinterpret_cast<int*>(Bs + FCG_STAGES * Cfg::B_STAGE);   // [Kt_pad] input row of k, -1 = none
    int* cols_s = rows_s + Kt_pad;                                          // [BM] column of tile row m, -1 = none
    __shared__ __align__(8) uint64_t b_bar[FCG_STAGES];                     // the weight rows of a stage land on these

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp % FCG_WARPS_M, wn = warp / FCG_WARPS_M;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.y * Cfg::BN;

    const int key = tile_key[blockIdx.x];
    const int h0 = key % KH - (wh - 1), w0 = key / KH - (ww - 1);
    const bool null_bin = key == KH * (W + ww - 1);     // columns whose window lies off the image
    const bool comp_pairs = comp != nullptr && comp_stride % 2 == 0 && (reinterpret_cast<uintptr_t>(comp) & 15) == 0;
    const int start = tile_start[blockIdx.x], count = tile_count[blockIdx.x];
    if (tid == 0) {
        for (int s = 0; s < FCG_STAGES; ++s) mbar_init(&b_bar[s], 1);
        mbar_init_fence();
    }
    // a weight row of the tile is one contiguous run of Wt: one bulk copy each (16-byte multiples: ldw is even)
    const uint32_t row_bytes = uint32_t(min(Cfg::BN, ldw - n0)) * 8u;
    for (int m = tid; m < Cfg::BM; m += Cfg::THREADS) cols_s[m] = m < count ? perm[start + m] : -1;
    for (int k = tid; k < Kt_pad; k += Cfg::THREADS) {
        int row = -1;
        if (k < Kt && !null_bin) {
            int hl, wl, c;
            if (comp != nullptr) {
                c = k % C;
                const int pos = k / C;
                hl = pos % wh;
                wl = pos / wh;
            } else {
                hl = k % wh;
                const int r2 = k / wh;
                wl = r2 % ww;
                c = r2 / ww;
            }
            const int h = h0 + hl, w = w0 + wl;
            if (h >= 0 && h < H && w >= 0 && w < W) row = h + H * (w + W * c);
        }
        rows_s[k] = row;
    }
    __syncthreads();

    auto load_stage = [&](int stage, int kt) {
        const int k0 = kt * FC_BK;
        double* a = As + stage * Cfg::A_STAGE;
        double* b = Bs + stage * Cfg::B_STAGE;
        if (comp != nullptr && comp_pairs) {
            // compact columns: a column's operand row is contiguous in the contraction order, 16 bytes a copy
            for (int c = tid; c < Cfg::BM * (FC_BK / 2); c += Cfg::THREADS) {
                const int m = c / (FC_BK / 2), kk = 2 * (c % (FC_BK / 2));
                const int r0 = rows_s[k0 + kk], r1 = rows_s[k0 + kk + 1], col = cols_s[m];
                double* d = a + m * FC_AST + kk;
                const double* src = col >= 0 ? comp + (int64_t(col) - comp_col0) * comp_stride + (k0 + kk) : comp;
                if (col >= 0 && r0 >= 0 && r1 >= 0) {
                    cp_async16(d, src, 16);
                } else {
                    const bool ok0 = col >= 0 && r0 >= 0, ok1 = col >= 0 && r1 >= 0;
                    cp_async8(d, ok0 ? src : comp, ok0 ? 8 : 0);
                    cp_async8(d + 1, ok1 ? src + 1 : comp, ok1 ? 8 : 0);
                }
            }
        } else {
            for (int c = tid; c < Cfg::BM * FC_BK; c += Cfg::THREADS) {
                const int m = c / FC_BK, kk = c % FC_BK;
                const int row = rows_s[k0 + kk], col = cols_s[m];
                const bool ok = row >= 0 && col >= 0;
                const double* src = comp != nullptr ? comp : Vin;
                if (ok) src = comp != nullptr ? comp + (int64_t(col) - comp_col0) * comp_stride + (k0 + kk)
                                              : Vin + int64_t(col) * ld_in + row;
                cp_async8(a + m * FC_AST + kk, src, ok ? 8 : 0);
            }
        }
        // B: the FC_BK weight rows of the chunk, one bulk copy per row issued by the lanes of warp 0; their bytes are
        // counted on the stage's barrier.  Positions off the image take the zero row.  Outputs past ldw are not
        // copied: they feed accumulator columns that are never stored.
        if (warp == 0) {
            if (lane == 0) {
                async_proxy_fence();
                mbar_expect_bytes(&b_bar[stage], row_bytes * FC_BK);
            }
            __syncwarp();
            if (lane < FC_BK) {
                const int row = rows_s[k0 + lane];
                bulk_copy_g2s(b + lane * Cfg::BST, Wt + int64_t(row >= 0 ? row : zero_row) * ldw + n0, row_bytes,
                              &b_bar[stage]);
            }
        }
    };

    double acc[FCG_WM][FCG_WN][4];
#pragma unroll
    for (int mi = 0; mi < FCG_WM; ++mi)
#pragma unroll
        for (int ni = 0; ni < FCG_WN; ++ni)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[mi][ni][r] = 0.0;

    const int KT = Kt_pad / FC_BK;
#pragma unroll
    for (int s = 0; s < FCG_STAGES - 1; ++s) {
        if (s < KT) load_stage(s, s);
        cp_async_commit();
    }
    for (int kt = 0; kt < KT; ++kt) {
        cp_async_wait<FCG_STAGES - 2>();
        mbar_wait(&b_bar[kt % FCG_STAGES], (kt / FCG_STAGES) & 1);      // stage kt % S is on its (kt / S)-th use
        __syncthreads();
        {
            const int nk = kt + FCG_STAGES - 1;
            if (nk < KT) load_stage(nk % FCG_STAGES, nk);
            cp_async_commit();
        }
        const double* a = As + (kt % FCG_STAGES) * Cfg::A_STAGE + (wm * FCG_WM * 16 + g) * FC_AST + t;
        const double* b = Bs + (kt % FCG_STAGES) * Cfg::B_STAGE + t * Cfg::BST + wn * FCG_WN * 8 + g;
#pragma unroll
        for (int kk = 0; kk < FC_BK; kk += 8) {
            double af[FCG_WM][4];
            double bf[FCG_WN][2];
#pragma unroll
            for (int mi = 0; mi < FCG_WM; ++mi) {
                const double* p = a + mi * 16 * FC_AST + kk;
                af[mi][0] = p[0];
                af[mi][1] = p[8 * FC_AST];
                af[mi][2] = p[4];
                af[mi][3] = p[8 * FC_AST + 4];
            }
#pragma unroll
            for (int ni = 0; ni < FCG_WN; ++ni) {
                const double* p = b + kk * Cfg::BST + ni * 8;
                bf[ni][0] = p[0];
                bf[ni][1] = p[4 * Cfg::BST];
            }
#pragma unroll
            for (int mi = 0; mi < FCG_WM; ++mi)
#pragma unroll
                for (int ni = 0; ni < FCG_WN; ++ni) dmma_16x8x8(acc[mi][ni], af[mi], bf[ni]);
        }
    }
    cp_async_wait<0>();

#pragma unroll
    for (int mi = 0; mi < FCG_WM; ++mi) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int col = cols_s[wm * FCG_WM * 16 + mi * 16 + g + half * 8];
            if (col < 0) continue;
            double* dst = Vout + int64_t(col) * ld_out;
#pragma unroll
            for (int ni = 0; ni < FCG_WN; ++ni) {
                const int o = n0 + wn * FCG_WN * 8 + ni * 8 + 2 * t;
                if (o >= Out) continue;
                if (o + 1 < Out)
                    *reinterpret_cast<double2*>(dst + o) = make_double2(acc[mi][ni][half * 2], acc[mi][ni][half * 2 + 1]);
                else
                    dst[o] = acc[mi][ni][half * 2];
            }
        }
    }
}

}  // namespace

size_t fc_gather_scratch_ints(int64_t n, int H, int W, int wh, int ww) {
    const int64_t nbins = int64_t(H + wh - 1) * (W + ww - 1) + 1;
    const int64_t max_tiles = ceil_div(n, FCG_BM) + nbins;
    return size_t(3 * nbins + 3 * max_tiles + n + 8);
}

bool fc_gather_fits(int C, int wh, int ww) { return round_up(int64_t(C) * wh * ww, FC_BK) <= 16384; }

int launch_fc_gather(cudaStream_t st, int H, int W, int C, int wh, int ww, int Out, const double* Wt, int ldw,
                     const int4* box, int64_t col0, int64_t n, const double* Vin, int64_t ld_in, double* Vout,
                     int64_t ld_out, int32_t* scratch, int64_t* launches, const double* comp, int64_t comp_stride) {
    if (n <= 0) return NNVB_OK;
    using Cfg = FcCfg<FCG_WM, FCG_WN, FCG_WARPS_M, FCG_WARPS_N>;
    const int KH = H + wh - 1;
    const int nbins = KH * (W + ww - 1) + 1;        // the last bin: windows off the image
    const int64_t max_tiles = ceil_div(n, FCG_BM) + nbins;
    int32_t* hist = scratch;
    int32_t* bin_start = hist + nbins;
    int32_t* cursor = bin_start + nbins;
    int32_t* tile_key = cursor + nbins;
    int32_t* tile_start = tile_key + max_tiles;
    int32_t* tile_count = tile_start + max_tiles;
    int32_t* n_tiles = tile_count + max_tiles;
    int32_t* perm = n_tiles + 8;
    NNVB_CUDA(cudaMemsetAsync(hist, 0, sizeof(int32_t) * nbins, st));
    fcg_hist_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, st>>>(col0, n, box, wh, ww, KH, nbins, hist);
    fcg_tiles_kernel<<<1, 1024, 0, st>>>(nbins, FCG_BM, hist, bin_start, cursor, tile_key, tile_start, tile_count, n_tiles);
    fcg_scatter_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, st>>>(col0, n, box, wh, ww, KH, nbins, bin_start, cursor, perm);
    const int Kt = C * wh * ww;
    const int Kt_pad = (int)round_up(Kt, FC_BK);
    const size_t smem = FCG_SMEM + size_t(Kt_pad + 128) * sizeof(int);
    static bool attr_set = false;
    if (!attr_set) {
        NNVB_CUDA(cudaFuncSetAttribute(fc_gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(FCG_SMEM + size_t(16384 + 128) * sizeof(int))));
        NNVB_CUDA(cudaFuncSetAttribute(fc_gather_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                       cudaSharedmemCarveoutMaxShared));
        attr_set = true;
    }
    dim3 grid((unsigned)max_tiles, (unsigned)ceil_div(Out, Cfg::BN));
    fc_gather_kernel<<<grid, Cfg::THREADS, smem, st>>>(H, W, C, wh, ww, KH, Kt, Kt_pad, Out, Wt, ldw, Vin, ld_in, Vout,
                                                      ld_out, tile_key, tile_start, tile_count, n_tiles, perm, comp,
                                                      comp_stride, col0, (int)round_up(int64_t(H) * W * C, 16));
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 4;
    return NNVB_OK;
}

size_t fc_skinny_scratch_doubles(int In, int Out, int ncols) { return size_t(ceil_div(In, SK_ROWS)) * ncols * Out; }

int launch_fc_skinny(cudaStream_t st, int In, int Out, const double* Wt, int ldw, const double* bias,
                     const double* Vin, int64_t ld_in, double* Vout, int64_t ld_out, int ncols, double* scratch,
                     int64_t* launches) {
    if (ncols <= 0) return NNVB_OK;
    const int n_slices = (int)ceil_div(In, SK_ROWS);
    dim3 grid((unsigned)ceil_div(Out, 32), (unsigned)n_slices);
    fc_skinny_kernel<<<grid, 256, 0, st>>>(In, Out, Wt, ldw, Vin, ld_in, ncols, scratch);
    NNVB_CUDA(cudaGetLastError());
    fc_skinny_reduce_kernel<<<(unsigned)ceil_div(int64_t(ncols) * Out, 256), 256, 0, st>>>(Out, ncols, n_slices, scratch,
                                                                                           bias, Vout, ld_out);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 2;
    return NNVB_OK;
}

int launch_fc_onehot(cudaStream_t st, int Out, const double* Wt, int ldw, const HotCols& hot, int64_t K_loc,
                     double* Vout, int64_t ld_out, int64_t* launches) {
    if (K_loc <= 0) return NNVB_OK;
    fc_onehot_kernel<<<(unsigned)K_loc, 128, 0, st>>>(Out, Wt, ldw, hot, Vout, ld_out);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

}  // namespace nnvb
