// Shared declarations of the sm_100a engine: error plumbing, device helpers
// and the launch signatures of the kernels (one .cu file per kernel family).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

#include "../../include/nnvb200.h"

namespace nnvb {

void set_error(const char* fmt, ...);

#define NNVB_CUDA(call)                                                          \
    do {                                                                         \
        cudaError_t e_ = (call);                                                 \
        if (e_ != cudaSuccess) {                                                 \
            nnvb::set_error("%s failed at %s:%d: %s", #call, __FILE__, __LINE__, \
                            cudaGetErrorString(e_));                             \
            return NNVB_E_CUDA;                                                  \
        }                                                                        \
    } while (0)

#define NNVB_TRY(call)                  \
    do {                                \
        int s_ = (call);                \
        if (s_ != NNVB_OK) return s_;   \
    } while (0)

#define NNVB_REQUIRE(cond, ...)         \
    do {                                \
        if (!(cond)) {                  \
            nnvb::set_error(__VA_ARGS__); \
            return NNVB_E_ARG;          \
        }                               \
    } while (0)

static inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }
static inline int64_t ceil_div(int64_t x, int64_t m) { return (x + m - 1) / m; }

// Leading dimension (doubles) of a generator matrix with N rows: columns start
// on 128-byte lines for large N, on 16-byte boundaries always.
static inline int64_t lead_dim(int64_t N) { return N >= 64 ? round_up(N, 16) : round_up(N, 2); }

// ---------------------------------------------------------------------------
// Kernel launch wrappers.  Every wrapper enqueues on `st`, returns the number of
// kernels it launched through *launches (added), and reports launch errors.

struct ConvGeom {
    int H, W, Cin;          // input image
    int Ho, Wo, Cout;       // output image
    int kh, kw;
    int pad_t, pad_l;
    int sh, sw, dh, dw;
};

// Pre-arranged convolution weights (see conv_f64.cu for the layout).
struct ConvWeights {
    double* w;              // device, arranged [n_tile][ci_chunk][tap][KC][CS]
    double* bias;           // device [Cout]
    int bn_tile;            // output channels per CTA tile (32, 64 or 128)
    int cs;                 // padded channel stride in shared memory (doubles)
    int n_tiles;            // ceil(Cout / bn_tile)
    int n_chunks;           // ceil(Cin / KC)
    // Filter footprints for unit-vector columns (unit stride and dilation only, else null): the image of the unit
    // vector of input channel ci, window only and channel fastest, [Cin][kw][kh][Cout]:
    // foot[((ci*kw + owl)*kh + ohl)*Cout + co] = W(kh-1-ohl, kw-1-owl, ci, co)
    double* foot = nullptr;
};

// Optional per-channel affine fused behind a contraction (BatchNormalization
// in eval mode): centre: ((x - mean) / den) * scale + offset, generators:
// (x / den) * scale.  All pointers device, length = channels; null = off.
struct ChanAffine {
    const double* mean;
    const double* den;      // sqrt(var + eps)
    const double* rden;     // 1 / den, used where the affine is fused behind a contraction
    const double* scale;
    const double* offset;
};

// Rows that a ReLU step cleared but did not zero in memory: for columns j < ncols, row i of column j
// reads as zero when state[col_q[j]*N + i] != 0.  state == nullptr: no mask.
struct RowMask {
    const uint8_t* state;
    const int32_t* col_q;
    int64_t ncols;
    int64_t N;
    // the same states in channel-fastest order, [q][(w*H + h)*C + c] (null: not made), for readers of compact storage
    const uint8_t* state_cf = nullptr;
};

// Column windows: column j (absolute index) is exactly zero outside its input window box[j] = {h0, w0, h
// extent, w extent} (may lie partly outside the image).  Memory outside a window may hold stale data, so
// every reader treats it as zero.  wh x ww > 0 is the size of the OUTPUT patch a windowed launch computes
// for each column; wh == 0 asks for the whole output image (dense launch).  box == nullptr: no windows.
struct ColWindows {
    const int4* box;        // per column {h0, w0, wh, ww} of its input window
    int wh, ww;
};
// A window that covers any image (dense columns).
#define NNVB_DENSE_ORIGIN (-(1 << 20))
#define NNVB_DENSE_EXTENT (1 << 21)

size_t conv_weights_doubles(const ConvGeom& g, int* bn_tile, int* cs, int* n_tiles, int* n_chunks);
// Host-side re-layout of W[kh,kw,Cin,Cout] (column-major) into the kernel's layout.
void conv_arrange_weights(const ConvGeom& g, const double* W, double* dst, int bn_tile, int cs,
                          int n_tiles, int n_chunks);

// Windowed generator columns (no centres) with the taps that read outside the wh_in x ww_in input window
// skipped; see conv_win_f64.cu.  *done stays false, and nothing is launched, for geometries it does not
// cover (the caller then uses launch_conv_f64).  pack (nullable): the launch also writes a window-only copy of
// its columns there, column j (from col_base) at j*wh*ww*Cout, entry (h, w, c) of the output window at
// ((w - w0)*wh + (h - h0))*Cout + c.  cin (nullable): the launch's input columns in the same compact form
// (column j at cin + j*cin_stride, window wh_in x ww_in), read instead of Vin.  Vout may be null when pack is
// given: the output then exists in compact form only.
int conv_win_wait_timeouts(cudaStream_t st, int* out);
int launch_conv_win(cudaStream_t st, const ConvGeom& g, const ConvWeights& w, const ChanAffine& bn, const RowMask& mask,
                    const ColWindows& win, int wh_in, int ww_in, int64_t col_base, const double* Vin, int64_t ld_in,
                    double* Vout, int64_t ld_out, int64_t ncols, double* pack, bool* done, int64_t* launches,
                    const double* cin = nullptr, int64_t cin_stride = 0);
// Processes columns [col_base, col_base + ncols) of Vin / Vout (pointers to column 0).
int launch_conv_f64(cudaStream_t st, const ConvGeom& g, const ConvWeights& w, const ChanAffine& bn,
                    const RowMask& mask, const ColWindows& win, int64_t col_base, const double* Vin, int64_t ld_in, double* Vout, int64_t ld_out,
                    int64_t ncols, int64_t n_center, int64_t* launches);

// The one-hot columns a ReLU step appended and no layer has written to memory yet: column t of this rank
// is scale[t] (1 where scale is null) times the unit vector of neuron idx[first + t*step].
struct HotCols {
    const int32_t* idx;
    int64_t first, step;
    const double* scale;
};
// Images of one-hot columns, written to Vout[ld_out x K_loc].
// zero_fill: clear the whole output block first (else only the columns' output windows are written).
// pack (nullable): also a window-only copy, column t at t*wh*ww*Cout, laid out as launch_conv_win's.
int launch_conv_onehot(cudaStream_t st, const ConvGeom& g, const ConvWeights& w, const ChanAffine& bn,
                       const HotCols& hot, int64_t K_loc, double* Vout, int64_t ld_out, bool zero_fill,
                       double* pack, int64_t* launches);
// Writes zero to every entry of columns [col0, col0+n) of V (an H x W x C image per column) that lies
// outside the column's window box[col]: afterwards the columns can be read without window tests.
int launch_zero_outside_windows(cudaStream_t st, int H, int W, int C, const int4* box, int64_t col0, int64_t n,
                                double* V, int64_t ld, int64_t* launches);
// FC on windowed columns [col0, col0+n) (all with an wh x ww window in the H x W x C input; origins in box):
// only the weight rows of each column's window are contracted.  scratch: fc_gather_scratch_ints() int32.
// comp (nullable): the columns in compact form (column col0 + j at comp + j*comp_stride), read instead of Vin.
size_t fc_gather_scratch_ints(int64_t n, int H, int W, int wh, int ww);
bool fc_gather_fits(int C, int wh, int ww);
int launch_fc_gather(cudaStream_t st, int H, int W, int C, int wh, int ww, int Out, const double* Wt, int ldw,
                     const int4* box, int64_t col0, int64_t n, const double* Vin, int64_t ld_in, double* Vout,
                     int64_t ld_out, int32_t* scratch, int64_t* launches, const double* comp = nullptr,
                     int64_t comp_stride = 0);
// FC for a few columns that are all points (bias on every column); used for witness points.
size_t fc_skinny_scratch_doubles(int In, int Out, int ncols);
int launch_fc_skinny(cudaStream_t st, int In, int Out, const double* Wt, int ldw, const double* bias,
                     const double* Vin, int64_t ld_in, double* Vout, int64_t ld_out, int ncols, double* scratch,
                     int64_t* launches);
int launch_fc_onehot(cudaStream_t st, int Out, const double* Wt, int ldw, const HotCols& hot, int64_t K_loc,
                     double* Vout, int64_t ld_out, int64_t* launches);

// FC: Vout[Out x ncols] = W * Vin[In x ncols]; bias (and the optional affine) on
// the first n_center columns.  Wt is the device copy arranged [In_pad][ldw]
// (ldw = Out rounded up to 8, zero filled).
int launch_fc_f64(cudaStream_t st, int In, int Out, const double* Wt, int ldw, const double* bias,
                  const double* Vin, int64_t ld_in, double* Vout, int64_t ld_out, int64_t ncols,
                  int64_t n_center, int64_t* launches);

// Per-channel affine (BatchNormalization) in place on V[N x ncols]; channel of
// row i is i / plane (plane = H*W).
int launch_bn_f64(cudaStream_t st, const ChanAffine& bn, int64_t plane, int64_t N, double* V,
                  int64_t ld, int64_t ncols, int64_t n_center, int64_t* launches);

struct PoolGeom {
    int H, W, C, Ho, Wo;
    int ph, pw, sh, sw, pad_t, pad_l;
    int clip;               // 1: the divisor counts only the window entries inside the image (padding excluded)
};
// Divisor of the average for the window whose first entry is (h0, w0) in unpadded coordinates.
__host__ __device__ inline double pool_divisor(const PoolGeom& g, int h0, int w0) {
    if (!g.clip) return double(g.ph * g.pw);
    const int h1 = h0 + g.ph < g.H ? h0 + g.ph : g.H, w1 = w0 + g.pw < g.W ? w0 + g.pw : g.W;
    const int n = (h1 - (h0 > 0 ? h0 : 0)) * (w1 - (w0 > 0 ? w0 : 0));
    return double(n > 0 ? n : 1);
}
// box (nullable): per-column input windows, indexed like Vin's columns; entries outside count as zero.
int launch_avgpool_f64(cudaStream_t st, const PoolGeom& g, const RowMask& mask, const int4* box, const double* Vin,
                       int64_t ld_in, double* Vout, int64_t ld_out, int64_t ncols, int64_t* launches);
// zero_fill: clear the whole output block first (else only the columns' output windows are written).
int launch_avgpool_onehot(cudaStream_t st, const PoolGeom& g, const HotCols& hot, int64_t K_loc, double* Vout,
                          int64_t ld_out, bool zero_fill, int64_t* launches);
// Pooling with windows that tile the image exactly (pool size = stride, no padding, H and W multiples of
// it) maps a scaled one-hot column to a scaled one-hot column: neuron (h, w, c) -> (h/sh, w/sw, c), scale
// -> (0 + scale) / (ph*pw), the value the pooling kernel computes for that column.  Writes the new neuron
// and scale of every column to dst_idx / dst_scale (which may be hot.idx / hot.scale when first = 0, step = 1);
// no column memory is touched.
bool pool_keeps_onehot(const PoolGeom& g);
int launch_pool_onehot_track(cudaStream_t st, const PoolGeom& g, const HotCols& hot, int64_t K_loc, int32_t* dst_idx,
                             double* dst_scale, int64_t* launches);

// ReLU approx-star step; see relu_star.cu.  All pointers are device pointers.
// A cohort of windowed columns [col0, col0+n): every column is zero outside a wh x ww window.  The bound
// reduction sorts them by window origin into KH x KW bins per query (KH = H + wh - 1: every origin whose
// window meets the image) and then visits, for each pixel, only the columns whose window covers it.
struct WinCohort {
    int64_t col0, n;
    int wh, ww, KH, KW;
    int64_t bin_base;          // offset of its [nq][KH*KW + 1] table in the bin arrays
    // window-only copy of the cohort's columns (ReluWork::win_pack), or pack_off < 0: entry (h, w, c) of column j
    // at pack_off + (j - col0)*pack_stride + ((w - w0_j)*wh + (h - h0_j))*C + c
    int64_t pack_off, pack_stride;
};
constexpr int MAX_WIN_COHORTS = 16;
constexpr int MAX_WIN_EXTENT = 32;       // largest window side handled this way
struct WinCohorts {
    int n;
    WinCohort c[MAX_WIN_COHORTS];
};
size_t range_windows_scratch_ints(const WinCohorts& wc, int nq, int64_t ncols);
int range_windows_slices(int H, int W, int C, int nq, int sm_count);

struct ReluWork {
    int nq;
    int64_t N, ld;
    double* V;                 // [ld x ncols]; column q (< nq) is the centre of query q
    const int64_t* qcol_off;   // [nq+1] offsets into qcol_idx
    const int32_t* qcol_idx;   // predicate-ordered generator columns of each query
    const double* pl;          // [ncols] predicate bounds by column
    const double* pu;
    const int4* box;           // [ncols] window of each column
    const int32_t* col_q;      // [ncols] query of each column
    int img_h, img_w, img_c;   // shape of the current tensor (rows are h-fastest, then w, then c)
    // cohorts whose columns are reduced through their windows (their columns are in no chunk)
    WinCohorts win;
    int win_slices;            // chunks per query the windowed cohorts fill (range_windows_slices())
    const double* win_pack;    // window-only copies of the windowed cohorts (all of them, or null: read V)
    int32_t* win_scratch;      // range_windows_scratch_ints() int32
    const int32_t* win_seg;    // [win.n][nq] first column of query q in windowed cohort k
    // chunk list for the bound reduction
    int n_chunks;
    const int64_t* chunk_beg;  // [n_chunks] positions in qcol_idx
    const int64_t* chunk_end;
    const int32_t* q_chunk_off;// [nq+1] chunks of query q are q_chunk_off[q] .. q_chunk_off[q+1]
    double* partial;           // [n_chunks][2][N]
    // outputs
    double* lb;                // [nq][N]
    double* ub;                // [nq][N]
    uint8_t* state;            // [nq][N] 0 keep, 1 dead, 2 crossing
    int32_t* rank;             // [nq][N] rank of a crossing neuron within its query
    int32_t* blk_cross;        // [nq][blocks] crossing count per row block, then its exclusive scan
    int64_t* q_cross;          // [nq] crossing count per query
    int64_t* q_dead;           // [nq]
    int64_t* q_new_off;        // [nq+1] exclusive scan of q_cross
};
// Per-layer record of the appended columns (K = total crossing neurons of the batch).
struct ReluRecord {
    int32_t* idx;              // [K] neuron index of new column c
    int32_t* q;                // [K] its query
    double* c;                 // [K] centre value of the row before zeroing
    double* l;                 // [K] estimated lower bound
    double* u;                 // [K] estimated upper bound
    double* G;                 // crossing rows before zeroing, per query a [k_q x P_q] column-major block (null: not kept)
    int64_t* G_off;            // [nq] start of each block
};
int relu_blocks_per_query(int64_t N);
int launch_estimate_ranges(cudaStream_t st, const ReluWork& w, int64_t* launches);
// Sharded generators: per-query sums of the chunk partials (no centre), [nq][2][N].
int launch_reduce_chunks(cudaStream_t st, const ReluWork& w, double* sums, int64_t* launches);
// Partial sums of all ranks in peer-mapped buffers, for the classification that adds them itself.
struct PeerSums {
    double* const* tab;        // device array [world]: every rank's buffer as mapped on this device
    int64_t slot_off;          // offset (doubles) of this call's [nq][2][N] sums in each buffer
    int rank, world;
    unsigned long long epoch;  // a rank's flag (64-bit word `rank` at the start of a buffer) reaches this value
                               // once its sums of this call are written
    int* status;               // [0] set to 1 when a wait ran out; [1] the rank waited for, [2] the epoch
    long long max_polls;
};
// sums = nullptr: combine the chunk partials directly; else classify from the (all-reduced) sums;
// peers != nullptr: wait for every rank's flag and add the ranks' sums from peer memory while classifying.
int launch_classify_scan(cudaStream_t st, const ReluWork& w, const double* sums, int64_t* launches,
                         const PeerSums* peers = nullptr);
int launch_rank_cross(cudaStream_t st, const ReluWork& w, const ReluRecord& rec, int64_t* launches);
// LP-tightened bounds: overwrite the bounds of the k listed neurons of one query (lb_q / ub_q point at the
// query's [N] arrays), then classify every query again from w.lb / w.ub (outputs as launch_classify_scan).
int launch_tighten_bounds(cudaStream_t st, int64_t k, int64_t N, const int32_t* idx, const double* xmin,
                          const double* xmax, double* lb_q, double* ub_q, int64_t* launches);
int launch_reclassify_scan(cudaStream_t st, const ReluWork& w, int64_t* launches);
// out[pos*k + t] = V[col][idx[t]] for the P listed columns (pos = col_pos[col]): rows of a query's matrix.
int launch_gather_rows(cudaStream_t st, int64_t k, int64_t P, const int32_t* idx, const int32_t* qcol,
                       const int64_t* col_pos, const double* V, int64_t ld, double* out, int64_t* launches);
// Zero dead and crossing rows in all existing columns; save crossing rows.
int launch_relu_zero_rows(cudaStream_t st, const ReluWork& w, int64_t ncols, const int32_t* col_q,
                          const ReluRecord& rec, const int64_t* col_pos, int64_t* launches);
// Append one one-hot column per crossing neuron with its predicate bounds and
// rebuild the per-query column lists.
// (rank, world) = generator shard; K_loc = new columns this rank holds; P_in = predicates per
// query entering the layer over all ranks (nullptr when unsharded).
// materialize = false leaves the new columns implicit (only their metadata is written).
int launch_relu_append(cudaStream_t st, const ReluWork& w, int64_t ncols_old, int64_t K_loc, int rank, int world,
                       bool materialize, const int64_t* P_in, const ReluRecord& rec, int32_t* col_q, double* pl, double* pu,
                       int64_t* col_pos, int img_h, int img_w, int4* box,
                       int64_t* new_qcol_off, int32_t* new_qcol_idx, int64_t* launches);

// Halfspace rows against output sets; see relu_star.cu.  Pair p tests row G[p] (length Nout)
// with offset g[p] on query pair_q[p]; margin (nullable, 2*n_pairs doubles): margin[p] = box minimum of
// G x - g, margin[n_pairs + p] = sum of the magnitudes of its terms;
// r_out (nullable) receives the predicate coefficients of pair p at r_off[p] + position.
int launch_halfspace_pairs(cudaStream_t st, int n_pairs, const int32_t* pair_q, int64_t Nout, int64_t ld,
                           const double* V, const int64_t* qcol_off, const int32_t* qcol_idx, const double* pl,
                           const double* pu, const double* G, const double* g, double* margin, double* r_out,
                           const int64_t* r_off, const int64_t* col_pos, int add_center, double* part,
                           int64_t* launches);
constexpr int HS_SPLIT = 32;     // slices of a query's column list; `part` holds 2 * n_pairs * HS_SPLIT doubles
// Back-substitution bound of halfspace rows through the recorded ReLU relaxations (see relu_star.cu): r holds
// each pair's row by predicate position (as launch_halfspace_pairs writes it) and is overwritten;
// bound[p] receives a lower bound of G x - g over the whole star set of the pair's query, bound[n_pairs + p]
// the sum of the magnitudes of its terms.
struct BacksubLayer {
    const double* G;            // crossing rows, per query a kq x P_in block (column-major) at G_off[q]
    const int64_t* G_off;       // [nq+1]
    const double* c;            // per new column: centre value, lower and upper bound of the pre-activation
    const double* l;
    const double* u;
    const int64_t* new_off;     // [nq+1] first new column of each query
    const int64_t* P_in;        // [nq] predicates entering the layer
};
constexpr int MAX_BACKSUB_LAYERS = 32;
struct BacksubLayers {
    int n;
    BacksubLayer L[MAX_BACKSUB_LAYERS];
};
int launch_backsub(cudaStream_t st, const BacksubLayers& layers, int n_pairs, const int32_t* pair_q, int64_t Nout,
                   int64_t ld, const double* V, const double* G, const double* g, double* r, const int64_t* r_off,
                   const int64_t* qcol_off, const int32_t* qcol_idx, const double* pl, const double* pu, double* bound,
                   int64_t* launches);
// Witness search kernels (one point per pair, X is [ld x n_pairs]).
int launch_witness_x0_bounds(cudaStream_t st, int n_pairs, const int32_t* pair_q, int64_t N, int64_t ld,
                             const double* lbub, const double* r, const int64_t* r_off, double* X,
                             int64_t* launches);
int launch_witness_x0_star(cudaStream_t st, int n_pairs, const int32_t* pair_q, int64_t N, int64_t ld, int64_t ld0,
                           const double* V0, const int64_t* gen0, const double* pl0, const double* pu0,
                           const double* r, const int64_t* r_off, const int64_t* pos0, int add_center, double* X,
                           int64_t* launches);
int launch_witness_relu(cudaStream_t st, int n_pairs, const int32_t* pair_q, int64_t N, int64_t ld, double* X,
                        const double* lb, const double* ub, const int32_t* rank, const int64_t* P_in,
                        const double* r, const int64_t* r_off, double* alpha, int64_t* launches);
// max(x, 0) in place on n concrete points X [ld x n] (NN.evaluate's ReLU).
int launch_relu_points(cudaStream_t st, int64_t n, int64_t N, int64_t ld, double* X, int64_t* launches);
int launch_witness_value(cudaStream_t st, int n_pairs, int64_t Nout, int64_t ld, const double* X, const double* G,
                         const double* g, double* value, double* scale, int64_t* launches);

// Build the input set of a bounds-form query batch: centres, and per generator its metadata and either
// its column in V (hot_idx null) or its (entry, half width) pair in hot_idx / hot_scale, indexed by
// column - nq, with the column's memory left untouched.
int launch_build_from_bounds(cudaStream_t st, int nq, int64_t N, int64_t ld, const double* lbub,
                             const int64_t* q_gen_off, int rank, int world, double* V, int32_t* col_q, double* pl,
                             double* pu, int32_t* qcol_idx, int64_t* col_pos, int img_h, int img_w, int4* box,
                             int32_t* hot_idx, double* hot_scale, int64_t* launches);
// Move the windows of columns [0, n) through a convolution / pooling layer (extent = (k-1)*dilation).
int launch_update_windows(cudaStream_t st, int64_t n, int4* box, int pad_t, int pad_l, int ext_h,
                          int ext_w, int sh, int sw, int64_t* launches);
// Mark columns [0, n) as dense (a window that covers any image).
int launch_fill_dense_windows(cudaStream_t st, int64_t n, int4* box, int64_t* launches);
// Average pooling of windowed columns [col_base, col_base+ncols): only the win.wh x win.ww output patch of
// each column is computed (the output block is zero filled by the caller).
int launch_avgpool_windowed(cudaStream_t st, const PoolGeom& g, const RowMask& mask, const ColWindows& win,
                            int64_t col_base, const double* Vin, int64_t ld_in, double* Vout, int64_t ld_out,
                            int64_t ncols, int64_t* launches);
// Compact (window-only, channel-fastest) storage of windowed columns; see elementwise.cu.  Column jj of the
// launch (absolute column col_base + jj) starts at comp + jj*stride.
int launch_avgpool_compact(cudaStream_t st, const PoolGeom& g, const RowMask& mask, const int4* box, int64_t col_base,
                           int64_t ncols, int wh_in, int ww_in, int wh_out, int ww_out, const double* comp_in,
                           int64_t stride_in, double* comp_out, int64_t stride_out, int64_t* launches);
int launch_state_channel_fastest(cudaStream_t st, int nq, int H, int W, int C, const uint8_t* state, uint8_t* cf,
                                 int64_t* launches);
// Writes the in-image entries of the compact windows into the full-length columns [col0, col0+n) of V
// (clear: the columns are zeroed first, else the memory outside the windows is left as it is).
int launch_expand_compact(cudaStream_t st, int H, int W, int C, const int4* box, int64_t col0, int64_t n, int wh, int ww,
                          const double* comp, int64_t stride, double* V, int64_t ld, bool clear, int64_t* launches);
int launch_count_bounds(cudaStream_t st, int nq, int64_t N, const double* lbub, int64_t* q_count,
                        int64_t* launches);

}  // namespace nnvb
