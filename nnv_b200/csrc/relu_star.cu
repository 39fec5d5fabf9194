// The LP-free PosLin (ReLU) approx-star step on a batch of star sets:
//   1. Star.estimateRanges (Star.m:1078-1106): lb/ub of every neuron from the
//      predicate box,
//   2. classification (PosLin.m:1594,1598): dead = ub <= 0, crossing = lb < 0 & ub > 0,
//      and a warp-ballot prefix scan that ranks the crossing neurons of each query
//      in ascending linear index,
//   3. Star.resetRow + multipleStepReachStarApprox_at_one (Star.m:1449-1450,
//      PosLin.m:698-740): zero dead and crossing rows of every existing column,
//      append a one-hot column per crossing neuron with predicate range [0, ub],
//      and save the crossing rows (before zeroing) that make up the new
//      constraint rows.
// All of it is HBM-bandwidth work: V is read once for the bounds and touched
// once more where rows are cleared.
#include "common.cuh"

namespace nnvb {

namespace {

// ---------------------------------------------------------------------------
// 1. partial bound sums.  A chunk is a run of one query's generator columns
//    (positions [beg,end) of its predicate-ordered column list).  Every thread
//    owns two adjacent rows and walks the chunk's columns in order, so the sum
//    of a chunk has a fixed order; chunks are combined in order by the finalize
//    kernel.  lo += max(v,0)*pl + min(v,0)*pu ; hi += max(v,0)*pu + min(v,0)*pl.
template <int UNROLL>
__global__ void __launch_bounds__(256)
range_partial_rows2_kernel(int64_t N, int64_t ld, const double* __restrict__ V,
                           const int32_t* __restrict__ qcol_idx, const double* __restrict__ pl,
                           const double* __restrict__ pu, const int64_t* __restrict__ chunk_beg,
                           const int64_t* __restrict__ chunk_end, double* __restrict__ partial) {
    const int chunk = blockIdx.x;
    const int64_t i = (int64_t(blockIdx.y) * blockDim.x + threadIdx.x) * 2;
    if (i >= N) return;
    const bool two = i + 1 < N;
    const int64_t beg = chunk_beg[chunk], end = chunk_end[chunk];
    double lo0 = 0.0, hi0 = 0.0, lo1 = 0.0, hi1 = 0.0;
    int64_t pos = beg;
    if (two) {
        for (; pos + UNROLL <= end; pos += UNROLL) {
            double2 v[UNROLL];
            double a[UNROLL], b[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int64_t col = qcol_idx[pos + u];
                v[u] = __ldcs(reinterpret_cast<const double2*>(V + col * ld + i));
                a[u] = pl[col];
                b[u] = pu[col];
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                // max(v,0)*pl + min(v,0)*pu == v * (v > 0 ? pl : pu): one product per bound
                const bool s0 = v[u].x > 0.0, s1 = v[u].y > 0.0;
                lo0 = fma(v[u].x, s0 ? a[u] : b[u], lo0);
                hi0 = fma(v[u].x, s0 ? b[u] : a[u], hi0);
                lo1 = fma(v[u].y, s1 ? a[u] : b[u], lo1);
                hi1 = fma(v[u].y, s1 ? b[u] : a[u], hi1);
            }
        }
    }
    for (; pos < end; ++pos) {
        const int64_t col = qcol_idx[pos];
        const double a = pl[col], b = pu[col];
        const double x = V[col * ld + i];
        const double p0 = fmax(x, 0.0), n0 = fmin(x, 0.0);
        lo0 = fma(p0, a, lo0); lo0 = fma(n0, b, lo0);
        hi0 = fma(p0, b, hi0); hi0 = fma(n0, a, hi0);
        if (two) {
            const double y = V[col * ld + i + 1];
            const double p1 = fmax(y, 0.0), n1 = fmin(y, 0.0);
            lo1 = fma(p1, a, lo1); lo1 = fma(n1, b, lo1);
            hi1 = fma(p1, b, hi1); hi1 = fma(n1, a, hi1);
        }
    }
    double* plo = partial + int64_t(chunk) * 2 * N;
    double* phi = plo + N;
    plo[i] = lo0;
    phi[i] = hi0;
    if (two) { plo[i + 1] = lo1; phi[i + 1] = hi1; }
}

// ---------------------------------------------------------------------------
// Windowed columns.  A column of a windowed cohort is exactly zero outside its window box[col] (the memory
// there may hold stale data), so it adds to the bounds of the pixels inside that window only.  The columns
// of each (query, cohort) are sorted by window origin; a block then takes a strip of TH pixels of one pixel
// column (all channels) and visits the columns whose origin lies in the ww x (TH + wh - 1) bins that can
// cover the strip: a few contiguous runs of the sorted order.  The sums are formed in that order (cohort,
// origin column, origin row, column index), which does not depend on the schedule.
//
// 1. count the columns of every (cohort, query, origin bin)
__global__ void win_hist_kernel(WinCohorts wc, int nq, const int4* __restrict__ box, const int32_t* __restrict__ col_q,
                                int32_t* __restrict__ bins) {
    const WinCohort co = wc.c[blockIdx.y];
    const int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= co.n) return;
    const int64_t col = co.col0 + t;
    const int4 bx = box[col];
    const int bh = bx.x + co.wh - 1, bw = bx.y + co.ww - 1;
    if (bh < 0 || bw < 0 || bh >= co.KH || bw >= co.KW) return;        // window off the image: an all-zero column
    atomicAdd(bins + co.bin_base + int64_t(col_q[col]) * (co.KH * co.KW + 1) + bh + co.KH * bw, 1);
}

// 2. exclusive scan of each (cohort, query) table in place; entry KH*KW receives the total
__global__ void __launch_bounds__(256) win_scan_kernel(WinCohorts wc, int32_t* __restrict__ bins) {
    const WinCohort co = wc.c[blockIdx.y];
    const int nb = co.KH * co.KW + 1;
    int32_t* b = bins + co.bin_base + int64_t(blockIdx.x) * nb;
    __shared__ int warp_tot[8];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int base = 0; base < nb; base += 256) {
        const int i = base + threadIdx.x;
        const int v = i < nb ? b[i] : 0;
        int inc = v;
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += n;
        }
        if (lane == 31) warp_tot[warp] = inc;
        __syncthreads();
        int before = carry;
        for (int w2 = 0; w2 < warp; ++w2) before += warp_tot[w2];
        if (i < nb) b[i] = before + inc - v;
        __syncthreads();
        if (threadIdx.x == 255) carry = before + inc;
        __syncthreads();
    }
}

// 3. scatter the columns into their bins (any order within a bin) ...
__global__ void win_scatter_kernel(WinCohorts wc, int nq, const int4* __restrict__ box, const int32_t* __restrict__ col_q,
                                   const int32_t* __restrict__ bins, int32_t* __restrict__ cursor,
                                   const int32_t* __restrict__ seg, int32_t* __restrict__ tmp) {
    const WinCohort co = wc.c[blockIdx.y];
    const int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= co.n) return;
    const int64_t col = co.col0 + t;
    const int4 bx = box[col];
    const int bh = bx.x + co.wh - 1, bw = bx.y + co.ww - 1;
    if (bh < 0 || bw < 0 || bh >= co.KH || bw >= co.KW) return;
    const int q = col_q[col];
    const int64_t e = co.bin_base + int64_t(q) * (co.KH * co.KW + 1) + bh + co.KH * bw;
    const int slot = bins[e] + atomicAdd(cursor + e, 1);
    tmp[seg[blockIdx.y * nq + q] + slot] = int32_t(col);
}

// 4. ... and order every bin by column index: an entry's place is the number of smaller entries in its bin
__global__ void win_rank_kernel(WinCohorts wc, int nq, const int4* __restrict__ box, const int32_t* __restrict__ col_q,
                                const int32_t* __restrict__ bins, const int32_t* __restrict__ seg,
                                const int32_t* __restrict__ tmp, int32_t* __restrict__ perm) {
    const WinCohort co = wc.c[blockIdx.y];
    const int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= co.n) return;
    const int64_t col = co.col0 + t;
    const int4 bx = box[col];
    const int bh = bx.x + co.wh - 1, bw = bx.y + co.ww - 1;
    if (bh < 0 || bw < 0 || bh >= co.KH || bw >= co.KW) return;
    const int q = col_q[col];
    const int64_t e = co.bin_base + int64_t(q) * (co.KH * co.KW + 1) + bh + co.KH * bw;
    const int s0 = seg[blockIdx.y * nq + q];
    const int b0 = bins[e], b1 = bins[e + 1];
    int rank = 0;
    for (int i = b0; i < b1; ++i) rank += tmp[s0 + i] < int32_t(col) ? 1 : 0;
    perm[s0 + b0 + rank] = int32_t(col);
}

// 5. the partial sums of the windowed cohorts: one chunk (the last) per query.
//    grid = (strips, nq); a thread owns RPT rows (pixel of the strip, channel), pixel fastest.
constexpr int RW_THREADS = 256;
constexpr int RW_RPT = 4;
constexpr int RW_MLP = 8;            // window loads a thread keeps in flight
constexpr int RW_MAX_RUNS = MAX_WIN_COHORTS * MAX_WIN_EXTENT;
// Four blocks per SM: at 64 registers the compiler keeps a few values of the prologue on the stack (about 60 bytes, none
// inside the candidate loop); 80 registers without any spill (three blocks per SM) measured 7 % slower: the kernel
// lives on loads in flight.
template <bool PACKED>
__global__ void __launch_bounds__(RW_THREADS, 4)
range_windows_kernel(int64_t N, int64_t ld, const double* __restrict__ V, const double* __restrict__ pl,
                     const double* __restrict__ pu, const int4* __restrict__ box, int H, int W, int C, int TH, int nq,
                     WinCohorts wc, const int32_t* __restrict__ bins, const int32_t* __restrict__ perm,
                     const int32_t* __restrict__ seg, const int32_t* __restrict__ q_chunk_off,
                     double* __restrict__ partial) {
    // blockIdx.z takes one slice of the strip's candidate list and fills one of the query's last gridDim.z chunks
    const int q = blockIdx.y;
    const int n_th = (H + TH - 1) / TH;
    const int w = blockIdx.x / n_th;
    const int hT = (blockIdx.x % n_th) * TH;

    __shared__ int run_src[RW_MAX_RUNS];      // first sorted entry of the run (index into perm)
    __shared__ int run_pre[RW_MAX_RUNS + 1];  // candidates before the run
    __shared__ int run_wh[RW_MAX_RUNS];
    __shared__ int run_co[PACKED ? RW_MAX_RUNS : 1];      // cohort of the run
    __shared__ int64_t s_off[PACKED ? RW_THREADS : 1];    // packed offset of entry (h = 0, w, c = 0) of a candidate
    __shared__ int n_runs_s;
    __shared__ int s_col[RW_THREADS], s_h0[RW_THREADS], s_wh[RW_THREADS];
    __shared__ double s_pl[RW_THREADS], s_pu[RW_THREADS];

    // runs: for every cohort and every origin column bw that can cover pixel column w, the bins of the
    // origin rows that can cover some pixel of the strip.  Slot k*MAX_WIN_EXTENT + d holds origin column
    // w + d of cohort k; the non-empty slots are then packed in slot order.
    for (int slot = threadIdx.x; slot < wc.n * MAX_WIN_EXTENT; slot += RW_THREADS) {
        const int k = slot / MAX_WIN_EXTENT, d = slot % MAX_WIN_EXTENT;
        const WinCohort& co = wc.c[k];
        int src = 0, len = 0;
        const int bw = w + d;
        if (d < co.ww && bw < co.KW) {
            const int32_t* b = bins + co.bin_base + int64_t(q) * (co.KH * co.KW + 1) + co.KH * bw;
            const int bh_hi = min(hT + TH - 1 + co.wh - 1, co.KH - 1);
            const int s0 = b[hT], s1 = b[bh_hi + 1];            // origin rows hT - wh + 1 .. hT + TH - 1
            src = seg[k * nq + q] + s0;
            len = s1 - s0;
        }
        run_src[slot] = src;
        run_wh[slot] = len;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int r = 0, total = 0;
        for (int k = 0; k < wc.n; ++k) {
            const int ww = wc.c[k].ww, wh = wc.c[k].wh;
            for (int d = 0; d < ww; ++d) {
                const int slot = k * MAX_WIN_EXTENT + d;
                const int src = run_src[slot], len = run_wh[slot];
                if (len <= 0) continue;
                // r <= slot: packing in place never overwrites an unread slot
                run_src[r] = src;
                run_pre[r] = total;
                run_wh[r] = wh;
                if (PACKED) run_co[r] = k;
                total += len;
                ++r;
            }
        }
        run_pre[r] = total;
        n_runs_s = r;
    }
    __syncthreads();
    const int n_runs = n_runs_s;
    const int total = run_pre[n_runs];
    const int per_slice = (total + gridDim.z - 1) / gridDim.z;
    const int c_lo = min(total, per_slice * int(blockIdx.z)), c_hi = min(total, c_lo + per_slice);

    // rows of this thread
    int64_t row[RW_RPT];
    int hh[RW_RPT];
    int cc[RW_RPT];
    double lo[RW_RPT], hi[RW_RPT];
#pragma unroll
    for (int r = 0; r < RW_RPT; ++r) {
        const int idx = threadIdx.x + r * RW_THREADS;
        // the window-only copies are channel-fastest: lanes along the channels there, along the pixels in V
        const int pix = PACKED ? idx / C : idx % TH, c = PACKED ? idx % C : idx / TH;
        hh[r] = hT + pix;
        row[r] = (c < C && pix < TH && hh[r] < H) ? hh[r] + int64_t(H) * (w + int64_t(W) * c) : int64_t(-1);
        if (PACKED) cc[r] = c;
        lo[r] = 0.0;
        hi[r] = 0.0;
    }

    for (int base = c_lo; base < c_hi; base += RW_THREADS) {
        const int i = base + threadIdx.x;
        if (i < c_hi) {
            int a = 0, b2 = n_runs - 1;                 // last run with run_pre <= i
            while (a < b2) {
                const int m = (a + b2 + 1) >> 1;
                if (run_pre[m] <= i) a = m; else b2 = m - 1;
            }
            const int col = perm[run_src[a] + (i - run_pre[a])];
            s_col[threadIdx.x] = col;
            const int4 bx = box[col];
            s_h0[threadIdx.x] = bx.x;
            s_wh[threadIdx.x] = run_wh[a];
            if (PACKED) {
                const WinCohort& co = wc.c[run_co[a]];
                s_off[threadIdx.x] = co.pack_off + (int64_t(col) - co.col0) * co.pack_stride +
                                     (int64_t(w - bx.y) * co.wh - bx.x) * C;
            }
            s_pl[threadIdx.x] = pl[col];
            s_pu[threadIdx.x] = pu[col];
        }
        __syncthreads();
        const int cnt = min(RW_THREADS, c_hi - base);
#pragma unroll
        for (int r = 0; r < RW_RPT; ++r) {
            if (row[r] < 0) continue;
            int j = 0;
            for (; j + RW_MLP <= cnt; j += RW_MLP) {    // RW_MLP loads in flight, added in candidate order
                double v[RW_MLP];
#pragma unroll
                for (int u = 0; u < RW_MLP; ++u) {
                    const bool in = unsigned(hh[r] - s_h0[j + u]) < unsigned(s_wh[j + u]);
                    v[u] = !in ? 0.0 : PACKED ? V[s_off[j + u] + int64_t(hh[r]) * C + cc[r]]
                                              : V[int64_t(s_col[j + u]) * ld + row[r]];
                }
#pragma unroll
                for (int u = 0; u < RW_MLP; ++u) {
                    // max(v,0)*pl + min(v,0)*pu == v * (v > 0 ? pl : pu): one product per bound
                    const bool pos = v[u] > 0.0;
                    lo[r] = fma(v[u], pos ? s_pl[j + u] : s_pu[j + u], lo[r]);
                    hi[r] = fma(v[u], pos ? s_pu[j + u] : s_pl[j + u], hi[r]);
                }
            }
            for (; j < cnt; ++j) {
                const bool in = unsigned(hh[r] - s_h0[j]) < unsigned(s_wh[j]);
                const double v = !in ? 0.0 : PACKED ? V[s_off[j] + int64_t(hh[r]) * C + cc[r]]
                                                    : V[int64_t(s_col[j]) * ld + row[r]];
                const bool pos = v > 0.0;
                lo[r] = fma(v, pos ? s_pl[j] : s_pu[j], lo[r]);
                hi[r] = fma(v, pos ? s_pu[j] : s_pl[j], hi[r]);
            }
        }
        __syncthreads();
    }

    double* plo = partial + int64_t(q_chunk_off[q + 1] - int(gridDim.z) + int(blockIdx.z)) * 2 * N;
    double* phi = plo + N;
#pragma unroll
    for (int r = 0; r < RW_RPT; ++r) {
        if (row[r] < 0) continue;
        plo[row[r]] = lo[r];
        phi[row[r]] = hi[r];
    }
}

// Narrow sets (few rows, many columns): a warp owns 32 rows, the 8 warps of a
// block split the chunk's columns round-robin and are combined in warp order.
__global__ void __launch_bounds__(256)
range_partial_narrow_kernel(int64_t N, int64_t ld, const double* __restrict__ V,
                            const int32_t* __restrict__ qcol_idx, const double* __restrict__ pl,
                            const double* __restrict__ pu, const int64_t* __restrict__ chunk_beg,
                            const int64_t* __restrict__ chunk_end, double* __restrict__ partial) {
    const int chunk = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t i = int64_t(blockIdx.y) * 32 + lane;
    const int64_t beg = chunk_beg[chunk], end = chunk_end[chunk];
    double lo = 0.0, hi = 0.0;
    if (i < N) {
        // four of the warp's columns in flight; the sums still run in column order
        for (int64_t pos = beg + warp; pos < end; pos += 32) {
            double x[4], a[4], b[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int64_t pu_ = pos + 8 * u;
                const int64_t col = pu_ < end ? qcol_idx[pu_] : -1;
                x[u] = col >= 0 ? V[col * ld + i] : 0.0;
                a[u] = col >= 0 ? pl[col] : 0.0;
                b[u] = col >= 0 ? pu[col] : 0.0;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (pos + 8 * u >= end) break;
                const double p0 = fmax(x[u], 0.0), n0 = fmin(x[u], 0.0);
                lo = fma(p0, a[u], lo); lo = fma(n0, b[u], lo);
                hi = fma(p0, b[u], hi); hi = fma(n0, a[u], hi);
            }
        }
    }
    __shared__ double slo[8][32], shi[8][32];
    slo[warp][lane] = lo;
    shi[warp][lane] = hi;
    __syncthreads();
    if (warp == 0 && i < N) {
        double l = 0.0, h = 0.0;
#pragma unroll
        for (int w = 0; w < 8; ++w) { l += slo[w][lane]; h += shi[w][lane]; }
        double* plo = partial + int64_t(chunk) * 2 * N;
        plo[i] = l;
        plo[N + i] = h;
    }
}

// ---------------------------------------------------------------------------
// 2a. finalize bounds and classify.  grid = (nq, row blocks of FIN_ROWS).
constexpr int FIN_THREADS = 256;
constexpr int FIN_ROWS = 256;    // rows per block (1 per thread)

__global__ void __launch_bounds__(FIN_THREADS)
range_finalize_kernel(int64_t N, int64_t ld, const double* __restrict__ V,
                      const int32_t* __restrict__ q_chunk_off, const double* __restrict__ partial,
                      double* __restrict__ lb, double* __restrict__ ub, uint8_t* __restrict__ state,
                      int32_t* __restrict__ blk_cross, unsigned long long* __restrict__ q_dead, int nblk) {
    const int q = blockIdx.x;
    const int c0 = q_chunk_off[q], c1 = q_chunk_off[q + 1];
    int n_cross = 0, n_dead = 0;
    for (int r = 0; r < FIN_ROWS / FIN_THREADS; ++r) {
        const int64_t i = int64_t(blockIdx.y) * FIN_ROWS + r * FIN_THREADS + threadIdx.x;
        if (i >= N) break;
        const double c = V[int64_t(q) * ld + i];     // centre column of query q is column q
        double lo = 0.0, hi = 0.0;
        int ch = c0;
        for (; ch + 8 <= c1; ch += 8) {            // eight chunk partials in flight, added in chunk order
            double a[8], bq[8];
#pragma unroll
            for (int u8 = 0; u8 < 8; ++u8) {
                const double* pp = partial + int64_t(ch + u8) * 2 * N;
                a[u8] = pp[i];
                bq[u8] = pp[N + i];
            }
#pragma unroll
            for (int u8 = 0; u8 < 8; ++u8) { lo += a[u8]; hi += bq[u8]; }
        }
        for (; ch < c1; ++ch) {
            const double* pp = partial + int64_t(ch) * 2 * N;
            lo += pp[i];
            hi += pp[N + i];
        }
        const double l = c + lo, u = c + hi;
        lb[int64_t(q) * N + i] = l;
        ub[int64_t(q) * N + i] = u;
        uint8_t s = 0;
        if (u <= 0.0) { s = 1; ++n_dead; }
        else if (l < 0.0 && u > 0.0) { s = 2; ++n_cross; }
        state[int64_t(q) * N + i] = s;
    }
    // block totals (integer: order-free)
    __shared__ int sc[FIN_THREADS / 32], sd[FIN_THREADS / 32];
    for (int o = 16; o; o >>= 1) {
        n_cross += __shfl_down_sync(0xffffffffu, n_cross, o);
        n_dead += __shfl_down_sync(0xffffffffu, n_dead, o);
    }
    if ((threadIdx.x & 31) == 0) { sc[threadIdx.x >> 5] = n_cross; sd[threadIdx.x >> 5] = n_dead; }
    __syncthreads();
    if (threadIdx.x == 0) {
        int tc = 0, td = 0;
        for (int w = 0; w < FIN_THREADS / 32; ++w) { tc += sc[w]; td += sd[w]; }
        blk_cross[int64_t(q) * nblk + blockIdx.y] = tc;
        if (td) atomicAdd(q_dead + q, (unsigned long long)td);
    }
}

// 2b. per query: exclusive scan of its block counts; total -> q_cross[q].
__global__ void scan_blocks_kernel(int nblk, int32_t* __restrict__ blk_cross, int64_t* __restrict__ q_cross) {
    const int q = blockIdx.x;
    int32_t* b = blk_cross + int64_t(q) * nblk;
    __shared__ int warp_tot[32];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int base = 0; base < nblk; base += blockDim.x) {
        const int i = base + threadIdx.x;
        const int v = i < nblk ? b[i] : 0;
        int inc = v;
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += n;
        }
        if (lane == 31) warp_tot[warp] = inc;
        __syncthreads();
        int before = carry;
        for (int w = 0; w < warp; ++w) before += warp_tot[w];
        if (i < nblk) b[i] = before + inc - v;
        __syncthreads();
        if (threadIdx.x == 0) {
            int tot = 0;
            for (int w = 0; w < nw; ++w) tot += warp_tot[w];
            carry += tot;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) q_cross[q] = carry;
}

// 2c. exclusive scan over queries (single block): q_new_off[0..nq].
__global__ void scan_queries_kernel(int nq, const int64_t* __restrict__ q_cross, int64_t* __restrict__ q_new_off) {
    __shared__ long long warp_tot[32];
    __shared__ long long carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int base = 0; base < nq; base += blockDim.x) {
        const int i = base + threadIdx.x;
        const long long v = i < nq ? q_cross[i] : 0;
        long long inc = v;
        for (int o = 1; o < 32; o <<= 1) {
            const long long n = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += n;
        }
        if (lane == 31) warp_tot[warp] = inc;
        __syncthreads();
        long long before = carry;
        for (int w = 0; w < warp; ++w) before += warp_tot[w];
        if (i < nq) q_new_off[i] = before + inc - v;
        __syncthreads();
        if (threadIdx.x == 0) {
            long long tot = 0;
            for (int w = 0; w < nw; ++w) tot += warp_tot[w];
            carry += tot;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) q_new_off[nq] = carry;
}

// 2d. rank crossing neurons (ascending index within the query) with a warp
// ballot scan, and write the per-new-column record.
__global__ void __launch_bounds__(FIN_THREADS)
rank_cross_kernel(int64_t N, int64_t ld, const double* __restrict__ V, const uint8_t* __restrict__ state,
                  const double* __restrict__ lb, const double* __restrict__ ub,
                  const int32_t* __restrict__ blk_off, int nblk, const int64_t* __restrict__ q_new_off,
                  int32_t* __restrict__ rank, int32_t* __restrict__ rec_idx, int32_t* __restrict__ rec_q,
                  double* __restrict__ rec_c, double* __restrict__ rec_l, double* __restrict__ rec_u) {
    const int q = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ int warp_cnt[FIN_THREADS / 32];
    int running = blk_off[int64_t(q) * nblk + blockIdx.y];
    const int64_t new0 = q_new_off[q];
    for (int r = 0; r < FIN_ROWS / FIN_THREADS; ++r) {
        const int64_t i = int64_t(blockIdx.y) * FIN_ROWS + r * FIN_THREADS + threadIdx.x;
        const bool is_cross = i < N && state[int64_t(q) * N + i] == 2;
        const unsigned bal = __ballot_sync(0xffffffffu, is_cross);
        if (lane == 0) warp_cnt[warp] = __popc(bal);
        __syncthreads();
        int before = running;
        int tot = 0;
        for (int w = 0; w < FIN_THREADS / 32; ++w) {
            if (w < warp) before += warp_cnt[w];
            tot += warp_cnt[w];
        }
        if (is_cross) {
            const int rk = before + __popc(bal & ((1u << lane) - 1u));
            rank[int64_t(q) * N + i] = rk;
            const int64_t c = new0 + rk;
            rec_idx[c] = int32_t(i);
            rec_q[c] = q;
            rec_c[c] = V[int64_t(q) * ld + i];
            rec_l[c] = lb[int64_t(q) * N + i];
            rec_u[c] = ub[int64_t(q) * N + i];
        }
        running += tot;
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// 3a. clear dead and crossing rows in every existing column; copy the crossing
// rows of generator columns into the layer's constraint record first.
// grid = (row blocks, column walkers).
__global__ void __launch_bounds__(256)
zero_rows_kernel(int nq, int64_t N, int64_t ld, double* __restrict__ V, int64_t ncols,
                 const int32_t* __restrict__ col_q, const uint8_t* __restrict__ state,
                 const int32_t* __restrict__ rank, double* __restrict__ rec_G,
                 const int64_t* __restrict__ rec_off, const int64_t* __restrict__ q_new_off,
                 const int64_t* __restrict__ col_pos) {
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= N) return;
    for (int64_t j = blockIdx.y; j < ncols; j += gridDim.y) {
        const int q = col_q[j];
        const uint8_t s = state[int64_t(q) * N + i];
        if (s == 0) continue;
        double* p = V + j * ld + i;
        if (s == 2 && rec_G != nullptr && j >= nq) {
            const int64_t kq = q_new_off[q + 1] - q_new_off[q];
            rec_G[rec_off[q] + col_pos[j] * kq + rank[int64_t(q) * N + i]] = *p;
        }
        *p = 0.0;
    }
}

// 3b. one-hot columns for the crossing neurons (the block was zero filled) and
// their predicate range [0, ub].  With the generators sharded over `world`
// ranks, new column c (numbered over the whole batch) lives on rank c % world;
// this rank materialises its K_loc columns t -> c = rank + t*world.
__global__ void append_cols_kernel(int64_t K_loc, int rank, int world, int write_v, int64_t ld, double* __restrict__ V,
                                   int64_t ncols_old, const int32_t* __restrict__ rec_idx,
                                   const int32_t* __restrict__ rec_q, const double* __restrict__ rec_u,
                                   const int64_t* __restrict__ q_new_off, const int64_t* __restrict__ qcol_off,
                                   const int64_t* __restrict__ P_in, int32_t* __restrict__ col_q,
                                   double* __restrict__ pl, double* __restrict__ pu,
                                   int64_t* __restrict__ col_pos, int img_h, int img_w, int4* __restrict__ box) {
    const int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= K_loc) return;
    const int64_t c = rank + t * world;
    const int64_t col = ncols_old + t;
    const int q = rec_q[c];
    if (write_v) V[col * ld + rec_idx[c]] = 1.0;     // else the column stays implicit until the next layer
    col_q[col] = q;
    pl[col] = 0.0;
    pu[col] = rec_u[c];
    // position in the query's predicate order (over all ranks)
    const int64_t p_in = P_in ? P_in[q] : (qcol_off[q + 1] - qcol_off[q]);
    col_pos[col] = p_in + (c - q_new_off[q]);
    box[col] = make_int4(rec_idx[c] % img_h, (rec_idx[c] / img_h) % img_w, 1, 1);   // a unit vector: one pixel
}

// 3c. new predicate-ordered column lists: old list of the query, then its new
// columns held by this rank (global numbers c = rank mod world within the query's range).
__global__ void rebuild_lists_kernel(int nq, int rank, int world, const int64_t* __restrict__ qcol_off,
                                     const int32_t* __restrict__ qcol_idx,
                                     const int64_t* __restrict__ q_new_off, int64_t ncols_old,
                                     int64_t* __restrict__ new_off, int32_t* __restrict__ new_idx) {
    const int q = blockIdx.x;
    const int64_t o0 = qcol_off[q], o1 = qcol_off[q + 1];
    const int64_t n0 = q_new_off[q], n1 = q_new_off[q + 1];
    // local new columns before / inside this query's range: t = (c - rank) / world for c = rank (mod world)
    auto first_t = [&](int64_t n) { return n <= rank ? int64_t(0) : (n - rank + world - 1) / world; };
    const int64_t t0 = first_t(n0), t1 = first_t(n1);
    const int64_t dst = o0 + t0;
    for (int64_t t = threadIdx.x; t < o1 - o0; t += blockDim.x) new_idx[dst + t] = qcol_idx[o0 + t];
    for (int64_t t = threadIdx.x; t < t1 - t0; t += blockDim.x)
        new_idx[dst + (o1 - o0) + t] = int32_t(ncols_old + t0 + t);
    if (threadIdx.x == 0) {
        new_off[q] = dst;
        if (q == nq - 1) new_off[nq] = o1 + t1;
    }
}

// Sharded generators: sum the chunk partials of each query (no centre) so that
// the ranks can add their sums before classifying.  grid = (nq, row blocks).
__global__ void __launch_bounds__(FIN_THREADS)
reduce_chunks_kernel(int64_t N, const int32_t* __restrict__ q_chunk_off, const double* __restrict__ partial,
                     double* __restrict__ sums) {
    const int q = blockIdx.x;
    const int c0 = q_chunk_off[q], c1 = q_chunk_off[q + 1];
    for (int r = 0; r < FIN_ROWS / FIN_THREADS; ++r) {
        const int64_t i = int64_t(blockIdx.y) * FIN_ROWS + r * FIN_THREADS + threadIdx.x;
        if (i >= N) break;
        double lo = 0.0, hi = 0.0;
        for (int ch = c0; ch < c1; ++ch) {
            const double* pp = partial + int64_t(ch) * 2 * N;
            lo += pp[i];
            hi += pp[N + i];
        }
        sums[(int64_t(q) * 2) * N + i] = lo;
        sums[(int64_t(q) * 2 + 1) * N + i] = hi;
    }
}

// ... and classify from the combined sums (same outputs as range_finalize_kernel).
__global__ void __launch_bounds__(FIN_THREADS)
classify_sums_kernel(int64_t N, int64_t ld, const double* __restrict__ V, const double* __restrict__ sums,
                     double* __restrict__ lb, double* __restrict__ ub, uint8_t* __restrict__ state,
                     int32_t* __restrict__ blk_cross, unsigned long long* __restrict__ q_dead, int nblk) {
    const int q = blockIdx.x;
    int n_cross = 0, n_dead = 0;
    for (int r = 0; r < FIN_ROWS / FIN_THREADS; ++r) {
        const int64_t i = int64_t(blockIdx.y) * FIN_ROWS + r * FIN_THREADS + threadIdx.x;
        if (i >= N) break;
        const double c = V[int64_t(q) * ld + i];
        const double l = c + sums[(int64_t(q) * 2) * N + i], u = c + sums[(int64_t(q) * 2 + 1) * N + i];
        lb[int64_t(q) * N + i] = l;
        ub[int64_t(q) * N + i] = u;
        uint8_t s = 0;
        if (u <= 0.0) { s = 1; ++n_dead; }
        else if (l < 0.0 && u > 0.0) { s = 2; ++n_cross; }
        state[int64_t(q) * N + i] = s;
    }
    __shared__ int sc[FIN_THREADS / 32], sd[FIN_THREADS / 32];
    for (int o = 16; o; o >>= 1) {
        n_cross += __shfl_down_sync(0xffffffffu, n_cross, o);
        n_dead += __shfl_down_sync(0xffffffffu, n_dead, o);
    }
    if ((threadIdx.x & 31) == 0) { sc[threadIdx.x >> 5] = n_cross; sd[threadIdx.x >> 5] = n_dead; }
    __syncthreads();
    if (threadIdx.x == 0) {
        int tc = 0, td = 0;
        for (int w = 0; w < FIN_THREADS / 32; ++w) { tc += sc[w]; td += sd[w]; }
        blk_cross[int64_t(q) * nblk + blockIdx.y] = tc;
        if (td) atomicAdd(q_dead + q, (unsigned long long)td);
    }
}

// The same classification with the sum over the ranks fused in: every rank's [nq][2][N] partial sums sit at
// slot_off in a buffer that all ranks have mapped (peer memory over NVLink).  A block first waits, with a
// bounded number of polls, until every rank has raised its flag for this call in THIS rank's buffer, then adds
// the ranks' sums in rank order with plain loads (L2-only, no multicast).  The order is the same on every rank,
// so all ranks classify identical numbers.  When a wait runs out the block records which rank it waited for in
// ps.status, writes "no crossing, no dead" for its rows and returns; the host reads the status word.
__global__ void __launch_bounds__(FIN_THREADS)
classify_peers_kernel(int64_t N, int64_t ld, const double* __restrict__ V, PeerSums ps,
                      double* __restrict__ lb, double* __restrict__ ub, uint8_t* __restrict__ state,
                      int32_t* __restrict__ blk_cross, unsigned long long* __restrict__ q_dead, int nblk) {
    const int q = blockIdx.x;
    __shared__ int s_bad;
    if (threadIdx.x == 0) s_bad = 0;
    __syncthreads();
    if (threadIdx.x < ps.world && threadIdx.x != ps.rank) {
        const volatile unsigned long long* flags = reinterpret_cast<const volatile unsigned long long*>(ps.tab[ps.rank]);
        long long polls = 0;
        while (flags[threadIdx.x] < ps.epoch) {
            if (++polls > ps.max_polls) {
                s_bad = 1;
                if (atomicCAS(ps.status, 0, 1) == 0) {
                    ps.status[1] = threadIdx.x;
                    ps.status[2] = int(ps.epoch);
                }
                break;
            }
            __nanosleep(polls < 64 ? 100 : 500);
        }
        __threadfence_system();          // the peer's sums were written before its flag
    }
    __syncthreads();
    const bool bad = s_bad != 0;
    int n_cross = 0, n_dead = 0;
    for (int r = 0; r < FIN_ROWS / FIN_THREADS; ++r) {
        const int64_t i = int64_t(blockIdx.y) * FIN_ROWS + r * FIN_THREADS + threadIdx.x;
        if (i >= N) break;
        const double c = V[int64_t(q) * ld + i];
        double lo = 0.0, hi = 0.0;
        if (!bad) {
            const int64_t o = ps.slot_off + (int64_t(q) * 2) * N + i;
            for (int rk = 0; rk < ps.world; ++rk) {
                const double* src = ps.tab[rk];
                lo += __ldcg(src + o);
                hi += __ldcg(src + o + N);
            }
        }
        const double l = c + lo, u = c + hi;
        lb[int64_t(q) * N + i] = l;
        ub[int64_t(q) * N + i] = u;
        uint8_t s = 0;
        if (!bad) {
            if (u <= 0.0) { s = 1; ++n_dead; }
            else if (l < 0.0 && u > 0.0) { s = 2; ++n_cross; }
        }
        state[int64_t(q) * N + i] = s;
    }
    __shared__ int sc[FIN_THREADS / 32], sd[FIN_THREADS / 32];
    for (int o = 16; o; o >>= 1) {
        n_cross += __shfl_down_sync(0xffffffffu, n_cross, o);
        n_dead += __shfl_down_sync(0xffffffffu, n_dead, o);
    }
    if ((threadIdx.x & 31) == 0) { sc[threadIdx.x >> 5] = n_cross; sd[threadIdx.x >> 5] = n_dead; }
    __syncthreads();
    if (threadIdx.x == 0) {
        int tc = 0, td = 0;
        for (int w = 0; w < FIN_THREADS / 32; ++w) { tc += sc[w]; td += sd[w]; }
        blk_cross[int64_t(q) * nblk + blockIdx.y] = tc;
        if (td) atomicAdd(q_dead + q, (unsigned long long)td);
    }
}

// LP-tightened bounds (PosLin.reach_star_approx2, PosLin.m:817-846): the caller solved the LPs of the neurons the
// estimates call crossing; their bounds replace the estimates ...
__global__ void tighten_bounds_kernel(int64_t k, int64_t N, const int32_t* __restrict__ idx, const double* __restrict__ xmin,
                                      const double* __restrict__ xmax, double* __restrict__ lb, double* __restrict__ ub) {
    const int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= k) return;
    lb[idx[t]] = xmin[t];
    ub[idx[t]] = xmax[t];
}

// ... and the layer is classified again from the bound arrays (same rule, same outputs as range_finalize_kernel).
__global__ void __launch_bounds__(FIN_THREADS)
reclassify_kernel(int64_t N, const double* __restrict__ lb, const double* __restrict__ ub, uint8_t* __restrict__ state,
                  int32_t* __restrict__ blk_cross, unsigned long long* __restrict__ q_dead, int nblk) {
    const int q = blockIdx.x;
    int n_cross = 0, n_dead = 0;
    for (int r = 0; r < FIN_ROWS / FIN_THREADS; ++r) {
        const int64_t i = int64_t(blockIdx.y) * FIN_ROWS + r * FIN_THREADS + threadIdx.x;
        if (i >= N) break;
        const double l = lb[int64_t(q) * N + i], u = ub[int64_t(q) * N + i];
        uint8_t s = 0;
        if (u <= 0.0) { s = 1; ++n_dead; }
        else if (l < 0.0 && u > 0.0) { s = 2; ++n_cross; }
        state[int64_t(q) * N + i] = s;
    }
    __shared__ int sc[FIN_THREADS / 32], sd[FIN_THREADS / 32];
    for (int o = 16; o; o >>= 1) {
        n_cross += __shfl_down_sync(0xffffffffu, n_cross, o);
        n_dead += __shfl_down_sync(0xffffffffu, n_dead, o);
    }
    if ((threadIdx.x & 31) == 0) { sc[threadIdx.x >> 5] = n_cross; sd[threadIdx.x >> 5] = n_dead; }
    __syncthreads();
    if (threadIdx.x == 0) {
        int tc = 0, td = 0;
        for (int w = 0; w < FIN_THREADS / 32; ++w) { tc += sc[w]; td += sd[w]; }
        blk_cross[int64_t(q) * nblk + blockIdx.y] = tc;
        if (td) atomicAdd(q_dead + q, (unsigned long long)td);
    }
}

// Rows idx[0..k) of the query's columns, in predicate order: out[pos*k + t] = V[col(pos)][idx[t]].
__global__ void gather_rows_kernel(int64_t k, int64_t P, const int32_t* __restrict__ idx, const int32_t* __restrict__ qcol,
                                   const int64_t* __restrict__ col_pos, const double* __restrict__ V, int64_t ld,
                                   double* __restrict__ out) {
    const int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= k) return;
    for (int64_t j = blockIdx.y; j < P; j += gridDim.y) {
        const int64_t col = qcol[j];
        out[col_pos[col] * k + t] = V[col * ld + idx[t]];
    }
}

// ---------------------------------------------------------------------------
// Halfspace rows and their minimum over the predicate box.  A "pair" is one
// halfspace row G_p x <= g_p tested against the output set of query pair_q[p].
// r_p[pos] = G_p . V[:, col(pos)] is the coefficient of predicate `pos` in the
// halfspace row of Star.intersectHalfSpace (Star.m:576); the minimum of
// G_p x - g_p over the predicate box is (G_p c - g_p) + sum_pos min(r*pl, r*pu).
// block = one pair; lanes stride over the query's columns.  r_out (optional)
// receives the coefficients at r_off[p] + pos.
__global__ void __launch_bounds__(256)
halfspace_pairs_kernel(const int32_t* __restrict__ pair_q, int64_t Nout, int64_t ld,
                       const double* __restrict__ V, const int64_t* __restrict__ qcol_off,
                       const int32_t* __restrict__ qcol_idx, const double* __restrict__ pl,
                       const double* __restrict__ pu, const double* __restrict__ G,
                       double* __restrict__ r_out, const int64_t* __restrict__ r_off,
                       const int64_t* __restrict__ col_pos, double* __restrict__ part) {
    const int p = blockIdx.x;
    const int q = pair_q[p];
    const double* Gr = G + int64_t(p) * Nout;
    double acc = 0.0, mag = 0.0;
    // blockIdx.y takes one contiguous slice of the query's column list
    const int64_t q0 = qcol_off[q], q1 = qcol_off[q + 1];
    const int64_t per = (q1 - q0 + gridDim.y - 1) / gridDim.y;
    const int64_t o0 = q0 + per * blockIdx.y, o1 = min(q1, o0 + per);
    for (int64_t pos = o0 + threadIdx.x; pos < o1; pos += blockDim.x) {
        const int64_t col = qcol_idx[pos];
        const double* v = V + col * ld;
        double r = 0.0;
        for (int64_t o = 0; o < Nout; ++o) r = fma(Gr[o], v[o], r);
        const double t = fmin(r * pl[col], r * pu[col]);
        acc += t;
        mag += fabs(t);
        if (r_out) r_out[r_off[p] + col_pos[col]] = r;     // position in the query's predicate order
    }
    __shared__ double s[256], sm[256];
    s[threadIdx.x] = acc;
    sm[threadIdx.x] = mag;
    __syncthreads();
    for (int o = 128; o; o >>= 1) {
        if (threadIdx.x < o) { s[threadIdx.x] += s[threadIdx.x + o]; sm[threadIdx.x] += sm[threadIdx.x + o]; }
        __syncthreads();
    }
    if (threadIdx.x == 0 && part) {
        part[(int64_t(p) * gridDim.y + blockIdx.y) * 2] = s[0];
        part[(int64_t(p) * gridDim.y + blockIdx.y) * 2 + 1] = sm[0];
    }
}

// margin[p] = (centre term) + the slices' partial minima, added in slice order; margin[n_pairs + p] = the sum
// of the magnitudes of every term that went into it (what a rounding guard on the sign of margin[p] scales with).
__global__ void halfspace_margin_kernel(int n_pairs, int n_split, const int32_t* __restrict__ pair_q, int64_t Nout,
                                        int64_t ld, const double* __restrict__ V, const double* __restrict__ G,
                                        const double* __restrict__ g, const double* __restrict__ part,
                                        double* __restrict__ margin, int add_center) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= n_pairs) return;
    double r = 0.0, mag = 0.0;
    if (add_center) {                          // with sharded generators only one rank adds the centre term
        const double* Gr = G + int64_t(p) * Nout;
        const double* v = V + int64_t(pair_q[p]) * ld;
        for (int64_t o = 0; o < Nout; ++o) {
            r = fma(Gr[o], v[o], r);
            mag += fabs(Gr[o] * v[o]);
        }
        r -= g[p];
        mag += fabs(g[p]);
    }
    double sum = 0.0;
    for (int s = 0; s < n_split; ++s) {
        sum += part[(int64_t(p) * n_split + s) * 2];
        mag += part[(int64_t(p) * n_split + s) * 2 + 1];
    }
    margin[p] = r + sum;
    margin[n_pairs + p] = mag;
}

// ---------------------------------------------------------------------------
// Back-substitution bound.  The box minimum above treats every predicate as free in its range.  With
// the crossing rows of every ReLU layer at hand (constraint records) the relaxation itself can be used:
// a new predicate y of a crossing neuron with pre-activation x = c + G alpha (alpha: the predicates
// that existed before its layer) satisfies y >= 0, y >= x and y <= a (x - l), a = u / (u - l)
// (PosLin.m:716-735).  A term rho*y of the halfspace row is therefore bounded from below by
// rho*lambda*x for any lambda in [0,1] when rho >= 0 (lambda = 1 if u >= -l, else 0) and by rho*a*(x - l)
// when rho < 0.  Substituting layer by layer, last layer first, leaves a row over the input predicates
// only, whose box minimum is a lower bound of the row over the whole star set: the minimum the
// emptiness LP of Star.isEmptySet (Star.m:1216-1232) would have to beat.  A positive bound proves the
// intersection empty.  One block per pair; r holds the row by predicate position and is overwritten.
__global__ void __launch_bounds__(256)
backsub_kernel(BacksubLayers layers, const int32_t* __restrict__ pair_q, int64_t Nout, int64_t ld,
               const double* __restrict__ V, const double* __restrict__ Gh, const double* __restrict__ gh,
               double* __restrict__ r, const int64_t* __restrict__ r_off, const int64_t* __restrict__ qcol_off,
               const int32_t* __restrict__ qcol_idx, const double* __restrict__ pl, const double* __restrict__ pu,
               double* __restrict__ bound) {
    const int p = blockIdx.x;
    const int q = pair_q[p];
    double* rp = r + r_off[p];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __shared__ double red[256], redm[256];
    double konst = 0.0, kmag = 0.0;         // kept by thread 0; kmag: magnitudes of the terms of the bound
    if (tid == 0) {
        const double* Gr = Gh + int64_t(p) * Nout;
        const double* v = V + int64_t(q) * ld;
        for (int64_t o = 0; o < Nout; ++o) {
            konst = fma(Gr[o], v[o], konst);
            kmag += fabs(Gr[o] * v[o]);
        }
        konst -= gh[p];
        kmag += fabs(gh[p]);
    }
    int64_t P_first = qcol_off[q + 1] - qcol_off[q];
    for (int L = layers.n - 1; L >= 0; --L) {
        const BacksubLayer& rec = layers.L[L];
        const int64_t c0 = rec.new_off[q];
        const int64_t kq = rec.new_off[q + 1] - c0;
        const int64_t Pin = rec.P_in[q];
        P_first = Pin;
        // weights of the pre-activations, stored over the coefficients they replace
        double part = 0.0, pmag = 0.0;
        for (int64_t t = tid; t < kq; t += 256) {
            const double rho = rp[Pin + t];
            const double l = rec.l[c0 + t], u = rec.u[c0 + t], c = rec.c[c0 + t];
            double w;
            if (rho >= 0.0) {
                w = (u >= -l) ? rho : 0.0;
                part += w * c;
                pmag += fabs(w * c);
            } else {
                w = rho * (u / (u - l));
                part += w * (c - l);
                pmag += fabs(w * c) + fabs(w * l);
            }
            rp[Pin + t] = w;
        }
        red[tid] = part;
        redm[tid] = pmag;
        __syncthreads();
        for (int o = 128; o; o >>= 1) {
            if (tid < o) { red[tid] += red[tid + o]; redm[tid] += redm[tid + o]; }
            __syncthreads();
        }
        if (tid == 0) { konst += red[0]; kmag += redm[0]; }
        // r[j] += sum_t w_t G[t, j]: a warp per earlier predicate, lanes over the layer's crossing neurons
        const double* Gq = rec.G + rec.G_off[q];
        for (int64_t j = warp; j < Pin; j += 8) {
            double acc = 0.0;
            for (int64_t t = lane; t < kq; t += 32) acc = fma(rp[Pin + t], Gq[j * kq + t], acc);
            for (int o = 16; o; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
            if (lane == 0) rp[j] += acc;
        }
        __syncthreads();
    }
    // box minimum over what is left: the predicates of the input set
    double part = 0.0, pmag = 0.0;
    for (int64_t j = tid; j < P_first; j += 256) {
        const int64_t col = qcol_idx[qcol_off[q] + j];
        const double t = fmin(rp[j] * pl[col], rp[j] * pu[col]);
        part += t;
        pmag += fabs(t);
    }
    red[tid] = part;
    redm[tid] = pmag;
    __syncthreads();
    for (int o = 128; o; o >>= 1) {
        if (tid < o) { red[tid] += red[tid + o]; redm[tid] += redm[tid + o]; }
        __syncthreads();
    }
    if (tid == 0) {
        bound[p] = konst + red[0];
        bound[gridDim.x + p] = kmag + redm[0];
    }
}

// ---------------------------------------------------------------------------
// Witness search: a point of the output set inside a halfspace proves the
// intersection non-empty.  Every point of an approx-star set is reached by
// picking the input predicates in their box and, neuron by neuron, a value of
// each new predicate between the lower envelope max(0,x) and the chord
// a*(x-l) of the triangle relaxation (PosLin.m:716-735); the greedy choice
// takes whichever end lowers the halfspace row, judged by the sign of the
// predicate's coefficient r.

// x0 for ImageStar(lb,ub) queries: entry i sits at lb or ub according to the
// sign of the coefficient of its predicate.  One block per pair.
__global__ void __launch_bounds__(256)
witness_x0_bounds_kernel(const int32_t* __restrict__ pair_q, int64_t N, int64_t ld,
                         const double* __restrict__ lbub, const double* __restrict__ r,
                         const int64_t* __restrict__ r_off, double* __restrict__ X) {
    const int p = blockIdx.x;
    const int q = pair_q[p];
    const double* lb = lbub + int64_t(q) * 2 * N;
    const double* ub = lb + N;
    const double* rp = r + r_off[p];
    __shared__ int warp_cnt[8];
    __shared__ int64_t running;
    if (threadIdx.x == 0) running = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t base = 0; base < N; base += blockDim.x) {
        const int64_t i = base + threadIdx.x;
        double l = 0.0, u = 0.0;
        bool has = false;
        if (i < N) {
            l = lb[i];
            u = ub[i];
            has = (0.5 * (u - l) != 0.0) || N == 1;
        }
        const unsigned bal = __ballot_sync(0xffffffffu, has);
        if (lane == 0) warp_cnt[warp] = __popc(bal);
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < 8; ++w) {
            if (w < warp) before += warp_cnt[w];
            total += warp_cnt[w];
        }
        if (i < N) {
            double x = 0.5 * (l + u);
            if (has) {
                const int64_t pos = running + before + __popc(bal & ((1u << lane) - 1u));
                const double hw = 0.5 * (u - l);
                x = rp[pos] > 0.0 ? x - hw : x + hw;       // predicate at -1 or +1
            }
            X[int64_t(p) * ld + i] = x;
        }
        __syncthreads();
        if (threadIdx.x == 0) running += total;
        __syncthreads();
    }
}

// x0 for general star queries: x0 = c + sum_j alpha_j G0_j with alpha_j = pl_j if
// r_j > 0 else pu_j.  V0 is the uploaded input matrix (centres first, then each
// query's generators from column gen0[q]).  grid = (pairs, row blocks).
__global__ void __launch_bounds__(256)
witness_x0_star_kernel(const int32_t* __restrict__ pair_q, int64_t N, int64_t ld, int64_t ld0,
                       const double* __restrict__ V0, const int64_t* __restrict__ gen0,
                       const double* __restrict__ pl0, const double* __restrict__ pu0,
                       const double* __restrict__ r, const int64_t* __restrict__ r_off,
                       const int64_t* __restrict__ pos0, int add_center, double* __restrict__ X) {
    const int p = blockIdx.x;
    const int q = pair_q[p];
    const int64_t i = int64_t(blockIdx.y) * blockDim.x + threadIdx.x;
    if (i >= N) return;
    const double* rp = r + r_off[p];
    const int64_t c0 = gen0[q], c1 = gen0[q + 1];
    double x = add_center ? V0[int64_t(q) * ld0 + i] : 0.0;
    for (int64_t col = c0; col < c1; ++col) {
        const double a = rp[pos0[col]] > 0.0 ? pl0[col] : pu0[col];
        x = fma(a, V0[col * ld0 + i], x);
    }
    X[int64_t(p) * ld + i] = x;
}

// relaxed ReLU on the witness points of one layer, in place.
__global__ void __launch_bounds__(256)
witness_relu_kernel(const int32_t* __restrict__ pair_q, int64_t N, int64_t ld, double* __restrict__ X,
                    const double* __restrict__ lb, const double* __restrict__ ub,
                    const int32_t* __restrict__ rank, const int64_t* __restrict__ P_in,
                    const double* __restrict__ r, const int64_t* __restrict__ r_off, double* __restrict__ alpha) {
    const int p = blockIdx.x;
    const int q = pair_q[p];
    const int64_t i = int64_t(blockIdx.y) * blockDim.x + threadIdx.x;
    if (i >= N) return;
    const double l = lb[int64_t(q) * N + i], u = ub[int64_t(q) * N + i];
    double* px = X + int64_t(p) * ld + i;
    const double x = *px;
    double y = x;
    if (u <= 0.0) {
        y = 0.0;
    } else if (l < 0.0) {
        const double lo = fmax(x, 0.0);
        const double rr = r[r_off[p] + P_in[q] + rank[int64_t(q) * N + i]];
        if (rr < 0.0) {
            const double a = u / (u - l);
            y = fmax(lo, a * x - a * l);
        } else {
            y = lo;
        }
        // the value of the neuron's new predicate at this point of the set
        if (alpha != nullptr) alpha[r_off[p] + P_in[q] + rank[int64_t(q) * N + i]] = y;
    }
    *px = y;
}

// ReLU of concrete points, in place: PosLin.evaluate (PosLin.m: max(x, 0)) on X [ld x n].
__global__ void __launch_bounds__(256)
relu_points_kernel(int64_t n, int64_t N, int64_t ld, double* __restrict__ X) {
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= N) return;
    for (int64_t p = blockIdx.y; p < n; p += gridDim.y) {
        double* px = X + p * ld + i;
        *px = fmax(*px, 0.0);
    }
}

// value[p] = G_p . x_p - g_p and a magnitude for the acceptance tolerance.
__global__ void witness_value_kernel(int n_pairs, int64_t Nout, int64_t ld, const double* __restrict__ X,
                                     const double* __restrict__ G, const double* __restrict__ g,
                                     double* __restrict__ value, double* __restrict__ scale) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= n_pairs) return;
    double v = 0.0, s = 0.0;
    for (int64_t o = 0; o < Nout; ++o) {
        const double t = G[int64_t(p) * Nout + o] * X[int64_t(p) * ld + o];
        v += t;
        s += fabs(t);
    }
    value[p] = v - g[p];
    scale[p] = s + fabs(g[p]);
}

}  // namespace

// Slices of a strip's candidate list (each its own block and chunk): enough blocks to fill the GPU.
// Strip height: at least 8 pixels (64 contiguous bytes per channel) where the block's rows allow it.
static int rw_strip_height(int H, int C) {
    const int cap = std::max(1, std::min(H, RW_THREADS * RW_RPT / std::max(1, C)));
    return std::min(cap, std::max(8, RW_THREADS / std::max(1, C)));
}

int range_windows_slices(int H, int W, int C, int nq, int sm_count) {
    const int TH = rw_strip_height(H, C);
    const int64_t blocks = ceil_div(H, TH) * int64_t(W) * nq;
    return (int)std::max<int64_t>(1, std::min<int64_t>(8, ceil_div(4 * int64_t(sm_count), blocks)));
}

size_t range_windows_scratch_ints(const WinCohorts& wc, int nq, int64_t ncols) {
    size_t bins = 0;
    for (int k = 0; k < wc.n; ++k) bins += size_t(nq) * (size_t(wc.c[k].KH) * wc.c[k].KW + 1);
    return 2 * bins + 2 * size_t(ncols) + 16;      // bins, cursors, unsorted and sorted columns
}

int launch_estimate_ranges(cudaStream_t st, const ReluWork& w, int64_t* launches) {
    if (w.n_chunks > 0) {
        if (w.N >= 2048) {
            dim3 grid((unsigned)w.n_chunks, (unsigned)ceil_div(ceil_div(w.N, 2), 256));
            range_partial_rows2_kernel<4><<<grid, 256, 0, st>>>(w.N, w.ld, w.V, w.qcol_idx, w.pl, w.pu,
                                                               w.chunk_beg, w.chunk_end, w.partial);
        } else {
            dim3 grid((unsigned)w.n_chunks, (unsigned)ceil_div(w.N, 32));
            range_partial_narrow_kernel<<<grid, 256, 0, st>>>(w.N, w.ld, w.V, w.qcol_idx, w.pl, w.pu,
                                                              w.chunk_beg, w.chunk_end, w.partial);
        }
        NNVB_CUDA(cudaGetLastError());
        if (launches) *launches += 1;
    }
    if (w.win.n > 0) {
        // the last win_slices chunks of every query (empty in the chunk list) take the windowed cohorts
        size_t n_bins = 0;
        int64_t max_n = 0, ncols = 0;
        for (int k = 0; k < w.win.n; ++k) {
            n_bins += size_t(w.nq) * (size_t(w.win.c[k].KH) * w.win.c[k].KW + 1);
            max_n = std::max(max_n, w.win.c[k].n);
            ncols = std::max(ncols, w.win.c[k].col0 + w.win.c[k].n);
        }
        int32_t* bins = w.win_scratch;
        int32_t* cursor = bins + n_bins;
        int32_t* tmp = cursor + n_bins;
        int32_t* perm = tmp + ncols;
        NNVB_CUDA(cudaMemsetAsync(bins, 0, sizeof(int32_t) * 2 * n_bins, st));
        dim3 gcol((unsigned)ceil_div(max_n, 256), (unsigned)w.win.n);
        win_hist_kernel<<<gcol, 256, 0, st>>>(w.win, w.nq, w.box, w.col_q, bins);
        win_scan_kernel<<<dim3((unsigned)w.nq, (unsigned)w.win.n), 256, 0, st>>>(w.win, bins);
        win_scatter_kernel<<<gcol, 256, 0, st>>>(w.win, w.nq, w.box, w.col_q, bins, cursor, w.win_seg, tmp);
        win_rank_kernel<<<gcol, 256, 0, st>>>(w.win, w.nq, w.box, w.col_q, bins, w.win_seg, tmp, perm);
        // strip height: a thread per (pixel, channel) where the channels allow it
        // the window-only copies hold a pixel's channels contiguously: short strips read them as well as long
        // ones and stage fewer candidates per block; a strip taller than the windows spends most of its
        // (row, candidate) pairs outside the candidate's window.  Measured on the 32x32x3 CNN (bound reduction of a
        // 128-image step): strips of 256 / C pixels (one row per thread) 8.8 ms, 128 / C (half the threads idle on
        // 32-channel layers) 9.3 ms, 512 / C 10.5 ms
        const int TH = w.win_pack != nullptr
                           ? std::min(rw_strip_height(w.img_h, w.img_c), std::max(4, 256 / std::max(1, w.img_c)))
                           : rw_strip_height(w.img_h, w.img_c);
        if (int64_t(TH) * w.img_c > int64_t(RW_THREADS) * RW_RPT) {
            set_error("range_windows: %d channels exceed the rows a block owns", w.img_c);
            return NNVB_E_UNSUPPORTED;
        }
        dim3 grid((unsigned)(ceil_div(w.img_h, TH) * w.img_w), (unsigned)w.nq, (unsigned)w.win_slices);
        if (w.win_pack != nullptr)
            range_windows_kernel<true><<<grid, RW_THREADS, 0, st>>>(w.N, w.ld, w.win_pack, w.pl, w.pu, w.box, w.img_h,
                                                                    w.img_w, w.img_c, TH, w.nq, w.win, bins, perm,
                                                                    w.win_seg, w.q_chunk_off, w.partial);
        else
            range_windows_kernel<false><<<grid, RW_THREADS, 0, st>>>(w.N, w.ld, w.V, w.pl, w.pu, w.box, w.img_h,
                                                                     w.img_w, w.img_c, TH, w.nq, w.win, bins, perm,
                                                                     w.win_seg, w.q_chunk_off, w.partial);
        NNVB_CUDA(cudaGetLastError());
        if (launches) *launches += 5;
    }
    return NNVB_OK;
}

int relu_blocks_per_query(int64_t N) { return (int)ceil_div(N, FIN_ROWS); }

int launch_reduce_chunks(cudaStream_t st, const ReluWork& w, double* sums, int64_t* launches) {
    const int nblk = relu_blocks_per_query(w.N);
    dim3 grid((unsigned)w.nq, (unsigned)nblk);
    reduce_chunks_kernel<<<grid, FIN_THREADS, 0, st>>>(w.N, w.q_chunk_off, w.partial, sums);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_classify_scan(cudaStream_t st, const ReluWork& w, const double* sums, int64_t* launches,
                         const PeerSums* peers) {
    const int nblk = relu_blocks_per_query(w.N);
    NNVB_CUDA(cudaMemsetAsync(w.q_dead, 0, sizeof(int64_t) * w.nq, st));
    dim3 grid((unsigned)w.nq, (unsigned)nblk);
    if (peers)
        classify_peers_kernel<<<grid, FIN_THREADS, 0, st>>>(w.N, w.ld, w.V, *peers, w.lb, w.ub, w.state, w.blk_cross,
                                                            reinterpret_cast<unsigned long long*>(w.q_dead), nblk);
    else if (sums)
        classify_sums_kernel<<<grid, FIN_THREADS, 0, st>>>(w.N, w.ld, w.V, sums, w.lb, w.ub, w.state, w.blk_cross,
                                                           reinterpret_cast<unsigned long long*>(w.q_dead), nblk);
    else
        range_finalize_kernel<<<grid, FIN_THREADS, 0, st>>>(w.N, w.ld, w.V, w.q_chunk_off, w.partial, w.lb,
                                                            w.ub, w.state, w.blk_cross,
                                                            reinterpret_cast<unsigned long long*>(w.q_dead), nblk);
    NNVB_CUDA(cudaGetLastError());
    scan_blocks_kernel<<<w.nq, 256, 0, st>>>(nblk, w.blk_cross, w.q_cross);
    NNVB_CUDA(cudaGetLastError());
    scan_queries_kernel<<<1, 1024, 0, st>>>(w.nq, w.q_cross, w.q_new_off);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 3;
    return NNVB_OK;
}

int launch_tighten_bounds(cudaStream_t st, int64_t k, int64_t N, const int32_t* idx, const double* xmin,
                          const double* xmax, double* lb_q, double* ub_q, int64_t* launches) {
    if (k <= 0) return NNVB_OK;
    tighten_bounds_kernel<<<(unsigned)ceil_div(k, 256), 256, 0, st>>>(k, N, idx, xmin, xmax, lb_q, ub_q);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_reclassify_scan(cudaStream_t st, const ReluWork& w, int64_t* launches) {
    const int nblk = relu_blocks_per_query(w.N);
    NNVB_CUDA(cudaMemsetAsync(w.q_dead, 0, sizeof(int64_t) * w.nq, st));
    dim3 grid((unsigned)w.nq, (unsigned)nblk);
    reclassify_kernel<<<grid, FIN_THREADS, 0, st>>>(w.N, w.lb, w.ub, w.state, w.blk_cross,
                                                    reinterpret_cast<unsigned long long*>(w.q_dead), nblk);
    NNVB_CUDA(cudaGetLastError());
    scan_blocks_kernel<<<w.nq, 256, 0, st>>>(nblk, w.blk_cross, w.q_cross);
    NNVB_CUDA(cudaGetLastError());
    scan_queries_kernel<<<1, 1024, 0, st>>>(w.nq, w.q_cross, w.q_new_off);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 3;
    return NNVB_OK;
}

int launch_gather_rows(cudaStream_t st, int64_t k, int64_t P, const int32_t* idx, const int32_t* qcol,
                       const int64_t* col_pos, const double* V, int64_t ld, double* out, int64_t* launches) {
    if (k <= 0 || P <= 0) return NNVB_OK;
    dim3 grid((unsigned)ceil_div(k, 128), (unsigned)std::min<int64_t>(P, 32768));
    gather_rows_kernel<<<grid, 128, 0, st>>>(k, P, idx, qcol, col_pos, V, ld, out);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_rank_cross(cudaStream_t st, const ReluWork& w, const ReluRecord& rec, int64_t* launches) {
    const int nblk = relu_blocks_per_query(w.N);
    dim3 grid((unsigned)w.nq, (unsigned)nblk);
    rank_cross_kernel<<<grid, FIN_THREADS, 0, st>>>(w.N, w.ld, w.V, w.state, w.lb, w.ub, w.blk_cross, nblk,
                                                    w.q_new_off, w.rank, rec.idx, rec.q, rec.c, rec.l, rec.u);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_relu_zero_rows(cudaStream_t st, const ReluWork& w, int64_t ncols, const int32_t* col_q,
                          const ReluRecord& rec, const int64_t* col_pos, int64_t* launches) {
    dim3 grid((unsigned)ceil_div(w.N, 256), (unsigned)std::min<int64_t>(ncols, 32768));
    zero_rows_kernel<<<grid, 256, 0, st>>>(w.nq, w.N, w.ld, w.V, ncols, col_q, w.state, w.rank, rec.G,
                                           rec.G_off, w.q_new_off, col_pos);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_relu_append(cudaStream_t st, const ReluWork& w, int64_t ncols_old, int64_t K_loc, int rank, int world,
                       bool materialize, const int64_t* P_in, const ReluRecord& rec, int32_t* col_q, double* pl, double* pu,
                       int64_t* col_pos, int img_h, int img_w, int4* box,
                       int64_t* new_qcol_off, int32_t* new_qcol_idx, int64_t* launches) {
    if (K_loc > 0) {
        if (materialize) NNVB_CUDA(cudaMemsetAsync(w.V + ncols_old * w.ld, 0, sizeof(double) * w.ld * K_loc, st));
        append_cols_kernel<<<(unsigned)ceil_div(K_loc, 256), 256, 0, st>>>(K_loc, rank, world, materialize ? 1 : 0,
                                                                          w.ld, w.V, ncols_old,
                                                                          rec.idx, rec.q, rec.u, w.q_new_off,
                                                                          w.qcol_off, P_in, col_q, pl, pu, col_pos, img_h,
                                                                          img_w, box);
        NNVB_CUDA(cudaGetLastError());
        if (launches) *launches += 1;
    }
    rebuild_lists_kernel<<<w.nq, 128, 0, st>>>(w.nq, rank, world, w.qcol_off, w.qcol_idx, w.q_new_off, ncols_old,
                                               new_qcol_off, new_qcol_idx);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_halfspace_pairs(cudaStream_t st, int n_pairs, const int32_t* pair_q, int64_t Nout, int64_t ld,
                           const double* V, const int64_t* qcol_off, const int32_t* qcol_idx, const double* pl,
                           const double* pu, const double* G, const double* g, double* margin, double* r_out,
                           const int64_t* r_off, const int64_t* col_pos, int add_center, double* part,
                           int64_t* launches) {
    if (n_pairs <= 0) return NNVB_OK;
    if (margin != nullptr && part == nullptr) {
        set_error("halfspace_pairs: margins need the partial-sum scratch");
        return NNVB_E_ARG;
    }
    dim3 grid((unsigned)n_pairs, HS_SPLIT);
    halfspace_pairs_kernel<<<grid, 256, 0, st>>>(pair_q, Nout, ld, V, qcol_off, qcol_idx, pl, pu, G, r_out, r_off,
                                                 col_pos, margin ? part : nullptr);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    if (margin) {
        halfspace_margin_kernel<<<(n_pairs + 127) / 128, 128, 0, st>>>(n_pairs, HS_SPLIT, pair_q, Nout, ld, V, G, g, part,
                                                                       margin, add_center);
        NNVB_CUDA(cudaGetLastError());
        if (launches) *launches += 1;
    }
    return NNVB_OK;
}

int launch_backsub(cudaStream_t st, const BacksubLayers& layers, int n_pairs, const int32_t* pair_q, int64_t Nout,
                   int64_t ld, const double* V, const double* G, const double* g, double* r, const int64_t* r_off,
                   const int64_t* qcol_off, const int32_t* qcol_idx, const double* pl, const double* pu, double* bound,
                   int64_t* launches) {
    if (n_pairs <= 0) return NNVB_OK;
    backsub_kernel<<<n_pairs, 256, 0, st>>>(layers, pair_q, Nout, ld, V, G, g, r, r_off, qcol_off, qcol_idx, pl, pu,
                                            bound);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_witness_x0_bounds(cudaStream_t st, int n_pairs, const int32_t* pair_q, int64_t N, int64_t ld,
                             const double* lbub, const double* r, const int64_t* r_off, double* X,
                             int64_t* launches) {
    witness_x0_bounds_kernel<<<n_pairs, 256, 0, st>>>(pair_q, N, ld, lbub, r, r_off, X);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_witness_x0_star(cudaStream_t st, int n_pairs, const int32_t* pair_q, int64_t N, int64_t ld, int64_t ld0,
                           const double* V0, const int64_t* gen0, const double* pl0, const double* pu0,
                           const double* r, const int64_t* r_off, const int64_t* pos0, int add_center, double* X,
                           int64_t* launches) {
    dim3 grid((unsigned)n_pairs, (unsigned)ceil_div(N, 256));
    witness_x0_star_kernel<<<grid, 256, 0, st>>>(pair_q, N, ld, ld0, V0, gen0, pl0, pu0, r, r_off, pos0, add_center, X);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_witness_relu(cudaStream_t st, int n_pairs, const int32_t* pair_q, int64_t N, int64_t ld, double* X,
                        const double* lb, const double* ub, const int32_t* rank, const int64_t* P_in,
                        const double* r, const int64_t* r_off, double* alpha, int64_t* launches) {
    dim3 grid((unsigned)n_pairs, (unsigned)ceil_div(N, 256));
    witness_relu_kernel<<<grid, 256, 0, st>>>(pair_q, N, ld, X, lb, ub, rank, P_in, r, r_off, alpha);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_relu_points(cudaStream_t st, int64_t n, int64_t N, int64_t ld, double* X, int64_t* launches) {
    dim3 grid((unsigned)ceil_div(N, 256), (unsigned)std::min<int64_t>(n, 65535));
    relu_points_kernel<<<grid, 256, 0, st>>>(n, N, ld, X);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_witness_value(cudaStream_t st, int n_pairs, int64_t Nout, int64_t ld, const double* X, const double* G,
                         const double* g, double* value, double* scale, int64_t* launches) {
    witness_value_kernel<<<(unsigned)ceil_div(n_pairs, 128), 128, 0, st>>>(n_pairs, Nout, ld, X, G, g, value, scale);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

}  // namespace nnvb
