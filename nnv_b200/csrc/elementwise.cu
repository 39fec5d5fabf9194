// Bandwidth-bound layer maps over every generator column: BatchNormalization
// (per-channel affine), AveragePooling2D, and construction of the dense input
// set ImageStar(lb, ub).
#include "common.cuh"

namespace nnvb {

namespace {

// BatchNormalizationLayer.reach_star_single_input, BatchNormalizationLayer.m:311-327:
// c -= mean; (c,G) = ((c,G).*1)/sqrt(var+eps); (c,G) .*= scale; c += offset.
// One thread per pair of rows, grid.y walks the columns.
__global__ void bn_f64_kernel(ChanAffine bn, int64_t plane, int64_t N, double* __restrict__ V,
                              int64_t ld, int64_t ncols, int64_t n_center) {
    const int64_t i = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) * 2;
    if (i >= N) return;
    const bool two = i + 1 < N;
    const int64_t c0 = i / plane;
    const int64_t c1 = two ? (i + 1) / plane : c0;
    const double den0 = bn.den[c0], den1 = bn.den[c1];
    const double sc0 = bn.scale[c0], sc1 = bn.scale[c1];
    const double mu0 = bn.mean[c0], mu1 = bn.mean[c1];
    const double of0 = bn.offset[c0], of1 = bn.offset[c1];
    for (int64_t j = blockIdx.y; j < ncols; j += gridDim.y) {
        double* p = V + j * ld + i;
        const bool is_center = j < n_center;
        if (two) {
            double2 v = *reinterpret_cast<double2*>(p);
            if (is_center) { v.x -= mu0; v.y -= mu1; }
            v.x = (v.x * 1.0) / den0;
            v.y = (v.y * 1.0) / den1;
            v.x *= sc0;
            v.y *= sc1;
            if (is_center) { v.x += of0; v.y += of1; }
            *reinterpret_cast<double2*>(p) = v;
        } else {
            double v = *p;
            if (is_center) v -= mu0;
            v = (v * 1.0) / den0;
            v *= sc0;
            if (is_center) v += of0;
            *p = v;
        }
    }
}

// AveragePooling2DLayer.evaluate, AveragePooling2DLayer.m:227-248 (semantics of compute_averageMap,
// :316-393): window sum in row-major order of the window, divided by ph*pw or, with g.clip, by the
// number of window entries inside the image (the two rules the reference's back ends use).
// One thread per output element of a column; grid.y walks the columns.
// Rows that the preceding ReLU step cleared are read as zero through `mask` (they were not zeroed in memory).
__global__ void avgpool_f64_kernel(PoolGeom g, RowMask mask, const int4* __restrict__ box,
                                   const double* __restrict__ Vin, int64_t ld_in,
                                   double* __restrict__ Vout, int64_t ld_out, int64_t ncols) {
    const int64_t o = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t n_out = int64_t(g.Ho) * g.Wo * g.C;
    if (o >= n_out) return;
    const int oh = int(o % g.Ho);
    const int ow = int((o / g.Ho) % g.Wo);
    const int c = int(o / (int64_t(g.Ho) * g.Wo));
    const int h0 = oh * g.sh - g.pad_t;
    const int w0 = ow * g.sw - g.pad_l;
    const double div = pool_divisor(g, h0, w0);
    const int64_t cbase = int64_t(c) * g.H * g.W;
    for (int64_t j = blockIdx.y; j < ncols; j += gridDim.y) {
        const double* src = Vin + j * ld_in + cbase;
        const uint8_t* st = (mask.state != nullptr && j < mask.ncols) ? mask.state + mask.col_q[j] * mask.N + cbase
                                                                      : nullptr;
        // entries outside the column's window count as zero whatever the memory holds there
        const int4 bx = box != nullptr ? box[j]
                                       : make_int4(NNVB_DENSE_ORIGIN, NNVB_DENSE_ORIGIN, NNVB_DENSE_EXTENT, NNVB_DENSE_EXTENT);
        double acc = 0.0;
        for (int a = 0; a < g.ph; ++a) {
            const int h = h0 + a;
            for (int b = 0; b < g.pw; ++b) {
                const int w = w0 + b;
                double v = 0.0;
                if (h >= 0 && h < g.H && w >= 0 && w < g.W && unsigned(h - bx.x) < unsigned(bx.z) &&
                    unsigned(w - bx.y) < unsigned(bx.w)) {
                    const int64_t o_in = h + int64_t(g.H) * w;
                    if (st == nullptr || st[o_in] == 0) v = src[o_in];
                }
                acc = acc + v;
            }
        }
        Vout[j * ld_out + o] = acc / div;
    }
}

// Average pooling of one-hot columns (unit vector of neuron (h,w,c)): 1/(ph*pw) at every output
// position of channel c whose window covers (h,w).  Every entry of the column's output window (all
// channels; origin and extent as update_windows_kernel derives them from a 1x1 input window) is written,
// zeros included; nothing outside it is touched.  One thread per (column, window entry).
__global__ void avgpool_onehot_kernel(PoolGeom g, HotCols hot, int64_t K_loc, double* __restrict__ Vout,
                                      int64_t ld_out) {
    const int wh = (g.ph - 1) / g.sh + 1, ww = (g.pw - 1) / g.sw + 1;
    const int per_col = wh * ww * g.C;
    const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= K_loc * per_col) return;
    const int64_t t = e / per_col;
    int r = int(e % per_col);
    const int cc = r % g.C;            // channel fastest: the writes of a column spread over its channel planes
    r /= g.C;
    const int ohl = r % wh, owl = r / wh;
    const int i = hot.idx[hot.first + t * hot.step];
    const double sc = hot.scale != nullptr ? hot.scale[t] : 1.0;
    const int h = i % g.H, w = (i / g.H) % g.W, c = i / (g.H * g.W);
    const int ah = h + g.pad_t - (g.ph - 1), aw = w + g.pad_l - (g.pw - 1);
    const int oh = (ah >= 0 ? (ah + g.sh - 1) / g.sh : -((-ah) / g.sh)) + ohl;
    const int ow = (aw >= 0 ? (aw + g.sw - 1) / g.sw : -((-aw) / g.sw)) + owl;
    if (oh < 0 || ow < 0 || oh >= g.Ho || ow >= g.Wo) return;
    const int h0 = oh * g.sh - g.pad_t, w0 = ow * g.sw - g.pad_l;
    const bool covers = cc == c && h >= h0 && h < h0 + g.ph && w >= w0 && w < w0 + g.pw;
    // same arithmetic as the dense kernel on this column: a sum of zeros and a single entry, then the division
    const double val = covers ? (0.0 + sc) / pool_divisor(g, h0, w0) : 0.0;
    Vout[t * ld_out + oh + int64_t(g.Ho) * (ow + int64_t(g.Wo) * cc)] = val;
}

// One-hot columns through a pooling layer whose windows tile the image: every neuron lies in exactly one
// window, so the pooled column is again a single entry.  Only the column's neuron and scale are rewritten.
__global__ void pool_onehot_track_kernel(PoolGeom g, HotCols hot, int64_t K_loc, int32_t* __restrict__ dst_idx,
                                         double* __restrict__ dst_scale) {
    const int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= K_loc) return;
    const int i = hot.idx[hot.first + t * hot.step];
    const double sc = hot.scale != nullptr ? hot.scale[t] : 1.0;
    const int h = i % g.H, w = (i / g.H) % g.W, c = i / (g.H * g.W);
    dst_idx[t] = h / g.sh + g.Ho * (w / g.sw + g.Wo * c);
    dst_scale[t] = (0.0 + sc) / double(g.ph * g.pw);
}

// Number of generators of ImageStar(lb,ub): entries with ub != lb (Box.m:36-43).
// One block per query.
__global__ void count_bounds_kernel(int64_t N, const double* __restrict__ lbub, int64_t* q_count) {
    const int q = blockIdx.x;
    const double* lb = lbub + int64_t(q) * 2 * N;
    const double* ub = lb + N;
    int cnt = 0;
    for (int64_t i = threadIdx.x; i < N; i += blockDim.x) cnt += (0.5 * (ub[i] - lb[i]) != 0.0 || N == 1) ? 1 : 0;
    __shared__ int s[32];
    for (int o = 16; o; o >>= 1) cnt += __shfl_down_sync(0xffffffffu, cnt, o);
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = cnt;
    __syncthreads();
    if (threadIdx.x < 32) {
        int v = threadIdx.x < (blockDim.x + 31) / 32 ? s[threadIdx.x] : 0;
        for (int o = 16; o; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
        if (threadIdx.x == 0) q_count[q] = v;
    }
}

// Fill centre and generator columns of ImageStar(lb,ub).  One block per query:
// centre = (lb+ub)/2; the r-th entry with nonzero half width gets generator
// column q_gen_off[q] + r holding that half width at its row (columns are zeroed
// beforehand).  Order of generators = ascending linear index, as diag() gives it.
__global__ void build_from_bounds_kernel(int nq, int rank, int world, int64_t N, int64_t ld,
                                         const double* __restrict__ lbub,
                                         const int64_t* __restrict__ q_gen_off, double* __restrict__ V,
                                         int32_t* __restrict__ col_q, double* __restrict__ pl,
                                         double* __restrict__ pu, int32_t* __restrict__ qcol_idx,
                                         int64_t* __restrict__ col_pos, int img_h, int img_w,
                                         int4* __restrict__ box, int32_t* __restrict__ hot_idx,
                                         double* __restrict__ hot_scale) {
    const int q = blockIdx.x;
    const double* lb = lbub + int64_t(q) * 2 * N;
    const double* ub = lb + N;
    const int64_t gen0 = q_gen_off[q];            // first generator column of this query (global index)
    const int64_t list0 = gen0 - nq;              // its position in qcol_idx (generators start at column nq)
    __shared__ int warp_cnt[32];
    __shared__ int64_t running;
    if (threadIdx.x == 0) running = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    for (int64_t base = 0; base < N; base += blockDim.x) {
        const int64_t i = base + threadIdx.x;
        double c = 0.0, hw = 0.0;
        bool has = false;
        if (i < N) {
            c = 0.5 * (lb[i] + ub[i]);
            hw = 0.5 * (ub[i] - lb[i]);
            has = hw != 0.0 || N == 1;
            V[int64_t(q) * ld + i] = c;
        }
        const unsigned bal = __ballot_sync(0xffffffffu, has);
        if (lane == 0) warp_cnt[warp] = __popc(bal);
        __syncthreads();
        int before = 0;
        for (int w = 0; w < warp; ++w) before += warp_cnt[w];
        int total = 0;
        for (int w = 0; w < nwarp; ++w) total += warp_cnt[w];
        const int64_t r = running + before + __popc(bal & ((1u << lane) - 1u));
        if (has && r % world == rank) {           // generator r of the query lives on rank r % world
            const int64_t t = r / world;
            const int64_t col = gen0 + t;
            if (hot_idx != nullptr) {             // the column stays implicit: half width times a unit vector
                hot_idx[col - nq] = int32_t(i);
                hot_scale[col - nq] = hw;
            } else {
                V[col * ld + i] = hw;
            }
            col_q[col] = q;
            pl[col] = -1.0;
            pu[col] = 1.0;
            qcol_idx[list0 + t] = int32_t(col);
            col_pos[col] = r;
            box[col] = make_int4(int(i % img_h), int((i / img_h) % img_w), 1, 1);   // non-zero at one pixel only
        }
        __syncthreads();
        if (threadIdx.x == 0) running += total;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        col_q[q] = q; pl[q] = 0.0; pu[q] = 0.0;
        box[q] = make_int4(NNVB_DENSE_ORIGIN, NNVB_DENSE_ORIGIN, NNVB_DENSE_EXTENT, NNVB_DENSE_EXTENT);
    }
}

}  // namespace

// Window origins after a convolution or pooling layer: an input window starting at h0 can reach outputs
// from ceil((h0 + pad - extent) / stride) on (extent = (k-1)*dilation).  One thread per column.
__global__ void update_windows_kernel(int64_t n, int4* __restrict__ box, int pad_t, int pad_l, int ext_h, int ext_w,
                                      int sh, int sw) {
    const int64_t j = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (j >= n) return;
    int4 bx = box[j];
    const int a = bx.x + pad_t - ext_h, b = bx.y + pad_l - ext_w;
    bx.x = a >= 0 ? (a + sh - 1) / sh : -((-a) / sh);
    bx.y = b >= 0 ? (b + sw - 1) / sw : -((-b) / sw);
    bx.z = (bx.z - 1 + ext_h) / sh + 1;
    bx.w = (bx.w - 1 + ext_w) / sw + 1;
    box[j] = bx;
}

__global__ void fill_dense_windows_kernel(int64_t n, int4* __restrict__ box) {
    const int64_t j = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (j < n) box[j] = make_int4(NNVB_DENSE_ORIGIN, NNVB_DENSE_ORIGIN, NNVB_DENSE_EXTENT, NNVB_DENSE_EXTENT);
}

// Windowed average pooling: a thread owns one (channel, patch position) and walks over the columns
// (blockIdx.y strided), so the index arithmetic is done once; same window sum as the dense kernel.
template <bool PAIRS>
__global__ void avgpool_windowed_kernel(PoolGeom g, RowMask mask, ColWindows win, int64_t col_base, int64_t ncols,
                                        const double* __restrict__ Vin, int64_t ld_in, double* __restrict__ Vout,
                                        int64_t ld_out, bool pad_rows) {
    const int per_col = win.wh * win.ww * g.C;
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= per_col) return;
    const int ohl = r % win.wh;
    const int r2 = r / win.wh;
    const int owl = r2 % win.ww;
    const int c = r2 / win.ww;
    const int64_t cbase = int64_t(c) * g.H * g.W;
    const int64_t obase = int64_t(g.Ho) * g.Wo * c;
    for (int64_t jj = blockIdx.y; jj < ncols; jj += gridDim.y) {
        const int64_t j = col_base + jj;
        const int4 bx = win.box[j];
        int oh, ow, h0, w0;
        if (PAIRS) {        // 2x2 windows, stride 2, no padding: the same origin formula with its constants folded
            const int a = bx.x - 1, b2 = bx.y - 1;
            oh = (a >= 0 ? (a + 1) >> 1 : -((-a) >> 1)) + ohl;
            ow = (b2 >= 0 ? (b2 + 1) >> 1 : -((-b2) >> 1)) + owl;
            h0 = 2 * oh;
            w0 = 2 * ow;
        } else {
            const int a = bx.x + g.pad_t - (g.ph - 1), b2 = bx.y + g.pad_l - (g.pw - 1);
            oh = (a >= 0 ? (a + g.sh - 1) / g.sh : -((-a) / g.sh)) + ohl;
            ow = (b2 >= 0 ? (b2 + g.sw - 1) / g.sw : -((-b2) / g.sw)) + owl;
            h0 = oh * g.sh - g.pad_t;
            w0 = ow * g.sw - g.pad_l;
        }
        if (oh < 0 || ow < 0 || oh >= g.Ho || ow >= g.Wo) continue;
        const double* src = Vin + j * ld_in + cbase;
        const uint8_t* st = (mask.state != nullptr && j < mask.ncols) ? mask.state + mask.col_q[j] * mask.N + cbase : nullptr;
        double acc = 0.0;
        if (PAIRS) {
            // 2x2 windows at stride 2 without padding on an even image height: the two rows of a window
            // column are one aligned 16-byte load (and one 2-byte load of their states); the four values
            // are added in the order of the general loop below
            double a[2][2];         // [row][column]
#pragma unroll
            for (int bb = 0; bb < 2; ++bb) {
                const int w = w0 + bb;
                a[0][bb] = 0.0;
                a[1][bb] = 0.0;
                if (w < g.W && unsigned(w - bx.y) < unsigned(bx.w)) {
                    const int64_t o_in = h0 + int64_t(g.H) * w;
                    const double2 v = *reinterpret_cast<const double2*>(src + o_in);
                    const unsigned s2 = st != nullptr ? *reinterpret_cast<const unsigned short*>(st + o_in) : 0u;
                    if (unsigned(h0 - bx.x) < unsigned(bx.z) && (s2 & 0xffu) == 0) a[0][bb] = v.x;
                    if (unsigned(h0 + 1 - bx.x) < unsigned(bx.z) && (s2 >> 8) == 0) a[1][bb] = v.y;
                }
            }
            acc = acc + a[0][0];
            acc = acc + a[0][1];
            acc = acc + a[1][0];
            acc = acc + a[1][1];
        } else {
            for (int aa = 0; aa < g.ph; ++aa) {
                const int h = h0 + aa;
                for (int bb = 0; bb < g.pw; ++bb) {
                    const int w = w0 + bb;
                    double v = 0.0;
                    if (h >= 0 && h < g.H && w >= 0 && w < g.W && unsigned(h - bx.x) < unsigned(bx.z) &&
                        unsigned(w - bx.y) < unsigned(bx.w)) {
                        const int64_t o_in = h + int64_t(g.H) * w;
                        if (st == nullptr || st[o_in] == 0) v = src[o_in];
                    }
                    acc = acc + v;
                }
            }
        }
        double* dst = Vout + j * ld_out + int64_t(g.Ho) * ow + obase;
        dst[oh] = PAIRS ? acc * 0.25 : acc / pool_divisor(g, h0, w0);       // a quotient by 4 is exact either way
        if (pad_rows) {
            // complete the 32-byte sectors at both ends of the window's run of rows with zeros (the dense
            // tensor is zero there): a partly written sector costs the memory system a read on top of the write
            const int first = oh - ohl;
            const int lo = max(first, 0), hi = min(first + win.wh, g.Ho);
            if (oh == lo)
                for (int r = lo & ~3; r < lo; ++r) dst[r] = 0.0;
            if (oh == hi - 1)
                for (int r = hi; r < ((hi + 3) & ~3); ++r) dst[r] = 0.0;
        }
    }
}

// 2x2 windows at stride 2 without padding, even image height: a thread owns two vertically adjacent outputs of
// one (patch column, channel), so the window, the pointers and the column tests of a column are worked out
// once for both.  Per output the same four values in the same order as avgpool_windowed_kernel.
__global__ void avgpool_windowed_2x2_kernel(PoolGeom g, RowMask mask, ColWindows win, int64_t col_base, int64_t ncols,
                                            const double* __restrict__ Vin, int64_t ld_in, double* __restrict__ Vout,
                                            int64_t ld_out, bool pad_rows) {
    const int slots = (win.wh + 1) / 2;
    const int per_col = slots * win.ww * g.C;
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= per_col) return;
    const int ohl = 2 * (r % slots);
    const int r2 = r / slots;
    const int owl = r2 % win.ww;
    const int c = r2 / win.ww;
    const int64_t cbase = int64_t(c) * g.H * g.W;
    const int64_t obase = int64_t(g.Ho) * g.Wo * c;
    const bool two = ohl + 1 < win.wh;
    for (int64_t jj = blockIdx.y; jj < ncols; jj += gridDim.y) {
        const int64_t j = col_base + jj;
        const int4 bx = win.box[j];
        const int a = bx.x - 1, b2 = bx.y - 1;
        const int first = a >= 0 ? (a + 1) >> 1 : -((-a) >> 1);         // first output row of the window
        const int ow = (b2 >= 0 ? (b2 + 1) >> 1 : -((-b2) >> 1)) + owl;
        const int oh0 = first + ohl;
        const bool ok0 = oh0 >= 0 && oh0 < g.Ho, ok1 = two && oh0 + 1 >= 0 && oh0 + 1 < g.Ho;
        if (ow < 0 || ow >= g.Wo || !(ok0 || ok1)) continue;
        const double* src = Vin + j * ld_in + cbase;
        const uint8_t* st = (mask.state != nullptr && j < mask.ncols) ? mask.state + mask.col_q[j] * mask.N + cbase : nullptr;
        const int w0 = 2 * ow;
        double v[2][2][2];          // [output][row][column]
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int h0 = 2 * (oh0 + k);
            const bool okk = k == 0 ? ok0 : ok1;
#pragma unroll
            for (int bb = 0; bb < 2; ++bb) {
                const int w = w0 + bb;
                v[k][0][bb] = 0.0;
                v[k][1][bb] = 0.0;
                if (okk && w < g.W && unsigned(w - bx.y) < unsigned(bx.w)) {
                    const int64_t o_in = h0 + int64_t(g.H) * w;
                    const double2 x = *reinterpret_cast<const double2*>(src + o_in);
                    const unsigned s2 = st != nullptr ? *reinterpret_cast<const unsigned short*>(st + o_in) : 0u;
                    if (unsigned(h0 - bx.x) < unsigned(bx.z) && (s2 & 0xffu) == 0) v[k][0][bb] = x.x;
                    if (unsigned(h0 + 1 - bx.x) < unsigned(bx.z) && (s2 >> 8) == 0) v[k][1][bb] = x.y;
                }
            }
        }
        double* dst = Vout + j * ld_out + int64_t(g.Ho) * ow + obase;
        const int lo = max(first, 0), hi = min(first + win.wh, g.Ho);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            if (!(k == 0 ? ok0 : ok1)) continue;
            const int oh = oh0 + k;
            double acc = 0.0;
            acc = acc + v[k][0][0];
            acc = acc + v[k][0][1];
            acc = acc + v[k][1][0];
            acc = acc + v[k][1][1];
            dst[oh] = acc * 0.25;           // the quotient by 4, exactly
            if (pad_rows) {                 // whole sectors at both ends of the window's run of rows
                if (oh == lo)
                    for (int rr = lo & ~3; rr < lo; ++rr) dst[rr] = 0.0;
                if (oh == hi - 1)
                    for (int rr = hi; rr < ((hi + 3) & ~3); ++rr) dst[rr] = 0.0;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// Compact storage of windowed columns.  Column j of a cohort [col0, col0+n) whose columns are zero outside a
// wh x ww window is kept as its window only, channel fastest: entry (h, w, c) at
//     base + (j - col0)*stride + ((w - w0_j)*wh + (h - h0_j))*C + c,     (h0_j, w0_j) = box[j].xy.
// A pixel's channels are contiguous (256-512 bytes for 32-64 channels), so readers and writers move whole
// sectors.  Entries of a window that hang over the image border are never read (every reader tests the
// image bounds), so writers may leave anything there.

// Average pooling, compact -> compact.  A thread owns one (output window position, channel), channel fastest, and
// walks over the columns (blockIdx.y strided), so the index arithmetic is done once.  Same window sum, in the same
// order, and the same divisor as avgpool_f64_kernel.  mask.state_cf: the row states in channel-fastest order, so that
// the lanes of a warp (neighbouring channels of one pixel) read neighbouring bytes.
__global__ void __launch_bounds__(256)
avgpool_compact_kernel(PoolGeom g, RowMask mask, const int4* __restrict__ box, int64_t col_base, int64_t ncols,
                       int wh_in, int ww_in, int wh_out, int ww_out, const double* __restrict__ Cin_, int64_t stride_in,
                       double* __restrict__ Cout_, int64_t stride_out) {
    const int per_col = wh_out * ww_out * g.C;
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= per_col) return;
    const int c = r % g.C;
    const int pos = r / g.C;
    const int ohl = pos % wh_out, owl = pos / wh_out;
    const int64_t plane = int64_t(g.H) * g.W;
    for (int64_t jj = blockIdx.y; jj < ncols; jj += gridDim.y) {
        const int64_t j = col_base + jj;
        const int4 bx = box[j];
        const int a0 = bx.x + g.pad_t - (g.ph - 1), b0 = bx.y + g.pad_l - (g.pw - 1);
        const int oh = (a0 >= 0 ? (a0 + g.sh - 1) / g.sh : -((-a0) / g.sh)) + ohl;
        const int ow = (b0 >= 0 ? (b0 + g.sw - 1) / g.sw : -((-b0) / g.sw)) + owl;
        double out = 0.0;
        if (oh >= 0 && ow >= 0 && oh < g.Ho && ow < g.Wo) {
            const int h0 = oh * g.sh - g.pad_t, w0 = ow * g.sw - g.pad_l;
            const double* src = Cin_ + jj * stride_in + c;
            const bool masked = mask.state != nullptr && j < mask.ncols;
            const uint8_t* st = masked ? (mask.state_cf != nullptr ? mask.state_cf + mask.col_q[j] * mask.N + c
                                                                  : mask.state + mask.col_q[j] * mask.N + c * plane)
                                       : nullptr;
            const bool cf = mask.state_cf != nullptr;
            double acc = 0.0;
            for (int a = 0; a < g.ph; ++a) {
                const int h = h0 + a;
                for (int b = 0; b < g.pw; ++b) {
                    const int w = w0 + b;
                    double v = 0.0;
                    if (h >= 0 && h < g.H && w >= 0 && w < g.W && unsigned(h - bx.x) < unsigned(wh_in) &&
                        unsigned(w - bx.y) < unsigned(ww_in)) {
                        const int64_t pix = h + int64_t(g.H) * w;
                        if (st == nullptr || st[cf ? pix * g.C : pix] == 0)
                            v = src[int64_t((w - bx.y) * wh_in + (h - bx.x)) * g.C];
                    }
                    acc = acc + v;
                }
            }
            out = acc / pool_divisor(g, h0, w0);
        }
        Cout_[jj * stride_out + r] = out;
    }
}

// The same for 2x2 windows at stride 2 without padding and an even channel count: a thread owns two neighbouring
// channels of one output position (16-byte loads and stores, the two row states as one 2-byte load), the window
// origin comes from shifts, and the four loads of a window are issued together.  Per output the same four values
// in the same order as the general kernel; the quotient by 4 is exact.
__global__ void __launch_bounds__(256)
avgpool_compact_2x2_kernel(PoolGeom g, RowMask mask, const int4* __restrict__ box, int64_t col_base, int64_t ncols,
                           int wh_in, int ww_in, int wh_out, int ww_out, const double* __restrict__ Cin_,
                           int64_t stride_in, double* __restrict__ Cout_, int64_t stride_out) {
    const int C2 = g.C / 2;
    const int per_col = wh_out * ww_out * C2;
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= per_col) return;
    const int c = 2 * (r % C2);
    const int pos = r / C2;
    const int ohl = pos % wh_out, owl = pos / wh_out;
    const bool cf = mask.state_cf != nullptr;
    const int64_t plane = int64_t(g.H) * g.W;
    // the window box and the query of the NEXT column are requested while this column is summed: they head the
    // dependent chain box -> addresses -> values, which otherwise costs a memory round trip per column
    int4 bx_n = make_int4(0, 0, 0, 0);
    int q_n = 0;
    if (int64_t(blockIdx.y) < ncols) {
        bx_n = box[col_base + blockIdx.y];
        if (mask.state != nullptr && col_base + blockIdx.y < mask.ncols) q_n = mask.col_q[col_base + blockIdx.y];
    }
    for (int64_t jj = blockIdx.y; jj < ncols; jj += gridDim.y) {
        const int64_t j = col_base + jj;
        const int4 bx = bx_n;
        const int q_j = q_n;
        if (jj + gridDim.y < ncols) {
            bx_n = box[j + gridDim.y];
            if (mask.state != nullptr && j + gridDim.y < mask.ncols) q_n = mask.col_q[j + gridDim.y];
        }
        const int a = bx.x - 1, b2 = bx.y - 1;
        const int oh = (a >= 0 ? (a + 1) >> 1 : -((-a) >> 1)) + ohl;
        const int ow = (b2 >= 0 ? (b2 + 1) >> 1 : -((-b2) >> 1)) + owl;
        double2 out = make_double2(0.0, 0.0);
        if (oh >= 0 && ow >= 0 && oh < g.Ho && ow < g.Wo) {
            const int h0 = 2 * oh, w0 = 2 * ow;
            const double* src = Cin_ + jj * stride_in + c;
            const bool masked = mask.state != nullptr && j < mask.ncols;
            const uint8_t* st = masked ? (cf ? mask.state_cf + q_j * mask.N + c
                                             : mask.state + q_j * mask.N + c * plane) : nullptr;
            double2 v[4];
            unsigned sbits[4];
            bool in[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int h = h0 + (k >> 1), w = w0 + (k & 1);
                in[k] = h < g.H && w < g.W && unsigned(h - bx.x) < unsigned(wh_in) && unsigned(w - bx.y) < unsigned(ww_in);
                v[k] = make_double2(0.0, 0.0);
                sbits[k] = 0u;
                if (in[k]) {
                    const int64_t pix = h + int64_t(g.H) * w;
                    if (st != nullptr)
                        sbits[k] = cf ? unsigned(*reinterpret_cast<const unsigned short*>(st + pix * g.C))
                                      : (unsigned(st[pix]) | (unsigned(st[pix + plane]) << 8));
                    v[k] = *reinterpret_cast<const double2*>(src + int64_t((w - bx.y) * wh_in + (h - bx.x)) * g.C);
                }
            }
            double a0 = 0.0, a1 = 0.0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                a0 = a0 + ((sbits[k] & 0xffu) == 0 ? v[k].x : 0.0);
                a1 = a1 + ((sbits[k] >> 8) == 0 ? v[k].y : 0.0);
            }
            out = make_double2(a0 * 0.25, a1 * 0.25);
        }
        *reinterpret_cast<double2*>(Cout_ + jj * stride_out + int64_t(pos) * g.C + c) = out;
    }
}

// Row states in channel-fastest order: cf[q][(w*H + h)*C + c] = state[q][h + H*(w + W*c)].
__global__ void __launch_bounds__(256)
state_channel_fastest_kernel(int nq, int H, int W, int C, const uint8_t* __restrict__ state, uint8_t* __restrict__ cf) {
    const int64_t N = int64_t(H) * W * C;
    const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= N * nq) return;
    const int64_t q = e / N, i = e % N;
    const int c = int(i % C);
    const int64_t pix = i / C;
    cf[e] = state[q * N + pix + int64_t(H) * W * c];
}

// Compact -> full-length columns: scatter of the in-image window entries.
__global__ void __launch_bounds__(256)
expand_compact_kernel(int H, int W, int C, const int4* __restrict__ box, int64_t col0, int64_t n, int wh, int ww,
                      const double* __restrict__ comp, int64_t stride, double* __restrict__ V, int64_t ld) {
    const int per_col = wh * ww * C;
    const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= n * per_col) return;
    const int64_t jj = e / per_col;
    int r = int(e % per_col);
    const int c = r % C;
    r /= C;
    const int hl = r % wh, wl = r / wh;
    const int4 bx = box[col0 + jj];
    const int h = bx.x + hl, w = bx.y + wl;
    if (h < 0 || h >= H || w < 0 || w >= W) return;
    V[(col0 + jj) * ld + h + int64_t(H) * (w + int64_t(W) * c)] = comp[jj * stride + e % per_col];
}

int launch_avgpool_compact(cudaStream_t st, const PoolGeom& g, const RowMask& mask, const int4* box, int64_t col_base,
                           int64_t ncols, int wh_in, int ww_in, int wh_out, int ww_out, const double* comp_in,
                           int64_t stride_in, double* comp_out, int64_t stride_out, int64_t* launches) {
    if (ncols <= 0) return NNVB_OK;
    const bool pairs = g.ph == 2 && g.pw == 2 && g.sh == 2 && g.sw == 2 && g.pad_t == 0 && g.pad_l == 0 && g.C % 2 == 0 &&
                       stride_in % 2 == 0 && stride_out % 2 == 0 && (reinterpret_cast<uintptr_t>(comp_in) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(comp_out) & 15) == 0 &&
                       (mask.state_cf == nullptr || mask.N % 2 == 0);
    static const bool one_row = getenv("NNVB_POOL_ONE_ROW") != nullptr;
    if (pairs && !one_row) {
        const int per2 = wh_out * ww_out * (g.C / 2);
        const int th2 = per2 >= 256 ? 256 : 128;
        dim3 grid2((unsigned)ceil_div(per2, th2), (unsigned)std::min<int64_t>(ncols, 65535));
        avgpool_compact_2x2_kernel<<<grid2, th2, 0, st>>>(g, mask, box, col_base, ncols, wh_in, ww_in, wh_out, ww_out,
                                                          comp_in, stride_in, comp_out, stride_out);
        NNVB_CUDA(cudaGetLastError());
        if (launches) *launches += 1;
        return NNVB_OK;
    }
    const int per_col = wh_out * ww_out * g.C;
    const int threads = per_col >= 256 ? 256 : 128;
    dim3 grid((unsigned)ceil_div(per_col, threads), (unsigned)std::min<int64_t>(ncols, 65535));
    avgpool_compact_kernel<<<grid, threads, 0, st>>>(g, mask, box, col_base, ncols, wh_in, ww_in, wh_out, ww_out, comp_in,
                                                     stride_in, comp_out, stride_out);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_state_channel_fastest(cudaStream_t st, int nq, int H, int W, int C, const uint8_t* state, uint8_t* cf,
                                 int64_t* launches) {
    const int64_t total = int64_t(nq) * H * W * C;
    if (total <= 0) return NNVB_OK;
    state_channel_fastest_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, st>>>(nq, H, W, C, state, cf);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_expand_compact(cudaStream_t st, int H, int W, int C, const int4* box, int64_t col0, int64_t n, int wh, int ww,
                          const double* comp, int64_t stride, double* V, int64_t ld, bool clear, int64_t* launches) {
    if (n <= 0) return NNVB_OK;
    if (clear) NNVB_CUDA(cudaMemsetAsync(V + col0 * ld, 0, sizeof(double) * ld * n, st));
    const int64_t total = n * wh * ww * C;
    expand_compact_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, st>>>(H, W, C, box, col0, n, wh, ww, comp, stride, V, ld);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_avgpool_windowed(cudaStream_t st, const PoolGeom& g, const RowMask& mask, const ColWindows& win,
                            int64_t col_base, const double* Vin, int64_t ld_in, double* Vout, int64_t ld_out,
                            int64_t ncols, int64_t* launches) {
    if (ncols <= 0) return NNVB_OK;
    const int per_col = win.wh * win.ww * g.C;
    const int threads = per_col >= 256 ? 256 : 128;
    dim3 grid((unsigned)ceil_div(per_col, threads), (unsigned)std::min<int64_t>(ncols, 8192));
    // the state array of a query starts at q*N: N even keeps the 2-byte state loads aligned
    const bool pairs = g.ph == 2 && g.pw == 2 && g.sh == 2 && g.sw == 2 && g.pad_t == 0 && g.pad_l == 0 &&
                       g.H % 2 == 0 && ld_in % 2 == 0 && (mask.state == nullptr || mask.N % 2 == 0);
    const bool pad_rows = g.Ho % 4 == 0 && ld_out % 4 == 0;      // image columns start on sector boundaries
    static const bool one_row = getenv("NNVB_POOL_ONE_ROW") != nullptr;
    if (pairs && !one_row) {
        const int per2 = (win.wh + 1) / 2 * win.ww * g.C;
        const int th2 = per2 >= 256 ? 256 : 128;
        dim3 grid2((unsigned)ceil_div(per2, th2), (unsigned)std::min<int64_t>(ncols, 8192));
        avgpool_windowed_2x2_kernel<<<grid2, th2, 0, st>>>(g, mask, win, col_base, ncols, Vin, ld_in, Vout, ld_out, pad_rows);
    } else if (pairs)
        avgpool_windowed_kernel<true><<<grid, threads, 0, st>>>(g, mask, win, col_base, ncols, Vin, ld_in, Vout, ld_out,
                                                                pad_rows);
    else
        avgpool_windowed_kernel<false><<<grid, threads, 0, st>>>(g, mask, win, col_base, ncols, Vin, ld_in, Vout, ld_out,
                                                                 pad_rows);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

// Zero outside the windows: thread per pair of rows, blockIdx.y strides over the columns.
__global__ void zero_outside_windows_kernel(int H, int W, int C, const int4* __restrict__ box, int64_t col0, int64_t n,
                                            double* __restrict__ V, int64_t ld) {
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t N = int64_t(H) * W * C;
    if (i >= N) return;
    const int o = int(i % (int64_t(H) * W));
    const int h = o % H, w = o / H;
    for (int64_t j = blockIdx.y; j < n; j += gridDim.y) {
        const int4 bx = box[col0 + j];
        const bool inside = unsigned(h - bx.x) < unsigned(bx.z) && unsigned(w - bx.y) < unsigned(bx.w);
        if (!inside) V[(col0 + j) * ld + i] = 0.0;
    }
}

int launch_zero_outside_windows(cudaStream_t st, int H, int W, int C, const int4* box, int64_t col0, int64_t n,
                                double* V, int64_t ld, int64_t* launches) {
    if (n <= 0) return NNVB_OK;
    const int64_t N = int64_t(H) * W * C;
    dim3 grid((unsigned)ceil_div(N, 256), (unsigned)std::min<int64_t>(n, 16384));
    zero_outside_windows_kernel<<<grid, 256, 0, st>>>(H, W, C, box, col0, n, V, ld);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_fill_dense_windows(cudaStream_t st, int64_t n, int4* box, int64_t* launches) {
    if (n <= 0) return NNVB_OK;
    fill_dense_windows_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, st>>>(n, box);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_update_windows(cudaStream_t st, int64_t n, int4* box, int pad_t, int pad_l, int ext_h,
                          int ext_w, int sh, int sw, int64_t* launches) {
    if (n <= 0) return NNVB_OK;
    update_windows_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, st>>>(n, box, pad_t, pad_l, ext_h, ext_w, sh, sw);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_bn_f64(cudaStream_t st, const ChanAffine& bn, int64_t plane, int64_t N, double* V,
                  int64_t ld, int64_t ncols, int64_t n_center, int64_t* launches) {
    if (ncols <= 0) return NNVB_OK;
    const int threads = 128;
    dim3 grid((unsigned)ceil_div(ceil_div(N, 2), threads), (unsigned)std::min<int64_t>(ncols, 65535));
    bn_f64_kernel<<<grid, threads, 0, st>>>(bn, plane, N, V, ld, ncols, n_center);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

bool pool_keeps_onehot(const PoolGeom& g) {
    return g.ph == g.sh && g.pw == g.sw && g.pad_t == 0 && g.pad_l == 0 && g.H == g.Ho * g.sh && g.W == g.Wo * g.sw;
}

int launch_pool_onehot_track(cudaStream_t st, const PoolGeom& g, const HotCols& hot, int64_t K_loc, int32_t* dst_idx,
                             double* dst_scale, int64_t* launches) {
    if (K_loc <= 0) return NNVB_OK;
    pool_onehot_track_kernel<<<(unsigned)ceil_div(K_loc, 256), 256, 0, st>>>(g, hot, K_loc, dst_idx, dst_scale);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_avgpool_onehot(cudaStream_t st, const PoolGeom& g, const HotCols& hot, int64_t K_loc, double* Vout,
                          int64_t ld_out, bool zero_fill, int64_t* launches) {
    if (K_loc <= 0) return NNVB_OK;
    if (zero_fill) NNVB_CUDA(cudaMemsetAsync(Vout, 0, sizeof(double) * ld_out * K_loc, st));
    const int64_t per_col = int64_t((g.ph - 1) / g.sh + 1) * ((g.pw - 1) / g.sw + 1) * g.C;
    avgpool_onehot_kernel<<<(unsigned)ceil_div(K_loc * per_col, 256), 256, 0, st>>>(g, hot, K_loc, Vout, ld_out);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_avgpool_f64(cudaStream_t st, const PoolGeom& g, const RowMask& mask, const int4* box, const double* Vin,
                       int64_t ld_in, double* Vout, int64_t ld_out, int64_t ncols, int64_t* launches) {
    if (ncols <= 0) return NNVB_OK;
    const int threads = 256;
    const int64_t n_out = int64_t(g.Ho) * g.Wo * g.C;
    dim3 grid((unsigned)ceil_div(n_out, threads), (unsigned)std::min<int64_t>(ncols, 65535));
    avgpool_f64_kernel<<<grid, threads, 0, st>>>(g, mask, box, Vin, ld_in, Vout, ld_out, ncols);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_count_bounds(cudaStream_t st, int nq, int64_t N, const double* lbub, int64_t* q_count,
                        int64_t* launches) {
    count_bounds_kernel<<<nq, 256, 0, st>>>(N, lbub, q_count);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

int launch_build_from_bounds(cudaStream_t st, int nq, int64_t N, int64_t ld, const double* lbub,
                             const int64_t* q_gen_off, int rank, int world, double* V, int32_t* col_q, double* pl,
                             double* pu, int32_t* qcol_idx, int64_t* col_pos, int img_h, int img_w, int4* box,
                             int32_t* hot_idx, double* hot_scale, int64_t* launches) {
    build_from_bounds_kernel<<<nq, 256, 0, st>>>(nq, rank, world, N, ld, lbub, q_gen_off, V, col_q, pl, pu, qcol_idx,
                                                 col_pos, img_h, img_w, box, hot_idx, hot_scale);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

}  // namespace nnvb
