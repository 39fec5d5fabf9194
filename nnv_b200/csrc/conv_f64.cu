// Conv2D layer over every generator slice at once as an implicit GEMM:
//   out(oh,ow,co,j) = sum_{kh,kw,ci} in(oh*sh - pt + kh*dh, ow*sw - pl + kw*dw, ci, j) * W(kh,kw,ci,co)
// bias on the centre slices only (Conv2DLayer.reach_star_single_input,
// Conv2DLayer.m:591-596; arithmetic of compute_featureMap, :1180-1197).
// An optional per-channel affine (the BatchNormalization layer that follows,
// BatchNormalizationLayer.m:311-327) is applied in the epilogue in the
// reference's operation order.
//
// Dense FP64 contraction on the DMMA tensor path:
//   M = output positions of a tile (TH x TW patch of NJ generator columns),
//   N = output channels (BN_TILE per CTA), K = taps x input channels.
// Per K chunk of KC = 8 input channels a stage holds
//   - the input halo of the tile, [KC][NJ][HW][HH] with h fastest (the set's own
//     layout, so global reads run along h), fetched with 8-byte cp.async and
//     zero-filled outside the image;
//   - the weights of the chunk, [tap][KC][CS], one contiguous pre-arranged block.
// The per-channel halo stride PS and the channel stride CS are = 4 (mod 8)
// doubles, which makes the A and B fragment reads bank-conflict free for
// stride-1 convolutions.  Every tap reuses the staged halo, so global traffic
// is that of the input itself, not of an im2col matrix.
#include "common.cuh"
#include "mma_f64.cuh"

#include <algorithm>
#include <cstdlib>
#include <vector>

namespace nnvb {

namespace {

constexpr int KC = 8;   // input channels per K chunk

struct ConvParams {
    ConvGeom g;
    int TH, TW, NJ;        // output tile: TH x TW positions of NJ columns
    int HH, HW;            // halo height / width
    int plane;             // NJ * HH * HW
    int PS;                // per-channel halo stride (doubles), = 4 mod 8
    int CS;                // weight channel stride (doubles)
    int n_th, n_tw;        // spatial tiles per image
    int n_chunks;
    int taps;
    int halo_stage;        // doubles
    int w_stage;           // doubles
    int64_t col_groups;    // ceil(ncols / NJ)
};

template <int WM_TILES, int WN_TILES, int WARPS_M, int WARPS_N, int STAGES, int MIN_BLOCKS>
__global__ void __launch_bounds__(WARPS_M* WARPS_N * 32, MIN_BLOCKS)
conv_f64_kernel(const ConvParams p, const double* __restrict__ Wg, const double* __restrict__ bias,
                const ChanAffine bn, const RowMask mask, const ColWindows win, int64_t col_base,
                const double* __restrict__ Vin, int64_t ld_in, double* __restrict__ Vout, int64_t ld_out,
                int64_t ncols, int64_t n_center) {
    constexpr int BN = WARPS_N * WN_TILES * 8;
    constexpr int THREADS = WARPS_M * WARPS_N * 32;
    constexpr int NWARPS = WARPS_M * WARPS_N;

    extern __shared__ __align__(16) double smem[];
    double* halo = smem;                                  // [STAGES][halo_stage]
    double* wts = smem + STAGES * p.halo_stage;           // [STAGES][w_stage]
    double* chan = wts + STAGES * p.w_stage;              // [5][BN]: bias, mean, 1/den, scale, offset
    int* gtab = reinterpret_cast<int*>(chan + 5 * BN);    // [plane]
    int* mtab = gtab + p.plane;                           // [plane] row-state offset, -1 = column not masked

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int wm = warp % WARPS_M;
    const int wn = warp / WARPS_M;
    const int g = lane >> 2;
    const int t = lane & 3;

    // tile coordinates: spatial tiles fastest, then column groups
    const int sp_tiles = p.n_th * p.n_tw;
    const int64_t cg = blockIdx.x / sp_tiles;
    const int sp = int(blockIdx.x % sp_tiles);
    const int oh0 = (sp % p.n_th) * p.TH;
    const int ow0 = (sp / p.n_th) * p.TW;
    const int64_t j0 = cg * p.NJ;
    const int n_tile = blockIdx.y;
    const int n0 = n_tile * BN;

    const int H = p.g.H, W = p.g.W;
    const int hw_in = H * W;

    // Origin of each column's output patch.  Dense columns: the spatial tile.  Windowed columns: every
    // column is zero outside a small window [h0, h0+wh) x [w0, w0+ww) of the input; the outputs that
    // can be non-zero form a TH x TW patch starting at ceil((h0 + pad - (k-1)*dil) / stride), and only
    // that patch is computed and written; the rest of the output column is left as it is.
    __shared__ int org_h[128], org_w[128];
    __shared__ int4 in_box[128];
    if (tid < p.NJ) {
        int a = oh0, b2 = ow0;
        int4 bx = make_int4(NNVB_DENSE_ORIGIN, NNVB_DENSE_ORIGIN, NNVB_DENSE_EXTENT, NNVB_DENSE_EXTENT);
        if (win.box != nullptr && j0 + tid < ncols) bx = win.box[col_base + j0 + tid];
        in_box[tid] = bx;
        if (win.wh > 0 && j0 + tid < ncols) {
            const int ah = bx.x + p.g.pad_t - (p.g.kh - 1) * p.g.dh;
            const int aw = bx.y + p.g.pad_l - (p.g.kw - 1) * p.g.dw;
            a = ah >= 0 ? (ah + p.g.sh - 1) / p.g.sh : -((-ah) / p.g.sh);
            b2 = aw >= 0 ? (aw + p.g.sw - 1) / p.g.sw : -((-aw) / p.g.sw);
        }
        org_h[tid] = a;
        org_w[tid] = b2;
    }
    __syncthreads();

    // table: halo element r -> offset in the input relative to column j0, channel 0
    for (int r = tid; r < p.plane; r += THREADS) {
        const int jl = r / (p.HH * p.HW);
        const int r2 = r - jl * (p.HH * p.HW);
        const int wl = r2 / p.HH;
        const int hl = r2 - wl * p.HH;
        const int hi = org_h[jl] * p.g.sh - p.g.pad_t + hl;
        const int wi = org_w[jl] * p.g.sw - p.g.pad_l + wl;
        int off = -1, moff = -1;
        // Outside its window a column is zero by construction; the memory there may hold stale data (the
        // producer wrote the window only), so such elements are zero filled like the padding.
        const int4 ib = in_box[jl];
        const bool in_win = unsigned(hi - ib.x) < unsigned(ib.z) && unsigned(wi - ib.y) < unsigned(ib.w);
        if (hi >= 0 && hi < H && wi >= 0 && wi < W && j0 + jl < ncols && in_win) {
            off = int(jl * ld_in) + hi + H * wi;
            // rows cleared by the preceding ReLU step are masked here instead of being zeroed in memory
            if (mask.state != nullptr && col_base + j0 + jl < mask.ncols)
                moff = int(mask.col_q[col_base + j0 + jl] * mask.N) + hi + H * wi;
        }
        gtab[r] = off;
        mtab[r] = moff;
    }
    // per-channel epilogue constants of this channel tile
    const bool has_bn = bn.rden != nullptr;
    for (int c = tid; c < BN; c += THREADS) {
        const int co = n0 + c;
        const bool ok = co < p.g.Cout;
        chan[c] = ok ? bias[co] : 0.0;
        chan[BN + c] = (ok && has_bn) ? bn.mean[co] : 0.0;
        chan[2 * BN + c] = (ok && has_bn) ? bn.rden[co] : 1.0;
        chan[3 * BN + c] = (ok && has_bn) ? bn.scale[co] : 1.0;
        chan[4 * BN + c] = (ok && has_bn) ? bn.offset[co] : 0.0;
    }
    __syncthreads();

    const double* in_base = Vin + (col_base + j0) * ld_in;
    const int64_t w_block = int64_t(p.w_stage);
    const double* w_base = Wg + (int64_t(n_tile) * p.n_chunks) * w_block;

    auto load_stage = [&](int stage, int chunk) {
        double* hs = halo + stage * p.halo_stage;
        // each warp fetches the halo planes of channels warp, warp+NWARPS, ...
        for (int cil = warp; cil < KC; cil += NWARPS) {
            const int ci = chunk * KC + cil;
            const bool ci_ok = ci < p.g.Cin;
            const double* src_c = in_base + int64_t(ci_ok ? ci : 0) * hw_in;
            double* dst_c = hs + cil * p.PS;
            if (mask.state == nullptr) {
                for (int r = lane; r < p.plane; r += 32) {
                    const int off = gtab[r];
                    const bool ok = ci_ok && off >= 0;
                    cp_async8(dst_c + r, ok ? (src_c + off) : Vin, ok ? 8 : 0);
                }
            } else {
                // four elements per lane at a time, so that the row-state loads are in flight together
                const uint8_t* st_c = mask.state + int64_t(ci_ok ? ci : 0) * hw_in;
                for (int r0 = lane; r0 < p.plane; r0 += 128) {
                    int off[4];
                    uint8_t sv[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int r = r0 + 32 * u;
                        off[u] = (r < p.plane && ci_ok) ? gtab[r] : -1;
                        const int moff = (r < p.plane && ci_ok) ? mtab[r] : -1;
                        sv[u] = moff >= 0 ? st_c[moff] : uint8_t(0);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int r = r0 + 32 * u;
                        if (r >= p.plane) break;
                        const bool ok = off[u] >= 0 && sv[u] == 0;
                        cp_async8(dst_c + r, ok ? (src_c + off[u]) : Vin, ok ? 8 : 0);
                    }
                }
            }
        }
        double* ws = wts + stage * p.w_stage;
        const double* wsrc = w_base + int64_t(chunk) * w_block;
        for (int c = tid; c < p.w_stage / 2; c += THREADS) cp_async16(ws + 2 * c, wsrc + 2 * c, 16);
    };

    // shared-memory base of the rows this lane owns in each m16 tile
    // and where its outputs go (relative to column j0, channel 0; -1 = nothing to store)
    int rowbase[WM_TILES][2];
    int outoff[WM_TILES][2];
#pragma unroll
    for (int mi = 0; mi < WM_TILES; ++mi) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            int m = wm * WM_TILES * 16 + mi * 16 + g + half * 8;
            const int per_col = p.TH * p.TW;
            int jl = m / per_col;
            int rem = m - jl * per_col;
            int owl = rem / p.TH;
            int ohl = rem - owl * p.TH;
            const int oh = org_h[jl < p.NJ ? jl : 0] + ohl, ow = org_w[jl < p.NJ ? jl : 0] + owl;
            const bool ok = jl < p.NJ && oh >= 0 && ow >= 0 && oh < p.g.Ho && ow < p.g.Wo && j0 + jl < ncols;
            outoff[mi][half] = ok ? int(jl * ld_out) + oh + p.g.Ho * ow : -1;
            if (jl >= p.NJ) { jl = 0; owl = 0; ohl = 0; }   // padding rows read a valid address
            rowbase[mi][half] = jl * (p.HH * p.HW) + (owl * p.g.sw) * p.HH + ohl * p.g.sh;
        }
    }

    double acc[WM_TILES][WN_TILES][4];
#pragma unroll
    for (int mi = 0; mi < WM_TILES; ++mi)
#pragma unroll
        for (int ni = 0; ni < WN_TILES; ++ni)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[mi][ni][r] = 0.0;

    const int NCH = p.n_chunks;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < NCH) load_stage(s, s);
        cp_async_commit();
    }

    for (int ch = 0; ch < NCH; ++ch) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        {
            const int nc = ch + STAGES - 1;
            if (nc < NCH) load_stage(nc % STAGES, nc);
            cp_async_commit();
        }
        const double* hs = halo + (ch % STAGES) * p.halo_stage + t * p.PS;
        const double* ws = wts + (ch % STAGES) * p.w_stage + t * p.CS + wn * WN_TILES * 8 + g;
        int tap = 0;
        for (int kwi = 0; kwi < p.g.kw; ++kwi) {
            for (int khi = 0; khi < p.g.kh; ++khi, ++tap) {
                // tap index follows W's memory order (kh fastest)
                const int tapoff = (kwi * p.g.dw) * p.HH + khi * p.g.dh;
                const double* wt = ws + tap * (KC * p.CS);
                double af[WM_TILES][4];
                double bf[WN_TILES][2];
#pragma unroll
                for (int mi = 0; mi < WM_TILES; ++mi) {
                    const double* p0 = hs + rowbase[mi][0] + tapoff;
                    const double* p1 = hs + rowbase[mi][1] + tapoff;
                    af[mi][0] = p0[0];
                    af[mi][1] = p1[0];
                    af[mi][2] = p0[4 * p.PS];
                    af[mi][3] = p1[4 * p.PS];
                }
#pragma unroll
                for (int ni = 0; ni < WN_TILES; ++ni) {
                    bf[ni][0] = wt[ni * 8];
                    bf[ni][1] = wt[ni * 8 + 4 * p.CS];
                }
#pragma unroll
                for (int mi = 0; mi < WM_TILES; ++mi)
#pragma unroll
                    for (int ni = 0; ni < WN_TILES; ++ni) dmma_16x8x8(acc[mi][ni], af[mi], bf[ni]);
            }
        }
    }
    cp_async_wait<0>();

    // epilogue: bias on the centre columns, the fused per-channel affine
    // ((x - mean) * (1/den)) * scale + offset in the reference's order, one
    // 8-byte store per element (8 lanes cover 64 contiguous bytes along h)
    const int64_t hw_out = int64_t(p.g.Ho) * p.g.Wo;
    const int per_col = p.TH * p.TW;
    double* out_base = Vout + (col_base + j0) * ld_out;
#pragma unroll
    for (int mi = 0; mi < WM_TILES; ++mi) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int off = outoff[mi][half];
            if (off < 0) continue;
            const int m = wm * WM_TILES * 16 + mi * 16 + g + half * 8;
            const bool is_center = col_base + j0 + m / per_col < n_center;
            double* dst = out_base + off;
#pragma unroll
            for (int ni = 0; ni < WN_TILES; ++ni) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int c = wn * WN_TILES * 8 + ni * 8 + 2 * t + e;
                    if (n0 + c >= p.g.Cout) continue;
                    double v = acc[mi][ni][half * 2 + e];
                    if (is_center) v = (v + chan[c]) - chan[BN + c];
                    v = (v * chan[2 * BN + c]) * chan[3 * BN + c];
                    if (is_center) v += chan[4 * BN + c];
                    dst[hw_out * (n0 + c)] = v;
                }
            }
        }
    }
}

// Convolution of one-hot columns.  A column the preceding ReLU step appended is the unit vector of
// neuron (h, w, ci); its image under the convolution is the filter footprint
//   out(oh, ow, co) = W(kh, kw, ci, co)   wherever oh*sh - pt + kh*dh = h and ow*sw - pl + kw*dw = w,
// times the generator part of the fused affine.  No products are formed, so the values equal what the
// dense contraction of that column gives (every other term of its sums is a product with zero).
// Every entry of the column's output window (origin and extent as update_windows_kernel derives them from
// a 1x1 input window) is written, zeros included; nothing outside it is touched.  One block per column,
// lanes over (window position, output channel).  A column with a scale (a generator of a bounds-form input set,
// a one-hot column that went through a pooling layer) gives scale times the footprint: the one product its dense contraction would form.
__global__ void __launch_bounds__(128)
conv_onehot_kernel(ConvGeom g, const double* __restrict__ Wg, int bn_tile, int cs, int n_chunks, ChanAffine bn,
                   HotCols hot, double* __restrict__ Vout, int64_t ld_out, double* __restrict__ pack, bool staged) {
    const int64_t t = blockIdx.x;
    const int i = hot.idx[hot.first + t * hot.step];
    const bool scaled = hot.scale != nullptr;
    const double sc = scaled ? hot.scale[t] : 1.0;
    const int h = i % g.H;
    const int w = (i / g.H) % g.W;
    const int ci = i / (g.H * g.W);
    const int taps = g.kh * g.kw;
    const int ch = ci / KC, cil = ci % KC;
    const int eh = (g.kh - 1) * g.dh, ew = (g.kw - 1) * g.dw;
    const int wh = eh / g.sh + 1, ww = ew / g.sw + 1;
    const int ah = h + g.pad_t - eh, aw = w + g.pad_l - ew;
    const int org_h = ah >= 0 ? (ah + g.sh - 1) / g.sh : -((-ah) / g.sh);
    const int org_w = aw >= 0 ? (aw + g.sw - 1) / g.sw : -((-aw) / g.sw);
    double* dst = Vout != nullptr ? Vout + t * ld_out : nullptr;
    // the tap value at output (oh, ow, co), zero where no tap maps it to input (h, w)
    auto entry = [&](int oh, int ow, int co) -> double {
        const int dh_ = h + g.pad_t - oh * g.sh, dw_ = w + g.pad_l - ow * g.sw;
        if (!(dh_ >= 0 && dw_ >= 0 && dh_ % g.dh == 0 && dw_ % g.dw == 0 && dh_ / g.dh < g.kh && dw_ / g.dw < g.kw))
            return 0.0;
        const int tap = dh_ / g.dh + g.kh * (dw_ / g.dw);
        const int nt = co / bn_tile, n = co % bn_tile;
        double v = Wg[((((int64_t(nt) * n_chunks + ch) * taps + tap) * KC + cil) * cs) + n];
        if (scaled) v = v * sc;
        if (bn.rden != nullptr) v = (v * bn.rden[co]) * bn.scale[co];
        return v;
    };
    // in front of a ReLU layer: the window-only copy the bound reduction reads, channel fastest.  With room in
    // shared memory the entries are computed once, here, and the writes below take them from there
    extern __shared__ double sv[];
    if (pack != nullptr) {
        double* pk = pack + t * (int64_t(wh) * ww * g.Cout);
        for (int e = threadIdx.x; e < wh * ww * g.Cout; e += blockDim.x) {
            const int co = e % g.Cout, pos = e / g.Cout;
            const double v = entry(org_h + pos % wh, org_w + pos / wh, co);
            pk[e] = v;
            if (staged) sv[e] = v;
        }
        if (staged) __syncthreads();
    }
    if (Vout == nullptr) return;          // the images exist in compact form only
    auto value = [&](int oh, int ow, int co) -> double {
        return staged ? sv[((ow - org_w) * wh + (oh - org_h)) * g.Cout + co] : entry(oh, ow, co);
    };
    const int lo = max(org_h, 0), hi = min(org_h + wh, g.Ho);     // window rows on the image
    if (hi <= lo) return;
    if (g.Ho % 4 == 0 && ld_out % 4 == 0) {
        // whole 32-byte sectors: the aligned groups of four rows that cover the window rows are written, with
        // zeros in the entries outside the window (which are zero in the dense tensor too); a partly written
        // sector costs the memory system a read on top of the write
        const int a0 = lo & ~3;
        const int ngr = (hi - a0 + 3) / 4;
        for (int e = threadIdx.x; e < ngr * ww * g.Cout; e += blockDim.x) {
            const int r0 = a0 + 4 * (e % ngr);
            const int e2 = e / ngr;
            const int co = e2 % g.Cout;
            const int ow = org_w + e2 / g.Cout;
            if (ow < 0 || ow >= g.Wo) continue;
            double v[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) v[r] = (r0 + r >= lo && r0 + r < hi) ? value(r0 + r, ow, co) : 0.0;
            double2* d2 = reinterpret_cast<double2*>(dst + r0 + int64_t(g.Ho) * (ow + int64_t(g.Wo) * co));
            d2[0] = make_double2(v[0], v[1]);
            d2[1] = make_double2(v[2], v[3]);
        }
        return;
    }
    // patch rows fastest: the lanes of one (patch column, channel) write consecutive addresses
    for (int e = threadIdx.x; e < wh * ww * g.Cout; e += blockDim.x) {
        const int oh = org_h + e % wh;
        const int e2 = e / wh;
        const int co = e2 % g.Cout;
        const int ow = org_w + e2 / g.Cout;
        if (oh < 0 || ow < 0 || oh >= g.Ho || ow >= g.Wo) continue;
        dst[oh + int64_t(g.Ho) * (ow + int64_t(g.Wo) * co)] = value(oh, ow, co);
    }
}

// The same images for unit stride and dilation, compact form only: a column's window is the filter flipped in
// both directions, read as one contiguous run from the footprint table (ConvWeights::foot) and scaled in the
// order of conv_onehot_kernel.  Four columns per block, lanes along (position, channel).
__global__ void __launch_bounds__(256)
conv_onehot_foot_kernel(ConvGeom g, const double* __restrict__ foot, ChanAffine bn, HotCols hot, int64_t K_loc,
                        double* __restrict__ pack) {
    const int per_col = g.kh * g.kw * g.Cout;
    const int64_t t = int64_t(blockIdx.x) * 4 + (threadIdx.x >> 6);
    if (t >= K_loc) return;
    const int i = hot.idx[hot.first + t * hot.step];
    const bool scaled = hot.scale != nullptr;
    const double sc = scaled ? hot.scale[t] : 1.0;
    const int ci = i / (g.H * g.W);
    const double* src = foot + int64_t(ci) * per_col;
    double* pk = pack + t * int64_t(per_col);
    for (int e = threadIdx.x & 63; e < per_col; e += 64) {
        const int co = e % g.Cout;
        double v = src[e];
        if (scaled) v = v * sc;
        if (bn.rden != nullptr) v = (v * bn.rden[co]) * bn.scale[co];
        pk[e] = v;
    }
}

int pad_stride(int n) {            // smallest s >= n with s = 4 (mod 8)
    int s = (n + 7) / 8 * 8 + 4;
    if (s - 8 >= n) s -= 8;
    return s;
}

int pick_bn_tile(int Cout) { return Cout <= 16 ? 16 : (Cout <= 32 ? 32 : 64); }

void pick_tile(const ConvGeom& g, int BM, int* TH, int* TW, int* NJ) {
    const int per_img = g.Ho * g.Wo;
    if (per_img * 2 <= BM) {       // several columns per tile
        *TH = g.Ho;
        *TW = g.Wo;
        *NJ = BM / per_img;
        return;
    }
    *NJ = 1;
    double best = -1.0;
    for (int th = 1; th <= std::min(g.Ho, BM); ++th) {
        int tw = std::min(g.Wo, BM / th);
        if (tw < 1) continue;
        const int64_t tiles = ceil_div(g.Ho, th) * ceil_div(g.Wo, tw);
        double eff = double(per_img) / double(tiles * BM);
        // prefer tall tiles (longer runs along the contiguous axis) on ties
        eff += 1e-6 * th;
        if (eff > best) { best = eff; *TH = th; *TW = tw; }
    }
}

template <int WM_TILES, int WN_TILES, int WARPS_M, int WARPS_N, int STAGES, int MIN_BLOCKS>
int launch_variant(cudaStream_t st, const ConvParams& p, dim3 grid, size_t smem, const ConvWeights& w,
                   const ChanAffine& bn, const RowMask& mask, const ColWindows& win, int64_t col_base,
                   const double* Vin, int64_t ld_in, double* Vout, int64_t ld_out, int64_t ncols, int64_t n_center) {
    auto kern = conv_f64_kernel<WM_TILES, WN_TILES, WARPS_M, WARPS_N, STAGES, MIN_BLOCKS>;
    NNVB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    // ask for the largest shared-memory carve-out so that MIN_BLOCKS CTAs really are resident
    NNVB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    kern<<<grid, WARPS_M * WARPS_N * 32, smem, st>>>(p, w.w, w.bias, bn, mask, win, col_base, Vin, ld_in, Vout, ld_out,
                                                     ncols, n_center);
    NNVB_CUDA(cudaGetLastError());
    return NNVB_OK;
}

template <int WM_TILES, int WN_TILES, int WARPS_M, int WARPS_N>
int launch_cfg(cudaStream_t st, const ConvGeom& g, const ConvWeights& w, const ChanAffine& bn, const RowMask& mask,
               const ColWindows& win, int64_t col_base, const double* Vin, int64_t ld_in, double* Vout,
               int64_t ld_out, int64_t ncols, int64_t n_center) {
    constexpr int BM = WARPS_M * WM_TILES * 16;
    constexpr int BN = WARPS_N * WN_TILES * 8;
    ConvParams p;
    p.g = g;
    if (win.wh > 0) {
        // one patch of wh x ww outputs per column, as many columns per tile as fit
        if (win.wh * win.ww > BM || win.wh < 1 || win.ww < 1) {
            set_error("conv: output window %dx%d does not fit a tile", win.wh, win.ww);
            return NNVB_E_ARG;
        }
        p.TH = win.wh;
        p.TW = win.ww;
        p.NJ = std::min(BM / (win.wh * win.ww), 128);
    } else {
        pick_tile(g, BM, &p.TH, &p.TW, &p.NJ);
    }
    p.HH = (p.TH - 1) * g.sh + (g.kh - 1) * g.dh + 1;
    p.HW = (p.TW - 1) * g.sw + (g.kw - 1) * g.dw + 1;
    p.plane = p.NJ * p.HH * p.HW;
    p.PS = pad_stride(p.plane);
    p.CS = w.cs;
    p.n_th = win.wh > 0 ? 1 : (int)ceil_div(g.Ho, p.TH);
    p.n_tw = win.wh > 0 ? 1 : (int)ceil_div(g.Wo, p.TW);
    p.n_chunks = w.n_chunks;
    p.taps = g.kh * g.kw;
    p.halo_stage = KC * p.PS;
    p.w_stage = p.taps * KC * p.CS;
    p.col_groups = ceil_div(ncols, p.NJ);
    if (w.bn_tile != BN) {
        set_error("conv: weight arrangement (%d) does not match kernel tile (%d)", w.bn_tile, BN);
        return NNVB_E_ARG;
    }
    if (int64_t(p.NJ) * std::max(ld_in, ld_out) >= (int64_t(1) << 31)) {
        set_error("conv: column stride too large for the tile offset table");
        return NNVB_E_UNSUPPORTED;
    }
    const size_t stage_bytes = size_t(p.halo_stage + p.w_stage) * sizeof(double);
    const size_t fixed_bytes = size_t(5 * BN) * sizeof(double) + size_t(2 * p.plane) * sizeof(int);
    const size_t limit = 227 * 1024;
    const int64_t blocks = p.col_groups * p.n_th * p.n_tw;
    if (blocks >= (int64_t(1) << 31)) {
        set_error("conv: grid too large");
        return NNVB_E_UNSUPPORTED;
    }
    dim3 grid((unsigned)blocks, (unsigned)w.n_tiles);
    // Two resident CTAs per SM (one runs its epilogue while the other contracts) when two
    // double-buffered CTAs fit in shared memory; else one CTA with a 3- or 2-deep ring.
    static const int variant = getenv("NNVB_CONV_VARIANT") ? atoi(getenv("NNVB_CONV_VARIANT")) : 0;
    const size_t two = 2 * stage_bytes + fixed_bytes;
    const size_t three = 3 * stage_bytes + fixed_bytes;
    if ((variant == 0 || variant == 2) && 2 * (two + 1024) <= limit)
        return launch_variant<WM_TILES, WN_TILES, WARPS_M, WARPS_N, 2, 2>(st, p, grid, two, w, bn, mask, win, col_base, Vin, ld_in, Vout,
                                                                         ld_out, ncols, n_center);
    if (three <= limit)
        return launch_variant<WM_TILES, WN_TILES, WARPS_M, WARPS_N, 3, 1>(st, p, grid, three, w, bn, mask, win, col_base, Vin, ld_in, Vout,
                                                                         ld_out, ncols, n_center);
    if (two <= limit)
        return launch_variant<WM_TILES, WN_TILES, WARPS_M, WARPS_N, 2, 1>(st, p, grid, two, w, bn, mask, win, col_base, Vin, ld_in, Vout,
                                                                         ld_out, ncols, n_center);
    set_error("conv: filter %dx%d with stride (%d,%d) needs %zu bytes of shared memory per stage", g.kh, g.kw, g.sh,
              g.sw, stage_bytes);
    return NNVB_E_UNSUPPORTED;
}

}  // namespace

size_t conv_weights_doubles(const ConvGeom& g, int* bn_tile, int* cs, int* n_tiles, int* n_chunks) {
    *bn_tile = pick_bn_tile(g.Cout);
    *cs = *bn_tile + 4;
    *n_tiles = (int)ceil_div(g.Cout, *bn_tile);
    *n_chunks = (int)ceil_div(g.Cin, KC);
    return size_t(*n_tiles) * (*n_chunks) * (g.kh * g.kw) * KC * (*cs);
}

void conv_arrange_weights(const ConvGeom& g, const double* W, double* dst, int bn_tile, int cs,
                          int n_tiles, int n_chunks) {
    // dst[n_tile][chunk][tap][cil][cs]; tap = kh + KH*kw (W's own order); zero padded
    const int taps = g.kh * g.kw;
    const size_t total = size_t(n_tiles) * n_chunks * taps * KC * cs;
    std::fill(dst, dst + total, 0.0);
    for (int nt = 0; nt < n_tiles; ++nt)
        for (int ch = 0; ch < n_chunks; ++ch)
            for (int tap = 0; tap < taps; ++tap)
                for (int cil = 0; cil < KC; ++cil) {
                    const int ci = ch * KC + cil;
                    if (ci >= g.Cin) continue;
                    double* row = dst + ((((size_t(nt) * n_chunks + ch) * taps + tap) * KC + cil) * cs);
                    for (int n = 0; n < bn_tile; ++n) {
                        const int co = nt * bn_tile + n;
                        if (co >= g.Cout) break;
                        row[n] = W[size_t(tap) + size_t(taps) * (ci + size_t(g.Cin) * co)];
                    }
                }
}

int launch_conv_f64(cudaStream_t st, const ConvGeom& g, const ConvWeights& w, const ChanAffine& bn,
                    const RowMask& mask, const ColWindows& win, int64_t col_base, const double* Vin, int64_t ld_in,
                    double* Vout, int64_t ld_out, int64_t ncols, int64_t n_center, int64_t* launches) {
    if (ncols <= 0) return NNVB_OK;
    int s;
    if (w.bn_tile == 16)
        s = launch_cfg<1, 2, 8, 1>(st, g, w, bn, mask, win, col_base, Vin, ld_in, Vout, ld_out, ncols, n_center);
    else if (w.bn_tile == 32)
        s = launch_cfg<2, 2, 4, 2>(st, g, w, bn, mask, win, col_base, Vin, ld_in, Vout, ld_out, ncols, n_center);
    else
        s = launch_cfg<2, 4, 4, 2>(st, g, w, bn, mask, win, col_base, Vin, ld_in, Vout, ld_out, ncols, n_center);
    if (s == NNVB_OK && launches) *launches += 1;
    return s;
}

int launch_conv_onehot(cudaStream_t st, const ConvGeom& g, const ConvWeights& w, const ChanAffine& bn,
                       const HotCols& hot, int64_t K_loc, double* Vout, int64_t ld_out, bool zero_fill,
                       double* pack, int64_t* launches) {
    if (K_loc <= 0) return NNVB_OK;
    if (Vout == nullptr && pack == nullptr) {
        set_error("conv_onehot: no output buffer");
        return NNVB_E_ARG;
    }
    if (zero_fill && Vout != nullptr) NNVB_CUDA(cudaMemsetAsync(Vout, 0, sizeof(double) * ld_out * K_loc, st));
    if (Vout == nullptr && w.foot != nullptr && g.sh == 1 && g.sw == 1 && g.dh == 1 && g.dw == 1) {
        conv_onehot_foot_kernel<<<(unsigned)ceil_div(K_loc, 4), 256, 0, st>>>(g, w.foot, bn, hot, K_loc, pack);
        NNVB_CUDA(cudaGetLastError());
        if (launches) *launches += 1;
        return NNVB_OK;
    }
    // the window of a column: (kh-1)*dh/sh + 1 rows, likewise columns, all output channels
    const size_t win_bytes = sizeof(double) * size_t((g.kh - 1) * g.dh / g.sh + 1) * ((g.kw - 1) * g.dw / g.sw + 1) * g.Cout;
    const bool staged = pack != nullptr && win_bytes <= 32768;
    // 64 threads per column: 32 blocks fill an SM (measured per step: 32 threads 1.01 ms, 64 1.03, 128 1.13, 256 1.40)
    conv_onehot_kernel<<<(unsigned)K_loc, 64, staged ? win_bytes : 0, st>>>(g, w.w, w.bn_tile, w.cs, w.n_chunks, bn, hot,
                                                                            Vout, ld_out, pack, staged);
    NNVB_CUDA(cudaGetLastError());
    if (launches) *launches += 1;
    return NNVB_OK;
}

}  // namespace nnvb
