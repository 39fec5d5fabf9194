// Convolution of windowed columns, FP64 on the DMMA pipe (sm_100a).
//
// A windowed column is zero outside a small wh_in x ww_in window of the input image, so its image
// under a unit-stride convolution is zero outside a (wh_in + kh - 1) x (ww_in + kw - 1) patch.  The
// dense kernel (conv_f64.cu) computes such a patch with the output positions as the rows of its
// tiles and runs every filter tap for every row, although for the rows near the patch border most
// taps read outside the input window: about half of its products are with structural zeros.
//
// Here the rows of an MMA tile are 16 COLUMNS at the same patch position.  All columns of a cohort
// share the window geometry, so whether tap (khi, kwi) of patch position (oh, ow) reads inside the
// input window is the same for the 16 rows of a tile, and the taps that do not are skipped
// altogether.  A block owns 16*WARPS_M columns, one patch column ow and up to 8 patch rows; warp
// (wm, wn) owns 16 columns and 8 output channels and keeps one accumulator tile per patch row.
// An input row fragment is loaded once and used by the (up to kh) taps that pair it with different
// output rows.
//
// Conv2DLayer.reach_star_single_input (Conv2DLayer.m:559-601) applies the layer to the centre
// with bias and to every generator without; this kernel is used for generator columns only.
#include <algorithm>

#include "common.cuh"
#include "mma_f64.cuh"
#include <type_traits>

namespace nnvb {
namespace {

constexpr int KC = 8;               // input channels per pipeline stage, as conv_arrange_weights lays them out
constexpr int CW_TH = 8;            // patch rows per block
constexpr int CW_THREADS = 512;
constexpr int CW_STAGES = 2;
constexpr int CW_MAX_STAGES = 4;    // warp-specialised form: 2 to 4 stages, as many as shared memory holds
// dynamic shared memory a block may ask for: the 227 KB of an SM less the kernels' static variables (barriers, flags)
constexpr size_t CW_SMEM_LIMIT = size_t(227) * 1024 - 256;

struct ConvWinParams {
    ConvGeom g;
    int wh_in, ww_in, wh_out, ww_out;
    int n_ohb;                      // row blocks per patch
    int ni_s;                       // input rows staged per origin column
    int CSI;                        // stride between the channels of a staged input row (doubles)
    int RS;                         // stride between staged input rows: 8 channels and one double, so that
                                    // the rows a warp fetches together fall on different banks
    int CS;                         // weight channel stride (doubles)
    int in_stage, w_stage;          // doubles per stage
    int n_chunks;
    int ncol;                       // columns per block
    int OSTR, CSTR;                 // epilogue staging strides: patch row, column (doubles)
    double* pack;                   // window-only copy of the launch's columns (null: none): entry (ohl, owl, co) of
    int64_t pack_stride;            // column j at j*pack_stride + (owl*wh_out + ohl)*Cout + co
    int tab_cap;                    // table entries
    int tail;                       // doubles before the constants and tables
    // compact input (null: Vin holds full-length columns): the launch's columns window-only and channel fastest,
    // entry (h, w, c) of column j at cin + j*cin_stride + ((w - w0)*wh_in + (h - h0))*Cin + c
    const double* cin;
    int64_t cin_stride;
    // persistent form: tiles = column groups x patch columns x row blocks x output-channel tiles, channel tiles fastest
    int n_ytiles;
    int64_t n_flat;
    int stages;                     // persistent form: pipeline depth
    int use_bits;                   // persistent form, at most 64 input channels: the row states of a table entry
                                    // are gathered once into a 64-bit word
};

// CIN: the input is read from compact storage (p.cin).  A (column, input position) then holds its 8-channel chunk
// in 64 contiguous bytes: one thread fetches it with four 16-byte copies into a staging row [column][8 channels]
// (channel index XOR 4 for every other column pair, which keeps the fragment loads free of bank conflicts without
// padding), and reads the eight row states of the chunk as one 8-byte word when they come in channel-fastest order.
// NROWS > 0: the input windows are NROWS rows high and one block covers all patch rows, so the rows a block meets
// are known at compile time and the unrolled product loop carries no range tests (0: any height, tested at run time).
template <int KH, int WARPS_M, int WARPS_N, bool CIN, int NROWS>
__global__ void __launch_bounds__(CW_THREADS, 1)
conv_win_kernel(const ConvWinParams p, const double* __restrict__ Wg, const ChanAffine bn, const RowMask mask,
                const int4* __restrict__ box, int64_t col_base, const double* __restrict__ Vin, int64_t ld_in,
                double* __restrict__ Vout, int64_t ld_out, int64_t ncols) {
    static_assert(WARPS_M * WARPS_N * 32 == CW_THREADS, "16 warps");
    constexpr int BN = WARPS_N * 8;
    constexpr int NI = CW_TH + KH - 1;              // input rows that can meet the block's output rows

    extern __shared__ __align__(16) double smem[];
    double* in_s = smem;                                        // [STAGES][in_stage]
    double* wts = smem + CW_STAGES * p.in_stage;                // [STAGES][w_stage]
    double* chan = smem + p.tail;                               // [2][BN]: 1/den, scale
    int* goff = reinterpret_cast<int*>(chan + 2 * BN);          // [tab_cap] input offset, -1 = zero
    int* soff = goff + p.tab_cap;                               // [tab_cap] staging offset
    int* moff = soff + p.tab_cap;                               // [tab_cap] row-state offset, -1 = none
    int4* s_box = reinterpret_cast<int4*>(moff + p.tab_cap);    // [ncol]

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int wm = warp % WARPS_M;
    const int wn = warp / WARPS_M;
    const int g = lane >> 2;
    const int t = lane & 3;

    const int per = p.ww_out * p.n_ohb;
    const int64_t cg = blockIdx.x / per;
    const int rem = int(blockIdx.x % per);
    const int owl = rem / p.n_ohb;
    const int ohb = rem % p.n_ohb;
    const int64_t j0 = cg * p.ncol;
    const int n_tile = blockIdx.y;
    const int n0 = n_tile * BN;
    const int H = p.g.H, W = p.g.W;
    const int hw_in = H * W;
    const int KW = p.g.kw;
    const int ext_h = KH - 1, ext_w = KW - 1;

    // input rows i (relative to ih_base) that lie in the window, and the output rows of this block
    const int ih_base = ohb * CW_TH - ext_h;
    const int i_lo = NROWS > 0 ? KH - 1 : max(0, -ih_base);
    const int i_hi = NROWS > 0 ? KH - 1 + NROWS : min(NI, p.wh_in - ih_base);
    const int n_i = i_hi - i_lo;
    const int th_cnt = min(CW_TH, p.wh_out - ohb * CW_TH);
    // origin columns kwi whose input column owl + kwi - ext_w lies in the window
    const int kw_lo = max(0, ext_w - owl);
    const int kw_hi = min(KW, p.ww_in + ext_w - owl);
    const int n_kw = kw_hi - kw_lo;

    for (int c = tid; c < p.ncol; c += CW_THREADS) {
        int4 bx = make_int4(0, 0, 0, 0);
        if (j0 + c < ncols) bx = box[col_base + j0 + c];
        s_box[c] = bx;
    }
    const bool has_bn = bn.rden != nullptr;
    for (int c = tid; c < BN; c += CW_THREADS) {
        const int co = n0 + c;
        const bool ok = co < p.g.Cout && has_bn;
        chan[c] = ok ? bn.rden[co] : 1.0;
        chan[BN + c] = ok ? bn.scale[co] : 1.0;
    }
    __shared__ unsigned row_used[WARPS_M];
    __shared__ __align__(8) uint64_t w_bar[CW_STAGES];      // one barrier per weight stage (bulk copies land on it)
    if (tid < WARPS_M) row_used[tid] = 0u;
    if (tid == 0) {
        for (int s = 0; s < CW_STAGES; ++s) mbar_init(&w_bar[s], 1);
        mbar_init_fence();
    }
    __syncthreads();

    // Patches near the image border hang over it.  Columns that lie next to each other in memory come from
    // neighbouring pixels, so whole tiles agree on which patch positions are off the image: a block whose
    // patch column is off the image for all of its columns has nothing to do, and a tile skips the patch
    // rows that are off the image for its 16 columns.
    bool col_on = false;
    if (tid < p.ncol && j0 + tid < ncols) {
        const int4 bx = s_box[tid];
        const int ow = bx.y + p.g.pad_l - ext_w + owl;
        col_on = ow >= 0 && ow < p.g.Wo;
        if (col_on) {
            unsigned m = 0u;
            for (int o = 0; o < th_cnt; ++o) {
                const int oh = bx.x + p.g.pad_t - ext_h + ohb * CW_TH + o;
                if (oh >= 0 && oh < p.g.Ho) m |= 1u << o;
            }
            if (m) atomicOr(&row_used[tid >> 4], m);
        }
    }
    if (__syncthreads_or(col_on ? 1 : 0) == 0) return;
    const unsigned rows_on = row_used[wm];

    // table: entry e = (column, origin column, input row), input row fastest (contiguous in memory)
    const int n_e = p.ncol * n_kw * n_i;
    for (int e = tid; e < n_e; e += CW_THREADS) {
        // full-length input: input row fastest (contiguous in memory); compact input: column fastest, so that
        // neighbouring lanes of the fetch write neighbouring 64-byte slots of the staging row
        int i_idx, kwi, col;
        if (CIN) {
            col = e % p.ncol;
            const int e2 = e / p.ncol;
            i_idx = e2 % n_i;
            kwi = kw_lo + e2 / n_i;
        } else {
            i_idx = e % n_i;
            const int e2 = e / n_i;
            kwi = kw_lo + e2 % n_kw;
            col = e2 / n_kw;
        }
        const int4 bx = s_box[col];
        const int hi = bx.x + ih_base + i_lo + i_idx;
        const int wi = bx.y + owl + kwi - ext_w;
        int off = -1, mo = -1;
        if (hi >= 0 && hi < H && wi >= 0 && wi < W && j0 + col < ncols) {
            off = CIN ? int(col * p.cin_stride) + ((wi - bx.y) * p.wh_in + (hi - bx.x)) * p.g.Cin
                      : int(col * ld_in) + hi + H * wi;
            if (mask.state != nullptr && col_base + j0 + col < mask.ncols) {
                const int q_off = int(mask.col_q[col_base + j0 + col] * mask.N);
                mo = (CIN && mask.state_cf != nullptr) ? q_off + (hi + H * wi) * p.g.Cin : q_off + hi + H * wi;
            }
        }
        goff[e] = off;
        moff[e] = mo;
        // CIN: [origin column][input row][column][8 channels], the swizzle bit of the column in bit 30
        soff[e] = CIN ? (((kwi * p.ni_s + i_idx) * p.ncol + col) * KC) | (((col >> 1) & 1) << 30)
                      : (kwi * p.ni_s + i_idx) * p.RS + col;
    }
    __syncthreads();

    const double* in_base = CIN ? p.cin + j0 * p.cin_stride : Vin + (col_base + j0) * ld_in;
    const double* zero_src = CIN ? p.cin : Vin;      // a valid address for the zero-size copies
    const double* w_base = Wg + (int64_t(n_tile) * p.n_chunks) * p.w_stage;

    auto load_stage = [&](int stage, int chunk) {
        double* is = in_s + stage * p.in_stage;
        if (CIN) {
            // one 16-byte channel pair of one (column, input position) per thread and round: four neighbouring
            // lanes fetch the 64 bytes of an entry, eight neighbouring entries are eight neighbouring columns, so a
            // warp's copies fill 512 contiguous bytes of the staging row (no bank conflicts)
            const int c0 = chunk * KC;
            const double* src_b = in_base + c0;
            const bool cf = mask.state_cf != nullptr;
            const bool pair_ok = cf && (p.g.Cin % 2 == 0) && (mask.N % 2 == 0);
            for (int it = tid; it < 4 * n_e; it += CW_THREADS) {
                const int e = it >> 2, u0 = 2 * (it & 3);
                const int off = goff[e], so_raw = soff[e], mo = moff[e];
                const int so = so_raw & 0x3fffffff;
                const int sw = (so_raw >> 30) & 1 ? 4 : 0;
                bool ok0 = off >= 0 && c0 + u0 < p.g.Cin, ok1 = off >= 0 && c0 + u0 + 1 < p.g.Cin;
                if (mo >= 0 && (ok0 || ok1)) {                   // rows the ReLU step cleared read as zero
                    if (pair_ok) {
                        const unsigned sv = *reinterpret_cast<const unsigned short*>(mask.state_cf + mo + c0 + u0);
                        ok0 = ok0 && (sv & 0xffu) == 0;
                        ok1 = ok1 && (sv >> 8) == 0;
                    } else {
                        if (ok0) ok0 = (cf ? mask.state_cf[mo + c0 + u0] : mask.state[mo + int64_t(c0 + u0) * hw_in]) == 0;
                        if (ok1) ok1 = (cf ? mask.state_cf[mo + c0 + u0 + 1] : mask.state[mo + int64_t(c0 + u0 + 1) * hw_in]) == 0;
                    }
                }
                double* d2 = is + so + (u0 ^ sw);
                if (ok0 && ok1) {
                    cp_async16(d2, src_b + off + u0, 16);
                } else {
                    cp_async8(d2, ok0 ? src_b + off + u0 : zero_src, ok0 ? 8 : 0);
                    cp_async8(d2 + 1, ok1 ? src_b + off + u0 + 1 : zero_src, ok1 ? 8 : 0);
                }
            }
        } else {
            // warp w fetches channel w % 8 of the chunk; the two warps of a channel split the table
            const int cil = warp & 7;
            const int ci = chunk * KC + cil;
            const bool ci_ok = ci < p.g.Cin;
            const double* src_c = in_base + int64_t(ci_ok ? ci : 0) * hw_in;
            const uint8_t* st_c = mask.state != nullptr ? mask.state + int64_t(ci_ok ? ci : 0) * hw_in : nullptr;
            double* dst_c = is + cil * p.CSI;
            for (int e0 = (warp >> 3) * 32 + lane; e0 < n_e; e0 += 256) {
                int off[4], so[4];
                uint8_t sv[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int e = e0 + 64 * u;
                    off[u] = (e < n_e && ci_ok) ? goff[e] : -1;
                    so[u] = e < n_e ? soff[e] : -1;
                    const int mo = (e < n_e && ci_ok && st_c != nullptr) ? moff[e] : -1;
                    sv[u] = mo >= 0 ? st_c[mo] : uint8_t(0);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (so[u] < 0) continue;
                    const bool ok = off[u] >= 0 && sv[u] == 0;
                    cp_async8(dst_c + so[u], ok ? (src_c + off[u]) : zero_src, ok ? 8 : 0);
                }
            }
        }
        // the chunk's weights are one contiguous block in memory and in the stage: a single bulk copy issued by
        // one thread moves it, and its bytes are counted on the stage's barrier
        if (tid == 0) {
            async_proxy_fence();
            mbar_expect_bytes(&w_bar[stage], uint32_t(p.w_stage) * 8u);
            bulk_copy_g2s(wts + stage * p.w_stage, w_base + int64_t(chunk) * p.w_stage, uint32_t(p.w_stage) * 8u,
                          &w_bar[stage]);
        }
    };

    double acc[CW_TH][4];
#pragma unroll
    for (int o = 0; o < CW_TH; ++o)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[o][r] = 0.0;

    // FULL: every patch row of the block is on the image for this warp's columns (the common case): the products
    // carry no per-row test, which would otherwise put a branch around every DMMA
    auto compute = [&](int ch, auto full_rows) {
        constexpr bool FULL = decltype(full_rows)::value;
        // row = column g (and g + 8), k = channel t (and t + 4)
        const int sw = CIN ? ((g >> 1) & 1) * 4 : 0;
        const double* is = CIN ? in_s + (ch & 1) * p.in_stage + (wm * 16 + g) * KC
                               : in_s + (ch & 1) * p.in_stage + t * p.CSI + wm * 16 + g;
        const int RSr = CIN ? p.ncol * KC : p.RS;                                    // stride between staged input rows
        const int o1 = CIN ? 8 * KC : 8, o2 = CIN ? ((t ^ sw) ^ 4) - (t ^ sw) : 4 * p.CSI;
        const int o0 = CIN ? (t ^ sw) : 0;
        const double* ws = wts + (ch & 1) * p.w_stage + t * p.CS + wn * 8 + g;      // k = channel t, n = g
        for (int kwi = kw_lo; kwi < kw_hi; ++kwi) {
            double bf[KH][2];
#pragma unroll
            for (int khi = 0; khi < KH; ++khi) {
                const double* wt = ws + (khi + KH * kwi) * (KC * p.CS);     // tap index: kh fastest
                bf[khi][0] = wt[0];
                bf[khi][1] = wt[4 * p.CS];
            }
            const double* a_col = is + (kwi * p.ni_s - i_lo) * RSr + o0;
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                if (i < i_lo || i >= i_hi) continue;
                const double* a = a_col + i * RSr;
                double af[4];
                af[0] = a[0];
                af[1] = a[o1];
                af[2] = a[o2];
                af[3] = a[o2 + o1];
                // input row i meets output row i - khi through tap khi
#pragma unroll
                for (int khi = 0; khi < KH; ++khi) {
                    const int o = i - khi;
                    if (o >= 0 && o < CW_TH) {
                        if (FULL || ((rows_on >> o) & 1u)) dmma_16x8x8(acc[o], af, bf[khi]);
                    }
                }
            }
        }
    };

    const int NCH = p.n_chunks;
    const unsigned row_bits = (1u << th_cnt) - 1u;
    const bool all_rows = (rows_on & row_bits) == row_bits;
    load_stage(0, 0);
    cp_async_commit();
    // Half of the warps fetch the next stage before their products, the other half after: while one half
    // waits on its table and row-state loads the other keeps the DMMA pipe busy.
    const bool load_first = (warp >> 3) == 0;
    for (int ch = 0; ch < NCH; ++ch) {
        cp_async_wait<0>();
        mbar_wait(&w_bar[ch & 1], (ch >> 1) & 1);       // stage ch % 2 is on its (ch / 2)-th use
        __syncthreads();
        if (load_first && ch + 1 < NCH) load_stage((ch + 1) & 1, ch + 1);
        if (all_rows) compute(ch, std::true_type{});
        else compute(ch, std::false_type{});
        if (!load_first && ch + 1 < NCH) load_stage((ch + 1) & 1, ch + 1);
        cp_async_commit();
    }
    cp_async_wait<0>();
    if (Vout == nullptr && p.pack != nullptr) {
        // Compact output only: straight from the accumulators.  A lane holds two neighbouring channels of a
        // (column, patch row), so its store is 16 bytes; the four lanes of a quad fill the 64 bytes of an
        // 8-channel group, whole sectors of the channel-fastest output without a pass through shared memory.
        const int nn = wn * 8 + 2 * t;
        if (n0 + nn < p.g.Cout) {
            const double r0 = chan[nn], s0 = chan[BN + nn], r1 = chan[nn + 1], s1 = chan[BN + nn + 1];
            const int64_t ca = j0 + wm * 16 + g, cb = ca + 8;
            double* da = p.pack + ca * p.pack_stride + int64_t(owl * p.wh_out + ohb * CW_TH) * p.g.Cout + n0 + nn;
            double* db = da + 8 * p.pack_stride;
#pragma unroll
            for (int o = 0; o < CW_TH; ++o) {
                if (o >= th_cnt) break;
                if (ca < ncols)
                    *reinterpret_cast<double2*>(da + int64_t(o) * p.g.Cout) =
                        make_double2((acc[o][0] * r0) * s0, (acc[o][1] * r1) * s1);
                if (cb < ncols)
                    *reinterpret_cast<double2*>(db + int64_t(o) * p.g.Cout) =
                        make_double2((acc[o][2] * r0) * s0, (acc[o][3] * r1) * s1);
            }
        }
        return;
    }
    __syncthreads();        // every warp is done with the stages: they become the output staging area

    // epilogue 1: accumulators -> staging [column][patch row][channel]; 16-byte stores
    double* out_s = smem;
    {
        const int c_lo = wm * 16 + g;
#pragma unroll
        for (int o = 0; o < CW_TH; ++o) {
            const int nn = wn * 8 + 2 * t;
            const double r0 = chan[nn], s0 = chan[BN + nn], r1 = chan[nn + 1], s1 = chan[BN + nn + 1];
            double2 lo2 = make_double2((acc[o][0] * r0) * s0, (acc[o][1] * r1) * s1);
            double2 hi2 = make_double2((acc[o][2] * r0) * s0, (acc[o][3] * r1) * s1);
            *reinterpret_cast<double2*>(out_s + c_lo * p.CSTR + o * p.OSTR + nn) = lo2;
            *reinterpret_cast<double2*>(out_s + (c_lo + 8) * p.CSTR + o * p.OSTR + nn) = hi2;
        }
    }
    __syncthreads();
    // epilogue 2: staging -> memory; 8 lanes write the 8 patch rows of one (column, channel): 64 contiguous bytes
    // (skipped when the launch keeps its output in compact form only)
    if (Vout != nullptr) {
        const int o = lane & 7;
        const int sub = lane >> 3;
        const int64_t hw_out = int64_t(p.g.Ho) * p.g.Wo;
        const int n_pairs = p.ncol * BN;
        for (int base = warp * 4; base < n_pairs; base += (CW_THREADS / 32) * 4) {
            const int pair = base + sub;
            const int col = pair / BN, n = pair % BN;
            if (j0 + col >= ncols || n0 + n >= p.g.Cout || o >= th_cnt) continue;
            const int4 bx = s_box[col];
            const int oh = bx.x + p.g.pad_t - ext_h + ohb * CW_TH + o;
            const int ow = bx.y + p.g.pad_l - ext_w + owl;
            if (oh < 0 || oh >= p.g.Ho || ow < 0 || ow >= p.g.Wo) continue;
            Vout[(col_base + j0 + col) * ld_out + oh + int64_t(p.g.Ho) * ow + hw_out * (n0 + n)] =
                out_s[col * p.CSTR + o * p.OSTR + n];
        }
    }
    // epilogue 3 (in front of a ReLU layer): the same tile into the window-only copy the bound reduction reads;
    // a warp writes the channels of one (column, patch row): contiguous in the copy and in the staging area
    if (p.pack != nullptr) {
        constexpr int LPR = BN / 2;          // lanes per (column, patch row), two channels each
        constexpr int RPI = 32 / LPR;        // (column, patch row) pairs per warp instruction
        const int items = p.ncol * th_cnt;
        const int n = 2 * (lane % LPR);
        for (int it = warp * RPI + lane / LPR; it < items; it += (CW_THREADS / 32) * RPI) {
            const int o = it % th_cnt, col = it / th_cnt;
            if (j0 + col >= ncols || n0 + n >= p.g.Cout) continue;
            const double2 v = *reinterpret_cast<const double2*>(out_s + col * p.CSTR + o * p.OSTR + n);
            double* dst = p.pack + (j0 + col) * p.pack_stride +
                          int64_t(owl * p.wh_out + ohb * CW_TH + o) * p.g.Cout + n0 + n;
            if (n0 + n + 1 < p.g.Cout) *reinterpret_cast<double2*>(dst) = v;     // Cout is even: 16-byte aligned
            else dst[0] = v.x;
        }
    }
}


// 4-byte async copy; src_bytes = 0 writes zero.
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem, int src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(src_bytes));
}

template <int KH, int WARPS_M, int WARPS_N, bool CIN, int NROWS = 0>
int launch_cfg(cudaStream_t st, const ConvGeom& g, const ConvWeights& w, const ChanAffine& bn, const RowMask& mask,
               const ColWindows& win, int wh_in, int ww_in, int64_t col_base, const double* Vin, int64_t ld_in,
               double* Vout, int64_t ld_out, int64_t ncols, double* pack, const double* cin, int64_t cin_stride,
               bool* done) {
    constexpr int BN = WARPS_N * 8;
    ConvWinParams p;
    p.g = g;
    p.cin = cin;
    p.cin_stride = cin_stride;
    if (Vout == nullptr && (pack == nullptr || g.Cout % 2 != 0)) return NNVB_OK;     // nowhere to write
    if (CIN && (int64_t(16 * WARPS_M) * cin_stride >= (int64_t(1) << 31) || g.Cin % 2 != 0 || cin_stride % 2 != 0 ||
                (reinterpret_cast<uintptr_t>(cin) & 15) != 0))
        return NNVB_OK;
    p.pack = g.Cout % 2 == 0 ? pack : nullptr;
    p.pack_stride = int64_t(win.wh) * win.ww * g.Cout;
    p.wh_in = wh_in; p.ww_in = ww_in;
    p.wh_out = win.wh; p.ww_out = win.ww;
    p.n_ohb = (int)ceil_div(win.wh, CW_TH);
    p.ni_s = std::min(wh_in, CW_TH + KH - 1);
    p.ncol = 16 * WARPS_M;
    p.CSI = p.ncol + 4;             // = 4 (mod 16): the four channel rows of a fragment fall on distinct banks
    p.CS = w.cs;
    p.RS = KC * p.CSI + 1;
    p.in_stage = CIN ? g.kw * p.ni_s * p.ncol * KC
                     : (g.kw * p.ni_s * p.RS + 1) / 2 * 2;  // even: the weights behind it are fetched 16 bytes at a time
    p.w_stage = g.kh * g.kw * KC * p.CS;
    p.n_chunks = w.n_chunks;
    p.OSTR = BN + 2;
    p.CSTR = CW_TH * p.OSTR + 8;
    if (p.CSTR % 16 != 8) p.CSTR += (8 - p.CSTR % 16 + 16) % 16;
    p.tab_cap = p.ncol * g.kw * p.ni_s;
    // the output staging area reuses the pipeline stages; the constants and tables follow the larger of the two
    const size_t pipe = size_t(CW_STAGES) * (p.in_stage + p.w_stage) * sizeof(double);
    const size_t stage_out = size_t(p.ncol) * p.CSTR * sizeof(double);
    p.tail = int(std::max(pipe, stage_out) / sizeof(double));
    const size_t smem = std::max(pipe, stage_out) + size_t(2 * BN) * sizeof(double) +
                        size_t(3 * p.tab_cap) * sizeof(int) + size_t(p.ncol) * sizeof(int4);
    if (smem > CW_SMEM_LIMIT) return NNVB_OK;
    if (int64_t(p.ncol) * std::max(ld_in, ld_out) >= (int64_t(1) << 31)) return NNVB_OK;
    const int64_t blocks = ceil_div(ncols, p.ncol) * p.ww_out * p.n_ohb;
    if (blocks >= (int64_t(1) << 31)) return NNVB_OK;
    if (NROWS > 0 && (p.n_ohb != 1 || wh_in != NROWS)) return NNVB_OK;
    auto kern = conv_win_kernel<KH, WARPS_M, WARPS_N, CIN, NROWS>;
    NNVB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)blocks, (unsigned)w.n_tiles);
    kern<<<grid, CW_THREADS, smem, st>>>(p, w.w, bn, mask, win.box, col_base, Vin, ld_in, Vout, ld_out, ncols);
    NNVB_CUDA(cudaGetLastError());
    *done = true;
    return NNVB_OK;
}


// Persistent, warp-specialised form of the compact-input, compact-output case (the hot one).  One block per SM walks
// the tiles with stride gridDim.x and treats (tile, channel chunk) pairs as ONE pipelined sequence, so the start-up
// of a tile (window boxes, flags, fetch table, first stage) runs underneath the products of the tile before it
// instead of in front of an idle DMMA pipe.  Sixteen consumer warps (four warpgroups) only multiply: they wait for a
// stage to be full, run its products, and hand the stage back; results leave straight from the accumulators
// (16-byte stores), so shared memory is never reused as an output staging area.  One producer warpgroup (four
// warps) does everything else: while tile t is multiplied it requests the boxes and query numbers of tile t+1's
// columns (chunk 0), derives tile t+1's flags and fetch table from them (chunk 1), and fills every stage — the input
// copies and the weight copy.  Stages are handed over through mbarriers (full: the producer's copies have landed;
// empty: all consumer warps are done with the stage), so there is no block-wide barrier in the main loop and a
// consumer warp never waits for another consumer warp.  The producers give most of their registers to the
// consumers.  The form needs three chunks per tile at least (the table of tile t+1 is built during chunk 1 of tile
// t and first used for its last chunk).  Every wait is bounded; a wait that runs out sets *err and lets the kernel
// finish.
constexpr int WS_CONSUMER_WARPS = 16;
constexpr int WS_PRODUCERS = 128;                                   // threads of the producer warpgroup
constexpr int WS_THREADS = WS_CONSUMER_WARPS * 32 + WS_PRODUCERS;   // 640
constexpr int WS_BAR_PRODUCERS = 1;                                 // named barrier of the producer warps

template <int KH, int WARPS_M, int WARPS_N, int NROWS>
__global__ void __launch_bounds__(WS_THREADS, 1)
conv_win_ws_kernel(const ConvWinParams p, const double* __restrict__ Wg, const ChanAffine bn, const RowMask mask,
                   const int4* __restrict__ box, int64_t col_base, int64_t ncols, int* __restrict__ err) {
    static_assert(WARPS_M * WARPS_N == WS_CONSUMER_WARPS, "16 consumer warps");
    constexpr int BN = WARPS_N * 8;
    constexpr int NI = CW_TH + KH - 1;

    extern __shared__ __align__(16) double smem[];
    const int S = p.stages;                                     // 2 to 4 pipeline stages, as many as fit
    double* in_s = smem;                                        // [S][in_stage]
    double* wts = smem + S * p.in_stage;                        // [S][w_stage]
    // fetch tables, [2 buffers][goff | soff | moff, or the row-state bits (two ints per entry)][tab_cap]
    int* tab = reinterpret_cast<int*>(smem + p.tail);
    int4* s_box = reinterpret_cast<int4*>(tab + 8 * p.tab_cap); // [2][ncol]
    int* s_q = reinterpret_cast<int*>(s_box + 2 * p.ncol);      // [2][ncol] query of the column
    unsigned* s_rows = reinterpret_cast<unsigned*>(s_q + 2 * p.ncol);   // [2][WARPS_M] patch rows on the image
    int* s_on = reinterpret_cast<int*>(s_rows + 2 * WARPS_M);   // [2] some column of the tile has its patch column on the image
    __shared__ __align__(8) uint64_t full_bar[CW_MAX_STAGES], empty_bar[CW_MAX_STAGES];
    __shared__ int s_abort;             // raised by the first wait that runs out: every role then leaves its loop

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int H = p.g.H, W = p.g.W;
    const int KW = p.g.kw;
    const int ext_h = KH - 1, ext_w = KW - 1;
    const int per = p.ww_out * p.n_ohb;
    const int NCH = p.n_chunks;

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < CW_MAX_STAGES; ++s) {
            mbar_init(&full_bar[s], WS_PRODUCERS + 1);      // every producer thread's copies, and the weight copy
            mbar_init(&empty_bar[s], WS_CONSUMER_WARPS);    // one arrival per consumer warp
        }
        mbar_init_fence();
    }
    __syncthreads();

    struct Tile { int n_tile, owl, ohb; int64_t j0; };
    auto decode = [&](int tile) {        // the tile count fits 31 bits (checked at launch)
        Tile x;
        x.n_tile = tile % p.n_ytiles;
        const int r = tile / p.n_ytiles;
        x.j0 = int64_t(r / per) * p.ncol;
        const int rem = r % per;
        x.owl = rem / p.n_ohb;
        x.ohb = rem % p.n_ohb;
        return x;
    };
    auto i_lo_of = [&](int ohb) { return NROWS > 0 ? KH - 1 : max(0, ext_h - ohb * CW_TH); };
    auto i_hi_of = [&](int ohb) { return NROWS > 0 ? KH - 1 + NROWS : min(NI, p.wh_in - (ohb * CW_TH - ext_h)); };
    auto kw_lo_of = [&](int owl) { return max(0, ext_w - owl); };
    auto kw_hi_of = [&](int owl) { return min(KW, p.ww_in + ext_w - owl); };

    if (warp >= WS_CONSUMER_WARPS) {
        // ------------------------------------------------------------------ producer warpgroup
        // the block owns 640 x 96 registers: 128 x 32 for the producers leave 512 x 112 for the consumers
        setmaxnreg_dec<32>();
        const int ptid = tid - WS_CONSUMER_WARPS * 32;
        const bool cf = mask.state_cf != nullptr;
        const bool pair_ok = cf && (p.g.Cin % 2 == 0) && (mask.N % 2 == 0);
        const int hw_in = H * W;

        // boxes and query numbers of a tile's columns into buffer b (async copies)
        auto prep_boxes = [&](const Tile& x, int b) {
            if (ptid < p.ncol) {
                const bool ok = x.j0 + ptid < ncols;
                cp_async16(&s_box[b * p.ncol + ptid], ok ? box + col_base + x.j0 + ptid : box, ok ? 16 : 0);
            } else if (ptid < 2 * p.ncol) {
                const int c = ptid - p.ncol;
                const int64_t gj = col_base + x.j0 + c;
                const bool ok = mask.state != nullptr && x.j0 + c < ncols && gj < mask.ncols;
                cp_async4(&s_q[b * p.ncol + c], ok ? static_cast<const void*>(mask.col_q + gj) : static_cast<const void*>(box),
                          ok ? 4 : 0);
            }
        };
        // flags and fetch table of the tile whose boxes are in buffer b
        auto prep_table = [&](const Tile& x, int b) {
            const int th_cnt = min(CW_TH, p.wh_out - x.ohb * CW_TH);
            // Patches near the image border hang over it: a tile none of whose columns has its patch column on the
            // image has nothing to do, and a consumer warp skips the patch rows that are off the image for its 16
            // columns.  Producer warp w works out the flags of column group w (of WARPS_M <= 4).
            const int pw = ptid >> 5;
            if (pw < WARPS_M) {
                unsigned m = 0u;
                if (lane < 16) {
                    const int c = pw * 16 + lane;
                    if (x.j0 + c < ncols) {
                        const int4 bx = s_box[b * p.ncol + c];
                        const int ow = bx.y + p.g.pad_l - ext_w + x.owl;
                        if (ow >= 0 && ow < p.g.Wo) {
                            m = 1u << 31;                       // the patch column is on the image
                            for (int o = 0; o < th_cnt; ++o) {
                                const int oh = bx.x + p.g.pad_t - ext_h + x.ohb * CW_TH + o;
                                if (oh >= 0 && oh < p.g.Ho) m |= 1u << o;
                            }
                        }
                    }
                }
                m = __reduce_or_sync(0xffffffffu, m);
                if (lane == 0) s_rows[b * WARPS_M + pw] = m;
            }
            named_bar_sync(WS_BAR_PRODUCERS, WS_PRODUCERS);
            unsigned any = 0u;
            for (int i = 0; i < WARPS_M; ++i) any |= s_rows[b * WARPS_M + i];
            const bool on = (any >> 31) != 0u;
            if (ptid == 0) s_on[b] = on ? 1 : 0;
            if (!on) return;
            const int ih_base = x.ohb * CW_TH - ext_h;
            const int i_lo = i_lo_of(x.ohb), n_i = i_hi_of(x.ohb) - i_lo;
            const int kw_lo = kw_lo_of(x.owl), n_kw = kw_hi_of(x.owl) - kw_lo;
            const int n_e = p.ncol * n_kw * n_i;
            int* goff = tab + b * 4 * p.tab_cap;
            int* soff = goff + p.tab_cap;
            int* moff = soff + p.tab_cap;
            unsigned long long* mbits = reinterpret_cast<unsigned long long*>(moff);
            // entry e = (origin column, input row, column), column fastest: neighbouring lanes of the fetch write
            // neighbouring 64-byte slots of the staging row
            for (int e = ptid; e < n_e; e += WS_PRODUCERS) {
                const int col = e % p.ncol;
                const int e2 = e / p.ncol;
                const int i_idx = e2 % n_i;
                const int kwi = kw_lo + e2 / n_i;
                const int4 bx = s_box[b * p.ncol + col];
                const int hi = bx.x + ih_base + i_lo + i_idx;
                const int wi = bx.y + x.owl + kwi - ext_w;
                int off = -1, mo = -1;
                if (hi >= 0 && hi < H && wi >= 0 && wi < W && x.j0 + col < ncols) {
                    off = int(col * p.cin_stride) + ((wi - bx.y) * p.wh_in + (hi - bx.x)) * p.g.Cin;
                    if (mask.state != nullptr && col_base + x.j0 + col < mask.ncols) {
                        const int q_off = int(s_q[b * p.ncol + col] * mask.N);
                        mo = cf ? q_off + (hi + H * wi) * p.g.Cin : q_off + hi + H * wi;
                    }
                }
                goff[e] = off;
                soff[e] = (((kwi * p.ni_s + i_idx) * p.ncol + col) * KC) | (((col >> 1) & 1) << 30);
                if (!p.use_bits) {
                    moff[e] = mo;
                    continue;
                }
                // the entry's row states, one bit per channel (bit c: channel c was cleared by the ReLU step): read
                // here once per tile instead of once per channel chunk, so that filling a stage depends on no
                // global load
                unsigned long long mb = 0ull;
                if (mo >= 0) {
                    const uint8_t* sp = mask.state_cf + mo;
                    if ((p.g.Cin & 7) == 0 && (reinterpret_cast<uintptr_t>(sp) & 7) == 0) {
                        for (int w8 = 0; w8 < p.g.Cin / 8; ++w8) {
                            const unsigned long long v = *reinterpret_cast<const unsigned long long*>(sp + 8 * w8);
                            // high bit of every non-zero byte, then the eight bits gathered into one byte
                            const unsigned long long y =
                                (((v & 0x7f7f7f7f7f7f7f7full) + 0x7f7f7f7f7f7f7f7full) | v) & 0x8080808080808080ull;
                            mb |= (((y >> 7) * 0x0102040810204080ull) >> 56) << (8 * w8);
                        }
                    } else {
                        for (int c = 0; c < p.g.Cin; ++c) mb |= (unsigned long long)(sp[c] != 0) << c;
                    }
                }
                mbits[e] = mb;
            }
        };
        // one stage of a tile: the chunk's weights by one bulk copy (a contiguous block; its bytes are counted on the
        // stage's full barrier), the inputs by 16-byte copies, one channel pair of one (column, input position) each
        auto fill_stage = [&](int stage, const Tile& x, int b, int chunk) {
            if (ptid == 0) {
                mbar_expect_bytes(&full_bar[stage], uint32_t(p.w_stage) * 8u);
                bulk_copy_g2s(wts + stage * p.w_stage, Wg + (int64_t(x.n_tile) * p.n_chunks + chunk) * p.w_stage,
                              uint32_t(p.w_stage) * 8u, &full_bar[stage]);
            }
            if (s_on[b]) {
                const int n_e = p.ncol * (kw_hi_of(x.owl) - kw_lo_of(x.owl)) * (i_hi_of(x.ohb) - i_lo_of(x.ohb));
                const int* goff = tab + b * 4 * p.tab_cap;
                const int* soff = goff + p.tab_cap;
                const int* moff = soff + p.tab_cap;
                const unsigned long long* mbits = reinterpret_cast<const unsigned long long*>(moff);
                double* is = in_s + stage * p.in_stage;
                const int c0 = chunk * KC;
                const double* src_b = p.cin + x.j0 * p.cin_stride + c0;
                for (int it = ptid; it < 4 * n_e; it += WS_PRODUCERS) {
                    const int e = it >> 2, u0 = 2 * (it & 3);
                    const int off = goff[e], so_raw = soff[e];
                    const int so = so_raw & 0x3fffffff;
                    const int sw = (so_raw >> 30) & 1 ? 4 : 0;
                    bool ok0 = off >= 0 && c0 + u0 < p.g.Cin, ok1 = off >= 0 && c0 + u0 + 1 < p.g.Cin;
                    const int mo = p.use_bits ? -1 : moff[e];
                    if (p.use_bits) {                                // rows the ReLU step cleared read as zero
                        const unsigned two = unsigned(mbits[e] >> (c0 + u0)) & 3u;
                        ok0 = ok0 && (two & 1u) == 0;
                        ok1 = ok1 && (two & 2u) == 0;
                    } else if (mo >= 0 && (ok0 || ok1)) {
                        if (pair_ok) {
                            const unsigned sv = *reinterpret_cast<const unsigned short*>(mask.state_cf + mo + c0 + u0);
                            ok0 = ok0 && (sv & 0xffu) == 0;
                            ok1 = ok1 && (sv >> 8) == 0;
                        } else {
                            if (ok0) ok0 = (cf ? mask.state_cf[mo + c0 + u0] : mask.state[mo + int64_t(c0 + u0) * hw_in]) == 0;
                            if (ok1) ok1 = (cf ? mask.state_cf[mo + c0 + u0 + 1] : mask.state[mo + int64_t(c0 + u0 + 1) * hw_in]) == 0;
                        }
                    }
                    double* d2 = is + so + (u0 ^ sw);
                    if (ok0 && ok1) {
                        cp_async16(d2, src_b + off + u0, 16);
                    } else {
                        cp_async8(d2, ok0 ? src_b + off + u0 : p.cin, ok0 ? 8 : 0);
                        cp_async8(d2 + 1, ok1 ? src_b + off + u0 + 1 : p.cin, ok1 ? 8 : 0);
                    }
                }
            }
            cp_async_arrive_on(&full_bar[stage]);       // this thread's part of the stage has landed
        };

        int tile = blockIdx.x;
        Tile cx = decode(tile), nx = cx;
        int buf = 0;
        prep_boxes(cx, 0);
        cp_async_wait_all();
        named_bar_sync(WS_BAR_PRODUCERS, WS_PRODUCERS);
        prep_table(cx, 0);
        named_bar_sync(WS_BAR_PRODUCERS, WS_PRODUCERS);
        int stage = 0;                  // the (tile, chunk) sequence walks the stages round robin;
        unsigned use = 0;               // use = how often the current stage has been filled before
        for (;;) {
            const int64_t next = int64_t(tile) + gridDim.x;
            const bool has_next = next < p.n_flat;
            if (has_next) nx = decode(int(next));
            for (int ch = 0; ch < NCH; ++ch) {
                // the consumers have left the stage (its previous use); passes at once on a stage's first use
                // (a wait that ran out raises the abort flag; the producers then run through the remaining items
                // without waiting, so that all four warps still meet at their named barriers, and the consumers leave)
                if (!mbar_wait_or_abort(&empty_bar[stage], (use & 1) ^ 1, &s_abort)) atomicExch(err, 1);
                fill_stage(stage, cx, buf, ch);
                if (++stage == S) { stage = 0; ++use; }
                // the next tile's start-up, spread over this tile's first chunks
                if (has_next && ch == 0) prep_boxes(nx, buf ^ 1);
                if (has_next && ch == 1) {
                    cp_async_wait_all();
                    named_bar_sync(WS_BAR_PRODUCERS, WS_PRODUCERS);
                    prep_table(nx, buf ^ 1);
                    named_bar_sync(WS_BAR_PRODUCERS, WS_PRODUCERS);
                }
            }
            if (!has_next) break;
            tile = int(next);
            cx = nx;
            buf ^= 1;
        }
        cp_async_wait_all();
        return;
    }
    // ---------------------------------------------------------------------- consumer warps
    setmaxnreg_inc<112>();
    const int wm = warp % WARPS_M;
    const int wn = warp / WARPS_M;
    const int g = lane >> 2;
    const int t = lane & 3;

    double acc[CW_TH][4];
#pragma unroll
    for (int o = 0; o < CW_TH; ++o)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[o][r] = 0.0;

    int tile = blockIdx.x;
    Tile cx = decode(tile);
    int buf = 0;
    int kw_lo = 0, kw_hi = 0, i_lo = 0, i_hi = 0;
    unsigned rows_on = 0u;
    bool all_rows = false, tile_on = false;
    auto enter_tile = [&]() {           // reads the flags the producers left in buffer buf (behind the full barrier)
        kw_lo = kw_lo_of(cx.owl); kw_hi = kw_hi_of(cx.owl);
        i_lo = i_lo_of(cx.ohb); i_hi = i_hi_of(cx.ohb);
        tile_on = s_on[buf] != 0;
        rows_on = tile_on ? (s_rows[buf * WARPS_M + wm] & 0xffu) : 0u;
        if (rows_on == 0u) kw_hi = kw_lo;         // nothing of this warp's columns is on the image
        const unsigned row_bits = (1u << min(CW_TH, p.wh_out - cx.ohb * CW_TH)) - 1u;
        all_rows = (rows_on & row_bits) == row_bits;
    };

    // FULL: every patch row of the tile is on the image for this warp's columns (the common case): the products
    // carry no per-row test, which would otherwise put a branch around every DMMA
    auto compute = [&](int stage, auto full_rows) {
        constexpr bool FULL = decltype(full_rows)::value;
        // row = column g (and g + 8), k = channel t (and t + 4); the channel index is XORed with 4 for every other
        // column pair (the staging swizzle)
        const int sw = ((g >> 1) & 1) * 4;
        const double* is = in_s + stage * p.in_stage + (wm * 16 + g) * KC;
        const int RSr = p.ncol * KC;                                                // stride between staged input rows
        constexpr int o1 = 8 * KC;
        const int o0 = t ^ sw, o2 = (o0 ^ 4) - o0;
        const double* ws = wts + stage * p.w_stage + t * p.CS + wn * 8 + g;         // k = channel t, n = g
        for (int kwi = kw_lo; kwi < kw_hi; ++kwi) {
            double bf[KH][2];
#pragma unroll
            for (int khi = 0; khi < KH; ++khi) {
                const double* wt = ws + (khi + KH * kwi) * (KC * p.CS);     // tap index: kh fastest
                bf[khi][0] = wt[0];
                bf[khi][1] = wt[4 * p.CS];
            }
            const double* a_col = is + (kwi * p.ni_s - i_lo) * RSr + o0;
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                if (i < i_lo || i >= i_hi) continue;
                const double* a = a_col + i * RSr;
                double af[4];
                af[0] = a[0];
                af[1] = a[o1];
                af[2] = a[o2];
                af[3] = a[o2 + o1];
                // input row i meets output row i - khi through tap khi
#pragma unroll
                for (int khi = 0; khi < KH; ++khi) {
                    const int o = i - khi;
                    if (o >= 0 && o < CW_TH) {
                        if (FULL || ((rows_on >> o) & 1u)) dmma_16x8x8(acc[o], af, bf[khi]);
                    }
                }
            }
        }
    };

    // results of the finished tile: a lane holds two neighbouring channels of a (column, patch row), so its store is
    // 16 bytes; the four lanes of a quad fill the 64 bytes of an 8-channel group of the channel-fastest output
    auto store_tile = [&]() {
        const int th_cnt = min(CW_TH, p.wh_out - cx.ohb * CW_TH);
        const int co = cx.n_tile * BN + wn * 8 + 2 * t;
        if (tile_on && co < p.g.Cout) {
            const bool has_bn = bn.rden != nullptr;
            const double r0 = has_bn ? bn.rden[co] : 1.0, s0 = has_bn ? bn.scale[co] : 1.0;
            const double r1 = has_bn ? bn.rden[co + 1] : 1.0, s1 = has_bn ? bn.scale[co + 1] : 1.0;
            const int64_t ca = cx.j0 + wm * 16 + g, cb = ca + 8;
            double* da = p.pack + ca * p.pack_stride + int64_t(cx.owl * p.wh_out + cx.ohb * CW_TH) * p.g.Cout + co;
            double* db = da + 8 * p.pack_stride;
#pragma unroll
            for (int o = 0; o < CW_TH; ++o) {
                if (o >= th_cnt) break;
                if (ca < ncols)
                    *reinterpret_cast<double2*>(da + int64_t(o) * p.g.Cout) =
                        make_double2((acc[o][0] * r0) * s0, (acc[o][1] * r1) * s1);
                if (cb < ncols)
                    *reinterpret_cast<double2*>(db + int64_t(o) * p.g.Cout) =
                        make_double2((acc[o][2] * r0) * s0, (acc[o][3] * r1) * s1);
            }
        }
#pragma unroll
        for (int o = 0; o < CW_TH; ++o)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[o][r] = 0.0;
    };

    int stage = 0;
    unsigned use = 0;
    for (;;) {
        for (int ch = 0; ch < NCH; ++ch) {
            if (!mbar_wait_or_abort(&full_bar[stage], use & 1, &s_abort)) {
                atomicExch(err, 1);
                return;
            }
            if (ch == 0) enter_tile();
            if (all_rows) compute(stage, std::true_type{});
            else compute(stage, std::false_type{});
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);      // this warp is done with the stage
            if (++stage == S) { stage = 0; ++use; }
        }
        store_tile();
        const int64_t next = int64_t(tile) + gridDim.x;
        if (next >= p.n_flat) break;
        tile = int(next);
        cx = decode(tile);
        buf ^= 1;
    }
}

int sm_count_of_current_device() {
    static int cached_dev = -1, cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached = n;
        cached_dev = dev;
    }
    return cached;
}

// set by the warp-specialised kernel when one of its bounded waits ran out (read by conv_win_wait_timeouts)
__device__ int g_ws_wait_timeout = 0;

template <int KH, int WARPS_M, int WARPS_N, int NROWS>
int launch_persist(cudaStream_t st, const ConvGeom& g, const ConvWeights& w, const ChanAffine& bn, const RowMask& mask,
                   const ColWindows& win, int wh_in, int ww_in, int64_t col_base, int64_t ncols, double* pack,
                   const double* cin, int64_t cin_stride, bool* done) {
    constexpr int BN = WARPS_N * 8;
    ConvWinParams p;
    p.g = g;
    p.cin = cin;
    p.cin_stride = cin_stride;
    if (int64_t(16 * WARPS_M) * cin_stride >= (int64_t(1) << 31) || g.Cin % 2 != 0 || cin_stride % 2 != 0 ||
        (reinterpret_cast<uintptr_t>(cin) & 15) != 0)
        return NNVB_OK;
    p.pack = pack;
    p.pack_stride = int64_t(win.wh) * win.ww * g.Cout;
    p.wh_in = wh_in; p.ww_in = ww_in;
    p.wh_out = win.wh; p.ww_out = win.ww;
    p.n_ohb = (int)ceil_div(win.wh, CW_TH);
    if (NROWS > 0 && (p.n_ohb != 1 || wh_in != NROWS)) return NNVB_OK;
    p.ni_s = std::min(wh_in, CW_TH + KH - 1);
    p.ncol = 16 * WARPS_M;
    p.CSI = 0; p.RS = 0; p.OSTR = 0; p.CSTR = 0;
    p.CS = w.cs;
    p.in_stage = g.kw * p.ni_s * p.ncol * KC;
    p.w_stage = g.kh * g.kw * KC * p.CS;
    p.n_chunks = w.n_chunks;
    p.tab_cap = p.ncol * g.kw * p.ni_s;
    p.n_ytiles = w.n_tiles;
    p.n_flat = ceil_div(ncols, p.ncol) * p.ww_out * p.n_ohb * w.n_tiles;
    if (p.n_flat >= (int64_t(1) << 31)) return NNVB_OK;
    p.use_bits = g.Cin <= 64 && (mask.state == nullptr || mask.state_cf != nullptr);
    // two to four stages, as many as fit beside the tables (four ints per table entry and buffer, the tiles' boxes,
    // query numbers and flags): where the stages are small the producers run further ahead of the consumers
    const size_t stage_bytes = size_t(p.in_stage + p.w_stage) * sizeof(double);
    const size_t fixed = size_t(8 * p.tab_cap) * sizeof(int) + size_t(2 * p.ncol) * (sizeof(int4) + sizeof(int)) +
                         size_t(2 * (CW_THREADS / 32) + 4) * sizeof(int);
    if (fixed + 2 * stage_bytes > CW_SMEM_LIMIT) return NNVB_OK;
    p.stages = int(std::min<size_t>(CW_MAX_STAGES, (CW_SMEM_LIMIT - fixed) / stage_bytes));
    p.tail = p.stages * (p.in_stage + p.w_stage);
    const size_t smem = fixed + p.stages * stage_bytes;
    const unsigned grid = (unsigned)std::min<int64_t>(p.n_flat, sm_count_of_current_device());
    static int* err = nullptr;
    if (err == nullptr) NNVB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&err), g_ws_wait_timeout));
    auto kern = conv_win_ws_kernel<KH, WARPS_M, WARPS_N, NROWS>;
    NNVB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, WS_THREADS, smem, st>>>(p, w.w, bn, mask, win.box, col_base, ncols, err);
    NNVB_CUDA(cudaGetLastError());
    *done = true;
    return NNVB_OK;
}

}  // namespace

// Number of launches of the warp-specialised kernel since the last call in which a bounded wait ran out (0 in a
// healthy run); synchronises the stream.
int conv_win_wait_timeouts(cudaStream_t st, int* out) {
    int v = 0;
    static const int zero = 0;
    NNVB_CUDA(cudaMemcpyFromSymbolAsync(&v, g_ws_wait_timeout, sizeof(int), 0, cudaMemcpyDeviceToHost, st));
    NNVB_CUDA(cudaStreamSynchronize(st));
    if (v != 0) NNVB_CUDA(cudaMemcpyToSymbolAsync(g_ws_wait_timeout, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, st));
    *out = v;
    return NNVB_OK;
}

// Windowed convolution with tap skipping.  *done is set when the launch was made; it stays false (and
// nothing is launched) for geometries this kernel does not cover: the caller then uses launch_conv_f64.
int launch_conv_win(cudaStream_t st, const ConvGeom& g, const ConvWeights& w, const ChanAffine& bn, const RowMask& mask,
                    const ColWindows& win, int wh_in, int ww_in, int64_t col_base, const double* Vin, int64_t ld_in,
                    double* Vout, int64_t ld_out, int64_t ncols, double* pack, bool* done, int64_t* launches,
                    const double* cin, int64_t cin_stride) {
    *done = false;
    if (ncols <= 0) { *done = true; return NNVB_OK; }
    if (g.sh != 1 || g.sw != 1 || g.dh != 1 || g.dw != 1 || g.kh != 3 || g.kw > 7 || win.box == nullptr) return NNVB_OK;
    if (win.wh != wh_in + g.kh - 1 || win.ww != ww_in + g.kw - 1) return NNVB_OK;
    int rc = NNVB_OK;
    // compact input, compact output, three channel chunks or more: the persistent form
    static const bool no_persist = getenv("NNVB_NO_PERSIST") != nullptr;
    if (!no_persist && cin != nullptr && Vout == nullptr && pack != nullptr && g.Cout % 2 == 0 && w.n_chunks >= 3 &&
        (w.bn_tile == 64 || w.bn_tile == 32)) {
#define NNVB_CP_ARGS st, g, w, bn, mask, win, wh_in, ww_in, col_base, ncols, pack, cin, cin_stride, done
        const int prow = (wh_in >= 3 && wh_in <= 6 && win.wh <= CW_TH) ? wh_in : 0;
        if (w.bn_tile == 64) {
            switch (prow) {
                case 3: rc = launch_persist<3, 2, 8, 3>(NNVB_CP_ARGS); break;
                case 4: rc = launch_persist<3, 2, 8, 4>(NNVB_CP_ARGS); break;
                case 5: rc = launch_persist<3, 2, 8, 5>(NNVB_CP_ARGS); break;
                case 6: rc = launch_persist<3, 2, 8, 6>(NNVB_CP_ARGS); break;
                default: rc = launch_persist<3, 2, 8, 0>(NNVB_CP_ARGS);
            }
        } else {
            switch (prow) {
                case 3: rc = launch_persist<3, 4, 4, 3>(NNVB_CP_ARGS); break;
                case 4: rc = launch_persist<3, 4, 4, 4>(NNVB_CP_ARGS); break;
                case 5: rc = launch_persist<3, 4, 4, 5>(NNVB_CP_ARGS); break;
                case 6: rc = launch_persist<3, 4, 4, 6>(NNVB_CP_ARGS); break;
                default: rc = launch_persist<3, 4, 4, 0>(NNVB_CP_ARGS);
            }
        }
#undef NNVB_CP_ARGS
        if (rc != NNVB_OK) return rc;
        if (*done) {
            if (launches) *launches += 1;
            return NNVB_OK;
        }
    }
#define NNVB_CW_ARGS st, g, w, bn, mask, win, wh_in, ww_in, col_base, Vin, ld_in, Vout, ld_out, ncols, pack, cin, cin_stride, done
    // window heights 3 to 6 with one row block (the windows of the first layers behind an input or a ReLU layer)
    // have their own instances of the compact-input kernel
    const int rows = (cin != nullptr && wh_in >= 3 && wh_in <= 6 && win.wh <= CW_TH) ? wh_in : 0;
    if (w.bn_tile == 64 && cin != nullptr) {
        switch (rows) {
            case 3: rc = launch_cfg<3, 2, 8, true, 3>(NNVB_CW_ARGS); break;
            case 4: rc = launch_cfg<3, 2, 8, true, 4>(NNVB_CW_ARGS); break;
            case 5: rc = launch_cfg<3, 2, 8, true, 5>(NNVB_CW_ARGS); break;
            case 6: rc = launch_cfg<3, 2, 8, true, 6>(NNVB_CW_ARGS); break;
            default: rc = launch_cfg<3, 2, 8, true>(NNVB_CW_ARGS);
        }
    } else if (w.bn_tile == 64) {
        rc = launch_cfg<3, 2, 8, false>(NNVB_CW_ARGS);
    } else if (w.bn_tile == 32 && cin != nullptr) {
        switch (rows) {
            case 3: rc = launch_cfg<3, 4, 4, true, 3>(NNVB_CW_ARGS); break;
            case 4: rc = launch_cfg<3, 4, 4, true, 4>(NNVB_CW_ARGS); break;
            case 5: rc = launch_cfg<3, 4, 4, true, 5>(NNVB_CW_ARGS); break;
            case 6: rc = launch_cfg<3, 4, 4, true, 6>(NNVB_CW_ARGS); break;
            default: rc = launch_cfg<3, 4, 4, true>(NNVB_CW_ARGS);
        }
    } else if (w.bn_tile == 32) {
        rc = launch_cfg<3, 4, 4, false>(NNVB_CW_ARGS);
    }
#undef NNVB_CW_ARGS
    if (rc == NNVB_OK && *done && launches) *launches += 1;
    return rc;
}

}  // namespace nnvb
