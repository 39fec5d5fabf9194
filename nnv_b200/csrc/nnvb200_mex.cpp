// MEX gateway: MATLAB <-> libnnvb200.so.  No arithmetic happens here; the file
// unpacks MATLAB arrays (read-only, column-major FP64, exactly the layout the C
// ABI takes), calls the C ABI, and packs the results into new MATLAB arrays.
//
//   h   = nnvb200_mex('create_net', layers, [H W C])   % layers: struct array, see below
//   R   = nnvb200_mex('reach', h, S)                   % S: struct with V,C,d,pred_lb,pred_ub
//                                                      %    or im_lb, im_ub (ImageStar(lb,ub))
//   out = nnvb200_mex('verify', h, S, target)          % 1 robust, 2 unknown, -1 undecided on device
//   st  = nnvb200_mex('stats', h)                      % per-ReLU-layer counters of the last reach
//         nnvb200_mex('destroy', h)
//
// layers(i) has the fields of the reference's layer objects: Type ('conv2d', 'fc',
// 'bn', 'avgpool', 'relu'), Weights, Bias, PaddingSize, Stride, DilationFactor,
// PoolSize, TrainedMean, TrainedVariance, Scale, Offset, Epsilon
// (code/nnv/engine/nn/layers/Conv2DLayer.m:84-144, FullyConnectedLayer.m:56-66,
//  BatchNormalizationLayer.m:72-77, AveragePooling2DLayer.m:109-131).
//
// Errors: the C ABI returns status codes; only this file turns them into
// mexErrMsgIdAndTxt (which does not return), after the C++ temporaries of the
// call have been released.  The CUDA context persists across calls (mexLock);
// mexAtExit tears it down.  MATLAB's 1-based target label becomes 0-based here.
#include "mex.h"

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/nnvb200.h"

namespace {

nnvb_ctx* g_ctx = nullptr;

struct NetHandle {
    nnvb_net* net = nullptr;
    nnvb_batch* last = nullptr;   // results of the most recent reach
    int64_t shape[3] = {0, 0, 0};
};
std::vector<NetHandle*> g_nets;

void at_exit() {
    for (NetHandle* h : g_nets) {
        if (!h) continue;
        nnvb_batch_destroy(h->last);
        nnvb_net_destroy(h->net);
        delete h;
    }
    g_nets.clear();
    nnvb_destroy(g_ctx);
    g_ctx = nullptr;
}

// Collects an error instead of raising it, so that destructors run first.
struct Err {
    std::string id, msg;
    bool set = false;
    void fail(const char* i, const std::string& m) { if (!set) { id = i; msg = m; set = true; } }
    void check(int status, const char* where) {
        // a batch that does not fit the arena gets its own identifier: the caller can split the list and retry
        if (status != NNVB_OK)
            fail(status == NNVB_E_CAPACITY ? "NNVB200:capacity" : "NNVB200:engine",
                 std::string(where) + ": " + nnvb_strerror(status) + " - " + nnvb_last_error());
    }
};

const double* field_doubles(const mxArray* s, mwIndex i, const char* name, size_t* n, Err& e) {
    const mxArray* f = mxGetField(s, i, name);
    if (!f || mxIsEmpty(f)) { if (n) *n = 0; return nullptr; }
    if (!mxIsDouble(f) || mxIsComplex(f)) { e.fail("NNVB200:type", std::string(name) + " must be a real double array"); return nullptr; }
    if (n) *n = mxGetNumberOfElements(f);
    return mxGetDoubles(f);
}

void fill_ints(const double* src, size_t n, int32_t* dst, size_t want, int32_t dflt) {
    for (size_t i = 0; i < want; ++i) dst[i] = (src && i < n) ? (int32_t)src[i] : dflt;
}

NetHandle* get_handle(const mxArray* a, Err& e) {
    if (!a || mxGetNumberOfElements(a) != 1) { e.fail("NNVB200:handle", "invalid network handle"); return nullptr; }
    const size_t idx = (size_t)mxGetScalar(a);
    if (idx == 0 || idx > g_nets.size() || !g_nets[idx - 1]) { e.fail("NNVB200:handle", "invalid network handle"); return nullptr; }
    return g_nets[idx - 1];
}

void create_net(int nlhs, mxArray* plhs[], int nrhs, const mxArray* prhs[], Err& e) {
    if (nrhs < 3 || !mxIsStruct(prhs[1])) { e.fail("NNVB200:args", "create_net needs a layer struct array and [H W C]"); return; }
    const size_t nl = mxGetNumberOfElements(prhs[1]);
    std::vector<nnvb_layer_desc> descs(nl);
    std::memset(descs.data(), 0, nl * sizeof(nnvb_layer_desc));
    for (size_t i = 0; i < nl && !e.set; ++i) {
        nnvb_layer_desc& d = descs[i];
        const mxArray* t = mxGetField(prhs[1], i, "Type");
        char* ts = t ? mxArrayToString(t) : nullptr;
        const std::string type = ts ? ts : "";
        if (ts) mxFree(ts);
        size_t n = 0;
        d.stride[0] = d.stride[1] = 1;
        d.dilation[0] = d.dilation[1] = 1;
        if (type == "conv2d") {
            d.type = NNVB_LAYER_CONV2D;
            const mxArray* w = mxGetField(prhs[1], i, "Weights");
            if (!w || !mxIsDouble(w)) { e.fail("NNVB200:type", "conv2d Weights must be double"); break; }
            const mwSize nd = mxGetNumberOfDimensions(w);
            const mwSize* dm = mxGetDimensions(w);
            d.kh = (int32_t)dm[0]; d.kw = (int32_t)dm[1];
            d.cin = nd > 2 ? (int32_t)dm[2] : 1; d.cout = nd > 3 ? (int32_t)dm[3] : 1;
            d.W = mxGetDoubles(w);
            d.b = field_doubles(prhs[1], i, "Bias", &n, e);
            const double* p = field_doubles(prhs[1], i, "PaddingSize", &n, e); fill_ints(p, n, d.pad, 4, 0);
            p = field_doubles(prhs[1], i, "Stride", &n, e); fill_ints(p, n, d.stride, 2, 1);
            p = field_doubles(prhs[1], i, "DilationFactor", &n, e); fill_ints(p, n, d.dilation, 2, 1);
        } else if (type == "fc") {
            d.type = NNVB_LAYER_FC;
            const mxArray* w = mxGetField(prhs[1], i, "Weights");
            if (!w || !mxIsDouble(w)) { e.fail("NNVB200:type", "fc Weights must be double"); break; }
            d.cout = (int32_t)mxGetM(w); d.cin = (int32_t)mxGetN(w);
            d.W = mxGetDoubles(w);
            d.b = field_doubles(prhs[1], i, "Bias", &n, e);
        } else if (type == "bn") {
            d.type = NNVB_LAYER_BN;
            d.bn_mean = field_doubles(prhs[1], i, "TrainedMean", &n, e); d.cout = (int32_t)n;
            d.bn_var = field_doubles(prhs[1], i, "TrainedVariance", &n, e);
            d.bn_scale = field_doubles(prhs[1], i, "Scale", &n, e);
            d.bn_offset = field_doubles(prhs[1], i, "Offset", &n, e);
            const double* eps = field_doubles(prhs[1], i, "Epsilon", &n, e);
            d.bn_eps = eps ? eps[0] : 1e-5;
        } else if (type == "avgpool") {
            d.type = NNVB_LAYER_AVGPOOL2D;
            const double* p = field_doubles(prhs[1], i, "PoolSize", &n, e); fill_ints(p, n, d.pool, 2, 2);
            p = field_doubles(prhs[1], i, "Stride", &n, e); fill_ints(p, n, d.stride, 2, 1);
            p = field_doubles(prhs[1], i, "PaddingSize", &n, e); fill_ints(p, n, d.pad, 4, 0);
            // how a padded window is averaged: a MATLAB host reaches this engine where its CPU path would call
            // vl_nnpool (entries inside the image); DivisorWindow = 1 selects ph*pw (the gpuArray path's avgpool)
            const double* dv = field_doubles(prhs[1], i, "DivisorWindow", &n, e);
            d.avgpool_divisor = (dv && dv[0] != 0.0) ? NNVB_POOL_DIV_WINDOW : NNVB_POOL_DIV_INSIDE;
        } else if (type == "relu") {
            d.type = NNVB_LAYER_RELU;
        } else {
            e.fail("NNVB200:layer", "layer type '" + type + "' is outside the approx-star path of this engine");
        }
    }
    if (e.set) return;
    if (mxGetNumberOfElements(prhs[2]) != 3) { e.fail("NNVB200:args", "input size must be [H W C]"); return; }
    const double* hwc = mxGetDoubles(prhs[2]);
    if (!g_ctx) {
        e.check(nnvb_init(0, 0, &g_ctx), "nnvb_init");
        if (e.set) return;
        mexLock();
        mexAtExit(at_exit);
    }
    NetHandle* h = new NetHandle();
    e.check(nnvb_net_create(g_ctx, descs.data(), (int)nl, (int64_t)hwc[0], (int64_t)hwc[1], (int64_t)hwc[2], &h->net),
            "nnvb_net_create");
    if (e.set) { delete h; return; }
    nnvb_net_out_shape(h->net, h->shape);
    g_nets.push_back(h);
    if (nlhs > 0) plhs[0] = mxCreateDoubleScalar((double)g_nets.size());
}

// stage one MATLAB set struct into batch slot 0
void stage_set(nnvb_batch* b, const mxArray* S, Err& e) {
    size_t nlb = 0, nub = 0;
    const double* lb = field_doubles(S, 0, "im_lb", &nlb, e);
    const double* ub = field_doubles(S, 0, "im_ub", &nub, e);
    const mxArray* V = mxGetField(S, 0, "V");
    if ((!V || mxIsEmpty(V)) && lb && ub) {
        if (nlb != nub) { e.fail("NNVB200:set", "Inconsistency between lower bound image and upper bound image"); return; }
        e.check(nnvb_batch_set_bounds(b, 0, lb, ub), "nnvb_batch_set_bounds");
        return;
    }
    if (!V || !mxIsDouble(V)) { e.fail("NNVB200:set", "set needs a double V or im_lb/im_ub"); return; }
    const mwSize nd = mxGetNumberOfDimensions(V);
    const mwSize* dm = mxGetDimensions(V);
    // ImageStar: [H W C P+1]; Star: [N P+1]
    const int64_t P = (nd == 2 ? (int64_t)dm[1] : (nd > 3 ? (int64_t)dm[3] : 1)) - 1;
    size_t n = 0, m = 0;
    const double* pl = field_doubles(S, 0, "pred_lb", &n, e);
    const double* pu = field_doubles(S, 0, "pred_ub", &n, e);
    const double* d = field_doubles(S, 0, "d", &m, e);
    const double* C = field_doubles(S, 0, "C", &n, e);
    if (e.set) return;
    e.check(nnvb_batch_set_star(b, 0, P, mxGetDoubles(V), pl, pu, C ? (int64_t)m : 0, C, d), "nnvb_batch_set_star");
}

void reach_or_verify(bool verify, int nlhs, mxArray* plhs[], int nrhs, const mxArray* prhs[], Err& e) {
    if (nrhs < (verify ? 4 : 3) || !mxIsStruct(prhs[2])) { e.fail("NNVB200:args", "usage: reach(h, S) / verify(h, S, target)"); return; }
    NetHandle* h = get_handle(prhs[1], e);
    if (!h) return;
    nnvb_batch_destroy(h->last);
    h->last = nullptr;
    e.check(nnvb_batch_create(h->net, 1, &h->last), "nnvb_batch_create");
    if (e.set) return;
    stage_set(h->last, prhs[2], e);
    if (e.set) return;
    e.check(nnvb_batch_upload(h->last), "nnvb_batch_upload");
    nnvb_opts o;
    std::memset(&o, 0, sizeof(o));
    o.keep_constraints = verify ? 0 : 1;
    o.keep_layer_bounds = 1;
    if (!e.set) e.check(nnvb_batch_reach(h->last, &o), "nnvb_batch_reach");
    if (e.set) return;
    if (verify) {
        const int32_t target = (int32_t)mxGetScalar(prhs[3]) - 1;      // MATLAB labels are 1-based
        int verdict = NNVB_UNDECIDED;
        e.check(nnvb_batch_verify_robust(h->last, &target, 0, &verdict, nullptr, nullptr), "nnvb_batch_verify_robust");
        if (!e.set && nlhs > 0) plhs[0] = mxCreateDoubleScalar((double)verdict);
        return;
    }
    int64_t P = 0, m = 0;
    e.check(nnvb_batch_out_dims(h->last, 0, &P, &m), "nnvb_batch_out_dims");
    if (e.set) return;
    const char* names[] = {"V", "C", "d", "pred_lb", "pred_ub"};
    mxArray* R = mxCreateStructMatrix(1, 1, 5, names);
    const mwSize vd[4] = {(mwSize)h->shape[0], (mwSize)h->shape[1], (mwSize)h->shape[2], (mwSize)(P + 1)};
    mxArray* V = mxCreateNumericArray(4, vd, mxDOUBLE_CLASS, mxREAL);
    mxArray* C = mxCreateDoubleMatrix((mwSize)m, (mwSize)P, mxREAL);
    mxArray* d = mxCreateDoubleMatrix((mwSize)m, 1, mxREAL);
    mxArray* pl = mxCreateDoubleMatrix((mwSize)P, 1, mxREAL);
    mxArray* pu = mxCreateDoubleMatrix((mwSize)P, 1, mxREAL);
    e.check(nnvb_batch_get_V(h->last, 0, mxGetDoubles(V)), "nnvb_batch_get_V");
    if (!e.set) e.check(nnvb_batch_get_constraints(h->last, 0, mxGetDoubles(C), mxGetDoubles(d)), "nnvb_batch_get_constraints");
    if (!e.set) e.check(nnvb_batch_get_pred_bounds(h->last, 0, mxGetDoubles(pl), mxGetDoubles(pu)), "nnvb_batch_get_pred_bounds");
    mxSetField(R, 0, "V", V); mxSetField(R, 0, "C", C); mxSetField(R, 0, "d", d);
    mxSetField(R, 0, "pred_lb", pl); mxSetField(R, 0, "pred_ub", pu);
    if (nlhs > 0) plhs[0] = R;
}

void stats(int nlhs, mxArray* plhs[], int nrhs, const mxArray* prhs[], Err& e) {
    NetHandle* h = nrhs > 1 ? get_handle(prhs[1], e) : nullptr;
    if (!h || !h->last) { e.fail("NNVB200:state", "no reach has been run on this network"); return; }
    int n = 0;
    nnvb_batch_relu_layers(h->last, &n);
    mxArray* out = mxCreateDoubleMatrix((mwSize)n, 4, mxREAL);
    double* p = mxGetDoubles(out);
    for (int i = 0; i < n && !e.set; ++i) {
        nnvb_relu_stats s;
        e.check(nnvb_batch_relu_stats(h->last, i, &s), "nnvb_batch_relu_stats");
        p[i] = (double)s.n_neurons; p[n + i] = (double)s.n_cross; p[2 * n + i] = (double)s.n_dead; p[3 * n + i] = (double)s.cols_after;
    }
    if (nlhs > 0) plhs[0] = out;
}

// Y = nnvb200_mex('evaluate', h, X): NN.evaluate (NN.m:130-145) on the columns of X [H*W*C x n] in one pass
void evaluate(int nlhs, mxArray* plhs[], int nrhs, const mxArray* prhs[], Err& e) {
    if (nrhs < 3 || !mxIsDouble(prhs[2]) || mxIsComplex(prhs[2])) { e.fail("NNVB200:args", "usage: evaluate(h, X) with a real double X"); return; }
    NetHandle* h = get_handle(prhs[1], e);
    if (!h) return;
    const size_t n = mxGetN(prhs[2]);
    const size_t n_out = (size_t)(h->shape[0] * h->shape[1] * h->shape[2]);
    mxArray* Y = mxCreateDoubleMatrix((mwSize)n_out, (mwSize)n, mxREAL);
    e.check(nnvb_net_evaluate(h->net, (int64_t)n, mxGetDoubles(prhs[2]), mxGetDoubles(Y)), "nnvb_net_evaluate");
    if (!e.set && nlhs > 0) plhs[0] = Y;
}

// id = nnvb200_mex('nccl_id') on worker 1; nnvb200_mex('set_shard', rank, world, id [, peer_memory]) on every worker
// (rank 1-based like spmdIndex): one set split along its generators over the workers' GPUs
void nccl_id(int nlhs, mxArray* plhs[], Err& e) {
    mxArray* id = mxCreateNumericMatrix(1, NNVB_NCCL_ID_BYTES / 8, mxUINT64_CLASS, mxREAL);
    e.check(nnvb_nccl_unique_id(mxGetData(id)), "nnvb_nccl_unique_id");
    if (!e.set && nlhs > 0) plhs[0] = id;
}

void set_shard(int nrhs, const mxArray* prhs[], Err& e) {
    if (nrhs < 4 || mxGetNumberOfElements(prhs[3]) * 8 != NNVB_NCCL_ID_BYTES) { e.fail("NNVB200:args", "usage: set_shard(rank, world, id)"); return; }
    if (!g_ctx) { e.fail("NNVB200:state", "create a network first: the context is made with it"); return; }
    const int rank = (int)mxGetScalar(prhs[1]) - 1, world = (int)mxGetScalar(prhs[2]);
    const int peer = nrhs > 4 ? (mxGetScalar(prhs[4]) != 0.0) : 0;     // NCCL measured faster than the fused form
    e.check(nnvb_set_shard_nccl(g_ctx, rank, world, mxGetData(prhs[3]), peer), "nnvb_set_shard_nccl");
}

}  // namespace

extern "C" void mexFunction(int nlhs, mxArray* plhs[], int nrhs, const mxArray* prhs[]) {
    Err e;
    {
        std::string cmd;
        if (nrhs >= 1 && mxIsChar(prhs[0])) {
            char* c = mxArrayToString(prhs[0]);
            if (c) { cmd = c; mxFree(c); }
        }
        if (cmd == "create_net") create_net(nlhs, plhs, nrhs, prhs, e);
        else if (cmd == "reach") reach_or_verify(false, nlhs, plhs, nrhs, prhs, e);
        else if (cmd == "verify") reach_or_verify(true, nlhs, plhs, nrhs, prhs, e);
        else if (cmd == "stats") stats(nlhs, plhs, nrhs, prhs, e);
        else if (cmd == "evaluate") evaluate(nlhs, plhs, nrhs, prhs, e);
        else if (cmd == "nccl_id") nccl_id(nlhs, plhs, e);
        else if (cmd == "set_shard") set_shard(nrhs, prhs, e);
        else if (cmd == "destroy") {
            NetHandle* h = nrhs > 1 ? get_handle(prhs[1], e) : nullptr;
            if (h) {
                nnvb_batch_destroy(h->last);
                nnvb_net_destroy(h->net);
                g_nets[(size_t)mxGetScalar(prhs[1]) - 1] = nullptr;
                delete h;
            }
        } else {
            e.fail("NNVB200:command", "unknown command '" + cmd + "'");
        }
    }   // every C++ temporary is gone before the (non-returning) error call
    if (e.set) mexErrMsgIdAndTxt(e.id.c_str(), "%s", e.msg.c_str());
}
