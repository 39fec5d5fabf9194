/*
 * nnvb200.h — C ABI of libnnvb200.so, the sm_100a engine for the approx-star
 * (estimated-bounds) reachability path of NNV.
 *
 * Everything crosses this boundary as plain pointers and sizes.  All floating
 * point is IEEE double; all tensors use MATLAB's column-major layout, i.e. an
 * image-shaped set is V[h + H*(w + W*(c + C*j))] for predicate column j
 * (j = 0 is the centre), exactly what mxGetDoubles returns for the reference's
 * ImageStar.V.  Indices are 0-based here; the MEX gateway converts.
 *
 * Every function returns an nnvb_status (0 = NNVB_OK); nothing throws, nothing
 * calls back.  Host buffers stay owned by the caller and are only read unless
 * the parameter is documented as an output.  Device memory lives behind the
 * opaque handles and is released by the matching *_destroy.
 *
 * Citations name the reference interface each entry point stands in for
 * (paths relative to the reference repository).
 */
#ifndef NNVB200_H
#define NNVB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    NNVB_OK = 0,
    NNVB_E_ARG = 1,        /* bad argument / inconsistent dimensions (the reference raises error(...)) */
    NNVB_E_CUDA = 2,       /* a CUDA runtime call failed; see nnvb_last_error */
    NNVB_E_CAPACITY = 3,   /* the set outgrew the context's arena; retry with a smaller batch or bigger arena */
    NNVB_E_STATE = 4,      /* call order violated (e.g. results requested before reach) */
    NNVB_E_UNSUPPORTED = 5 /* layer type / option outside the engine's path */
} nnvb_status;

typedef struct nnvb_ctx nnvb_ctx;
typedef struct nnvb_net nnvb_net;
typedef struct nnvb_batch nnvb_batch;

/* ---- layer descriptions ------------------------------------------------- */

typedef enum {
    NNVB_LAYER_CONV2D = 1,   /* code/nnv/engine/nn/layers/Conv2DLayer.m */
    NNVB_LAYER_FC = 2,       /* code/nnv/engine/nn/layers/FullyConnectedLayer.m */
    NNVB_LAYER_BN = 3,       /* code/nnv/engine/nn/layers/BatchNormalizationLayer.m */
    NNVB_LAYER_AVGPOOL2D = 4,/* code/nnv/engine/nn/layers/AveragePooling2DLayer.m */
    NNVB_LAYER_RELU = 5      /* code/nnv/engine/nn/layers/ReluLayer.m */
} nnvb_layer_type;

/* One layer.  Parameter layouts are the reference's own:
 *   CONV2D   W[kh,kw,Cin,Cout] column-major, b[Cout], pad = [t b l r], stride, dilation
 *            (Conv2DLayer.m:84-144)
 *   FC       W[Out,In] column-major, b[Out]; In is indexed h-fastest
 *            (FullyConnectedLayer.m:56-66, :312)
 *   BN       mean/var/scale/offset[C], eps (BatchNormalizationLayer.m:311-327)
 *   AVGPOOL  pool[2], stride[2], pad[4] (AveragePooling2DLayer.m:109-131).  The
 *            reference averages a padded window in two different ways:
 *            reach_star_single_input calls evaluate (:227-248), which on host
 *            arrays is MatConvNet's vl_nnpool(..., 'Method', 'avg') — the sum is
 *            divided by the number of window entries inside the image — and on
 *            gpuArray inputs is avgpool with zero padding, which divides by
 *            ph*pw like the pure-MATLAB compute_averageMap (:316-393).
 *            avgpool_divisor selects the rule: NNVB_POOL_DIV_WINDOW (0) = ph*pw,
 *            NNVB_POOL_DIV_INSIDE (1) = entries inside the image.  Without
 *            padding the two agree.
 *   RELU     no parameters
 * Unused fields are ignored. */
#define NNVB_POOL_DIV_WINDOW 0
#define NNVB_POOL_DIV_INSIDE 1
typedef struct {
    int32_t type;
    int32_t kh, kw, cin, cout;       /* conv: filter dims; fc: cout = Out, cin = In */
    int32_t pad[4];                  /* t b l r */
    int32_t stride[2];
    int32_t dilation[2];
    int32_t pool[2];
    const double* W;
    const double* b;
    const double* bn_mean;
    const double* bn_var;
    const double* bn_scale;
    const double* bn_offset;
    double bn_eps;
    int32_t avgpool_divisor;         /* NNVB_POOL_DIV_* */
    int32_t reserved;
} nnvb_layer_desc;

/* ---- options and statistics -------------------------------------------- */

/* Counterpart of the reachOptions struct parsed in NN.reach (NN.m:189-247).
 * Only the LP-free bound mode exists here: reachMethod 'approx-star' with
 * estimated ranges == 'relax-star-*' with relaxFactor = 1 (PosLin.m:1588-1646). */
typedef struct {
    int32_t keep_constraints;  /* 1: record the rows needed to emit C,d (Star.C / Star.d) */
    int32_t keep_layer_bounds; /* 1: keep lb/ub and crossing lists of every ReLU layer for download */
    int32_t reserved[6];
} nnvb_opts;

/* Per-ReLU-layer counters summed over the batch; maps onto the reference's
 * per-layer tic/toc record obj.reachTime (NN.m:1542-1545). */
typedef struct {
    int64_t n_neurons;   /* N of the layer */
    int64_t n_cross;     /* crossing neurons, summed over queries */
    int64_t n_dead;      /* ub <= 0 neurons, summed over queries */
    int64_t cols_after;  /* total columns in the batch after the layer */
} nnvb_relu_stats;

/* ---- context ------------------------------------------------------------ */

/* Bind a context to one CUDA device and reserve `arena_bytes` of device memory
 * for set tensors (two ping-pong generator buffers plus records).  One context
 * per process per GPU; mirrors the reference's reachOptions.device switch
 * (NN.m:216-222) and params2gpu (NN.m:1257-1263). */
int nnvb_init(int device, size_t arena_bytes, nnvb_ctx** out);
int nnvb_destroy(nnvb_ctx* ctx);
/* Text of the most recent failure on this thread (never NULL). */
const char* nnvb_last_error(void);
const char* nnvb_strerror(int status);
/* Version of this ABI; bumps when a signature changes. */
int nnvb_abi_version(void);
/* The stream every kernel of the context is launched on (a cudaStream_t cast
 * to void*), so a host harness can record events on it. */
void* nnvb_stream(nnvb_ctx* ctx);
/* Number of kernels this library has launched on the context so far. */
int64_t nnvb_launch_count(nnvb_ctx* ctx);

/* Device time per kernel family, the counterpart of the reference's per-layer
 * tic/toc record obj.reachTime (NN.m:1542-1545).  While enabled, every launch
 * group is bracketed by CUDA events on the context stream.  nnvb_profile_read
 * returns, since the last enable: accumulated milliseconds, kernels launched,
 * and the algorithmic work of those launches — floating-point operations for the
 * contractions (2*Ho*Wo*Cout*kh*kw*Cin*columns, 2*Out*In*columns), bytes for
 * the bandwidth-bound families (each tensor read or written once).  For columns
 * that are zero outside a small window only the window counts: positions of the
 * input window for a convolution (each meets kh*kw taps), rows of the window for
 * an FC layer, bytes of the windows for pooling and the bound reduction. */
#define NNVB_PROF_CONV 0      /* Conv2D implicit GEMM (+ fused BatchNormalization) */
#define NNVB_PROF_FC 1        /* FullyConnected GEMM */
#define NNVB_PROF_BN 2        /* stand-alone BatchNormalization */
#define NNVB_PROF_AVGPOOL 3   /* AveragePooling2D */
#define NNVB_PROF_RANGES 4    /* Star.estimateRanges + classification scans */
#define NNVB_PROF_RELAX 5     /* row clearing, column append, list rebuild */
#define NNVB_PROF_VERIFY 6    /* halfspace rows, box minimum, witness pass */
#define NNVB_PROF_ONEHOT 7    /* images of the unit-vector columns a ReLU step appended (bytes written) */
#define NNVB_PROF_ALLREDUCE 8  /* generator sharding: sum of the partial bound sums over the ranks (bytes per rank) */
#define NNVB_PROF_FAMILIES 9
int nnvb_profile_enable(nnvb_ctx* ctx, int on);
int nnvb_profile_read(nnvb_ctx* ctx, int family, double* ms, int64_t* launches, double* work);

/* ---- one set sharded over several GPUs ----------------------------------- */

/* Generator sharding: a single large set is split along its predicate
 * (generator) dimension over `world` processes, one GPU each.  Rank r holds the
 * generator columns whose position in the predicate order is = r (mod world);
 * the centre is replicated.  Every affine layer works on the local columns; in
 * the ReLU step each rank reduces its own columns to partial bound sums, the
 * sums are added over the ranks through the hook below, and every rank then
 * classifies the same numbers, clears its own columns' rows and materialises
 * the new columns numbered = r (mod world).  The reference has no counterpart
 * (its only parallel axis is parfor over independent sets, NN.m:1371-1413).
 *
 * The hook must sum `count` doubles at device pointer `dev_buf` over all ranks
 * in place (an NCCL all-reduce), ordered after prior work on `stream` (a
 * cudaStream_t) and before later work on it; it returns 0 on success.  It is
 * called from nnvb_batch_reach and the result getters of a sharded context, at
 * the same points on every rank.  Call nnvb_set_shard before creating batches.
 * With world > 1: nnvb_batch_out_dims reports sizes over all ranks; get_V and
 * get_pred_bounds fill only this rank's columns (centre on rank 0) into the
 * full-size output, zeros elsewhere, so the sum over ranks is the set;
 * constraint records (keep_constraints, get_constraints) are not available. */
typedef int (*nnvb_allreduce_fn)(void* user, double* dev_buf, int64_t count, void* stream);
int nnvb_set_shard(nnvb_ctx* ctx, int rank, int world, nnvb_allreduce_fn fn, void* user);

/* The same sharding with the collective inside the library, for hosts without
 * a collective of their own (a MATLAB session per GPU): NCCL is bound at run
 * time (libnccl.so.2) and ncclAllReduce(ncclDouble, ncclSum) runs on the
 * context's stream.  Rank 0 obtains a communicator id with
 * nnvb_nccl_unique_id (NNVB_NCCL_ID_BYTES bytes) and hands it to the other
 * ranks by any host-side means (a file, a socket); then every rank calls
 * nnvb_set_shard_nccl with its own context current on its own GPU — the call
 * is collective and returns when the communicator is up.
 * peer_memory != 0 additionally maps every rank's sum buffer into every other
 * rank (CUDA IPC, GPUs of one node linked by NVLink): the ReLU step then
 * writes its partial sums there, raises a flag at the peers, and the
 * classification kernel adds the ranks' sums in rank order straight from peer
 * memory — one pass instead of reduce + all-reduce + classify.  A rank waits
 * for a peer's flag at most about two seconds; after that the reach returns
 * NNVB_E_STATE and the context stays usable.  If the mapping cannot be set
 * up on some rank, all ranks use the NCCL all-reduce.  Measured on 2 and on
 * 8 B200s the NCCL all-reduce is the faster of the two (every rank of the
 * peer-memory form reads all ranks' sums): pass 0 unless measuring. */
#define NNVB_NCCL_ID_BYTES 128
int nnvb_nccl_unique_id(void* id_out);
int nnvb_set_shard_nccl(nnvb_ctx* ctx, int rank, int world, const void* nccl_id, int peer_memory);

/* ---- network ------------------------------------------------------------ */

/* Copy the layer parameters to the device once and pre-arrange them for the
 * kernels.  Stands in for constructing NN({layers...}) (NN.m:99-105) followed by
 * params2gpu.  (in_h,in_w,in_c) is the input image size; a vector input of
 * length n is (n,1,1). */
int nnvb_net_create(nnvb_ctx* ctx, const nnvb_layer_desc* layers, int n_layers,
                    int64_t in_h, int64_t in_w, int64_t in_c, nnvb_net** out);
int nnvb_net_destroy(nnvb_net* net);
/* NN.evaluate (NN.m:130-145) on n_points concrete inputs at once: X is
 * [H*W*C x n_points] column-major on the host, Y receives [N_out x n_points].
 * ReLU layers apply max(x, 0).  This is what falsification (NN.falsify,
 * NN.m:930-988) and the harness pre-check of the bound images
 * (examples/Tutorial/SPIE/Classification2D/verifySample.m:5-20) evaluate. */
int nnvb_net_evaluate(nnvb_net* net, int64_t n_points, const double* X, double* Y);
/* Output size (H,W,C) of the network. */
int nnvb_net_out_shape(const nnvb_net* net, int64_t shape[3]);

/* ---- batches of input sets ---------------------------------------------- */

/* A batch is a list of independent input sets (queries) pushed through the same
 * network together; a single NN.reach call is a batch of one.  Stands in for
 * the array-of-sets handling of reach_star_multipleInputs
 * (e.g. Conv2DLayer.m:862-886). */
int nnvb_batch_create(nnvb_net* net, int n_queries, nnvb_batch** out);
int nnvb_batch_destroy(nnvb_batch* b);

/* Query q := ImageStar(lb, ub) (ImageStar.m:302-343 -> Star.m:220-237 ->
 * Box.m:16-58): centre (lb+ub)/2, one generator per entry with ub != lb, each
 * predicate in [-1,1], C = zeros(1,P), d = 0.  lb/ub have H*W*C entries. */
int nnvb_batch_set_bounds(nnvb_batch* b, int q, const double* lb, const double* ub);

/* Query q := ImageStar(V, C, d, pred_lb, pred_ub) (ImageStar.m:172-227).
 * V is [N x (P+1)] column-major, Cmat is [m x P] column-major (may be NULL when
 * m = 0), pl/pu have P entries.  C and d are kept on the host side of the
 * record: no layer reads them (they only enter the final feasibility system). */
int nnvb_batch_set_star(nnvb_batch* b, int q, int64_t P, const double* V,
                        const double* pl, const double* pu,
                        int64_t m, const double* Cmat, const double* d);

/* The same for n queries q0 .. q0+n-1 in one call (arrays of sets, e.g. the 16 384
 * attack sets of a brightening study built by ImageStar.m:172-227 in a loop):
 * set k reads lb + k*stride / ub + k*stride (stride >= H*W*C doubles), or, for
 * stars that share P and m, V + k*N*(P+1), pl/pu + k*P, Cmat + k*m*P, d + k*m. */
int nnvb_batch_set_bounds_many(nnvb_batch* b, int q0, int n, const double* lb, const double* ub, int64_t stride);
int nnvb_batch_set_stars(nnvb_batch* b, int q0, int n, int64_t P, int64_t m, const double* V, const double* pl,
                         const double* pu, const double* Cmat, const double* d);

/* Copy all staged queries to the device (asynchronous on the context stream). */
int nnvb_batch_upload(nnvb_batch* b);

/* Run every layer on the uploaded batch: NN.reach / reach_noConns
 * (NN.m:189-278, :1529-1551) with the LP-free ReLU step.  Can be called again
 * on the same uploaded inputs. */
int nnvb_batch_reach(nnvb_batch* b, const nnvb_opts* opts);

/* ---- LP-tightened bounds (the reference's default 'approx-star') ---------- */

/* PosLin.reach_star_approx2 (PosLin.m:747-857) uses the estimated ranges only
 * to pre-select: every neuron they call crossing gets its exact upper bound by
 * an LP over the set's constraints (Star.getMaxs, Star.m:898-970), those still
 * above zero their exact lower bound (Star.getMins, :784-856), and the
 * relaxation is built from the LP bounds.  The LP solver stays on the host, as
 * in the reference (lpsolver.m); the engine calls `fn` once per ReLU layer that
 * has such neurons, from inside nnvb_batch_reach, after the classification by
 * estimated ranges.  Inside the hook the caller may use, for that layer:
 *   nnvb_batch_get_crossing        the listed neurons of a query and their estimated bounds
 *   nnvb_batch_get_crossing_rows   their rows of the generator matrix and centre values (the LP objectives)
 *   nnvb_batch_get_constraints_before / nnvb_batch_out_dims / nnvb_batch_get_pred_bounds
 *                                  the constraint system and predicate box entering the layer
 *   nnvb_batch_tighten_crossing    hand back xmin / xmax for the listed neurons of a query
 * and the engine then classifies again: xmax <= 0 clears the row, xmin >= 0
 * leaves it untouched, otherwise the neuron is relaxed with [xmin, xmax].
 * The reach must keep constraint records (opts.keep_constraints).  fn returns
 * 0 on success.  NULL removes the hook. */
typedef int (*nnvb_bounds_fn)(void* user, nnvb_batch* b, int relu_layer);
int nnvb_batch_set_bounds_hook(nnvb_batch* b, nnvb_bounds_fn fn, void* user);
/* Rows of query q's generator matrix at the listed neurons of the running
 * layer: G is [k x P_in] column-major in the reference's predicate order, c[k]
 * the centre values.  Only valid inside the hook, for its relu_layer. */
int nnvb_batch_get_crossing_rows(nnvb_batch* b, int q, int relu_layer, double* G, double* c);
/* Constraint system of query q entering ReLU layer relu_layer: *m rows, P_in
 * columns (what nnvb_batch_get_constraints would give after the layers before
 * it).  Cmat / d may be NULL to ask for *m only. */
int nnvb_batch_get_constraints_before(nnvb_batch* b, int q, int relu_layer, int64_t* m, double* Cmat, double* d);
/* LP bounds of the k listed neurons of query q, in the order of
 * nnvb_batch_get_crossing.  Only valid inside the hook. */
int nnvb_batch_tighten_crossing(nnvb_batch* b, int q, int relu_layer, const double* xmin, const double* xmax);

/* ---- results of a reach -------------------------------------------------- */

/* Number of predicates P and of constraint rows m of query q's output set. */
int nnvb_batch_out_dims(const nnvb_batch* b, int q, int64_t* P, int64_t* m);
/* Output generator matrix of query q, [N_out x (P+1)] column-major, columns in
 * the reference's predicate order (ImageStar.V of the returned set). */
int nnvb_batch_get_V(nnvb_batch* b, int q, double* V);
/* pred_lb / pred_ub of the output set (P entries each). */
int nnvb_batch_get_pred_bounds(nnvb_batch* b, int q, double* pl, double* pu);
/* Star.estimateRanges (Star.m:1078-1106) of the output set: N_out entries each. */
int nnvb_batch_get_ranges(nnvb_batch* b, int q, double* lb, double* ub);
/* Dense constraint system [m x P] column-major and d[m] of the output set, as
 * PosLin.multipleStepReachStarApprox_at_one stacks it (PosLin.m:711-735).
 * Requires opts.keep_constraints. */
int nnvb_batch_get_constraints(nnvb_batch* b, int q, double* Cmat, double* d);
/* Number of ReLU layers, and the per-layer counters. */
int nnvb_batch_relu_layers(const nnvb_batch* b, int* n);
int nnvb_batch_relu_stats(const nnvb_batch* b, int relu_layer, nnvb_relu_stats* st);
/* Crossing neurons of query q at ReLU layer `relu_layer`: count, then (when the
 * pointers are non-NULL) their ascending 0-based linear indices and estimated
 * bounds — map2 / lb / ub of PosLin.m:1598-1607.  Requires opts.keep_layer_bounds. */
int nnvb_batch_get_crossing(nnvb_batch* b, int q, int relu_layer, int64_t* k,
                            int64_t* idx, double* lb, double* ub);
/* Estimated bounds of all N neurons of query q entering ReLU layer `relu_layer`. */
int nnvb_batch_get_layer_ranges(nnvb_batch* b, int q, int relu_layer, double* lb, double* ub);

/* ---- output specification ------------------------------------------------ */

/* Verdict codes follow verify_specification.m: 1 = every halfspace
 * intersection is empty (robust / safe), 2 = some intersection is non-empty
 * (unknown for an over-approximation).  NNVB_UNDECIDED marks a halfspace the
 * device-side tests could not settle; the caller finishes it with the
 * feasibility LP of Star.isEmptySet (Star.m:1216-1232).
 *
 * Device-side tests per halfspace row G_h x <= g_h:
 *   - the minimum of G_h x - g_h over the output set's predicate box; a
 *     positive minimum proves the intersection empty (NNVB_VERDICT_EMPTY).
 *     "Positive" means above 1e-6 * (1 + the sum of the magnitudes of the terms
 *     of the minimum): the guard covers the rounding of a sum of 1e4..1e5 terms
 *     and the feasibility tolerance of the LP solver that decides the same
 *     question in the reference; rows nearer to zero stay undecided;
 *   - after a reach with opts.keep_constraints, a tighter lower bound of the
 *     row over the whole set: every ReLU predicate is replaced, last layer
 *     first, through its own relaxation rows (PosLin.m:716-735) by the affine
 *     form of its pre-activation, and the row left over the input predicates
 *     is minimised over their box; positive (same guard) proves the
 *     intersection empty and is returned as the margin;
 *   - a witness: a point of the output set (input predicates at a corner of
 *     their box, each ReLU predicate at the lower envelope max(0,x) or on the
 *     chord of its triangle, whichever lowers the row) evaluated by a forward
 *     pass; a point inside the halfspace proves it non-empty
 *     (NNVB_VERDICT_NONEMPTY).  The witness needs opts.keep_layer_bounds. */
#define NNVB_VERDICT_EMPTY 1
#define NNVB_VERDICT_NONEMPTY 2
#define NNVB_UNDECIDED (-1)

/* For query q and halfspaces G x <= g (G is [nh x N_out] column-major): the
 * minimum of G x - g over the output set's predicate box, one value per
 * halfspace.  A positive value proves Star.intersectHalfSpace (Star.m:555-589)
 * empty without an LP.  status[h] receives NNVB_VERDICT_EMPTY,
 * NNVB_VERDICT_NONEMPTY or NNVB_UNDECIDED. */
int nnvb_batch_halfspace_margins(nnvb_batch* b, int q, const double* G, const double* g,
                                 int nh, double* margin_lo, int* status);

/* Robustness form of the same test for the whole batch: for query q the
 * halfspaces are NN.robustness_set(target[q], kind) (NN.m:1334-1368), kind 0 =
 * 'max', 1 = 'min'.  status is [n_queries x (N_out-1)] row-major per query;
 * margin_lo likewise (may be NULL).  verdict[q] = 1 when all rows are empty, 2
 * when some row is proven non-empty, else NNVB_UNDECIDED. */
int nnvb_batch_verify_robust(nnvb_batch* b, const int32_t* target, int kind,
                             int* verdict, int* status, double* margin_lo);

/* The witness point the device builds for one halfspace row G x <= g of query
 * q (G has N_out entries), for callers that want to check it against the
 * constraint system of the set themselves: alpha[P] is the point's predicate
 * vector in the reference's predicate order — input predicates at the end of
 * their range that lowers the row, each ReLU predicate at max(0, x) or on the
 * chord a*(x - l) of its triangle (PosLin.m:716-735) — x_out[N_out] (nullable)
 * the network output the forward pass reached at that point, and *value
 * (nullable) G x_out - g.  By construction x_out = c + V alpha of the output
 * set and alpha satisfies pred_lb <= alpha <= pred_ub and C alpha <= d up to
 * rounding.  Needs a reach with opts.keep_layer_bounds; not available with
 * sharded generators (NNVB_E_UNSUPPORTED). */
int nnvb_batch_halfspace_witness(nnvb_batch* b, int q, const double* G, double g,
                                 double* alpha, double* x_out, double* value);

/* ---- single-layer entry points ------------------------------------------- */

/* One layer applied to one host-resident set, result back on the host:
 * L.reach(in_set, 'approx-star') for the affine layers
 * (Conv2DLayer.m:559-601, FullyConnectedLayer.m:295-317,
 * BatchNormalizationLayer.m:287-329, AveragePooling2DLayer.m:424-438).
 * V_in is [H*W*C x ncols] column-major (column 0 = centre), V_out must hold
 * Ho*Wo*Co x ncols doubles; out_shape receives (Ho,Wo,Co). */
int nnvb_layer_apply(nnvb_ctx* ctx, const nnvb_layer_desc* layer,
                     int64_t H, int64_t W, int64_t C, int64_t ncols,
                     const double* V_in, double* V_out, int64_t out_shape[3]);

/* Star.estimateRanges on a host-resident set: V is [N x (P+1)]. */
int nnvb_estimate_ranges(nnvb_ctx* ctx, int64_t N, int64_t P, const double* V,
                         const double* pl, const double* pu, double* lb, double* ub);

/* ---- allocation-free entry point ------------------------------------------ */

/* No counterpart in the reference: it exists for hosts that cannot let this
 * library allocate device memory — a MATLAB session whose gpuArray pool owns the
 * GPU, or a service with a fixed pre-sized arena — and therefore only lend it
 * pointers.  Computes Star.estimateRanges like nnvb_estimate_ranges, but every
 * pointer is a DEVICE pointer supplied by the caller and the call performs no
 * cudaMalloc/cudaFree (nor any allocating library call): its scratch is a fixed
 * array of NNVB_NOALLOC_SCRATCH_DOUBLES doubles (4 MiB) inside the loaded
 * module, held by every GPU that loads the library until the process exits.
 *   V_dev   [ld x (P+1)] column-major, column 0 = centre, ld >= N
 *   pl_dev, pu_dev  [P] predicate bounds;  lb_dev, ub_dev  [N] outputs
 *   stream  a cudaStream_t (NULL = default stream); the call returns after
 *           enqueueing two kernels on it.
 * Limit: 2*N <= NNVB_NOALLOC_SCRATCH_DOUBLES (N <= 262144); larger sets are
 * refused with NNVB_E_CAPACITY and a message.  The current device is used.  The
 * first call on a device loads the module's device data (the 4 MiB appear
 * on that GPU then, under lazy module loading) and looks up the scratch address
 * (cudaGetSymbolAddress), which is cached for the life of the process and does
 * not survive a cudaDeviceReset of that device; make that first call before
 * starting any stream capture.  All calls on a
 * device share the scratch: calls that overlap on the GPU race, so issue them on
 * one stream or otherwise one after the other.  Nothing in the scratch needs to
 * be cleared between calls. */
#define NNVB_NOALLOC_SCRATCH_DOUBLES 524288
int nnvb_estimate_ranges_noalloc(void* stream, int64_t N, int64_t P, const double* V_dev, int64_t ld,
                                 const double* pl_dev, const double* pu_dev, double* lb_dev, double* ub_dev);

#ifdef __cplusplus
}
#endif
#endif /* NNVB200_H */
