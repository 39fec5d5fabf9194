"""CPU restatement of the reference's approx-star (estimated-bounds) path.

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA engine:
only the tests, the smoke check and the benchmark's CPU-baseline leg may
import it.  The shipped package never does.

Parity status: the reference is MATLAB-only and cannot run where this code
runs, so the restatement is pinned (a) against the reference's own known-answer
tests and stored ``.mat`` baselines for the individual operations (fixtures in
tests/golden/reference_kats.npz) and (b) by following the reference source
function by function, cited below.  No reference test stores approx-star
generator tensors, bounds, crossing sets or verdicts at non-toy size, so parity
of the composed pipeline beyond those fixtures is unpinned.

All arithmetic is FP64 NumPy in the reference's operation order where the
order is visible in its source.  Arrays use MATLAB index semantics: image
tensors are ``[H, W, C, P+1]``; flattening is column-major (h fastest).

Bounds mode: the estimated (LP-free) ranges of Star.estimateRanges drive the
ReLU step, i.e. PosLin.reach_relaxed_star_static with relaxFactor = 1
(code/nnv/engine/nn/funcs/PosLin.m:1588-1646), which is also
PosLin.reach_star_approx2 (:747-857) with its two LP calls replaced by the
estimates.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import scipy.sparse as sp
from scipy.optimize import linprog

# --------------------------------------------------------------------------
# set types


@dataclass
class ImageStar:
    """code/nnv/engine/set/ImageStar.m:47-94 (fields) — V[H,W,C,P+1], C[m,P],
    d[m], pred_lb/pred_ub[P].  A vector Star (Star.m:13-24) is the same object
    with shape (N,1,1); ImageStar.toStar / Star.toImageStar (ImageStar.m:569-592,
    Star.m:1398-1418) are reshapes."""
    V: np.ndarray
    C: object          # scipy.sparse.csr_matrix [m, P]
    d: np.ndarray
    pl: np.ndarray
    pu: np.ndarray
    trace: list = field(default_factory=list)   # one dict per ReLU layer

    @property
    def shape(self):
        return self.V.shape[:3]

    @property
    def P(self):
        return self.V.shape[3] - 1

    def mat(self):
        """N x (P+1) matrix view (column-major flatten of each slice)."""
        h, w, c, p1 = self.V.shape
        return self.V.reshape(h * w * c, p1, order="F")


def star_from_bounds(lb, ub):
    """ImageStar(lb_im, ub_im): ImageStar.m:302-343 -> Star(lb,ub) Star.m:220-237
    -> Box Box.m:16-58 (centre (lb+ub)/2, generators diag((ub-lb)/2) with all-zero
    columns removed) -> Zono.toStar Zono.m:301-309 (pred in [-1,1]); the Star
    ctor then installs C = zeros(1,P), d = 0."""
    lb = np.asarray(lb, dtype=np.float64)
    ub = np.asarray(ub, dtype=np.float64)
    if lb.ndim == 1:
        lb = lb.reshape(-1, 1, 1)
        ub = ub.reshape(-1, 1, 1)
    if lb.ndim == 2:
        lb = lb[:, :, None]
        ub = ub[:, :, None]
    h, w, c = lb.shape
    n = h * w * c
    lbv = lb.reshape(n, order="F")
    ubv = ub.reshape(n, order="F")
    center = 0.5 * (lbv + ubv)
    vec = 0.5 * (ubv - lbv)
    nz = np.nonzero(vec != 0)[0]
    if n == 1:          # numel(gens) > 1 guard in Box.m:41
        nz = np.arange(1)
    P = len(nz)
    M = np.zeros((n, P + 1), order="F")
    M[:, 0] = center
    M[nz, np.arange(1, P + 1)] = vec[nz]
    V = M.reshape(h, w, c, P + 1, order="F")
    return ImageStar(V, sp.csr_matrix((1, P)), np.zeros(1), -np.ones(P), np.ones(P))


def star_from_query(q):
    """Build the input set of a workload query (see nnv_b200/configs.py)."""
    if "lb" in q:
        return star_from_bounds(q["lb"], q["ub"])
    V = np.asfortranarray(np.asarray(q["V"], dtype=np.float64))
    if V.ndim == 2:
        V = V.reshape(V.shape[0], 1, 1, V.shape[1], order="F")
    return ImageStar(V, sp.csr_matrix(np.atleast_2d(q["C"])), np.asarray(q["d"], float).ravel(),
                     np.asarray(q["pl"], float).ravel(), np.asarray(q["pu"], float).ravel())


# --------------------------------------------------------------------------
# affine layers


def zero_pad(x, pad):
    """Conv2DLayer.get_zero_padding_input, Conv2DLayer.m:1064-1108."""
    t, b, l, r = pad
    width = [(t, b), (l, r)] + [(0, 0)] * (x.ndim - 2)
    return np.pad(x, width)


def conv_out_size(hp, k, dil, stride):
    """Conv2DLayer.get_size_featureMap, Conv2DLayer.m:1227-1228 (hp = padded size)."""
    return (hp - (k - 1) * dil - 1) // stride + 1


CONV_BACKEND = "numpy"


def set_conv_backend(name):
    """"numpy" (default): im2col + GEMM written out below.  "torch": the same cross-correlation through
    torch.nn.functional.conv2d on the CPU in FP64 (about 4x faster on large generator tensors; results agree
    with the NumPy form to rounding, which tests/test_oracle_kats.py checks).  Used where a full-size
    workload has to finish in a test's or a benchmark sample's time."""
    global CONV_BACKEND
    if name not in ("numpy", "torch"):
        raise ValueError(name)
    CONV_BACKEND = name


def _conv2d_slices_torch(X, W, pad, stride, dilation, chunk=2048):
    import torch
    import torch.nn.functional as F
    t, b, l, r = pad
    w = torch.from_numpy(np.ascontiguousarray(W.transpose(3, 2, 0, 1)))          # [Cout, Cin, kh, kw]
    outs = []
    for c0 in range(0, X.shape[3], chunk):
        x = torch.from_numpy(np.ascontiguousarray(X[:, :, :, c0:c0 + chunk].transpose(3, 2, 0, 1)))   # [cols, Cin, H, W]
        x = F.pad(x, (l, r, t, b))
        outs.append(F.conv2d(x, w, None, tuple(stride), 0, tuple(dilation)).numpy().transpose(2, 3, 1, 0))
    return np.asfortranarray(np.concatenate(outs, axis=3))


def conv2d_slices(X, W, pad, stride, dilation, chunk=32):
    """Cross-correlation of every slice X[:,:,:,j] with W[kh,kw,Cin,Cout]; the
    arithmetic of Conv2DLayer.compute_featureMap (Conv2DLayer.m:1111-1204)
    extended over channels and filters as dlconv does at :591-592.  No bias."""
    if CONV_BACKEND == "torch":
        return _conv2d_slices_torch(X, W, pad, stride, dilation)
    kh, kw, cin, cout = W.shape
    assert X.shape[2] == cin
    Xp = zero_pad(X, pad)
    sh, sw = stride
    dh, dw = dilation
    ho = conv_out_size(Xp.shape[0], kh, dh, sh)
    wo = conv_out_size(Xp.shape[1], kw, dw, sw)
    ncol = X.shape[3]
    out = np.zeros((ho, wo, cout, ncol), order="F")
    for c0 in range(0, ncol, chunk):
        c1 = min(ncol, c0 + chunk)
        cols = np.empty((ho, wo, c1 - c0, kh, kw, cin))
        for i in range(kh):
            for j in range(kw):
                patch = Xp[i * dh: i * dh + (ho - 1) * sh + 1: sh,
                           j * dw: j * dw + (wo - 1) * sw + 1: sw, :, c0:c1]
                cols[:, :, :, i, j, :] = patch.transpose(0, 1, 3, 2)
        A = cols.reshape(ho * wo * (c1 - c0), kh * kw * cin)
        Wc = W.reshape(kh * kw * cin, cout)      # rows (kh, kw, ci), ci fastest, like A's columns
        Y = A @ Wc
        out[:, :, :, c0:c1] = Y.reshape(ho, wo, c1 - c0, cout).transpose(0, 1, 3, 2)
    return out


def conv2d_reach(S, L):
    """Conv2DLayer.reach_star_single_input, Conv2DLayer.m:559-601,780: bias on
    slice 0 only; C, d, predicate bounds unchanged."""
    Y = conv2d_slices(S.V, L["W"], L["pad"], L["stride"], L["dilation"])
    Y[:, :, :, 0] += np.asarray(L["b"]).reshape(1, 1, -1)
    return ImageStar(np.asfortranarray(Y), S.C, S.d, S.pl, S.pu, S.trace)


def fc_reach(S, L):
    """FullyConnectedLayer.reach_star_single_input, FullyConnectedLayer.m:295-317
    (ImageStar branch) / Star.affineMap Star.m:313-343: V' = W*reshape(V,N,P+1),
    bias added to column 1.  Result is a 1x1xOut image."""
    M = L["W"] @ S.mat()
    M[:, 0] += L["b"]
    out = M.shape[0]
    return ImageStar(np.asfortranarray(M.reshape(1, 1, out, -1, order="F")), S.C, S.d, S.pl, S.pu, S.trace)


def bn_reach(S, L):
    """BatchNormalizationLayer.reach_star_single_input ImageStar branch,
    BatchNormalizationLayer.m:305-328: four per-channel passes —
    c -= mean; (c,G) = ((c,G).*1)/sqrt(var+eps); (c,G) .*= scale; c += offset."""
    V = S.V.copy(order="F")
    h, w, c, _ = V.shape
    if len(L["mean"]) != c:
        # BatchNormalizationLayer.m:289-302: 1x1xN set with N parameters
        assert h == 1 and w == 1
    mean = np.asarray(L["mean"]).reshape(1, 1, -1)
    V[:, :, :, 0] = V[:, :, :, 0] - mean
    den = np.sqrt(np.asarray(L["var"]) + L["eps"]).reshape(1, 1, -1, 1)
    V = (V * 1.0) / den
    V = V * np.asarray(L["scale"]).reshape(1, 1, -1, 1)
    V[:, :, :, 0] = V[:, :, :, 0] + np.asarray(L["offset"]).reshape(1, 1, -1)
    return ImageStar(np.asfortranarray(V), S.C, S.d, S.pl, S.pu, S.trace)


def avgpool_slices(X, pool, stride, pad, divisor="window"):
    """AveragePooling2DLayer.compute_averageMap, AveragePooling2DLayer.m:316-393:
    zero-pad, sum the window row by row, divide by ph*pw (padding counted) —
    divisor="window", the rule of the pure-MATLAB map and of avgpool on gpuArray
    inputs (AveragePooling2DLayer.m:242-245).  divisor="inside" divides by the
    number of window entries inside the image instead: the rule of MatConvNet's
    vl_nnpool(..., 'Method', 'avg'), which evaluate calls on host arrays (:247);
    that routine ships as a binary only, so this rule is restated from its
    published source (matconvnet, pooling_cpu: the accumulator is built with the
    window clipped to the image) and is not pinned by a reference test."""
    ph, pw = pool
    sh, sw = stride
    Xp = zero_pad(X, pad)
    ho = (Xp.shape[0] - ph) // sh + 1
    wo = (Xp.shape[1] - pw) // sw + 1
    acc = np.zeros((ho, wo) + X.shape[2:], order="F")
    for i in range(ph):
        for j in range(pw):
            acc = acc + Xp[i: i + (ho - 1) * sh + 1: sh, j: j + (wo - 1) * sw + 1: sw]
    if divisor == "window":
        return acc / (ph * pw)
    if divisor != "inside":
        raise ValueError(divisor)
    H, W = X.shape[:2]
    h0 = np.arange(ho) * sh - pad[0]
    w0 = np.arange(wo) * sw - pad[2]
    nh = np.minimum(h0 + ph, H) - np.maximum(h0, 0)
    nw = np.minimum(w0 + pw, W) - np.maximum(w0, 0)
    cnt = np.maximum(np.outer(nh, nw), 1).astype(np.float64)
    return acc / cnt.reshape((ho, wo) + (1,) * (X.ndim - 2))


def avgpool_reach(S, L):
    """AveragePooling2DLayer.reach_star_single_input, AveragePooling2DLayer.m:424-438:
    evaluate applied to V (centre and generators).  L["divisor"] names the rule for padded
    windows (see avgpool_slices); the default is the host-array back end's."""
    Y = avgpool_slices(S.V, L["pool"], L["stride"], L["pad"], L.get("divisor", "inside"))
    return ImageStar(np.asfortranarray(Y), S.C, S.d, S.pl, S.pu, S.trace)


# --------------------------------------------------------------------------
# ReLU approx step


def estimate_ranges(M, pl, pu):
    """Star.estimateRanges, Star.m:1078-1106: four products formed separately,
    lb = c + pos*pl + neg*pu, ub = c + pos*pu + neg*pl (in that order)."""
    G = M[:, 1:]
    pos = np.maximum(G, 0.0)
    neg = np.minimum(G, 0.0)
    if pl.size == 0:
        pl = -np.ones(G.shape[1])
        pu = np.ones(G.shape[1])
    xmin1 = pos @ pl
    xmax1 = pos @ pu
    xmin2 = neg @ pu
    xmax2 = neg @ pl
    lb = M[:, 0] + xmin1 + xmin2
    ub = M[:, 0] + xmax1 + xmax2
    return lb, ub


def relu_reach(S, keep_constraints=True):
    """ReluLayer.reach_star_single_input (ReluLayer.m:103-118) -> PosLin.reach with
    the LP-free construction: PosLin.m:1588-1646 at relaxFactor = 1, built from
    Star.estimateRanges (Star.m:1078-1106), Star.resetRow (Star.m:1442-1461) and
    PosLin.multipleStepReachStarApprox_at_one (PosLin.m:685-742)."""
    h, w, c, p1 = S.V.shape
    N = h * w * c
    P = p1 - 1
    M = S.mat()
    lb, ub = estimate_ranges(M, S.pl, S.pu)
    dead = np.nonzero(ub <= 0)[0]                      # map1
    cross = np.nonzero((lb < 0) & (ub > 0))[0]         # map2 (ascending linear index)
    k = len(cross)
    lbc = lb[cross]
    ubc = ub[cross]
    In = M.copy(order="F")
    In[dead, :] = 0.0                                  # resetRow
    c_idx = In[cross, 0].copy()                        # pre-zeroing rows of the crossing neurons
    G_idx = In[cross, 1:].copy()
    V1 = In
    V1[cross, :] = 0.0
    newM = np.zeros((N, P + 1 + k), order="F")
    newM[:, :P + 1] = V1
    newM[cross, P + 1 + np.arange(k)] = 1.0
    a = ubc / (ubc - lbc)
    b = a * lbc
    new_pl = np.concatenate([S.pl, np.zeros(k)])
    new_pu = np.concatenate([S.pu, ubc])
    if keep_constraints:
        Ik = sp.identity(k, format="csr")
        Gs = sp.csr_matrix(G_idx)
        aG = sp.csr_matrix(G_idx * (-a)[:, None])
        m0 = S.C.shape[0]
        C0 = sp.hstack([S.C, sp.csr_matrix((m0, k))], format="csr")
        C1 = sp.hstack([sp.csr_matrix((k, P)), -Ik], format="csr")
        C2 = sp.hstack([Gs, -Ik], format="csr")
        C3 = sp.hstack([aG, Ik], format="csr")
        newC = sp.vstack([C0, C1, C2, C3], format="csr")
        newd = np.concatenate([S.d, np.zeros(k), -c_idx, a * c_idx - b])
    else:
        newC, newd = S.C, S.d
    trace = S.trace + [{"N": N, "lb": lb, "ub": ub, "dead": dead, "cross": cross,
                        "P_in": P, "P_out": P + k}]
    return ImageStar(newM.reshape(h, w, c, P + 1 + k, order="F"), newC, newd, new_pl, new_pu, trace)


def lp_extreme(f, c0, C, d, pl, pu, maximize):
    """Star.getMax / Star.getMin (Star.m:859-895, :745-781): optimum of c0 + f alpha over C alpha <= d,
    pl <= alpha <= pu through lpsolver (lpsolver.m): all-zero f returns c0, an all-zero C with d >= 0 the
    closed-form box optimum (:34-49), else an LP (HiGHS standing in for linprog)."""
    f = np.asarray(f, dtype=np.float64).ravel()
    if not np.any(f):
        return c0
    sgn = -1.0 if maximize else 1.0
    if (C.shape[0] == 0 or C.nnz == 0) and np.all(np.isfinite(pl)) and np.all(np.isfinite(pu)) and np.all(d >= 0):
        ff = sgn * f
        return sgn * float(np.sum(np.minimum(ff * pl, ff * pu))) + c0
    res = linprog(sgn * f, A_ub=C, b_ub=d, bounds=list(zip(pl, pu)), method="highs")
    if res.status != 0:
        raise RuntimeError("Cannot find an optimal solution, status %d (%s)" % (res.status, res.message))
    return sgn * res.fun + c0


def relu_reach_lp(S):
    """PosLin.reach_star_approx2, PosLin.m:747-857 — the reference's default 'approx-star': the estimated
    ranges only pre-select; every neuron they call crossing gets its true upper bound by an LP (getMaxs,
    :817), those still above zero their true lower bound (getMins, :842); neurons whose LP bounds no longer
    cross are cleared (xmax <= 0) or left untouched (xmin >= 0); the rest is relaxed with the LP bounds by
    multipleStepReachStarApprox_at_one (:685-742), ascending index order."""
    h, w, c, p1 = S.V.shape
    N = h * w * c
    P = p1 - 1
    M = S.mat()
    lb, ub = estimate_ranges(M, S.pl, S.pu)
    map1 = np.nonzero(ub <= 0)[0]
    map2 = np.nonzero((lb < 0) & (ub > 0))[0]
    C = sp.csr_matrix(S.C)
    xmax = np.array([lp_extreme(M[i, 1:], M[i, 0], C, S.d, S.pl, S.pu, True) for i in map2])
    map4 = map2[xmax <= 0] if len(map2) else map2
    dead = np.concatenate([map1, map4]).astype(np.int64)
    keep5 = xmax > 0 if len(map2) else np.zeros(0, bool)
    map6 = map2[keep5]
    xmax1 = xmax[keep5]
    xmin = np.array([lp_extreme(M[i, 1:], M[i, 0], C, S.d, S.pl, S.pu, False) for i in map6])
    keep7 = xmin < 0 if len(map6) else np.zeros(0, bool)
    cross = map6[keep7]
    lbc = xmin[keep7]
    ubc = xmax1[keep7]
    k = len(cross)
    In = M.copy(order="F")
    In[dead, :] = 0.0
    c_idx = In[cross, 0].copy()
    G_idx = In[cross, 1:].copy()
    In[cross, :] = 0.0
    newM = np.zeros((N, P + 1 + k), order="F")
    newM[:, :P + 1] = In
    newM[cross, P + 1 + np.arange(k)] = 1.0
    a = ubc / (ubc - lbc)
    b = a * lbc
    Ik = sp.identity(k, format="csr")
    m0 = S.C.shape[0]
    newC = sp.vstack([sp.hstack([S.C, sp.csr_matrix((m0, k))], format="csr"),
                      sp.hstack([sp.csr_matrix((k, P)), -Ik], format="csr"),
                      sp.hstack([sp.csr_matrix(G_idx), -Ik], format="csr"),
                      sp.hstack([sp.csr_matrix(G_idx * (-a)[:, None]), Ik], format="csr")], format="csr")
    newd = np.concatenate([S.d, np.zeros(k), -c_idx, a * c_idx - b])
    trace = S.trace + [{"N": N, "lb": lb, "ub": ub, "dead": np.sort(dead), "cross": cross, "cross_est": map2,
                        "lb_lp": lbc, "ub_lp": ubc, "P_in": P, "P_out": P + k}]
    return ImageStar(newM.reshape(h, w, c, P + 1 + k, order="F"), newC, newd,
                     np.concatenate([S.pl, np.zeros(k)]), np.concatenate([S.pu, ubc]), trace)


def _matlab_round(x):
    """MATLAB round: halves away from zero (Python's round goes to even)."""
    return int(np.floor(x + 0.5)) if x >= 0 else -int(np.floor(-x + 0.5))


def relax_selection(method, relax_factor, lb2, ub2, rng=None):
    """Which of the neurons the estimated ranges call crossing get LP-optimised ranges, and the order of the rest:
    n1 = round((1 - relaxFactor) * numel(map2)) neurons, picked by
      'relax-star-area'   largest triangle area 0.5*|ub|*|lb| first   (PosLin.m:1044-1052)
      'relax-star-range'  largest ub - lb first                        (PosLin.m:929-936)
      'relax-star-static' the first n1 in index order                  (PosLin.m:1599-1607)
      'relax-star-random' randperm (not reproducible across RNGs)      (PosLin.m:1483-1491)
    (MATLAB's sort is stable: ties keep index order).  Returns (positions of map21, positions of map22) within
    map2, each in the reference's order."""
    k = len(lb2)
    n1 = _matlab_round((1.0 - relax_factor) * k)
    if method == "relax-star-area":
        order = np.argsort(-(0.5 * np.abs(ub2) * np.abs(lb2)), kind="stable")
    elif method == "relax-star-range":
        order = np.argsort(-(ub2 - lb2), kind="stable")
    elif method == "relax-star-static":
        order = np.arange(k)
    elif method == "relax-star-random":
        rng = rng or np.random.default_rng(0)
        pick = rng.permutation(k)[:n1]
        rest = np.setdiff1d(np.arange(k), pick)              # setdiff(map2, map21, 'stable'): index order
        return pick, rest
    else:
        raise ValueError(method)
    return order[:n1], order[n1:]


def relu_reach_relaxed(S, method, relax_factor, rng=None):
    """PosLin.reach_relaxed_star_area / _range / _static / _random (PosLin.m:986-1105, 863-984, 1541-1646,
    1425-1539): estimated ranges classify; of the crossing neurons only the selected share gets LP bounds
    (getMaxs, then getMins where the maximum is positive); the others keep the estimated bounds.  New predicates
    are appended in the reference's order map9 = [map22; map8]: first the neurons without optimised ranges (in
    selection order), then the optimised ones that still cross."""
    h, w, c, p1 = S.V.shape
    N = h * w * c
    P = p1 - 1
    M = S.mat()
    lb, ub = estimate_ranges(M, S.pl, S.pu)
    map1 = np.nonzero(ub <= 0)[0]
    map2 = np.nonzero((lb < 0) & (ub > 0))[0]
    p21, p22 = relax_selection(method, relax_factor, lb[map2], ub[map2], rng)
    map21, map22 = map2[p21], map2[p22]
    C = sp.csr_matrix(S.C)
    xmax = np.array([lp_extreme(M[i, 1:], M[i, 0], C, S.d, S.pl, S.pu, True) for i in map21])
    map4 = map21[xmax <= 0] if len(map21) else map21
    dead = np.concatenate([map1, map4]).astype(np.int64)
    keep5 = xmax > 0 if len(map21) else np.zeros(0, bool)
    map6 = map21[keep5]
    xmax1 = xmax[keep5]
    xmin = np.array([lp_extreme(M[i, 1:], M[i, 0], C, S.d, S.pl, S.pu, False) for i in map6])
    keep7 = xmin < 0 if len(map6) else np.zeros(0, bool)
    map8 = map6[keep7]
    cross = np.concatenate([map22, map8]).astype(np.int64)                      # map9
    lbc = np.concatenate([lb[map22], xmin[keep7] if len(map6) else np.zeros(0)])
    ubc = np.concatenate([ub[map22], xmax1[keep7] if len(map6) else np.zeros(0)])
    k = len(cross)
    In = M.copy(order="F")
    In[dead, :] = 0.0
    c_idx = In[cross, 0].copy()
    G_idx = In[cross, 1:].copy()
    In[cross, :] = 0.0
    newM = np.zeros((N, P + 1 + k), order="F")
    newM[:, :P + 1] = In
    newM[cross, P + 1 + np.arange(k)] = 1.0
    a = ubc / (ubc - lbc)
    b = a * lbc
    Ik = sp.identity(k, format="csr")
    m0 = S.C.shape[0]
    newC = sp.vstack([sp.hstack([S.C, sp.csr_matrix((m0, k))], format="csr"),
                      sp.hstack([sp.csr_matrix((k, P)), -Ik], format="csr"),
                      sp.hstack([sp.csr_matrix(G_idx), -Ik], format="csr"),
                      sp.hstack([sp.csr_matrix(G_idx * (-a)[:, None]), Ik], format="csr")], format="csr")
    newd = np.concatenate([S.d, np.zeros(k), -c_idx, a * c_idx - b])
    trace = S.trace + [{"N": N, "lb": lb, "ub": ub, "dead": np.sort(dead), "cross": cross, "cross_est": map2,
                        "optimised": map21, "lb_lp": lbc, "ub_lp": ubc, "P_in": P, "P_out": P + k}]
    return ImageStar(newM.reshape(h, w, c, P + 1 + k, order="F"), newC, newd,
                     np.concatenate([S.pl, np.zeros(k)]), np.concatenate([S.pu, ubc]), trace)


# --------------------------------------------------------------------------
# network driver and verdict


def image_input_reach(S, L):
    """ImageInputLayer.reach_star_single_input, ImageInputLayer.m:121-168, with ImageStar.affineMap
    (ImageStar.m:431-460: generators scaled, offset added to the centre).  L: {"normalization", "mean",
    "std", "min", "max"} (the last four may be None)."""
    V = S.V.copy()
    norm = L.get("normalization", "none")

    def arr(x):
        a = np.asarray(x, dtype=np.float64)
        return a.reshape(a.shape + (1,) * (3 - a.ndim)) if a.ndim < 3 else a

    if norm == "none":
        pass
    elif norm == "zerocenter":
        V[..., 0] = V[..., 0] + (-arr(L["mean"]))
    elif norm == "zscore":
        V[..., 0] = V[..., 0] + (-arr(L["mean"]))
        std = np.asarray(L["std"], dtype=np.float64).ravel()
        for nc in range(V.shape[2]):
            V[:, :, nc, :] = V[:, :, nc, :] / std[nc if std.size > 1 else 0]
    elif norm == "rescale-zero-one":
        if L.get("min") is not None and L.get("max") is not None:
            V[..., 0] = V[..., 0] + (-arr(L["min"]))
            V = V * (1.0 / (float(L["max"]) - float(L["min"])))
        else:
            V = V * (1 / 255)
    elif norm == "rescale-symmetric":
        if L.get("min") is not None and L.get("max") is not None:
            V[..., 0] = V[..., 0] + (-arr(L["min"]))
            V = V * (2.0 / (float(L["max"]) - float(L["min"])))
            V[..., 0] = V[..., 0] + (-1)
        else:
            V = V * (2 / 255)
            V[..., 0] = V[..., 0] + (-1)
    else:
        raise ValueError("The normalization method is not supported yet.")
    return ImageStar(V, S.C, S.d, S.pl, S.pu, S.trace)


def flatten_order(shape, kind):
    """Source index (column-major position in the H x W x C image) of every entry of the flattened vector,
    FlattenLayer.evaluate, FlattenLayer.m:105-164.  'nnet.cnn.layer.FlattenLayer' is a plain reshape;
    'nnet.keras.layer.FlattenCStyleLayer' permutes [3 2 1] first, the ONNX types [2 1 3]."""
    h, w, c = shape
    idx = np.arange(h * w * c).reshape((h, w, c), order="F")
    if kind == "nnet.cnn.layer.FlattenLayer":
        return idx.reshape(-1, order="F")
    if kind == "nnet.keras.layer.FlattenCStyleLayer":
        return np.transpose(idx, (2, 1, 0)).reshape(-1, order="F")
    if kind in ("nnet.onnx.layer.FlattenLayer", "nnet.onnx.layer.FlattenInto2dLayer",
                "nnet.onnx.layer.Flatten3dInto2dLayer"):
        return np.transpose(idx, (1, 0, 2)).reshape(-1, order="F")
    raise ValueError("Unknown type of flatten layer")


def flatten_reach(S, L):
    """FlattenLayer.reach_single_input (FlattenLayer.m:172-183): evaluate applied to every slice of V;
    the result is a 1 x 1 x N ImageStar."""
    src = flatten_order(S.shape, L["kind"])
    M = S.mat()[src, :]
    return ImageStar(M.reshape((1, 1, M.shape[0], M.shape[1]), order="F"), S.C, S.d, S.pl, S.pu, S.trace)


def reach(layers, S, keep_constraints=True, lp_bounds=False, relax=None):
    """NN.reach_noConns layer loop, NN.m:1529-1551.  lp_bounds: the ReLU layers use the LP-tightened
    step (reference default 'approx-star', relaxFactor = 0) instead of the estimated bounds.  relax =
    (method, relaxFactor): the 'relax-star-*' step with LPs for a share of the crossing neurons."""
    for L in layers:
        t = L["type"]
        if t == "imageinput":
            S = image_input_reach(S, L)
        elif t == "flatten":
            S = flatten_reach(S, L)
        elif t == "conv2d":
            S = conv2d_reach(S, L)
        elif t == "fc":
            S = fc_reach(S, L)
        elif t == "bn":
            S = bn_reach(S, L)
        elif t == "avgpool":
            S = avgpool_reach(S, L)
        elif t == "relu":
            if relax is not None:
                S = relu_reach_relaxed(S, relax[0], relax[1])
            else:
                S = relu_reach_lp(S) if lp_bounds else relu_reach(S, keep_constraints)
        else:
            raise ValueError(t)
    return S


def robustness_set(n_out, target, class_type="max"):
    """NN.robustness_set, NN.m:1334-1368 (target 0-based here): n_out-1 halfspaces
    G x <= 0; 'max': x_target - x_i <= 0 ... encoded as row e_target - e_i;
    'min': row e_i - e_target."""
    G = np.eye(n_out)
    G = np.delete(G, target, axis=0)
    if class_type == "max":
        G = -G
        G[:, target] = 1.0
    elif class_type == "min":
        G[:, target] = -1.0
    else:
        raise ValueError(class_type)
    return G, np.zeros(G.shape[0])


def is_empty_set(C, d, pl, pu):
    """Star.isEmptySet, Star.m:1216-1232 -> lpsolver(0, C, d, [], [], pl, pu)
    (lpsolver.m:99-128; box-only closed form :34-49).  HiGHS stands in for
    linprog/glpk."""
    C = sp.csr_matrix(C)
    d = np.asarray(d, float).ravel()
    P = C.shape[1]
    if C.nnz == 0 and pl.size and np.all(np.isfinite(pl)) and np.all(np.isfinite(pu)) and np.all(d >= 0):
        return False                                   # box-only fast path: feasible
    bounds = list(zip(pl, pu)) if pl.size else [(None, None)] * P
    res = linprog(np.zeros(P), A_ub=C, b_ub=d, bounds=bounds, method="highs")
    if res.status == 0:
        return False
    if res.status == 2:
        return True
    raise RuntimeError("LP solver status %d: %s" % (res.status, res.message))


def intersect_halfspace_system(S, H, g):
    """Star.intersectHalfSpace, Star.m:555-589: C1 = H*V(:,2:end),
    d1 = g - H*V(:,1); returns the stacked system ([C; C1], [d; d1])."""
    M = S.mat()
    H = np.atleast_2d(H)
    C1 = H @ M[:, 1:]
    d1 = np.asarray(g, float).ravel() - H @ M[:, 0]
    newC = sp.vstack([S.C, sp.csr_matrix(C1)], format="csr")
    newd = np.concatenate([S.d, d1])
    return newC, newd


def verify_specification(S, G, g):
    """verify_specification.m:36-79 with NN.checkRobust (NN.m:617-648): OR over
    halfspaces; 1 iff every intersection is empty, 2 at the first non-empty."""
    for i in range(G.shape[0]):
        C, d = intersect_halfspace_system(S, G[i:i + 1], g[i:i + 1])
        if not is_empty_set(C, d, S.pl, S.pu):
            return 2
    return 1


def verify_robustness(layers, q, keep_trace=False):
    """NN.verify_robustness, NN.m:651-667, for one workload query."""
    S = reach(layers, star_from_query(q))
    n_out = S.mat().shape[0]
    G, g = robustness_set(n_out, q["target"], q.get("spec", "max"))
    v = verify_specification(S, G, g)
    return (v, S) if keep_trace else v


def evaluate(layers, x):
    """NN.evaluate (NN.m:130-145 -> evaluate_noConns :1416-1425): each layer's evaluate on one concrete input
    x[H,W,C] (or a vector): the affine layer maps above applied to a set without generators, and
    PosLin.evaluate = max(x, 0) for ReLU.  Returns the output, column-major flattened."""
    x = np.asarray(x, dtype=np.float64)
    if x.ndim == 1:
        x = x.reshape(-1, 1, 1)
    if x.ndim == 2:
        x = x[:, :, None]
    S = ImageStar(np.asfortranarray(x[..., None]), sp.csr_matrix((0, 0)), np.zeros(0), np.zeros(0), np.zeros(0))
    for L in layers:
        t = L["type"]
        if t == "relu":
            S = ImageStar(np.maximum(S.V, 0.0), S.C, S.d, S.pl, S.pu)
        elif t == "imageinput":
            S = image_input_reach(S, L)
        elif t == "flatten":
            S = flatten_reach(S, L)
        elif t == "conv2d":
            S = conv2d_reach(S, L)
        elif t == "fc":
            S = fc_reach(S, L)
        elif t == "bn":
            S = bn_reach(S, L)
        elif t == "avgpool":
            S = avgpool_reach(S, L)
        else:
            raise ValueError(t)
    return S.V[..., 0].reshape(-1, order="F")


def halfspace_contains(G, g, y):
    """HalfSpace.contains (HalfSpace.m:35-55): no entry of g - G*y is negative."""
    return not np.any(np.asarray(g, float).ravel() - np.atleast_2d(G) @ y < 0)


def falsify(layers, points, G, g):
    """NN.falsify (NN.m:930-988) on given sample points (the reference draws them with Star.sample /
    MATLAB's rand; a caller hands the same points to both implementations): the points whose output lies in
    one of the halfspaces G[j] x <= g[j]."""
    out = []
    for x in points:
        y = evaluate(layers, x)
        if any(halfspace_contains(G[j:j + 1], g[j:j + 1], y) for j in range(G.shape[0])):
            out.append(x)
    return out


def verify_sample(layers, q, image, verdict_fn=None):
    """examples/Tutorial/SPIE/Classification2D/verifySample.m:1-32 for a bounds-form workload query: -1
    misclassified image, 0 when the upper- or lower-bound image is classified differently, else
    verify_robustness."""
    t = q["target"]
    if int(np.argmax(evaluate(layers, image))) != t:
        return -1
    if int(np.argmax(evaluate(layers, q["ub"]))) != t or int(np.argmax(evaluate(layers, q["lb"]))) != t:
        return 0
    return (verdict_fn or verify_robustness)(layers, q)


def output_ranges(S):
    """Star.estimateRanges of the final set."""
    return estimate_ranges(S.mat(), S.pl, S.pu)
