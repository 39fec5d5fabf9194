"""Pin the CPU oracle against the reference's own known-answer tests and stored
.mat baselines (fixtures: tests/golden/reference_kats.npz, written by
tests/golden/make_golden.py with the file:line of every item)."""
import numpy as np
import scipy.sparse as sp
from scipy.optimize import linprog

from oracle import nnv_oracle as O


def test_conv_feature_map_kat(kats):
    X = kats["conv_I"][:, :, None, None]
    W = kats["conv_W"][:, :, None, None]
    Y = O.conv2d_slices(X, W, (0, 0, 0, 0), (1, 1), (1, 1))
    assert np.array_equal(Y[:, :, 0, 0], kats["conv_expected"])


def test_zero_padding_kat(kats):
    vol = kats["pad_vol"]
    I = O.zero_pad(vol, (1, 1, 1, 1))
    assert I.shape == (7, 7, 3)
    assert np.array_equal(I[1:-1, 1:-1, :], vol)
    assert not I[0].any() and not I[-1].any() and not I[:, 0].any() and not I[:, -1].any()


def test_avgpool_kats(kats):
    Y = O.avgpool_slices(kats["avg_I"][:, :, None, None], (2, 2), (2, 2), (0, 0, 0, 0))[:, :, 0, 0]
    I = kats["avg_I"]
    chk = np.array([[I[0:2, 0:2].sum() / 4, I[0:2, 2:4].sum() / 4], [I[2:4, 0:2].sum() / 4, I[2:4, 2:4].sum() / 4]])
    assert np.array_equal(Y, chk)
    assert np.array_equal(Y, kats["avg_expected_mat"])          # stored MATLAB output
    Y2 = O.avgpool_slices(kats["avg2_I"][:, :, None, None], (2, 2), (2, 2), (0, 0, 0, 0))[:, :, 0, 0]
    assert np.abs(Y2 - kats["avg2_expected"]).max() < 1e-10
    vol = kats["avg_vol"]
    Y3 = O.avgpool_slices(vol[:, :, :, None], (3, 3), (2, 2), (0, 0, 0, 0))[:, :, :, 0]
    for i in range(3):
        for j in range(2):
            for k in range(2):
                assert abs(Y3[j, k, i] - vol[2 * j:2 * j + 3, 2 * k:2 * k + 3, i].sum() / 9) <= 10 * np.finfo(float).eps


def test_fc_kat(kats):
    S = O.ImageStar(kats["fc_x"].reshape(2, 1, 1, 1), sp.csr_matrix((0, 0)), np.zeros(0), np.zeros(0), np.zeros(0))
    R = O.fc_reach(S, {"W": kats["fc_W"], "b": kats["fc_b"]})
    assert np.abs(R.mat()[:, 0] - kats["fc_expected"]).max() < 1e-10


def test_bn_closed_form(kats):
    mean, var, eps, scale, offset = kats["bn_params"]
    rng = np.random.default_rng(42)
    x = rng.uniform(size=(4, 4, 1, 2))
    S = O.ImageStar(np.asfortranarray(x), sp.csr_matrix((1, 1)), np.zeros(1), -np.ones(1), np.ones(1))
    L = {"mean": [mean], "var": [var], "eps": eps, "scale": [scale], "offset": [offset]}
    R = O.bn_reach(S, L)
    exp_c = scale * (x[..., 0] - mean) / np.sqrt(var + eps) + offset
    exp_g = scale * x[..., 1] / np.sqrt(var + eps)
    assert np.abs(R.V[..., 0] - exp_c).max() < 1e-10
    assert np.abs(R.V[..., 1] - exp_g).max() < 1e-10
    ident = {"mean": np.zeros(5), "var": np.ones(5), "eps": 0.0, "scale": np.ones(5), "offset": np.zeros(5)}
    S5 = O.ImageStar(np.arange(1., 6.).reshape(1, 1, 5, 1), sp.csr_matrix((0, 0)), np.zeros(0), np.zeros(0), np.zeros(0))
    assert np.array_equal(O.bn_reach(S5, ident).V, S5.V)


def test_relu_evaluate_kats(kats):
    assert np.array_equal(np.maximum(kats["relu_IM"], 0), kats["relu_IM_out"])
    assert np.array_equal(np.maximum(kats["poslin_x"], 0), kats["poslin_y"])


def test_identity_maps_and_sign_cases():
    # code/nnv/tests/soundness/test_regression_reachability.m:6-79
    c = np.array([1., 2., 3.])
    S = O.ImageStar(np.hstack([c[:, None], np.eye(3)]).reshape(3, 1, 1, 4, order="F"),
                    sp.csr_matrix(np.vstack([np.eye(3), -np.eye(3)])), np.ones(6), -np.ones(3), np.ones(3))
    R = O.fc_reach(S, {"W": np.eye(3), "b": np.zeros(3)})
    assert np.abs(R.mat()[:, 0] - c).max() < 1e-10
    V = np.zeros((3, 3, 1, 2))
    V[:, :, 0, 0] = np.arange(1., 10.).reshape(3, 3)
    V[:, :, 0, 1] = 0.05
    Si = O.ImageStar(np.asfortranarray(V), sp.csr_matrix([[1.], [-1.]]), np.ones(2), -np.ones(1), np.ones(1))
    W = np.ones((1, 1, 1, 2))
    R = O.conv2d_reach(Si, {"W": W, "b": np.zeros(2), "pad": (0, 0, 0, 0), "stride": (1, 1), "dilation": (1, 1)})
    assert np.abs(R.V[:, :, 0, 0] - V[:, :, 0, 0]).max() < 1e-10
    for sign in (+1, -1):
        c = sign * np.array([2., 3., 4.])
        S = O.ImageStar(np.hstack([c[:, None], 0.1 * np.eye(3)]).reshape(3, 1, 1, 4, order="F"),
                        sp.csr_matrix(np.vstack([np.eye(3), -np.eye(3)])), 0.5 * np.ones(6), -0.5 * np.ones(3),
                        0.5 * np.ones(3))
        R = O.relu_reach(S)
        assert R.P == 3                                   # no crossing neuron, no new predicate
        assert np.abs(R.mat()[:, 0] - np.maximum(c, 0)).max() < 1e-10


def test_relu_reach_attack_set(kats):
    # code/nnv/tests/nn/layers/ReluLayer/test_layers_relu.m:36-55: ImageStar(IM, LB, UB) -> approx-star reach
    IM, LB, UB = kats["relu_reach_IM"], kats["relu_reach_LB"], kats["relu_reach_UB"]
    # ImageStar(IM, LB, UB) (ImageStar.m:229-300) is the box IM+LB .. IM+UB
    S = O.star_from_bounds(IM + LB, IM + UB)
    assert S.P == 6                                      # six perturbed pixels
    R = O.relu_reach(S)
    lb, ub = O.output_ranges(R)
    assert np.all(lb >= -1e-12)
    # only pixel (1,1,2) = 0 +- 0.1 crosses zero; the other five stay positive
    assert list(R.trace[0]["cross"]) == [16] and R.P == 7


def test_is_empty_set_baseline(kats):
    C, d = kats["empty_S_C"], kats["empty_S_d"].ravel()
    assert O.is_empty_set(C, d, np.zeros(0), np.zeros(0)) == bool(kats["empty_b_nonempty"][0, 0])
    C1, d1 = kats["empty_S1_C"], kats["empty_S1_d"].ravel()
    assert O.is_empty_set(C1, d1, np.zeros(0), np.zeros(0)) == bool(kats["empty_b_empty"][0, 0])


def test_intersect_halfspace_baseline(kats):
    V = kats["hs_S_V"]
    C_all, d_all = kats["hs_S1_C"], kats["hs_S1_d"].ravel()
    S = O.ImageStar(V.reshape(2, 1, 1, 4, order="F"), sp.csr_matrix(C_all[:-1]), d_all[:-1], np.zeros(0), np.zeros(0))
    C, d = O.intersect_halfspace_system(S, kats["hs_H"], kats["hs_g"])
    assert np.array_equal(C.toarray(), C_all)
    assert np.array_equal(d, d_all)
    assert O.is_empty_set(C, d, np.zeros(0), np.zeros(0)) == bool(kats["hs_S1_isEmpty"][0, 0])


def test_affine_map_baseline(kats):
    V = kats["aff_S_V"]
    S = O.ImageStar(V.reshape(2, 1, 1, 4, order="F"), sp.csr_matrix((0, 3)), np.zeros(0), -np.ones(3), np.ones(3))
    R = O.fc_reach(S, {"W": kats["aff_W"], "b": kats["aff_b"].ravel()})
    assert np.abs(R.mat() - kats["aff_S1_V"]).max() < 1e-12
    # Star(lb,ub) -> affineMap(W2) -> ranges (test_star_affineMap.m:58-66, :91): a box star's exact
    # ranges equal its estimated ranges
    S3 = O.star_from_bounds(np.array([0., -1., 0.]), np.array([1., 1., 1.]))
    S4 = O.fc_reach(S3, {"W": kats["aff_W2"], "b": np.zeros(3)})
    lb, ub = O.output_ranges(S4)
    assert np.abs(lb - kats["aff_S4_lb"].ravel()).max() < 1e-6     # baseline tolerance of the reference
    assert np.abs(ub - kats["aff_S4_ub"].ravel()).max() < 1e-6


def test_get_box_fast_baseline(kats):
    # Star.getBoxFast (Star.m:658-677): predicate bounds of the polytope (an LP per predicate), then the
    # zonotope box == estimateRanges with those bounds.
    V, C, d = kats["box_I1_V"], kats["box_I1_C"], kats["box_I1_d"].ravel()
    P = C.shape[1]
    pl, pu = np.zeros(P), np.zeros(P)
    for i in range(P):
        e = np.zeros(P)
        e[i] = 1
        pl[i] = linprog(e, A_ub=C, b_ub=d, bounds=[(None, None)] * P, method="highs").fun
        pu[i] = -linprog(-e, A_ub=C, b_ub=d, bounds=[(None, None)] * P, method="highs").fun
    lb, ub = O.estimate_ranges(V, pl, pu)
    assert np.abs(lb - kats["box_B2_lb"].ravel()).max() < 1e-6
    assert np.abs(ub - kats["box_B2_ub"].ravel()).max() < 1e-6


def test_box_to_star_construction():
    # Box.m:16-58 / Star.m:220-237: zero-width entries produce no generator
    lb = np.array([0., 1., -1., 2.])
    ub = np.array([1., 1., 1., 2.])
    S = O.star_from_bounds(lb, ub)
    assert S.P == 2
    M = S.mat()
    assert np.array_equal(M[:, 0], [0.5, 1., 0., 2.])
    assert np.array_equal(M[:, 1], [0.5, 0, 0, 0]) and np.array_equal(M[:, 2], [0, 0, 1., 0])
    assert S.C.shape == (1, 2) and S.C.nnz == 0 and np.array_equal(S.d, [0.])
    assert np.array_equal(S.pl, [-1, -1]) and np.array_equal(S.pu, [1, 1])


def test_avgpool_divisor_rules():
    """Padded windows: "window" divides by ph*pw (compute_averageMap), "inside" by the entries inside the image
    (the host-array back end of AveragePooling2DLayer.evaluate); without padding the two agree."""
    rng = np.random.default_rng(5)
    X = rng.standard_normal((7, 9, 2, 3))
    pool, stride, pad = (3, 2), (2, 1), (1, 0, 1, 1)
    Xp = np.pad(X, ((1, 0), (1, 1), (0, 0), (0, 0)))
    ho, wo = (8 - 3) // 2 + 1, (11 - 2) // 1 + 1
    for rule in ("window", "inside"):
        Y = O.avgpool_slices(X, pool, stride, pad, rule)
        assert Y.shape == (ho, wo, 2, 3)
        for oh in range(ho):
            for ow in range(wo):
                win = Xp[oh * 2: oh * 2 + 3, ow: ow + 2]
                h0, w0 = oh * 2 - 1, ow - 1
                inside = (min(h0 + 3, 7) - max(h0, 0)) * (min(w0 + 2, 9) - max(w0, 0))
                ref = win.sum(axis=(0, 1)) / (6 if rule == "window" else inside)
                assert np.allclose(Y[oh, ow], ref, rtol=1e-14, atol=1e-15)
    a = O.avgpool_slices(X, (2, 2), (2, 2), (0, 0, 0, 0), "window")
    b = O.avgpool_slices(X, (2, 2), (2, 2), (0, 0, 0, 0), "inside")
    assert np.array_equal(a, b)


def test_conv_backends_agree():
    rng = np.random.default_rng(6)
    X = np.asfortranarray(rng.standard_normal((9, 7, 5, 40)))
    W = rng.standard_normal((3, 2, 5, 6))
    a = O.conv2d_slices(X, W, (1, 0, 2, 1), (2, 1), (1, 2))
    O.set_conv_backend("torch")
    try:
        b = O.conv2d_slices(X, W, (1, 0, 2, 1), (2, 1), (1, 2))
    finally:
        O.set_conv_backend("numpy")
    assert a.shape == b.shape and np.abs(a - b).max() <= 1e-13 * np.abs(a).max()


def test_relax_star_selection_and_limits():
    """The 'relax-star-*' step with an LP share (PosLin.m:863-1105, 1541-1646) pinned at its two ends and on a
    hand-worked selection: relaxFactor = 0 with the static order is reach_star_approx2 (every crossing neuron
    optimised, ascending order); relaxFactor = 1 optimises nothing and is the LP-free step up to the order of
    the new predicates; n1 = round((1 - relaxFactor) * count) rounds halves up as MATLAB does."""
    from nnv_b200.configs import make_config
    lb2 = np.array([-1.0, -4.0, -2.0, -1.0, -3.0])
    ub2 = np.array([2.0, 1.0, 2.0, 2.0, 1.0])
    # areas 1, 2, 2, 1, 1.5 -> descending, ties in index order: 1, 2, 4, 0, 3; n1 = round(0.5 * 5) = 3
    p21, p22 = O.relax_selection("relax-star-area", 0.5, lb2, ub2)
    assert list(p21) == [1, 2, 4] and list(p22) == [0, 3]
    # ranges 3, 5, 4, 3, 4 -> 1, 2, 4, 0, 3; n1 = round(0.75 * 5) = 4
    p21, p22 = O.relax_selection("relax-star-range", 0.25, lb2, ub2)
    assert list(p21) == [1, 2, 4, 0] and list(p22) == [3]
    p21, p22 = O.relax_selection("relax-star-static", 0.5, lb2, ub2)
    assert list(p21) == [0, 1, 2] and list(p22) == [3, 4]
    cfg = make_config("fc5", n_queries=3)
    for qu in cfg["queries"]:
        S0 = O.star_from_query(qu)
        A = O.reach(cfg["layers"], S0, lp_bounds=True)
        B = O.reach(cfg["layers"], S0, relax=("relax-star-static", 0.0))
        assert A.V.shape == B.V.shape and np.array_equal(A.V, B.V) and np.array_equal(A.pu, B.pu)
        E = O.reach(cfg["layers"], S0)
        F = O.reach(cfg["layers"], S0, relax=("relax-star-area", 1.0))
        assert E.V.shape == F.V.shape
        for te, tf in zip(E.trace, F.trace):
            assert np.array_equal(np.sort(tf["cross"]), te["cross"]) and len(tf["optimised"]) == 0
        # same set, new predicates permuted: the output ranges agree
        le, ue = O.estimate_ranges(E.mat(), E.pl, E.pu)
        lf, uf = O.estimate_ranges(F.mat(), F.pl, F.pu)
        assert np.allclose(le, lf, rtol=1e-12, atol=1e-12) and np.allclose(ue, uf, rtol=1e-12, atol=1e-12)
