"""Host-side mirror of the reference API (no GPU needed): constructors, their
error behaviour, the robustness specification and option validation."""
import numpy as np
import pytest

from nnv_b200 import nn
from nnv_b200.configs import make_config, out_shape
from oracle import nnv_oracle as O


def test_imagestar_from_bounds_matches_oracle():
    rng = np.random.default_rng(0)
    lb = rng.uniform(size=(4, 3, 2))
    ub = lb + rng.uniform(size=(4, 3, 2)) * (rng.uniform(size=(4, 3, 2)) > 0.3)
    I = nn.ImageStar(lb, ub)
    S = O.star_from_bounds(lb, ub)
    assert I.numPred == S.P
    assert np.array_equal(I.V, S.V)
    assert np.array_equal(I.pred_lb, S.pl) and np.array_equal(I.pred_ub, S.pu)
    assert I.C.shape == (1, S.P) and not I.C.any() and np.array_equal(I.d, [0.0])
    St = I.toStar()
    assert St.dim == 24 and St.nVar == S.P and np.array_equal(St.V, S.mat())


def test_imagestar_constructor_errors():
    with pytest.raises(ValueError, match="Inconsistency between lower bound image and upper bound image"):
        nn.ImageStar(np.zeros((2, 2, 1)), np.zeros((2, 3, 1)))
    with pytest.raises(ValueError, match="Invalid number of input arguments"):
        nn.ImageStar(np.zeros((2, 2, 1)))
    V = np.zeros((2, 2, 1, 3))
    with pytest.raises(ValueError, match="constraint matrix"):
        nn.ImageStar(V, np.zeros((1, 5)), np.zeros(1), -np.ones(2), np.ones(2))
    with pytest.raises(ValueError, match="predicate"):
        nn.ImageStar(V, np.zeros((1, 2)), np.zeros(1), -np.ones(3), np.ones(3))


def test_star_constructor_errors():
    with pytest.raises(ValueError, match="Inconsistency between basic matrix and constraint matrix"):
        nn.Star(np.zeros((2, 3)), np.zeros((1, 3)), np.zeros(1))
    with pytest.raises(ValueError, match="constraint vector"):
        nn.Star(np.zeros((2, 3)), np.zeros((2, 2)), np.zeros(1))
    with pytest.raises(ValueError, match="Inconsistent dimensions between lb and ub"):
        nn.Star(np.zeros(2), np.zeros(3))
    S = nn.Star(np.array([0., -1.]), np.array([1., 1.]))
    assert S.dim == 2 and S.nVar == 2
    with pytest.raises(ValueError, match="Inconsistent dimension in the ImageStar"):
        S.toImageStar(3, 1, 1)


def test_layer_constructor_errors():
    with pytest.raises(ValueError, match="filter weights and filter biases"):
        nn.Conv2DLayer(np.zeros((3, 3, 1, 2)), np.zeros(3))
    with pytest.raises(ValueError, match="Invalid padding size"):
        nn.Conv2DLayer(np.zeros((3, 3, 1, 2)), np.zeros(2), PaddingSize=(1, 1))
    with pytest.raises(ValueError, match="weight matrix and bias vector"):
        nn.FullyConnectedLayer(np.zeros((2, 3)), np.zeros(3))
    with pytest.raises(ValueError):
        nn.AveragePooling2DLayer((2,), (2, 2))


def test_robustness_set_matches_reference_construction():
    net = nn.NN([nn.FullyConnectedLayer(np.zeros((4, 3)), np.zeros(4))])
    for kind in ("max", "min"):
        for t in range(1, 5):
            hs = net.robustness_set(t, kind)
            G = np.vstack([h.G for h in hs])
            Go, go = O.robustness_set(4, t - 1, kind)
            assert np.array_equal(G, Go) and all(h.g[0] == 0 for h in hs)
    # NN.m:1343-1345
    with pytest.raises(ValueError, match="Target idx must be less than or equal"):
        net.robustness_set(5)


def test_reach_option_validation():
    v = nn._validate_reach_options
    assert v(None)["reachMethod"] == "approx-star"
    assert v({"reachMethod": "relax-star-area", "relaxFactor": 1})["relaxFactor"] == 1
    with pytest.raises(NotImplementedError):
        v({"reachMethod": "exact-star"})
    assert v({"reachMethod": "relax-star-range", "relaxFactor": 0.5})["relaxFactor"] == 0.5
    with pytest.raises(NotImplementedError):      # upper and lower bounds of different neurons: not built
        v({"reachMethod": "relax-star-ub", "relaxFactor": 0.5})
    with pytest.raises(ValueError, match="relax factor"):
        v({"reachMethod": "relax-star-area", "relaxFactor": 1.5})
    with pytest.raises(TypeError, match="Wrong input set type"):
        nn.NN([nn.ReluLayer()]).reach(np.zeros(3))


def test_halfspace_and_lp_emptiness(kats):
    H = nn.HalfSpace([[1.0, 0.0]], [0.5])
    assert H.dim == 2
    with pytest.raises(ValueError):
        nn.HalfSpace(np.zeros((2, 2)), np.zeros(3))
    # stored baseline of the reference's isEmptySet test
    S = nn.Star(kats["empty_S_V"], kats["empty_S_C"], kats["empty_S_d"].ravel())
    S1 = nn.Star(kats["empty_S1_V"], kats["empty_S1_C"], kats["empty_S1_d"].ravel())
    assert S.isEmptySet() == bool(kats["empty_b_nonempty"][0, 0])
    assert S1.isEmptySet() == bool(kats["empty_b_empty"][0, 0])


def test_config_shapes():
    for name in ("fc5", "cnn28", "cnn32", "bright28"):
        cfg = make_config(name, n_queries=1, small=(name != "fc5"))
        h, w, c = out_shape(cfg["layers"], cfg["in_shape"])
        assert (h, w) == (1, 1) and c in (5, 10)
    cfg = make_config("cnn28", n_queries=1)
    fc = [l for l in cfg["layers"] if l["type"] == "fc"][0]
    assert fc["W"].shape == (128, 2704)          # 13 x 13 x 16 after the stride-2 convolution
    cfg = make_config("cnn32", n_queries=1)
    fc = [l for l in cfg["layers"] if l["type"] == "fc"][0]
    assert fc["W"].shape == (256, 4096)


def test_flatten_layer_types_fold_into_the_next_fc_layer():
    """FlattenLayer.m:105-164: the plain type is the column-major order itself, the Keras C-style and ONNX
    types permute first; the host folds the permutation into the FC weight columns."""
    rng = np.random.default_rng(0)
    shape = (4, 3, 2)
    x = rng.standard_normal(shape)
    S = O.star_from_bounds(x - 0.1, x + 0.1)
    for kind in nn.FlattenLayer.TYPES:
        W, b = rng.standard_normal((5, 24)), rng.standard_normal(5)
        ref = O.reach([{"type": "flatten", "kind": kind}, {"type": "fc", "W": W, "b": b}], S)
        folded = nn.NN([nn.FlattenLayer(Type=kind), nn.FullyConnectedLayer(W, b)])._layer_dicts(shape)
        assert [d["type"] for d in folded] == ["fc"]
        got = O.reach(folded, S)
        assert np.abs(got.mat() - ref.mat()).max() < 1e-13
    # the evaluate semantics of the permuting types on a concrete image (MATLAB permute + reshape)
    img = np.arange(24.0).reshape(shape, order="F")
    keras = nn.FlattenLayer(Type="nnet.keras.layer.FlattenCStyleLayer").source_index(shape)
    assert np.array_equal(img.reshape(-1, order="F")[keras], np.transpose(img, (2, 1, 0)).reshape(-1, order="F"))
    assert np.array_equal(img.reshape(-1, order="F")[keras], img.reshape(-1, order="C"))      # C-style order
    with pytest.raises(NotImplementedError):
        nn.NN([nn.FlattenLayer(Type="nnet.keras.layer.FlattenCStyleLayer"), nn.ReluLayer()])._layer_dicts(shape)
    with pytest.raises(ValueError):
        nn.FlattenLayer(Type="something else")


def test_image_input_layer_normalisations_match_the_oracle():
    """ImageInputLayer.m:121-168 on a set given by bounds and on a set given by V."""
    rng = np.random.default_rng(1)
    shape = (3, 4, 2)
    x = rng.uniform(0, 255, shape)
    lb, ub = x - 2.0, x + 2.0
    S = O.star_from_bounds(lb, ub)
    mean = rng.uniform(100, 150, shape)
    cases = [("none", {}), ("zerocenter", {"Mean": mean}), ("zscore", {"Mean": mean, "StandardDeviation": [50.0, 60.0]}),
             ("rescale-zero-one", {}), ("rescale-zero-one", {"Min": 10.0, "Max": 240.0}),
             ("rescale-symmetric", {}), ("rescale-symmetric", {"Min": 10.0, "Max": 240.0})]
    for norm, kw in cases:
        L = nn.ImageInputLayer(shape, norm, **kw)
        ref = O.image_input_reach(S, {"normalization": norm, "mean": kw.get("Mean"), "std": kw.get("StandardDeviation"),
                                      "min": kw.get("Min"), "max": kw.get("Max")})
        by_bounds = L.apply(nn.ImageStar(lb, ub))
        got = O.star_from_bounds(by_bounds.im_lb, by_bounds.im_ub) if norm != "none" else S
        assert np.abs(got.V - ref.V).max() <= 1e-12 * np.abs(ref.V).max()
        by_V = L.apply(nn.ImageStar(S.V, S.C.toarray(), S.d, S.pl, S.pu))
        assert np.abs(by_V.V - ref.V).max() <= 1e-12 * np.abs(ref.V).max()
    with pytest.raises(ValueError):
        nn.ImageInputLayer(shape, "zerophase")


def test_relax_star_selection_matches_the_oracle():
    """The host hook and the oracle pick the same neurons for LP-optimised ranges (ties, rounding of halves)."""
    from oracle import nnv_oracle as O
    rng = np.random.default_rng(5)
    for k in (1, 2, 5, 8, 33):
        lb = -np.round(rng.uniform(0.1, 3.0, k), 1)         # rounded: ties occur
        ub = np.round(rng.uniform(0.1, 3.0, k), 1)
        for method in ("relax-star-area", "relax-star-range", "relax-star-static"):
            for rf in (0.0, 0.25, 0.5, 0.75, 1.0):
                sel = nn.relax_select(method, rf, lb, ub)
                p21, p22 = O.relax_selection(method, rf, lb, ub)
                assert list(sel) == list(p21), (k, method, rf)
                assert sorted(list(p21) + list(p22)) == list(range(k))
