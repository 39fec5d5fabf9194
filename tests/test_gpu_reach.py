"""End-to-end parity of the CUDA reach (through the C ABI and the reference-shaped
host API) against the CPU oracle and the committed fixtures: generator tensors,
predicate bounds, constraint systems and output ranges within 1e-9 relative;
crossing-neuron index lists, predicate counts and verdicts identical."""
import numpy as np
import pytest

from nnv_b200 import nn
from nnv_b200.configs import forward_concrete, make_config
from nnv_b200.engine import Batch, Network
from oracle import nnv_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-9
CASES = [("fc5", False, 6), ("cnn28", True, 3), ("cnn32", True, 3), ("bright28", True, 4), ("vgg224", True, 1)]


def _rel(a, b):
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-300)


@pytest.mark.parametrize("name,small,nq", CASES)
def test_reach_parity_vs_oracle(ctx, golden, name, small, nq):
    cfg = make_config(name, n_queries=nq, small=small)
    net = Network(ctx, cfg["layers"], cfg["in_shape"])
    b = Batch(net, cfg["queries"])
    b.upload()
    b.reach(keep_constraints=True, keep_layer_bounds=True)
    for q, qu in enumerate(cfg["queries"]):
        S = O.reach(cfg["layers"], O.star_from_query(qu))
        V = b.get_V(q)
        assert V.shape == S.V.shape
        assert _rel(V, S.V) < TOL
        lb, ub = b.get_ranges(q)
        rl, ru = O.output_ranges(S)
        scale = max(np.abs(rl).max(), np.abs(ru).max())
        assert np.abs(lb - rl).max() / scale < TOL and np.abs(ub - ru).max() / scale < TOL
        assert np.allclose(lb, golden["%s_q%d_lb" % (name, q)], rtol=0, atol=TOL * scale)
        assert np.allclose(ub, golden["%s_q%d_ub" % (name, q)], rtol=0, atol=TOL * scale)
        for li, t in enumerate(S.trace):
            idx, cl, cu = b.get_crossing(q, li)
            assert np.array_equal(idx, t["cross"])                       # bit-exact index work
            assert np.array_equal(idx, golden["%s_q%d_cross%d" % (name, q, li)])
            bscale = max(np.abs(t["lb"]).max(), np.abs(t["ub"]).max())
            assert np.abs(cl - t["lb"][t["cross"]]).max(initial=0) / bscale < TOL
            assert np.abs(cu - t["ub"][t["cross"]]).max(initial=0) / bscale < TOL
            ll, lu = b.get_layer_ranges(q, li, t["N"])
            assert np.abs(ll - t["lb"]).max() / bscale < TOL and np.abs(lu - t["ub"]).max() / bscale < TOL
            assert np.array_equal(np.nonzero(lu <= 0)[0], t["dead"])
        pl, pu = b.get_pred_bounds(q)
        assert np.array_equal(pl, S.pl) and _rel(pu, S.pu) < TOL
        Cm, d = b.get_constraints(q)
        Cd = S.C.toarray()
        assert Cm.shape == Cd.shape and _rel(Cm, Cd) < TOL and np.abs(d - S.d).max() <= TOL * max(np.abs(S.d).max(), 1)
        P, m = b.out_dims(q)
        assert P == S.P and m == S.C.shape[0]
    stats = b.relu_stats()
    assert len(stats) == sum(1 for l in cfg["layers"] if l["type"] == "relu")
    b.close()
    net.close()


@pytest.mark.parametrize("name,small,nq", CASES)
def test_default_path_parity_vs_oracle(ctx, name, small, nq):
    """The path a verification run takes (no constraint records): windowed layer kernels that write
    only the columns' windows, rows cleared by masks in the next layer, implicit unit-vector columns,
    the window-sorted bound reduction."""
    cfg = make_config(name, n_queries=nq, small=small)
    net = Network(ctx, cfg["layers"], cfg["in_shape"])
    b = Batch(net, cfg["queries"])
    b.upload()
    b.reach(keep_layer_bounds=True)
    for q, qu in enumerate(cfg["queries"]):
        S = O.reach(cfg["layers"], O.star_from_query(qu))
        V = b.get_V(q)
        assert V.shape == S.V.shape
        assert _rel(V, S.V) < TOL
        lb, ub = b.get_ranges(q)
        rl, ru = O.output_ranges(S)
        scale = max(np.abs(rl).max(), np.abs(ru).max())
        assert np.abs(lb - rl).max() / scale < TOL and np.abs(ub - ru).max() / scale < TOL
        for li, t in enumerate(S.trace):
            idx, cl, cu = b.get_crossing(q, li)
            assert np.array_equal(idx, t["cross"])
            bscale = max(np.abs(t["lb"]).max(), np.abs(t["ub"]).max())
            ll, lu = b.get_layer_ranges(q, li, t["N"])
            assert np.abs(ll - t["lb"]).max() / bscale < TOL and np.abs(lu - t["ub"]).max() / bscale < TOL
            assert np.array_equal(np.nonzero(lu <= 0)[0], t["dead"])
        pl, pu = b.get_pred_bounds(q)
        assert np.array_equal(pl, S.pl) and _rel(pu, S.pu) < TOL
    b.close()
    net.close()


def test_results_belong_to_the_last_reach_on_a_context(ctx):
    from nnv_b200._lib import NNVError
    cfg = make_config("fc5", n_queries=2)
    net = Network(ctx, cfg["layers"], cfg["in_shape"])
    b1 = Batch(net, cfg["queries"][:1])
    b2 = Batch(net, cfg["queries"][1:])
    for b in (b1, b2):
        b.upload()
    b1.reach()
    b2.reach()
    b2.get_V(0)
    with pytest.raises(NNVError):
        b1.get_V(0)                 # overwritten by the later reach: refused, not garbage
    b1.reach()
    b1.get_V(0)
    b1.close()
    b2.close()
    net.close()


def test_reach_is_deterministic_and_batch_invariant(ctx):
    cfg = make_config("cnn32", n_queries=3, small=True)
    net = Network(ctx, cfg["layers"], cfg["in_shape"])
    b = Batch(net, cfg["queries"])
    b.upload()
    b.reach()
    first = [b.get_V(q) for q in range(3)]
    b.reach()                                                # same uploaded inputs, second pass
    for q in range(3):
        assert np.array_equal(b.get_V(q), first[q])
    b.close()
    for q in range(3):                                       # one query at a time
        b1 = Batch(net, [cfg["queries"][q]])
        b1.upload()
        b1.reach()
        assert np.array_equal(b1.get_V(0), first[q])
        b1.close()
    net.close()


@pytest.mark.parametrize("name,small,nq", [("fc5", False, 6), ("cnn28", True, 3), ("cnn32", True, 3), ("bright28", True, 4)])
def test_verdicts_match_oracle(ctx, golden, name, small, nq):
    cfg = make_config(name, n_queries=nq, small=small)
    net = nn.NN(cfg["layers"], ctx=ctx)
    sets = []
    for qu in cfg["queries"]:
        if "lb" in qu:
            sets.append(nn.ImageStar(qu["lb"], qu["ub"]))
        else:
            sets.append(nn.ImageStar(qu["V"], qu["C"], qu["d"], qu["pl"], qu["pu"]))
    targets = [qu["target"] + 1 for qu in cfg["queries"]]
    kind = cfg["queries"][0]["spec"]
    stats = {}
    got = net.verify_robustness_batch(sets, {"reachMethod": "approx-star"}, targets, kind, stats)
    assert np.array_equal(got, golden[name + "_verdicts"])
    assert stats["n_prefilter"] + stats["n_witness"] + stats["n_lp_queries"] == nq


@pytest.mark.parametrize("name,small,nq", [("cnn28", True, 6), ("cnn28", False, 10), ("bright28", True, 4),
                                           ("cnn32", True, 3)])
def test_device_verdicts_per_halfspace_row_are_sound(ctx, name, small, nq):
    """Every row the device decides agrees with the emptiness LP of the oracle on that row: box minimum
    and back-substitution bound (EMPTY), witness point (NONEMPTY).  With the crossing rows recorded the
    back-substitution bound leaves no more rows open than the run without them."""
    from nnv_b200 import _lib as L
    cfg = make_config(name, n_queries=nq, small=small)
    net = Network(ctx, cfg["layers"], cfg["in_shape"])
    b = Batch(net, cfg["queries"])
    b.upload()
    tg = [qu["target"] for qu in cfg["queries"]]
    kind = cfg["queries"][0]["spec"]
    b.reach(keep_layer_bounds=True)
    _, s0, _ = b.verify_robust(tg, kind)
    s0 = np.array(s0).copy()
    b.reach(keep_constraints=True, keep_layer_bounds=True)
    _, s1, m1 = b.verify_robust(tg, kind)
    s1 = np.array(s1)
    assert (s1 == L.UNDECIDED).sum() <= (s0 == L.UNDECIDED).sum()
    for q, qu in enumerate(cfg["queries"]):
        S = O.reach(cfg["layers"], O.star_from_query(qu))
        G, g = O.robustness_set(S.mat().shape[0], qu["target"], kind)
        for i in range(G.shape[0]):
            if s0[q][i] == L.UNDECIDED and s1[q][i] == L.UNDECIDED:
                continue
            C, d = O.intersect_halfspace_system(S, G[i:i + 1], g[i:i + 1])
            empty = O.is_empty_set(C, d, S.pl, S.pu)
            for st in (s0[q][i], s1[q][i]):
                if st == L.VERDICT_EMPTY:
                    assert empty, (q, i)
                elif st == L.VERDICT_NONEMPTY:
                    assert not empty, (q, i)
    b.close()
    net.close()


def test_reference_shaped_api_single_set(ctx):
    cfg = make_config("cnn28", n_queries=1, small=True)
    qu = cfg["queries"][0]
    layers = []
    for L in cfg["layers"]:
        if L["type"] == "conv2d":
            layers.append(nn.Conv2DLayer(L["W"], L["b"], L["pad"], L["stride"], L["dilation"]))
        elif L["type"] == "fc":
            layers.append(nn.FullyConnectedLayer(L["W"], L["b"]))
        elif L["type"] == "relu":
            layers.append(nn.ReluLayer())
    net = nn.NN(layers, ctx=ctx)
    I = nn.ImageStar(qu["lb"], qu["ub"])
    R = net.reach(I, {"reachMethod": "relax-star-area", "relaxFactor": 1})
    S = O.reach(cfg["layers"], O.star_from_query(qu))
    assert isinstance(R, nn.ImageStar) and R.numPred == S.P
    assert _rel(R.V, S.V) < TOL and _rel(R.C, S.C.toarray()) < TOL
    assert net.verify_robustness(I, {"reachMethod": "approx-star"}, qu["target"] + 1) == O.verify_robustness(cfg["layers"], qu)
    # layer-level reach contract: L.reach(set, method)
    R1 = layers[0].reach(I, "approx-star")
    assert _rel(R1.V, O.conv2d_reach(O.star_from_query(qu), cfg["layers"][0]).V) < TOL


def test_relu_layer_reach_kat(ctx, kats):
    # code/nnv/tests/nn/layers/ReluLayer/test_layers_relu.m:36-55 through ReluLayer.reach
    IM, LB, UB = kats["relu_reach_IM"], kats["relu_reach_LB"], kats["relu_reach_UB"]
    R = nn.ReluLayer().reach(nn.ImageStar(IM + LB, IM + UB), "approx-star")
    S = O.relu_reach(O.star_from_bounds(IM + LB, IM + UB))
    assert R.numPred == 7 and np.array_equal(R.V, S.V)
    assert np.allclose(R.C, S.C.toarray(), rtol=1e-12, atol=1e-15) and np.allclose(R.d, S.d, rtol=1e-12, atol=1e-15)
    # all-positive and all-negative stars (code/nnv/tests/soundness/test_regression_reachability.m:47-79)
    for sign in (1, -1):
        c = sign * np.array([2., 3., 4.])
        St = nn.Star(np.hstack([c[:, None], 0.1 * np.eye(3)]), np.vstack([np.eye(3), -np.eye(3)]), 0.5 * np.ones(6),
                     -0.5 * np.ones(3), 0.5 * np.ones(3))
        Rs = nn.ReluLayer().reach(St, "approx-star")
        assert isinstance(Rs, nn.Star) and Rs.nVar == 3
        assert np.abs(Rs.V[:, 0] - np.maximum(c, 0)).max() < 1e-10


def test_soundness_by_sampling_on_gpu(ctx):
    cfg = make_config("cnn32", n_queries=2, small=True)
    net = Network(ctx, cfg["layers"], cfg["in_shape"])
    b = Batch(net, cfg["queries"])
    b.upload()
    b.reach()
    rng = np.random.default_rng(3)
    for q, qu in enumerate(cfg["queries"]):
        lb, ub = b.get_ranges(q)
        for _ in range(8):
            x = rng.uniform(qu["lb"], qu["ub"])
            y = forward_concrete(cfg["layers"], x)
            assert np.all(y >= lb - 1e-9) and np.all(y <= ub + 1e-9)
    b.close()
    net.close()


def test_edge_cases(ctx):
    from nnv_b200._lib import NNVError
    # a point set (no generators) through a whole network
    cfg = make_config("cnn28", n_queries=1, small=True)
    x = cfg["queries"][0]["lb"]
    net = Network(ctx, cfg["layers"], cfg["in_shape"])
    b = Batch(net, [{"lb": x, "ub": x}])
    b.upload()
    b.reach(keep_constraints=True)
    assert b.out_dims(0) == (0, 1)
    lb, ub = b.get_ranges(0)
    y = forward_concrete(cfg["layers"], x)
    assert np.abs(lb - y).max() < 1e-12 and np.array_equal(lb, ub)
    # results before reach, bad query index, unset query
    b2 = Batch(net, n_queries=2)
    b2.set_bounds(0, x, x)
    with pytest.raises(NNVError, match="never set"):
        b2.upload()
    with pytest.raises(NNVError):
        b2.get_ranges(0)
    with pytest.raises(NNVError, match="lb > ub"):
        b2.set_bounds(1, x + 1, x)
    b.close()
    b2.close()
    net.close()


@pytest.mark.parametrize("tail", ["conv", "relu", "pool", "bn"])
def test_networks_that_end_in_an_image_layer(ctx, tail):
    """The set handed out after a convolution / ReLU / pooling / BN layer (no FC behind it) is the dense
    tensor of the reference although the engine holds only the columns' windows at that point.  Also covers
    strides, dilation, uneven padding and a 5x3 filter, which take the patch-tiled convolution."""
    from nnv_b200.configs import _conv, _bn, _pool2, RELU
    rng = np.random.default_rng(11)
    shape = (24, 20, 3)
    layers = [_conv(rng, 3, 3, 3, 8, (1, 1, 1, 1)), RELU, _conv(rng, 5, 3, 8, 8, (2, 1, 0, 1), (2, 1)), RELU, _pool2()]
    layers[2]["dilation"] = (1, 2)
    if tail == "conv":
        layers.append(_conv(rng, 3, 3, 8, 4, (1, 1, 1, 1)))
    elif tail == "relu":
        layers += [_conv(rng, 3, 3, 8, 4, (1, 1, 1, 1)), RELU]
    elif tail == "bn":
        layers += [_conv(rng, 3, 3, 8, 4, (1, 1, 1, 1)), RELU, _bn(rng, 4)]
    queries = []
    for _ in range(3):
        x = rng.uniform(0, 1, shape)
        queries.append({"lb": np.maximum(x - 0.02, 0), "ub": np.minimum(x + 0.02, 1)})
    net = Network(ctx, layers, shape)
    b = Batch(net, queries)
    b.upload()
    b.reach()
    for q, qu in enumerate(queries):
        S = O.reach(layers, O.star_from_query(qu))
        V = b.get_V(q)
        assert V.shape == S.V.shape and _rel(V, S.V) < TOL
        lb, ub = b.get_ranges(q)
        rl, ru = O.output_ranges(S)
        scale = max(np.abs(rl).max(), np.abs(ru).max())
        assert np.abs(lb - rl).max() / scale < TOL and np.abs(ub - ru).max() / scale < TOL
    b.close()
    net.close()


def test_windowed_convolution_with_ragged_channel_counts(ctx):
    """Channel counts that fill neither the 8-channel input chunks nor the 32/64-channel output tiles of the
    windowed convolution kernel, a 3x5 filter, and image borders on every side of the windows."""
    from nnv_b200.configs import _conv, _bn, _pool2, _fc, RELU
    rng = np.random.default_rng(12)
    shape = (18, 14, 3)
    layers = [_conv(rng, 3, 3, 3, 20, (1, 1, 1, 1)), RELU,
              _conv(rng, 3, 5, 20, 40, (1, 1, 2, 2)), _bn(rng, 40), RELU,
              _conv(rng, 3, 3, 40, 24, (1, 1, 1, 1)), RELU, _pool2()]
    layers += [_fc(rng, 9 * 7 * 24, 30), RELU, _fc(rng, 30, 6)]
    queries = []
    for k in range(3):
        x = rng.uniform(0, 1, shape)
        e = np.zeros(shape)
        e[k::3, ::2, :] = 0.01                      # a third of the rows, every other pixel column
        e[0, 0, :] = e[-1, -1, :] = e[0, -1, :] = e[-1, 0, :] = 0.01
        queries.append({"lb": np.maximum(x - e, 0), "ub": np.minimum(x + e, 1)})
    net = Network(ctx, layers, shape)
    b = Batch(net, queries)
    b.upload()
    b.reach(keep_layer_bounds=True)
    for q, qu in enumerate(queries):
        S = O.reach(layers, O.star_from_query(qu))
        V = b.get_V(q)
        assert V.shape == S.V.shape and _rel(V, S.V) < TOL
        for li, t in enumerate(S.trace):
            idx, _, _ = b.get_crossing(q, li)
            assert np.array_equal(idx, t["cross"])
            ll, lu = b.get_layer_ranges(q, li, t["N"])
            bscale = max(np.abs(t["lb"]).max(), np.abs(t["ub"]).max())
            assert np.abs(ll - t["lb"]).max() / bscale < TOL and np.abs(lu - t["ub"]).max() / bscale < TOL
    b.close()
    net.close()


def _pool(ph, pw, sh, sw, pad=(0, 0, 0, 0)):
    return {"type": "avgpool", "pool": (ph, pw), "stride": (sh, sw), "pad": pad}


@pytest.mark.parametrize("case", ["tiling", "chain", "ragged", "overlap"])
def test_unit_vector_columns_through_pooling_layers(ctx, case):
    """The columns a ReLU layer appends reach the layer after a pooling layer as scaled unit vectors when the
    pooling windows tile the image (their memory is first written by that next layer); with a ragged image,
    overlapping windows or padding they are written by the pooling layer.  Same sets either way."""
    from nnv_b200.configs import _conv, _bn, _fc, RELU, out_shape
    rng = np.random.default_rng(31)
    if case == "tiling":          # ReLU -> 2x2/2 -> convolution, ReLU -> 3x2/3x2 -> FC
        shape = (12, 12, 2)
        layers = [_conv(rng, 3, 3, 2, 12, (1, 1, 1, 1)), RELU, _pool(2, 2, 2, 2),
                  _conv(rng, 3, 3, 12, 10, (1, 1, 1, 1)), _bn(rng, 10), RELU, _pool(3, 2, 3, 2)]
    elif case == "chain":         # two pooling layers in a row, the second one followed by a convolution
        shape = (16, 8, 2)
        layers = [_conv(rng, 3, 3, 2, 9, (1, 1, 1, 1)), RELU, _pool(2, 2, 2, 2), _pool(2, 1, 2, 1),
                  _conv(rng, 3, 3, 9, 8, (1, 1, 1, 1)), RELU, _pool(2, 2, 2, 2)]
    elif case == "ragged":        # 7 rows do not split into 2-row windows; the second pooling layer is padded
        shape = (7, 9, 2)
        layers = [_conv(rng, 3, 3, 2, 8, (1, 1, 1, 1)), RELU, _pool(2, 2, 2, 2),
                  _conv(rng, 3, 3, 8, 8, (1, 1, 1, 1)), RELU, _pool(2, 2, 2, 2, (1, 0, 0, 0))]
    else:                         # 3x3 windows with stride 2
        shape = (11, 11, 2)
        layers = [_conv(rng, 3, 3, 2, 8, (1, 1, 1, 1)), RELU, _pool(3, 3, 2, 2),
                  _conv(rng, 3, 3, 8, 8, (1, 1, 1, 1)), RELU, _pool(2, 2, 2, 2)]
    h, w, c = out_shape(layers, shape)
    layers += [_fc(rng, h * w * c, 20), RELU, _fc(rng, 20, 5)]
    queries = []
    for k in range(2):
        x = rng.uniform(0, 1, shape)
        e = np.zeros(shape)
        e[k::2, 1::3, :] = 0.05
        queries.append({"lb": np.maximum(x - e, 0), "ub": np.minimum(x + e, 1)})
    net = Network(ctx, layers, shape)
    b = Batch(net, queries)
    b.upload()
    b.reach(keep_layer_bounds=True)
    for q, qu in enumerate(queries):
        S = O.reach(layers, O.star_from_query(qu))
        V = b.get_V(q)
        assert V.shape == S.V.shape and _rel(V, S.V) < TOL
        assert any(len(t["cross"]) > 0 for t in S.trace[:2])
        for li, t in enumerate(S.trace):
            idx, _, _ = b.get_crossing(q, li)
            assert np.array_equal(idx, t["cross"])
            ll, lu = b.get_layer_ranges(q, li, t["N"])
            bscale = max(np.abs(t["lb"]).max(), np.abs(t["ub"]).max())
            assert np.abs(ll - t["lb"]).max() / bscale < TOL and np.abs(lu - t["ub"]).max() / bscale < TOL
    b.close()
    net.close()


def test_verification_of_a_list_that_exceeds_the_arena_is_split():
    """verify_robustness_batch halves the list when the generator tensors of all sets do not fit the arena."""
    from nnv_b200.engine import Context
    cfg = make_config("cnn28", n_queries=12)
    sets = [nn.ImageStar(qu["lb"], qu["ub"]) for qu in cfg["queries"]]
    targets = [qu["target"] + 1 for qu in cfg["queries"]]
    big = Context(0, 2 << 30)
    ref_stats = {}
    ref_model = nn.NN(cfg["layers"], ctx=big)
    ref = ref_model.verify_robustness_batch(sets, {"reachMethod": "approx-star"}, targets, "max", ref_stats)
    ref_model.close()
    big.close()
    small = Context(0, 160 << 20)                    # room for a few of the twelve sets at a time
    model = nn.NN(cfg["layers"], ctx=small)
    with pytest.raises(Exception):
        model.reach_batch(sets, {"reachMethod": "approx-star"})
    stats = {}
    got = model.verify_robustness_batch(sets, {"reachMethod": "approx-star"}, targets, "max", stats)
    assert np.array_equal(got, ref)
    assert stats["n_prefilter"] == ref_stats["n_prefilter"] and stats["n_witness"] == ref_stats["n_witness"]
    model.close()
    small.close()


def test_image_input_and_flatten_layers_around_the_path(ctx):
    """A network as an importer would hand it over: ImageInputLayer (zscore), convolution, ReLU, pooling, a
    Keras C-style FlattenLayer and two FC layers, against the oracle's own restatement of those layers."""
    from nnv_b200.configs import _conv, _fc, _pool2, RELU
    rng = np.random.default_rng(13)
    shape = (12, 10, 3)
    mean = rng.uniform(0.3, 0.6, shape)
    std = [0.2, 0.25, 0.3]
    conv = _conv(rng, 3, 3, 3, 8, (1, 1, 1, 1))
    fc1, fc2 = _fc(rng, 6 * 5 * 8, 20), _fc(rng, 20, 4)
    kind = "nnet.keras.layer.FlattenCStyleLayer"
    oracle_layers = [{"type": "imageinput", "normalization": "zscore", "mean": mean, "std": std}, conv, RELU, _pool2(),
                     {"type": "flatten", "kind": kind}, fc1, RELU, fc2]
    model = nn.NN([nn.ImageInputLayer(shape, "zscore", Mean=mean, StandardDeviation=std),
                   nn.Conv2DLayer(conv["W"], conv["b"], conv["pad"], conv["stride"], conv["dilation"]), nn.ReluLayer(),
                   nn.AveragePooling2DLayer((2, 2), (2, 2)), nn.FlattenLayer(Type=kind),
                   nn.FullyConnectedLayer(fc1["W"], fc1["b"]), nn.ReluLayer(), nn.FullyConnectedLayer(fc2["W"], fc2["b"])],
                  ctx=ctx)
    for _ in range(2):
        x = rng.uniform(0, 1, shape)
        lb, ub = np.maximum(x - 0.01, 0), np.minimum(x + 0.01, 1)
        S = O.reach(oracle_layers, O.star_from_bounds(lb, ub))
        R = model.reach(nn.ImageStar(lb, ub), {"reachMethod": "approx-star"})
        assert R.numPred == S.P
        assert _rel(R.V.reshape(S.V.shape, order="F"), S.V) < TOL
        assert _rel(R.C, S.C.toarray()) < TOL
    model.close()


def test_capacity_error_is_reported_not_fatal():
    from nnv_b200._lib import NNVError, NNVB_E_CAPACITY
    from nnv_b200.engine import Context
    small_ctx = Context(0, 1 << 20)                         # 1 MiB arena
    cfg = make_config("cnn28", n_queries=4)
    net = Network(small_ctx, cfg["layers"], cfg["in_shape"])
    b = Batch(net, cfg["queries"])
    b.upload()
    with pytest.raises(NNVError) as ei:
        b.reach()
    assert ei.value.status == NNVB_E_CAPACITY
    b.close()
    net.close()
    small_ctx.close()


@pytest.mark.parametrize("pool_pad", [False, True])
def test_compact_storage_chain(ctx, pool_pad):
    """Channel counts the tap-skipping convolution covers (more than 16 output channels), so that the windowed
    cohorts travel in compact form (window only, channel fastest) from the first convolution through ReLU
    layers, two pooling layers and into the gathered FC layer, with windows that hang over every image border.
    With a padded pooling layer the second half of the chain falls back to full-length columns."""
    from nnv_b200.configs import _conv, _bn, _fc, RELU, out_shape
    rng = np.random.default_rng(41)
    shape = (16, 12, 3)
    layers = [_conv(rng, 3, 3, 3, 32, (1, 1, 1, 1)), _bn(rng, 32), RELU,
              _conv(rng, 3, 3, 32, 36, (1, 1, 1, 1)), RELU, _pool(2, 2, 2, 2),
              _conv(rng, 3, 5, 36, 66, (1, 1, 2, 2)), _bn(rng, 66), RELU,
              _pool(2, 2, 2, 2, (1, 1, 0, 0) if pool_pad else (0, 0, 0, 0))]
    h, w, c = out_shape(layers, shape)
    layers += [_fc(rng, h * w * c, 24), RELU, _fc(rng, 24, 5)]
    queries = []
    for k in range(3):
        x = rng.uniform(0, 1, shape)
        e = np.zeros(shape)
        e[k::4, 1::3, :] = 0.02
        e[0, 0, :] = e[-1, -1, :] = e[0, -1, :] = e[-1, 0, :] = 0.02
        queries.append({"lb": np.maximum(x - e, 0), "ub": np.minimum(x + e, 1)})
    net = Network(ctx, layers, shape)
    b = Batch(net, queries)
    b.upload()
    b.reach(keep_layer_bounds=True)
    for q, qu in enumerate(queries):
        S = O.reach(layers, O.star_from_query(qu))
        V = b.get_V(q)
        assert V.shape == S.V.shape and _rel(V, S.V) < TOL
        assert sum(len(t["cross"]) for t in S.trace) > 20
        for li, t in enumerate(S.trace):
            idx, _, _ = b.get_crossing(q, li)
            assert np.array_equal(idx, t["cross"]), li
            ll, lu = b.get_layer_ranges(q, li, t["N"])
            bscale = max(np.abs(t["lb"]).max(), np.abs(t["ub"]).max())
            assert np.abs(ll - t["lb"]).max() / bscale < TOL and np.abs(lu - t["ub"]).max() / bscale < TOL
    b.close()
    net.close()
    # a network that ends while its cohorts are in compact form: the set handed out is the dense tensor
    net = Network(ctx, layers[:6], shape)
    b = Batch(net, queries[:1])
    b.upload()
    b.reach()
    S = O.reach(layers[:6], O.star_from_query(queries[0]))
    assert _rel(b.get_V(0), S.V) < TOL
    b.close()
    net.close()


def test_halfspace_row_with_zero_margin_is_left_to_the_lp(ctx):
    """A row whose minimum over the set is exactly zero touches the halfspace: the intersection is not empty
    (Star.isEmptySet finds the point), so the device must not call it empty because of a rounding error of either
    sign — it leaves the row undecided; rows that are clearly apart are decided."""
    from nnv_b200 import _lib as L
    W = np.array([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]])
    layers = [{"type": "fc", "W": W, "b": np.zeros(3)}]
    net = Network(ctx, layers, (2, 1, 1))
    b = Batch(net, [{"lb": np.array([-1.0, -1.0]).reshape(2, 1, 1), "ub": np.array([1.0, 1.0]).reshape(2, 1, 1)}])
    b.upload()
    b.reach(keep_constraints=True, keep_layer_bounds=True)
    G = np.array([[-1.0, 0.0, 0.0],        # -x1 <= -1: touches the set at x1 = 1, minimum of G x - g is exactly 0
                  [-1.0, 0.0, 0.0],        # -x1 <= -1.5: empty, minimum 0.5
                  [0.0, 0.0, 1.0]])        # x1 + x2 <= 0: half of the set
    g = np.array([-1.0, -1.5, 0.0])
    margin, status = b.halfspace_margins(0, G, g)
    assert margin[0] == 0.0 and status[0] == L.UNDECIDED
    assert margin[1] == 0.5 and status[1] == L.VERDICT_EMPTY
    assert status[2] == L.VERDICT_NONEMPTY
    S = O.reach(layers, O.star_from_bounds(np.array([-1.0, -1.0]), np.array([1.0, 1.0])))
    for i, want in enumerate([False, True, False]):
        C, d = O.intersect_halfspace_system(S, G[i:i + 1], g[i:i + 1])
        assert O.is_empty_set(C, d, S.pl, S.pu) == want
    b.close()
    net.close()


@pytest.mark.parametrize("name", ["cnn28", "bright28"])
def test_bulk_set_entry_points_equal_the_per_set_ones(ctx, name):
    """A uniform list of eight or more sets crosses the ABI in one call (nnvb_batch_set_bounds_many for
    ImageStar(lb, ub) lists, nnvb_batch_set_stars for stars that share their predicate and constraint counts);
    the batch must be the one the per-set calls build."""
    cfg = make_config(name, n_queries=9, small=True)
    net = Network(ctx, cfg["layers"], cfg["in_shape"])
    bulk = Batch(net, cfg["queries"])                  # nine sets: the bulk path
    one = Batch(net, n_queries=9)
    for q, qu in enumerate(cfg["queries"]):
        one.set_query(q, qu)
    for b in (bulk, one):
        b.upload()
        b.reach()
    res = {}
    for key, b in (("bulk", bulk), ("one", one)):
        b.reach()                                       # results belong to the batch reached last
        res[key] = [(b.get_V(q), b.get_pred_bounds(q), b.get_ranges(q)) for q in range(9)]
    for (V, (pl, pu), (lb, ub)), (V1, (pl1, pu1), (lb1, ub1)) in zip(res["bulk"], res["one"]):
        assert np.array_equal(V, V1) and np.array_equal(pl, pl1) and np.array_equal(pu, pu1)
        assert np.array_equal(lb, lb1) and np.array_equal(ub, ub1)
    bulk.close()
    one.close()
    net.close()
