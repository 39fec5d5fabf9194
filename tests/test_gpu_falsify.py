"""Concrete evaluation and falsification around the reach: NN.evaluate as one batched forward pass on the
device, NN.falsify / NN.verify_safety (verdict 0, "unsafe"), and the pre-check of the bound images that the
reference's example harness runs before verify_robustness.  Checked against the oracle's restatements on the
same sample points."""
import numpy as np
import pytest

from nnv_b200 import nn
from nnv_b200.configs import make_config
from oracle import nnv_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,small", [("cnn32", True), ("cnn28", False), ("fc5", False), ("vgg224", True)])
def test_evaluate_matches_oracle(ctx, name, small):
    cfg = make_config(name, n_queries=1, small=small)
    model = nn.NN(cfg["layers"], ctx=ctx)
    rng = np.random.default_rng(3)
    xs = [rng.uniform(0, 1, cfg["in_shape"]) for _ in range(5)]
    ys = model.evaluate(xs)
    for x, y in zip(xs, ys):
        ref = O.evaluate(cfg["layers"], x)
        assert np.abs(y - ref).max() <= 1e-12 * max(1.0, np.abs(ref).max())
    assert np.array_equal(model.evaluate(xs[0]), ys[0])
    model.close()


def test_sample_precheck_produces_every_verdict(ctx):
    """-1 (misclassified), 0 (a bound image changes class), 1 / 2 from the reach: same as the oracle's harness."""
    cfg = make_config("cnn28", n_queries=8, small=True, eps=0.1)
    model = nn.NN(cfg["layers"], ctx=ctx)
    sets = [nn.ImageStar(q["lb"], q["ub"]) for q in cfg["queries"]]
    images = [0.5 * (q["lb"] + q["ub"]) for q in cfg["queries"]]
    got = model.verify_sample_batch(sets, images, [q["target"] + 1 for q in cfg["queries"]], {"reachMethod": "approx-star"})
    ref = np.array([O.verify_sample(cfg["layers"], q, im) for q, im in zip(cfg["queries"], images)])
    assert np.array_equal(got, ref)
    assert -1 in got and 0 in got
    model.close()


def test_falsify_and_verify_safety(ctx):
    cfg = make_config("cnn28", n_queries=8, small=True, eps=0.2)
    model = nn.NN(cfg["layers"], ctx=ctx)
    found = 0
    for q in cfg["queries"][4:]:
        I = nn.ImageStar(q["lb"], q["ub"])
        U = model.robustness_set(q["target"] + 1, "max")
        pts = I.sample(40, np.random.default_rng(5))                      # the points both sides evaluate
        assert len(pts) == 40 and all(np.all(p >= q["lb"] - 1e-15) and np.all(p <= q["ub"] + 1e-15) for p in pts)
        G, g = O.robustness_set(10, q["target"], "max")
        ref = O.falsify(cfg["layers"], pts, G, g)
        got = model.falsify(I, U, 40, np.random.default_rng(5))
        assert len(got) == len(ref) and all(np.array_equal(a, b) for a, b in zip(got, ref))
        res, counter = model.verify_safety(I, U, {"reachMethod": "approx-star"}, 40, np.random.default_rng(5))
        assert res == (0 if ref else 2) and len(counter) == len(ref)
        found += bool(ref)
    assert found > 0, "no query of this seed has a counterexample among its samples"
    # a set that is provably safe needs no samples
    q = make_config("cnn28", n_queries=1, small=True, eps=1e-4)["queries"][0]
    res, counter = model.verify_safety(nn.ImageStar(q["lb"], q["ub"]), model.robustness_set(q["target"] + 1, "max"),
                                       {"reachMethod": "approx-star"}, 10)
    assert res == 1 and counter == []
    model.close()


def test_star_sample_and_contains(ctx):
    # a general star (its constraints cut the predicate box): samples lie in the set; points outside do not
    V = np.array([[0.0, 1.0, 0.5], [1.0, -0.5, 1.0]])
    S = nn.Star(V, np.array([[1.0, 1.0]]), np.array([0.5]), -np.ones(2), np.ones(2))
    X = S.sample(20, np.random.default_rng(1))
    assert X.shape[0] == 2 and 0 < X.shape[1] <= 20
    assert all(S.contains(X[:, i]) for i in range(X.shape[1]))
    assert not S.contains(np.array([10.0, 10.0]))
    H = nn.HalfSpace(np.array([[1.0, 0.0]]), np.array([0.0]))
    assert H.contains(np.array([-1.0, 5.0])) and not H.contains(np.array([1.0, 0.0]))


def test_imagestar_affine_map(ctx):
    """ImageStar.affineMap: per-channel scale of every slice, offset on the centre (ImageStar.m:431-460)."""
    rng = np.random.default_rng(8)
    V = rng.standard_normal((6, 5, 3, 9))
    I = nn.ImageStar(V, np.zeros((1, 8)), np.zeros(1), -np.ones(8), np.ones(8))
    scale = rng.uniform(0.5, 2.0, (1, 1, 3))
    offset = rng.standard_normal((1, 1, 3))
    R = I.affineMap(scale, offset, ctx)
    ref = scale[..., None] * V
    ref[..., 0] += offset
    assert np.allclose(R.V, ref, rtol=1e-15, atol=0) and R.numPred == 8
    R2 = I.affineMap(0.25, rng.standard_normal((6, 5, 3)), ctx)           # scalar scale, offset image
    assert np.array_equal(R2.V[..., 1:], 0.25 * V[..., 1:])
    R3 = I.affineMap(None, 1.5, ctx)
    assert np.array_equal(R3.V[..., 1:], V[..., 1:]) and np.allclose(R3.V[..., 0], V[..., 0] + 1.5, rtol=1e-15)
    with pytest.raises(ValueError):
        I.affineMap(np.ones((1, 1, 2)), None, ctx)
