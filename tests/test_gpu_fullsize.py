"""Parity of the CUDA verification path with the CPU oracle at the sizes the benchmark runs:
the 32x32x3 CNN (image 0 of the workload; 3072 input predicates growing to ~20 000), the 28x28 CNN on 8
images, the brightening sets on 64, and all 100 queries of the 5-50x6-5 FC network.

The engine is driven the way a verification run drives it (reach with layer bounds kept, no constraint
records: windowed layer kernels, rows cleared by masks, implicit unit-vector columns, window-only copies,
the window-sorted bound reduction) and compared with a live oracle run: per ReLU layer the crossing index
list (bit-exact), the predicate count, the bounds of every neuron (1e-9 relative); the output set's
generator matrix, predicate bounds and ranges (1e-9 relative); the verdict.  Where the device proves a
halfspace intersection non-empty, the witness point behind that answer is checked against the ORACLE's
constraint system: C alpha <= d, pred_lb <= alpha <= pred_ub and G (c + V alpha) <= g, a sparse
matrix-vector product instead of an LP with 20 000 variables.
"""
import numpy as np
import pytest

from nnv_b200 import _lib as L
from nnv_b200.configs import make_config
from nnv_b200.engine import Batch, Context, Network
from oracle import nnv_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-9


@pytest.fixture(scope="module")
def big_ctx():
    c = Context(0, 16 << 30)
    yield c
    c.close()


def _rel(a, b):
    return np.abs(a - b).max(initial=0) / max(np.abs(b).max(initial=0), 1e-300)


def _compare_reach(b, q, S):
    """Engine results of query q against the oracle's output set S (with its per-layer trace)."""
    for li, t in enumerate(S.trace):
        idx, cl, cu = b.get_crossing(q, li)
        assert np.array_equal(idx, t["cross"]), "crossing set of ReLU layer %d differs" % li
        bscale = max(np.abs(t["lb"]).max(), np.abs(t["ub"]).max())
        ll, lu = b.get_layer_ranges(q, li, t["N"])
        assert np.abs(ll - t["lb"]).max() / bscale < TOL and np.abs(lu - t["ub"]).max() / bscale < TOL
        assert np.array_equal(np.nonzero(lu <= 0)[0], t["dead"])
        assert np.abs(cl - t["lb"][t["cross"]]).max(initial=0) / bscale < TOL
        assert np.abs(cu - t["ub"][t["cross"]]).max(initial=0) / bscale < TOL
    P, _ = b.out_dims(q)
    assert P == S.P
    V = b.get_V(q)
    assert V.shape == S.V.shape and _rel(V, S.V) < TOL
    pl, pu = b.get_pred_bounds(q)
    assert np.array_equal(pl, S.pl) and _rel(pu, S.pu) < TOL
    lb, ub = b.get_ranges(q)
    rl, ru = O.output_ranges(S)
    scale = max(np.abs(rl).max(), np.abs(ru).max())
    assert np.abs(lb - rl).max() / scale < TOL and np.abs(ub - ru).max() / scale < TOL


def _check_witness(b, q, S, Grow, g):
    """The device's witness point for the row lies in the oracle's star set and inside the halfspace."""
    alpha, x, val = b.halfspace_witness(q, Grow, g)
    M = S.mat()
    assert np.all(alpha >= S.pl - 1e-12) and np.all(alpha <= S.pu + 1e-9 * np.maximum(1.0, np.abs(S.pu)))
    # the constraint rows scale with the generator rows they were built from
    resid = S.C @ alpha - S.d
    row_scale = abs(S.C) @ np.abs(alpha) + np.abs(S.d) + 1.0
    assert np.all(resid <= 1e-9 * row_scale), "witness violates C alpha <= d by %g" % (resid / row_scale).max()
    y = M[:, 0] + M[:, 1:] @ alpha                       # the point of the oracle's set
    yscale = np.abs(M[:, 0]).max() + (np.abs(M[:, 1:]) @ np.abs(alpha)).max()
    assert np.abs(y - x).max() <= 1e-9 * yscale, "forward pass and affine form disagree"
    assert Grow @ y - g < 0 and val < 0


def test_cnn32_image0_full_size(big_ctx):
    O.set_conv_backend("torch")
    try:
        cfg = make_config("cnn32", n_queries=1)
        qu = cfg["queries"][0]
        S = O.reach(cfg["layers"], O.star_from_query(qu), keep_constraints=True)
    finally:
        O.set_conv_backend("numpy")
    # predicate columns (centre included) after every ReLU layer of seeded image 0
    assert [t["P_out"] + 1 for t in S.trace] == [4623, 7812, 10834, 20394, 20650]
    net = Network(big_ctx, cfg["layers"], cfg["in_shape"])
    b = Batch(net, cfg["queries"])
    b.upload()
    b.reach(keep_layer_bounds=True)
    _compare_reach(b, 0, S)
    verdict, status, margin = b.verify_robust([qu["target"]], "max")
    G, g = O.robustness_set(10, qu["target"], "max")
    M = S.mat()
    r = G @ M
    box_min = r[:, 0] + np.minimum(r[:, 1:] * S.pl, r[:, 1:] * S.pu).sum(axis=1) - g
    n_witness = 0
    for i in range(G.shape[0]):
        if status[0][i] == L.VERDICT_EMPTY:
            assert box_min[i] > 0
        elif status[0][i] == L.VERDICT_NONEMPTY:
            _check_witness(b, 0, S, G[i], g[i])
            n_witness += 1
    # one non-empty intersection makes the verdict "unknown" (verify_specification.m:56-79)
    assert (verdict[0] == L.VERDICT_NONEMPTY) == (n_witness > 0)
    assert n_witness > 0, "bounds this loose (output widths ~100) leave no row provably empty"
    b.close()
    net.close()


@pytest.mark.parametrize("name,nq", [("cnn28", 8), ("bright28", 64), ("fc5", 100)])
def test_full_size_workloads(big_ctx, name, nq):
    cfg = make_config(name, n_queries=nq)
    net = Network(big_ctx, cfg["layers"], cfg["in_shape"])
    b = Batch(net, cfg["queries"])
    b.upload()
    b.reach(keep_layer_bounds=True)
    kind = cfg["queries"][0]["spec"]
    tg = [qu["target"] for qu in cfg["queries"]]
    verdict, status, _ = b.verify_robust(tg, kind)
    status = np.array(status)
    n_out = int(np.prod(net.out_shape))
    decided = 0
    for q, qu in enumerate(cfg["queries"]):
        S = O.reach(cfg["layers"], O.star_from_query(qu), keep_constraints=True)
        _compare_reach(b, q, S)
        G, g = O.robustness_set(n_out, qu["target"], kind)
        ref = O.verify_specification(S, G, g)                      # the reference's LP verdict
        if verdict[q] != L.UNDECIDED:
            assert verdict[q] == ref, (q, verdict[q], ref)
            decided += 1
        for i in np.nonzero(status[q] == L.VERDICT_NONEMPTY)[0][:2]:
            _check_witness(b, q, S, G[i], g[i])
    assert decided > 0
    b.close()
    net.close()


def test_full_size_verdicts_through_the_host_api(big_ctx):
    """verify_robustness_batch (device tests, back-substitution pass, host LP for what is left) gives the
    oracle's verdict on every query."""
    from nnv_b200 import nn
    for name, nq in (("fc5", 100), ("cnn28", 16), ("bright28", 64)):
        cfg = make_config(name, n_queries=nq)
        model = nn.NN(cfg["layers"], ctx=big_ctx)
        sets = [nn.ImageStar(qu["lb"], qu["ub"]) if "lb" in qu else
                nn.ImageStar(qu["V"], qu["C"], qu["d"], qu["pl"], qu["pu"]) for qu in cfg["queries"]]
        kind = cfg["queries"][0]["spec"]
        got = model.verify_robustness_batch(sets, {"reachMethod": "approx-star"},
                                            [qu["target"] + 1 for qu in cfg["queries"]], kind)
        ref = np.array([O.verify_robustness(cfg["layers"], qu) for qu in cfg["queries"]])
        assert np.array_equal(got, ref), name
        model.close()
