"""LP-tightened bounds: the reference's default 'approx-star' (PosLin.reach_star_approx2, PosLin.m:747-857).
The engine pre-selects by estimated ranges on the device, the host solves the LPs of the pre-selected neurons
(Star.getMaxs / getMins) inside the reach, and the relaxation is built from the LP bounds.  Against the
oracle's restatement of the same function: crossing sets identical, sets and constraint systems to 1e-9,
verdicts identical."""
import numpy as np
import pytest

from nnv_b200 import nn
from nnv_b200.configs import make_config
from oracle import nnv_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-9
LP = {"reachMethod": "approx-star", "bounds": "lp"}


def _rel(a, b):
    return np.abs(a - b).max(initial=0) / max(np.abs(b).max(initial=0), 1e-300)


def _sets(cfg):
    return [nn.ImageStar(q["lb"], q["ub"]) if "lb" in q else nn.ImageStar(q["V"], q["C"], q["d"], q["pl"], q["pu"])
            for q in cfg["queries"]]


@pytest.mark.parametrize("name,small,nq", [("fc5", False, 6), ("cnn28", True, 3), ("cnn32", True, 2), ("bright28", True, 3)])
def test_lp_bounds_reach_matches_oracle(ctx, name, small, nq):
    cfg = make_config(name, n_queries=nq, small=small)
    model = nn.NN(cfg["layers"], ctx=ctx)
    b = model.reach_batch(_sets(cfg), LP, keep_layer_bounds=True)
    tightened = 0
    for q, qu in enumerate(cfg["queries"]):
        S = O.reach(cfg["layers"], O.star_from_query(qu), lp_bounds=True)
        for li, t in enumerate(S.trace):
            idx, cl, cu = b.get_crossing(q, li)
            assert np.array_equal(idx, t["cross"]), (q, li)
            sc = max(np.abs(t["lb"]).max(), np.abs(t["ub"]).max())
            assert np.abs(cl - t["lb_lp"]).max(initial=0) <= 1e-7 * sc      # LP optima: solver tolerance
            assert np.abs(cu - t["ub_lp"]).max(initial=0) <= 1e-7 * sc
            tightened += len(t["cross_est"]) - len(t["cross"])
        P, m = b.out_dims(q)
        assert P == S.P and m == S.C.shape[0]
        V = b.get_V(q)
        assert V.shape == S.V.shape and _rel(V, S.V) < TOL
        pl, pu = b.get_pred_bounds(q)
        assert np.array_equal(pl, S.pl) and np.abs(pu - S.pu).max(initial=0) <= 1e-7 * max(1.0, np.abs(S.pu).max())
        Cm, d = b.get_constraints(q)
        Cd = S.C.toarray()
        assert Cm.shape == Cd.shape and _rel(Cm, Cd) < 1e-6 and np.abs(d - S.d).max() <= 1e-6 * max(np.abs(S.d).max(), 1)
    b.close()
    if name in ("fc5", "cnn28"):
        assert tightened > 0, "no neuron of these queries is decided by its LP bounds: the case is not exercised"
    model.close()


@pytest.mark.parametrize("name,small,nq", [("fc5", False, 12), ("cnn28", True, 4)])
def test_lp_bounds_verdicts_match_oracle(ctx, name, small, nq):
    cfg = make_config(name, n_queries=nq, small=small)
    model = nn.NN(cfg["layers"], ctx=ctx)
    kind = cfg["queries"][0]["spec"]
    got = model.verify_robustness_batch(_sets(cfg), LP, [q["target"] + 1 for q in cfg["queries"]], kind)
    ref = []
    for qu in cfg["queries"]:
        S = O.reach(cfg["layers"], O.star_from_query(qu), lp_bounds=True)
        G, g = O.robustness_set(S.mat().shape[0], qu["target"], kind)
        ref.append(O.verify_specification(S, G, g))
    assert np.array_equal(got, np.array(ref))
    model.close()


def test_hook_errors_surface_as_status(ctx):
    from nnv_b200._lib import NNVError
    from nnv_b200.engine import Batch
    cfg = make_config("fc5", n_queries=2)
    model = nn.NN(cfg["layers"], ctx=ctx)
    net = model._network(cfg["in_shape"])
    b = Batch(net, cfg["queries"])
    b.upload()

    def bad(batch, layer):
        raise RuntimeError("solver unavailable")
    b.set_bounds_hook(bad)
    with pytest.raises(NNVError, match="bounds hook failed"):
        b.reach(keep_constraints=True)
    b.set_bounds_hook(None)
    b.reach(keep_constraints=True)                     # the context and the batch stay usable
    b.close()
    model.close()


def _oracle_in_engine_order(S):
    """The oracle appends a layer's new predicates in the reference's order (neurons without optimised ranges
    first), the engine in ascending neuron order: the column permutation that turns the first into the second,
    layer by layer, and the per-layer crossing lists in ascending order."""
    perm = list(range(1 + S.trace[0]["P_in"]))
    crossings = []
    for t in S.trace:
        order = np.argsort(t["cross"], kind="stable")
        base = 1 + t["P_in"]
        perm.extend(int(base + o) for o in order)
        crossings.append((t["cross"][order], t["lb_lp"][order], t["ub_lp"][order]))
    return np.array(perm, dtype=np.int64), crossings


@pytest.mark.parametrize("method,rf", [("relax-star-area", 0.5), ("relax-star-range", 0.25), ("relax-star-static", 0.5),
                                       ("relax-star-area", 0.0)])
@pytest.mark.parametrize("name,small,nq", [("fc5", False, 5), ("cnn28", True, 2)])
def test_relax_star_with_lp_share_matches_oracle(ctx, name, small, nq, method, rf):
    """'relax-star-*' with relaxFactor < 1 (PosLin.m:863-1105, 1541-1646): a share of the crossing neurons,
    chosen by the method's heuristic on the estimated ranges, gets LP bounds.  Same neurons optimised, same
    crossing sets, same set up to the order of the new predicate variables."""
    cfg = make_config(name, n_queries=nq, small=small)
    model = nn.NN(cfg["layers"], ctx=ctx)
    opts = {"reachMethod": method, "relaxFactor": rf}
    b = model.reach_batch(_sets(cfg), opts, keep_layer_bounds=True)
    n_opt = n_est = 0
    for q, qu in enumerate(cfg["queries"]):
        S = O.reach(cfg["layers"], O.star_from_query(qu), relax=(method, rf))
        perm, crossings = _oracle_in_engine_order(S)
        for li, (t, (cr, cl_o, cu_o)) in enumerate(zip(S.trace, crossings)):
            idx, cl, cu = b.get_crossing(q, li)
            assert np.array_equal(idx, cr), (q, li)
            sc = max(np.abs(t["lb"]).max(), np.abs(t["ub"]).max())
            assert np.abs(cl - cl_o).max(initial=0) <= 1e-7 * sc and np.abs(cu - cu_o).max(initial=0) <= 1e-7 * sc
            n_opt += len(t["optimised"])
            n_est += len(t["cross_est"])
        V = b.get_V(q)
        Vo = S.V[..., perm]
        assert V.shape == Vo.shape and _rel(V, Vo) < TOL
        pl, pu = b.get_pred_bounds(q)
        assert np.array_equal(pl, S.pl[perm[1:] - 1])
        assert np.abs(pu - S.pu[perm[1:] - 1]).max(initial=0) <= 1e-7 * max(1.0, np.abs(S.pu).max())
    b.close()
    model.close()
    assert n_opt > 0
    if rf >= 0.5:       # (layers with one or two crossing neurons round a share of 0.75 up to all of them)
        assert n_opt < n_est, "the share must be a proper part of the crossing neurons for the case to count"


def test_relax_star_verdicts_match_oracle(ctx):
    cfg = make_config("fc5", n_queries=10)
    model = nn.NN(cfg["layers"], ctx=ctx)
    opts = {"reachMethod": "relax-star-area", "relaxFactor": 0.5}
    kind = cfg["queries"][0]["spec"]
    got = model.verify_robustness_batch(_sets(cfg), opts, [q["target"] + 1 for q in cfg["queries"]], kind)
    ref = []
    for qu in cfg["queries"]:
        S = O.reach(cfg["layers"], O.star_from_query(qu), relax=("relax-star-area", 0.5))
        G, g = O.robustness_set(S.mat().shape[0], qu["target"], kind)
        ref.append(O.verify_specification(S, G, g))
    assert np.array_equal(got, np.array(ref))
    model.close()
