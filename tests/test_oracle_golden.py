"""The oracle reproduces its committed outputs, and its reach sets are sound
(sampled concrete executions stay inside the estimated output ranges) — the
reference's own correctness notion (code/nnv/tests/soundness/soundness_test_utils.m)."""
import numpy as np
import pytest

from nnv_b200.configs import forward_concrete, make_config
from oracle import nnv_oracle as O

CASES = [("fc5", False, 6), ("cnn28", True, 3), ("cnn32", True, 3), ("bright28", True, 4), ("vgg224", True, 1)]


@pytest.mark.parametrize("name,small,nq", CASES)
def test_oracle_matches_committed_outputs(golden, name, small, nq):
    cfg = make_config(name, n_queries=nq, small=small)
    for q, qu in enumerate(cfg["queries"]):
        S = O.reach(cfg["layers"], O.star_from_query(qu))
        lb, ub = O.output_ranges(S)
        assert np.allclose(lb, golden["%s_q%d_lb" % (name, q)], rtol=1e-12, atol=1e-13)
        assert np.allclose(ub, golden["%s_q%d_ub" % (name, q)], rtol=1e-12, atol=1e-13)
        assert np.array_equal([t["P_out"] for t in S.trace], golden["%s_q%d_P" % (name, q)])
        for li, t in enumerate(S.trace):
            assert np.array_equal(t["cross"], golden["%s_q%d_cross%d" % (name, q, li)])


@pytest.mark.parametrize("name,small", [("fc5", False), ("cnn28", True), ("cnn32", True), ("bright28", True)])
def test_oracle_soundness_by_sampling(name, small):
    cfg = make_config(name, n_queries=2, small=small)
    rng = np.random.default_rng(7)
    for qu in cfg["queries"]:
        S0 = O.star_from_query(qu)
        S = O.reach(cfg["layers"], S0)
        lb, ub = O.output_ranges(S)
        M0 = S0.mat()
        for trial in range(12):
            if trial < 4:
                a = np.where(rng.uniform(size=S0.P) < 0.5, S0.pl, S0.pu)       # corners
            else:
                a = rng.uniform(S0.pl, S0.pu)
            x = (M0[:, 0] + M0[:, 1:] @ a).reshape(S0.shape, order="F")
            y = forward_concrete(cfg["layers"], x)
            assert np.all(y >= lb - 1e-9) and np.all(y <= ub + 1e-9)


def test_verdict_golden(golden):
    cfg = make_config("cnn28", n_queries=3, small=True)
    got = [O.verify_robustness(cfg["layers"], q) for q in cfg["queries"]]
    assert np.array_equal(got, golden["cnn28_verdicts"])
