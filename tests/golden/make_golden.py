"""Generate the committed fixtures under tests/golden/.

Two files are written:

reference_kats.npz
    Known-answer items of the reference's own test-suite for the operations on
    the approx-star path: literal inputs/expected values transcribed from its
    test files, and arrays read from its stored ``.mat`` baselines (needs the
    reference checkout: pass its root as argv[1] or in NNV_REFERENCE_ROOT).
    Each key is documented with the file:line it comes from.

oracle_small.npz
    Outputs of the CPU oracle (oracle/nnv_oracle.py) on the small seeded
    workloads: output ranges, predicate counts and crossing index lists per
    ReLU layer, verdicts.  The GPU tests compare against these as well as
    against a live oracle run.

Run from the repository root:  python tests/golden/make_golden.py <reference root>
"""
import os
import sys

import numpy as np
import scipy.io as sio

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from nnv_b200.configs import make_config  # noqa: E402
from oracle import nnv_oracle as O  # noqa: E402

SMALL_CASES = [("fc5", False, 6), ("cnn28", True, 3), ("cnn32", True, 3), ("bright28", True, 4),
               ("vgg224", True, 1)]


def reference_kats(ref_root):
    k = {}
    # code/nnv/tests/nn/layers/Conv2DLayer/test_layers_Conv2D.m:14-27 (compute_featureMap KAT)
    I = np.array([[1, 1, 1, 0, 0], [0, 1, 1, 1, 0], [0, 0, 1, 1, 1], [0, 0, 1, 1, 0], [0, 1, 1, 0, 0]], float)
    W = np.array([[1, 0, 1], [0, 1, 0], [1, 0, 1]], float)
    chk = np.zeros((3, 3))
    for i in range(3):
        for j in range(3):
            chk[i, j] = I[i, j] + I[i, j + 2] + I[i + 1, j + 1] + I[i + 2, j] + I[i + 2, j + 2]
    k["conv_I"], k["conv_W"], k["conv_expected"] = I, W, chk
    # test_layers_Conv2D.m:55-74 (zero padding of a 5x5x3 volume with [1 1 1 1])
    vol = np.zeros((5, 5, 3))
    vol[:, :, 0] = [[2, 0, 1, 2, 1], [1, 0, 2, 2, 2], [1, 2, 2, 0, 2], [1, 2, 0, 0, 1], [1, 0, 1, 1, 2]]
    vol[:, :, 1] = [[0, 0, 1, 0, 1], [0, 0, 2, 1, 1], [1, 1, 0, 1, 1], [1, 1, 0, 2, 2], [2, 1, 2, 0, 0]]
    vol[:, :, 2] = [[1, 2, 2, 1, 0], [2, 0, 0, 2, 0], [0, 0, 1, 0, 1], [1, 2, 0, 2, 0], [1, 0, 2, 1, 0]]
    k["pad_vol"] = vol
    # code/nnv/tests/nn/layers/AveragePooling2DLayer/test_layers_averagePooling.m:13-22 and the stored
    # baseline results/tests/baselines/nn/test_layers_averagePooling_results.mat (averageMap)
    k["avg_I"] = np.array([[1, 0, 2, 3], [4, 6, 6, 8], [3, 1, 1, 0], [1, 2, 2, 4]], float)
    m = sio.loadmat(os.path.join(ref_root, "results/tests/baselines/nn/test_layers_averagePooling_results.mat"))
    k["avg_expected_mat"] = m["averageMap"].astype(float)
    # test_layers_averagePooling.m:34-54 (evaluate: 3x3 pool, stride 2, on a 5x5x3 volume vs block means)
    v2 = np.zeros((5, 5, 3))
    v2[:, :, 0] = [[0, 0, 2, 0, 0], [1, 2, 0, 2, 0], [0, 0, 2, 2, 0], [0, 2, 2, 2, 2], [2, 2, 2, 1, 1]]
    v2[:, :, 1] = [[1, 2, 2, 1, 2], [2, 1, 2, 0, 2], [2, 2, 2, 0, 1], [1, 1, 1, 0, 0], [1, 0, 2, 2, 1]]
    v2[:, :, 2] = [[0, 0, 2, 2, 1], [0, 2, 1, 1, 2], [0, 2, 0, 0, 1], [0, 2, 1, 0, 1], [1, 2, 1, 0, 0]]
    k["avg_vol"] = v2
    # code/nnv/tests/soundness/test_regression_layers.m:52-65 (FC), :103-115 (avg-pool)
    k["fc_W"], k["fc_b"], k["fc_x"], k["fc_expected"] = (np.array([[1., 2.], [3., 4.]]), np.array([0.5, 1.0]),
                                                          np.array([1., 1.]), np.array([3.5, 8.0]))
    k["avg2_I"] = np.tile(np.array([2., 4., 6., 8.]), (4, 1))
    k["avg2_expected"] = np.array([[3., 7.], [3., 7.]])
    # code/nnv/tests/soundness/test_soundness_BatchNormalizationLayer.m:6-23 (closed form, tol 1e-10)
    k["bn_params"] = np.array([0.5, 0.1, 1e-5, 1.2, 0.1])      # mean, var, eps, scale, offset
    # code/nnv/tests/nn/layers/ReluLayer/test_layers_relu.m:19-33 and baseline test_layers_relu_results.mat
    # (the stored IM is a later variable of that script; the evaluate input is transcribed, the expected
    # output IM_out is read from the baseline)
    IMe = np.zeros((4, 4, 3))
    IMe[:, :, 0] = [[-1, 1, 0, -1], [0, 0, 1, -1], [1, 0, -1, 0], [1, -1, -1, 1]]
    IMe[:, :, 1] = [[0, 1, 0, 0], [1, 0, 0, -1], [0, 1, -1, 0], [0, 1, 0, -1]]
    IMe[:, :, 2] = [[1, -1, 1, 1], [1, -1, 0, 1], [0, 1, -1, 0], [1, 0, -1, 0]]
    m = sio.loadmat(os.path.join(ref_root, "results/tests/baselines/nn/test_layers_relu_results.mat"))
    k["relu_IM"], k["relu_IM_out"] = IMe, m["IM_out"].astype(float)
    m = sio.loadmat(os.path.join(ref_root, "results/tests/baselines/nn/test_funcs_poslin_results.mat"))
    k["poslin_x"], k["poslin_y"] = m["x_input"].astype(float).ravel(), m["y_output"].astype(float).ravel()
    # test_layers_relu.m:36-46: ImageStar(IM, LB, UB) attack set for the approx-star reach smoke test
    IM = np.zeros((4, 4, 3))
    IM[:, :, 0] = [[1, 1, 0, 1], [0, 0, 1, 1], [1, 0, 1, 0], [1, 1, 1, 1]]
    IM[:, :, 1] = [[0, 1, 0, 0], [1, 0, 0, 1], [0, 1, 1, 0], [0, 0, 0, 1]]
    IM[:, :, 2] = [[1, 1, 1, 1], [1, 1, 0, 1], [0, 1, 1, 0], [1, 0, 1, 0]]
    LB = np.zeros((4, 4, 3))
    LB[0, 0, 0], LB[0, 1, 0] = -0.1, -0.2
    LB[0, 0, 1], LB[0, 1, 1] = -0.1, -0.15
    LB[:, :, 2] = LB[:, :, 1]
    k["relu_reach_IM"], k["relu_reach_LB"], k["relu_reach_UB"] = IM, LB, -LB
    # results/tests/baselines/set/test_star_isEmptySet_results.mat (code/nnv/tests/set/star/test_star_isEmptySet.m)
    m = sio.loadmat(os.path.join(ref_root, "results/tests/baselines/set/test_star_isEmptySet_results.mat"))
    for key in ("S_V", "S_C", "S_d", "S1_V", "S1_C", "S1_d", "b_nonempty", "b_empty"):
        k["empty_" + key] = m[key].astype(float)
    # results/tests/baselines/set/test_star_intersect_halfSpace_results.mat
    m = sio.loadmat(os.path.join(ref_root, "results/tests/baselines/set/test_star_intersect_halfSpace_results.mat"))
    for key in ("H", "g", "S_V", "S1_C", "S1_d", "S1_isEmpty"):
        k["hs_" + key] = m[key].astype(float)
    # results/tests/baselines/set/test_star_affineMap_results.mat (code/nnv/tests/set/star/test_star_affineMap.m)
    m = sio.loadmat(os.path.join(ref_root, "results/tests/baselines/set/test_star_affineMap_results.mat"))
    for key in ("W", "b", "S_V", "S1_V", "W2", "S4_lb", "S4_ub"):
        k["aff_" + key] = m[key].astype(float)
    # results/tests/baselines/set/test_star_getBoxFast_results.mat (code/nnv/tests/set/star/test_star_getBoxFast.m)
    m = sio.loadmat(os.path.join(ref_root, "results/tests/baselines/set/test_star_getBoxFast_results.mat"))
    for key in ("I1_V", "I1_C", "I1_d", "B2_lb", "B2_ub"):
        k["box_" + key] = m[key].astype(float)
    return k


def oracle_small():
    out = {}
    for name, small, nq in SMALL_CASES:
        cfg = make_config(name, n_queries=nq, small=small)
        tag = name
        verdicts = []
        for q, qu in enumerate(cfg["queries"]):
            S = O.reach(cfg["layers"], O.star_from_query(qu))
            lb, ub = O.output_ranges(S)
            out["%s_q%d_lb" % (tag, q)] = lb
            out["%s_q%d_ub" % (tag, q)] = ub
            out["%s_q%d_P" % (tag, q)] = np.array([t["P_out"] for t in S.trace], dtype=np.int64)
            for li, t in enumerate(S.trace):
                out["%s_q%d_cross%d" % (tag, q, li)] = t["cross"].astype(np.int64)
            G, g = O.robustness_set(len(lb), qu["target"], qu["spec"])
            verdicts.append(O.verify_specification(S, G, g))
        out[tag + "_verdicts"] = np.array(verdicts, dtype=np.int64)
    return out


if __name__ == "__main__":
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NNV_REFERENCE_ROOT")
    if not ref_root:
        sys.exit("usage: make_golden.py <root of the reference checkout>")
    np.savez_compressed(os.path.join(HERE, "reference_kats.npz"), **reference_kats(ref_root))
    np.savez_compressed(os.path.join(HERE, "oracle_small.npz"), **oracle_small())
    for f in ("reference_kats.npz", "oracle_small.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")
