"""Per-layer parity of the CUDA kernels (through the C ABI) against the CPU
oracle: every affine layer map and Star.estimateRanges, over shapes that hit
ragged tiles, strides, dilation, padding and the column-packed small images.
Tolerance: 1e-9 relative to the largest magnitude of the result (FP64)."""
import numpy as np
import pytest
import scipy.sparse as sp

from oracle import nnv_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-9


def _rel(a, b):
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-300)


def _star(V):
    P = V.shape[3] - 1
    return O.ImageStar(np.asfortranarray(V), sp.csr_matrix((0, P)), np.zeros(0), -np.ones(P), np.ones(P))


CONV_CASES = [
    # H, W, Cin, Cout, k, pad, stride, dil, ncols
    (5, 5, 1, 1, 3, (0, 0, 0, 0), (1, 1), (1, 1), 1),
    (32, 32, 3, 32, 3, (1, 1, 1, 1), (1, 1), (1, 1), 37),
    (32, 32, 32, 32, 3, (1, 1, 1, 1), (1, 1), (1, 1), 9),
    (16, 16, 32, 64, 3, (1, 1, 1, 1), (1, 1), (1, 1), 130),
    (28, 28, 1, 8, 3, (1, 1, 1, 1), (1, 1), (1, 1), 21),
    (28, 28, 8, 16, 3, (0, 0, 0, 0), (2, 2), (1, 1), 33),
    (8, 8, 16, 16, 3, (1, 1, 1, 1), (1, 1), (1, 1), 19),      # two columns per tile
    (4, 4, 5, 70, 3, (1, 1, 1, 1), (1, 1), (1, 1), 67),       # many columns per tile, two channel tiles
    (13, 11, 7, 10, 3, (2, 1, 0, 2), (1, 2), (1, 1), 5),      # asymmetric padding, mixed stride
    (17, 17, 4, 6, 3, (2, 2, 2, 2), (1, 1), (2, 2), 6),       # dilation
    (9, 9, 3, 5, 1, (0, 0, 0, 0), (1, 1), (1, 1), 4),         # 1x1 filter
    (12, 12, 2, 3, 5, (2, 2, 2, 2), (1, 1), (1, 1), 3),       # 5x5 filter
    (40, 40, 3, 130, 3, (1, 1, 1, 1), (1, 1), (1, 1), 3),     # three channel tiles, ragged spatial tiles
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_parity(ctx, case):
    H, W, Cin, Cout, k, pad, stride, dil, ncols = case
    rng = np.random.default_rng(hash(case) % (2 ** 31))
    V = rng.standard_normal((H, W, Cin, ncols))
    V[..., ncols // 2] *= (rng.uniform(size=(H, W, Cin)) > 0.7)       # a sparse generator
    L = {"type": "conv2d", "W": rng.standard_normal((k, k, Cin, Cout)), "b": rng.standard_normal(Cout),
         "pad": pad, "stride": stride, "dilation": dil}
    ref = O.conv2d_reach(_star(V), L).V
    got = ctx.layer_apply(L, V)
    assert got.shape == ref.shape
    assert _rel(got, ref) < TOL


def test_conv_kat_on_gpu(ctx, kats):
    # code/nnv/tests/nn/layers/Conv2DLayer/test_layers_Conv2D.m:14-27
    L = {"type": "conv2d", "W": kats["conv_W"][:, :, None, None], "b": np.zeros(1), "pad": (0, 0, 0, 0),
         "stride": (1, 1), "dilation": (1, 1)}
    got = ctx.layer_apply(L, kats["conv_I"][:, :, None, None])
    assert np.array_equal(got[:, :, 0, 0], kats["conv_expected"])


@pytest.mark.parametrize("nin,nout,ncols", [(5, 50, 6), (50, 50, 13), (50, 5, 40), (2704, 128, 70), (4096, 256, 150),
                                             (128, 10, 300), (33, 17, 129), (1, 1, 1), (7, 3, 1)])
def test_fc_parity(ctx, nin, nout, ncols):
    rng = np.random.default_rng(nin * 1000 + nout)
    V = rng.standard_normal((nin, 1, 1, ncols))
    L = {"type": "fc", "W": rng.standard_normal((nout, nin)), "b": rng.standard_normal(nout)}
    ref = O.fc_reach(_star(V), L).V
    got = ctx.layer_apply(L, V)
    assert got.shape == ref.shape and _rel(got, ref) < TOL


def test_fc_kats_on_gpu(ctx, kats):
    # code/nnv/tests/soundness/test_regression_layers.m:52-65 and the stored affineMap baseline
    got = ctx.layer_apply({"type": "fc", "W": kats["fc_W"], "b": kats["fc_b"]}, kats["fc_x"].reshape(2, 1, 1, 1))
    assert np.abs(got.ravel() - kats["fc_expected"]).max() < 1e-10
    got = ctx.layer_apply({"type": "fc", "W": kats["aff_W"], "b": kats["aff_b"].ravel()},
                          kats["aff_S_V"].reshape(2, 1, 1, 4, order="F"))
    assert np.abs(got.reshape(2, 4, order="F") - kats["aff_S1_V"]).max() < 1e-12


@pytest.mark.parametrize("shape,ncols", [((6, 5, 3), 4), ((32, 32, 32), 7), ((1, 1, 9), 5), ((3, 3, 1), 1)])
def test_bn_parity(ctx, shape, ncols):
    rng = np.random.default_rng(sum(shape))
    c = shape[2]
    V = rng.standard_normal(shape + (ncols,))
    L = {"type": "bn", "mean": rng.standard_normal(c), "var": rng.uniform(0.1, 2, c), "scale": rng.uniform(0.5, 1.5, c),
         "offset": rng.standard_normal(c), "eps": 1e-5}
    ref = O.bn_reach(_star(V), L).V
    got = ctx.layer_apply(L, V)
    assert np.array_equal(got, ref)          # same operation order: bit-identical


def test_bn_after_conv_is_fused_and_matches(ctx):
    from nnv_b200.engine import Batch, Network
    rng = np.random.default_rng(5)
    V = rng.standard_normal((10, 9, 3, 6))
    conv = {"type": "conv2d", "W": rng.standard_normal((3, 3, 3, 12)), "b": rng.standard_normal(12),
            "pad": (1, 1, 1, 1), "stride": (1, 1), "dilation": (1, 1)}
    bn = {"type": "bn", "mean": rng.standard_normal(12), "var": rng.uniform(0.1, 2, 12),
          "scale": rng.uniform(0.5, 1.5, 12), "offset": rng.standard_normal(12), "eps": 1e-5}
    ref = O.bn_reach(O.conv2d_reach(_star(V), conv), bn).V
    net = Network(ctx, [conv, bn], (10, 9, 3))
    b = Batch(net, [{"V": V, "pl": -np.ones(5), "pu": np.ones(5)}])
    b.upload()
    b.reach()
    assert _rel(b.get_V(0), ref) < TOL


@pytest.mark.parametrize("shape,pool,stride,pad,ncols,divisor", [
    ((4, 4, 1), (2, 2), (2, 2), (0, 0, 0, 0), 1, "inside"),
    ((5, 5, 3), (3, 3), (2, 2), (0, 0, 0, 0), 2, "window"),
    ((32, 32, 32), (2, 2), (2, 2), (0, 0, 0, 0), 9, "inside"),
    ((7, 9, 2), (3, 2), (2, 1), (1, 0, 1, 1), 5, "window"),
    ((7, 9, 2), (3, 2), (2, 1), (1, 0, 1, 1), 5, "inside"),
    ((8, 8, 3), (3, 3), (2, 2), (1, 2, 2, 1), 4, "inside"),
])
def test_avgpool_parity(ctx, shape, pool, stride, pad, ncols, divisor):
    rng = np.random.default_rng(sum(shape) + ncols)
    V = rng.standard_normal(shape + (ncols,))
    L = {"type": "avgpool", "pool": pool, "stride": stride, "pad": pad, "divisor": divisor}
    ref = O.avgpool_reach(_star(V), L).V
    got = ctx.layer_apply(L, V)
    assert got.shape == ref.shape and np.array_equal(got, ref)      # same summation order


def test_avgpool_kats_on_gpu(ctx, kats):
    L = {"type": "avgpool", "pool": (2, 2), "stride": (2, 2), "pad": (0, 0, 0, 0)}
    assert np.array_equal(ctx.layer_apply(L, kats["avg_I"][:, :, None, None])[:, :, 0, 0], kats["avg_expected_mat"])
    assert np.array_equal(ctx.layer_apply(L, kats["avg2_I"][:, :, None, None])[:, :, 0, 0], kats["avg2_expected"])


@pytest.mark.parametrize("N,P", [(1, 0), (1, 1), (10, 951), (50, 12), (128, 930), (256, 3000), (257, 4), (6272, 785),
                                  (32768, 300), (1023, 1025)])
def test_estimate_ranges_parity(ctx, N, P):
    rng = np.random.default_rng(N + P)
    M = rng.standard_normal((N, P + 1)) * (rng.uniform(size=(N, P + 1)) > 0.5)
    pl = -rng.uniform(0, 1, P)
    pu = rng.uniform(0, 1, P)
    rl, ru = O.estimate_ranges(M, pl, pu)
    lb, ub = ctx.estimate_ranges(M, pl, pu)
    scale = np.abs(M).sum(axis=1).max() + 1e-300
    assert np.abs(lb - rl).max() / scale < 1e-12
    assert np.abs(ub - ru).max() / scale < 1e-12
    # rows without generators: lb = ub = centre exactly
    M[0, 1:] = 0
    lb, ub = ctx.estimate_ranges(M, pl, pu)
    assert lb[0] == M[0, 0] and ub[0] == M[0, 0]


def test_estimate_ranges_default_predicate_box(ctx):
    # Star.m:1091-1096: empty predicate bounds default to [-1, 1]
    M = np.array([[1., 2., -3.], [0., 0.5, 0.25]])
    lb, ub = ctx.estimate_ranges(M)
    assert np.array_equal(lb, [-4., -0.75]) and np.array_equal(ub, [6., 0.75])


def test_get_box_fast_baseline_on_gpu(ctx, kats):
    from scipy.optimize import linprog
    V, C, d = kats["box_I1_V"], kats["box_I1_C"], kats["box_I1_d"].ravel()
    P = C.shape[1]
    pl, pu = np.zeros(P), np.zeros(P)
    for i in range(P):
        e = np.zeros(P)
        e[i] = 1
        pl[i] = linprog(e, A_ub=C, b_ub=d, bounds=[(None, None)] * P, method="highs").fun
        pu[i] = -linprog(-e, A_ub=C, b_ub=d, bounds=[(None, None)] * P, method="highs").fun
    lb, ub = ctx.estimate_ranges(V, pl, pu)
    assert np.abs(lb - kats["box_B2_lb"].ravel()).max() < 1e-6
    assert np.abs(ub - kats["box_B2_ub"].ravel()).max() < 1e-6


def test_bad_layer_arguments(ctx):
    from nnv_b200._lib import NNVError
    V = np.zeros((4, 4, 2, 1))
    with pytest.raises(NNVError, match="channels"):
        ctx.layer_apply({"type": "conv2d", "W": np.zeros((3, 3, 3, 4)), "b": np.zeros(4)}, V)
    with pytest.raises(NNVError, match="InputSize"):
        ctx.layer_apply({"type": "fc", "W": np.zeros((3, 5)), "b": np.zeros(3)}, V)
    with pytest.raises(NNVError, match="larger than padded input"):
        ctx.layer_apply({"type": "conv2d", "W": np.zeros((7, 7, 2, 1)), "b": np.zeros(1)}, V)
