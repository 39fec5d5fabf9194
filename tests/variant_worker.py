"""One process of the kernel-variant equivalence check (launched by tests/test_gpu_variants.py with an
environment switch set): reach two seeded workloads on the default path and save the output sets."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    from nnv_b200.configs import make_config
    from nnv_b200.engine import Batch, Context, Network

    out = sys.argv[1]
    ctx = Context(0, 2 << 30)
    res = {}
    for name, nq in (("cnn32", 3), ("cnn28", 2), ("vgg224", 1)):
        cfg = make_config(name, n_queries=nq, small=True)
        net = Network(ctx, cfg["layers"], cfg["in_shape"])
        b = Batch(net, cfg["queries"])
        b.upload()
        b.reach(keep_layer_bounds=True)
        n_relu = sum(1 for l in cfg["layers"] if l["type"] == "relu")
        for q in range(nq):
            res["%s_V%d" % (name, q)] = b.get_V(q)
            lb, ub = b.get_ranges(q)
            res["%s_lb%d" % (name, q)] = lb
            res["%s_ub%d" % (name, q)] = ub
            for li in range(n_relu):
                idx, cl, cu = b.get_crossing(q, li)
                res["%s_cross%d_%d" % (name, q, li)] = idx
        verdict, status, margin = b.verify_robust([qu["target"] for qu in cfg["queries"]], cfg["queries"][0]["spec"])
        res["%s_verdict" % name] = np.asarray(verdict)
        b.close()
        net.close()
    # channel counts of three 8-channel chunks and more: the windowed convolution then runs in its persistent,
    # warp-specialised form (the small configurations above have too few channels for it)
    from nnv_b200.configs import _conv, _bn, _fc, RELU, out_shape
    rng = np.random.default_rng(43)
    shape = (14, 12, 3)
    pool = {"type": "avgpool", "pool": (2, 2), "stride": (2, 2), "pad": (0, 0, 0, 0)}
    layers = [_conv(rng, 3, 3, 3, 32, (1, 1, 1, 1)), _bn(rng, 32), RELU,
              _conv(rng, 3, 3, 32, 40, (1, 1, 1, 1)), RELU, dict(pool),
              _conv(rng, 3, 5, 40, 64, (1, 1, 2, 2)), _bn(rng, 64), RELU, dict(pool)]
    h, w, c = out_shape(layers, shape)
    layers += [_fc(rng, h * w * c, 24), RELU, _fc(rng, 24, 5)]
    queries = []
    for k in range(3):
        x = rng.uniform(0, 1, shape)
        e = np.zeros(shape)
        e[k::4, 1::3, :] = 0.02
        e[0, 0, :] = e[-1, -1, :] = 0.02
        queries.append({"lb": np.maximum(x - e, 0), "ub": np.minimum(x + e, 1)})
    net = Network(ctx, layers, shape)
    b = Batch(net, queries)
    b.upload()
    b.reach(keep_layer_bounds=True)
    for q in range(len(queries)):
        res["wide_V%d" % q] = b.get_V(q)
        lb, ub = b.get_ranges(q)
        res["wide_lb%d" % q] = lb
        res["wide_ub%d" % q] = ub
        for li in range(4):
            res["wide_cross%d_%d" % (q, li)] = b.get_crossing(q, li)[0]
    b.close()
    net.close()
    ctx.close()
    np.savez(out, **res)


if __name__ == "__main__":
    main()
