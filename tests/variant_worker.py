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
    ctx.close()
    np.savez(out, **res)


if __name__ == "__main__":
    main()
