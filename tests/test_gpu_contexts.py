"""Two engine contexts on one GPU, driven from two host threads at the same time (what ``bench.py --contexts``
does): the library keeps its state per context (stream, arena, working buffers; the error text per thread), so
both threads must get the sets a single context gets."""
import threading

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _reach_all(device, cfg, out, key, rounds):
    from nnv_b200.engine import Batch, Context, Network
    ctx = Context(device, 1 << 30)
    net = Network(ctx, cfg["layers"], cfg["in_shape"])
    res = None
    for _ in range(rounds):
        b = Batch(net, cfg["queries"])
        b.upload()
        b.reach(keep_layer_bounds=True)
        res = [(b.get_V(q), b.get_ranges(q), b.get_crossing(q, 0)[0]) for q in range(len(cfg["queries"]))]
        b.close()
    net.close()
    ctx.close()
    out[key] = res


def test_two_contexts_in_two_threads_agree_with_one():
    from nnv_b200.configs import make_config
    cfg = make_config("cnn32", n_queries=3, small=True)
    out = {}
    _reach_all(0, cfg, out, "single", 1)
    threads = [threading.Thread(target=_reach_all, args=(0, cfg, out, k, 4)) for k in ("a", "b")]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert set(out) == {"single", "a", "b"}
    for k in ("a", "b"):
        for (V, (lb, ub), cr), (V0, (lb0, ub0), cr0) in zip(out[k], out["single"]):
            assert np.array_equal(cr, cr0)
            assert np.array_equal(V, V0) and np.array_equal(lb, lb0) and np.array_equal(ub, ub0)
