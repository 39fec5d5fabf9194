"""Generator sharding of a set over two GPUs (NCCL all-reduce of the partial bound sums per ReLU
layer) against the CPU oracle.  Needs two GPUs; on a single-GPU box only the world-size-1 form of
the same entry points is checked."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run_ranks(mode, port):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port),
                        os.path.join(ROOT, "tests", "sharded_worker.py"), mode],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


@pytest.mark.parametrize("mode,port", [("hook", 29533), ("nccl", 29534), ("peer", 29535)])
def test_two_rank_generator_sharding_matches_oracle(mode, port):
    """hook: the caller's all-reduce callback; nccl: the library's own NCCL all-reduce; peer: partial sums in
    peer-mapped buffers, added inside the classification kernel."""
    assert "SHARDED PARITY OK" in _run_ranks(mode, port)


def test_capacity_stop_is_the_same_on_every_rank():
    """One rank's arena is too small for its share: all ranks return the capacity status together."""
    assert "SHARDED CAPACITY OK" in _run_ranks("capacity", 29536)


def test_world_size_one_shard_is_the_plain_path(ctx):
    from nnv_b200.configs import make_config
    from nnv_b200.engine import Batch, Network
    cfg = make_config("cnn28", n_queries=2, small=True)
    net = Network(ctx, cfg["layers"], cfg["in_shape"])
    b = Batch(net, cfg["queries"])
    b.upload()
    b.reach()
    ref = [b.get_V(q) for q in range(2)]
    b.close()
    ctx.set_shard(0, 1)
    b = Batch(net, cfg["queries"])
    b.upload()
    b.reach()
    for q in range(2):
        assert np.array_equal(b.get_V(q), ref[q])
    b.close()
    net.close()
