"""World-size-2 check (gloo, CPU) of the generator-sharding scheme the CUDA engine uses on several
GPUs: predicate j on rank j % world, centre replicated, partial bound sums all-reduced before each
ReLU classification, new column c on rank c % world.  Each rank runs the oracle's layer maps on its
own columns; the union of the ranks' columns must reproduce the unsharded oracle set."""
import os
import socket

import numpy as np
import pytest
import scipy.sparse as sp

from nnv_b200 import sharding
from nnv_b200.configs import make_config
from oracle import nnv_oracle as O


def test_index_helpers():
    for world in (1, 2, 3, 8):
        for P in (0, 1, 5, 17):
            allpos = np.concatenate([sharding.shard_positions(P, r, world) for r in range(world)])
            assert sorted(allpos.tolist()) == list(range(P))
            assert [sharding.shard_count(P, r, world) for r in range(world)] == \
                [len(sharding.shard_positions(P, r, world)) for r in range(world)]
    new_off = np.array([0, 3, 3, 10])
    for world in (2, 4):
        for q in range(3):
            cs = np.concatenate([sharding.local_new_columns(new_off, q, r, world) for r in range(world)])
            assert sorted(cs.tolist()) == list(range(new_off[q], new_off[q + 1]))
            for r in range(world):
                assert all(c % world == r for c in sharding.local_new_columns(new_off, q, r, world))


def _sharded_reach(rank, world, layers, query, dist):
    """One rank of a generator-sharded reach, written with the oracle's layer maps."""
    import torch
    S = O.star_from_query(query)
    pos = sharding.shard_positions(S.P, rank, world)            # predicate positions held here
    V = np.concatenate([S.V[..., :1], S.V[..., 1 + pos]], axis=3)
    pl, pu = S.pl[pos], S.pu[pos]
    P_glob = S.P
    crossings = []
    for L in layers:
        loc = O.ImageStar(np.asfortranarray(V), sp.csr_matrix((0, V.shape[3] - 1)), np.zeros(0), pl, pu)
        t = L["type"]
        if t == "conv2d":
            V = O.conv2d_reach(loc, L).V
        elif t == "fc":
            V = O.fc_reach(loc, L).V
        elif t == "bn":
            V = O.bn_reach(loc, L).V
        elif t == "avgpool":
            V = O.avgpool_reach(loc, L).V
        elif t == "relu":
            M = loc.mat()
            G = M[:, 1:]
            part = np.stack([np.maximum(G, 0) @ pl + np.minimum(G, 0) @ pu,
                             np.maximum(G, 0) @ pu + np.minimum(G, 0) @ pl])
            tt = torch.from_numpy(part)
            dist.all_reduce(tt)                                  # the one collective of the path
            lb, ub = M[:, 0] + tt[0].numpy(), M[:, 0] + tt[1].numpy()
            dead = np.nonzero(ub <= 0)[0]
            cross = np.nonzero((lb < 0) & (ub > 0))[0]
            crossings.append(cross)
            M = M.copy()
            M[dead, :] = 0
            M[cross, :] = 0
            mine = sharding.local_new_columns(np.array([0, len(cross)]), 0, rank, world)
            newc = np.zeros((M.shape[0], len(mine)))
            newc[cross[mine], np.arange(len(mine))] = 1.0
            M = np.hstack([M, newc])
            pos = np.concatenate([pos, P_glob + mine])
            pl = np.concatenate([pl, np.zeros(len(mine))])
            pu = np.concatenate([pu, ub[cross[mine]]])
            P_glob += len(cross)
            V = M.reshape(loc.V.shape[:3] + (M.shape[1],), order="F")
    return V, pos, pl, pu, P_glob, crossings


def _worker(rank, world, port, name, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = make_config(name, n_queries=1, small=True)
        V, pos, pl, pu, P_glob, crossings = _sharded_reach(rank, world, cfg["layers"], cfg["queries"][0], dist)
        # every rank contributes its columns at their predicate positions; the sum is the set
        import torch
        n = int(np.prod(V.shape[:3]))
        full = np.zeros((n, P_glob + 1))
        M = V.reshape(n, -1, order="F")
        if rank == 0:
            full[:, 0] = M[:, 0]
        full[:, 1 + pos] = M[:, 1:]
        bounds = np.zeros((2, P_glob))
        bounds[0, pos], bounds[1, pos] = pl, pu
        tf, tb = torch.from_numpy(full), torch.from_numpy(bounds)
        dist.all_reduce(tf)
        dist.all_reduce(tb)
        if rank == 0:
            ref = O.reach(cfg["layers"], O.star_from_query(cfg["queries"][0]))
            assert ref.P == P_glob
            for a, t in zip(crossings, ref.trace):
                assert np.array_equal(a, t["cross"])
            scale = np.abs(ref.mat()).max()
            assert np.abs(tf.numpy() - ref.mat()).max() / scale < 1e-12
            assert np.array_equal(tb[0].numpy(), ref.pl)
            assert np.abs(tb[1].numpy() - ref.pu).max() <= 1e-12 * max(1.0, np.abs(ref.pu).max())
            q.put("ok")
    except Exception as exc:      # pragma: no cover - reported through the queue
        if rank == 0:
            q.put("fail: %r" % (exc,))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name", ["cnn28", "cnn32"])
def test_sharded_scheme_two_ranks_gloo(name):
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, name, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert all(p.exitcode == 0 for p in procs)
    assert q.get(timeout=5) == "ok"


def _agree_worker(rank, world, port, q):
    """The go / no-go protocol of a sharded reach: every rank contributes "I cannot go on" (its share does
    not fit its arena), the sum comes back, and all ranks stop at the same point or none does."""
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        arena = [1 << 30, 1 << 20][rank]                 # rank 1 has the small arena
        cols = [sharding.shard_count(3000, rank, world) + 1, sharding.shard_count(7000, rank, world) + 1]
        stopped_at = None
        for layer, (n_rows, c) in enumerate(zip([4096, 4096], cols)):
            flag = torch.tensor([1.0 if n_rows * c * 8 > arena // 2 else 0.0], dtype=torch.float64)
            dist.all_reduce(flag)                        # the one-double sum every rank takes part in
            if flag.item() > 0:
                stopped_at = layer
                break
        q.put((rank, stopped_at))
    finally:
        dist.destroy_process_group()


def test_capacity_stop_is_agreed_on_by_all_ranks_gloo():
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_agree_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert all(p.exitcode == 0 for p in procs)
    got = dict(q.get(timeout=5) for _ in range(2))
    assert got[0] == got[1] == 0                         # rank 0 fits, yet it stops where rank 1 does
