"""One rank of the generator-sharded GPU parity check (launched by tests/test_gpu_sharded.py through
torch.distributed.run, one process per GPU, NCCL).  Every rank reaches its share of each query's
generators; the sum over ranks of the per-rank outputs must match the CPU oracle's unsharded set.

argv[1] picks the transport of the bound sums: "hook" (the caller's all-reduce callback), "nccl" (the
library's own NCCL all-reduce), "peer" (peer-mapped buffers added inside the classification kernel), or
"capacity": rank 1 gets an arena too small for its share, and every rank must come back with the capacity
status instead of one of them waiting in a collective for the rank that stopped."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist

    from nnv_b200 import _lib
    from nnv_b200.configs import make_config
    from nnv_b200.engine import Batch, Context, Network
    from oracle import nnv_oracle as O

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    mode = sys.argv[1] if len(sys.argv) > 1 else "hook"
    if mode == "capacity":
        ctx = Context(local, (4 << 30) if rank != 1 else (1 << 20))
        ctx.set_shard_nccl(rank, world, peer_memory=True)
        cfg = make_config("cnn32", n_queries=2, small=True)
        net = Network(ctx, cfg["layers"], cfg["in_shape"])
        b = Batch(net, cfg["queries"])
        b.upload()
        try:
            b.reach(keep_layer_bounds=True)
            status = 0
        except _lib.NNVError as e:
            status = e.status
        flag = torch.tensor([1 if status == _lib.NNVB_E_CAPACITY else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            print("SHARDED CAPACITY OK" if int(flag) == 1 else "SHARDED CAPACITY FAIL (status %d)" % status, flush=True)
        b.close()
        net.close()
        ctx.close()
        dist.destroy_process_group()
        sys.exit(0 if int(flag) == 1 else 1)
    ctx = Context(local, 4 << 30)
    if mode == "hook":
        ctx.set_shard(rank, world)
    else:
        ctx.set_shard_nccl(rank, world, peer_memory=(mode == "peer"))
    ok = True
    for name, nq in (("cnn32", 2), ("vgg224", 1), ("bright28", 3), ("fc5", 4)):
        cfg = make_config(name, n_queries=nq, small=(name != "fc5"))
        net = Network(ctx, cfg["layers"], cfg["in_shape"])
        b = Batch(net, cfg["queries"])
        b.upload()
        b.reach(keep_layer_bounds=True)
        verdict, status, margin = b.verify_robust([q["target"] for q in cfg["queries"]], cfg["queries"][0]["spec"])
        for q, qu in enumerate(cfg["queries"]):
            S = O.reach(cfg["layers"], O.star_from_query(qu))
            P, _ = b.out_dims(q)
            Vloc = b.get_V(q)
            Vt = torch.from_numpy(np.ascontiguousarray(Vloc.reshape(-1, order="F"))).cuda()
            dist.all_reduce(Vt)
            Vsum = Vt.cpu().numpy().reshape(Vloc.shape, order="F")
            pl, pu = b.get_pred_bounds(q)
            pt = torch.from_numpy(np.stack([pl, pu])).cuda()
            dist.all_reduce(pt)
            lb, ub = b.get_ranges(q)
            rl, ru = O.output_ranges(S)
            scale = max(np.abs(rl).max(), np.abs(ru).max())
            good = P == S.P and Vsum.shape == S.V.shape
            good = good and np.abs(Vsum - S.V).max() / np.abs(S.V).max() < 1e-9
            good = good and np.abs(lb - rl).max() / scale < 1e-9 and np.abs(ub - ru).max() / scale < 1e-9
            good = good and np.array_equal(pt[0].cpu().numpy(), S.pl)
            good = good and np.abs(pt[1].cpu().numpy() - S.pu).max() <= 1e-9 * max(1.0, np.abs(S.pu).max())
            for li, t in enumerate(S.trace):
                idx, _, _ = b.get_crossing(q, li)
                good = good and np.array_equal(idx, t["cross"])
            G, g = O.robustness_set(len(rl), qu["target"], qu["spec"])
            ref = O.verify_specification(S, G, g)
            good = good and verdict[q] in (ref, _lib.UNDECIDED)
            if not good:
                print("rank %d: %s query %d MISMATCH (P %d vs %d, verdict %d vs %d)" % (rank, name, q, P, S.P, verdict[q], ref),
                      flush=True)
            ok = ok and good
        # every rank must see the same verdicts and margins
        vt = torch.from_numpy(margin.copy()).cuda()
        v0 = vt.clone()
        dist.broadcast(v0, 0)
        ok = ok and bool(torch.equal(vt, v0))
        b.close()
        net.close()
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("SHARDED PARITY OK" if int(flag) == 1 else "SHARDED PARITY FAIL", flush=True)
    ctx.close()
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
