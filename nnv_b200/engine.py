"""Thin object wrappers over the C ABI: Context, Network, Batch.

These hold the opaque handles and move NumPy arrays (FP64, column-major) across
the boundary.  The reference-shaped API (NN, ImageStar, layers ...) in
``nnv_b200.nn`` is written on top of them.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L


def _dp(a):
    # the address as an integer: the double* parameters are declared void* on the Python side, which accepts it
    # without building a typed pointer object per call (this sits on the per-set path of large batches)
    return a.__array_interface__["data"][0] if a is not None else None


def _f64(a, order="F"):
    if type(a) is np.ndarray and a.dtype == np.float64:
        f = a.flags
        if f.aligned and (f.f_contiguous if order == "F" else f.c_contiguous):
            return a
    return np.require(np.asarray(a, dtype=np.float64), requirements=["F" if order == "F" else "C", "A"])


class Context:
    """One GPU context (``nnvb_init``): a stream and the generator arena."""

    def __init__(self, device=0, arena_bytes=0):
        self.lib = L.load()
        h = C.c_void_p()
        L.check(self.lib.nnvb_init(int(device), int(arena_bytes), C.byref(h)), "nnvb_init")
        self.handle = h
        self.device = device

    def close(self):
        if getattr(self, "handle", None):
            self.lib.nnvb_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def stream(self):
        return self.lib.nnvb_stream(self.handle)

    @property
    def launch_count(self):
        return int(self.lib.nnvb_launch_count(self.handle))

    def set_shard(self, rank, world, group=None):
        """Shard the generators of every later batch over ``world`` ranks (this process is
        ``rank``); the partial bound sums are added with torch.distributed on ``group``."""
        from .sharding import make_allreduce_hook
        self._hook = make_allreduce_hook(group) if world > 1 else L.ALLREDUCE_FN(0)
        L.check(self.lib.nnvb_set_shard(self.handle, int(rank), int(world), self._hook, None), "nnvb_set_shard")
        self.rank, self.world = int(rank), int(world)

    def set_shard_nccl(self, rank, world, peer_memory=False, group=None):
        """The same sharding with the collective inside the library (``nnvb_set_shard_nccl``): NCCL bound by
        the library itself and, with ``peer_memory``, the fused sum-and-classify kernel over peer-mapped
        buffers.  torch.distributed only carries the 128-byte communicator id from rank 0 to the others."""
        buf = C.create_string_buffer(L.NCCL_ID_BYTES)
        if world > 1:
            import torch
            import torch.distributed as dist
            if rank == 0:
                L.check(self.lib.nnvb_nccl_unique_id(buf), "nnvb_nccl_unique_id")
            t = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8).clone()
            if dist.get_backend(group) == "nccl":
                t = t.cuda()
            dist.broadcast(t, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            buf = C.create_string_buffer(bytes(t.cpu().numpy().tobytes()), L.NCCL_ID_BYTES)
        L.check(self.lib.nnvb_set_shard_nccl(self.handle, int(rank), int(world), buf, int(bool(peer_memory))),
                "nnvb_set_shard_nccl")
        self.rank, self.world = int(rank), int(world)

    def profile_enable(self, on=True):
        """Start (and zero) or stop the per-kernel-family device timers."""
        L.check(self.lib.nnvb_profile_enable(self.handle, int(bool(on))), "nnvb_profile_enable")

    def profile_read(self):
        """{family: {"ms", "launches", "work"}} accumulated since profile_enable."""
        out = {}
        for i, name in enumerate(L.PROF_FAMILIES):
            ms, n, work = C.c_double(), C.c_int64(), C.c_double()
            L.check(self.lib.nnvb_profile_read(self.handle, i, C.byref(ms), C.byref(n), C.byref(work)),
                    "nnvb_profile_read")
            out[name] = {"ms": ms.value, "launches": n.value, "work": work.value}
        return out

    # single-layer entry points ------------------------------------------------
    def layer_apply(self, layer, V):
        """Apply one affine layer to V[H,W,C,ncols]; returns the output tensor."""
        V = _f64(V)
        h, w, c, ncols = V.shape
        keep = []
        desc = make_layer_desc(layer, keep)
        # output size: ask a throw-away network
        net = Network(self, [layer], (h, w, c))
        ho, wo, co = net.out_shape
        net.close()
        out = np.empty((ho, wo, co, ncols), dtype=np.float64, order="F")
        shp = (C.c_int64 * 3)()
        L.check(self.lib.nnvb_layer_apply(self.handle, C.byref(desc), h, w, c, ncols, _dp(V), _dp(out), shp),
                "nnvb_layer_apply")
        assert tuple(shp) == (ho, wo, co)
        return out

    def estimate_ranges(self, M, pl=None, pu=None):
        """Star.estimateRanges of the N x (P+1) matrix M."""
        M = _f64(M)
        n, p1 = M.shape
        pl = None if pl is None else _f64(pl).ravel()
        pu = None if pu is None else _f64(pu).ravel()
        lb = np.empty(n)
        ub = np.empty(n)
        L.check(self.lib.nnvb_estimate_ranges(self.handle, n, p1 - 1, _dp(M), _dp(pl), _dp(pu), _dp(lb), _dp(ub)),
                "nnvb_estimate_ranges")
        return lb, ub


def make_layer_desc(layer, keep):
    """Translate a neutral layer dict into an nnvb_layer_desc; arrays that must
    outlive the call are appended to ``keep``."""
    d = L.LayerDesc()
    t = layer["type"]
    if t == "conv2d":
        W = _f64(layer["W"])
        if W.ndim != 4:
            raise ValueError("conv2d weights must be [kh,kw,Cin,Cout]")
        b = _f64(layer["b"]).ravel()
        keep += [W, b]
        d.type = L.LAYER_CONV2D
        d.kh, d.kw, d.cin, d.cout = W.shape
        d.pad = (C.c_int32 * 4)(*[int(x) for x in layer.get("pad", (0, 0, 0, 0))])
        d.stride = (C.c_int32 * 2)(*[int(x) for x in layer.get("stride", (1, 1))])
        d.dilation = (C.c_int32 * 2)(*[int(x) for x in layer.get("dilation", (1, 1))])
        d.W, d.b = _dp(W), _dp(b)
    elif t == "fc":
        W = _f64(layer["W"])
        b = _f64(layer["b"]).ravel()
        keep += [W, b]
        d.type = L.LAYER_FC
        d.cout, d.cin = W.shape
        d.W, d.b = _dp(W), _dp(b)
    elif t == "bn":
        arrs = [_f64(layer[k]).ravel() for k in ("mean", "var", "scale", "offset")]
        keep += arrs
        d.type = L.LAYER_BN
        d.cout = arrs[0].size
        d.bn_mean, d.bn_var, d.bn_scale, d.bn_offset = (_dp(a) for a in arrs)
        d.bn_eps = float(layer.get("eps", 1e-5))
    elif t == "avgpool":
        d.type = L.LAYER_AVGPOOL2D
        d.pool = (C.c_int32 * 2)(*[int(x) for x in layer["pool"]])
        d.stride = (C.c_int32 * 2)(*[int(x) for x in layer.get("stride", layer["pool"])])
        d.pad = (C.c_int32 * 4)(*[int(x) for x in layer.get("pad", (0, 0, 0, 0))])
        div = layer.get("divisor", "inside")
        if div not in ("window", "inside"):
            raise ValueError("avgpool divisor must be 'window' or 'inside'")
        d.avgpool_divisor = L.POOL_DIV_INSIDE if div == "inside" else L.POOL_DIV_WINDOW
    elif t == "relu":
        d.type = L.LAYER_RELU
    else:
        raise ValueError("layer type %r is outside the approx-star path of this engine" % (t,))
    return d


class Network:
    """Device copy of a layer list (``nnvb_net_create``)."""

    def __init__(self, ctx, layers, in_shape):
        self.ctx = ctx
        self.lib = ctx.lib
        self.layers = list(layers)
        self.in_shape = tuple(int(x) for x in in_shape)
        self.n_in = int(np.prod(self.in_shape))
        keep = []
        descs = (L.LayerDesc * max(len(layers), 1))()
        for i, layer in enumerate(layers):
            descs[i] = make_layer_desc(layer, keep)
        h = C.c_void_p()
        L.check(self.lib.nnvb_net_create(ctx.handle, descs, len(layers), *self.in_shape, C.byref(h)),
                "nnvb_net_create")
        self.handle = h
        shp = (C.c_int64 * 3)()
        L.check(self.lib.nnvb_net_out_shape(h, shp), "nnvb_net_out_shape")
        self.out_shape = tuple(shp)
        self.n_relu = sum(1 for l in layers if l["type"] == "relu")

    def evaluate(self, X):
        """Concrete forward pass of the columns of X [N_in x n] (or one vector); returns [N_out x n]."""
        X = _f64(X)
        one = X.ndim == 1
        X = X.reshape(int(np.prod(self.in_shape)), -1, order="F")
        Y = np.empty((int(np.prod(self.out_shape)), X.shape[1]), dtype=np.float64, order="F")
        L.check(self.lib.nnvb_net_evaluate(self.handle, X.shape[1], _dp(X), _dp(Y)), "nnvb_net_evaluate")
        return Y[:, 0] if one else Y

    def close(self):
        if getattr(self, "handle", None):
            self.lib.nnvb_net_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Batch:
    """A list of input sets pushed through a network together."""

    def __init__(self, net, queries=None, n_queries=None):
        self.net = net
        self.lib = net.lib
        n = len(queries) if queries is not None else int(n_queries)
        self.nq = n
        h = C.c_void_p()
        L.check(self.lib.nnvb_batch_create(net.handle, n, C.byref(h)), "nnvb_batch_create")
        self.handle = h
        if queries is not None:
            if n < 8 or not self._set_many(queries):
                for q, qu in enumerate(queries):
                    self.set_query(q, qu)

    def _set_many(self, queries):
        """All sets of a uniform list in one call across the ABI (``nnvb_batch_set_bounds_many`` /
        ``nnvb_batch_set_stars``); False when the list is not uniform (mixed forms, different predicate or
        constraint counts, shapes that do not fit): the per-set path then reports what is wrong."""
        n, N = len(queries), self.net.n_in
        try:
            if all("lb" in q for q in queries):
                LB, UB = np.empty((n, N)), np.empty((n, N))
                for k, q in enumerate(queries):
                    LB[k] = np.asarray(q["lb"], dtype=np.float64).ravel(order="F")
                    UB[k] = np.asarray(q["ub"], dtype=np.float64).ravel(order="F")
                L.check(self.lib.nnvb_batch_set_bounds_many(self.handle, 0, n, _dp(LB), _dp(UB), N),
                        "nnvb_batch_set_bounds_many")
                return True
            if any("lb" in q for q in queries):
                return False
            V0 = np.asarray(queries[0]["V"])
            if V0.size % N:
                return False
            P = V0.size // N - 1
            C0 = queries[0].get("C")
            m = 0 if C0 is None or np.size(C0) == 0 else int(np.atleast_2d(C0).shape[0])
            Vs, PL, PU = np.empty((n, N * (P + 1))), np.empty((n, P)), np.empty((n, P))
            Cs, Ds = np.empty((n, m * P)), np.empty((n, m))
            for k, q in enumerate(queries):
                Vk = np.asarray(q["V"], dtype=np.float64)
                Ck = q.get("C")
                mk = 0 if Ck is None or np.size(Ck) == 0 else int(np.atleast_2d(Ck).shape[0])
                if Vk.size != N * (P + 1) or mk != m or np.size(q["pl"]) != P or np.size(q["pu"]) != P:
                    return False
                Vs[k] = Vk.ravel(order="F")
                PL[k] = np.asarray(q["pl"], dtype=np.float64).ravel()
                PU[k] = np.asarray(q["pu"], dtype=np.float64).ravel()
                if m:
                    Ck = np.atleast_2d(np.asarray(Ck, dtype=np.float64))
                    if Ck.shape[1] != P or np.size(q["d"]) != m:
                        return False
                    Cs[k] = Ck.ravel(order="F")
                    Ds[k] = np.asarray(q["d"], dtype=np.float64).ravel()
            L.check(self.lib.nnvb_batch_set_stars(self.handle, 0, n, P, m, _dp(Vs), _dp(PL) if P else None,
                                                  _dp(PU) if P else None, _dp(Cs) if m else None, _dp(Ds) if m else None),
                    "nnvb_batch_set_stars")
            return True
        except (ValueError, TypeError, KeyError):
            return False

    def close(self):
        if getattr(self, "handle", None):
            self.lib.nnvb_batch_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # inputs -------------------------------------------------------------------
    def set_bounds(self, q, lb, ub):
        lb = _f64(lb).ravel(order="F")
        ub = _f64(ub).ravel(order="F")
        n = self.net.n_in
        if lb.size != n or ub.size != n:
            raise ValueError("Inconsistency between lower bound image and upper bound image")
        L.check(self.lib.nnvb_batch_set_bounds(self.handle, q, _dp(lb), _dp(ub)), "nnvb_batch_set_bounds")

    def set_star(self, q, V, pl, pu, Cm=None, d=None):
        V = _f64(V)
        n = self.net.n_in
        M = V.reshape(n, -1, order="F")
        P = M.shape[1] - 1
        pl = _f64(pl).ravel()
        pu = _f64(pu).ravel()
        if pl.size != P or pu.size != P:
            raise ValueError("Inconsistency between number of predicate variables and predicate bounds")
        if Cm is None or np.size(Cm) == 0:
            m, Cm, d = 0, None, None
        else:
            Cm = _f64(np.atleast_2d(Cm))
            d = _f64(d).ravel()
            m = Cm.shape[0]
            if Cm.shape[1] != P or d.size != m:
                raise ValueError("Inconsistency between basic matrix and constraint matrix")
        L.check(self.lib.nnvb_batch_set_star(self.handle, q, P, _dp(M), _dp(pl), _dp(pu), m, _dp(Cm), _dp(d)),
                "nnvb_batch_set_star")

    def set_query(self, q, query):
        if "lb" in query:
            self.set_bounds(q, query["lb"], query["ub"])
        else:
            self.set_star(q, query["V"], query["pl"], query["pu"], query.get("C"), query.get("d"))

    def upload(self):
        L.check(self.lib.nnvb_batch_upload(self.handle), "nnvb_batch_upload")

    def reach(self, keep_constraints=False, keep_layer_bounds=False):
        o = L.Opts()
        o.keep_constraints = int(bool(keep_constraints))
        o.keep_layer_bounds = int(bool(keep_layer_bounds))
        L.check(self.lib.nnvb_batch_reach(self.handle, C.byref(o)), "nnvb_batch_reach")

    # LP-tightened bounds --------------------------------------------------------
    def set_bounds_hook(self, fn):
        """``fn(batch, relu_layer)`` is called inside reach for every ReLU layer with neurons the estimated
        ranges call crossing (``None`` removes it); see ``lp_bounds_hook``."""
        if fn is None:
            self._hook = L.BOUNDS_FN(0)
        else:
            def tramp(user, handle, layer):
                try:
                    fn(self, int(layer))
                    return 0
                except Exception as exc:          # never let an exception cross the C boundary
                    import sys
                    print("nnv_b200 bounds hook failed: %r" % (exc,), file=sys.stderr)
                    self._hook_error = exc
                    return 1
            self._hook = L.BOUNDS_FN(tramp)
        L.check(self.lib.nnvb_batch_set_bounds_hook(self.handle, self._hook, None), "nnvb_batch_set_bounds_hook")

    def get_crossing_rows(self, q, relu_layer, k, P):
        G = np.empty((k, P), dtype=np.float64, order="F")
        c = np.empty(k)
        L.check(self.lib.nnvb_batch_get_crossing_rows(self.handle, q, relu_layer, _dp(G), _dp(c)),
                "nnvb_batch_get_crossing_rows")
        return G, c

    def get_constraints_before(self, q, relu_layer, P):
        m = C.c_int64()
        L.check(self.lib.nnvb_batch_get_constraints_before(self.handle, q, relu_layer, C.byref(m), None, None),
                "nnvb_batch_get_constraints_before")
        Cm = np.empty((m.value, P), dtype=np.float64, order="F")
        d = np.empty(m.value)
        L.check(self.lib.nnvb_batch_get_constraints_before(self.handle, q, relu_layer, C.byref(m), _dp(Cm), _dp(d)),
                "nnvb_batch_get_constraints_before")
        return Cm, d

    def tighten_crossing(self, q, relu_layer, xmin, xmax):
        xmin, xmax = _f64(xmin).ravel(), _f64(xmax).ravel()
        L.check(self.lib.nnvb_batch_tighten_crossing(self.handle, q, relu_layer, _dp(xmin), _dp(xmax)),
                "nnvb_batch_tighten_crossing")

    # results ------------------------------------------------------------------
    def out_dims(self, q):
        P = C.c_int64()
        m = C.c_int64()
        L.check(self.lib.nnvb_batch_out_dims(self.handle, q, C.byref(P), C.byref(m)), "nnvb_batch_out_dims")
        return P.value, m.value

    def get_V(self, q):
        P, _ = self.out_dims(q)
        h, w, c = self.net.out_shape
        V = np.empty((h, w, c, P + 1), dtype=np.float64, order="F")
        L.check(self.lib.nnvb_batch_get_V(self.handle, q, _dp(V)), "nnvb_batch_get_V")
        return V

    def get_pred_bounds(self, q):
        P, _ = self.out_dims(q)
        pl = np.empty(P)
        pu = np.empty(P)
        L.check(self.lib.nnvb_batch_get_pred_bounds(self.handle, q, _dp(pl), _dp(pu)), "nnvb_batch_get_pred_bounds")
        return pl, pu

    def get_ranges(self, q):
        n = int(np.prod(self.net.out_shape))
        lb = np.empty(n)
        ub = np.empty(n)
        L.check(self.lib.nnvb_batch_get_ranges(self.handle, q, _dp(lb), _dp(ub)), "nnvb_batch_get_ranges")
        return lb, ub

    def get_constraints(self, q):
        P, m = self.out_dims(q)
        Cm = np.empty((m, P), dtype=np.float64, order="F")
        d = np.empty(m)
        L.check(self.lib.nnvb_batch_get_constraints(self.handle, q, _dp(Cm), _dp(d)), "nnvb_batch_get_constraints")
        return Cm, d

    def relu_stats(self):
        out = []
        for i in range(self.net.n_relu):
            st = L.ReluStats()
            L.check(self.lib.nnvb_batch_relu_stats(self.handle, i, C.byref(st)), "nnvb_batch_relu_stats")
            out.append({"N": st.n_neurons, "n_cross": st.n_cross, "n_dead": st.n_dead, "cols_after": st.cols_after})
        return out

    def get_crossing(self, q, relu_layer):
        k = C.c_int64()
        L.check(self.lib.nnvb_batch_get_crossing(self.handle, q, relu_layer, C.byref(k), None, None, None),
                "nnvb_batch_get_crossing")
        idx = np.empty(k.value, dtype=np.int64)
        lb = np.empty(k.value)
        ub = np.empty(k.value)
        if k.value:
            L.check(self.lib.nnvb_batch_get_crossing(self.handle, q, relu_layer, C.byref(k),
                                                     idx.ctypes.data_as(L.c_int64_p), _dp(lb), _dp(ub)),
                    "nnvb_batch_get_crossing")
        return idx, lb, ub

    def get_layer_ranges(self, q, relu_layer, n):
        lb = np.empty(n)
        ub = np.empty(n)
        L.check(self.lib.nnvb_batch_get_layer_ranges(self.handle, q, relu_layer, _dp(lb), _dp(ub)),
                "nnvb_batch_get_layer_ranges")
        return lb, ub

    def halfspace_margins(self, q, G, g):
        G = _f64(np.atleast_2d(G))
        g = _f64(g).ravel()
        nh = G.shape[0]
        margin = np.empty(nh)
        status = (C.c_int * nh)()
        L.check(self.lib.nnvb_batch_halfspace_margins(self.handle, q, _dp(G), _dp(g), nh, _dp(margin), status),
                "nnvb_batch_halfspace_margins")
        return margin, np.array(status[:], dtype=np.int32)

    def halfspace_witness(self, q, G, g):
        """(alpha[P], x_out[N_out], G x_out - g) of the device's witness point for the row G x <= g."""
        G = _f64(G).ravel()
        P, _ = self.out_dims(q)
        alpha = np.empty(P)
        x = np.empty(G.size)
        val = C.c_double()
        L.check(self.lib.nnvb_batch_halfspace_witness(self.handle, q, _dp(G), float(g), _dp(alpha), _dp(x),
                                                      C.cast(C.byref(val), L.c_double_p)),
                "nnvb_batch_halfspace_witness")
        return alpha, x, val.value

    def verify_robust(self, targets, kind="max"):
        t = np.ascontiguousarray(np.asarray(targets, dtype=np.int32).ravel())
        if t.size != self.nq:
            raise ValueError("one target per query expected")
        nh = int(np.prod(self.net.out_shape)) - 1
        verdict = (C.c_int * self.nq)()
        status = (C.c_int * (self.nq * nh))()
        margin = np.empty((self.nq, nh))
        L.check(self.lib.nnvb_batch_verify_robust(self.handle, t.ctypes.data_as(L.c_int32_p),
                                                  0 if kind == "max" else 1, verdict, status, _dp(margin)),
                "nnvb_batch_verify_robust")
        return (np.array(verdict[:], dtype=np.int32), np.array(status[:], dtype=np.int32).reshape(self.nq, nh),
                margin)
