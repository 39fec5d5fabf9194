"""Seeded synthetic workloads for the approx-star hot path.

Every workload is a *neutral description* shared by the CUDA engine, the CPU
oracle and the tests: a list of layer dicts (NumPy arrays with MATLAB index
semantics) plus a list of query dicts.  Nothing here touches the GPU.

Layer dicts (shapes follow the reference's parameter layouts,
code/nnv/engine/nn/layers/Conv2DLayer.m:84-144, FullyConnectedLayer.m:56-66,
BatchNormalizationLayer.m:72-77, AveragePooling2DLayer.m:109-131):

    {"type": "conv2d", "W": [kh,kw,Cin,Cout], "b": [Cout],
     "pad": (t,b,l,r), "stride": (sh,sw), "dilation": (dh,dw)}
    {"type": "fc", "W": [Out,In], "b": [Out]}          # In indexed h-fastest
    {"type": "bn", "mean","var","scale","offset": [C], "eps": float}
    {"type": "avgpool", "pool": (ph,pw), "stride": (sh,sw), "pad": (t,b,l,r),
     "divisor": "inside" | "window"}    # padded windows: entries inside the image (default) or ph*pw
    {"type": "relu"}

Query dicts describe one input set and its specification:

    {"lb": [H,W,C], "ub": [H,W,C]}                      # box -> ImageStar(lb,ub)
    {"V": [H,W,C,P+1], "C": [m,P], "d": [m], "pl": [P], "pu": [P]}
    plus "target" (0-based class) and "spec" ("max" or "min").

The five full-size workloads restate the benchmark configurations in seeded
NumPy; images are uniform random stand-ins for the datasets the reference's
examples use.  ``small=True`` variants keep the layer structure but shrink
the image so that CPU checks finish in seconds.
"""
from __future__ import annotations

import numpy as np

__all__ = ["make_config", "CONFIG_NAMES", "input_shape", "forward_concrete"]

CONFIG_NAMES = ("fc5", "cnn28", "cnn32", "bright28", "vgg224")


def _he(rng, shape, fan_in):
    return rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)


def _conv(rng, kh, kw, cin, cout, pad, stride=(1, 1)):
    return {
        "type": "conv2d",
        "W": np.asfortranarray(_he(rng, (kh, kw, cin, cout), kh * kw * cin)),
        "b": rng.standard_normal(cout) * 0.01,
        "pad": tuple(pad),
        "stride": tuple(stride),
        "dilation": (1, 1),
    }


def _fc(rng, nin, nout):
    return {
        "type": "fc",
        "W": np.asfortranarray(_he(rng, (nout, nin), nin)),
        "b": rng.standard_normal(nout) * 0.01,
    }


def _bn(rng, c):
    return {
        "type": "bn",
        "mean": np.zeros(c),
        "var": np.ones(c),
        "scale": rng.uniform(0.5, 1.5, c),
        "offset": rng.standard_normal(c) * 0.1,
        "eps": 1e-5,
    }


def _pool2():
    return {"type": "avgpool", "pool": (2, 2), "stride": (2, 2), "pad": (0, 0, 0, 0)}


RELU = {"type": "relu"}


def out_shape(layers, shape):
    """Propagate an (H, W, C) shape through the layer list."""
    h, w, c = shape
    for L in layers:
        t = L["type"]
        if t == "conv2d":
            kh, kw, cin, cout = L["W"].shape
            assert cin == c, (cin, c)
            pt, pb, pl, pr = L["pad"]
            sh, sw = L["stride"]
            dh, dw = L["dilation"]
            h = (h + pt + pb - (kh - 1) * dh - 1) // sh + 1
            w = (w + pl + pr - (kw - 1) * dw - 1) // sw + 1
            c = cout
        elif t == "avgpool":
            ph, pw = L["pool"]
            pt, pb, pl, pr = L["pad"]
            sh, sw = L["stride"]
            h = (h + pt + pb - ph) // sh + 1
            w = (w + pl + pr - pw) // sw + 1
        elif t == "fc":
            assert L["W"].shape[1] == h * w * c, (L["W"].shape, h, w, c)
            h, w, c = 1, 1, L["W"].shape[0]
    return h, w, c


def forward_concrete(layers, x):
    """Concrete forward pass of one image ``x[H,W,C]`` (evaluate semantics of
    the in-scope layers); used to pick the target class of a query."""
    x = np.asarray(x, dtype=np.float64)
    if x.ndim == 1:
        x = x.reshape(-1, 1, 1)
    for L in layers:
        t = L["type"]
        if t == "conv2d":
            W = L["W"]
            kh, kw, cin, cout = W.shape
            pt, pb, pl, pr = L["pad"]
            sh, sw = L["stride"]
            dh, dw = L["dilation"]
            xp = np.pad(x, ((pt, pb), (pl, pr), (0, 0)))
            ho = (xp.shape[0] - (kh - 1) * dh - 1) // sh + 1
            wo = (xp.shape[1] - (kw - 1) * dw - 1) // sw + 1
            y = np.zeros((ho, wo, cout))
            for i in range(kh):
                for j in range(kw):
                    patch = xp[i * dh: i * dh + (ho - 1) * sh + 1: sh,
                               j * dw: j * dw + (wo - 1) * sw + 1: sw, :]
                    y += patch @ W[i, j]
            x = y + L["b"].reshape(1, 1, -1)
        elif t == "fc":
            x = (L["W"] @ x.reshape(-1, order="F") + L["b"]).reshape(1, 1, -1)
        elif t == "bn":
            x = (x - L["mean"]) / np.sqrt(L["var"] + L["eps"]) * L["scale"] + L["offset"]
        elif t == "avgpool":
            ph, pw = L["pool"]
            pt, pb, pl, pr = L["pad"]
            sh, sw = L["stride"]
            xp = np.pad(x, ((pt, pb), (pl, pr), (0, 0)))
            ho = (xp.shape[0] - ph) // sh + 1
            wo = (xp.shape[1] - pw) // sw + 1
            y = np.zeros((ho, wo, x.shape[2]))
            for i in range(ph):
                for j in range(pw):
                    y += xp[i: i + (ho - 1) * sh + 1: sh, j: j + (wo - 1) * sw + 1: sw, :]
            if L.get("divisor", "inside") == "inside":
                h0, w0 = np.arange(ho) * sh - pt, np.arange(wo) * sw - pl
                nh = np.minimum(h0 + ph, x.shape[0]) - np.maximum(h0, 0)
                nw = np.minimum(w0 + pw, x.shape[1]) - np.maximum(w0, 0)
                x = y / np.maximum(np.outer(nh, nw), 1)[:, :, None]
            else:
                x = y / (ph * pw)
        elif t == "relu":
            x = np.maximum(x, 0.0)
        else:
            raise ValueError(t)
    return x.reshape(-1, order="F")


def input_shape(name, small=False):
    return {
        "fc5": (5, 1, 1),
        "cnn28": (12, 12, 1) if small else (28, 28, 1),
        "cnn32": (8, 8, 3) if small else (32, 32, 3),
        "bright28": (12, 12, 1) if small else (28, 28, 1),
        "vgg224": (32, 32, 3) if small else (224, 224, 3),
    }[name]


def _net_fc5(rng):
    layers = []
    nin = 5
    for _ in range(6):
        layers += [_fc(rng, nin, 50), RELU]
        nin = 50
    layers.append(_fc(rng, nin, 5))
    return layers


def _net_cnn28(rng, shape):
    layers = [_conv(rng, 3, 3, 1, 8, (1, 1, 1, 1)), RELU,
              _conv(rng, 3, 3, 8, 16, (0, 0, 0, 0), (2, 2)), RELU]
    h, w, c = out_shape(layers, shape)
    layers += [_fc(rng, h * w * c, 128), RELU, _fc(rng, 128, 10)]
    return layers


def _net_cnn32(rng, shape, widths=(32, 64), nfc=256):
    layers = []
    cin = shape[2]
    for cw in widths:
        for _ in range(2):
            layers += [_conv(rng, 3, 3, cin, cw, (1, 1, 1, 1)), _bn(rng, cw), RELU]
            cin = cw
        layers.append(_pool2())
    h, w, c = out_shape(layers, shape)
    layers += [_fc(rng, h * w * c, nfc), RELU, _fc(rng, nfc, 10)]
    return layers


def _net_vgg(rng, shape, small):
    plan = [(64, 2), (128, 2), (256, 3), (512, 3), (512, 3)]
    if small:
        plan = [(8, 2), (16, 2), (32, 3), (64, 3), (64, 3)]
    layers = []
    cin = shape[2]
    for cw, reps in plan:
        for _ in range(reps):
            layers += [_conv(rng, 3, 3, cin, cw, (1, 1, 1, 1)), RELU]
            cin = cw
        layers.append(_pool2())
    h, w, c = out_shape(layers, shape)
    nfc = 64 if small else 4096
    nout = 10 if small else 1000
    layers += [_fc(rng, h * w * c, nfc), RELU, _fc(rng, nfc, nfc), RELU, _fc(rng, nfc, nout)]
    return layers


def make_config(name, n_queries=None, small=False, eps=None):
    """Return ``{"name", "layers", "in_shape", "queries"}`` for one workload.

    name        one of CONFIG_NAMES
    n_queries   number of input sets (default: the benchmark's count)
    small       shrink the image / widths (structure kept) for CPU-sized checks
    eps         override the perturbation radius
    """
    shape = input_shape(name, small)
    if name == "fc5":
        rng = np.random.default_rng(0)
        layers = _net_fc5(rng)
        nq = 100 if n_queries is None else n_queries
        hw = 0.01 if eps is None else eps
        queries = []
        for _ in range(nq):
            x = rng.uniform(-1.0, 1.0, 5).reshape(5, 1, 1)
            queries.append({"lb": x - hw, "ub": x + hw, "target": 0, "spec": "min"})
    elif name in ("cnn28", "bright28"):
        rng = np.random.default_rng(1)
        layers = _net_cnn28(rng, shape)
        if name == "cnn28":
            nq = 256 if n_queries is None else n_queries
            e = 1.0 / 255 if eps is None else eps
            queries = []
            for _ in range(nq):
                x = rng.uniform(0.0, 1.0, shape)
                q = {"lb": np.maximum(x - e, 0.0), "ub": np.minimum(x + e, 1.0), "spec": "max"}
                q["target"] = int(np.argmax(forward_concrete(layers, x)))
                queries.append(q)
        else:
            rng = np.random.default_rng(4)
            nq = 16384 if n_queries is None else n_queries
            amax = 0.05 if eps is None else eps
            queries = []
            for _ in range(nq):
                x = rng.uniform(0.0, 1.0, shape)
                bright = rng.uniform(0.0, 1.0, shape) < 0.15
                x = np.where(bright, rng.uniform(0.8, 1.0, shape), x)
                dgen = np.where(x > 0.8, 1.0 - x, 0.0)
                V = np.asfortranarray(np.stack([x, dgen], axis=3))
                q = {"V": V, "C": np.array([[1.0], [-1.0]]), "d": np.array([amax, 0.0]),
                     "pl": np.array([0.0]), "pu": np.array([amax]), "spec": "max"}
                q["target"] = int(np.argmax(forward_concrete(layers, x)))
                queries.append(q)
    elif name == "cnn32":
        rng = np.random.default_rng(2)
        layers = _net_cnn32(rng, shape, widths=(8, 16) if small else (32, 64),
                            nfc=32 if small else 256)
        nq = 128 if n_queries is None else n_queries
        e = 2.0 / 255 if eps is None else eps
        queries = []
        for _ in range(nq):
            x = rng.uniform(0.0, 1.0, shape)
            q = {"lb": x - e, "ub": x + e, "spec": "max"}
            q["target"] = int(np.argmax(forward_concrete(layers, x)))
            queries.append(q)
    elif name == "vgg224":
        rng = np.random.default_rng(3)
        layers = _net_vgg(rng, shape, small)
        nq = 8 if n_queries is None else n_queries
        e = 2.0 / 255 if eps is None else eps
        npix = 16 if small else 64
        queries = []
        n = int(np.prod(shape))
        for _ in range(nq):
            x = rng.uniform(0.0, 1.0, shape)
            pick = rng.choice(n, size=npix, replace=False)
            lb = x.copy().reshape(-1, order="F")
            ub = lb.copy()
            lb[pick] -= e
            ub[pick] += e
            q = {"lb": lb.reshape(shape, order="F"), "ub": ub.reshape(shape, order="F"),
                 "spec": "max"}
            q["target"] = int(np.argmax(forward_concrete(layers, x)))
            queries.append(q)
    else:
        raise ValueError(name)
    return {"name": name, "small": small, "layers": layers, "in_shape": shape, "queries": queries}
