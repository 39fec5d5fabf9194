"""ctypes binding of libnnvb200.so (the C ABI declared in include/nnvb200.h).

The library is built in-tree by ``nnv_b200/csrc/Makefile`` (or
``__graft_entry__.build()``).  There is no CPU fallback: if the shared object
is missing, or no sm_100a device is present when a context is created, the
caller gets an exception.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnnvb200.so")

NNVB_OK = 0
NNVB_E_ARG = 1
NNVB_E_CUDA = 2
NNVB_E_CAPACITY = 3
NNVB_E_STATE = 4
NNVB_E_UNSUPPORTED = 5

LAYER_CONV2D, LAYER_FC, LAYER_BN, LAYER_AVGPOOL2D, LAYER_RELU = 1, 2, 3, 4, 5

POOL_DIV_WINDOW, POOL_DIV_INSIDE = 0, 1
NCCL_ID_BYTES = 128

PROF_FAMILIES = ("conv", "fc", "bn", "avgpool", "ranges", "relax", "verify", "onehot", "allreduce")

VERDICT_EMPTY = 1
VERDICT_NONEMPTY = 2
UNDECIDED = -1

c_double_p = C.c_void_p          # double*: callers pass array addresses
c_int_p = C.POINTER(C.c_int)
c_int32_p = C.POINTER(C.c_int32)
c_int64_p = C.POINTER(C.c_int64)


class LayerDesc(C.Structure):
    _fields_ = [
        ("type", C.c_int32),
        ("kh", C.c_int32), ("kw", C.c_int32), ("cin", C.c_int32), ("cout", C.c_int32),
        ("pad", C.c_int32 * 4),
        ("stride", C.c_int32 * 2),
        ("dilation", C.c_int32 * 2),
        ("pool", C.c_int32 * 2),
        ("W", c_double_p), ("b", c_double_p),
        ("bn_mean", c_double_p), ("bn_var", c_double_p), ("bn_scale", c_double_p), ("bn_offset", c_double_p),
        ("bn_eps", C.c_double),
        ("avgpool_divisor", C.c_int32), ("reserved", C.c_int32),
    ]


class Opts(C.Structure):
    _fields_ = [("keep_constraints", C.c_int32), ("keep_layer_bounds", C.c_int32), ("reserved", C.c_int32 * 6)]


class ReluStats(C.Structure):
    _fields_ = [("n_neurons", C.c_int64), ("n_cross", C.c_int64), ("n_dead", C.c_int64), ("cols_after", C.c_int64)]


# int (*nnvb_allreduce_fn)(void* user, double* dev_buf, int64_t count, void* stream)
ALLREDUCE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p)


# int (*nnvb_bounds_fn)(void* user, nnvb_batch* b, int relu_layer)
BOUNDS_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_int)


class NNVError(RuntimeError):
    """A non-zero status from the C ABI; ``status`` holds the nnvb_status code."""

    def __init__(self, status, where, text):
        super().__init__("%s: status %d (%s)" % (where, status, text))
        self.status = status


# every exported symbol with (restype, argtypes); the CPU tests check this list
# against the header and against the shared object
SIGNATURES = {
    "nnvb_init": (C.c_int, [C.c_int, C.c_size_t, C.POINTER(C.c_void_p)]),
    "nnvb_destroy": (C.c_int, [C.c_void_p]),
    "nnvb_last_error": (C.c_char_p, []),
    "nnvb_strerror": (C.c_char_p, [C.c_int]),
    "nnvb_abi_version": (C.c_int, []),
    "nnvb_stream": (C.c_void_p, [C.c_void_p]),
    "nnvb_launch_count": (C.c_int64, [C.c_void_p]),
    "nnvb_profile_enable": (C.c_int, [C.c_void_p, C.c_int]),
    "nnvb_profile_read": (C.c_int, [C.c_void_p, C.c_int, c_double_p, c_int64_p, c_double_p]),
    "nnvb_set_shard": (C.c_int, [C.c_void_p, C.c_int, C.c_int, ALLREDUCE_FN, C.c_void_p]),
    "nnvb_nccl_unique_id": (C.c_int, [C.c_void_p]),
    "nnvb_set_shard_nccl": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int]),
    "nnvb_net_create": (C.c_int, [C.c_void_p, C.POINTER(LayerDesc), C.c_int, C.c_int64, C.c_int64, C.c_int64,
                                  C.POINTER(C.c_void_p)]),
    "nnvb_net_destroy": (C.c_int, [C.c_void_p]),
    "nnvb_net_evaluate": (C.c_int, [C.c_void_p, C.c_int64, c_double_p, c_double_p]),
    "nnvb_net_out_shape": (C.c_int, [C.c_void_p, c_int64_p]),
    "nnvb_batch_create": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_void_p)]),
    "nnvb_batch_destroy": (C.c_int, [C.c_void_p]),
    "nnvb_batch_set_bounds": (C.c_int, [C.c_void_p, C.c_int, c_double_p, c_double_p]),
    "nnvb_batch_set_star": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, c_double_p, c_double_p, c_double_p,
                                      C.c_int64, c_double_p, c_double_p]),
    "nnvb_batch_set_bounds_many": (C.c_int, [C.c_void_p, C.c_int, C.c_int, c_double_p, c_double_p, C.c_int64]),
    "nnvb_batch_set_stars": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_int64, c_double_p, c_double_p,
                                       c_double_p, c_double_p, c_double_p]),
    "nnvb_batch_upload": (C.c_int, [C.c_void_p]),
    "nnvb_batch_reach": (C.c_int, [C.c_void_p, C.POINTER(Opts)]),
    "nnvb_batch_set_bounds_hook": (C.c_int, [C.c_void_p, BOUNDS_FN, C.c_void_p]),
    "nnvb_batch_get_crossing_rows": (C.c_int, [C.c_void_p, C.c_int, C.c_int, c_double_p, c_double_p]),
    "nnvb_batch_get_constraints_before": (C.c_int, [C.c_void_p, C.c_int, C.c_int, c_int64_p, c_double_p, c_double_p]),
    "nnvb_batch_tighten_crossing": (C.c_int, [C.c_void_p, C.c_int, C.c_int, c_double_p, c_double_p]),
    "nnvb_batch_out_dims": (C.c_int, [C.c_void_p, C.c_int, c_int64_p, c_int64_p]),
    "nnvb_batch_get_V": (C.c_int, [C.c_void_p, C.c_int, c_double_p]),
    "nnvb_batch_get_pred_bounds": (C.c_int, [C.c_void_p, C.c_int, c_double_p, c_double_p]),
    "nnvb_batch_get_ranges": (C.c_int, [C.c_void_p, C.c_int, c_double_p, c_double_p]),
    "nnvb_batch_get_constraints": (C.c_int, [C.c_void_p, C.c_int, c_double_p, c_double_p]),
    "nnvb_batch_relu_layers": (C.c_int, [C.c_void_p, c_int_p]),
    "nnvb_batch_relu_stats": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(ReluStats)]),
    "nnvb_batch_get_crossing": (C.c_int, [C.c_void_p, C.c_int, C.c_int, c_int64_p, c_int64_p, c_double_p,
                                          c_double_p]),
    "nnvb_batch_get_layer_ranges": (C.c_int, [C.c_void_p, C.c_int, C.c_int, c_double_p, c_double_p]),
    "nnvb_batch_halfspace_margins": (C.c_int, [C.c_void_p, C.c_int, c_double_p, c_double_p, C.c_int, c_double_p,
                                               c_int_p]),
    "nnvb_batch_halfspace_witness": (C.c_int, [C.c_void_p, C.c_int, c_double_p, C.c_double, c_double_p, c_double_p,
                                               c_double_p]),
    "nnvb_batch_verify_robust": (C.c_int, [C.c_void_p, c_int32_p, C.c_int, c_int_p, c_int_p, c_double_p]),
    "nnvb_layer_apply": (C.c_int, [C.c_void_p, C.POINTER(LayerDesc), C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                   c_double_p, c_double_p, c_int64_p]),
    "nnvb_estimate_ranges": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, c_double_p, c_double_p, c_double_p,
                                       c_double_p, c_double_p]),
    # device pointers travel as integers (c_void_p)
    "nnvb_estimate_ranges_noalloc": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p,
                                               C.c_void_p, C.c_void_p, C.c_void_p]),
}

_lib = None


def load():
    """Load the shared object once and attach the signatures."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libnnvb200.so is not built (expected at %s); run `make -C nnv_b200/csrc` or "
            "`python -c 'import __graft_entry__ as g; g.build()'`. There is no CPU fallback." % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status, where):
    if status != NNVB_OK:
        lib = load()
        detail = lib.nnvb_last_error().decode("utf-8", "replace")
        kind = lib.nnvb_strerror(status).decode()
        raise NNVError(status, where, "%s: %s" % (kind, detail))
