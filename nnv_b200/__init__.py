"""nnv_b200 — sm_100a engine for NNV's approx-star (estimated-bounds) reachability path.

``nnv_b200.nn`` mirrors the reference's host API (NN, ImageStar, Star, layers);
``nnv_b200.engine`` wraps the C ABI of libnnvb200.so; ``nnv_b200.configs`` holds
the seeded synthetic workloads.  Importing the package does not touch the GPU.
"""
from .configs import CONFIG_NAMES, make_config  # noqa: F401

__version__ = "0.1.0"
