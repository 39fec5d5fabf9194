"""The allocation-free Star.estimateRanges entry point.

Hosts that own all device memory themselves (a MATLAB session whose gpuArray pool
holds the GPU, a service with a fixed arena) cannot let the library call
cudaMalloc; for them ``nnvb_estimate_ranges_noalloc`` works on caller-owned
device buffers plus a fixed 4 MiB scratch array inside the module.  This test
drives it through the C ABI on two calls in a row — the second smaller than the
first, so stale scratch contents would show — and checks each result against the
ordinary entry point ``nnvb_estimate_ranges`` with the tolerance the other
range tests use.  It is collected last on purpose.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run_noalloc(lib, torch, M, pl, pu):
    n, p1 = M.shape
    dV = torch.from_numpy(np.ascontiguousarray(M.T)).cuda()          # [P+1, N] row-major == N x (P+1) column-major
    dpl = torch.from_numpy(pl).cuda()
    dpu = torch.from_numpy(pu).cuda()
    dlb = torch.empty(n, dtype=torch.float64, device="cuda")
    dub = torch.empty(n, dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    st = torch.cuda.current_stream().cuda_stream
    s = lib.nnvb_estimate_ranges_noalloc(st, n, p1 - 1, dV.data_ptr(), n, dpl.data_ptr(), dpu.data_ptr(),
                                         dlb.data_ptr(), dub.data_ptr())
    assert s == 0, lib.nnvb_last_error()
    torch.cuda.synchronize()
    return dlb.cpu().numpy(), dub.cpu().numpy()


def test_noalloc_matches_regular_entry_point_twice(ctx):
    import torch
    from nnv_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(11)
    for n, p in [(6272, 785), (300, 41)]:                            # two calls in a row, second one smaller
        M = rng.standard_normal((n, p + 1)) * (rng.uniform(size=(n, p + 1)) > 0.4)
        pl = -rng.uniform(0, 1, p)
        pu = rng.uniform(0, 1, p)
        ref_lb, ref_ub = ctx.estimate_ranges(M, pl, pu)              # existing entry point
        lb, ub = _run_noalloc(lib, torch, M, pl, pu)
        scale = np.abs(M).sum(axis=1).max()
        assert np.abs(lb - ref_lb).max() / scale < 1e-12
        assert np.abs(ub - ref_ub).max() / scale < 1e-12


def test_noalloc_rejects_oversized_sets():
    import torch
    from nnv_b200 import _lib
    lib = _lib.load()
    n = 524288 // 2 + 1
    buf = torch.zeros(8, dtype=torch.float64, device="cuda")
    s = lib.nnvb_estimate_ranges_noalloc(None, n, 1, buf.data_ptr(), n, buf.data_ptr(), buf.data_ptr(),
                                         buf.data_ptr(), buf.data_ptr())
    assert s == _lib.NNVB_E_CAPACITY
    assert b"exceeds the fixed scratch" in lib.nnvb_last_error()
