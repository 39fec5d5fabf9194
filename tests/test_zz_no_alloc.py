"""The allocation-free Star.estimateRanges entry point.

Hosts that own all device memory themselves (a MATLAB session whose gpuArray pool
holds the GPU, a service with a fixed arena) cannot let the library call
cudaMalloc; for them ``nnvb_estimate_ranges_noalloc`` works on caller-owned
device buffers plus a fixed 4 MiB scratch array inside the module.  This test
drives it through the C ABI on two calls in a row — the second smaller than the
first, so stale scratch contents would show — and checks each result against the
ordinary entry point ``nnvb_estimate_ranges`` and against the CPU oracle's
Star.estimateRanges with the tolerance the other range tests use; the free
device memory must be the same before and after the second call.  It is
collected last on purpose.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run_noalloc(lib, torch, M, pl, pu, pad_rows=0, check_free=False):
    n, p1 = M.shape
    ld = n + pad_rows
    Mp = np.full((p1, ld), np.nan)                                   # [P+1, ld] row-major == ld x (P+1) column-major
    Mp[:, :n] = M.T
    dV = torch.from_numpy(Mp).cuda()
    dpl = torch.from_numpy(np.ascontiguousarray(pl) if pl.size else np.zeros(1)).cuda()
    dpu = torch.from_numpy(np.ascontiguousarray(pu) if pu.size else np.zeros(1)).cuda()
    dlb = torch.empty(n, dtype=torch.float64, device="cuda")
    dub = torch.empty(n, dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    st = torch.cuda.current_stream().cuda_stream
    free0 = torch.cuda.mem_get_info()[0]
    s = lib.nnvb_estimate_ranges_noalloc(st, n, p1 - 1, dV.data_ptr(), ld, dpl.data_ptr(), dpu.data_ptr(),
                                         dlb.data_ptr(), dub.data_ptr())
    assert s == 0, lib.nnvb_last_error()
    torch.cuda.synchronize()
    if check_free:                                                   # the call itself took no device memory
        assert torch.cuda.mem_get_info()[0] == free0
    return dlb.cpu().numpy(), dub.cpu().numpy()


def test_noalloc_matches_regular_entry_point_twice(ctx):
    import torch
    from nnv_b200 import _lib
    lib = _lib.load()
    from oracle import nnv_oracle as O
    rng = np.random.default_rng(11)
    for k, (n, p) in enumerate([(6272, 785), (300, 41)]):            # two calls in a row, second one smaller
        M = rng.standard_normal((n, p + 1)) * (rng.uniform(size=(n, p + 1)) > 0.4)
        pl = -rng.uniform(0, 1, p)
        pu = rng.uniform(0, 1, p)
        ref_lb, ref_ub = ctx.estimate_ranges(M, pl, pu)              # existing entry point
        lb, ub = _run_noalloc(lib, torch, M, pl, pu, check_free=k == 1)
        scale = np.abs(M).sum(axis=1).max()
        assert np.abs(lb - ref_lb).max() / scale < 1e-12
        assert np.abs(ub - ref_ub).max() / scale < 1e-12
        olb, oub = O.estimate_ranges(M, pl, pu)                      # Star.m:1078-1106 on the CPU
        assert np.abs(lb - olb).max() / scale < 1e-12 and np.abs(ub - oub).max() / scale < 1e-12


def test_noalloc_padded_columns_and_no_predicates():
    """Columns longer than the set (ld > N; the padding holds NaN and must not be read into a result) and a
    set without predicates, whose bounds are its centre."""
    import torch
    from nnv_b200 import _lib
    from oracle import nnv_oracle as O
    lib = _lib.load()
    rng = np.random.default_rng(12)
    M = rng.standard_normal((1000, 58))
    pl, pu = -rng.uniform(0, 1, 57), rng.uniform(0, 1, 57)
    lb, ub = _run_noalloc(lib, torch, M, pl, pu, pad_rows=16)
    olb, oub = O.estimate_ranges(M, pl, pu)
    scale = np.abs(M).sum(axis=1).max()
    assert np.abs(lb - olb).max() / scale < 1e-12 and np.abs(ub - oub).max() / scale < 1e-12
    c = rng.standard_normal((77, 1))
    lb, ub = _run_noalloc(lib, torch, c, np.zeros(0), np.zeros(0), pad_rows=3)
    assert np.array_equal(lb, c[:, 0]) and np.array_equal(ub, c[:, 0])


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
