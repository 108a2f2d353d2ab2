"""The allocation-free entry point, rlxq_matmul_static_scratch, against rlxq_matmul.

Who needs it: a caller that cannot get device memory at the moment it needs a GEMV — a decode loop
running after the process froze its allocations, a host whose whole device budget belongs to another
allocator, code held to a "no cudaMalloc after start-up" rule.  rlxq_matmul asks such a caller for a
workspace it may not have; this entry point keeps the workspace in a fixed 2 MiB array inside the
library's device image instead.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.  The test calls the new entry point through the C ABI twice in a row (the second
call reuses the array with the first call's leftovers in it) and compares each result with what the
existing entry point gives for the same inputs.  Both run the same two kernels with the same plan,
so the results are expected to be identical; the assertion uses the tolerance of the other GEMV
tests (2e-5 of |x| |w_row|) and additionally reports exact equality.  Because a fault common to both
entry points would pass that comparison, each result is also held against the CPU oracle.
"""
import ctypes as C

import numpy as np
import pytest

import rlx_b200 as R
from rlx_b200._lib import lib
from oracle import oracle as O
from tests.helpers import assert_within_tolerance, bound, make_case

pytestmark = pytest.mark.gpu

CASES = [("q4_0", 1, 4096, 11008), ("q4_k", 2, 2048, 300), ("q8_0", 1, 1024, 77), ("q6_k", 2, 4096, 130)]


def _static(xd, wd, s, n, out_dtype):
    import torch
    m, k = xd.shape
    y = torch.empty((m, n), dtype=out_dtype, device=xd.device)
    dt = lambda t: 0 if t.dtype == torch.float32 else 1   # noqa: E731
    st = lib.rlxq_matmul_static_scratch(torch.cuda.current_stream().cuda_stream, s, xd.data_ptr(), dt(xd),
                                        wd.data_ptr(), y.data_ptr(), dt(y), m, k, n)
    assert st == 0, (st, lib.rlxq_last_error().decode())
    return y


@pytest.mark.parametrize("sch,m,k,n", CASES)
def test_static_scratch_matches_workspace_entry_point_twice_in_a_row(sch, m, k, n):
    import torch
    s = O.SCHEMES[sch]
    w, x1 = make_case(s, m, k, n, seed=700 + n)
    _, x2 = make_case(s, m, k, n, seed=800 + n)
    wd = torch.from_numpy(w).cuda()
    xs = [torch.from_numpy(x1).cuda(), torch.from_numpy(x2).cuda()]
    # two calls back to back on one stream, no synchronisation in between
    got = [_static(xd, wd, s, n, torch.float32) for xd in xs]
    torch.cuda.synchronize()
    R.set_option("gemv_kernel", 3)
    try:
        want = [R.matmul(xd, wd, s, n) for xd in xs]
    finally:
        R.set_option("gemv_kernel", 0)
    R.device_status()
    for g, wnt, x in zip(got, want, (x1, x2)):
        g, wnt = g.cpu().numpy(), wnt.cpu().numpy()
        err = np.abs(g.astype(np.float64) - wnt.astype(np.float64)) / bound(s, w, x, n)
        assert err.max() <= 2e-5, f"{sch}: static-scratch result differs from rlxq_matmul by {err.max():.2e}"
        assert np.array_equal(g, wnt), f"{sch}: same kernels, same plan: results should be identical"
        ref = O.matmul_bt_mt(x, w, m, k, n, s)
        assert_within_tolerance(g, ref, bound(s, w, x, n), tol=2e-5, what=f"static scratch vs oracle {sch}")


def test_static_scratch_timeouts_are_visible_to_device_status():
    """rlxq_device_status covers the error word this entry point uses, whichever it is: after a clean call it
    reports no error, and it can be called by a process that has made allocation-free calls only."""
    import torch
    s, m, k, n = O.Q4_0, 1, 2048, 64
    w, x = make_case(s, m, k, n, seed=5)
    y = _static(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), s, n, torch.float32)
    code = C.c_int(-1)
    assert lib.rlxq_device_status(C.byref(code)) == 0 and code.value == 0
    assert_within_tolerance(y.cpu().numpy(), O.matmul_bt_mt(x, w, m, k, n, s), bound(s, w, x, n), tol=2e-5)


def test_static_scratch_bf16_in_and_out():
    import torch
    s, m, k, n = O.Q4_K, 1, 4096, 512
    w, x = make_case(s, m, k, n, seed=31, x_bf16=True)
    wd = torch.from_numpy(w).cuda()
    xd = torch.from_numpy(x).cuda().to(torch.bfloat16)
    a = _static(xd, wd, s, n, torch.bfloat16)
    b = R.matmul(xd, wd, s, n, out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    assert torch.equal(a, b)


def test_static_scratch_rejects_what_it_cannot_hold():
    import torch
    z = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    p = z.data_ptr()
    # batch above 2 is not this entry point's job
    assert lib.rlxq_matmul_static_scratch(stream, O.Q4_0, p, 0, p, p, 0, 3, 256, 16) == -2
    # k not a multiple of 256
    assert lib.rlxq_matmul_static_scratch(stream, O.Q4_0, p, 0, p, p, 0, 1, 96, 16) == -2
    # a shape whose partial tiles would not fit the 2 MiB array: rejected before any pointer is touched
    assert lib.rlxq_matmul_static_scratch(stream, O.Q4_0, p, 0, p, p, 0, 2, 4096, 4_000_000) == -11
    assert b"scratch" in lib.rlxq_last_error()
    assert lib.rlxq_matmul_static_scratch(stream, 99, p, 0, p, p, 0, 1, 256, 16) == -1
    assert lib.rlxq_matmul_static_scratch(stream, O.Q4_0, None, 0, p, p, 0, 1, 256, 16) == -3
