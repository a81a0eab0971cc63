"""The allocation-free BN+ReLU backward entry point (trb200_bnrelu_bwd_static).

It serves hosts that cannot allocate device memory when they call the operator, so its
scratch is a fixed array inside the library.  The test calls it through the C ABI, twice in
a row (the array keeps what the previous call left in it, and nothing is cleared in
between), and compares with the workspace-taking entry point on the same inputs.  The
file name sorts last so that a failure here cannot hide the other tests in a run that
stops at the first failure."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, m, c):
    g = torch.Generator(device="cuda").manual_seed(seed)
    dy = torch.randn((m, c), generator=g, device="cuda").half()
    x = (torch.randn((m, c), generator=g, device="cuda") * 1.3 + 0.2).half()
    bits = torch.randint(0, 256, (m * c // 8,), generator=g, device="cuda", dtype=torch.int32).to(torch.uint8)
    gamma = 1 + 0.2 * torch.randn(c, generator=g, device="cuda")
    mean = x.float().mean(dim=0)
    inv = 1.0 / torch.sqrt(x.float().var(dim=0, unbiased=False) + 1e-5)
    return dy, bits, x, gamma, mean, inv


def _static(lib, check, dy, bits, x, gamma, mean, inv):
    m, c = dy.shape
    dconv = torch.empty_like(dy)
    dg = torch.empty(c, device="cuda")
    db = torch.empty(c, device="cuda")
    check(lib.trb200_bnrelu_bwd_static(dy.data_ptr(), bits.data_ptr(), x.data_ptr(), gamma.data_ptr(),
                                       mean.data_ptr(), inv.data_ptr(), dconv.data_ptr(), dg.data_ptr(),
                                       db.data_ptr(), m, c, C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return dconv, dg, db


@pytest.mark.parametrize("shapes", [[(50000, 64), (3001, 256)], [(777, 4096), (4096, 512)]])
def test_two_calls_in_a_row_match_the_workspace_entry_point(shapes):
    from renaissance_b200 import _lib, ops
    lib = _lib.load()
    for i, (m, c) in enumerate(shapes):
        args = _inputs(40 + i, m, c)
        got = _static(lib, _lib.check, *args)
        ref = ops.bnrelu_bwd(*args)
        torch.cuda.synchronize()
        for a, b, tol in ((got[1], ref[1], 1e-4), (got[2], ref[2], 1e-4)):
            assert float((a - b).abs().max() / b.abs().max()) < tol      # channel sums: 1e-4 relative
        d = (got[0].float() - ref[0].float()).norm() / ref[0].float().norm()
        assert float(d) < 2e-3                                            # half dconv


def test_rejects_more_channels_than_the_fixed_scratch_covers():
    from renaissance_b200 import _lib
    lib = _lib.load()
    args = _inputs(3, 16, 8)
    big = 8192
    rc = lib.trb200_bnrelu_bwd_static(args[0].data_ptr(), args[1].data_ptr(), args[2].data_ptr(), args[3].data_ptr(),
                                      args[4].data_ptr(), args[5].data_ptr(), None, args[3].data_ptr(),
                                      args[3].data_ptr(), 16, big, None)
    assert rc == _lib.ERR_UNSUPPORTED
    assert b"4096" in lib.trb200_last_error()
