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


def test_strip_cap_of_the_fixed_scratch_and_no_allocation():
    """(8192, 4096): the ordinary plan would use more strips than strips * 2 * c floats fit the fixed 4 MiB array, so the
    entry point runs with fewer, longer strips (its only code of its own).  Compared with float64 sums taken by torch,
    since the strip plan differs from the workspace entry point's.  Free device memory is the same before and after
    the second call: nothing was allocated."""
    from renaissance_b200 import _lib
    lib = _lib.load()
    m, c = 8192, 4096
    assert lib.trb200_bnrelu_bwd_workspace_bytes(m, c) > 4 << 20         # the workspace entry point would need more
    dy, bits, x, gamma, mean, inv = _inputs(77, m, c)
    _static(lib, _lib.check, dy, bits, x, gamma, mean, inv)             # first call on the device: address look-up
    torch.cuda.synchronize()
    dconv = torch.empty_like(dy)
    dg = torch.empty(c, device="cuda")
    db = torch.empty(c, device="cuda")
    free_before = torch.cuda.mem_get_info()[0]
    _lib.check(lib.trb200_bnrelu_bwd_static(dy.data_ptr(), bits.data_ptr(), x.data_ptr(), gamma.data_ptr(),
                                            mean.data_ptr(), inv.data_ptr(), dconv.data_ptr(), dg.data_ptr(),
                                            db.data_ptr(), m, c, C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    idx = torch.arange(m * c, device="cuda")
    keep = ((bits[idx >> 3].to(torch.int32) >> (idx & 7).to(torch.int32)) & 1).reshape(m, c).double()
    dym = dy.double() * keep
    ref_db = dym.sum(dim=0)
    ref_dg = (dym * (x.double() - mean.double()) * inv.double()).sum(dim=0)
    assert float((dg.double() - ref_dg).abs().max() / ref_dg.abs().max()) < 1e-4
    assert float((db.double() - ref_db).abs().max() / ref_db.abs().max()) < 1e-4
    xhat = (x.double() - mean.double()) * inv.double()
    ref_dx = gamma.double() * inv.double() * (dym - ref_db / m - xhat * ref_dg / m)
    assert float((dconv.double() - ref_dx).norm() / ref_dx.norm()) < 2e-3


def test_same_plan_gives_the_same_bits():
    """Where the fixed scratch does not force a different strip plan the two entry points run the same kernels on the
    same plan: identical bits."""
    from renaissance_b200 import _lib, ops
    lib = _lib.load()
    for seed, (m, c) in enumerate([(50000, 64), (4096, 512)]):
        args = _inputs(60 + seed, m, c)
        got = _static(lib, _lib.check, *args)
        ref = ops.bnrelu_bwd(*args)
        torch.cuda.synchronize()
        assert torch.equal(got[1], ref[1]) and torch.equal(got[2], ref[2]) and torch.equal(got[0], ref[0])


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
    # the mask is required here (the workspace entry point takes NULL for a BN with no ReLU behind it)
    rc = lib.trb200_bnrelu_bwd_static(args[0].data_ptr(), None, args[2].data_ptr(), args[3].data_ptr(),
                                      args[4].data_ptr(), args[5].data_ptr(), None, args[3].data_ptr(),
                                      args[3].data_ptr(), 16, 8, None)
    assert rc == _lib.ERR_INVALID_ARGUMENT
