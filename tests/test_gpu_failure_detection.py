"""Failure detection without a GPU fault: every wait of the tcgen05 kernels is bounded, and a wait that runs out
returns a status the host reads.  The self-test entry point makes that happen on purpose (a barrier nothing arrives
on, a short limit) with the kernels' own wait routine."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_reports_a_status_and_leaves_the_context_usable(orc):
    import numpy as np
    from renaissance_b200 import _lib, ops
    ops.device_status()                                    # clean before
    out = ops.selftest_wait_timeout(limit_ns=1_000_000)    # 1 ms
    torch.cuda.synchronize()
    got0, ns0, got1, ns1 = (int(v) for v in out.cpu())
    assert got0 == 0 and got1 == 0                         # neither warp got the barrier
    assert 1_000_000 <= ns0 < 50_000_000                   # warp 0 gave up after its limit
    assert ns1 < 50_000_000                                # warp 1 (one-second limit) left on the abort flag, not after 1 s
    with pytest.raises(_lib.Trb200Error) as e:
        ops.device_status()
    assert e.value.code == _lib.ERR_DEVICE_TIMEOUT
    ops.device_status()                                    # the word is cleared by the read
    # the next tensor-core launch on the same context is clean
    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, 8, 8, 64)).astype(np.float16)
    w = (rng.standard_normal((64, 3, 3, 64)) * 0.05).astype(np.float16)
    g = ops.ConvGeometry(2, 8, 8, 64, 64)
    y = ops.conv_fprop(g, torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda())
    torch.cuda.synchronize()
    ops.device_status()
    ref = orc.conv_fwd(x.astype(np.float32), w.astype(np.float32))
    assert float(np.abs(y.cpu().numpy().astype(np.float32) - ref).max()) < 2e-2


def test_limit_outside_the_allowed_range_is_refused():
    from renaissance_b200 import _lib
    lib = _lib.load()
    out = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert lib.trb200_selftest_wait_timeout(10, out.data_ptr(), None) == _lib.ERR_INVALID_ARGUMENT
    assert lib.trb200_selftest_wait_timeout(10**10, out.data_ptr(), None) == _lib.ERR_INVALID_ARGUMENT
    assert lib.trb200_selftest_wait_timeout(10**6, None, None) == _lib.ERR_INVALID_ARGUMENT
