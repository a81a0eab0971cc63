"""BN+ReLU backward of the block on the GPU against the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import rel_l2, rel_max
from gpu_util import dev, host

pytestmark = pytest.mark.gpu


def _case(orc, seed, m, c, p_keep=0.5):
    rng = np.random.default_rng(seed)
    dy = rng.standard_normal((m, c)).astype(np.float16)
    x = (rng.standard_normal((m, c)) * 1.5 + 0.3).astype(np.float16)
    mask = (rng.random((m, c)) < p_keep).astype(np.int8)
    bits = orc.mask_pack(mask)
    gamma = (1.0 + 0.2 * rng.standard_normal(c)).astype(np.float32)
    xf = x.astype(np.float32)
    mean = xf.mean(axis=0).astype(np.float32)
    inv_std = (1.0 / np.sqrt(xf.var(axis=0) + 1e-5)).astype(np.float32)
    return dy, x, bits, gamma, mean, inv_std


@pytest.mark.parametrize("m,c", [(1, 8), (7, 8), (64, 64), (1000, 24), (4096, 64), (3001, 256),
                                 (515, 512), (130, 2048), (33, 4096)])
def test_matches_oracle(orc, m, c):
    from renaissance_b200 import ops
    dy, x, bits, gamma, mean, inv_std = _case(orc, 100 + c + m, m, c)
    ref_dx, ref_dg, ref_db = orc.bnrelu_bwd_amp(dy, bits, x, gamma, mean, inv_std)
    dconv, dg, db = ops.bnrelu_bwd(dev(dy), dev(bits), dev(x), dev(gamma), dev(mean), dev(inv_std))
    torch.cuda.synchronize()
    # fp32-accumulated channel reductions: 1e-4 relative
    assert rel_max(host(dg), ref_dg) < 1e-4
    assert rel_max(host(db), ref_db) < 1e-4
    # half dx: 2e-2 relative L2
    assert rel_l2(host(dconv).astype(np.float32), ref_dx.astype(np.float32)) < 2e-2
    assert rel_l2(host(dconv).astype(np.float32), ref_dx.astype(np.float32)) < 2e-3   # what it really reaches


def test_all_masked_and_none_masked(orc):
    from renaissance_b200 import ops
    for keep in (0.0, 1.0):
        dy, x, bits, gamma, mean, inv_std = _case(orc, 7, 257, 64, p_keep=keep)
        ref_dx, ref_dg, ref_db = orc.bnrelu_bwd_amp(dy, bits, x, gamma, mean, inv_std)
        dconv, dg, db = ops.bnrelu_bwd(dev(dy), dev(bits), dev(x), dev(gamma), dev(mean), dev(inv_std))
        if keep == 0.0:
            assert float(dg.abs().max()) == 0.0 and float(db.abs().max()) == 0.0
            assert float(dconv.abs().max()) == 0.0
        else:
            assert rel_max(host(dg), ref_dg) < 1e-4 and rel_max(host(db), ref_db) < 1e-4
            assert rel_l2(host(dconv).astype(np.float32), ref_dx.astype(np.float32)) < 2e-3


def test_sums_only_and_bitwise_reproducible(orc):
    from renaissance_b200 import ops
    dy, x, bits, gamma, mean, inv_std = _case(orc, 11, 20000, 128)
    args = [dev(a) for a in (dy, bits, x, gamma, mean, inv_std)]
    none, dg0, db0 = ops.bnrelu_bwd(*args, want_dconv=False)
    assert none is None
    d1, dg1, db1 = ops.bnrelu_bwd(*args)
    d2, dg2, db2 = ops.bnrelu_bwd(*args)
    assert torch.equal(dg0, dg1) and torch.equal(dg1, dg2) and torch.equal(db0, db2)
    assert torch.equal(d1, d2)


def test_full_size_properties():
    """BASELINE.json configuration 2 size (N=256, 56x56, C=64): properties that need no oracle.
    sum_rows(dconv) = 0 and sum_rows(dconv * xhat) = 0 per channel (the BN backward
    projects both out), and dbeta / dgamma against torch float64 sums."""
    from renaissance_b200 import ops
    m, c = 256 * 56 * 56, 64
    g = torch.Generator(device="cuda").manual_seed(3)
    dy = torch.randn((m, c), generator=g, device="cuda", dtype=torch.float32).half()
    x = (torch.randn((m, c), generator=g, device="cuda", dtype=torch.float32) * 1.2 + 0.1).half()
    bits = torch.randint(0, 256, (m * c // 8,), generator=g, device="cuda", dtype=torch.int32).to(torch.uint8)
    gamma = 1 + 0.2 * torch.randn(c, generator=g, device="cuda")
    mean = x.float().mean(dim=0)
    inv_std = 1.0 / torch.sqrt(x.float().var(dim=0, unbiased=False) + 1e-5)
    dconv, dg, db = ops.bnrelu_bwd(dy, bits, x, gamma, mean, inv_std)
    shifts = torch.arange(8, device="cuda", dtype=torch.uint8)
    mask = ((bits.view(-1, 1) >> shifts) & 1).view(m, c).double()
    dym = dy.double() * mask
    xhat = (x.double() - mean.double()) * inv_std.double()
    ref_db = dym.sum(dim=0)
    ref_dg = (dym * xhat).sum(dim=0)
    assert float((db.double() - ref_db).abs().max() / ref_db.abs().max()) < 1e-4
    assert float((dg.double() - ref_dg).abs().max() / ref_dg.abs().max()) < 1e-4
    ref = gamma.double() * inv_std.double() * (dym - ref_db / m - xhat * ref_dg / m)
    err = (dconv.double() - ref).norm() / ref.norm()
    assert float(err) < 2e-3
    # projections: small compared with the size of the terms they cancel
    scale = float(dym.abs().sum(dim=0).max())
    assert float(dconv.double().sum(dim=0).abs().max()) / scale < 1e-3


@pytest.mark.parametrize("m,c,dtype,with_mask", [
    (592 * 128 + 77, 64, torch.float16, True),       # the smallest tensor on the bulk-copy ring, 77 rows past the last item
    (80011, 256, torch.float16, True),
    (40003, 512, torch.float16, False),              # no ReLU behind the BN (mask absent)
    (592 * 128 + 5, 64, torch.bfloat16, True),
    (30001, 2048, torch.bfloat16, False),
])
def test_ring_kernels_with_ragged_tails(m, c, dtype, with_mask):
    """Tensors of four or more 1024-vector items per SM run on the bulk-copy ring kernels; rows past the last whole
    item are handled by one block with plain loads.  Against float64 sums taken by torch on the same GPU; two runs
    give the same bits."""
    from renaissance_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(m + c)
    dy = torch.randn((m, c), generator=g, device="cuda", dtype=torch.float32).to(dtype)
    x = (torch.randn((m, c), generator=g, device="cuda", dtype=torch.float32) * 1.2 + 0.1).to(dtype)
    bits = torch.randint(0, 256, (m * c // 8,), generator=g, device="cuda", dtype=torch.int32).to(torch.uint8)
    gamma = 1 + 0.2 * torch.randn(c, generator=g, device="cuda")
    mean = x.float().mean(dim=0)
    inv_std = 1.0 / torch.sqrt(x.float().var(dim=0, unbiased=False) + 1e-5)
    dconv, dg, db = ops.bnrelu_bwd(dy, bits if with_mask else None, x, gamma, mean, inv_std)
    dconv2, dg2, db2 = ops.bnrelu_bwd(dy, bits if with_mask else None, x, gamma, mean, inv_std)
    assert torch.equal(dconv, dconv2) and torch.equal(dg, dg2) and torch.equal(db, db2)
    if with_mask:
        shifts = torch.arange(8, device="cuda", dtype=torch.uint8)
        mask = ((bits.view(-1, 1) >> shifts) & 1).view(m, c).double()
    else:
        mask = 1.0
    dym = dy.double() * mask
    xhat = (x.double() - mean.double()) * inv_std.double()
    ref_db = dym.sum(dim=0)
    ref_dg = (dym * xhat).sum(dim=0)
    assert float((db.double() - ref_db).abs().max() / ref_db.abs().max()) < 1e-4
    assert float((dg.double() - ref_dg).abs().max() / ref_dg.abs().max()) < 1e-4
    ref = gamma.double() * inv_std.double() * (dym - ref_db / m - xhat * ref_dg / m)
    tol = 2e-3 if dtype == torch.float16 else 1e-2
    assert float((dconv.double() - ref).norm() / ref.norm()) < tol
    # the last rows (the ragged tail) on their own
    assert float((dconv[-100:].double() - ref[-100:]).norm() / ref[-100:].norm()) < tol


def test_ring_kernels_replay_from_a_cuda_graph():
    """The bulk-copy ring kernels enqueue only: after one eager call (which sets the kernels' shared-memory
    attribute) the same call is captured into a CUDA graph in thread-local mode and replayed; the replay's results
    equal the eager ones bit for bit."""
    from renaissance_b200 import ops
    m, c = 256 * 56 * 56, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    dy = torch.randn((m, c), generator=g, device="cuda", dtype=torch.float32).half()
    x = (torch.randn((m, c), generator=g, device="cuda", dtype=torch.float32) * 1.2 + 0.1).half()
    bits = torch.randint(0, 256, (m * c // 8,), generator=g, device="cuda", dtype=torch.int32).to(torch.uint8)
    gamma = 1 + 0.2 * torch.randn(c, generator=g, device="cuda")
    mean = x.float().mean(dim=0)
    inv_std = 1.0 / torch.sqrt(x.float().var(dim=0, unbiased=False) + 1e-5)
    ws = ops.Workspace(torch.device("cuda"))
    eager = ops.bnrelu_bwd(dy, bits, x, gamma, mean, inv_std, workspace=ws)
    torch.cuda.synchronize()
    out = torch.empty_like(dy)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
            replayed = ops.bnrelu_bwd(dy, bits, x, gamma, mean, inv_std, dconv=out, workspace=ws, stream=side)
    torch.cuda.current_stream().wait_stream(side)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(replayed[0], eager[0]) and torch.equal(replayed[1], eager[1]) and torch.equal(replayed[2], eager[2])
    ops.device_status()
