"""Whole Conv+BN+ReLU block backward through trb200_cbr_bwd, one stream and three."""
import numpy as np
import pytest
import torch

from conftest import golden, rel_l2, rel_max
from gpu_util import block_inputs, dev, host

pytestmark = pytest.mark.gpu


def _run(orc, ops, b, first_layer, streams):
    n, h, w, c = b["x"].shape
    k = b["w"].shape[0]
    g = ops.ConvGeometry(n, h, w, c, k)
    ref = orc.cbr_bwd_amp(b["dy"], b["w"], b["gamma"], b["saved_mean"], b["saved_inv_std"], b["mask_bits"],
                          b["x"], b["conv_out"], first_layer=first_layer)
    xd = dev(b["x"])
    x_before = xd.clone()
    st = ops.BlockStreams.create() if streams else None
    if st is not None:
        torch.cuda.synchronize()
    out = ops.cbr_amp_bwd(g, dev(b["dy"]), dev(b["w"]), dev(b["gamma"]), dev(b["saved_mean"]),
                          dev(b["saved_inv_std"]), dev(b["mask_bits"]), xd, dev(b["conv_out"]),
                          first_layer=first_layer, streams=st)
    ops.device_status()
    assert rel_max(host(out["dgamma"]), ref["dgamma"]) < 1e-4
    assert rel_max(host(out["dbeta"]), ref["dbeta"]) < 1e-4
    assert rel_l2(host(out["dconv"]).astype(np.float32), ref["dconv"].astype(np.float32)) < 2e-3
    assert rel_l2(host(out["dw"]).astype(np.float32), ref["dw"].astype(np.float32)) < 2e-3
    if first_layer:
        assert out["dx"] is None and torch.equal(xd, x_before)       # the input buffer is not written
    else:
        assert out["dx"].data_ptr() == xd.data_ptr()                 # dX in place over X
        assert rel_l2(host(out["dx"]).astype(np.float32), ref["dx"].astype(np.float32)) < 2e-3


@pytest.mark.parametrize("streams", [False, True])
@pytest.mark.parametrize("n,h,w,c,k,first", [(4, 8, 8, 16, 32, False), (2, 8, 8, 4, 16, True),
                                             (2, 14, 14, 64, 64, False), (3, 12, 12, 64, 128, False),
                                             (2, 16, 16, 4, 64, True)])
def test_block_backward_matches_oracle(orc, n, h, w, c, k, first, streams):
    from renaissance_b200 import ops
    b = block_inputs(orc, 17 + n + c, n, h, w, c, k)
    _run(orc, ops, b, first, streams)


@pytest.mark.parametrize("name", ["cbr_block_small", "cbr_block_first"])
def test_block_backward_matches_golden(orc, name):
    """Against PyTorch autograd of conv -> batch_norm(training) -> relu on the same
    half inputs (the unfused composition the reference's CBR test compares with)."""
    from renaissance_b200 import ops
    g = golden(name)
    n, h, w, c, k, first = (int(v) for v in g["params"])
    fwd = orc.cbr_fwd_amp(g["x"], g["w"], g["gamma"], g["beta"])
    bits = orc.mask_pack(g["mask"])
    geo = ops.ConvGeometry(n, h, w, c, k)
    out = ops.cbr_amp_bwd(geo, dev(g["dy"]), dev(g["w"]), dev(g["gamma"]), dev(fwd["saved_mean"]),
                          dev(fwd["saved_inv_std"]), dev(bits), dev(g["x"]), dev(fwd["conv_out"]),
                          first_layer=bool(first))
    ops.device_status()
    assert rel_max(host(out["dgamma"]), g["dgamma"]) < 2e-3
    assert rel_max(host(out["dbeta"]), g["dbeta"]) < 2e-3
    assert rel_l2(host(out["dw"]).astype(np.float32), g["dw"]) < 2e-2
    if not first:
        assert rel_l2(host(out["dx"]).astype(np.float32), g["dx"]) < 2e-2


def test_block_backward_with_fused_pool(orc):
    """trb200_cbr_bwd with pool_argmax: dy is the gradient of the pooled output."""
    from renaissance_b200 import ops
    b = block_inputs(orc, 31, 2, 12, 12, 64, 64)
    n, h, w, c = b["x"].shape
    g = ops.ConvGeometry(n, h, w, c, 64)
    relu = b["relu_out"]
    _, am = orc.maxpool2x2_fwd(relu)
    rng = np.random.default_rng(9)
    dyp = rng.standard_normal((n, h // 2, w // 2, 64)).astype(np.float16)
    dy_full = orc.maxpool2x2_bwd(dyp, am, relu.shape)
    ref = orc.cbr_bwd_amp(dy_full, b["w"], b["gamma"], b["saved_mean"], b["saved_inv_std"], b["mask_bits"], b["x"],
                          b["conv_out"])
    xd = dev(b["x"])
    out = ops.cbr_amp_bwd(g, dev(dyp), dev(b["w"]), dev(b["gamma"]), dev(b["saved_mean"]), dev(b["saved_inv_std"]),
                          dev(b["mask_bits"]), xd, dev(b["conv_out"]), pool_argmax=dev(am),
                          streams=ops.BlockStreams.create())
    ops.device_status()
    assert rel_max(host(out["dgamma"]), ref["dgamma"]) < 1e-4 and rel_max(host(out["dbeta"]), ref["dbeta"]) < 1e-4
    assert rel_l2(host(out["dw"]).astype(np.float32), ref["dw"].astype(np.float32)) < 2e-3
    assert rel_l2(host(out["dx"]).astype(np.float32), ref["dx"].astype(np.float32)) < 2e-3


def test_block_backward_inside_cuda_graph(orc):
    """The reference replays the op from a captured CUDA graph after one warm-up call
    outside capture (src/graph/captured_graph.cpp:241-329).  Same discipline here:
    warm-up, capture on the three streams, replay twice, compare with the eager result."""
    from renaissance_b200 import ops
    b = block_inputs(orc, 5, 2, 14, 14, 64, 64)
    n, h, w, c = b["x"].shape
    g = ops.ConvGeometry(n, h, w, c, 64)
    t = {k: dev(b[k]) for k in ("dy", "w", "gamma", "saved_mean", "saved_inv_std", "mask_bits", "conv_out")}
    x0 = dev(b["x"])
    x = x0.clone()
    st = ops.BlockStreams.create()
    scratch = torch.empty_like(t["dy"])
    dw = torch.empty_like(t["w"])
    ws = ops.Workspace()

    def call():
        return ops.cbr_amp_bwd(g, t["dy"], t["w"], t["gamma"], t["saved_mean"], t["saved_inv_std"], t["mask_bits"],
                               x, t["conv_out"], bn_scratch=scratch, dw=dw, streams=st, workspace=ws)

    torch.cuda.synchronize()
    with torch.cuda.stream(st.bn):
        eager = call()                                  # warm-up outside capture (sizes the workspace)
    torch.cuda.synchronize()
    eager_dx, eager_dw = eager["dx"].clone(), eager["dw"].clone()
    x.copy_(x0)
    graph = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.graph(graph, stream=st.bn):
        out = call()
    for _ in range(2):
        x.copy_(x0)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out["dx"], eager_dx) and torch.equal(out["dw"], eager_dw)
    ops.device_status()
