"""The reference's cuDNN path, rebuilt for measurement only.

The reference runs its fused block through cuDNN-frontend graphs (src/backend/ops/dtensor/cbr_op.cpp):
conv_fprop + genstats (:430-718), conv_wgrad (:763-840), conv_dgrad (:842-917) and
MUL(dY, mask) -> batchnorm_backward (:1259-1353), each finalized the way
include/renaissance/backend/cudnn_utils.h:108-115 does it: heuristics mode B, then FALLBACK, engines
with the NONDETERMINISTIC note deselected, the heuristics' first plan built.  This module builds the same
graphs with the cudnn-frontend Python package on the same NHWC / KRSC buffers so that the kernel sweep can time
the library kernels the reference would run on this GPU beside this repository's kernels.

Library kernels: a baseline, not the product.  Nothing on the product path imports this file, and it is only
usable where the `cudnn` package and a GPU are present.
"""
from __future__ import annotations

import torch

_handle = None


def available() -> bool:
    try:
        import cudnn  # noqa: F401
        return torch.cuda.is_available()
    except Exception:
        return False


def _h():
    global _handle
    import cudnn
    if _handle is None:
        _handle = cudnn.create_handle()
    cudnn.set_stream(handle=_handle, stream=torch.cuda.current_stream().cuda_stream)
    return _handle


def _nhwc(n, c, h, w):
    return [n, c, h, w], [h * w * c, 1, w * c, c]


class _Graph:
    """A finalized graph with its device pointers; call it to enqueue one execution on the current stream."""

    def __init__(self, graph, pack, keep):
        self.graph, self.pack, self.keep = graph, pack, keep
        self.workspace = torch.empty(max(int(graph.get_workspace_size()), 16), dtype=torch.uint8, device="cuda")

    def __call__(self):
        self.graph.execute(self.pack, self.workspace, handle=_h())


def _io_type(t):
    import cudnn
    return cudnn.data_type.BFLOAT16 if t.dtype == torch.bfloat16 else cudnn.data_type.HALF


def _new_graph(io=None):
    import cudnn
    return cudnn.pygraph(io_data_type=io or cudnn.data_type.HALF, intermediate_data_type=cudnn.data_type.FLOAT,
                         compute_data_type=cudnn.data_type.FLOAT, handle=_h())


def _finalize(g):
    import cudnn
    g.validate()
    g.build_operation_graph()
    g.create_execution_plans([cudnn.heur_mode.B, cudnn.heur_mode.FALLBACK])
    g.deselect_numeric_notes([cudnn.numerical_note.NONDETERMINISTIC])
    g.check_support()
    g.build_plans(cudnn.build_plan_policy.HEURISTICS_CHOICE)


def _krsc(k, c, r):
    return [k, c, r, r], [r * r * c, 1, r * c, c]


def conv_fprop(x, w, y, genstats=None, pad=1, stride=1):
    """x [n,h,w,c], w [k,r,r,c], y [n,oh,ow,k] (half or bfloat16, contiguous).  genstats = (sum, sqsum) float [k]
    adds the statistics node the reference fuses behind the convolution."""
    import cudnn
    n, h, wd, c = x.shape
    k, r = w.shape[0], w.shape[1]
    io = _io_type(x)
    g = _new_graph(io)
    dx, sx = _nhwc(n, c, h, wd)
    X = g.tensor(name="X", dim=dx, stride=sx, data_type=io)
    dwt, swt = _krsc(k, c, r)
    W = g.tensor(name="W", dim=dwt, stride=swt, data_type=io)
    Y = g.conv_fprop(image=X, weight=W, padding=[pad, pad], stride=[stride, stride], dilation=[1, 1],
                     compute_data_type=cudnn.data_type.FLOAT)
    dy, sy = _nhwc(n, k, y.shape[1], y.shape[2])
    Y.set_output(True).set_dim(dy).set_stride(sy).set_data_type(io)
    pack = {X: x.data_ptr(), W: w.data_ptr(), Y: y.data_ptr()}
    if genstats is not None:
        S, Q = g.genstats(input=Y, compute_data_type=cudnn.data_type.FLOAT)
        for t, buf in ((S, genstats[0]), (Q, genstats[1])):
            t.set_output(True).set_dim([1, k, 1, 1]).set_stride([k, 1, k, k]).set_data_type(cudnn.data_type.FLOAT)
            pack[t] = buf.data_ptr()
    _finalize(g)
    return _Graph(g, pack, (x, w, y, genstats))


def conv_dgrad(dy, w, dx, pad=1, stride=1):
    import cudnn
    n, oh, ow, k = dy.shape
    c, r = w.shape[3], w.shape[1]
    io = _io_type(dy)
    g = _new_graph(io)
    ddy, sdy = _nhwc(n, k, oh, ow)
    DY = g.tensor(name="dY", dim=ddy, stride=sdy, data_type=io)
    dwt, swt = _krsc(k, c, r)
    W = g.tensor(name="W", dim=dwt, stride=swt, data_type=io)
    DX = g.conv_dgrad(loss=DY, filter=W, padding=[pad, pad], stride=[stride, stride], dilation=[1, 1],
                      compute_data_type=cudnn.data_type.FLOAT)
    ddx, sdx = _nhwc(n, c, dx.shape[1], dx.shape[2])
    DX.set_output(True).set_dim(ddx).set_stride(sdx).set_data_type(io)
    _finalize(g)
    return _Graph(g, {DY: dy.data_ptr(), W: w.data_ptr(), DX: dx.data_ptr()}, (dy, w, dx))


def conv_wgrad(x, dy, dw, pad=1, stride=1):
    import cudnn
    n, h, wd, c = x.shape
    k, r = dy.shape[3], dw.shape[1]
    io = _io_type(x)
    g = _new_graph(io)
    dx_, sx = _nhwc(n, c, h, wd)
    ddy, sdy = _nhwc(n, k, dy.shape[1], dy.shape[2])
    X = g.tensor(name="X", dim=dx_, stride=sx, data_type=io)
    DY = g.tensor(name="dY", dim=ddy, stride=sdy, data_type=io)
    DW = g.conv_wgrad(image=X, loss=DY, padding=[pad, pad], stride=[stride, stride], dilation=[1, 1],
                      compute_data_type=cudnn.data_type.FLOAT)
    dwt, swt = _krsc(k, c, r)
    DW.set_output(True).set_dim(dwt).set_stride(swt).set_data_type(io)
    _finalize(g)
    return _Graph(g, {X: x.data_ptr(), DY: dy.data_ptr(), DW: dw.data_ptr()}, (x, dy, dw))


def bnrelu_bwd(dy, mask_bits, x, scale, mean, inv_var, dx, dscale, dbias, nhw=None):
    """dy, x, dx [m, c] half, m = n*h*w rows; nhw = (n, h, w) gives the tensor's logical extents (default:
    (m, 1, 1)); mask_bits the bit-packed BOOLEAN ReLU mask; scale / mean / inv_var / dscale / dbias float [c]."""
    import cudnn
    m, c = dy.shape
    n, h, w = nhw if nhw is not None else (m, 1, 1)
    assert n * h * w == m
    g = _new_graph()
    d4, s4 = _nhwc(n, c, h, w)
    DY = g.tensor(name="dY", dim=d4, stride=s4, data_type=cudnn.data_type.HALF)
    MASK = g.tensor(name="mask", dim=d4, stride=s4, data_type=cudnn.data_type.BOOLEAN)
    X = g.tensor(name="X", dim=d4, stride=s4, data_type=cudnn.data_type.HALF)

    def param(name):
        return g.tensor(name=name, dim=[1, c, 1, 1], stride=[c, 1, c, c], data_type=cudnn.data_type.FLOAT)

    SC, MU, IV = param("scale"), param("saved_mean"), param("saved_inv_var")
    DYM = g.mul(a=DY, b=MASK, compute_data_type=cudnn.data_type.FLOAT)
    DYM.set_data_type(cudnn.data_type.HALF)
    DX, DS, DB = g.batchnorm_backward(grad=DYM, input=X, scale=SC, mean=MU, inv_variance=IV,
                                      compute_data_type=cudnn.data_type.FLOAT)
    DX.set_output(True).set_dim(d4).set_stride(s4).set_data_type(cudnn.data_type.HALF)
    for t in (DS, DB):
        t.set_output(True).set_dim([1, c, 1, 1]).set_stride([c, 1, c, c]).set_data_type(cudnn.data_type.FLOAT)
    _finalize(g)
    pack = {DY: dy.data_ptr(), MASK: mask_bits.data_ptr(), X: x.data_ptr(), SC: scale.data_ptr(), MU: mean.data_ptr(),
            IV: inv_var.data_ptr(), DX: dx.data_ptr(), DS: dscale.data_ptr(), DB: dbias.data_ptr()}
    return _Graph(g, pack, (dy, mask_bits, x, scale, mean, inv_var, dx, dscale, dbias))
