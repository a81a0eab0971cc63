"""The two kernels either side of the gradient all-reduce: half -> float cast with the mean factor folded in
(RANGE_CAST_FP16_TO_FP32, cast_op.cu:18-37) and the in-place scale (tr_scale_fp32_kernel, infra_kernels.cu:82-96)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [1, 7, 8, 1001, 4096, 1 << 20, (1 << 22) + 3])
@pytest.mark.parametrize("factor", [1.0, 0.125, 1.0 / 3.0])
def test_cast_half_to_float_with_factor(n, factor):
    from renaissance_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(n)
    src = (torch.randn(n + 9, generator=g, device="cuda") * 100).half()
    src[0] = 65504.0
    dst = torch.full((n + 2,), -7.0, device="cuda")
    view = src[1:1 + n] if n % 2 else src[:n]            # odd sizes also get an address that is only 2-byte aligned
    ops.cast_f16_to_f32(view, dst[1:1 + n], factor=factor)
    torch.cuda.synchronize()
    expect = view.float() * np.float32(factor)           # one float multiply: bit-exact
    assert torch.equal(dst[1:1 + n], expect)
    assert float(dst[0]) == -7.0 and float(dst[-1]) == -7.0


@pytest.mark.parametrize("n", [1, 5, 4096, (1 << 21) + 1])
def test_scale_in_place(n):
    from renaissance_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(n)
    buf = torch.randn(n + 8, generator=g, device="cuda")
    ref = buf.clone()
    ops.scale_f32(buf[4:4 + n], 1.0 / 8.0)                # the range starts on a 16-byte boundary, as the entry point asks
    torch.cuda.synchronize()
    assert torch.equal(buf[4:4 + n], ref[4:4 + n] * np.float32(0.125))
    assert torch.equal(buf[:4], ref[:4]) and torch.equal(buf[4 + n:], ref[4 + n:])
    with pytest.raises(Exception):
        ops.scale_f32(buf[1:1 + n], 0.5)                  # a start that is not 16-byte aligned is refused, not mis-scaled
