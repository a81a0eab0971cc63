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


def _buckets_rank(rank, world, port, out_path):
    """One rank of the two-GPU bucket test: the VGG16-BN driver's layout in small (float-born head, half middle,
    float-born tail) through GradientBuckets with the library's cast and scale kernels and NCCL's own mean."""
    import datetime
    import os
    import torch.distributed as dist
    from renaissance_b200 import ops
    from renaissance_b200.ddp import GradientBuckets
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=60))
    try:
        head, half_n, tail = 3000 * 8, 2000 * 8, 40 * 8
        total = head + half_n + tail
        gen = torch.Generator().manual_seed(50 + rank)
        f32 = torch.randn(total, generator=gen)
        h16 = torch.randn(half_n, generator=gen).half()
        g32 = f32.cuda()
        gb = GradientBuckets(h16.cuda(), g32, head + half_n, bucket_bytes=4 * 1024 * 8, group=None,
                             cast=lambda src, dst, factor: ops.cast_f16_to_f32(src, dst, factor=factor),
                             scale=lambda t, factor: ops.scale_f32(t, factor), half_begin=head)
        assert gb.native_mean
        gb.begin_step()
        gb.mark_ready(head)
        n_head = len(gb.issued)
        gb.mark_ready(head + half_n)
        gb.finish()
        torch.cuda.synchronize()
        res = g32.cpu().numpy()
        np.save(out_path, np.concatenate([res, np.array([n_head], dtype=np.float32)]))
    finally:
        dist.destroy_process_group()


def test_gradient_buckets_mean_on_two_gpus(tmp_path):
    """GradientBuckets over NCCL on two GPUs (one process each, NVLS off): both ranks end with the same floats, the
    mean of the two ranks' gradients, with the half range passing through the cast kernel and the float-born ranges
    untouched before the collective."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import os
    import socket
    import subprocess
    import sys
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    outs = [str(tmp_path / f"rank{r}.npy") for r in range(2)]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ("import sys; sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r}); "
            "import test_gpu_allreduce_side as t; t._buckets_rank({rank}, 2, {port}, {out!r})")
    procs = [subprocess.Popen([sys.executable, "-c", code.format(root=root, tests=os.path.join(root, "tests"), rank=r,
                                                                  port=port, out=outs[r])], env=env)
             for r in range(2)]
    for p in procs:
        assert p.wait(timeout=180) == 0
    a, b = np.load(outs[0]), np.load(outs[1])
    assert np.array_equal(a, b)
    head, half_n, tail = 3000 * 8, 2000 * 8, 40 * 8
    assert a[-1] == 2.0                                   # two whole buckets lie inside the float-born head
    exp = np.zeros(head + half_n + tail, dtype=np.float64)
    for r in range(2):
        gen = torch.Generator().manual_seed(50 + r)
        f = torch.randn(head + half_n + tail, generator=gen).double().numpy()
        h = torch.randn(half_n, generator=gen).half().double().numpy()
        f[head:head + half_n] = h
        exp += f / 2
    assert np.max(np.abs(a[:-1] - exp)) < 1e-6
