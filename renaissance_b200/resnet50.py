"""ResNet-50 training step composed from the library's entry points (BASELINE.json configuration 4: bottleneck
3-4-6-3, NHWC, bfloat16 or half tensors with float master weights).

The reference names this network (its layer list is scripts/resnet50_conv.json, its block descriptors are in
src/graph/layer_descriptor_registry.cpp:1313-1580) but has no backend for it, so this driver is not a drop-in for
anything: it exists to run every operator the network needs, in the order and on the shapes the network uses them,
through the same C ABI as the VGG16-BN path.  One stream, no fusion across operators beyond the statistics epilogue
of the stride-1 convolutions; it is a correctness composition, not a tuned step.

    forward   conv (tcgen05 kernels) -> batch statistics -> BN apply (+ ReLU + mask)      per conv + BN unit
              3x3 stride-2 max pool after the 7x7 stem, add + ReLU + mask at every residual join,
              global average pool, classifier GEMM (torch matmul on the 16-bit tensors), fused softmax cross-entropy
    backward  the same operators' gradients in reverse; the BN in front of a join and the shortcut BN take the
              BN backward without a mask
    update    SGD with momentum on the float master weights (torch element-wise ops), 16-bit copies refreshed

torch supplies device memory, the classifier's matmul and the optimizer arithmetic; every convolution, BN, pooling,
join and loss kernel is libtrb200's.
"""
from __future__ import annotations

import torch

from . import ops

# mid channels, output channels, stride of the first block of each stage; blocks per stage of ResNet-50
STAGES = [(64, 256, 1), (128, 512, 2), (256, 1024, 2), (512, 2048, 2)]
RESNET50_BLOCKS = (3, 4, 6, 3)


class ConvBN:
    """One convolution + batch norm: float master weights, a 16-bit working copy, gamma / beta in float."""

    def __init__(self, cin, cout, k, stride, pad, gen, dtype, device):
        self.cin, self.cout, self.k, self.stride, self.pad, self.dtype = cin, cout, k, stride, pad, dtype
        fan_in = k * k * cin
        self.w32 = torch.randn((cout, k, k, cin), generator=gen, device=device) * (2.0 / fan_in) ** 0.5
        self.gamma = torch.ones(cout, device=device)
        self.beta = torch.zeros(cout, device=device)
        self.w = self.w32.to(dtype)
        self.grads = {}

    def geometry(self, n, h, w):
        return ops.ConvGeometry(n, h, w, self.cin, self.cout, self.k, self.k, self.pad, self.stride, dtype=self.dtype)

    def forward(self, x, relu):
        n, h, w, _ = x.shape
        g = self.geometry(n, h, w)
        if self.stride == 1 and self.cin % 64 == 0:
            # the batch statistics come out of the convolution kernel's epilogue
            y, st = ops.conv_fprop_bn_stats(g, x, self.w, self.gamma, self.beta)
        else:
            # stride 2 and the stem go through a resampling / lowering pass: statistics by a pass of their own
            y = ops.conv_fprop(g, x, self.w)
            st = ops.bn_stats_finalize(y, self.gamma, self.beta)
        out, mask = ops.bn_apply(y, st["eq_scale"], st["eq_bias"], relu=relu)
        self.ctx = dict(g=g, x=x, y=y, st=st, mask=mask)
        return out

    def backward(self, dout, need_dx=True):
        """dout: gradient of this unit's output (after the ReLU when it has one).  Returns dx."""
        c = self.ctx
        dconv, dgamma, dbeta = ops.bnrelu_bwd(dout, c["mask"], c["y"], self.gamma, c["st"]["saved_mean"],
                                              c["st"]["saved_inv_std"])
        self.grads = dict(w=ops.conv_wgrad(c["g"], dconv, c["x"]), gamma=dgamma, beta=dbeta)
        dx = ops.conv_dgrad(c["g"], dconv, self.w) if need_dx else None
        self.ctx = None
        return dx


class Bottleneck:
    def __init__(self, cin, mid, cout, stride, gen, dtype, device):
        self.c1 = ConvBN(cin, mid, 1, 1, 0, gen, dtype, device)
        self.c2 = ConvBN(mid, mid, 3, stride, 1, gen, dtype, device)
        self.c3 = ConvBN(mid, cout, 1, 1, 0, gen, dtype, device)
        self.down = ConvBN(cin, cout, 1, stride, 0, gen, dtype, device) if (stride != 1 or cin != cout) else None

    def units(self):
        return [u for u in (self.c1, self.c2, self.c3, self.down) if u is not None]

    def forward(self, x):
        main = self.c3.forward(self.c2.forward(self.c1.forward(x, True), True), False)
        shortcut = x if self.down is None else self.down.forward(x, False)
        out, self.mask = ops.add_relu_mask(main, shortcut)
        return out

    def backward(self, dout):
        g = ops.relu_mask_bwd(dout, self.mask)                 # gradient of the sum, the same for both branches
        dx_main = self.c1.backward(self.c2.backward(self.c3.backward(g)))
        dx_short = g if self.down is None else self.down.backward(g)
        return ops.add16(dx_main, dx_short)


class ResNet50:
    def __init__(self, classes=1000, dtype=torch.bfloat16, seed=0, device="cuda", blocks=RESNET50_BLOCKS):
        """blocks: bottlenecks per stage; (3, 4, 6, 3) is ResNet-50.  Shallower variants exist for tests: at random
        initialisation every block multiplies the rounding differences between two 16-bit evaluations by about 1.3,
        so a comparison with a float reference is only tight for a few blocks."""
        gen = torch.Generator(device=device).manual_seed(seed)
        self.dtype, self.classes = dtype, classes
        self.stem = ConvBN(4, 64, 7, 2, 3, gen, dtype, device)          # 3 image channels + 1 zero channel
        self.blocks = []
        cin = 64
        for (mid, cout, stride), count in zip(STAGES, blocks):
            for i in range(count):
                self.blocks.append(Bottleneck(cin, mid, cout, stride if i == 0 else 1, gen, dtype, device))
                cin = cout
        self.fc_w32 = torch.randn((classes, cin), generator=gen, device=device) * (1.0 / cin) ** 0.5
        self.fc_b32 = torch.zeros(classes, device=device)
        self.fc_w = self.fc_w32.to(dtype)
        self.fc_grads = {}
        self.momentum = {}

    def units(self):
        return [self.stem] + [u for b in self.blocks for u in b.units()]

    # ---------------------------------------------------------------- one step
    def forward_backward(self, images, labels, loss_scale=1024.0, label_smoothing=0.0):
        """images [n, h, w, 4] of the network's 16-bit type, labels int32 [n].  Leaves the gradients (float, loss
        scale removed) in every unit's .grads and in .fc_grads; returns the mean loss as a 1-element tensor."""
        n = images.shape[0]
        dev = images.device
        x = self.stem.forward(images, True)
        stem_shape = tuple(x.shape)
        x, pool_argmax = ops.maxpool_fwd(x, 3, 2, 1)
        for b in self.blocks:
            x = b.forward(x)
        _, fh, fw, _ = x.shape
        feat = ops.avgpool_global_fwd(x)
        logits = (torch.matmul(feat, self.fc_w.t()).float() + self.fc_b32).to(self.dtype).contiguous()
        scale = torch.tensor([loss_scale], device=dev)
        ls = torch.tensor([label_smoothing], device=dev)
        out = ops.softmax_ce_amp_fused(logits, labels, scale, ls)
        dlogits = out["dlogits"]                               # d(mean loss) / d logits, times the loss scale
        inv = 1.0 / loss_scale
        self.fc_grads = dict(w=torch.matmul(dlogits.t().float(), feat.float()) * inv, b=dlogits.float().sum(dim=0) * inv)
        dfeat = torch.matmul(dlogits, self.fc_w).contiguous()
        dx = ops.avgpool_global_bwd(dfeat, fh, fw)
        for b in reversed(self.blocks):
            dx = b.backward(dx)
        dx = ops.maxpool_bwd(dx, pool_argmax, stem_shape, 3, 2, 1)
        self.stem.backward(dx, need_dx=False)
        for u in self.units():
            u.grads = {k: v.float() * inv for k, v in u.grads.items()}
        ops.device_status()
        return out["loss"]

    def allreduce_gradients(self, group=None):
        """Data parallelism: the mean over the ranks of every gradient, as one NCCL all-reduce of a flat float
        buffer (RANGE_MEAN_ALLREDUCE of the reference, allreduce_op.cpp:37-105; not bucketed or overlapped here).
        A single process is a no-op."""
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
            return
        tensors = [u.grads[k] for u in self.units() for k in ("w", "gamma", "beta")]
        tensors += [self.fc_grads["w"], self.fc_grads["b"]]
        flat = torch.cat([t.reshape(-1) for t in tensors])
        dist.all_reduce(flat, group=group)
        ops.scale_f32(flat, 1.0 / dist.get_world_size(group))
        off = 0
        for t in tensors:
            t.copy_(flat[off:off + t.numel()].view_as(t))
            off += t.numel()

    def sgd_step(self, lr=0.1, momentum=0.9, weight_decay=1e-4):
        def upd(key, p, g, decay):
            if decay:
                g = g + weight_decay * p
            m = self.momentum.get(key)
            m = g.clone() if m is None else m.mul_(momentum).add_(g)
            self.momentum[key] = m
            p.sub_(lr * m)

        for i, u in enumerate(self.units()):
            upd((i, "w"), u.w32, u.grads["w"], True)
            upd((i, "g"), u.gamma, u.grads["gamma"], False)
            upd((i, "b"), u.beta, u.grads["beta"], False)
            u.w = u.w32.to(self.dtype)
        upd("fcw", self.fc_w32, self.fc_grads["w"], True)
        upd("fcb", self.fc_b32, self.fc_grads["b"], False)
        self.fc_w = self.fc_w32.to(self.dtype)


def synthetic_batch(n, image=224, classes=1000, dtype=torch.bfloat16, seed=1, device="cuda"):
    """images ~ N(0, 1) in 3 channels + 1 zero channel, labels uniform."""
    gen = torch.Generator(device=device).manual_seed(seed)
    img = torch.randn((n, image, image, 4), generator=gen, device=device)
    img[..., 3] = 0
    labels = torch.randint(0, classes, (n,), generator=gen, device=device, dtype=torch.int32)
    return img.to(dtype).contiguous(), labels


def main():
    import argparse
    import json
    ap = argparse.ArgumentParser(description="ResNet-50 step timing (information only; the benchmark is bench.py)")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f16"])
    args = ap.parse_args()
    import os
    import torch.distributed as dist
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    if world > 1:                                               # launched by torchrun: one process per GPU
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl")
    net = ResNet50(dtype=dtype)                                 # same seed: the ranks start from the same weights
    img, lab = synthetic_batch(args.batch, dtype=dtype, seed=1 + rank)

    def step():
        loss = net.forward_backward(img, lab)
        net.allreduce_gradients()
        net.sgd_step(lr=0.01)
        return float(loss)

    losses = [step() for _ in range(2)]
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    a.record()
    losses += [step() for _ in range(args.steps)]
    b.record()
    torch.cuda.synchronize()
    ms = torch.tensor([a.elapsed_time(b) / args.steps], device="cuda")
    check = torch.stack([net.stem.w32.double().sum(), net.fc_w32.double().sum()])   # equal on every rank if in step
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        lo, hi = check.clone(), check.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        assert torch.equal(lo, hi), "the ranks' weights have diverged"
    if rank == 0:
        print(json.dumps({"model": "resnet50", "dtype": args.dtype, "n_gpus": world, "batch_per_gpu": args.batch,
                          "ms_per_step": round(float(ms), 2),
                          "images_per_sec": round(world * args.batch / float(ms) * 1e3, 1),
                          "losses_rank0": [round(v, 4) for v in losses],
                          "note": "untuned composition on one stream, same batch every step, all-reduce not overlapped"}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
