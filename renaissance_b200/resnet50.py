"""ResNet-50 training step composed from the library's entry points (BASELINE.json configuration 4: bottleneck
3-4-6-3, NHWC, bfloat16 or half tensors with float master weights, bucketed all-reduce overlapped with backward).

The reference names this network (its layer list is scripts/resnet50_conv.json, its block descriptors are in
src/graph/layer_descriptor_registry.cpp:1313-1580) but has no backend for it, so this driver is not a drop-in for
anything: it runs every operator the network needs, in the order and on the shapes the network uses them, through
the same C ABI as the VGG16-BN path.

    forward   conv (tcgen05 kernels; stride 2 through stepped tensor maps) -> batch statistics (the conv epilogue
              for stride-1 layers) -> BN apply (+ ReLU + mask)                               per conv + BN unit
              3x3 stride-2 max pool after the 7x7 stem, add + ReLU + mask at every residual join,
              global average pool, classifier (the skinny tcgen05 GEMM + bias pass), fused softmax cross-entropy
    backward  the same operators' gradients in reverse; the BN in front of a join and the shortcut BN take the
              BN backward without a mask
    exchange  float master weights, float gradients, momentum and the 16-bit working weights are four flat buffers
              laid out in the order in which backward completes the parameters (classifier, last block ... stem, then
              every BN vector); ~25 MB buckets are cast to float and all-reduced (NCCL) as soon as backward has passed
              them (ddp.GradientBuckets, the schedule of the VGG16-BN driver)
    update    non-finite check, SGD with momentum on the whole flat range in one sweep (the loss scale is removed
              there), loss-scale back-off

torch supplies device memory and the 16-bit copy of the weights in bfloat16; every convolution, BN, pooling, join,
classifier, loss and optimizer kernel is libtrb200's.
"""
from __future__ import annotations

import torch

from . import ops
from .ddp import GradientBuckets

# mid channels, output channels, stride of the first block of each stage; blocks per stage of ResNet-50
STAGES = [(64, 256, 1), (128, 512, 2), (256, 1024, 2), (512, 2048, 2)]
RESNET50_BLOCKS = (3, 4, 6, 3)


class ConvBN:
    """One convolution + batch norm.  Its tensors are views into the network's flat buffers (ResNet50._flatten)."""

    def __init__(self, cin, cout, k, stride, pad, gen, dtype, device):
        self.cin, self.cout, self.k, self.stride, self.pad, self.dtype = cin, cout, k, stride, pad, dtype
        fan_in = k * k * cin
        self.w32 = torch.randn((cout, k, k, cin), generator=gen, device=device) * (2.0 / fan_in) ** 0.5
        self.gamma = torch.ones(cout, device=device)
        self.beta = torch.zeros(cout, device=device)
        self.w = self.w32.to(dtype)
        self.dw16 = self.dgamma = self.dbeta = None
        self.net = None
        self.ctx = None

    def geometry(self, n, h, w):
        return ops.ConvGeometry(n, h, w, self.cin, self.cout, self.k, self.k, self.pad, self.stride, dtype=self.dtype)

    def forward(self, x, relu):
        n, h, w, _ = x.shape
        g = self.geometry(n, h, w)
        if self.cin % 64 == 0:
            # the batch statistics come out of the convolution kernel's epilogue (stride 1 and 2)
            y, st = ops.conv_fprop_bn_stats(g, x, self.w, self.gamma, self.beta)
        else:
            y = ops.conv_fprop(g, x, self.w)
            st = ops.bn_stats_finalize(y, self.gamma, self.beta)
        out, mask = ops.bn_apply(y, st["eq_scale"], st["eq_bias"], relu=relu)
        self.ctx = dict(g=g, x=x, y=y, st=st, mask=mask)
        return out

    def backward(self, dout, need_dx=True):
        """dout: gradient of this unit's output (after the ReLU when it has one).  Returns dx."""
        c = self.ctx
        net = self.net
        tev = None
        if net is not None and net.timing_bn is not None:
            tev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            tev[0].record()
        dconv, dgamma, dbeta = ops.bnrelu_bwd(dout, c["mask"], c["y"], self.gamma, c["st"]["saved_mean"],
                                              c["st"]["saved_inv_std"])
        if tev is not None:
            tev[1].record()
            net.timing_bn.append((tev, dout.numel(), c["mask"] is not None))
        self.dgamma.copy_(dgamma)
        self.dbeta.copy_(dbeta)
        ops.conv_wgrad(c["g"], dconv, c["x"], dw=self.dw16)
        dx = ops.conv_dgrad(c["g"], dconv, self.w) if need_dx else None
        self.ctx = None
        if net is not None:
            net.unit_done(self)
        return dx

    @property
    def grads(self):
        """float gradients with the loss scale removed (for tests; the step itself works on the flat buffers)"""
        inv = 1.0 / self.net.loss_scale_value()
        return dict(w=self.dw16.float() * inv, gamma=self.dgamma * inv, beta=self.dbeta * inv)


class Bottleneck:
    def __init__(self, cin, mid, cout, stride, gen, dtype, device):
        self.c1 = ConvBN(cin, mid, 1, 1, 0, gen, dtype, device)
        self.c2 = ConvBN(mid, mid, 3, stride, 1, gen, dtype, device)
        self.c3 = ConvBN(mid, cout, 1, 1, 0, gen, dtype, device)
        self.down = ConvBN(cin, cout, 1, stride, 0, gen, dtype, device) if (stride != 1 or cin != cout) else None

    def units(self):
        return [u for u in (self.c1, self.c2, self.c3, self.down) if u is not None]

    def backward_order(self):
        return [u for u in (self.c3, self.c2, self.c1, self.down) if u is not None]

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
    def __init__(self, classes=1000, dtype=torch.bfloat16, seed=0, device="cuda", blocks=RESNET50_BLOCKS,
                 loss_scale=1024.0, bucket_mb=25.0, group=None):
        """blocks: bottlenecks per stage; (3, 4, 6, 3) is ResNet-50.  Shallower variants exist for tests: at random
        initialisation every block multiplies the rounding differences between two 16-bit evaluations by about 1.3,
        so a comparison with a float reference is only tight for a few blocks."""
        gen = torch.Generator(device=device).manual_seed(seed)
        self.dtype, self.classes, self.device = dtype, classes, device
        self.stem = ConvBN(4, 64, 7, 2, 3, gen, dtype, device)          # 3 image channels + 1 zero channel
        self.blocks = []
        cin = 64
        for (mid, cout, stride), count in zip(STAGES, blocks):
            for i in range(count):
                self.blocks.append(Bottleneck(cin, mid, cout, stride if i == 0 else 1, gen, dtype, device))
                cin = cout
        fc_w32 = torch.randn((classes, cin), generator=gen, device=device) * (1.0 / cin) ** 0.5
        self.scaling = torch.tensor([float(loss_scale)], device=device)
        self.nan_flag = torch.zeros(1, dtype=torch.int32, device=device)
        self.label_smoothing = torch.zeros(1, device=device)
        self.timing_bn = None      # list of ((start, stop) events, elements, has mask) per BN backward when enabled
        self._flatten(fc_w32, bucket_mb, group)

    def units(self):
        return [self.stem] + [u for b in self.blocks for u in b.units()]

    def loss_scale_value(self):
        return float(self.scaling.item())

    # ---------------------------------------------------------------- flat parameter buffers
    def _flatten(self, fc_w32, bucket_mb, group):
        """Master weights, gradients, momentum and 16-bit weights as flat buffers in backward completion order:
        [classifier weight, conv weights of the last block ... first block, stem | every gamma, beta, classifier bias].
        The part before the bar has 16-bit gradients (the weight-gradient kernels write the network's type), the
        part after it float ones."""
        order = [u for b in reversed(self.blocks) for u in b.backward_order()] + [self.stem]
        sizes16 = [fc_w32.numel()] + [u.w32.numel() for u in order]
        half_numel = sum(sizes16)
        tail = sum(2 * u.cout for u in order) + self.classes
        total = half_numel + tail
        dev = self.device
        self.w32 = torch.empty(total, device=dev)
        self.g32 = torch.zeros(total, device=dev)
        self.m32 = torch.zeros(total, device=dev)
        self.w16 = torch.empty(half_numel, dtype=self.dtype, device=dev)
        self.g16 = torch.zeros(half_numel, dtype=self.dtype, device=dev)
        self.half_numel = half_numel
        off = 0

        def take(buf, n, shape):
            return buf[off:off + n].view(shape)

        n = fc_w32.numel()
        self.fc_w32 = take(self.w32, n, fc_w32.shape); self.fc_w32.copy_(fc_w32)
        self.fc_w = take(self.w16, n, fc_w32.shape)
        self.fc_dw16 = take(self.g16, n, fc_w32.shape)
        off += n
        self._end = {}
        self._end["fc"] = off
        for u in order:
            n = u.w32.numel()
            shape = u.w32.shape
            w = take(self.w32, n, shape); w.copy_(u.w32); u.w32 = w
            u.w = take(self.w16, n, shape)
            u.dw16 = take(self.g16, n, shape)
            off += n
            self._end[id(u)] = off
            u.net = self
        for u in order:
            for name in ("gamma", "beta"):
                p = take(self.w32, u.cout, (u.cout,)); p.copy_(getattr(u, name)); setattr(u, name, p)
                setattr(u, "d" + name, take(self.g32, u.cout, (u.cout,)))
                off += u.cout
        self.fc_b32 = take(self.w32, self.classes, (self.classes,)); self.fc_b32.zero_()
        self.fc_db = take(self.g32, self.classes, (self.classes,))
        off += self.classes
        assert off == total
        self.w16.copy_(self.w32[:half_numel])
        cast = None
        if self.dtype == torch.float16:
            cast = lambda src, dst, factor: ops.cast_f16_to_f32(src, dst, factor)
        self.buckets = GradientBuckets(self.g16, self.g32, half_numel, bucket_bytes=bucket_mb * 1024 * 1024, group=group,
                                       cast=cast, scale=lambda t, factor: ops.scale_f32(t, factor))

    def unit_done(self, u):
        self.buckets.mark_ready(self._end[id(u)])

    @property
    def fc_grads(self):
        inv = 1.0 / self.loss_scale_value()
        return dict(w=self.fc_dw16.float() * inv, b=self.fc_db * inv)

    # ---------------------------------------------------------------- one step
    def forward_backward(self, images, labels, label_smoothing=0.0):
        """images [n, h, w, 4] of the network's 16-bit type, labels int32 [n].  Leaves the gradients (times the loss
        scale; averaged over the ranks) in the flat float buffer; returns the mean loss as a 1-element tensor."""
        self.buckets.begin_step()
        if label_smoothing:
            self.label_smoothing.fill_(label_smoothing)
        x = self.stem.forward(images, True)
        stem_shape = tuple(x.shape)
        x, pool_argmax = ops.maxpool_fwd(x, 3, 2, 1)
        for b in self.blocks:
            x = b.forward(x)
        _, fh, fw, _ = x.shape
        feat = ops.avgpool_global_fwd(x)
        logits = ops.fc_amp_fwd(feat, self.fc_w, self.fc_b32)
        out = ops.softmax_ce_amp_fused(logits, labels, self.scaling, self.label_smoothing)
        dlogits = out["dlogits"]                               # d(mean loss) / d logits, times the loss scale
        dfeat, _, _ = ops.fc_amp_bwd(dlogits, self.fc_w, feat, dw=self.fc_dw16, db=self.fc_db)
        self.buckets.mark_ready(self._end["fc"])
        dx = ops.avgpool_global_bwd(dfeat, fh, fw)
        for b in reversed(self.blocks):
            dx = b.backward(dx)
        dx = ops.maxpool_bwd(dx, pool_argmax, stem_shape, 3, 2, 1)
        self.stem.backward(dx, need_dx=False)
        self.buckets.finish()
        return out["loss"]

    def sgd_step(self, lr=0.1, momentum=0.9, weight_decay=1e-4):
        """Non-finite guard, one momentum-SGD sweep over the flat range (the loss scale is removed there), the 16-bit
        working weights, loss-scale back-off (optimizer_op.cu:40-60, check_op.cu:15-52, grad_scaling_op.cu:15-22)."""
        ops.check_nonfinite(self.g32, self.nan_flag)
        half = self.dtype == torch.float16
        n16 = self.half_numel
        ops.sgd_momentum(self.w32[:n16], self.g32[:n16], self.m32[:n16], self.w16 if half else None, lr, weight_decay,
                         momentum, scaling=self.scaling, skip_flag=self.nan_flag)
        ops.sgd_momentum(self.w32[n16:], self.g32[n16:], self.m32[n16:], None, lr, 0.0, momentum, scaling=self.scaling,
                         skip_flag=self.nan_flag)
        if not half:
            self.w16.copy_(self.w32[:n16])
        ops.grad_scaling(self.nan_flag, self.scaling, clear_flag=True)

    def step(self, images, labels, lr=0.01):
        loss = self.forward_backward(images, labels)
        self.sgd_step(lr=lr)
        return loss

    def weights_checksum(self):
        return self.w32.double().sum()


def synthetic_batch(n, image=224, classes=1000, dtype=torch.bfloat16, seed=1, device="cuda"):
    """images ~ N(0, 1) in 3 channels + 1 zero channel, labels uniform."""
    gen = torch.Generator(device=device).manual_seed(seed)
    img = torch.randn((n, image, image, 4), generator=gen, device=device)
    img[..., 3] = 0
    labels = torch.randint(0, classes, (n,), generator=gen, device=device, dtype=torch.int32)
    return img.to(dtype).contiguous(), labels
