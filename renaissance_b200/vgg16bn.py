"""VGG16-BN AMP training step: the caller of the hot path.

This is the host-side schedule of one data-parallel training step, the role the
reference's ``DeepLearningTask::run_train_epoch_gpu`` plays
(src/task/deep_learning_task.cpp:1162-1217), reduced to what the benchmark needs:

    H2D (side stream, double buffered)                      TransferStation
    forward : 13 x [conv with BN statistics in its epilogue -> bn_finalize -> BN apply + ReLU + mask
              (+ 2x2 max pool fused in for the 5 pooled blocks)],
              FC 25088-4096-4096-1000 with ReLU + dropout, softmax-CE
    backward: softmax-CE, FC, 13 x CBR_AMP_BWD (first layer without dgrad; max-pool backward fused into
              the BN stage of the pooled blocks)
    gradients: FC weights in float from their GEMM, conv weights half -> float per bucket (>= 50 MB, ending at
              tensor ends) in backward order, NCCL all-reduce
              per bucket overlapped with the rest of backward, non-finite check,
              SGD with momentum on float master weights + half working copy

Every kernel of the step runs in libtrb200.so: the named hot path (block backward,
softmax-CE), the convolution forward, BN forward, pooling, casts, the optimizer, and the
classifier (the three FC layers on the library's own tensor-core GEMMs with bias, ReLU and
dropout folded into one pass; the reference uses cublasGemmEx there,
src/backend/ops/dtensor/fc_op.cpp:259-480).  torch supplies device memory, streams and
torch.distributed only.

Gradients follow the reference's in-place rule: dX of a block overwrites the block's
input buffer (src/graph/compiler.cpp:1390-1396).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from . import ops
from .ddp import GradientBuckets

VGG16_CFG = [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"]


@dataclass
class ParamSlot:
    name: str
    shape: tuple
    offset: int          # element offset in the flat buffers
    numel: int
    half_grad: bool      # gradient produced in half (conv weights) or float (FC weights and biases, BN vectors)
    stored: int = 0      # elements the slot holds (>= numel: an FC matrix keeps zero rows up to a GEMM-friendly count)


@dataclass
class ConvLayer:
    idx: int
    h: int
    c: int
    k: int
    pool_after: bool
    w: ParamSlot = None
    gamma: ParamSlot = None
    beta: ParamSlot = None
    buf: dict = field(default_factory=dict)


def _align(n, a=64):
    return (n + a - 1) // a * a


def _fc_width(n):
    """Rows an FC weight matrix is stored with: the tensor-core GEMMs take 64, 128 or a multiple of 256."""
    return 64 if n <= 64 else (128 if n <= 128 else _align(n, 256))


class Vgg16BnTrainer:
    def __init__(self, batch=256, image=224, classes=1000, lr=0.01, momentum=0.9, weight_decay=5e-4,
                 loss_scale=1024.0, label_smoothing=0.0, bucket_mb=50.0, seed=0, device=None,
                 process_group=None, dropout=0.5, fc_width=4096, nccl_registered=None, bucket_plan="tensors"):
        self.dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.batch, self.image, self.classes = batch, image, classes
        self.lr, self.beta, self.wd = lr, momentum, weight_decay
        self.dropout = dropout
        self.seed = seed
        self.steps_done = 0
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if (dist.is_available() and dist.is_initialized()) else 1

        # ---- layers
        self.convs: list[ConvLayer] = []
        h, c = image, 4                       # 3 input channels padded to 4 (arch_plan_normalize.cpp:39)
        for i, v in enumerate(VGG16_CFG):
            if v == "M":
                self.convs[-1].pool_after = True
                h //= 2
            else:
                self.convs.append(ConvLayer(len(self.convs), h, c, v, False))
                c = v
        self.feat_hw = h
        self.fc_dims = [(h * h * c, fc_width), (fc_width, fc_width), (fc_width, classes)]

        # ---- flat parameter space in BACKWARD completion order: fc3, fc2, fc1, conv13 .. conv1, then all BN vectors
        slots, off = [], 0

        def add(name, shape, half_grad, rows_stored=None):
            """`rows_stored` > shape[0]: the slot holds that many rows (the extra ones stay zero)."""
            nonlocal off
            n = int(math.prod(shape))
            stored = n if rows_stored is None else n // shape[0] * rows_stored
            s = ParamSlot(name, tuple(shape), off, n, half_grad, stored)
            off += _align(stored)
            slots.append(s)
            return s

        # an FC layer's weight is stored with a row count the tensor-core GEMMs take (1000 classes -> 1024 rows,
        # the extra rows zero); its gradient is written in float, as the reference's FC_AMP_BWD does
        # (fc_op.cpp:434-446: cublasGemmEx with a CUDA_R_32F output), so no cast pass follows it; its bias and bias
        # gradient are float too (fc_op.cpp:281-347) and sit with the BN vectors
        self.classes_pad = _fc_width(classes)
        self.fc = []
        for j in reversed(range(3)):
            i_f, o_f = self.fc_dims[j]
            self.fc.insert(0, dict(w=add(f"fc{j}.w", (o_f, i_f), False, rows_stored=_fc_width(o_f)), out_pad=_fc_width(o_f)))
        self.half_begin = off                 # the half gradients (conv weights) start here
        for L in reversed(self.convs):
            L.w = add(f"conv{L.idx}.w", (L.k, 3, 3, L.c), True)
        self.half_numel = off                 # ... and end here
        for L in reversed(self.convs):
            L.gamma = add(f"bn{L.idx}.gamma", (L.k,), False)
            L.beta = add(f"bn{L.idx}.beta", (L.k,), False)
        for j, f in enumerate(self.fc):
            f["b"] = add(f"fc{j}.b", (self.fc_dims[j][1],), False, rows_stored=f["out_pad"])
        self.total = off
        self.slots = slots

        d = self.dev
        self.w32 = torch.zeros(self.total, dtype=torch.float32, device=d)
        self.g32 = self._alloc_gradients(nccl_registered, process_group)
        self.m32 = torch.zeros(self.total, dtype=torch.float32, device=d)
        self.w16 = torch.zeros(self.total, dtype=torch.float16, device=d)
        self.g16 = torch.zeros(self.half_numel - self.half_begin, dtype=torch.float16, device=d)
        self._init_params(seed)

        # ---- buckets over the flat float gradient buffer, all-reduced as backward passes them
        self.buckets = GradientBuckets(
            self.g16, self.g32, self.half_numel, bucket_bytes=bucket_mb * 1024 * 1024, group=process_group,
            cast=lambda src, dst, factor: ops.cast_f16_to_f32(src, dst, factor=factor),
            scale=lambda t, factor: ops.scale_f32(t, factor), half_begin=self.half_begin,
            # "tensors": a bucket ends only where a weight gradient ends (each is ready in one piece), as soon as it
            # holds bucket_mb; "uniform": equal buckets of bucket_mb
            cuts=[s_.offset + _align(s_.stored) for s_ in slots if s_.offset < self.half_numel]
            if bucket_plan == "tensors" else None)

        # ---- scalars that the reference keeps as DTensors
        self.scaling = torch.tensor([loss_scale], dtype=torch.float32, device=d)
        self.label_smoothing = torch.tensor([label_smoothing], dtype=torch.float32, device=d)
        self.nan_flag = torch.zeros(1, dtype=torch.int32, device=d)

        # ---- activations
        n = batch
        for L in self.convs:
            e = (n, L.h, L.h, L.k)
            L.buf["conv_out"] = torch.empty(e, dtype=torch.float16, device=d)
            if not self._pool_after(L):
                L.buf["relu_out"] = torch.empty(e, dtype=torch.float16, device=d)
            L.buf["mask"] = torch.empty(n * L.h * L.h * L.k // 8, dtype=torch.uint8, device=d)
            for nm in ("saved_mean", "saved_inv_std", "eq_scale", "eq_bias"):
                L.buf[nm] = torch.empty(L.k, dtype=torch.float32, device=d)
            L.buf["running_mean"] = torch.zeros(L.k, dtype=torch.float32, device=d)
            L.buf["running_var"] = torch.ones(L.k, dtype=torch.float32, device=d)
            if L.pool_after:
                pe = (n, L.h // 2, L.h // 2, L.k)
                L.buf["pool_out"] = torch.empty(pe, dtype=torch.float16, device=d)
                L.buf["argmax"] = torch.empty(pe, dtype=torch.uint8, device=d)
        big = max(L.buf["conv_out"].numel() for L in self.convs)
        # the blocks' bn_output scratch
        self.bn_scratch = torch.empty(big, dtype=torch.float16, device=d)
        self.images = [torch.zeros((n, image, image, 4), dtype=torch.float16, device=d) for _ in range(2)]
        self.labels = [torch.zeros(n, dtype=torch.int32, device=d) for _ in range(2)]
        # logits and their gradient live in rows of classes_pad elements (the row stride the softmax kernels take);
        # the padding columns of d_logits stay zero, so the padded rows of the last layer's dW are zero too
        self.logits_rows = torch.zeros((n, self.classes_pad), dtype=torch.float16, device=d)
        self.dlogits_rows = torch.zeros((n, self.classes_pad), dtype=torch.float16, device=d)
        self.logits = self.logits_rows[:, :classes]
        self.dlogits = self.dlogits_rows[:, :classes]
        self.fc_out = [torch.empty((n, self.fc[j]["out_pad"]), dtype=torch.float16, device=d) for j in range(2)]
        self.fc_dx = [torch.empty((n, self.fc_dims[j][0]), dtype=torch.float16, device=d) for j in range(3)]
        self.loss_partial = torch.empty(n, dtype=torch.float32, device=d)
        self.loss = torch.zeros(1, dtype=torch.float32, device=d)
        self.inv_scaling = torch.zeros(1, dtype=torch.float32, device=d)
        self.ws = ops.Workspace(d)
        self.copy_stream = torch.cuda.Stream(device=d)
        self.copy_done = [torch.cuda.Event(), torch.cuda.Event()]
        self.slot_free = [torch.cuda.Event(), torch.cuda.Event()]
        self.timing = None        # list of (start event, stop event, flop, bytes) per forward conv launch when enabled
        self.timing_bwd = None    # list of (layer, [start, after BN, after wgrad, after dgrad] events) per block backward
        self.debug_hook = None    # called as hook(layer, dy, x) before every block backward (tests)

    @staticmethod
    def _pool_after(L):
        return L.pool_after

    # ------------------------------------------------------------------ parameters
    def view(self, buf, slot: ParamSlot):
        return buf[slot.offset:slot.offset + slot.numel].view(slot.shape)

    def _alloc_gradients(self, mode, group):
        """The flat float gradient buffer.  `mode` "user" / "symm": from NCCL's own allocator and registered with the
        communicator (a user buffer / a symmetric window), which lets NCCL's NVLink-SHARP and peer paths read and
        write it in place; None: an ordinary allocation."""
        if mode in ("user", "symm") and self.world > 1 and dist.get_backend(group) == "nccl":
            backend = (group or dist.group.WORLD)._get_backend(self.dev)
            self._nccl_pool = torch.cuda.MemPool(backend.mem_allocator)
            with torch.cuda.use_mem_pool(self._nccl_pool):
                g32 = torch.zeros(self.total, dtype=torch.float32, device=self.dev)
            backend.register_mem_pool(self._nccl_pool, mode == "symm")
            return g32
        return torch.zeros(self.total, dtype=torch.float32, device=self.dev)

    def half_grad(self, slot: ParamSlot):
        """A conv weight's gradient in the half buffer (whose element 0 is flat element half_begin)."""
        o = slot.offset - self.half_begin
        return self.g16[o:o + slot.numel].view(slot.shape)

    def stored(self, buf, slot: ParamSlot):
        """The slot with the rows it is stored with (an FC matrix padded to a GEMM-friendly row count)."""
        rows = slot.stored // (slot.numel // slot.shape[0])
        return buf[slot.offset:slot.offset + slot.stored].view((rows,) + tuple(slot.shape[1:]))

    def _init_params(self, seed):
        g = torch.Generator(device=self.dev).manual_seed(seed)
        for L in self.convs:
            fan_in = 9 * (3 if L.idx == 0 else L.c)
            w = torch.randn(L.w.shape, generator=g, device=self.dev) * math.sqrt(2.0 / fan_in)   # Kaiming normal
            if L.idx == 0:
                w[..., 3] = 0.0                 # the padded input channel carries no weight
            self.view(self.w32, L.w).copy_(w)
            self.view(self.w32, L.gamma).fill_(1.0)
            self.view(self.w32, L.beta).zero_()
        for f, (i_f, o_f) in zip(self.fc, self.fc_dims):
            self.view(self.w32, f["w"]).copy_(torch.randn((o_f, i_f), generator=g, device=self.dev) * math.sqrt(2.0 / i_f))
            self.view(self.w32, f["b"]).zero_()
        self.w16.copy_(self.w32)

    def load_params(self, params):
        """Master weights from numpy arrays: dict(convs=[dict(w, gamma, beta)], fcs=[dict(w, b)])."""
        for L, p in zip(self.convs, params["convs"]):
            self.view(self.w32, L.w).copy_(torch.from_numpy(p["w"]))
            self.view(self.w32, L.gamma).copy_(torch.from_numpy(p["gamma"]))
            self.view(self.w32, L.beta).copy_(torch.from_numpy(p["beta"]))
        for f, p in zip(self.fc, params["fcs"]):
            self.view(self.w32, f["w"]).copy_(torch.from_numpy(p["w"]))
            self.view(self.w32, f["b"]).copy_(torch.from_numpy(p["b"]))
        self.w16.copy_(self.w32)
        self.m32.zero_()

    def params(self):
        """Float master weights as numpy arrays (same structure as load_params takes)."""
        cp = lambda slot: self.view(self.w32, slot).detach().cpu().numpy().copy()
        return dict(convs=[dict(w=cp(L.w), gamma=cp(L.gamma), beta=cp(L.beta)) for L in self.convs],
                    fcs=[dict(w=cp(f["w"]), b=cp(f["b"])) for f in self.fc])

    # ------------------------------------------------------------------ input
    def upload(self, slot, host_images, host_labels):
        """Async H2D of one batch from pinned host memory into buffer `slot` on the copy stream."""
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self.slot_free[slot])
            self.images[slot].copy_(host_images, non_blocking=True)
            self.labels[slot].copy_(host_labels, non_blocking=True)
            self.copy_done[slot].record(self.copy_stream)

    # ------------------------------------------------------------------ one step
    def step(self, slot=0, wait_copy=False):
        """Forward + backward + all-reduce + SGD on input buffer `slot`.  Returns the device loss tensor."""
        cur = torch.cuda.current_stream()
        if wait_copy:
            cur.wait_event(self.copy_done[slot])
        self._forward(self.images[slot], self.labels[slot])
        self._backward(self.images[slot], self.labels[slot])
        self.slot_free[slot].record(cur)
        self.steps_done += 1
        return self.loss

    def _forward(self, images, labels):
        n = self.batch
        x = images
        for L in self.convs:
            b = L.buf
            w16 = self.view(self.w16, L.w)
            geo = ops.ConvGeometry(n, L.h, L.h, L.c, L.k)
            gamma, beta = self.view(self.w32, L.gamma), self.view(self.w32, L.beta)
            # conv with the batch statistics taken in its epilogue, then bn_finalize.  The 3(+1)->64 first
            # layer runs as a 1x1 GEMM over the pixels' 3x3 neighbourhoods, built in shared memory.
            if self.timing is not None and L.k >= 256:
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record()
            ops.conv_fprop_bn_stats(geo, x, w16, gamma, beta, y=b["conv_out"], out=b,
                                    running_mean=b["running_mean"], running_var=b["running_var"],
                                    workspace=self.ws)
            if self.timing is not None and L.k >= 256:
                t1.record()
                self.timing.append((t0, t1, 2.0 * n * L.h * L.h * L.c * L.k * 9,
                                    2.0 * (n * L.h * L.h * (L.c + L.k) + 9 * L.c * L.k)))
            if L.pool_after:
                # the pool is fused into the BN-apply kernel: the full-resolution ReLU output is never stored
                ops.bn_apply_relu_mask_pool(b["conv_out"], b["eq_scale"], b["eq_bias"], mask_bits=b["mask"],
                                            pool_out=b["pool_out"], argmax=b["argmax"])
                x = b["pool_out"]
            else:
                ops.bn_apply_relu_mask(b["conv_out"], b["eq_scale"], b["eq_bias"], relu_out=b["relu_out"],
                                       mask_bits=b["mask"])
                x = b["relu_out"]
        # classifier: flatten is a view of the NHWC pool output; bias, ReLU and dropout ride on the GEMM's output pass
        a = x.reshape(n, -1)
        self.fc_in = [a]
        for j, f in enumerate(self.fc):
            last = j == 2
            y = self.logits_rows if last else self.fc_out[j]
            ops.fc_amp_fwd(a, self.stored(self.w16, f["w"]), self.stored(self.w32, f["b"]), y=y, relu=not last,
                           dropout_p=0.0 if last else self.dropout, seed=self.seed,
                           offset=self.steps_done * 2 + j, workspace=self.ws)
            if not last:
                self.fc_in.append(y)
                a = y
        # loss + d_logits in one kernel (the FWD and BWD softmax-CE nodes fused)
        ops_out = ops.softmax_ce_amp_fused(self.logits, labels, self.scaling, self.label_smoothing,
                                           dlogits=self.dlogits)
        self.loss, self.inv_scaling = ops_out["loss"], ops_out["inv_scaling"]

    def _backward(self, images, labels):
        n = self.batch
        self.buckets.begin_step()
        # ---- classifier: db, dW, dx of each layer, then ReLU + dropout backward from the layer input's own values
        dz = self.dlogits_rows
        keep_scale = 1.0 / (1.0 - self.dropout)
        for j in reversed(range(3)):
            f = self.fc[j]
            # the layer's input carries the ReLU + dropout of the layer below: its backward rides on the dx pass
            ops.fc_amp_bwd(dz, self.stored(self.w16, f["w"]), self.fc_in[j], dx=self.fc_dx[j],
                           dw=self.stored(self.g32, f["w"]), db=self.stored(self.g32, f["b"]),
                           act=self.fc_in[j] if j > 0 else None, act_scale=keep_scale, workspace=self.ws)
            dz = self.fc_dx[j]
            self.buckets.mark_ready(self._end_of(f))
        # ---- feature extractor, last block first
        grad = dz.view(n, self.feat_hw, self.feat_hw, self.convs[-1].k)
        for L in reversed(self.convs):
            b = L.buf
            x = images if L.idx == 0 else (self.convs[L.idx - 1].buf["pool_out"] if self.convs[L.idx - 1].pool_after
                                           else self.convs[L.idx - 1].buf["relu_out"])
            geo = ops.ConvGeometry(n, L.h, L.h, L.c, L.k)
            if self.debug_hook is not None:
                self.debug_hook(L, grad, x)
            tev = None
            if self.timing_bwd is not None:
                tev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
                self.timing_bwd.append((L, tev))
            out = ops.cbr_amp_bwd(geo, grad, self.view(self.w16, L.w), self.view(self.w32, L.gamma),
                                  b["saved_mean"], b["saved_inv_std"], b["mask"], x, b["conv_out"],
                                  bn_scratch=self.bn_scratch[:b["conv_out"].numel()].view_as(b["conv_out"]),
                                  dw=self.half_grad(L.w), first_layer=(L.idx == 0), workspace=self.ws,
                                  dgamma=self.view(self.g32, L.gamma), dbeta=self.view(self.g32, L.beta),
                                  pool_argmax=b["argmax"] if L.pool_after else None,   # pool backward fused in
                                  timing_events=tev)
            grad = out["dx"]
            self.buckets.mark_ready(self._end_of(dict(w=L.w)))
        # BN gradients are float already and sit after every half-gradient slot
        self.buckets.finish()
        # ---- guard + optimizer over the whole flat range, then the loss-scale back-off (a step that saw a non-finite
        # gradient is skipped, halves the scale and resets the flag for the next step)
        ops.check_nonfinite(self.g32, self.nan_flag)
        ops.sgd_momentum(self.w32, self.g32, self.m32, self.w16, self.lr, self.wd, self.beta,
                         scaling=self.scaling, skip_flag=self.nan_flag)
        ops.grad_scaling(self.nan_flag, self.scaling, clear_flag=True)

    def sync_weights_from_rank0(self):
        """Every rank takes rank 0's master weights and momentum (after a diagnostic that let the ranks drift)."""
        if self.world > 1:
            dist.broadcast(self.w32, src=0, group=self.pg)
            dist.broadcast(self.m32, src=0, group=self.pg)
            self.w16.copy_(self.w32)

    def _end_of(self, group):
        """End offset (exclusive) of the flat range whose half gradients are complete once `group` is done."""
        last = group["w"]
        return last.offset + _align(getattr(last, "stored", last.numel))
