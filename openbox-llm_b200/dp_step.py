"""Data-parallel training step around the NSA model: one process per GPU, replicas kept in step by
a bucketed gradient all-reduce that overlaps the backward pass, then a clip + AdamW step that runs
as two kernels over flat fp32 buffers without a host synchronisation.

The reference trains on one GPU (train.py:246-264: autocast bf16 forward, backward,
clip_grad_norm_, AdamW betas (0.9, 0.95)); this is the same step for N replicas.  Gradients are
summed over ranks by NCCL and divided by the world size inside the optimizer kernel, so every
rank applies the mean gradient of the global batch."""
import torch
import torch.distributed as dist

from . import _lib as L


class FlatParams:
    """The distinct fp32 parameters of a module as views into one flat buffer, with a flat
    gradient buffer of the same layout (every p.grad is a view into it and stays one)."""

    def __init__(self, module):
        seen, self.params = set(), []
        for p in module.parameters():
            if p.requires_grad and id(p) not in seen:      # tied weights appear once
                seen.add(id(p))
                self.params.append(p)
        assert self.params, "no trainable parameters"
        dev = self.params[0].device
        assert all(p.dtype == torch.float32 and p.device == dev for p in self.params), \
            "parameters must be fp32 on one device"
        self.offsets, n = [], 0
        for p in self.params:
            self.offsets.append(n)
            n += (p.numel() + 3) // 4 * 4                  # 16-byte aligned slices
        self.numel = n
        self.flat = torch.zeros(n, dtype=torch.float32, device=dev)
        self.grad = torch.zeros(n, dtype=torch.float32, device=dev)
        for p, off in zip(self.params, self.offsets):
            self.flat[off:off + p.numel()].copy_(p.data.reshape(-1))
            p.data = self.flat[off:off + p.numel()].view(p.shape)
            p.grad = self.grad[off:off + p.numel()].view(p.shape)

    def zero_grad(self):
        self.grad.zero_()                                   # the views stay attached


class GradBuckets:
    """Contiguous ranges of the flat gradient buffer, filled from the last parameter backwards
    (the order backward produces gradients).  A post-accumulate hook on every parameter counts
    its bucket down; a full bucket is all-reduced (sum) at once on a side stream, so the
    transfer overlaps the rest of the backward pass.  With NVSwitch every bucket sees the full
    bandwidth, so buckets are sized for launch latency and overlap (default 64 MB)."""

    def __init__(self, flat: FlatParams, group=None, bucket_bytes=64 << 20):
        self.flat, self.group = flat, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.ranges, self.bucket_of, self.pending0 = [], {}, []
        hi, count = flat.numel, 0
        for i in range(len(flat.params) - 1, -1, -1):
            self.bucket_of[id(flat.params[i])] = len(self.ranges)
            count += 1
            lo = flat.offsets[i]
            if (hi - lo) * 4 >= bucket_bytes or i == 0:
                self.ranges.append((lo, hi))
                self.pending0.append(count)
                hi, count = lo, 0
        self.is_cuda = flat.grad.is_cuda
        self.comm_stream = torch.cuda.Stream(flat.grad.device) if self.is_cuda and self.world > 1 else None
        self.pending, self.handles = list(self.pending0), []
        self.enabled = True            # False: the hooks do nothing (gradients reduced in one piece)
        for p in flat.params:
            p.register_post_accumulate_grad_hook(self._ready)

    def reduce_all(self):
        """The whole flat gradient in one all-reduce on the current stream (no overlap)."""
        if self.world > 1:
            dist.all_reduce(self.flat.grad, op=dist.ReduceOp.SUM, group=self.group)

    def start(self):
        self.pending, self.handles = list(self.pending0), []

    def _ready(self, p):
        if not self.enabled:
            return
        b = self.bucket_of[id(p)]
        self.pending[b] -= 1
        if self.pending[b] == 0 and self.world > 1:
            lo, hi = self.ranges[b]
            view = self.flat.grad[lo:hi]
            if self.comm_stream is not None:
                self.comm_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.comm_stream):
                    self.handles.append(dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.group,
                                                        async_op=True))
            else:
                self.handles.append(dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.group,
                                                    async_op=True))

    def finish(self):
        """Every bucket reduced; the current stream may read the summed gradients."""
        assert all(c == 0 for c in self.pending) or self.world == 1 or not self.handles, \
            "a parameter received no gradient: its bucket was never reduced"
        for h in self.handles:
            h.wait()
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        self.handles = []


class FusedAdamW:
    """clip_grad_norm_ + AdamW (train.py:148-149, :262-264) as two kernels over the flat buffers."""

    def __init__(self, flat: FlatParams, lr, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, grad_clip=1.0):
        self.flat, self.lr, self.betas, self.eps = flat, lr, betas, eps
        self.weight_decay, self.grad_clip = weight_decay, grad_clip
        self.m = torch.zeros_like(flat.flat)
        self.v = torch.zeros_like(flat.flat)
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=flat.flat.device)
        self.t = 0

    def step(self, grad_scale=1.0, lr=None):
        with torch.cuda.device(self.flat.flat.device):    # the buffers' device, whatever is current
            self._step(grad_scale, lr)

    def _step(self, grad_scale, lr):
        f = self.flat
        self.t += 1
        self.sumsq.zero_()
        L.check(L.lib().nsa_sumsq_f32(L.ptr(f.grad), f.numel, L.ptr(self.sumsq), L.stream()))
        L.check(L.lib().nsa_adamw_step_f32(
            L.ptr(f.flat), L.ptr(f.grad), L.ptr(self.m), L.ptr(self.v), f.numel,
            float(self.lr if lr is None else lr), self.betas[0], self.betas[1], self.eps,
            self.weight_decay, self.t, L.ptr(self.sumsq), float(self.grad_clip or 0.0),
            float(grad_scale), L.stream()))

    def grad_norm(self, grad_scale=1.0):
        """Norm of the (scaled) gradient of the last step; reads the device value (synchronises)."""
        return float(self.sumsq.sqrt().item()) * grad_scale


class DataParallelStep:
    """One training step of a replica: forward under bf16 autocast, backward with overlapped
    gradient all-reduce, clip + AdamW.  Returns the loss as a device tensor (no host sync).

    use_graph=True replays forward + backward from a CUDA graph (captured on the first call
    after `graph_warmup` eager steps; the batch shape must not change): at the model's size the
    eager step is bound by the ~3000 launches the host has to issue, not by the GPU.  The
    gradients are then reduced in one all-reduce after the replay (NCCL stays outside the
    capture), which costs a millisecond of exposed transfer at this parameter count."""

    def __init__(self, model, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, grad_clip=1.0,
                 bucket_bytes=64 << 20, group=None, use_graph=False, graph_warmup=3, status_every=50):
        self.model = model
        self.flat = FlatParams(model)
        self.buckets = GradBuckets(self.flat, group, bucket_bytes)
        self.opt = FusedAdamW(self.flat, lr, betas, eps, weight_decay, grad_clip)
        self.use_graph, self.graph_warmup = use_graph, graph_warmup
        self.graph, self.calls = None, 0
        # every `status_every` steps the device status word is read (one stream synchronisation):
        # a kernel that gave up a bounded wait makes every later attention kernel return at entry,
        # which would otherwise go unnoticed for the rest of the run
        self.status_every = status_every

    def _forward_backward(self, idx, targets):
        self.flat.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            _, loss = self.model(idx, targets)
        loss.backward()
        return loss.detach()

    def step(self, idx, targets, lr=None):
        self.calls += 1
        if not self.use_graph:
            self.buckets.start()
            loss = self._forward_backward(idx, targets)
            self.buckets.finish()
        else:
            self.buckets.enabled = False
            if self.graph is None and self.calls <= self.graph_warmup:
                loss = self._forward_backward(idx, targets)          # eager: lazy initialisations happen here
            else:
                if self.graph is None:
                    self.g_idx, self.g_tgt = idx.clone(), targets.clone()
                    self.graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(self.graph):
                        self.g_loss = self._forward_backward(self.g_idx, self.g_tgt)
                self.g_idx.copy_(idx, non_blocking=True)
                self.g_tgt.copy_(targets, non_blocking=True)
                self.graph.replay()
                loss = self.g_loss
            self.buckets.reduce_all()
        self.opt.step(grad_scale=1.0 / self.buckets.world, lr=lr)
        if self.status_every and self.calls % self.status_every == 0:
            self.check_status()
        return loss

    def check_status(self):
        """Raise NsaError when a kernel of this device gave up a bounded wait since the last check."""
        with torch.cuda.device(self.flat.flat.device):
            L.check_device_status()
