"""Batch-sharded (data-parallel) use of the butterfly multiply on one multi-GPU box.

Rows of the batch are independent in the forward pass and in the input gradient; only the
twiddle gradient is a sum over rows.  So the layout is: one process per GPU, the batch cut
into contiguous row ranges, the twiddle replicated, no traffic between GPUs in the forward,
and exactly one all-reduce(SUM) of d_twiddle in the backward (SUM, not mean: it reproduces
the single-GPU gradient of the concatenated batch).  The reference library has no
distributed code on this path.
"""
import torch
import torch.distributed as dist


def shard_rows(batch: int, rank: int, world_size: int) -> slice:
    """Contiguous row range of `rank`: the first (batch % world_size) ranks get one extra row."""
    base, extra = divmod(batch, world_size)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def allreduce_twiddle_grad(d_twiddle: torch.Tensor, group=None) -> torch.Tensor:
    """In-place all-reduce(SUM) of a local twiddle gradient over the ranks (no-op without a process group)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        if d_twiddle.is_complex():
            dist.all_reduce(torch.view_as_real(d_twiddle), op=dist.ReduceOp.SUM, group=group)
        else:
            dist.all_reduce(d_twiddle, op=dist.ReduceOp.SUM, group=group)
    return d_twiddle


class _SyncTwiddleGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, twiddle, group):
        ctx.group = group
        return twiddle.view_as(twiddle)

    @staticmethod
    def backward(ctx, grad):
        return allreduce_twiddle_grad(grad.contiguous(), ctx.group), None


def sync_twiddle_grad(twiddle: torch.Tensor, group=None) -> torch.Tensor:
    """Identity in the forward pass; in the backward pass the gradient that flows into `twiddle`
    is all-reduced (SUM) over the ranks.  Use it on the replicated parameter of a batch-sharded
    layer:  ``y = butterfly_multiply(sync_twiddle_grad(layer.twiddle), x_local, True)``."""
    return _SyncTwiddleGrad.apply(twiddle, group)


class AsyncTwiddleReducer:
    """All-reduce(SUM) of twiddle gradients on a side stream, off the compute stream's critical path.

    The all-reduce of a latency-sized message (the twiddle gradient is a few hundred KB) costs
    tens of microseconds that nothing on the compute stream needs to wait for: the reduced
    gradient is only read by the optimizer step.  ``submit(d_twiddle)`` makes the side stream wait
    for the kernels that produce the gradient (an event on the current stream) and enqueues the
    all-reduce there; the next step's forward starts at once.  ``wait()`` makes the current stream
    (and therefore whatever reads the gradients next) wait for every all-reduce submitted so far.
    Without a process group both are no-ops.
    """

    def __init__(self, device, group=None):
        self.device = torch.device(device)
        self.group = group
        self.active = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        # CUDA: a side stream.  CPU tensors (gloo): the collective's own asynchronous handle.
        self.stream = torch.cuda.Stream(self.device) if self.active and self.device.type == "cuda" else None
        self.pending = []
        self.handles = []

    def submit(self, d_twiddle: torch.Tensor) -> torch.Tensor:
        if not self.active:
            return d_twiddle
        if self.stream is None:
            flat = torch.view_as_real(d_twiddle) if d_twiddle.is_complex() else d_twiddle
            self.handles.append(dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            self.pending.append(d_twiddle)
            return d_twiddle
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        d_twiddle.record_stream(self.stream)
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ready)
            allreduce_twiddle_grad(d_twiddle, self.group)
        self.pending.append(d_twiddle)
        return d_twiddle

    def wait(self):
        if self.active and self.stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
        for h in self.handles:
            h.wait()
        self.handles = []
        done, self.pending = self.pending, []
        return done
