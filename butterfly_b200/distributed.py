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
