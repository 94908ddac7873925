"""The batch-sharded path with two gloo ranks on the CPU: row sharding, and the single
all-reduce(SUM) of the twiddle gradient reproducing the full-batch gradient.  The local
compute of each rank stands in for the CUDA operator (the oracle here), the plumbing under
test is butterfly_b200.distributed."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from butterfly_b200 import distributed as bd
    torch.manual_seed(0)  # same twiddle and same full batch on every rank
    S, nb, log_n, B = 2, 2, 6, 13
    n = 1 << log_n
    for dtype in (torch.float32, torch.complex64):
        tw = torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dtype)
        x = torch.randn(B, S, n, dtype=dtype)
        g = torch.randn(B, S, n, dtype=dtype)
        rows = bd.shard_rows(B, rank, world)
        d_tw_local, d_x_local = oracle.multiply_bw(tw, x[rows], g[rows], True)
        d_tw = bd.allreduce_twiddle_grad(d_tw_local.clone())
        d_tw_full, d_x_full = oracle.multiply_bw(tw, x, g, True)
        # same terms summed in a different order: equal up to float rounding of the sums
        assert (d_tw - d_tw_full).abs().max() <= 2e-6 * d_tw_full.abs().max()
        assert torch.equal(d_x_local, d_x_full[rows])   # no cross-rank term in the input gradient
        # the same sum through the reducer that runs off the critical path (submit now, wait later)
        red = bd.AsyncTwiddleReducer("cpu")
        assert red.active
        mine = red.submit(d_tw_local.clone())
        other = red.submit(torch.full((3,), float(rank + 1)))
        done = red.wait()
        assert len(done) == 2 and red.wait() == []
        assert torch.equal(mine, d_tw) and torch.equal(other, torch.full((3,), float(sum(range(1, world + 1)))))
    # the autograd hook: gradient of a replicated parameter is summed over ranks
    p = torch.ones(4, requires_grad=True)
    loss = (bd.sync_twiddle_grad(p) * (rank + 1)).sum()
    loss.backward()
    assert torch.equal(p.grad, torch.full((4,), float(sum(range(1, world + 1)))))
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(out_dir, "ok%d" % rank), "w").write("ok")


def test_shard_rows_partition():
    from butterfly_b200.distributed import shard_rows
    for batch in (0, 1, 7, 8, 65536):
        for world in (1, 2, 3, 8):
            parts = [shard_rows(batch, r, world) for r in range(world)]
            assert parts[0].start == 0 and parts[-1].stop == batch
            assert all(a.stop == b.start for a, b in zip(parts, parts[1:]))
            sizes = [p.stop - p.start for p in parts]
            assert max(sizes) - min(sizes) <= 1


@pytest.mark.timeout(300)
def test_two_rank_gloo_twiddle_grad_allreduce(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / ("ok%d" % r)) for r in range(world))
