"""Two NCCL ranks on two GPUs: the batch-sharded backward, its twiddle gradient all-reduced on
the side stream (butterfly_b200.distributed.AsyncTwiddleReducer), against the single-GPU
gradient of the concatenated batch and the double-precision oracle.  Skips with fewer than
two devices.  The ranks are child processes; each leaves between steps, with nothing in flight."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import butterfly_b200 as bb
    import oracle
    from butterfly_b200 import distributed as bd
    from conftest import assert_sum_accuracy
    oracle.build()
    red = bd.AsyncTwiddleReducer(dev)
    assert red.active
    # config 5's shapes at a batch the oracle finishes quickly: four stacks of n = 1024, the
    # input broadcast over the stacks (stride 0), two blocks; and a complex case
    for dtype, S, nb, log_n, B, bcast in ((torch.float32, 4, 2, 10, 192, True), (torch.complex64, 1, 1, 9, 150, False)):
        torch.manual_seed(3)  # same twiddle and same full batch on every rank
        n = 1 << log_n
        tw = torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dtype) / 2 ** 0.5
        x = torch.randn(B, 1 if bcast else S, n, dtype=dtype).expand(B, S, n)
        g = torch.randn(B, S, n, dtype=dtype)
        rows = bd.shard_rows(B, rank, world)
        twd = tw.to(dev)
        d_tw, d_x = bb.butterfly_multiply_bw(twd, x[rows].to(dev), g[rows].to(dev), True)
        red.submit(d_tw)
        # the next step's forward may start while the all-reduce runs
        y = bb.butterfly_multiply_fw(twd, x[rows].to(dev), True)
        red.wait()
        torch.cuda.synchronize()
        assert torch.equal(y.cpu(), bb.butterfly_multiply_fw(twd, x.to(dev), True)[rows].cpu())
        d_tw_one, d_x_one = bb.butterfly_multiply_bw(twd, x.to(dev), g.to(dev), True)  # the whole batch on this GPU
        assert torch.equal(d_x.cpu(), d_x_one[rows].cpu())
        ref32, _ = oracle.multiply_bw(tw, x.contiguous(), g, True)
        ref64, _ = oracle.multiply_bw(tw.to(torch.complex128 if dtype.is_complex else torch.float64),
                                      x.contiguous().to(torch.complex128 if dtype.is_complex else torch.float64),
                                      g.to(torch.complex128 if dtype.is_complex else torch.float64), True)
        assert_sum_accuracy(d_tw, ref32, ref64, "all-reduced d_twiddle, rank %d" % rank)
        assert_sum_accuracy(d_tw_one, ref32, ref64, "single-GPU d_twiddle")
        scale = d_tw_one.abs().max().item()
        assert (d_tw - d_tw_one).abs().max().item() <= 2e-5 * scale
        # every rank holds the same bits after the all-reduce
        gathered = [torch.empty_like(torch.view_as_real(d_tw) if dtype.is_complex else d_tw) for _ in range(world)]
        dist.all_gather(gathered, torch.view_as_real(d_tw) if dtype.is_complex else d_tw)
        assert all(torch.equal(gathered[0], t) for t in gathered[1:])
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(out_dir, "ok%d" % rank), "w").write("ok")


@pytest.mark.timeout(600)
def test_two_gpu_sharded_backward_matches_single_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    world = 2
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / ("ok%d" % r)) for r in range(world))
