"""The no-allocation backward entry point (collected last on purpose: if it fails, a run that
stops at the first failure has already run everything else).

``bfly_bw_f32_noalloc`` serves hosts that cannot give the library device scratch at the call
site -- a plugin inside a framework that owns all device memory, a real-time or graph-captured
loop where an allocation would stall the device.  It must give the same gradients as
``bfly_bw_f32`` (which takes a caller-provided workspace), on every call, although all calls
share one built-in buffer that keeps the previous call's contents.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a - b).abs().max() / (b.abs().max() + 1e-30)).item()


def test_noalloc_backward_matches_workspace_backward_twice_in_a_row(oracle_mod):
    from butterfly_b200 import abi
    assert torch.cuda.is_available()
    dev = torch.device("cuda", 0)
    torch.manual_seed(11)
    # n = 4096 with two blocks: three backward phases, i.e. the scratch buffer is really used
    S, nblocks, log_n = 1, 2, 12
    n = 1 << log_n
    need = abi.bw_workspace_bytes(torch.float32, 512, S, log_n, nblocks)
    assert 0 < need <= abi.NOALLOC_SCRATCH_BYTES
    tw = (torch.randn(S, nblocks, log_n, n // 2, 2, 2) / 2 ** 0.5).to(dev)
    results = []
    for call, (B, in_size, out_size) in enumerate([(512, n, n), (300, n - 7, n - 3)]):
        x = torch.randn(B, S, in_size, device=dev)
        g = torch.randn(B, S, out_size, device=dev)
        ref_dtw, ref_dx, _ = abi.bw(tw, x, g, True)
        d_tw = torch.empty_like(tw)
        d_x = torch.empty(B, S, max(in_size, n), device=dev)
        if call == 0:
            # the first call on a device looks up the buffer's address; do it before measuring
            abi.bw_noalloc(tw, x, g, True, d_twiddle=d_tw, d_x=d_x)
        torch.cuda.synchronize()
        torch_allocs = torch.cuda.memory_stats(dev)["allocation.all.allocated"]
        free_before, _ = torch.cuda.mem_get_info(dev)
        got_dtw, got_dx, rc = abi.bw_noalloc(tw, x, g, True, d_twiddle=d_tw, d_x=d_x)
        torch.cuda.synchronize()
        assert rc == 0
        # the call took nothing from torch's allocator and nothing from the driver
        assert torch.cuda.memory_stats(dev)["allocation.all.allocated"] == torch_allocs
        assert torch.cuda.mem_get_info(dev)[0] == free_before
        # d_input is deterministic; d_twiddle differs only by the order of the final atomic adds
        assert torch.equal(got_dx[:, :, :in_size], ref_dx[:, :, :in_size]), "call %d" % call
        assert _rel(got_dtw, ref_dtw) < 2e-5, "call %d" % call
        if call == 1:
            # and once against the CPU oracle (not only against the other CUDA entry point)
            o_dtw, o_dx = oracle_mod.multiply_bw(tw.cpu(), x.cpu(), g.cpu(), True)
            assert _rel(got_dx[:, :, :in_size].cpu(), o_dx) < 2e-5 and _rel(got_dtw.cpu(), o_dtw) < 2e-5
        results.append(got_dtw)
    assert not torch.equal(results[0], results[1])  # two different problems were really solved


def test_noalloc_backward_rejects_problems_beyond_its_buffer():
    from butterfly_b200 import abi
    dev = torch.device("cuda", 0)
    S, nblocks, log_n, B = 1, 2, 12, 8192  # needs 2-3 snapshots of 128 MiB
    n = 1 << log_n
    assert abi.bw_workspace_bytes(torch.float32, B, S, log_n, nblocks) > abi.NOALLOC_SCRATCH_BYTES
    tw = torch.randn(S, nblocks, log_n, n // 2, 2, 2, device=dev)
    x = torch.randn(B, S, n, device=dev)
    d_tw = torch.full_like(tw, 7.0)
    _, _, rc = abi.bw_noalloc(tw, x, x, True, d_twiddle=d_tw, check=False)
    assert rc == -7
    assert "scratch" in abi.strerror(rc)
    assert (d_tw == 7.0).all()  # a rejected call touches nothing
    # a single-phase shape needs no scratch at all and is accepted at any batch size
    tw1 = torch.randn(1, 1, 8, 128, 2, 2, device=dev)
    x1 = torch.randn(80000, 1, 256, device=dev)
    a, b, rc = abi.bw_noalloc(tw1, x1, x1, True)
    ra, rb, _ = abi.bw(tw1, x1, x1, True)
    assert rc == 0 and torch.equal(b, rb) and _rel(a, ra) < 2e-5
