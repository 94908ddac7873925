"""The nn.Module layers and exact-transform constructions on top of the CUDA operators
(what the reference checks in tests/test_butterfly.py and tests/test_special.py)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda", 0)


def _matrix(layer, n_in, dtype, dev, **kw):
    """Dense matrix of a bias-free layer: apply it to the identity."""
    eye = torch.eye(n_in, dtype=dtype, device=dev)
    return layer(eye, **kw).t()


def test_butterfly_shapes_and_linear_compat(dev):
    import butterfly_b200 as bb
    for in_size, out_size in [(7, 15), (15, 7), (100, 300), (1024, 4096)]:
        for complex in (False, True):
            for nblocks in (1, 2, 3):
                b = bb.Butterfly(in_size, out_size, bias=True, complex=complex, nblocks=nblocks).to(dev)
                x = torch.randn(5, 3, in_size, dtype=b.twiddle.dtype, device=dev)
                y = b(x)
                assert y.shape == (5, 3, out_size)
                assert torch.isfinite(torch.view_as_real(y) if complex else y).all()


def test_transpose_conjugate_flags_match_explicit_matrix(dev):
    import butterfly_b200 as bb
    n = 16
    for complex in (False, True):
        for inc in (True, False):
            for nblocks in (1, 2, 3):
                b = bb.Butterfly(n, n, bias=False, complex=complex, increasing_stride=inc, nblocks=nblocks).to(dev)
                dt = b.twiddle.dtype
                m = _matrix(b, n, dt, dev)
                assert torch.allclose(_matrix(b, n, dt, dev, transpose=True), m.t(), atol=1e-5)
                assert torch.allclose(_matrix(b, n, dt, dev, conjugate=True), m.conj(), atol=1e-5)
                assert torch.allclose(_matrix(b, n, dt, dev, transpose=True, conjugate=True), m.t().conj(), atol=1e-5)


def test_fft_ifft_hadamard_circulant(dev):
    import butterfly_b200 as bb
    from butterfly_b200 import special
    for n in (2, 16, 256, 2048):
        x = torch.randn(6, n, dtype=torch.complex64, device=dev)
        for normalized in (False, True):
            norm = "ortho" if normalized else None
            for br_first in (True, False):
                f = special.fft(n, normalized=normalized, br_first=br_first).to(dev)
                fi = special.ifft(n, normalized=normalized, br_first=br_first).to(dev)
                scale = torch.fft.fft(x, norm=norm).abs().max()
                assert (f(x) - torch.fft.fft(x, norm=norm)).abs().max() < 2e-5 * scale + 1e-5
                assert (fi(x) - torch.fft.ifft(x, norm=norm)).abs().max() < 1e-5
                assert (fi(f(x)) - x * (1 if True else 1)).abs().max() < 1e-4 if normalized else True
    # 'fft_no_br' init of a plain Butterfly
    n = 64
    b = bb.Butterfly(n, n, bias=False, complex=True, init="fft_no_br").to(dev)
    x = torch.randn(4, n, dtype=torch.complex64, device=dev)
    br = bb.permutation.bitreversal_permutation(n).to(dev)
    assert (b(x[:, br]) - torch.fft.fft(x, norm="ortho")).abs().max() < 1e-5
    # Hadamard against the Sylvester construction
    for n in (2, 8, 128):
        h = torch.tensor([[1.0]])
        while h.shape[0] < n:
            h = torch.cat((torch.cat((h, h), 1), torch.cat((h, -h), 1)), 0)
        x = torch.randn(5, n, device=dev)
        for inc in (True, False):
            assert torch.allclose(special.hadamard(n, increasing_stride=inc).to(dev)(x), x @ h.to(dev).t(), atol=1e-4)
    # circulant against the explicit matrix
    n = 32
    col = torch.randn(n)
    c = special.circulant(col).to(dev)
    mat = torch.stack([torch.roll(col, j) for j in range(n)], dim=1).to(dev)  # column j = col rolled by j
    x = torch.randn(7, n, device=dev)
    assert torch.allclose(c(x), x @ mat.t(), atol=1e-4)


def test_bmm_equals_loop_of_butterflies_exactly(dev):
    import butterfly_b200 as bb
    torch.manual_seed(0)
    in_size, out_size, mb = 24, 40, 3
    for complex in (False, True):
        bmm = bb.ButterflyBmm(in_size, out_size, matrix_batch=mb, bias=True, complex=complex, nblocks=2).to(dev)
        x = torch.randn(9, mb, in_size, dtype=bmm.twiddle.dtype, device=dev)
        y = bmm(x)
        S = bmm.nstacks
        for i in range(mb):
            single = bb.Butterfly(in_size, out_size, bias=True, complex=complex, nblocks=2,
                                  init=bmm.twiddle[i * S:(i + 1) * S].detach().clone()).to(dev)
            with torch.no_grad():
                single.bias.copy_(bmm.bias[i])
            assert torch.equal(single(x[:, i]), y[:, i])


def test_to_base4_and_unitary_and_scaling(dev):
    import butterfly_b200 as bb
    torch.manual_seed(1)
    for in_size, out_size, nblocks in [(16, 16, 1), (20, 50, 2), (128, 128, 3)]:
        b = bb.Butterfly(in_size, out_size, bias=True, nblocks=nblocks).to(dev)
        b4 = b.to_base4()
        x = torch.randn(11, in_size, device=dev)
        assert torch.allclose(b(x), b4(x), rtol=1e-4, atol=1e-4)
        y = b(x)
        b *= 3.0
        assert torch.allclose((b(x) - b.bias) , 3.0 * (y - b.bias), rtol=1e-4, atol=1e-4)
    # complex layers: the base-4 form runs the complex64 base-4 operator, forward and backward
    for n, nblocks in [(32, 1), (64, 2)]:
        b = bb.Butterfly(n, n, bias=False, complex=True, nblocks=nblocks).to(dev)
        b4 = b.to_base4()
        x = torch.randn(9, n, dtype=torch.complex64, device=dev)
        xa = x.clone().requires_grad_(True)
        xb = x.clone().requires_grad_(True)
        ya, yb = b(xa), b4(xb)
        assert torch.allclose(ya, yb, rtol=1e-4, atol=1e-4)
        w = torch.randn_like(ya)
        (ya * w).real.sum().backward()
        (yb * w).real.sum().backward()
        assert torch.allclose(xa.grad, xb.grad, rtol=1e-4, atol=1e-4)
        assert b4.twiddle4.grad is not None and torch.isfinite(torch.view_as_real(b4.twiddle4.grad)).all()
    u = bb.ButterflyUnitary(32, 32, bias=False, nblocks=2).to(dev)
    m = _matrix(u, 32, torch.complex64, dev)
    assert torch.allclose(m @ m.t().conj(), torch.eye(32, dtype=torch.complex64, device=dev), atol=1e-5)
    # subtwiddle: a shorter input uses the leading part of the parameters
    b = bb.Butterfly(64, 64, bias=False).to(dev)
    x = torch.randn(3, 16, device=dev)
    small = bb.Butterfly(16, 16, bias=False, init=b.twiddle[:, :, :4, :8].detach().clone()).to(dev)
    assert torch.allclose(b(x, subtwiddle=True), small(x), atol=1e-6)


def test_training_step_decreases_loss(dev):
    """A Butterfly layer learns a fixed random orthogonal map with plain SGD."""
    import butterfly_b200 as bb
    torch.manual_seed(2)
    n = 64
    target = torch.linalg.qr(torch.randn(n, n))[0].to(dev)
    layer = bb.Butterfly(n, n, bias=False, nblocks=2, init="ortho").to(dev)
    opt = torch.optim.SGD(layer.parameters(), lr=0.05)
    x = torch.randn(512, n, device=dev)
    losses = []
    for _ in range(60):
        loss = ((layer(x) - x @ target.t()) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.7 * losses[0]
    assert all(math.isfinite(v) for v in losses)


def test_unitary_twiddle_kernels_match_the_torch_chain(dev):
    """bfly_unitary_twiddle_fw / _bw (through the C ABI and through the differentiable torch
    operator) against the reference's cos / sin / stack chain and autograd's backward of it
    (torch_butterfly/butterfly.py:271-280); ButterflyUnitary trains through them."""
    import math
    import butterfly_b200 as bb
    from butterfly_b200 import abi
    from conftest import assert_rtol_atol, unitary_chain
    torch.manual_seed(4)
    shape = (3, 2, 11, 1024)
    angles = torch.cat([torch.asin(torch.sqrt(torch.rand(shape + (1,)))), torch.rand(shape + (3,)) * 2 * math.pi], dim=-1).to(dev)
    a = angles.clone().requires_grad_(True)
    ref = unitary_chain(a)
    g = torch.randn(shape + (2, 2), dtype=torch.complex64, device=dev)
    ref.backward(g)
    launches = abi.launch_count()
    tw, rc = abi.unitary_twiddle_fw(angles)
    d, rc2 = abi.unitary_twiddle_bw(angles, g)
    assert rc == 0 and rc2 == 0 and abi.launch_count() - launches == 2
    assert_rtol_atol(tw, ref.detach(), "unitary twiddle", rtol=1e-5, atol=1e-6)
    assert_rtol_atol(d, a.grad, "unitary twiddle gradient", rtol=1e-5, atol=2e-6)
    # the differentiable operator, with a lazily conjugated gradient
    a2 = angles.clone().requires_grad_(True)
    bb.unitary_twiddle(a2).backward(g.conj().conj())
    assert torch.equal(a2.grad, d)
    # empty tensors, misaligned pointers
    assert abi.unitary_twiddle_fw(angles[:0])[0].shape == (0, 2, 11, 1024, 2, 2)
    bad = torch.empty(4 * 8 + 1, device=dev)[1:].view(8, 4)
    assert abi.unitary_twiddle_fw(bad, check=False)[1] == -3
    # the layer: unitary matrix, gradients reach the angles
    layer = bb.ButterflyUnitary(64, 64, bias=False).to(dev)
    m = layer(torch.eye(64, dtype=torch.complex64, device=dev)).t()
    assert (m @ m.conj().t() - torch.eye(64, device=dev)).abs().max() < 1e-5
    x = torch.randn(32, 64, dtype=torch.complex64, device=dev)
    layer(x).abs().pow(2).sum().backward()
    ref_layer = bb.ButterflyUnitary(64, 64, bias=False).to(dev)
    with torch.no_grad():
        ref_layer.twiddle.copy_(layer.twiddle)
    tw_ref = unitary_chain(ref_layer.twiddle)
    bb.butterfly_multiply(tw_ref, x.unsqueeze(1), True).squeeze(1).abs().pow(2).sum().backward()
    assert_rtol_atol(layer.twiddle.grad, ref_layer.twiddle.grad, "angle gradients through the layer", rtol=1e-4, atol=1e-4)


def test_host_pipeline_results_and_give_up_flag(dev, oracle_mod):
    """HostPipeline.fw_bw from pinned host memory: after wait() the host buffers hold the results (read at
    once, no other synchronisation); a raised give-up flag makes wait() raise and is cleared."""
    import butterfly_b200 as bb
    from butterfly_b200 import abi
    from butterfly_b200.host import HostPipeline
    from conftest import rel_err
    torch.manual_seed(6)
    B, S, log_n, nb = 100, 2, 9, 2
    n = 1 << log_n
    tw = torch.randn(S, nb, log_n, n // 2, 2, 2) / 2 ** 0.5
    x = torch.randn(B, S, n).pin_memory()
    g = torch.randn(B, S, n).pin_memory()
    out = torch.empty(B, S, n).pin_memory()
    d_x = torch.empty(B, S, n).pin_memory()
    d_tw = torch.empty_like(tw).pin_memory()
    pipe = HostPipeline(dev, chunks=3)
    pipe.fw_bw(tw.to(dev), x, g, True, out, d_x, d_tw)
    pipe.wait()
    yr = oracle_mod.multiply_fw(tw, x, True)
    dtr, dxr = oracle_mod.multiply_bw(tw, x, g, True)
    assert rel_err(out, yr) < 2e-5 and rel_err(d_x, dxr) < 2e-5 and rel_err(d_tw, dtr) < 2e-5
    # a kernel that gave up (the library's self-test warp) is reported at the pipeline's sync point
    abi.selftest_bounded_wait(2048)
    pipe.fw_bw(tw.to(dev), x, g, True, out, d_x, d_tw)
    with pytest.raises(RuntimeError, match="gave up"):
        pipe.wait()
    assert abi.device_error() == 0
    pipe.fw_bw(tw.to(dev), x, g, True, out, d_x, d_tw)
    pipe.wait()
    assert rel_err(out, yr) < 2e-5
