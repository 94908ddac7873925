"""combine.py and kops.py on the GPU: butterflies folded with diagonals, multiplied together, and
as 2-D maps -- the tensor product run as ONE multiply against the reference's two-pass form
(what the reference checks in tests/test_combine.py:16-95)."""
import copy
import math

import pytest
import torch
import torch.nn.functional as F

from conftest import assert_rtol_atol

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda", 0)


def _dtype(cplx):
    return torch.complex64 if cplx else torch.float32


@pytest.mark.parametrize("cplx", [False, True])
@pytest.mark.parametrize("increasing_stride", [True, False])
@pytest.mark.parametrize("nblocks", [1, 2, 3])
def test_diagonal_butterfly(dev, cplx, increasing_stride, nblocks):
    import butterfly_b200 as bb
    torch.manual_seed(0)
    for in_size, out_size in ((32, 32), (27, 32), (32, 20)):
        b = bb.Butterfly(in_size, out_size, False, cplx, increasing_stride, nblocks=nblocks).to(dev)
        x = torch.randn(9, in_size, dtype=_dtype(cplx), device=dev)
        for diag_first in (True, False):
            d = torch.randn(in_size if diag_first else out_size, dtype=_dtype(cplx), device=dev)
            want = b(x * d) if diag_first else b(x) * d
            bd = bb.combine.diagonal_butterfly(b, d, diag_first, inplace=False)
            assert_rtol_atol(bd(x), want, "diagonal folded into the butterfly", rtol=1e-4, atol=1e-4)
            b2 = copy.deepcopy(b)
            assert b2.diagonal_multiply_(d, diag_first) is b2   # the method form, in place
            assert torch.equal(b2.twiddle, bd.twiddle)


@pytest.mark.parametrize("cplx", [False, True])
def test_butterfly_product_and_flip(dev, cplx):
    import butterfly_b200 as bb
    torch.manual_seed(1)
    n = 64
    x = torch.randn(7, n, dtype=_dtype(cplx), device=dev)
    for inc1 in (True, False):
        for inc2 in (True, False):
            for nb1, nb2 in ((1, 1), (2, 1), (1, 3)):
                b1 = bb.Butterfly(n, n, False, cplx, inc1, nblocks=nb1).to(dev)
                b2 = bb.Butterfly(n, n, False, cplx, inc2, nblocks=nb2).to(dev)
                prod = bb.combine.butterfly_product(b1, b2)
                assert_rtol_atol(prod(x), b2(b1(x)), "product of two butterflies", rtol=1e-4, atol=1e-4)
        b = bb.Butterfly(n, n, False, cplx, inc1, nblocks=2).to(dev)
        assert_rtol_atol(bb.combine.flip_increasing_stride(b)(x), b(x), "flipped stride direction", rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("cplx", [False, True])
@pytest.mark.parametrize("increasing_stride", [True, False])
@pytest.mark.parametrize("nblocks", [1, 2, 3])
def test_tensor_product_as_one_multiply(dev, cplx, increasing_stride, nblocks):
    """The fused TensorProduct (one multiply of size n2 * n1 with the Kronecker twiddle) against the
    two-pass form around a transpose: outputs, and gradients of both parameters and the input."""
    import butterfly_b200 as bb
    from butterfly_b200 import abi
    torch.manual_seed(2)
    n1, n2 = 16, 64
    b1 = bb.Butterfly(n1, n1, False, cplx, increasing_stride, nblocks=nblocks).to(dev)
    b2 = bb.Butterfly(n2, n2, False, cplx, increasing_stride, nblocks=nblocks).to(dev)
    tp = bb.combine.TensorProduct(b1, b2)
    two_pass = bb.combine.TensorProduct(b1, b2, fused=False)
    assert tp.fusible()
    x = torch.randn(3, 5, n2, n1, dtype=_dtype(cplx), device=dev, requires_grad=True)
    g = torch.randn(3, 5, n2, n1, dtype=_dtype(cplx), device=dev)
    launches = abi.launch_count()
    y = tp(x)
    fused_launches = abi.launch_count() - launches
    y.backward(g)
    got = (y.detach(), x.grad.clone(), b1.twiddle.grad.clone(), b2.twiddle.grad.clone())
    x.grad = b1.twiddle.grad = b2.twiddle.grad = None
    launches = abi.launch_count()
    y2 = two_pass(x)
    # one multiply (for float32 rows of 512 or more columns preceded by its twiddle re-ordering kernel) against two
    assert fused_launches == (1 if cplx else 2) and abi.launch_count() - launches == 2
    y2.backward(g)
    want = (y2.detach(), x.grad, b1.twiddle.grad, b2.twiddle.grad)
    for a, b, what in zip(got, want, ("output", "d_input", "d_twiddle of map1", "d_twiddle of map2")):
        assert_rtol_atol(a, b, "tensor product, " + what, rtol=1e-4, atol=2e-4)
    # the same matrix as a stand-alone Butterfly on flattened images
    kron = bb.combine.butterfly_kronecker(b1, b2)
    assert_rtol_atol(kron(x.detach().reshape(15, n2 * n1)).reshape(3, 5, n2, n1), want[0], "butterfly_kronecker", rtol=1e-4, atol=2e-4)
    # smaller images are zero-padded per dimension, as the two maps would do one after the other
    xs = torch.randn(4, n2 - 3, n1 - 5, dtype=_dtype(cplx), device=dev)
    assert_rtol_atol(tp(xs), two_pass(xs), "tensor product of a smaller image", rtol=1e-4, atol=2e-4)
    # maps that do not line up run in two passes
    b3 = bb.Butterfly(n2, n2, False, cplx, not increasing_stride, nblocks=nblocks).to(dev)
    assert not bb.combine.TensorProduct(b1, b3).fusible()
    assert bb.combine.TensorProduct(b1, b3)(x).shape == x.shape


def test_permutation_kronecker(dev):
    import butterfly_b200 as bb
    torch.manual_seed(3)
    n1, n2 = 8, 4
    p1 = bb.permutation.FixedPermutation(torch.randperm(n1)).to(dev)
    p2 = bb.permutation.FixedPermutation(torch.randperm(n2)).to(dev)
    x = torch.randn(6, n2, n1, device=dev)
    want = p2(p1(x).transpose(-1, -2)).transpose(-1, -2)
    got = bb.combine.permutation_kronecker(p1, p2)(x.reshape(6, n2 * n1)).reshape(6, n2, n1)
    assert torch.equal(got, want)


@pytest.mark.parametrize("nblocks", [1, 2])
def test_kop2d_fft_init_is_the_circular_convolution(dev, nblocks):
    """KOP2d initialised to the FFT computes Conv2d with circular padding exactly; each of its
    three 2-D maps is one multiply launch."""
    import butterfly_b200 as bb
    from butterfly_b200 import abi
    torch.manual_seed(4)
    h, w, cin, cout, k = 16, 32, 3, 5, 3
    layer = bb.kops.KOP2d((h, w), cin, cout, k, complex=True, init="fft", nblocks=nblocks).to(dev)
    x = torch.randn(4, cin, h, w, device=dev)
    launches = abi.launch_count()
    y = layer(x)
    assert abi.launch_count() - launches == 3
    conv_w = layer.weight.detach().flip([-1, -2])
    pad = (k - 1) // 2
    want = F.conv2d(F.pad(x, (pad, pad, pad, pad), mode="circular"), conv_w)
    assert_rtol_atol(y, want, "KOP2d against Conv2d", rtol=1e-4, atol=1e-4)
    # it trains: gradients reach the weight and all six butterflies
    y.square().mean().backward()
    assert layer.weight.grad is not None and all(p.grad is not None and torch.isfinite(torch.view_as_real(p.grad) if p.grad.is_complex() else p.grad).all()
                                                 for p in layer.parameters())
    # radix-4 maps (two-pass execution) give the same function
    layer4 = bb.kops.KOP2d((h, w), cin, cout, k, complex=True, init="fft", nblocks=nblocks, base=4).to(dev)
    with torch.no_grad():
        layer4.weight.copy_(layer.weight)
    assert_rtol_atol(layer4(x), want, "KOP2d base 4 against Conv2d", rtol=1e-4, atol=1e-4)
    assert math.isfinite(y.sum().item())
