"""Exact fast transforms written as Butterfly layers.

Counterparts in the reference: ``fft``, ``ifft``, ``hadamard``, ``circulant``
(torch_butterfly/special.py:19-117, 248-301, 304-327).  They only build twiddles and call the
layers of butterfly.py, so they exercise the operators end to end.
"""
import math

import torch
from torch import nn

from .butterfly import Butterfly
from .permutation import FixedPermutation, bitreversal_permutation


def fft_twiddle(n, inverse=False, normalized=False, br_first=True, dtype=torch.complex64):
    """Twiddle (1, 1, log_n, n/2, 2, 2) of the radix-2 (i)FFT without its bit-reversal permutation.

    br_first=True is decimation in time: the input is expected bit-reversed and the factors run
    with increasing stride; stage s (stride 2^s) has blocks [[1, w], [1, -w]], w = exp(-+2 pi i k / 2^(s+1)).
    br_first=False is decimation in frequency: factors run with decreasing stride, blocks
    [[1, 1], [w, -w]], and the output comes out bit-reversed.
    """
    log_n = int(math.log2(n))
    assert n == 1 << log_n
    sign = 1.0 if inverse else -1.0
    factors = []
    for s in range(log_n):
        size = 1 << (s + 1)
        k = torch.arange(size // 2, dtype=torch.float64)
        w = torch.exp(sign * 2j * math.pi * k / size)
        one = torch.ones_like(w)
        if br_first:
            block = torch.stack((torch.stack((one, w), dim=-1), torch.stack((one, -w), dim=-1)), dim=-2)
        else:
            block = torch.stack((torch.stack((one, one), dim=-1), torch.stack((w, -w), dim=-1)), dim=-2)
        factors.append(block.repeat(n // size, 1, 1))  # (n/2, 2, 2), pair index = position with bit s removed
    if not br_first:
        factors = factors[::-1]
    tw = torch.stack(factors, dim=0)
    if normalized:
        tw = tw / math.sqrt(2)
    elif inverse:
        tw = tw / 2
    return tw.reshape(1, 1, log_n, n // 2, 2, 2).to(dtype)


def _transform(n, inverse, normalized, br_first, with_br_perm):
    tw = fft_twiddle(n, inverse=inverse, normalized=normalized, br_first=br_first)
    b = Butterfly(n, n, bias=False, complex=True, increasing_stride=br_first, init=tw)
    if not with_br_perm:
        return b
    br = FixedPermutation(bitreversal_permutation(n))
    return nn.Sequential(br, b) if br_first else nn.Sequential(b, br)


def fft(n, normalized=False, br_first=True, with_br_perm=True):
    """Module computing torch.fft.fft(x, norm='ortho' if normalized else None) along the last dim."""
    return _transform(n, False, normalized, br_first, with_br_perm)


def ifft(n, normalized=False, br_first=True, with_br_perm=True):
    """Module computing torch.fft.ifft along the last dim."""
    return _transform(n, True, normalized, br_first, with_br_perm)


def hadamard(n, normalized=False, increasing_stride=True):
    """Module multiplying by the n x n Walsh-Hadamard matrix (Sylvester order)."""
    log_n = int(math.log2(n))
    assert n == 1 << log_n
    h = torch.tensor([[1.0, 1.0], [1.0, -1.0]])
    if normalized:
        h = h / math.sqrt(2)
    tw = h.reshape(1, 1, 1, 1, 2, 2).expand(1, 1, log_n, n // 2, 2, 2).contiguous()
    return Butterfly(n, n, bias=False, complex=False, increasing_stride=increasing_stride, init=tw)


class _Circulant(nn.Module):
    """x -> irfft-free circular convolution with a fixed first column: ifft(diag(fft(col)) fft(x))."""

    def __init__(self, col):
        super().__init__()
        n = col.shape[-1]
        self.n = n
        self.real = not col.is_complex()
        self.fft = fft(n, br_first=False, with_br_perm=False)   # output bit-reversed
        self.ifft = ifft(n, br_first=True, with_br_perm=False)  # input bit-reversed: the permutations cancel
        spectrum = torch.fft.fft(col.to(torch.complex64))
        self.register_buffer("diag", spectrum[bitreversal_permutation(n)].contiguous())

    def forward(self, x):
        y = self.ifft(self.fft(x.to(torch.complex64)) * self.diag)
        return y.real if self.real else y


def circulant(col):
    """Module multiplying by the circulant matrix whose first column is `col` (n a power of two)."""
    return _Circulant(col)
