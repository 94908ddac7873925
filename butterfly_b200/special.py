"""Exact fast transforms written as Butterfly layers.

Counterparts in the reference: ``fft``, ``ifft``, ``hadamard``, ``circulant``
(torch_butterfly/special.py:19-117, 248-301, 304-327).  They build twiddles and chain the layers
of butterfly.py with permutation / diagonal / real-complex modules; by default the chain is then
rewritten by glue.fuse so that those modules run inside the butterflies' kernel launches.
"""
import math

import torch
from torch import nn

from torch.nn import functional as F

from .butterfly import Butterfly
from .complex_utils import Complex2Real, Real2Complex, real2complex
from .diagonal import Diagonal
from .glue import fuse
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


def _transform(n, inverse, normalized, br_first, with_br_perm, fused=True):
    tw = fft_twiddle(n, inverse=inverse, normalized=normalized, br_first=br_first)
    b = Butterfly(n, n, bias=False, complex=True, increasing_stride=br_first, init=tw)
    if not with_br_perm:
        return b
    br = FixedPermutation(bitreversal_permutation(n))
    chain = nn.Sequential(br, b) if br_first else nn.Sequential(b, br)
    return fuse(chain) if fused else chain


def fft(n, normalized=False, br_first=True, with_br_perm=True, fused=True):
    """Module computing torch.fft.fft(x, norm='ortho' if normalized else None) along the last dim.
    fused: the bit-reversal runs inside the butterfly's launch (glue.ButterflyPipeline) instead of
    as a gather module of its own."""
    return _transform(n, False, normalized, br_first, with_br_perm, fused)


def ifft(n, normalized=False, br_first=True, with_br_perm=True, fused=True):
    """Module computing torch.fft.ifft along the last dim."""
    return _transform(n, True, normalized, br_first, with_br_perm, fused)


def hadamard(n, normalized=False, increasing_stride=True):
    """Module multiplying by the n x n Walsh-Hadamard matrix (Sylvester order)."""
    log_n = int(math.log2(n))
    assert n == 1 << log_n
    h = torch.tensor([[1.0, 1.0], [1.0, -1.0]])
    if normalized:
        h = h / math.sqrt(2)
    tw = h.reshape(1, 1, 1, 1, 2, 2).expand(1, 1, log_n, n // 2, 2, 2).contiguous()
    return Butterfly(n, n, bias=False, complex=False, increasing_stride=increasing_stride, init=tw)


def circulant(col, transposed=False, separate_diagonal=True, fused=True):
    """Module multiplying by the circulant matrix whose first column is `col` (its first row when
    `transposed`): ifft(diag(fft(col)) fft(x)), the FFT leaving its output bit-reversed and the
    inverse taking it that way, so no permutation is needed.

    separate_diagonal: Butterfly, Diagonal, Butterfly (the spectrum stays a parameter of its own);
    otherwise the diagonal is folded into the first butterfly and the two become one Butterfly of
    two blocks.  A length that is not a power of two is embedded in a circulant of the next power
    of two doubled.  fused: real <-> complex conversion and the diagonal run inside the butterflies'
    launches (two launches for the whole chain)."""
    assert col.dim() == 1
    cplx = col.is_complex()
    n = col.shape[0]
    log_n = int(math.ceil(math.log2(n)))
    n_ext = n if n == 1 << log_n else 1 << (log_n + 1)
    b_fft = fft(n_ext, normalized=True, br_first=False, with_br_perm=False).to(col.device)
    b_ifft = ifft(n_ext, normalized=True, br_first=True, with_br_perm=False).to(col.device)
    b_fft.in_size, b_ifft.out_size = n, n
    if n < n_ext:  # [a, b, c] -> [a, b, c, 0, 0, a, b, c]: the leading n x n corner of the larger circulant
        col = torch.cat((F.pad(col, (0, 2 * ((1 << log_n) - n))), col))
    spectrum = torch.fft.fft(real2complex(col))
    if transposed:  # the first row is the first column reversed (element 0 stays): same reversal of the spectrum
        spectrum = torch.cat((spectrum[:1], spectrum[1:].flip([0])))
    diag = spectrum[bitreversal_permutation(n_ext).to(col.device)].to(torch.complex64)
    if separate_diagonal:
        chain = [b_fft, Diagonal(diagonal_init=diag), b_ifft]
    else:
        from .combine import butterfly_product, diagonal_butterfly
        b = butterfly_product(diagonal_butterfly(b_fft, diag, diag_first=False), b_ifft)
        b.in_size, b.out_size = n, n
        chain = [b]
    if not cplx:
        chain = [Real2Complex()] + chain + [Complex2Real()]
    seq = nn.Sequential(*chain)
    if fused:
        seq = fuse(seq)
    return seq if len(seq) > 1 else seq[0]
