"""Kaleidoscope-operator 2-D convolution layer.

Counterpart in the reference: ``KOP2d`` (convolution/models/kops.py:15-100): a convolution
computed as K2( K1(x) * Kd(weight) ) where K1, Kd, K2 are learnable 2-D butterfly maps
initialised to the 2-D FFT / inverse FFT (without bit reversal: the permutations cancel) or to
random orthogonal factors.  Each of the three maps is a ``combine.TensorProduct`` and runs as ONE
butterfly multiply over the flattened image; the channel contraction between them is a batched
complex GEMM (torch.einsum, a library GEMM).
"""
import math

import torch
from torch import nn

from .butterfly import Butterfly
from .combine import TensorProduct
from .permutation import bitreversal_permutation


class KOP2d(nn.Module):
    """in_size: image size (int or (h, w), powers of two); in_ch / out_ch: channels; kernel_size: int or pair.
    init 'fft' starts as an exact circular convolution with `weight` (zero_pad=True centres the
    kernel like Conv2d's padding = (k - 1) // 2 by a phase ramp folded into Kd), 'ortho' as random
    orthogonal butterflies.  base 4 converts the maps to radix-4 layers (two-pass execution)."""

    def __init__(self, in_size, in_ch, out_ch, kernel_size, complex=True, init="ortho", nblocks=1, base=2, zero_pad=True):
        super().__init__()
        self.in_size = (in_size, in_size) if isinstance(in_size, int) else tuple(in_size)
        self.kernel_size = (kernel_size, kernel_size) if isinstance(kernel_size, int) else tuple(kernel_size)
        self.in_ch, self.out_ch, self.complex, self.nblocks, self.base, self.zero_pad = in_ch, out_ch, complex, nblocks, base, zero_pad
        assert init in ("ortho", "fft") and base in (2, 4)
        assert init != "fft" or complex, "fft init requires complex=True"
        self.init = init
        self.padding = ((self.kernel_size[0] - 1) // 2, (self.kernel_size[1] - 1) // 2)
        conv = nn.Conv2d(in_ch, out_ch, self.kernel_size, padding=self.padding, bias=False)  # for its weight initialisation
        self.weight = nn.Parameter(conv.weight.detach().flip([-1, -2]).clone())
        h, w = self.in_size

        def pair(increasing_stride, kind):
            return TensorProduct(
                Butterfly(w, w, bias=False, complex=complex, increasing_stride=increasing_stride, init=kind, nblocks=nblocks),
                Butterfly(h, h, bias=False, complex=complex, increasing_stride=increasing_stride, init=kind, nblocks=nblocks))
        kinds = ["ortho"] * 3 if init == "ortho" else ["fft_no_br", "fft_no_br", "ifft_no_br"]
        self.Kd, self.K1, self.K2 = pair(False, kinds[0]), pair(False, kinds[1]), pair(True, kinds[2])
        with torch.no_grad():
            self.Kd.map1 *= math.sqrt(w)
            self.Kd.map2 *= math.sqrt(h)
            if zero_pad and complex:
                # shift theorem: rolling the kernel by -padding multiplies its spectrum by a phase ramp;
                # the spectrum comes out bit-reversed, and the ramp goes into the rows of the last factor of the first block
                for m, n, pad in ((self.Kd.map1, w, self.padding[1]), (self.Kd.map2, h, self.padding[0])):
                    ramp = torch.exp(2j * math.pi / n * pad * torch.arange(n))[bitreversal_permutation(n)].to(m.twiddle.dtype)
                    m.twiddle[:, 0, -1, :, 0, :] *= ramp[0::2].unsqueeze(-1)
                    m.twiddle[:, 0, -1, :, 1, :] *= ramp[1::2].unsqueeze(-1)
        if base == 4:
            for tp in (self.Kd, self.K1, self.K2):
                tp.map1, tp.map2 = tp.map1.to_base4(), tp.map2.to_base4()

    def forward(self, x):
        """x (batch, in_ch, h, w) real -> (batch, out_ch, h, w) real."""
        cplx = torch.complex64 if x.dtype == torch.float32 else torch.complex128
        x_f = self.K1(x.to(cplx) if self.complex else x)
        w_f = self.Kd(self.weight.to(cplx) if self.complex else self.weight)
        prod = torch.einsum("bihw,oihw->bohw", x_f, w_f)  # per frequency: (batch, in_ch) x (in_ch, out_ch)
        out = self.K2(prod)
        return out.real if self.complex else out
