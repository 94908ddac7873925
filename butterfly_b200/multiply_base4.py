"""Base-4 (radix-4) butterfly multiply.

The reference computes this product with PyTorch view/permute/sum calls only
(``torch_butterfly/multiply_base4.py:7-41``); here it is a native operator with its own
backward.  ``twiddle_base2_to_base4`` (``multiply_base4.py:44-71`` there) is set-up time
parameter algebra and stays in PyTorch.

    twiddle4: (nstacks, nblocks, log_n // 2, n/4, 4, 4)
    twiddle2: (nstacks, nblocks, log_n % 2,  n/2, 2, 2)
"""
from typing import Optional, Tuple

import torch


def butterfly_multiply_base4_fw(twiddle4, twiddle2, input, increasing_stride: bool = True,
                                output_size: Optional[int] = None) -> torch.Tensor:
    return torch.ops.torch_butterfly.butterfly_multiply_base4_fw(twiddle4, twiddle2, input, increasing_stride,
                                                                 output_size)


def butterfly_multiply_base4_bw(twiddle4, twiddle2, input, grad,
                                increasing_stride: bool = True) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (d_twiddle4, d_twiddle2, d_input)."""
    return torch.ops.torch_butterfly.butterfly_multiply_base4_bw(twiddle4, twiddle2, input, grad, increasing_stride)


def butterfly_multiply_base4(twiddle4, twiddle2, input, increasing_stride: bool = True,
                             output_size: Optional[int] = None) -> torch.Tensor:
    """Differentiable base-4 product; same call signature as the reference's
    ``butterfly_multiply_base4_torch``."""
    return torch.ops.torch_butterfly.butterfly_multiply_base4(twiddle4, twiddle2, input, increasing_stride,
                                                              output_size)


def twiddle_base2_to_base4(twiddle: torch.Tensor, increasing_stride: bool = True):
    """Fuse consecutive pairs of radix-2 factors into radix-4 factors.

    For every block, factors (2i, 2i+1) act on the bit pair (b, b+1) (b = 2i when the block
    runs with increasing stride, log_n-2-2i otherwise).  Their product restricted to the four
    positions {base + j*stride, j = 0..3} is the 4x4 matrix returned in ``twiddle4``; when
    log_n is odd the last factor of each block is returned unchanged in ``twiddle2``.
    """
    nstacks, nblocks, log_n = twiddle.shape[:3]
    n = 1 << log_n
    assert twiddle.shape == (nstacks, nblocks, log_n, n // 2, 2, 2)
    twiddle2 = (twiddle[:, :, -1:] if log_n % 2 == 1
                else twiddle.new_empty(nstacks, nblocks, 0, n // 2, 2, 2))
    twiddle4 = twiddle.new_empty(nstacks, nblocks, log_n // 2, n // 4, 4, 4)
    inc = increasing_stride
    for block in range(nblocks):
        for idx in range(log_n // 2):
            b = 2 * idx if inc else log_n - 2 - 2 * idx
            s = 1 << b
            # pair index i of a radix-2 factor on bit beta is the position with bit beta removed.
            # View both factors as (groups g, hi/lo bit h, offset k, 2, 2).
            first = twiddle[:, block, 2 * idx]        # acts first
            second = twiddle[:, block, 2 * idx + 1]   # acts second
            if inc:   # first on bit b (pairs j0), second on bit b+1 (pairs j1)
                # first:  index = g*2s + j1*s + k  -> (g, j1, k);  second: index = g*2s + j0*s + k -> (g, j0, k)
                f = first.reshape(nstacks, n // (4 * s), 2, s, 2, 2)    # [g, j1, k, r, c]: y[j0=r] from x[j0=c]
                g2 = second.reshape(nstacks, n // (4 * s), 2, s, 2, 2)  # [g, j0, k, r, c]: z[j1=r] from y[j1=c]
                # out[(r1,r0),(c1,c0)] = second[g, j0=r0, k, r1, c1] * first[g, j1=c1, k, r0, c0]
                prod = torch.einsum('sgakbc,sgckad->sgkbacd', g2, f)
            else:     # first on bit b+1, second on bit b
                f = first.reshape(nstacks, n // (4 * s), 2, s, 2, 2)    # [g, j0, k, r, c] on j1
                g2 = second.reshape(nstacks, n // (4 * s), 2, s, 2, 2)  # [g, j1, k, r, c] on j0
                # out[(r1,r0),(c1,c0)] = second[g, j1=r1, k, r0, c0] * first[g, j0=c0, k, r1, c1]
                prod = torch.einsum('sgbkad,sgdkbc->sgkbacd', g2, f)
            twiddle4[:, block, idx].copy_(prod.reshape(nstacks, n // 4, 4, 4))
        inc = not inc
    return twiddle4, twiddle2
