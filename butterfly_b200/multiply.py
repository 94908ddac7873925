"""Functional interface of the radix-2 butterfly multiply.

Mirrors ``torch_butterfly/multiply.py:8-24`` of the reference: three thin wrappers over
the registered operators, same names, argument order and defaults.

    twiddle: (nstacks, nblocks, log_n, n/2, 2, 2)
    input:   (batch_size, nstacks, input_size)   zero-padded / trimmed to n columns
    output:  (batch_size, nstacks, output_size)  output_size defaults to n
"""
from typing import Optional, Tuple

import torch


def butterfly_multiply_fw(twiddle: torch.Tensor, input: torch.Tensor, increasing_stride: bool,
                          output_size: Optional[int] = None) -> torch.Tensor:
    """Forward only (no autograd graph)."""
    return torch.ops.torch_butterfly.butterfly_multiply_fw(twiddle, input, increasing_stride, output_size)


def butterfly_multiply_bw(twiddle: torch.Tensor, input: torch.Tensor, grad: torch.Tensor,
                          increasing_stride: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (d_twiddle, d_input) for the output gradient ``grad``."""
    return torch.ops.torch_butterfly.butterfly_multiply_bw(twiddle, input, grad, increasing_stride)


def butterfly_multiply(twiddle: torch.Tensor, input: torch.Tensor, increasing_stride: bool,
                       output_size: Optional[int] = None) -> torch.Tensor:
    """Differentiable product of the nblocks * log_n butterfly factors with ``input``."""
    return torch.ops.torch_butterfly.butterfly_multiply(twiddle, input, increasing_stride, output_size)
