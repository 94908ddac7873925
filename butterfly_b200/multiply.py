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


def butterfly_linear(twiddle: torch.Tensor, input: torch.Tensor, bias: Optional[torch.Tensor], increasing_stride: bool,
                     out_size: int) -> torch.Tensor:
    """Butterfly as a linear layer, fused (float32): ``input`` (batch, in_size) is shared by all stacks,
    the result is the first ``out_size`` columns of the stacks' outputs side by side plus ``bias``.
    Replaces the expand / flatten / slice / bias-add glue of the reference's module
    (torch_butterfly/butterfly.py:152-169) and, in the backward, the reductions autograd derives
    from it (input gradient summed over the stacks, bias gradient)."""
    return torch.ops.torch_butterfly.butterfly_linear(twiddle, input, bias, increasing_stride, out_size)


def butterfly_linear_fw(twiddle: torch.Tensor, input: torch.Tensor, bias: Optional[torch.Tensor], increasing_stride: bool,
                        out_size: int) -> torch.Tensor:
    return torch.ops.torch_butterfly.butterfly_linear_fw(twiddle, input, bias, increasing_stride, out_size)


def butterfly_linear_bw(twiddle: torch.Tensor, input: torch.Tensor, grad: torch.Tensor, increasing_stride: bool,
                        need_bias: bool = True) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (d_twiddle, d_input (batch, in_size), d_bias (out_size))."""
    return torch.ops.torch_butterfly.butterfly_linear_bw(twiddle, input, grad, increasing_stride, need_bias)


def unitary_twiddle(angles: torch.Tensor) -> torch.Tensor:
    """(..., 4) float32 angles (phi, alpha, psi, chi) -> (..., 2, 2) complex64 unitary blocks
    [[cos(phi) e^{i(alpha+psi)}, sin(phi) e^{i(alpha+chi)}], [-sin(phi) e^{i(alpha-chi)}, cos(phi) e^{i(alpha-psi)}]],
    differentiable; one kernel each way in place of the cos / sin / stack chain of the reference's
    ButterflyUnitary.forward (torch_butterfly/butterfly.py:271-280)."""
    return torch.ops.torch_butterfly.unitary_twiddle(angles)


def unitary_twiddle_fw(angles: torch.Tensor) -> torch.Tensor:
    return torch.ops.torch_butterfly.unitary_twiddle_fw(angles)


def unitary_twiddle_bw(angles: torch.Tensor, grad: torch.Tensor) -> torch.Tensor:
    """Gradient of the angles for the gradient ``grad`` (..., 2, 2) of the blocks."""
    return torch.ops.torch_butterfly.unitary_twiddle_bw(angles, grad)
