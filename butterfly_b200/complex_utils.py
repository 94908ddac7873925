"""Real / complex conversions and last-dimension gathers as modules.

Counterparts in the reference: ``Real2Complex``, ``Complex2Real``, ``real2complex``,
``index_last_dim`` (torch_butterfly/complex_utils.py:100-142).  On their own each is a pass over
the rows; ``butterfly_b200.glue.fuse`` folds them into the neighbouring Butterfly's launch.
"""
import torch
from torch import nn

_COMPLEX = {torch.float32: torch.complex64, torch.float64: torch.complex128}


def real2complex(x: torch.Tensor) -> torch.Tensor:
    """Real tensor -> complex tensor with zero imaginary part (autograd returns the real part of the gradient)."""
    return x if x.is_complex() else x.to(_COMPLEX[x.dtype])


def index_last_dim(x: torch.Tensor, permutation: torch.Tensor) -> torch.Tensor:
    """x[..., permutation]."""
    return x[..., permutation]


class Real2Complex(nn.Module):
    def forward(self, input):
        return real2complex(input)


class Complex2Real(nn.Module):
    def forward(self, input):
        return input.real
