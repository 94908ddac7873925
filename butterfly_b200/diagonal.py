"""Learnable diagonal matrix.  Counterpart in the reference: ``Diagonal``
(torch_butterfly/diagonal.py:11-38)."""
import torch
from torch import nn

_COMPLEX = {torch.float32: torch.complex64, torch.float64: torch.complex128}


class Diagonal(nn.Module):
    """input (..., size) -> input * diagonal.  Either a size (random normal init) or an initial vector."""

    def __init__(self, size=None, complex=False, diagonal_init=None):
        super().__init__()
        if diagonal_init is not None:
            self.size = diagonal_init.shape
            self.diagonal = nn.Parameter(diagonal_init.detach().clone())
            self.complex = self.diagonal.is_complex()
        else:
            assert size is not None
            self.size = size
            dtype = torch.get_default_dtype()
            self.diagonal = nn.Parameter(torch.randn(size, dtype=_COMPLEX[dtype] if complex else dtype))
            self.complex = complex

    def forward(self, input):
        return input * self.diagonal
