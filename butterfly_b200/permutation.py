"""Index permutations used by the exact-transform constructions.

Counterparts in the reference: ``bitreversal_permutation`` and ``FixedPermutation``
(torch_butterfly/permutation.py:15-26, 58-75).
"""
import math

import torch
from torch import nn


def bitreversal_permutation(n: int) -> torch.Tensor:
    """perm[i] = i with its log2(n) bits reversed, as a LongTensor (n a power of two)."""
    log_n = int(math.log2(n))
    assert n == 1 << log_n, "n must be a power of 2"
    idx = torch.arange(n)
    out = torch.zeros(n, dtype=torch.long)
    for b in range(log_n):
        out |= ((idx >> b) & 1) << (log_n - 1 - b)
    return out


class FixedPermutation(nn.Module):
    """Gather along the last dimension with a fixed index vector: out[..., i] = x[..., perm[i]]."""

    def __init__(self, permutation: torch.Tensor) -> None:
        super().__init__()
        self.register_buffer("permutation", permutation.long())

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return input[..., self.permutation]
