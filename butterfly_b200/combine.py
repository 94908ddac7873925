"""Butterflies combined with diagonals, with each other, and as 2-D (tensor product) maps.

Counterparts in the reference: ``diagonal_butterfly``, ``butterfly_product``, ``TensorProduct``,
``butterfly_kronecker``, ``permutation_kronecker``, ``flip_increasing_stride``
(torch_butterfly/combine.py:11-159).

What is new here is the execution of ``TensorProduct``.  The reference applies map1 along the
last dimension, transposes, applies map2, and transposes back: two passes of the multiply over the
data plus two strided copies.  When both maps are butterflies of the same direction and block
count, the 2-D map on (n2, n1) images IS one butterfly of size n2 * n1 on the flattened image:
the factors of map1 act on the low log2(n1) bits of the flat index, the factors of map2 on the
high log2(n2) bits, the two sets commute, and inside each block they line up as one monotone run
of strides.  ``kronecker_twiddle`` builds that butterfly's twiddle from the two small ones with
expand / cat only (so autograd sums the gradient back onto the two parameters), and the data
makes ONE pass through the multiply kernel: no transposes, one read and one write of the image.
"""
import copy

import torch
from torch import nn
from torch.nn import functional as F

from .butterfly import Butterfly
from .multiply import butterfly_multiply
from .permutation import FixedPermutation, bitreversal_permutation


def _last_block_increasing(b: Butterfly) -> bool:
    return b.increasing_stride != ((b.nblocks - 1) % 2 == 1)


def diagonal_butterfly(butterfly: Butterfly, diagonal: torch.Tensor, diag_first: bool, inplace: bool = True) -> Butterfly:
    """Fold a diagonal matrix into the first (diag_first: x -> diag -> butterfly) or last
    (x -> butterfly -> diag) factor of a bias-free single-stack Butterfly.  A diagonal shorter
    than n is extended with ones."""
    assert butterfly.nstacks == 1 and butterfly.bias is None
    out = butterfly if inplace else copy.deepcopy(butterfly)
    n = out.n
    d = diagonal.to(out.twiddle.device)
    if d.shape[-1] < n:
        d = F.pad(d, (0, n - d.shape[-1]), value=1)
    with torch.no_grad():
        tw = out.twiddle
        if diag_first:
            # the first factor pairs positions (2i, 2i+1) when it has stride 1, (i, i + n/2) when it has stride n/2;
            # a diagonal before the factor scales the COLUMNS of each 2x2 block
            lo, hi = (d[0::2], d[1::2]) if out.increasing_stride else (d[:n // 2], d[n // 2:])
            tw[:, 0, 0, :, :, 0] *= lo.unsqueeze(-1)
            tw[:, 0, 0, :, :, 1] *= hi.unsqueeze(-1)
        else:
            # a diagonal after the last factor scales the ROWS of each 2x2 block
            lo, hi = (d[:n // 2], d[n // 2:]) if _last_block_increasing(out) else (d[0::2], d[1::2])
            tw[:, -1, -1, :, 0, :] *= lo.unsqueeze(-1)
            tw[:, -1, -1, :, 1, :] *= hi.unsqueeze(-1)
    return out


def butterfly_product(butterfly1: Butterfly, butterfly2: Butterfly) -> Butterfly:
    """x -> butterfly2(butterfly1(x)) as one Butterfly whose blocks are those of the two, with an
    identity block in between when the directions would not alternate."""
    assert butterfly1.bias is None and butterfly2.bias is None
    assert butterfly1.complex == butterfly2.complex and butterfly1.nstacks == butterfly2.nstacks
    assert butterfly1.log_n == butterfly2.log_n
    tw1, tw2 = butterfly1.twiddle.detach(), butterfly2.twiddle.detach()
    if _last_block_increasing(butterfly1) == butterfly2.increasing_stride:
        # the next block must run the other way: put an identity block between the two
        eye = torch.eye(2, dtype=tw1.dtype, device=tw1.device).expand(tw1.shape[0], 1, *tw1.shape[2:])
        tw1 = torch.cat((tw1, eye), dim=1)
    tw = torch.cat((tw1, tw2.to(tw1.device)), dim=1).contiguous()
    n = 1 << butterfly1.log_n
    out = Butterfly(n, n, bias=False, complex=butterfly1.complex, increasing_stride=butterfly1.increasing_stride,
                    init=tw.cpu(), nblocks=tw.shape[1]).to(tw.device)
    out.in_size, out.out_size = butterfly1.in_size, butterfly2.out_size
    return out


def kronecker_twiddle(twiddle1: torch.Tensor, twiddle2: torch.Tensor, increasing_stride: bool) -> torch.Tensor:
    """Twiddle (S, nblocks, log_n1 + log_n2, n1 n2 / 2, 2, 2) of the butterfly that applies the
    butterfly of twiddle1 (size n1) along the low bits and that of twiddle2 (size n2) along the high
    bits of a flat index of n2 * n1 positions.  Both have the same stack and block counts and the
    same direction.  Built from views and one cat, so gradients flow back to both."""
    S, nb, l1, h1 = twiddle1.shape[:4]
    S2, nb2, l2, h2 = twiddle2.shape[:4]
    assert (S, nb) == (S2, nb2) and twiddle1.dtype == twiddle2.dtype
    n1, n2 = 2 * h1, 2 * h2
    # a factor of map1 pairs positions inside a row of the image: pair index = row * n1/2 + own pair index
    t1 = twiddle1.unsqueeze(3).expand(S, nb, l1, n2, h1, 2, 2).reshape(S, nb, l1, n2 * h1, 2, 2)
    # a factor of map2 pairs rows: pair index = own pair index * n1 + column
    t2 = twiddle2.unsqueeze(4).expand(S, nb, l2, h2, n1, 2, 2).reshape(S, nb, l2, h2 * n1, 2, 2)
    blocks = []
    for j in range(nb):
        inc = increasing_stride != (j % 2 == 1)
        blocks.append(torch.cat((t1[:, j], t2[:, j]) if inc else (t2[:, j], t1[:, j]), dim=1))
    return torch.stack(blocks, dim=1)


def butterfly_kronecker(butterfly1: Butterfly, butterfly2: Butterfly) -> Butterfly:
    """The Kronecker product butterfly2 (x) butterfly1 as one Butterfly of size n1 * n2 acting on
    flattened (n2, n1) inputs (any block count; the reference supports one block)."""
    assert butterfly1.increasing_stride == butterfly2.increasing_stride and butterfly1.complex == butterfly2.complex
    assert butterfly1.bias is None and butterfly2.bias is None
    assert butterfly1.nstacks == 1 and butterfly2.nstacks == 1 and butterfly1.nblocks == butterfly2.nblocks
    tw = kronecker_twiddle(butterfly1.twiddle.detach(), butterfly2.twiddle.detach(), butterfly1.increasing_stride).contiguous()
    n = butterfly1.n * butterfly2.n
    out = Butterfly(n, n, bias=False, complex=butterfly1.complex, increasing_stride=butterfly1.increasing_stride,
                    init=tw.cpu(), nblocks=butterfly1.nblocks).to(tw.device)
    out.in_size = butterfly1.in_size * butterfly2.in_size
    out.out_size = butterfly1.out_size * butterfly2.out_size
    return out


class TensorProduct(nn.Module):
    """map1 on the last dimension, then map2 on the next to last: input (*, n2, n1) -> (*, n2', n1').

    Two plain square Butterfly layers of the same direction and block count run as ONE multiply of
    size n2 * n1 (see the module docstring); anything else runs as the reference does, one map
    after the other around a transpose.  ``fused`` = False forces the two-pass form."""

    def __init__(self, map1, map2, fused: bool = True) -> None:
        super().__init__()
        self.map1 = map1
        self.map2 = map2
        self.fused = fused

    def fusible(self) -> bool:
        a, b = self.map1, self.map2
        if type(a) is not Butterfly or type(b) is not Butterfly:
            return False
        square = all(m.in_size == m.n and m.out_size == m.n and m.bias is None and m.nstacks == 1 for m in (a, b))
        return (square and a.complex == b.complex and a.increasing_stride == b.increasing_stride
                and a.nblocks == b.nblocks and a.log_n + b.log_n <= 24)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        a, b = self.map1, self.map2
        if self.fused and self.fusible() and input.is_cuda and input.dtype == a.twiddle.dtype:
            assert input.shape[-1] <= a.n and input.shape[-2] <= b.n
            if input.shape[-1] < a.n or input.shape[-2] < b.n:  # the operator's zero padding, per dimension
                input = F.pad(input, (0, a.n - input.shape[-1], 0, b.n - input.shape[-2]))
            tw = kronecker_twiddle(a.twiddle, b.twiddle, a.increasing_stride)
            rows = input.reshape(-1, 1, a.n * b.n)
            return butterfly_multiply(tw, rows, a.increasing_stride).reshape(input.shape)
        out = a(input)
        return b(out.transpose(-1, -2)).transpose(-1, -2)


def permutation_kronecker(perm1: FixedPermutation, perm2: FixedPermutation) -> FixedPermutation:
    """The permutation of flattened (n2, n1) inputs that applies perm1 inside rows and perm2 to the rows."""
    p1, p2 = perm1.permutation, perm2.permutation
    n1 = p1.shape[-1]
    return FixedPermutation((p2.unsqueeze(1) * n1 + p1.unsqueeze(0)).reshape(-1))


def flip_increasing_stride(butterfly: Butterfly) -> nn.Module:
    """The same matrix with the opposite stride direction: bit-reverse the input, run the factors
    with their pair indices bit-reversed, bit-reverse the output."""
    assert butterfly.bias is None and butterfly.in_size == butterfly.n and butterfly.out_size == butterfly.n
    n = butterfly.n
    new = copy.deepcopy(butterfly)
    new.increasing_stride = not butterfly.increasing_stride
    half = bitreversal_permutation(n // 2).to(new.twiddle.device) if n > 2 else torch.zeros(1, dtype=torch.long, device=new.twiddle.device)
    with torch.no_grad():
        new.twiddle.copy_(new.twiddle[:, :, :, half])
    br = bitreversal_permutation(n)
    return nn.Sequential(FixedPermutation(br), new, FixedPermutation(br))
