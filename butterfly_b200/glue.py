"""A Butterfly and the element-wise / gather modules around it as ONE kernel launch.

The reference builds its exact transforms as ``nn.Sequential`` chains -- ``FixedPermutation``
(torch_butterfly/permutation.py:65-75), ``Real2Complex`` / ``Complex2Real``
(torch_butterfly/complex_utils.py:100-122), ``Diagonal`` (torch_butterfly/diagonal.py:11-38) around
``Butterfly`` modules (torch_butterfly/special.py: fft, ifft, circulant, ...).  Every link of such a
chain reads and writes all rows in device memory.  Here the forward kernel does the links on the
tile it already holds in shared memory: the real rows are widened as they are loaded, the gather
runs inside the tile before the first factor, the diagonal and the second gather after the last
factor, and only real parts are stored when the chain ends in ``Complex2Real``.

``fuse(sequential)`` rewrites such a chain into ``ButterflyPipeline`` modules (sharing the
parameters of the original); ``butterfly_multiply_glue`` is the differentiable operator.  The
backward composes the existing operators (scatter, multiply backward, scatter): it is not fused.
Rows that do not fit a tile (n > 4096 float32, n > 2048 complex64) run link by link as before.
"""
from typing import Optional

import torch
from torch import nn

from .butterfly import Butterfly
from .complex_utils import Complex2Real, Real2Complex
from .diagonal import Diagonal
from .multiply import butterfly_multiply, butterfly_multiply_bw, butterfly_multiply_fw
from .permutation import FixedPermutation


def _unfused(twiddle, input, increasing_stride, in_perm, out_diag, out_perm, out_real):
    x = input.to(twiddle.dtype)
    if in_perm is not None:
        x = x[..., in_perm.long()]
    y = butterfly_multiply(twiddle, x, increasing_stride)
    if out_diag is not None:
        y = y * out_diag
    if out_perm is not None:
        y = y[..., out_perm.long()]
    return y.real if out_real else y


class _Glue(torch.autograd.Function):
    @staticmethod
    def forward(ctx, twiddle, input, increasing_stride, in_perm, out_diag, out_perm, out_real):
        y = torch.ops.torch_butterfly.butterfly_multiply_glue_fw(twiddle, input, increasing_stride, in_perm, out_diag,
                                                                 out_perm, out_real)
        if y is None:  # a shape the fused launch does not cover: the same links one by one (the backward below fits both)
            with torch.no_grad():
                y = _unfused(twiddle, input, increasing_stride, in_perm, out_diag, out_perm, out_real).contiguous()
        ctx.save_for_backward(twiddle, input, in_perm, out_diag, out_perm)
        ctx.increasing_stride = increasing_stride
        return y

    @staticmethod
    def backward(ctx, grad):
        twiddle, input, in_perm, out_diag, out_perm = ctx.saved_tensors
        inc = ctx.increasing_stride
        g = grad.to(twiddle.dtype)
        if out_perm is not None:  # adjoint of the gather: scatter
            g = torch.empty_like(g).index_copy_(-1, out_perm.long(), g)
        x = input.to(twiddle.dtype)
        if in_perm is not None:
            x = x[..., in_perm.long()]
        d_diag = None
        if out_diag is not None:
            if ctx.needs_input_grad[4]:
                y = butterfly_multiply_fw(twiddle, x, inc)  # the product before the diagonal
                d_diag = (g * y.conj()).sum(dim=(0, 1)) if y.is_complex() else (g * y).sum(dim=(0, 1))
            g = g * out_diag.conj() if out_diag.is_complex() else g * out_diag
        d_twiddle, d_x = butterfly_multiply_bw(twiddle, x, g.contiguous(), inc)
        if in_perm is not None:
            d_x = torch.empty_like(d_x).index_copy_(-1, in_perm.long(), d_x)
        if not input.is_complex() and d_x.is_complex():
            d_x = d_x.real
        return d_twiddle, d_x, None, None, d_diag, None, None


def butterfly_multiply_glue(twiddle: torch.Tensor, input: torch.Tensor, increasing_stride: bool,
                            in_perm: Optional[torch.Tensor] = None, out_diag: Optional[torch.Tensor] = None,
                            out_perm: Optional[torch.Tensor] = None, out_real: bool = False) -> torch.Tensor:
    """real(  ( butterfly(twiddle) @ complex(input)[..., in_perm] * out_diag )[..., out_perm]  ), each
    link optional, as one launch.  input (batch, nstacks, n) with the dtype of twiddle, or float32
    for a complex twiddle; in_perm / out_perm int32 vectors of n entries; out_diag n entries."""
    n = 1 << twiddle.shape[2]
    limit = 2048 if twiddle.is_complex() else 4096
    if n > limit or input.shape[-1] != n or not input.is_cuda:
        return _unfused(twiddle, input, increasing_stride, in_perm, out_diag, out_perm, out_real)
    return _Glue.apply(twiddle, input, increasing_stride, in_perm, out_diag, out_perm, out_real)


class ButterflyPipeline(nn.Module):
    """[Real2Complex] [FixedPermutation] Butterfly [Diagonal] [FixedPermutation] [Complex2Real] as one
    module and one launch.  The Butterfly (square, single stack, no bias) and the Diagonal are the
    given modules, so their parameters stay shared with whoever else holds them."""

    def __init__(self, butterfly: Butterfly, in_perm: Optional[torch.Tensor] = None, diagonal: Optional[Diagonal] = None,
                 out_perm: Optional[torch.Tensor] = None, real_in: bool = False, real_out: bool = False):
        super().__init__()
        assert butterfly.nstacks == 1 and butterfly.bias is None and butterfly.in_size == butterfly.n == butterfly.out_size
        assert butterfly.complex or not (real_in or real_out)
        self.butterfly = butterfly
        self.diagonal = diagonal
        self.real_in, self.real_out = real_in, real_out
        self.register_buffer("in_perm", None if in_perm is None else in_perm.to(torch.int32))
        self.register_buffer("out_perm", None if out_perm is None else out_perm.to(torch.int32))

    def forward(self, input):
        b = self.butterfly
        rows = input.reshape(-1, 1, b.n)
        if not self.real_in and b.complex and not rows.is_complex():
            rows = rows.to(b.twiddle.dtype)
        diag = None if self.diagonal is None else self.diagonal.diagonal
        y = butterfly_multiply_glue(b.twiddle, rows, b.increasing_stride, self.in_perm, diag, self.out_perm, self.real_out)
        return y.reshape(*input.shape[:-1], b.n)


def _fusible_butterfly(m) -> bool:
    return (type(m) is Butterfly and m.nstacks == 1 and m.bias is None and m.in_size == m.n == m.out_size
            and m.twiddle.dtype in (torch.float32, torch.complex64))


def fuse(chain: nn.Sequential) -> nn.Sequential:
    """The same function as `chain` with every run of
    [Real2Complex] [FixedPermutation] Butterfly [Diagonal] [FixedPermutation] [Complex2Real]
    replaced by one ButterflyPipeline.  Links that do not fit the pattern are kept as they are."""
    mods = list(chain)
    out, i = [], 0
    while i < len(mods):
        j, real_in, in_perm = i, False, None
        if isinstance(mods[j], Real2Complex) and j + 1 < len(mods):
            real_in, j = True, j + 1
        if isinstance(mods[j], FixedPermutation) and j + 1 < len(mods):
            in_perm, j = mods[j].permutation, j + 1
        if not _fusible_butterfly(mods[j]) or (real_in and not mods[j].complex) or (
                in_perm is not None and in_perm.shape[-1] != mods[j].n):
            out.append(mods[i])
            i += 1
            continue
        b, j = mods[j], j + 1
        diagonal, out_perm, real_out = None, None, False
        if j < len(mods) and isinstance(mods[j], Diagonal) and mods[j].diagonal.shape == (b.n,) \
                and mods[j].diagonal.dtype == b.twiddle.dtype:
            diagonal, j = mods[j], j + 1
        if j < len(mods) and isinstance(mods[j], FixedPermutation) and mods[j].permutation.shape[-1] == b.n:
            out_perm, j = mods[j].permutation, j + 1
        if j < len(mods) and isinstance(mods[j], Complex2Real) and b.complex:
            real_out, j = True, j + 1
        out.append(ButterflyPipeline(b, in_perm, diagonal, out_perm, real_in, real_out))
        i = j
    return nn.Sequential(*out)
