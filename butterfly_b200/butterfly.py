"""nn.Module layers on top of the butterfly multiply operators.

Same constructor arguments, parameter names/shapes and forward() flags as the reference's
``Butterfly`` / ``ButterflyUnitary`` / ``ButterflyBmm`` (torch_butterfly/butterfly.py:15-397)
and ``ButterflyBase4`` (torch_butterfly/butterfly_base4.py:12-72), so state dicts carry over.
The layers run on CUDA tensors only: the operators underneath have no CPU path.
"""
import math
import numbers

import torch
from torch import nn

from .multiply import butterfly_linear, butterfly_multiply, unitary_twiddle
from .multiply_base4 import butterfly_multiply_base4, twiddle_base2_to_base4

_COMPLEX = {torch.float32: torch.complex64, torch.float64: torch.complex128}


def _as_rows(x, width):
    """(..., width) -> (N, width); complex tensors cannot be .view()ed when strided, so reshape."""
    return x.reshape(-1, width)


def _random_orthogonal_twiddle(core_shape, complex):
    """2x2 blocks drawn from O(2) (rotations/reflections) or from the Haar measure on U(2)."""
    if not complex:
        theta = torch.rand(core_shape) * 2 * math.pi
        c, s = torch.cos(theta), torch.sin(theta)
        det = torch.randint(0, 2, core_shape, dtype=c.dtype) * 2 - 1
        return torch.stack((torch.stack((det * c, -det * s), dim=-1), torch.stack((s, c), dim=-1)), dim=-2)
    phi = torch.asin(torch.sqrt(torch.rand(core_shape)))
    c, s = torch.cos(phi), torch.sin(phi)
    alpha, psi, chi = torch.rand((3,) + tuple(core_shape)) * 2 * math.pi
    a = torch.exp(1j * (alpha + psi)) * c
    b = torch.exp(1j * (alpha + chi)) * s
    cc = -torch.exp(1j * (alpha - chi)) * s
    d = torch.exp(1j * (alpha - psi)) * c
    return torch.stack((torch.stack((a, b), dim=-1), torch.stack((cc, d), dim=-1)), dim=-2)


class Butterfly(nn.Module):
    """Product of nblocks * log2(n) butterfly factors; a drop-in for ``nn.Linear(in_size, out_size)``.

    in_size is rounded up to n = 2^ceil(log2 in_size) (the input is zero-padded inside the
    operator); out_size > n is served by ceil(out_size / n) independent stacks.
    init: 'randn', 'ortho', 'identity', 'fft_no_br', 'ifft_no_br', 'empty', or a twiddle tensor.
    """

    def __init__(self, in_size, out_size, bias=True, complex=False, increasing_stride=True, init="randn",
                 nblocks=1):
        super().__init__()
        self._configure(in_size, out_size, complex, increasing_stride, nblocks)
        dtype = self._dtype()
        shape = (self.nstacks, nblocks, self.log_n, self.n // 2, 2, 2)
        self._make_params(shape, dtype, init, (out_size,) if bias else None)
        self.reset_parameters()

    # ---- construction helpers shared by the subclasses
    def _configure(self, in_size, out_size, complex, increasing_stride, nblocks):
        assert nblocks >= 1
        self.in_size = in_size
        self.log_n = max(1, int(math.ceil(math.log2(in_size))))
        self.n = 1 << self.log_n
        self.out_size = out_size
        self.nstacks = int(math.ceil(out_size / self.n))
        self.complex = complex
        self.increasing_stride = increasing_stride
        self.nblocks = nblocks

    def _dtype(self):
        d = torch.get_default_dtype()
        return _COMPLEX[d] if self.complex else d

    def _make_params(self, shape, dtype, init, bias_shape):
        if isinstance(init, torch.Tensor):
            assert init.shape == shape and init.dtype == dtype
            self.init = None
            self.twiddle = nn.Parameter(init.clone())
        else:
            assert init in ("empty", "randn", "ortho", "identity", "fft_no_br", "ifft_no_br")
            self.init = init
            self.twiddle = nn.Parameter(torch.empty(shape, dtype=dtype))
        self.twiddle._is_structured = True  # optimizers may exclude structured weights from weight decay
        if bias_shape is not None:
            self.bias = nn.Parameter(torch.empty(bias_shape, dtype=dtype))
        else:
            self.register_parameter("bias", None)

    def reset_parameters(self):
        if self.bias is not None:
            bound = 1 / math.sqrt(self.in_size)
            nn.init.uniform_(self.bias, -bound, bound)
        tw = self.twiddle
        with torch.no_grad():
            if self.init in (None, "empty"):
                return
            if self.init == "randn":
                tw.copy_(torch.randn(tw.shape, dtype=tw.dtype) / math.sqrt(2))
            elif self.init == "ortho":
                tw.copy_(_random_orthogonal_twiddle(tw.shape[:-2], self.complex))
            elif self.init == "identity":
                tw.copy_(torch.eye(2, dtype=tw.dtype).expand(tw.shape))
            else:  # fft_no_br / ifft_no_br: first block is the (i)FFT without bit reversal, the rest identity
                assert self.complex, "fft_no_br / ifft_no_br need a complex Butterfly"
                from . import special
                tw.copy_(torch.eye(2, dtype=tw.dtype).expand(tw.shape))
                tw[:, 0] = special.fft_twiddle(self.n, inverse=self.init == "ifft_no_br", normalized=True,
                                               br_first=self.increasing_stride, dtype=tw.dtype)[0, 0]

    # ---- forward
    def _effective_twiddle(self):
        return self.twiddle

    def forward(self, input, transpose=False, conjugate=False, subtwiddle=False):
        """input (..., in_size) -> (..., out_size).

        transpose / conjugate apply the transposed / conjugated matrix; subtwiddle uses the
        leading part of the parameters for a shorter input (the output then has the n' columns of
        the first stack, as in the reference: torch_butterfly/butterfly.py:147-150)."""
        twiddle = self._effective_twiddle()
        if (not subtwiddle and twiddle.dtype == torch.float32 and input.dtype == torch.float32 and input.is_cuda
                and type(self).pre_process is Butterfly.pre_process and type(self).post_process is Butterfly.post_process):
            # real float32 layer: one fused operator instead of expand / multiply / flatten / slice / bias
            inc = self.increasing_stride
            if transpose:
                twiddle = twiddle.transpose(-1, -2).flip([1, 2])
                inc = not (self.increasing_stride != ((self.nblocks - 1) % 2 == 1))
            rows = _as_rows(input, input.size(-1))
            out = butterfly_linear(twiddle, rows, self.bias, inc, self.out_size)
            return out.reshape(*input.shape[:-1], self.out_size)
        rows = self.pre_process(input)
        output_size = self.out_size if self.nstacks == 1 else None
        if subtwiddle:
            log_n = max(1, int(math.ceil(math.log2(input.size(-1)))))
            n = 1 << log_n
            twiddle = twiddle[:, :, :log_n, :n // 2] if self.increasing_stride else twiddle[:, :, -log_n:, :n // 2]
            output_size = None
        if conjugate and self.complex:
            twiddle = twiddle.conj()
        if not transpose:
            out = butterfly_multiply(twiddle, rows, self.increasing_stride, output_size)
        else:
            # (B_k ... B_1)^T = B_1^T ... B_k^T: reverse blocks and factors, transpose every 2x2
            twiddle = twiddle.transpose(-1, -2).flip([1, 2])
            last_increasing = self.increasing_stride != ((self.nblocks - 1) % 2 == 1)
            out = butterfly_multiply(twiddle, rows, not last_increasing, output_size)
        return self.post_process(input, out, out_size=out.size(-1) if subtwiddle else None)

    def pre_process(self, input):
        rows = _as_rows(input, input.size(-1))
        return rows.unsqueeze(1).expand(rows.shape[0], self.nstacks, rows.shape[1])  # stack stride 0, no copy

    def post_process(self, input, output, out_size=None):
        out_size = self.out_size if out_size is None else out_size
        batch = output.shape[0]
        output = output.reshape(batch, self.nstacks * output.size(-1))
        if out_size != output.shape[-1]:
            output = output[:, :out_size]
        if self.bias is not None:
            output = output + self.bias[:out_size]
        return output.reshape(*input.shape[:-1], out_size)

    def __imul__(self, scale):
        """Scale the whole matrix by a non-negative number by scaling every factor equally."""
        assert isinstance(scale, numbers.Number) and scale >= 0
        with torch.no_grad():
            self.twiddle *= scale ** (1.0 / (self.twiddle.shape[1] * self.twiddle.shape[2]))
        return self

    def diagonal_multiply_(self, diagonal, diag_first):
        """Fold a diagonal into this (single-stack, bias-free) layer in place: input -> diagonal -> butterfly when
        diag_first, else input -> butterfly -> diagonal (torch_butterfly/butterfly.py:181-190 of the reference)."""
        from .combine import diagonal_butterfly
        return diagonal_butterfly(self, diagonal, diag_first, inplace=True)

    def to_base4(self):
        """The same matrix as a ButterflyBase4 layer (pairs of factors fused into 4x4 blocks)."""
        with torch.no_grad():
            twiddle4, twiddle2 = twiddle_base2_to_base4(self.twiddle, self.increasing_stride)
        new = ButterflyBase4(self.in_size, self.out_size, self.bias is not None, self.complex,
                             self.increasing_stride, init=(twiddle4, twiddle2), nblocks=self.nblocks)
        new = new.to(self.twiddle.device)
        if new.bias is not None:
            with torch.no_grad():
                new.bias.copy_(self.bias)
        return new

    def extra_repr(self):
        return "in_size={}, out_size={}, bias={}, complex={}, increasing_stride={}, init={}, nblocks={}".format(
            self.in_size, self.out_size, self.bias is not None, self.complex, self.increasing_stride, self.init,
            self.nblocks)


class ButterflyUnitary(Butterfly):
    """Butterfly whose 2x2 blocks are unitary by construction: each block is parameterised by four
    angles (phi, alpha, psi, chi); ``twiddle`` has shape (nstacks, nblocks, log_n, n/2, 4)."""

    def __init__(self, in_size, out_size, bias=True, increasing_stride=True, nblocks=1):
        nn.Module.__init__(self)
        self._configure(in_size, out_size, True, increasing_stride, nblocks)
        self.init = "ortho"
        self.twiddle = nn.Parameter(torch.empty(self.nstacks, nblocks, self.log_n, self.n // 2, 4))
        self.twiddle._is_structured = True
        if bias:
            self.bias = nn.Parameter(torch.empty(out_size, dtype=self._dtype()))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self):
        core = self.twiddle.shape[:-1]
        phi = torch.asin(torch.sqrt(torch.rand(core)))
        alpha, psi, chi = torch.rand((3,) + tuple(core)) * 2 * math.pi
        with torch.no_grad():
            self.twiddle.copy_(torch.stack([phi, alpha, psi, chi], dim=-1))
        if self.bias is not None:
            bound = 1 / math.sqrt(self.in_size)
            nn.init.uniform_(self.bias, -bound, bound)

    def _effective_twiddle(self):
        if self.twiddle.is_cuda and self.twiddle.dtype == torch.float32:
            return unitary_twiddle(self.twiddle)  # one kernel each way
        phi, alpha, psi, chi = torch.unbind(self.twiddle, -1)
        c, s = torch.cos(phi), torch.sin(phi)

        def polar(r, ang):  # r * exp(i ang) through cos/sin so that autograd stays in real arithmetic
            return torch.stack((r * torch.cos(ang), r * torch.sin(ang)), dim=-1)
        a, b = polar(c, alpha + psi), polar(s, alpha + chi)
        cc, d = polar(-s, alpha - chi), polar(c, alpha - psi)
        tw = torch.stack([torch.stack([a, b], dim=-2), torch.stack([cc, d], dim=-2)], dim=-3)
        return torch.view_as_complex(tw)

    __imul__ = None
    to_base4 = None

    def extra_repr(self):
        return "in_size={}, out_size={}, bias={}, increasing_stride={}, nblocks={}".format(
            self.in_size, self.out_size, self.bias is not None, self.increasing_stride, self.nblocks)


class ButterflyBmm(Butterfly):
    """matrix_batch independent butterfly matrices applied to input (..., matrix_batch, in_size)."""

    def __init__(self, in_size, out_size, matrix_batch=1, bias=True, complex=False, increasing_stride=True,
                 init="randn", nblocks=1):
        nn.Module.__init__(self)
        self._configure(in_size, out_size, complex, increasing_stride, nblocks)
        self.matrix_batch = matrix_batch
        shape = (matrix_batch * self.nstacks, nblocks, self.log_n, self.n // 2, 2, 2)
        self._make_params(shape, self._dtype(), init, (matrix_batch, out_size) if bias else None)
        self.reset_parameters()

    def forward(self, input, transpose=False, conjugate=False):
        return super().forward(input, transpose, conjugate, subtwiddle=False)

    def pre_process(self, input):
        assert input.size(-2) == self.matrix_batch
        rows = input.reshape(-1, self.matrix_batch, input.size(-1))
        batch = rows.shape[0]
        rows = rows.unsqueeze(2).expand(batch, self.matrix_batch, self.nstacks, rows.shape[-1])
        return rows.reshape(batch, self.matrix_batch * self.nstacks, rows.shape[-1])

    def post_process(self, input, output, out_size=None):
        out_size = self.out_size if out_size is None else out_size
        batch = output.shape[0]
        output = output.reshape(batch, self.matrix_batch, self.nstacks * output.size(-1))
        if out_size != output.shape[-1]:
            output = output[:, :, :out_size]
        if self.bias is not None:
            output = output + self.bias[:, :out_size]
        return output.reshape(*input.shape[:-2], self.matrix_batch, self.out_size)

    to_base4 = None

    def extra_repr(self):
        return ("in_size={}, out_size={}, matrix_batch={}, bias={}, complex={}, increasing_stride={}, init={}, "
                "nblocks={}").format(self.in_size, self.out_size, self.matrix_batch, self.bias is not None,
                                     self.complex, self.increasing_stride, self.init, self.nblocks)


class ButterflyBase4(Butterfly):
    """Butterfly stored as radix-4 factors (twiddle4) plus one radix-2 factor per block when log_n is
    odd (twiddle2); multiplies with the native base-4 operator (float32 or complex64)."""

    def __init__(self, *args, init="randn", **kwargs):
        init_pair = None
        if isinstance(init, tuple):
            assert len(init) == 2 and all(isinstance(t, torch.Tensor) for t in init)
            init_pair, init = init, "empty"
        super().__init__(*args, init=init, **kwargs)
        with torch.no_grad():
            twiddle4, twiddle2 = init_pair if init_pair is not None else twiddle_base2_to_base4(
                self.twiddle, self.increasing_stride)
        del self.twiddle
        self.twiddle4 = nn.Parameter(twiddle4.clone())
        self.twiddle2 = nn.Parameter(twiddle2.clone())
        self.twiddle4._is_structured = True
        self.twiddle2._is_structured = True

    def forward(self, input):
        rows = self.pre_process(input)
        output_size = self.out_size if self.nstacks == 1 else None
        out = butterfly_multiply_base4(self.twiddle4, self.twiddle2, rows, self.increasing_stride, output_size)
        return self.post_process(input, out)

    def __imul__(self, scale):
        assert isinstance(scale, numbers.Number) and scale >= 0
        with torch.no_grad():
            per_factor = scale ** (1.0 / (self.twiddle4.shape[1] * (2 * self.twiddle4.shape[2] + self.twiddle2.shape[2])))
            self.twiddle4 *= per_factor ** 2  # a radix-4 factor is the product of two radix-2 factors
            self.twiddle2 *= per_factor
        return self

    to_base4 = None
