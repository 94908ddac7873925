"""butterfly_b200 -- the butterfly multiply of HazyResearch/butterfly's ``torch_butterfly``,
rebuilt for NVIDIA B200 (sm_100a).

Importing the package loads the native libraries built by ``butterfly_b200._build``:
``libbfly_b200.so`` (CUDA kernels behind the C ABI of ``include/bfly.h``) and the torch
operator layer ``_butterfly.so`` / ``_version.so``, which registers the same operators as
the reference (``torch.ops.torch_butterfly.butterfly_multiply_fw / _bw /
butterfly_multiply``, csrc/butterfly.cpp:127-131 there) plus native base-4 operators.

The operators accept CUDA tensors only.  Nothing here falls back to a CPU or pure-PyTorch
implementation: if the native libraries are missing the import fails.
"""
import os

import torch

__version__ = "0.1.0"

_HERE = os.path.dirname(os.path.abspath(__file__))


def _load_native():
    missing = [f for f in ("libbfly_b200.so", "_version.so", "_butterfly.so")
               if not os.path.exists(os.path.join(_HERE, f))]
    if missing:
        raise ImportError(
            "butterfly_b200: native libraries not built (%s missing). Run "
            "`python -m butterfly_b200._build` (needs nvcc and g++; no GPU needed to build)."
            % ", ".join(missing))
    # same order as the reference package: the version operator first, then the operators
    for name in ("_version.so", "_butterfly.so"):
        torch.ops.load_library(os.path.join(_HERE, name))


_load_native()

from .multiply import (  # noqa: E402,F401
    butterfly_multiply, butterfly_multiply_fw, butterfly_multiply_bw, butterfly_linear, butterfly_linear_fw, butterfly_linear_bw,
    unitary_twiddle, unitary_twiddle_fw, unitary_twiddle_bw,
)
from .multiply_base4 import (  # noqa: E402,F401
    butterfly_multiply_base4, butterfly_multiply_base4_fw, butterfly_multiply_base4_bw, twiddle_base2_to_base4,
)
from . import abi  # noqa: E402,F401
from .butterfly import Butterfly, ButterflyUnitary, ButterflyBmm, ButterflyBase4  # noqa: E402,F401
from . import permutation, complex_utils, diagonal, glue, special, host, distributed, combine, kops  # noqa: E402,F401
from .glue import butterfly_multiply_glue  # noqa: E402,F401

__all__ = [
    "butterfly_multiply", "butterfly_multiply_fw", "butterfly_multiply_bw",
    "butterfly_linear", "butterfly_linear_fw", "butterfly_linear_bw",
    "unitary_twiddle", "unitary_twiddle_fw", "unitary_twiddle_bw",
    "butterfly_multiply_base4", "butterfly_multiply_base4_fw", "butterfly_multiply_base4_bw",
    "twiddle_base2_to_base4", "abi", "__version__", "Butterfly", "ButterflyUnitary", "ButterflyBmm", "ButterflyBase4",
    "permutation", "special", "combine", "kops", "complex_utils", "diagonal", "glue", "butterfly_multiply_glue",
]
