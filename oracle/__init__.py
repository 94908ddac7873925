"""Test infrastructure, not product code: the CPU oracle for the butterfly multiply.

``oracle`` wraps ``libbfly_oracle.so`` (a plain-C restatement of the reference's CPU
algorithm, see ``bfly_oracle.c``) and, when it has been built, the reference's own CPU
operator compiled from the reference tree (``_ref/_butterfly_ref_cpu.so``).

Only the tests, the smoke check and the benchmark's CPU-baseline leg may import this
package; the shipped CUDA path never does.
"""
from .oracle import (  # noqa: F401
    multiply_fw, multiply_bw, base4_fw, base4_bw, build, load_reference_ops, reference_available, reference_dir, REF_PKG,
)
