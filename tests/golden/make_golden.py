"""Generates the golden fixtures in this directory from the REFERENCE implementation.

Run where the reference tree is available (BFLY_REFERENCE_DIR, or a directory `reference` beside
this repository) and the reference's CPU operator has been compiled by `make -C oracle refcpu`:

    python tests/golden/make_golden.py

It imports, by file path, the reference's pure-PyTorch definitions
(torch_butterfly/multiply.py:28-51 `butterfly_multiply_torch`,
torch_butterfly/multiply_base4.py:7-41 `butterfly_multiply_base4_torch`, :44-71
`twiddle_base2_to_base4`) and calls its compiled CPU operator
(csrc/cpu/butterfly_cpu.cpp), and stores seeded inputs together with their outputs:

  radix2_*.npz   twiddle, input, grad -> output, d_twiddle, d_input of the reference CPU op
                 (forward and backward), plus the forward of butterfly_multiply_torch
  base4_*.npz    twiddle4, twiddle2, input, grad -> output of butterfly_multiply_base4_torch
                 and its autograd gradients, evaluated in double precision

The reference's own tests hold no golden vectors (every check there compares two
implementations on unseeded random inputs: tests/test_multiply.py:19-90,
tests/test_multiply_base4.py:21-44), so these files are the pin.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

REF = oracle.reference_dir()  # BFLY_REFERENCE_DIR, or the sibling directory `reference`


def _load_reference_python():
    src = open(os.path.join(REF, "torch_butterfly", "multiply.py")).read()
    src = src[src.index("def butterfly_multiply_torch"):]  # skip the jit wrappers: they need the compiled ops
    ns = {"torch": torch, "F": torch.nn.functional}
    exec(compile(src, "multiply.py", "exec"), ns)
    ns4 = {}
    exec(compile(open(os.path.join(REF, "torch_butterfly", "multiply_base4.py")).read(), "multiply_base4.py", "exec"), ns4)
    return ns["butterfly_multiply_torch"], ns4["butterfly_multiply_base4_torch"], ns4["twiddle_base2_to_base4"]


def np_(t):
    t = t.detach()
    if t.is_complex():
        return torch.view_as_real(t.resolve_conj()).numpy().copy()
    return t.numpy().copy()


def main():
    import oracle
    ref = oracle.load_reference_ops()
    bmt, b4t, b2to4 = _load_reference_python()
    cases = []
    seed = 0
    # (dtype, log_n, nstacks, nblocks, batch, increasing_stride, input_size, output_size)
    for dt in (torch.float32, torch.complex64):
        for log_n, S, nb, B, inc in [(1, 1, 1, 3, True), (2, 2, 2, 3, False), (3, 2, 3, 5, True), (5, 2, 3, 6, False),
                                     (6, 1, 2, 4, True), (7, 1, 1, 3, False)]:
            n = 1 << log_n
            for insz, outsz in [(n, n), (max(1, n // 2 - 1), max(1, n - 1)), (2 * n + 3, max(1, n // 2))]:
                cases.append((dt, log_n, S, nb, B, inc, insz, outsz))
    for i, (dt, log_n, S, nb, B, inc, insz, outsz) in enumerate(cases):
        g = torch.Generator().manual_seed(seed + i)
        n = 1 << log_n
        tw = torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dt, generator=g) / 2 ** 0.5
        x = torch.randn(B, S, insz, dtype=dt, generator=g)
        grad = torch.randn(B, S, outsz, dtype=dt, generator=g)
        out = ref.butterfly_multiply_fw(tw, x, inc, outsz)
        d_tw, d_x = ref.butterfly_multiply_bw(tw, x, grad, inc)
        out_torch = bmt(tw, x, inc, outsz)
        name = "radix2_%s_%02d.npz" % ("f32" if dt == torch.float32 else "c64", i)
        np.savez_compressed(os.path.join(HERE, name), twiddle=np_(tw), input=np_(x), grad=np_(grad), output=np_(out),
                            d_twiddle=np_(d_tw), d_input=np_(d_x), output_torch=np_(out_torch),
                            meta=np.array([log_n, S, nb, B, int(inc), insz, outsz, int(dt == torch.complex64)]))
    # base-4: double-precision torch + autograd as truth, float32 inputs stored
    k = 0
    for dt in (torch.float32, torch.complex64):
        for log_n, S, nb, B, inc in [(1, 1, 1, 3, True), (2, 2, 2, 3, False), (3, 1, 2, 4, True), (4, 2, 3, 4, False),
                                     (5, 1, 1, 5, True), (6, 1, 2, 3, False), (7, 1, 2, 3, True)]:
            n = 1 << log_n
            for insz, outsz in [(n, n), (max(1, n // 2 - 1), max(1, n - 1))]:
                g = torch.Generator().manual_seed(1000 + k)
                tw = torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dt, generator=g) / 2 ** 0.5
                tw4, tw2 = b2to4(tw, inc)
                tw4 = torch.randn(tw4.shape, dtype=dt, generator=g) / 2  # generic 4x4 blocks, not products of 2x2s
                tw2 = tw2.clone()
                x = torch.randn(B, S, insz, dtype=dt, generator=g)
                grad = torch.randn(B, S, outsz, dtype=dt, generator=g)
                hi = torch.complex128 if dt.is_complex else torch.float64
                t4 = tw4.to(hi).requires_grad_(True)
                t2 = tw2.to(hi).requires_grad_(True)
                xx = x.to(hi).requires_grad_(True)
                out = b4t(t4, t2, xx, inc, outsz)
                gs = torch.autograd.grad(out, [t4, t2, xx], grad.to(hi), allow_unused=True)
                d4 = gs[0] if gs[0] is not None else torch.zeros_like(t4)
                d2 = gs[1] if gs[1] is not None else torch.zeros_like(t2)
                name = "base4_%s_%02d.npz" % ("f32" if dt == torch.float32 else "c64", k)
                np.savez_compressed(os.path.join(HERE, name), twiddle4=np_(tw4), twiddle2=np_(tw2), input=np_(x),
                                    grad=np_(grad), output=np_(out.to(dt)), d_twiddle4=np_(d4.to(dt)),
                                    d_twiddle2=np_(d2.to(dt)), d_input=np_(gs[2].to(dt)),
                                    meta=np.array([log_n, S, nb, B, int(inc), insz, outsz, int(dt == torch.complex64)]))
                k += 1
    print("wrote %d radix-2 and %d base-4 fixtures to %s" % (len(cases), k, HERE))


if __name__ == "__main__":
    main()
