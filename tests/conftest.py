import glob
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _t(a, cplx):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return torch.view_as_complex(t) if cplx else t


def load_golden(path):
    z = np.load(path)
    meta = [int(v) for v in z["meta"]]
    cplx = bool(meta[7])
    d = {k: _t(z[k], cplx) for k in z.files if k != "meta"}
    d.update(log_n=meta[0], nstacks=meta[1], nblocks=meta[2], batch=meta[3], increasing_stride=bool(meta[4]),
             input_size=meta[5], output_size=meta[6], complex=cplx, name=os.path.basename(path))
    return d


def golden_files(prefix):
    return sorted(glob.glob(os.path.join(GOLDEN, prefix + "_*.npz")))


def rel_err(a, b):
    a = a.detach().cpu()
    b = b.detach().cpu()
    return ((a - b).abs().max() / (b.abs().max() + 1e-30)).item() if b.numel() else 0.0


def tol_ratio(a, b, rtol=1e-5, atol=1e-5):
    """Per-component |a - b| / (atol + rtol |b|) (complex: real and imaginary parts separately).
    <= 1 everywhere means agreement within rtol / atol."""
    a = a.detach().cpu()
    b = b.detach().cpu()
    a = torch.view_as_real(a) if a.is_complex() else a
    b = torch.view_as_real(b) if b.is_complex() else b
    return (a - b).abs() / (atol + rtol * b.abs())


def assert_rtol_atol(a, b, what="", rtol=1e-5, atol=1e-5, outliers=0.0, worst_allowed=1.0):
    """Per-component rtol 1e-5 / atol 1e-5 (the tolerance the product is specified to).  Strict by
    default; `outliers` = fraction of components that may exceed it, up to `worst_allowed` times
    the tolerance (for comparisons of two different float32 evaluation orders over very many
    components, where a few land just outside)."""
    if not b.numel():
        return
    r = tol_ratio(a, b, rtol, atol)
    worst = r.max().item()
    frac = (r > 1).float().mean().item()
    assert frac <= outliers and worst <= max(worst_allowed, 1.0), (
        "%s: %.4f %% of components outside rtol %g / atol %g, worst %.2fx the tolerance" % (what, 100.0 * frac, rtol, atol, worst))


def assert_sum_accuracy(ours, ref32, ref64, what=""):
    """Grade a float32 twiddle gradient (a sum over the batch) against the double-precision
    oracle: per component it must be as close to it as the float32 oracle is, or within 1e-5 of
    the gradient's scale -- two valid summation orders of thousands of float32 terms differ by
    more than rtol 1e-5 on the entries whose true sum is near zero."""
    if not ref64.numel():
        return
    o = ours.detach().cpu()
    o = (torch.view_as_real(o) if o.is_complex() else o).double()
    r32 = (torch.view_as_real(ref32) if ref32.is_complex() else ref32).double()
    r64 = (torch.view_as_real(ref64) if ref64.is_complex() else ref64).double()
    scale = r64.abs().max().item()
    # the float32 oracle's own error, as a floor per component and over the tensor
    allowed = torch.maximum((r32 - r64).abs(), torch.full_like(r64, 1e-5 * scale))
    err = (o - r64).abs()
    bad = err > allowed
    assert not bad.any(), "%s: %d components further from the double-precision oracle than allowed (worst %.3g, scale %.3g)" % (
        what, int(bad.sum()), (err - allowed).max().item(), scale)


def unitary_chain(angles):
    """The reference's construction (torch_butterfly/butterfly.py:271-280) in plain torch."""
    phi, alpha, psi, chi = torch.unbind(angles, -1)
    c, s = torch.cos(phi), torch.sin(phi)
    A = torch.stack((c * torch.cos(alpha + psi), c * torch.sin(alpha + psi)), dim=-1)
    B = torch.stack((s * torch.cos(alpha + chi), s * torch.sin(alpha + chi)), dim=-1)
    C = torch.stack((-s * torch.cos(alpha - chi), -s * torch.sin(alpha - chi)), dim=-1)
    D = torch.stack((c * torch.cos(alpha - psi), c * torch.sin(alpha - psi)), dim=-1)
    return torch.view_as_complex(torch.stack([torch.stack([A, B], dim=-2), torch.stack([C, D], dim=-2)], dim=-3))


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    oracle.build()
    return oracle


class library_option:
    """Sets a development switch of libbfly_b200.so (butterfly_b200.abi.set_option) or of the
    host emulator for the duration of a `with` block and puts the old value back."""

    def __init__(self, setter, getter, name, value):
        self.setter, self.getter, self.name, self.value = setter, getter, name, value

    def __enter__(self):
        self.old = self.getter(self.name)
        self.setter(self.name, self.value)
        return self

    def __exit__(self, *exc):
        self.setter(self.name, self.old)
        return False


def abi_option(name, value):
    from butterfly_b200 import abi
    return library_option(abi.set_option, abi.get_option, name, value)
