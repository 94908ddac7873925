"""The reference's own Python package and test files, unchanged, on CUDA over the new libraries.

`make -C oracle refpy` stages torch_butterfly/*.py and three test files of the reference under
oracle/_ref/pkg (git-ignored).  Here a scratch directory gets symlinks to those files plus this
repository's `_butterfly.so` / `_version.so` under the names the reference package loads
(torch_butterfly/__init__.py:8-11), and a fresh interpreter imports it.  The new operator has no CPU
implementation, so inside that interpreter CPU tensors are routed to the reference's own
pure-PyTorch definition (`butterfly_multiply_torch`, torch_butterfly/multiply.py:28-51) -- the CPU
iterations of the reference's tests then compare that definition with itself, the CUDA iterations
exercise the new kernels.
"""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

from conftest import ROOT

pytestmark = pytest.mark.gpu

PROLOGUE = textwrap.dedent('''
    import sys
    sys.path.insert(0, %(shim)r)
    import torch
    import torch_butterfly
    import torch_butterfly.multiply as M
    _op = M.butterfly_multiply
    def _routed(twiddle, input, increasing_stride=True, output_size=None):
        if not twiddle.is_cuda:
            return M.butterfly_multiply_torch(twiddle, input, increasing_stride, output_size)
        return _op(twiddle, input, increasing_stride, output_size)
    for mod in (torch_butterfly, M, torch_butterfly.butterfly, torch_butterfly.butterfly_base4):
        if hasattr(mod, "butterfly_multiply"):
            mod.butterfly_multiply = _routed
''')


@pytest.fixture(scope="module")
def shim(tmp_path_factory):
    import oracle
    pkg = os.path.join(oracle.REF_PKG, "torch_butterfly")
    if not os.path.isdir(pkg):
        pytest.skip("reference package not staged (make -C oracle refpy REF=<reference tree>)")
    root = tmp_path_factory.mktemp("refpkg")
    d = root / "torch_butterfly"
    d.mkdir()
    for f in os.listdir(pkg):
        if f.endswith(".py"):
            os.symlink(os.path.join(pkg, f), d / f)
    for f in ("_butterfly.so", "_version.so"):
        os.symlink(os.path.join(ROOT, "butterfly_b200", f), d / f)
    return str(root)


def _run(shim, body, timeout=900):
    code = PROLOGUE % {"shim": shim} + textwrap.dedent(body)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    return r.stdout


def test_reference_modules_run_on_the_new_operator(shim):
    """torch_butterfly.Butterfly as a 1024 -> 4096 layer (forward + backward) against the reference's
    PyTorch definition on the same device, and special.fft(2048) against torch.fft."""
    out = _run(shim, '''
        torch.manual_seed(0)
        dev = torch.device("cuda", 0)
        before = torch.ops.torch_butterfly.b200_launch_count()
        layer = torch_butterfly.Butterfly(1024, 4096, bias=True, nblocks=2).to(dev)
        x = torch.randn(512, 1024, device=dev, requires_grad=True)
        y = layer(x)
        assert y.shape == (512, 4096)
        y.backward(torch.randn_like(y))
        # the same layer through the reference's pure-PyTorch multiply
        tw = layer.twiddle.detach().clone().requires_grad_(True)
        xr = x.detach().clone().requires_grad_(True)
        rows = xr.unsqueeze(1).expand(512, 4, 1024)
        yr = M.butterfly_multiply_torch(tw, rows, True).reshape(512, 4096) + layer.bias
        torch.manual_seed(0)
        assert torch.allclose(y, yr, rtol=1e-4, atol=1e-4), (y - yr).abs().max().item()
        b = torch_butterfly.special.fft(2048, normalized=False).to(dev)
        z = torch.randn(64, 2048, dtype=torch.complex64, device=dev)
        err = (b(z) - torch.fft.fft(z)).abs().max().item() / torch.fft.fft(z).abs().max().item()
        assert err < 1e-5, err
        assert torch.ops.torch_butterfly.b200_launch_count() > before   # the new kernels ran
        print("modules ok", err)
    ''')
    assert "modules ok" in out


@pytest.mark.parametrize("test_file,selection", [("test_multiply.py", ""), ("test_multiply_base4.py", ""), ("test_butterfly.py", "")])
def test_reference_test_files_pass_unchanged(shim, test_file, selection):
    """The reference's own test files, as they are.  test_transpose_conjugate_multiply fails with the
    reference's operator on current PyTorch (it ignores the lazy conjugate bit of `twiddle.conj()`);
    the new operator resolves it at the boundary, so the test passes here."""
    import oracle
    path = os.path.join(oracle.REF_PKG, "tests", test_file)
    out = _run(shim, '''
        import pytest
        # The reference's tests draw unseeded inputs and hold float32 twiddle gradients of un-normalised
        # products (sums of cancelling terms of magnitude ~60) to atol 1e-5 against another summation
        # order; about one seed in ten lands an entry just outside, whatever the implementation.  A fixed
        # seed makes the run repeatable.
        torch.manual_seed(0)
        args = [%r, "-q", "-p", "no:cacheprovider"]
        if %r:
            args += ["-k", %r]
        rc = pytest.main(args)
        print("pytest exit", int(rc))
        sys.exit(int(rc))
    ''' % (path, selection, selection), timeout=1800)
    assert "pytest exit 0" in out
