"""The C-ABI library loads and exports every symbol include/bfly.h declares; calls that
need no device behave as documented.  (No compute calls here: those are the GPU tests.)"""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "bfly.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bfly4?_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    from butterfly_b200 import abi
    lib = abi.lib()
    names = declared_symbols()
    assert len(names) >= 12
    for nm in names:
        assert hasattr(lib, nm), nm
    assert set(names) == set(abi.SYMBOLS)


def test_status_text_and_versions():
    from butterfly_b200 import abi
    assert abi.strerror(0) == "success"
    for rc in range(-6, 0):
        assert abi.strerror(rc) and abi.strerror(rc) != "unknown status"
    assert abi.strerror(-99) == "unknown status"
    assert abi.lib().bfly_version() >= 100
    assert abi.lib().bfly_cuda_version() >= 12000


def test_workspace_query_and_argument_errors():
    from butterfly_b200 import abi
    assert abi.bw_workspace_bytes(torch.float32, 256, 1, 8, 1) == 0           # 8 stages: one phase, no scratch
    # the forward's optional scratch: a twiddle-sized buffer for float rows of 512 .. 4096 columns
    assert abi.fw_workspace_bytes(torch.float32, 256, 1, 10, 1) == 10 * 512 * 16
    assert abi.fw_workspace_bytes(torch.float32, 256, 3, 12, 2) == 3 * 2 * 12 * 2048 * 16
    assert abi.fw_workspace_bytes(torch.float32, 256, 1, 8, 1) == 0
    # rows of 8192 columns run in one launch on a 512-thread CTA (twiddle-sized scratch, or room for the
    # panel passes that serve as its fallback); wider single-stack rows run pass by pass on 4096-column
    # panels: room for the largest pass (24 stages)
    assert abi.fw_workspace_bytes(torch.float32, 256, 1, 13, 1) == 24 * 8 * 8192
    assert abi.fw_workspace_bytes(torch.float32, 256, 2, 13, 3) == 2 * 3 * 13 * 8 * 8192
    assert abi.fw_workspace_bytes(torch.float32, 256, 1, 14, 1) == 24 * 8 * 16384
    assert abi.fw_workspace_bytes(torch.float32, 256, 2, 14, 1) == 0
    assert abi.fw_workspace_bytes(torch.complex64, 256, 1, 10, 1) == 0
    # 10 stages: two phases = one snapshot, plus the scratch of the forward pass that writes it
    assert abi.bw_workspace_bytes(torch.float32, 256, 1, 10, 1) == 256 * 1024 * 4 + 10 * 512 * 16
    # n = 4096, two blocks: 24 stages = three phases of 8, i.e. two snapshots (the query covers both directions)
    fws = abi.fw_workspace_bytes(torch.float32, 16384, 1, 12, 2)
    assert abi.bw_workspace_bytes(torch.float32, 16384, 1, 12, 2) in (2 * 16384 * 4096 * 4 + fws, 3 * 16384 * 4096 * 4 + fws)
    assert abi.bw_workspace_bytes(torch.float32, 4, 1, 0, 1) == -1      # log_n < 1
    assert abi.bw_workspace_bytes(torch.float32, 4, 0, 5, 1) == -1      # no stacks
    assert abi.bw_workspace_bytes(torch.complex64, 4, 1, 5, 1, base4=True) >= 0   # complex base-4 is supported
    assert abi.launch_count() >= 0


def test_torch_operators_are_registered_and_refuse_cpu_tensors():
    import butterfly_b200 as bb
    ops = torch.ops.torch_butterfly
    for name in ("butterfly_multiply_fw", "butterfly_multiply_bw", "butterfly_multiply", "butterfly_multiply_base4_fw",
                 "butterfly_multiply_base4_bw", "butterfly_multiply_base4", "cuda_version"):
        assert hasattr(ops, name)
    # the reference's import check compares this with torch.version.cuda (torch_butterfly/__init__.py:13-31)
    v = ops.cuda_version()
    major, minor = [int(s) for s in torch.version.cuda.split(".")]
    assert v // 1000 == major and (v % 1000) // 10 == minor
    tw = torch.randn(1, 1, 3, 4, 2, 2)
    x = torch.randn(2, 1, 8)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        bb.butterfly_multiply(tw, x, True)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        bb.butterfly_multiply_bw(tw, x, x, True)


def test_reference_package_imports_on_top_of_these_libraries(tmp_path):
    """The reference's unmodified Python package loads `_version` and `_butterfly` from its own
    directory (torch_butterfly/__init__.py:8-11); link its .py files beside our libraries and
    import it in a fresh interpreter."""
    import oracle
    ref = oracle.reference_dir()
    pkg = os.path.join(ref, "torch_butterfly") if ref else os.path.join(oracle.REF_PKG, "torch_butterfly")
    if not os.path.isdir(pkg):
        pytest.skip("reference tree not present and not staged (make -C oracle refpy)")
    import subprocess
    import sys
    shim = tmp_path / "torch_butterfly"
    shim.mkdir()
    for f in os.listdir(pkg):
        if f.endswith(".py"):
            os.symlink(os.path.join(pkg, f), shim / f)
    for f in ("_butterfly.so", "_version.so"):
        os.symlink(os.path.join(ROOT, "butterfly_b200", f), shim / f)
    code = ("import sys; sys.path.insert(0, %r); import torch, torch_butterfly; "
            "b = torch_butterfly.Butterfly(16, 16); print('imported', torch_butterfly.butterfly_multiply is not None)" % str(tmp_path))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "imported True" in r.stdout
