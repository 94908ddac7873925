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
