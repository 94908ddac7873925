"""ctypes front-end of the C oracle (test infrastructure, not product code).

Functions take and return CPU ``torch`` tensors so that parity tests read like the
reference's own tests (tests/test_multiply.py:19-90 of the reference compare the operator
with ``butterfly_multiply_torch`` in exactly this shape convention):

    twiddle (nstacks, nblocks, log_n, n/2, 2, 2), input (batch, nstacks, input_size)
"""
import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libbfly_oracle.so")
_REF_CPU = os.path.join(_HERE, "_ref", "_butterfly_ref_cpu.so")
_REF_CUDA = os.path.join(_HERE, "_ref", "_butterfly_ref_cuda.so")
_lib = None

_SUFFIX = {torch.float32: "f32", torch.float64: "f64", torch.complex64: "c64", torch.complex128: "c128"}


def build(force=False):
    """Compile the C oracle (and the reference CPU operator when the reference tree is there)."""
    if force or not os.path.exists(_LIB_PATH) or (
            os.path.getmtime(_LIB_PATH) < max(os.path.getmtime(os.path.join(_HERE, f))
                                              for f in ("bfly_oracle.c", "bfly_oracle_impl.h"))):
        subprocess.check_call(["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared",
                               os.path.join(_HERE, "bfly_oracle.c"), "-o", _LIB_PATH])
    ref_src = reference_dir()
    if ref_src and os.path.exists(os.path.join(ref_src, "csrc", "cpu", "butterfly_cpu.cpp")):
        if not os.path.exists(_REF_CPU):
            subprocess.check_call(["make", "-C", _HERE, "refcpu", f"REF={ref_src}"])
        if not os.path.exists(os.path.join(REF_PKG, "torch_butterfly", "__init__.py")):
            subprocess.check_call(["make", "-C", _HERE, "refpy", f"REF={ref_src}"])


# the reference's Python package and three of its test files, staged by `make refpy`
REF_PKG = os.path.join(_HERE, "_ref", "pkg")


def reference_dir():
    """Root of the reference tree: $BFLY_REFERENCE_DIR, else a directory named `reference` beside
    this repository; None when neither exists."""
    cand = os.environ.get("BFLY_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isdir(cand) else None


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def reference_available(cuda=False):
    return os.path.exists(_REF_CUDA if cuda else _REF_CPU)


_ref_loaded = None


def load_reference_ops(cuda=False):
    """Load the reference's own kernels (namespace ``torch.ops.torch_butterfly_ref``).

    The CUDA build also contains the CPU kernels, so it is preferred when asked for and
    present; only one of the two libraries may be loaded per process.
    """
    global _ref_loaded
    if _ref_loaded is None:
        path = _REF_CUDA if (cuda and os.path.exists(_REF_CUDA)) else _REF_CPU
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        torch.ops.load_library(path)
        _ref_loaded = path
    if cuda and _ref_loaded != _REF_CUDA:
        raise RuntimeError("reference CPU library already loaded in this process; CUDA build unavailable")
    return torch.ops.torch_butterfly_ref


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _prep_x(x):
    x = x.detach().cpu().resolve_conj()
    if x.stride(2) != 1:
        x = x.contiguous()
    return x


def _shape(twiddle, x):
    S, nblocks, log_n = twiddle.shape[:3]
    n = 1 << log_n
    assert tuple(twiddle.shape) == (S, nblocks, log_n, n // 2, 2, 2), twiddle.shape
    B, Sx, input_size = x.shape
    assert Sx == S
    return B, S, log_n, nblocks, n, input_size


def multiply_fw(twiddle, x, increasing_stride=True, output_size=None):
    twiddle = twiddle.detach().cpu().resolve_conj().contiguous()
    x = _prep_x(x).to(twiddle.dtype)
    B, S, log_n, nblocks, n, input_size = _shape(twiddle, x)
    output_size = n if output_size is None else output_size
    out = torch.empty(B, S, output_size, dtype=twiddle.dtype)
    fn = getattr(_load(), "bfly_oracle_fw_" + _SUFFIX[twiddle.dtype])
    rc = fn(_ptr(twiddle), _ptr(x), ctypes.c_int64(x.stride(0)), ctypes.c_int64(x.stride(1)), _ptr(out),
            ctypes.c_int64(B), ctypes.c_int64(S), ctypes.c_int(log_n), ctypes.c_int(nblocks),
            ctypes.c_int64(input_size), ctypes.c_int64(output_size), ctypes.c_int(int(increasing_stride)))
    if rc != 0:
        raise RuntimeError(f"oracle fw failed ({rc})")
    return out


def multiply_bw(twiddle, x, grad, increasing_stride=True):
    twiddle = twiddle.detach().cpu().resolve_conj().contiguous()
    x = _prep_x(x).to(twiddle.dtype)
    grad = grad.detach().cpu().resolve_conj().contiguous().to(twiddle.dtype)
    B, S, log_n, nblocks, n, input_size = _shape(twiddle, x)
    output_size = grad.shape[2]
    assert tuple(grad.shape) == (B, S, output_size)
    d_tw = torch.empty_like(twiddle)
    d_x = torch.empty(B, S, input_size, dtype=twiddle.dtype)
    fn = getattr(_load(), "bfly_oracle_bw_" + _SUFFIX[twiddle.dtype])
    rc = fn(_ptr(twiddle), _ptr(x), ctypes.c_int64(x.stride(0)), ctypes.c_int64(x.stride(1)), _ptr(grad),
            _ptr(d_tw), _ptr(d_x), ctypes.c_int64(B), ctypes.c_int64(S), ctypes.c_int(log_n),
            ctypes.c_int(nblocks), ctypes.c_int64(input_size), ctypes.c_int64(output_size),
            ctypes.c_int(int(increasing_stride)))
    if rc != 0:
        raise RuntimeError(f"oracle bw failed ({rc})")
    return d_tw, d_x


def _shape4(twiddle4, twiddle2, x):
    S, nblocks = twiddle4.shape[:2]
    log_n = twiddle4.shape[2] * 2 + twiddle2.shape[2]
    n = 1 << log_n
    if log_n // 2 > 0:
        assert tuple(twiddle4.shape) == (S, nblocks, log_n // 2, n // 4, 4, 4), twiddle4.shape
    if log_n % 2 == 1:
        assert tuple(twiddle2.shape) == (S, nblocks, 1, n // 2, 2, 2), twiddle2.shape
    B, Sx, input_size = x.shape
    assert Sx == S
    return B, S, log_n, nblocks, n, input_size


def base4_fw(twiddle4, twiddle2, x, increasing_stride=True, output_size=None):
    twiddle4 = twiddle4.detach().cpu().resolve_conj().contiguous()
    twiddle2 = twiddle2.detach().cpu().resolve_conj().contiguous().to(twiddle4.dtype)
    x = _prep_x(x).to(twiddle4.dtype)
    B, S, log_n, nblocks, n, input_size = _shape4(twiddle4, twiddle2, x)
    output_size = n if output_size is None else output_size
    out = torch.empty(B, S, output_size, dtype=twiddle4.dtype)
    fn = getattr(_load(), "bfly_oracle_base4_fw_" + _SUFFIX[twiddle4.dtype])
    rc = fn(_ptr(twiddle4), _ptr(twiddle2), _ptr(x), ctypes.c_int64(x.stride(0)), ctypes.c_int64(x.stride(1)),
            _ptr(out), ctypes.c_int64(B), ctypes.c_int64(S), ctypes.c_int(log_n), ctypes.c_int(nblocks),
            ctypes.c_int64(input_size), ctypes.c_int64(output_size), ctypes.c_int(int(increasing_stride)))
    if rc != 0:
        raise RuntimeError(f"oracle base4 fw failed ({rc})")
    return out


def base4_bw(twiddle4, twiddle2, x, grad, increasing_stride=True):
    twiddle4 = twiddle4.detach().cpu().resolve_conj().contiguous()
    twiddle2 = twiddle2.detach().cpu().resolve_conj().contiguous().to(twiddle4.dtype)
    x = _prep_x(x).to(twiddle4.dtype)
    grad = grad.detach().cpu().resolve_conj().contiguous().to(twiddle4.dtype)
    B, S, log_n, nblocks, n, input_size = _shape4(twiddle4, twiddle2, x)
    output_size = grad.shape[2]
    d4 = torch.empty_like(twiddle4)
    d2 = torch.empty_like(twiddle2)
    d_x = torch.empty(B, S, input_size, dtype=twiddle4.dtype)
    fn = getattr(_load(), "bfly_oracle_base4_bw_" + _SUFFIX[twiddle4.dtype])
    rc = fn(_ptr(twiddle4), _ptr(twiddle2), _ptr(x), ctypes.c_int64(x.stride(0)), ctypes.c_int64(x.stride(1)),
            _ptr(grad), _ptr(d4), _ptr(d2), _ptr(d_x), ctypes.c_int64(B), ctypes.c_int64(S),
            ctypes.c_int(log_n), ctypes.c_int(nblocks), ctypes.c_int64(input_size),
            ctypes.c_int64(output_size), ctypes.c_int(int(increasing_stride)))
    if rc != 0:
        raise RuntimeError(f"oracle base4 bw failed ({rc})")
    return d4, d2, d_x
