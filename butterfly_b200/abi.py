"""ctypes view of the C ABI (``include/bfly.h``) for callers that hold raw device pointers.

The torch operators go through the same entry points from C++; this module exists so that
tests and benchmarks can drive ``libbfly_b200.so`` directly, the way a non-torch host
(the reference's own FFI, a C++ server) would.  All functions take torch CUDA tensors only
to obtain device pointers and strides; nothing is copied.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbfly_b200.so")

F32, C64 = 0, 1

# every symbol include/bfly.h declares
SYMBOLS = (
    "bfly_strerror", "bfly_version", "bfly_cuda_version", "bfly_fw_f32", "bfly_fw_c64", "bfly_fw_workspace_bytes",
    "bfly_bw_workspace_bytes", "bfly_bw_f32", "bfly_bw_c64", "bfly4_fw_f32", "bfly4_bw_workspace_bytes",
    "bfly4_bw_f32", "bfly_launch_count", "bfly_profile_enable", "bfly_profile_collect", "bfly_bw_f32_noalloc",
    "bfly_linear_fw_f32", "bfly_linear_bw_f32", "bfly_linear_bw_workspace_bytes", "bfly_device_error", "bfly_set_option", "bfly_get_option", "bfly4_fw_c64", "bfly4_bw_c64", "bfly_fw_f32_saving", "bfly_fw_c64_saving", "bfly_bw_f32_saved", "bfly_bw_c64_saved",
    "bfly_unitary_twiddle_fw", "bfly_unitary_twiddle_bw", "bfly_fw_glue_f32", "bfly_fw_glue_c64",
    "bfly_selftest_bounded_wait", "bfly_device_error_async",
)

NOALLOC_SCRATCH_BYTES = 32 << 20

_lib = None


def lib():
    """The loaded library (raises if it has not been built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("libbfly_b200.so not built; run `python -m butterfly_b200._build`")
        L = ctypes.CDLL(LIB_PATH)
        L.bfly_strerror.restype = ctypes.c_char_p
        L.bfly_strerror.argtypes = [ctypes.c_int]
        L.bfly_bw_workspace_bytes.restype = ctypes.c_int64
        L.bfly_fw_workspace_bytes.restype = ctypes.c_int64
        L.bfly_linear_bw_workspace_bytes.restype = ctypes.c_int64
        L.bfly4_bw_workspace_bytes.restype = ctypes.c_int64
        L.bfly_launch_count.restype = ctypes.c_int64
        _lib = L
    return _lib


def strerror(rc):
    return lib().bfly_strerror(int(rc)).decode()


class BflyError(RuntimeError):
    def __init__(self, rc, what):
        super().__init__("%s failed: %s (status %d)" % (what, strerror(rc), rc))
        self.status = rc


def _p(t):
    return ctypes.c_void_p(t.data_ptr() if (t is not None and t.numel() > 0) else 0)


def _i64(v):
    return ctypes.c_int64(int(v))


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check_rows(t):
    assert t.is_cuda and t.dim() == 3 and (t.size(2) <= 1 or t.stride(2) == 1)


def fw_workspace_bytes(dtype, B, S, log_n, nblocks):
    code = F32 if dtype == torch.float32 else C64
    return int(lib().bfly_fw_workspace_bytes(code, int(B), int(S), int(log_n), int(nblocks)))


def fw(twiddle, x, increasing_stride=True, output_size=None, out=None, check=True, workspace="auto"):
    """``bfly_fw_f32`` / ``bfly_fw_c64``.  Returns the (batch, nstacks, n) output buffer and the status.

    ``workspace``: a uint8 CUDA tensor of ``fw_workspace_bytes`` bytes, ``None`` (the call then runs on
    the generic kernel) or ``"auto"`` (allocated here when the shape can use one)."""
    _check_rows(x)
    S, nblocks, log_n = twiddle.shape[:3]
    n = 1 << log_n
    B, _, in_size = x.shape
    output_size = n if output_size is None else output_size
    if out is None:
        out = torch.empty(B, S, n, dtype=x.dtype, device=x.device)
    if isinstance(workspace, str):
        need = fw_workspace_bytes(x.dtype, B, S, log_n, nblocks)
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device) if need > 0 else None
    ws_bytes = 0 if workspace is None else workspace.numel()
    fn = lib().bfly_fw_f32 if x.dtype == torch.float32 else lib().bfly_fw_c64
    rc = fn(_p(twiddle), _p(x), _i64(x.stride(0)), _i64(x.stride(1)), _p(out), int(B), int(S), int(log_n),
            int(nblocks), int(in_size), int(output_size), int(bool(increasing_stride)), _p(workspace),
            ctypes.c_size_t(ws_bytes), _stream())
    if check and rc != 0:
        raise BflyError(rc, "bfly_fw")
    return out, rc


def bw_workspace_bytes(dtype, B, S, log_n, nblocks, base4=False):
    code = F32 if dtype == torch.float32 else C64
    fn = lib().bfly4_bw_workspace_bytes if base4 else lib().bfly_bw_workspace_bytes
    return int(fn(code, int(B), int(S), int(log_n), int(nblocks)))


def bw(twiddle, x, grad, increasing_stride=True, workspace=None, d_twiddle=None, d_x=None, check=True):
    """``bfly_bw_f32`` / ``bfly_bw_c64``.  Returns (d_twiddle, d_x buffer (batch, nstacks, max(in, n)), status)."""
    _check_rows(x)
    _check_rows(grad)
    S, nblocks, log_n = twiddle.shape[:3]
    n = 1 << log_n
    B, _, in_size = x.shape
    out_size = grad.shape[2]
    if d_twiddle is None:
        d_twiddle = torch.empty_like(twiddle)
    if d_x is None:
        d_x = torch.empty(B, S, max(in_size, n), dtype=x.dtype, device=x.device)
    need = bw_workspace_bytes(x.dtype, B, S, log_n, nblocks)
    if need < 0:
        if check:
            raise BflyError(need, "bfly_bw_workspace_bytes")
        return d_twiddle, d_x, need
    if workspace is None and need > 0:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    ws_bytes = 0 if workspace is None else workspace.numel()
    fn = lib().bfly_bw_f32 if x.dtype == torch.float32 else lib().bfly_bw_c64
    rc = fn(_p(twiddle), _p(x), _i64(x.stride(0)), _i64(x.stride(1)), _p(grad), _i64(grad.stride(0)),
            _i64(grad.stride(1)), _p(d_twiddle), _p(d_x), int(B), int(S), int(log_n), int(nblocks), int(in_size),
            int(out_size), int(bool(increasing_stride)), _p(workspace), ctypes.c_size_t(ws_bytes), _stream())
    if check and rc != 0:
        raise BflyError(rc, "bfly_bw")
    return d_twiddle, d_x, rc


def fw_saving(twiddle, x, increasing_stride=True, output_size=None, out=None, snapshots=None, check=True):
    """``bfly_fw_f32_saving`` / ``bfly_fw_c64_saving``: the forward that also writes the activations
    the backward starts its phases from.  Returns (output buffer, snapshots, status)."""
    _check_rows(x)
    S, nblocks, log_n = twiddle.shape[:3]
    n = 1 << log_n
    B, _, in_size = x.shape
    output_size = n if output_size is None else output_size
    if out is None:
        out = torch.empty(B, S, n, dtype=x.dtype, device=x.device)
    need = bw_workspace_bytes(x.dtype, B, S, log_n, nblocks)
    if need < 0:
        if check:
            raise BflyError(need, "bfly_bw_workspace_bytes")
        return out, snapshots, need
    if snapshots is None:
        snapshots = torch.empty(need, dtype=torch.uint8, device=x.device)
    fn = lib().bfly_fw_f32_saving if x.dtype == torch.float32 else lib().bfly_fw_c64_saving
    rc = fn(_p(twiddle), _p(x), _i64(x.stride(0)), _i64(x.stride(1)), _p(out), int(B), int(S), int(log_n),
            int(nblocks), int(in_size), int(output_size), int(bool(increasing_stride)), _p(snapshots),
            ctypes.c_size_t(snapshots.numel()), _stream())
    if check and rc != 0:
        raise BflyError(rc, "bfly_fw_saving")
    return out, snapshots, rc


def bw_saved(twiddle, x, grad, snapshots, increasing_stride=True, d_twiddle=None, d_x=None, check=True):
    """``bfly_bw_f32_saved`` / ``bfly_bw_c64_saved``: the backward that starts from the snapshots the
    matching ``fw_saving`` call wrote.  Returns (d_twiddle, d_x buffer, status)."""
    _check_rows(x)
    _check_rows(grad)
    S, nblocks, log_n = twiddle.shape[:3]
    n = 1 << log_n
    B, _, in_size = x.shape
    out_size = grad.shape[2]
    if d_twiddle is None:
        d_twiddle = torch.empty_like(twiddle)
    if d_x is None:
        d_x = torch.empty(B, S, max(in_size, n), dtype=x.dtype, device=x.device)
    fn = lib().bfly_bw_f32_saved if x.dtype == torch.float32 else lib().bfly_bw_c64_saved
    rc = fn(_p(twiddle), _p(x), _i64(x.stride(0)), _i64(x.stride(1)), _p(grad), _i64(grad.stride(0)),
            _i64(grad.stride(1)), _p(d_twiddle), _p(d_x), int(B), int(S), int(log_n), int(nblocks), int(in_size),
            int(out_size), int(bool(increasing_stride)), _p(snapshots), ctypes.c_size_t(snapshots.numel()), _stream())
    if check and rc != 0:
        raise BflyError(rc, "bfly_bw_saved")
    return d_twiddle, d_x, rc


def bw_noalloc(twiddle, x, grad, increasing_stride=True, d_twiddle=None, d_x=None, check=True):
    """``bfly_bw_f32_noalloc``: the float32 backward with the library's built-in scratch buffer.

    For hosts that cannot hand the library any device scratch at the call site.  The outputs are
    passed in by the caller as usual (allocated here only when omitted, for convenience in tests);
    the call itself allocates nothing.  Returns (d_twiddle, d_x buffer, status); status is
    ``-7`` (BFLY_E_TOOLARGE) when the shape needs more than ``NOALLOC_SCRATCH_BYTES``.
    """
    _check_rows(x)
    _check_rows(grad)
    assert x.dtype == torch.float32
    S, nblocks, log_n = twiddle.shape[:3]
    n = 1 << log_n
    B, _, in_size = x.shape
    out_size = grad.shape[2]
    if d_twiddle is None:
        d_twiddle = torch.empty_like(twiddle)
    if d_x is None:
        d_x = torch.empty(B, S, max(in_size, n), dtype=x.dtype, device=x.device)
    rc = lib().bfly_bw_f32_noalloc(_p(twiddle), _p(x), _i64(x.stride(0)), _i64(x.stride(1)), _p(grad),
                                   _i64(grad.stride(0)), _i64(grad.stride(1)), _p(d_twiddle), _p(d_x), int(B),
                                   int(S), int(log_n), int(nblocks), int(in_size), int(out_size),
                                   int(bool(increasing_stride)), _stream())
    if check and rc != 0:
        raise BflyError(rc, "bfly_bw_f32_noalloc")
    return d_twiddle, d_x, rc


def linear_fw(twiddle, x2d, bias=None, increasing_stride=True, output_size=None, check=True):
    """``bfly_linear_fw_f32``: x2d (batch, in) -> the (batch, nstacks * n) output buffer (the layer's output
    is its first output_size columns, bias included) and the status."""
    assert x2d.is_cuda and x2d.dim() == 2 and x2d.dtype == torch.float32 and x2d.stride(1) == 1
    S, nblocks, log_n = twiddle.shape[:3]
    n = 1 << log_n
    B, in_size = x2d.shape
    output_size = S * n if output_size is None else output_size
    out = torch.empty(B, S * n, dtype=x2d.dtype, device=x2d.device)
    need = fw_workspace_bytes(x2d.dtype, B, S, log_n, nblocks)
    ws = torch.empty(need, dtype=torch.uint8, device=x2d.device) if need > 0 else None
    rc = lib().bfly_linear_fw_f32(_p(twiddle), _p(x2d), _i64(x2d.stride(0)), _p(out), _p(bias), int(B), int(S), int(log_n),
                                  int(nblocks), int(in_size), int(output_size), int(bool(increasing_stride)), _p(ws),
                                  ctypes.c_size_t(need if ws is not None else 0), _stream())
    if check and rc != 0:
        raise BflyError(rc, "bfly_linear_fw_f32")
    return out, rc


def linear_bw(twiddle, x2d, grad2d, increasing_stride=True, with_bias=True, check=True):
    """``bfly_linear_bw_f32``: (d_twiddle, d_input (batch, in), d_bias or None, status).  Status -2
    (BFLY_E_UNSUPPORTED) = the fused route does not apply; nothing was written."""
    S, nblocks, log_n = twiddle.shape[:3]
    B, in_size = x2d.shape
    out_size = grad2d.shape[1]
    d_tw = torch.empty_like(twiddle)
    d_in = torch.empty(B, in_size, dtype=x2d.dtype, device=x2d.device)
    d_b = torch.empty(out_size, dtype=x2d.dtype, device=x2d.device) if with_bias else None
    need = int(lib().bfly_linear_bw_workspace_bytes(int(B), int(S), int(log_n), int(nblocks)))
    if need < 0:
        if check:
            raise BflyError(need, "bfly_linear_bw_workspace_bytes")
        return d_tw, d_in, d_b, need
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=x2d.device)
    rc = lib().bfly_linear_bw_f32(_p(twiddle), _p(x2d), _i64(x2d.stride(0)), _p(grad2d), _i64(grad2d.stride(0)), _p(d_tw),
                                  _p(d_in), _i64(d_in.stride(0)), _p(d_b), int(B), int(S), int(log_n), int(nblocks),
                                  int(in_size), int(out_size), int(bool(increasing_stride)), _p(ws),
                                  ctypes.c_size_t(ws.numel()), _stream())
    if check and rc != 0:
        raise BflyError(rc, "bfly_linear_bw_f32")
    return d_tw, d_in, d_b, rc


def fw_glue(twiddle, x, increasing_stride=True, in_perm=None, out_diag=None, out_perm=None, out_real=False, check=True):
    """``bfly_fw_glue_f32`` / ``bfly_fw_glue_c64``: the forward with gather / diagonal / real-complex
    links folded into its launch.  x float32 with a complex twiddle = real input rows."""
    _check_rows(x)
    S, nblocks, log_n = twiddle.shape[:3]
    n = 1 << log_n
    B, _, in_size = x.shape
    cplx = twiddle.is_complex()
    x_real = cplx and not x.is_complex()
    out = torch.empty((B, S, n), dtype=torch.float32 if (out_real or not cplx) else torch.complex64, device=x.device)
    if cplx:
        rc = lib().bfly_fw_glue_c64(_p(twiddle), _p(x), int(x_real), _i64(x.stride(0)), _i64(x.stride(1)), _p(out), int(out_real),
                                    _p(in_perm), _p(out_diag), _p(out_perm), B, S, log_n, nblocks, in_size, n,
                                    int(increasing_stride), _stream())
    else:
        rc = lib().bfly_fw_glue_f32(_p(twiddle), _p(x), _i64(x.stride(0)), _i64(x.stride(1)), _p(out), _p(in_perm), _p(out_diag),
                                    _p(out_perm), B, S, log_n, nblocks, in_size, n, int(increasing_stride), _stream())
    if check and rc:
        raise BflyError(rc, "bfly_fw_glue")
    return out, rc


def unitary_twiddle_fw(angles, check=True):
    """``bfly_unitary_twiddle_fw``: (..., 4) float32 angles -> (..., 2, 2) complex64 blocks."""
    a = angles.contiguous()
    tw = torch.empty(a.shape[:-1] + (2, 2), dtype=torch.complex64, device=a.device)
    rc = lib().bfly_unitary_twiddle_fw(_p(a), _p(tw), _i64(a.numel() // 4), _stream())
    if check and rc:
        raise BflyError(rc, "bfly_unitary_twiddle_fw")
    return tw, rc


def unitary_twiddle_bw(angles, d_twiddle, check=True):
    """``bfly_unitary_twiddle_bw``: gradient of the angles from the gradient of the blocks."""
    a, g = angles.contiguous(), d_twiddle.contiguous()
    d = torch.empty_like(a)
    rc = lib().bfly_unitary_twiddle_bw(_p(a), _p(g), _p(d), _i64(a.numel() // 4), _stream())
    if check and rc:
        raise BflyError(rc, "bfly_unitary_twiddle_bw")
    return d, rc


def fw_base4(twiddle4, twiddle2, x, increasing_stride=True, output_size=None, out=None, check=True):
    """``bfly4_fw_f32`` / ``bfly4_fw_c64``."""
    _check_rows(x)
    S, nblocks = twiddle4.shape[:2]
    log_n = twiddle4.shape[2] * 2 + twiddle2.shape[2]
    n = 1 << log_n
    B, _, in_size = x.shape
    output_size = n if output_size is None else output_size
    if out is None:
        out = torch.empty(B, S, n, dtype=x.dtype, device=x.device)
    fn = lib().bfly4_fw_f32 if x.dtype == torch.float32 else lib().bfly4_fw_c64
    rc = fn(_p(twiddle4), _p(twiddle2), _p(x), _i64(x.stride(0)), _i64(x.stride(1)), _p(out), int(B),
                            int(S), int(log_n), int(nblocks), int(in_size), int(output_size),
                            int(bool(increasing_stride)), _stream())
    if check and rc != 0:
        raise BflyError(rc, "bfly4_fw")
    return out, rc


def bw_base4(twiddle4, twiddle2, x, grad, increasing_stride=True, workspace=None, check=True):
    """``bfly4_bw_f32`` / ``bfly4_bw_c64``.  Returns (d_twiddle4, d_twiddle2, d_x buffer, status)."""
    _check_rows(x)
    _check_rows(grad)
    S, nblocks = twiddle4.shape[:2]
    log_n = twiddle4.shape[2] * 2 + twiddle2.shape[2]
    n = 1 << log_n
    B, _, in_size = x.shape
    out_size = grad.shape[2]
    d4 = torch.empty_like(twiddle4)
    d2 = torch.empty_like(twiddle2)
    d_x = torch.empty(B, S, max(in_size, n), dtype=x.dtype, device=x.device)
    need = bw_workspace_bytes(x.dtype, B, S, log_n, nblocks, base4=True)
    if need < 0:
        if check:
            raise BflyError(need, "bfly4_bw_workspace_bytes")
        return d4, d2, d_x, need
    if workspace is None and need > 0:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    ws_bytes = 0 if workspace is None else workspace.numel()
    fn = lib().bfly4_bw_f32 if x.dtype == torch.float32 else lib().bfly4_bw_c64
    rc = fn(_p(twiddle4), _p(twiddle2), _p(x), _i64(x.stride(0)), _i64(x.stride(1)), _p(grad),
                            _i64(grad.stride(0)), _i64(grad.stride(1)), _p(d4), _p(d2), _p(d_x), int(B), int(S),
                            int(log_n), int(nblocks), int(in_size), int(out_size), int(bool(increasing_stride)),
                            _p(workspace), ctypes.c_size_t(ws_bytes), _stream())
    if check and rc != 0:
        raise BflyError(rc, "bfly4_bw")
    return d4, d2, d_x, rc


def set_option(name, value):
    """``bfly_set_option``: change a development / test switch of the library (see include/bfly.h)."""
    rc = lib().bfly_set_option(name.encode(), int(value))
    if rc != 0:
        raise BflyError(rc, "bfly_set_option(%s)" % name)


def get_option(name):
    v = ctypes.c_int(0)
    rc = lib().bfly_get_option(name.encode(), ctypes.byref(v))
    if rc != 0:
        raise BflyError(rc, "bfly_get_option(%s)" % name)
    return int(v.value)


def launch_count():
    return int(lib().bfly_launch_count())


def selftest_bounded_wait(polls=4096):
    """``bfly_selftest_bounded_wait``: one warp waits on a barrier that never completes, gives up after `polls` polls."""
    rc = lib().bfly_selftest_bounded_wait(int(polls), _stream())
    if rc:
        raise BflyError(rc, "bfly_selftest_bounded_wait")


def device_error_async(host_flag):
    """``bfly_device_error_async``: enqueue a copy of the give-up flag into `host_flag` (a pinned int32 tensor of
    one element) on the current stream; read it after the next synchronisation."""
    assert host_flag.dtype == torch.int32 and host_flag.numel() == 1 and not host_flag.is_cuda
    rc = lib().bfly_device_error_async(ctypes.c_void_p(host_flag.data_ptr()), _stream())
    if rc:
        raise BflyError(rc, "bfly_device_error_async")


def device_error():
    """Non-zero if a kernel gave up since the last call (its output is invalid): 1 = a bounded wait
    ran out, 2 = misaligned shared-memory window; else 0."""
    rc = int(lib().bfly_device_error())
    if rc < 0:
        raise BflyError(rc, "bfly_device_error")
    return rc


KERNEL_NAMES = ("bfly_fw_kernel", "bfly_bw_kernel", "bfly_fw2_kernel", "bfly_bw2_kernel", "bfly_bw3_kernel")


def profile_enable(on=True):
    lib().bfly_profile_enable(int(bool(on)))


def profile_collect():
    """{kernel name: (launches, total device ms)} for the launches recorded since the last call."""
    n = len(KERNEL_NAMES)
    launches = (ctypes.c_int64 * n)()
    total = (ctypes.c_double * n)()
    rc = lib().bfly_profile_collect(launches, total, n)
    if rc != 0:
        raise BflyError(rc, "bfly_profile_collect")
    return {KERNEL_NAMES[i]: (int(launches[i]), float(total[i])) for i in range(n)}
