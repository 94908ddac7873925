"""Host logic without a GPU: the launch planner and the kernels' per-thread tile routines,
executed thread by thread on the CPU by tests/emul/bfly_emul.cpp behind the same driver
that plans the GPU launches, compared with the oracle.  This checks panels, unit
decomposition, twiddle addressing, padding/slicing and the phase plan of the backward; it
is a test of index arithmetic, not a CPU implementation of the product."""
import ctypes
import math
import os
import subprocess

import pytest
import torch

from conftest import ROOT, assert_rtol_atol, golden_files, load_golden, rel_err, unitary_chain

EMUL_SRC = os.path.join(ROOT, "tests", "emul", "bfly_emul.cpp")
EMUL_LIB = os.path.join(ROOT, "tests", "emul", "libbfly_emul.so")
CSRC = os.path.join(ROOT, "butterfly_b200", "csrc")


@pytest.fixture(scope="module")
def emul():
    deps = [EMUL_SRC] + [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(".h")]
    if not os.path.exists(EMUL_LIB) or os.path.getmtime(EMUL_LIB) < max(os.path.getmtime(f) for f in deps):
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wno-unknown-pragmas", "-I", CSRC,
                               EMUL_SRC, "-o", EMUL_LIB])
    return ctypes.CDLL(EMUL_LIB)


def emul_option(lib, name, value):
    from conftest import library_option
    return library_option(lambda n, v: lib.bfly_emul_set_option(n.encode(), int(v)),
                          lambda n: lib.bfly_emul_get_option(n.encode()), name, value)


def P(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None and t.numel() else 0)


I64 = ctypes.c_int64


def emul_fw(lib, tw2, tw4, x, inc, out_size, log_n, nblocks, base4, threads=64, tail_untouched=True):
    B, S, insz = x.shape
    n = 1 << log_n
    out = torch.full((B, S, n), float("nan"), dtype=x.dtype)
    rc = lib.bfly_emul_fw(int(x.is_complex()), int(base4), P(tw2), P(tw4), P(x), I64(x.stride(0)), I64(x.stride(1)),
                          P(out), B, S, log_n, nblocks, insz, out_size, int(inc), threads)
    assert rc == 0, rc
    # columns >= out_size must stay untouched (a product that runs in several passes uses them as
    # working space)
    if tail_untouched:
        assert torch.isnan(out[:, :, out_size:]).all()
    return out[:, :, :out_size]


def emul_bw(lib, tw2, tw4, x, g, inc, log_n, nblocks, base4, threads=64, sms=7):
    B, S, insz = x.shape
    n = 1 << log_n
    d2 = torch.full_like(tw2, float("nan")) if tw2 is not None else None
    d4 = torch.full_like(tw4, float("nan")) if tw4 is not None else None
    dx = torch.full((B, S, max(insz, n)), float("nan"), dtype=x.dtype)
    g = g.contiguous()
    rc = lib.bfly_emul_bw(int(x.is_complex()), int(base4), P(tw2), P(tw4), P(x), I64(x.stride(0)), I64(x.stride(1)),
                          P(g), I64(g.stride(0)), I64(g.stride(1)), P(d2), P(d4), P(dx), B, S, log_n, nblocks, insz,
                          g.shape[2], int(inc), threads, sms)
    assert rc == 0, rc
    return d2, d4, dx[:, :, :insz]


@pytest.mark.parametrize("dtype", [torch.float32, torch.complex64], ids=["f32", "c64"])
@pytest.mark.parametrize("log_n", [1, 2, 3, 4, 5, 7, 9, 10, 11, 12])
def test_radix2_plan_and_indexing(emul, oracle_mod, dtype, log_n):
    torch.manual_seed(log_n)
    n = 1 << log_n
    shapes = [(n, n), (max(1, n // 2 - 1), max(1, n - 5)), (2 * n + 7, max(1, n // 2 - 2))] if log_n <= 7 else [(n, n)]
    for nb, inc in [(1, True), (1, False), (2, True), (3, False)]:
        if log_n >= 11 and nb == 3:
            continue
        S = 2 if log_n < 8 else 1
        B = 5 if log_n < 10 else 3
        for insz, outsz in shapes:
            tw = torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dtype) / 2 ** 0.5
            x = torch.randn(B, S, insz, dtype=dtype)
            g = torch.randn(B, S, outsz, dtype=dtype)
            thr = 64 if log_n < 10 else 256
            y = emul_fw(emul, tw, None, x, inc, outsz, log_n, nb, False, thr)
            assert rel_err(y, oracle_mod.multiply_fw(tw, x, inc, outsz)) < 2e-5
            d2, _, dx = emul_bw(emul, tw, None, x, g, inc, log_n, nb, False, thr)
            dtr, dxr = oracle_mod.multiply_bw(tw, x, g, inc)
            assert rel_err(d2, dtr) < 2e-5 and rel_err(dx, dxr) < 2e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.complex64], ids=["f32", "c64"])
@pytest.mark.parametrize("log_n", [1, 2, 3, 4, 5, 6, 7, 10, 11])
def test_base4_plan_and_indexing(emul, oracle_mod, log_n, dtype):
    torch.manual_seed(100 + log_n)
    n = 1 << log_n
    for nb, inc in [(1, True), (1, False), (2, True), (3, False)]:
        S, B = 2, 4
        for insz, outsz in [(n, n), (max(1, n // 2 - 1), max(1, n - 5)), (2 * n + 7, max(1, n // 2 - 2))]:
            tw4 = torch.randn(S, nb, log_n // 2, n // 4, 4, 4, dtype=dtype) / 2
            tw2 = torch.randn(S, nb, log_n % 2, n // 2, 2, 2, dtype=dtype) / 2 ** 0.5
            x = torch.randn(B, S, insz, dtype=dtype)
            g = torch.randn(B, S, outsz, dtype=dtype)
            y = emul_fw(emul, tw2, tw4, x, inc, outsz, log_n, nb, True)
            assert rel_err(y, oracle_mod.base4_fw(tw4, tw2, x, inc, outsz)) < 2e-5
            d2, d4, dx = emul_bw(emul, tw2, tw4, x, g, inc, log_n, nb, True)
            d4r, d2r, dxr = oracle_mod.base4_bw(tw4, tw2, x, g, inc)
            assert rel_err(dx, dxr) < 2e-5
            if tw4.numel():
                assert rel_err(d4, d4r) < 2e-5
            if tw2.numel():
                assert rel_err(d2, d2r) < 2e-5


def test_stack_broadcast_and_ragged_slices(emul, oracle_mod):
    torch.manual_seed(7)
    tw = torch.randn(3, 2, 6, 32, 2, 2) / 2 ** 0.5
    x = torch.randn(11, 1, 64).expand(11, 3, 64)  # stride 0 over stacks
    g = torch.randn(11, 3, 64)
    y = emul_fw(emul, tw, None, x, True, 64, 6, 2, False)
    assert rel_err(y, oracle_mod.multiply_fw(tw, x, True)) < 2e-5
    for sms in (1, 3, 7, 64):  # different row-slice splits must give the same sums
        d2, _, dx = emul_bw(emul, tw, None, x, g, True, 6, 2, False, sms=sms)
        dtr, dxr = oracle_mod.multiply_bw(tw, x, g, True)
        assert rel_err(d2, dtr) < 2e-5 and rel_err(dx, dxr) < 2e-5


@pytest.mark.parametrize("logc", [6, 7, 8])
def test_forward_passes_over_panels(emul, oracle_mod, logc):
    """Rows wider than a tile run as several forward launches over panels, in place; the
    fw_logcmax switch forces that path at sizes the emulator handles (the product path takes
    it for rows beyond one SM's shared memory)."""
    with emul_option(emul, "fw_logcmax", logc):
        _forward_passes_over_panels(emul, oracle_mod, logc)


def _forward_passes_over_panels(emul, oracle_mod, logc):
    torch.manual_seed(40 + logc)
    for dtype in (torch.float32, torch.complex64):
        for log_n, nb, inc in [(9, 1, True), (9, 2, False), (10, 2, True), (11, 1, False)]:
            n = 1 << log_n
            for insz, outsz in [(n, n), (n // 2 + 32, n - 64)]:
                S, B = 2, 3
                tw = torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dtype) / 2 ** 0.5
                x = torch.randn(B, S, insz, dtype=dtype)
                g = torch.randn(B, S, outsz, dtype=dtype)
                y = emul_fw(emul, tw, None, x, inc, outsz, log_n, nb, False, 64, tail_untouched=False)
                assert rel_err(y, oracle_mod.multiply_fw(tw, x, inc, outsz)) < 2e-5
                d2, _, dx = emul_bw(emul, tw, None, x, g, inc, log_n, nb, False, 64)
                dtr, dxr = oracle_mod.multiply_bw(tw, x, g, inc)
                assert rel_err(d2, dtr) < 2e-5 and rel_err(dx, dxr) < 2e-5
    # base-4, odd and even log_n (a radix-4 stage needs two panel bits plus 32-column segments)
    for log_n, nb, inc in ([(9, 2, True), (10, 1, False)] if logc >= 7 else []):
        n = 1 << log_n
        tw4 = torch.randn(1, nb, log_n // 2, n // 4, 4, 4) / 2
        tw2 = torch.randn(1, nb, log_n % 2, n // 2, 2, 2) / 2 ** 0.5
        x = torch.randn(3, 1, n)
        y = emul_fw(emul, tw2, tw4, x, inc, n, log_n, nb, True, tail_untouched=False)
        assert rel_err(y, oracle_mod.base4_fw(tw4, tw2, x, inc, n)) < 2e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.complex64], ids=["f32", "c64"])
def test_forward_that_saves_snapshots_feeds_the_backward(emul, oracle_mod, dtype):
    """bfly_fw_*_saving + bfly_bw_*_saved: the forward leaves the phase-boundary activations, the
    backward starts from them; results as from the recomputing pair."""
    torch.manual_seed(77)
    for log_n, nb, inc, thr in [(6, 3, True, 64), (10, 2, False, 256), (11, 2, True, 256), (4, 1, True, 64)]:
        n = 1 << log_n
        for insz, outsz in [(n, n), (max(1, n // 2 - 1), max(1, n - 5))]:
            S, B = 2, 5
            tw = torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dtype) / 2 ** 0.5
            x = torch.randn(B, S, insz, dtype=dtype)
            g = torch.randn(B, S, outsz, dtype=dtype)
            out = torch.full((B, S, n), float("nan"), dtype=dtype)
            d_tw = torch.full_like(tw, float("nan"))
            dx = torch.full((B, S, max(insz, n)), float("nan"), dtype=dtype)
            rc = emul.bfly_emul_fw_bw_saved(int(dtype.is_complex), P(tw), P(x), I64(x.stride(0)), I64(x.stride(1)), P(out),
                                            P(g), I64(g.stride(0)), I64(g.stride(1)), P(d_tw), P(dx), B, S, log_n, nb,
                                            insz, outsz, int(inc), thr, 7)
            assert rc == 0, rc
            assert rel_err(out[:, :, :outsz], oracle_mod.multiply_fw(tw, x, inc, outsz)) < 2e-5
            dtr, dxr = oracle_mod.multiply_bw(tw, x, g, inc)
            assert rel_err(d_tw, dtr) < 2e-5 and rel_err(dx[:, :, :insz], dxr) < 2e-5


def test_backward_in_chunks_of_phases(emul, oracle_mod):
    """More phases than one forward launch has snapshot slots for (here 9 and 11 blocks of 8 stages
    at n = 256): the backward runs in chunks, each with its own forward pass from the input."""
    torch.manual_seed(3)
    log_n, S, B = 8, 2, 5
    n = 1 << log_n
    for nb, inc in [(11, True), (9, False), (19, True)]:
        tw = torch.randn(S, nb, log_n, n // 2, 2, 2) / 2 ** 0.5
        x = torch.randn(B, S, n - 3)
        g = torch.randn(B, S, n - 7)
        # products of more than 40 stage groups run as several forward launches, in place on `out`
        y = emul_fw(emul, tw, None, x, inc, n - 7, log_n, nb, False, 64, tail_untouched=False)
        assert rel_err(y, oracle_mod.multiply_fw(tw, x, inc, n - 7)) < 5e-5
        d2, _, dx = emul_bw(emul, tw, None, x, g, inc, log_n, nb, False, 64)
        dtr, dxr = oracle_mod.multiply_bw(tw, x, g, inc)
        assert rel_err(d2, dtr) < 5e-5 and rel_err(dx, dxr) < 5e-5
    ws = ctypes.c_int64(0)
    assert emul.bfly_emul_bw_plan(0, 0, 16, 1, 10, 9, 1, ctypes.byref(ws)) > 9  # 90 stages: chunked
    assert ws.value == 9 * 16 * 1024 * 4 + 9 * 10 * 512 * 16  # 9 planes + the forward pass's re-ordered twiddles


def test_backward_phase_plan_sizes(emul):
    ws = ctypes.c_int64(0)
    # float: a phase holds at most 8 stages (4 sub-groups of 2) on a panel of 1024 columns
    assert emul.bfly_emul_bw_plan(0, 0, 64, 1, 8, 1, 1, ctypes.byref(ws)) == 1 and ws.value == 0
    assert emul.bfly_emul_bw_plan(0, 0, 64, 1, 10, 1, 1, ctypes.byref(ws)) == 2 and ws.value == 64 * 1024 * 4 + 10 * 512 * 16
    # n = 4096, two blocks: 24 stages = three phases of 8 -> two (B,S,n) float snapshots
    assert emul.bfly_emul_bw_plan(0, 0, 16384, 1, 12, 2, 1, ctypes.byref(ws)) == 3
    assert ws.value == 2 * 16384 * 4096 * 4 + 24 * 2048 * 16  # two snapshots + re-ordered twiddles of the forward pass
    # complex, n >= 1024: panels of 1024 columns, two 2-stage sub-groups (4 stages) per phase
    nph = emul.bfly_emul_bw_plan(1, 0, 8192, 1, 11, 1, 1, ctypes.byref(ws))
    assert nph == 3 and ws.value == 2 * 8192 * 2048 * 8
    # complex, n < 1024: panels of 512 columns, up to 10 one-stage sub-groups per phase
    nph = emul.bfly_emul_bw_plan(1, 0, 64, 1, 9, 2, 1, ctypes.byref(ws))
    assert nph == 2 and ws.value == 64 * 512 * 8
    with emul_option(emul, "bw_c64_kw2", 0):
        nph = emul.bfly_emul_bw_plan(1, 0, 8192, 1, 11, 1, 1, ctypes.byref(ws))
        assert nph == 2 and ws.value == 8192 * 2048 * 8


def test_complex_backward_on_two_stage_subgroups(emul, oracle_mod):
    """complex64 products of n >= 1024 run their backward phases on the tensor-memory kernel's step
    routines with 2-bit windows (two sub-groups of two stages); emulated here against the oracle."""
    torch.manual_seed(13)
    for log_n, nb, B, S, inc in ((10, 1, 9, 1, True), (11, 2, 6, 1, False), (12, 1, 5, 2, True)):
        n = 1 << log_n
        tw = torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=torch.complex64) / 2 ** 0.5
        x = torch.randn(B, S, n - 5, dtype=torch.complex64)
        g = torch.randn(B, S, n - 9, dtype=torch.complex64)
        d2, _, dx = emul_bw(emul, tw, None, x, g, inc, log_n, nb, False, 256)
        dtr, dxr = oracle_mod.multiply_bw(tw, x, g, inc)
        assert rel_err(d2, dtr) < 2e-5 and rel_err(dx, dxr) < 2e-5, (log_n, nb)


def test_twiddle_stacks_beyond_32bit_offsets_are_refused(emul):
    """The kernels address twiddles with 32-bit element offsets inside a stack: the planner and
    the library's size queries refuse a stack of 2^31 elements or more instead of wrapping."""
    from butterfly_b200 import abi
    ws = ctypes.c_int64(0)
    # n = 2^20: a stack holds nblocks * 20 * 2^21 elements -- 51 blocks fit under 2^31, 52 do not
    assert emul.bfly_emul_bw_plan(0, 0, 4, 1, 20, 51, 1, ctypes.byref(ws)) > 0
    assert emul.bfly_emul_bw_plan(0, 0, 4, 1, 20, 52, 1, ctypes.byref(ws)) == -2
    assert emul.bfly_emul_bw_plan(1, 0, 4, 1, 24, 6, 1, ctypes.byref(ws)) == -2
    assert abi.bw_workspace_bytes(torch.float32, 4, 1, 20, 51) > 0
    assert abi.bw_workspace_bytes(torch.float32, 4, 1, 20, 52) == -2
    assert abi.fw_workspace_bytes(torch.float32, 4, 1, 20, 52) == -2
    assert abi.bw_workspace_bytes(torch.float32, 4, 1, 24, 3, base4=True) == -2  # 3 * 12 * 2^22 * 16 elements


@pytest.mark.parametrize("path", golden_files("radix2")[::4], ids=lambda p: p.split("/")[-1])
def test_emulated_kernels_on_golden(emul, path):
    d = load_golden(path)
    y = emul_fw(emul, d["twiddle"], None, d["input"], d["increasing_stride"], d["output_size"], d["log_n"],
                d["nblocks"], False)
    assert rel_err(y, d["output"]) < 2e-5
    d2, _, dx = emul_bw(emul, d["twiddle"], None, d["input"], d["grad"], d["increasing_stride"], d["log_n"],
                        d["nblocks"], False)
    assert rel_err(d2, d["d_twiddle"]) < 2e-5 and rel_err(dx, d["d_input"]) < 2e-5


def test_shared_memory_accesses_are_bank_conflict_free(emul):
    """With 256 threads per CTA, every register-window access of the planned groups (forward) and
    sub-groups (backward) must hit 32 distinct banks per wavefront, for the window widths the
    kernels use by default (3 bits float / 2 bits complex) at the benchmark sizes."""
    for dtype, kmax in ((0, 3), (1, 2)):
        for log_n in (10, 11, 12, 13):
            for nblocks, inc in ((1, 1), (2, 1), (2, 0)):
                deg = emul.bfly_emul_max_conflicts(dtype, 0, log_n, nblocks, inc, kmax)
                assert deg == 1, (dtype, log_n, nblocks, inc, deg)
    # base-4 (float): radix-4 windows of 2 bits
    for log_n in (10, 12, 14):
        assert emul.bfly_emul_max_conflicts(0, 1, log_n, 1, 1, 2) == 1


@pytest.mark.parametrize("log_n", [9, 10, 11, 12])
def test_packed_pair_forward_path(emul, oracle_mod, log_n):
    """Float rows of 512 .. 4096 columns take the packed-pair forward kernel (two columns per
    64-bit register, warps that own a 512-column chunk of the tile).  Its per-thread routines run
    here thread by thread; with the kernel switched off the generic kernel must give the same bits
    (both evaluate a butterfly output as fma(own, x, rn(partner * z)))."""
    torch.manual_seed(700 + log_n)
    emul.bfly_emul_fw2_calls.restype = ctypes.c_long
    n = 1 << log_n
    for nb, inc in [(1, True), (2, False), (3, True)]:
        for B, S, insz, outsz in [(2, 1, n, n), (37, 2, n - 32, n - 64), (9, 3, n + 3, 64)]:
            tw = torch.randn(S, nb, log_n, n // 2, 2, 2) / 2 ** 0.5
            x = torch.randn(B, S, insz)
            before = emul.bfly_emul_fw2_calls()
            y = emul_fw(emul, tw, None, x, inc, outsz, log_n, nb, False, 256)
            assert emul.bfly_emul_fw2_calls() == before + 1
            with emul_option(emul, "fw2", 0):
                y0 = emul_fw(emul, tw, None, x, inc, outsz, log_n, nb, False, 256)
            assert emul.bfly_emul_fw2_calls() == before + 1
            assert torch.equal(y, y0)
            assert rel_err(y, oracle_mod.multiply_fw(tw, x, inc, outsz)) < 2e-5
    # a ragged width (not a multiple of 32 columns) cannot be described to the TMA unit: generic kernel
    x = torch.randn(3, 1, n - 5)
    tw = torch.randn(1, 1, log_n, n // 2, 2, 2) / 2 ** 0.5
    before = emul.bfly_emul_fw2_calls()
    y = emul_fw(emul, tw, None, x, True, n, log_n, 1, False, 256)
    assert emul.bfly_emul_fw2_calls() == before
    assert rel_err(y, oracle_mod.multiply_fw(tw, x, True, n)) < 2e-5


@pytest.mark.parametrize("log_n", [10, 11, 12])
def test_packed_pair_backward_path(emul, oracle_mod, log_n):
    """Float radix-2 phases on full 1024-column panels take the packed-pair backward kernel (two
    columns per 64-bit register, twiddles and accumulators paired in tensor memory).  Its step
    routines run here thread by thread; with the kernel switched off the scalar kernels must give
    the same input gradient bits (same rounding order) and the same twiddle gradient up to the
    order of the row sums."""
    torch.manual_seed(800 + log_n)
    emul.bfly_emul_bw3_calls.restype = ctypes.c_long
    n = 1 << log_n
    for nb, inc in [(1, True), (2, False), (2, True)]:
        for B, S, insz, outsz in [(5, 1, n, n), (23, 2, n - 32, n - 64), (9, 1, n + 32, 64)]:
            tw = torch.randn(S, nb, log_n, n // 2, 2, 2) / 2 ** 0.5
            x = torch.randn(B, S, insz)
            g = torch.randn(B, S, outsz)
            before = emul.bfly_emul_bw3_calls()
            with emul_option(emul, "bw3_min_rows", 0):  # small batches would take the scalar kernel otherwise
                d2, _, dx = emul_bw(emul, tw, None, x, g, inc, log_n, nb, False, 256)
            assert emul.bfly_emul_bw3_calls() > before
            with emul_option(emul, "bw3", 0):
                mid = emul.bfly_emul_bw3_calls()
                d2s, _, dxs = emul_bw(emul, tw, None, x, g, inc, log_n, nb, False, 256)
                assert emul.bfly_emul_bw3_calls() == mid
            dtr, dxr = oracle_mod.multiply_bw(tw, x, g, inc)
            assert torch.equal(dx, dxs)
            assert rel_err(d2, d2s) < 1e-5
            assert rel_err(d2, dtr) < 2e-5 and rel_err(dx, dxr) < 2e-5


@pytest.mark.parametrize("log_n,S", [(10, 4), (11, 2), (12, 1)])
def test_fused_linear_layer(emul, oracle_mod, log_n, S):
    """Butterfly as a linear layer, fused: the forward adds the bias in its store epilogue, the backward
    sums the input gradient over the stacks in its last store and collects the bias gradient from
    the gradient tiles -- against the oracle composed with the reference's PyTorch glue
    (torch_butterfly/butterfly.py:152-169: expand, flatten, slice, add bias)."""
    torch.manual_seed(900 + log_n)
    n = 1 << log_n
    for nb, inc in [(1, True), (2, True), (2, False)]:
        for B, in_size in [(5, n), (23, n - 64)]:
            out_total = S * n
            tw = torch.randn(S, nb, log_n, n // 2, 2, 2) / 2 ** 0.5
            x = torch.randn(B, in_size)
            bias = torch.randn(out_total)
            g = torch.randn(B, out_total)
            # the unfused composition on the oracle
            xe = x.unsqueeze(1).expand(B, S, in_size)
            yr = oracle_mod.multiply_fw(tw, xe, inc).reshape(B, S * n) + bias
            dtr, dxr = oracle_mod.multiply_bw(tw, xe, g.reshape(B, S, n), inc)
            dxr, dbr = dxr.sum(1), g.sum(0)
            out = torch.full((B, S * n), float("nan"))
            rc = emul.bfly_emul_linear_fw(P(tw), P(x), I64(x.stride(0)), P(out), P(bias), B, S, log_n, nb, in_size, out_total, int(inc))
            assert rc == 0
            assert rel_err(out, yr) < 2e-5
            d_tw = torch.full_like(tw, float("nan")); d_in = torch.full((B, in_size), float("nan")); d_b = torch.full((out_total,), float("nan"))
            rc = emul.bfly_emul_linear_bw(P(tw), P(x), I64(x.stride(0)), P(g), I64(g.stride(0)), P(d_tw), P(d_in), I64(d_in.stride(0)),
                                          P(d_b), B, S, log_n, nb, in_size, out_total, int(inc), 7)
            if rc == -2:
                # a phase on strided column segments takes only rows that are whole groups of segments
                # (what the TMA descriptors can express): refused before anything is written
                assert in_size != n and torch.isnan(d_in).all() and torch.isnan(d_tw).all()
                continue
            assert rc == 0
            assert rel_err(d_tw, dtr) < 2e-5 and rel_err(d_in, dxr) < 2e-5 and rel_err(d_b, dbr) < 2e-5
    # a ragged input width is refused before anything is written
    x = torch.randn(8, n - 3); g = torch.randn(8, S * n); d_in = torch.full((8, n - 3), 7.0)
    tw = torch.randn(S, 1, log_n, n // 2, 2, 2)
    d_tw = torch.full_like(tw, 7.0)
    rc = emul.bfly_emul_linear_bw(P(tw), P(x), I64(x.stride(0)), P(g), I64(g.stride(0)), P(d_tw), P(d_in), I64(d_in.stride(0)),
                                  P(None), 8, S, log_n, 1, n - 3, S * n, 1, 7)
    assert rc == -2 and (d_in == 7.0).all() and (d_tw == 7.0).all()


def test_unitary_twiddle_arithmetic(emul):
    """The per-block arithmetic of the unitary twiddle kernels against the reference's chain of
    torch operators and autograd's backward of it."""
    torch.manual_seed(2)
    shape = (2, 2, 5, 16)
    angles = torch.cat([torch.asin(torch.sqrt(torch.rand(shape + (1,)))), torch.rand(shape + (3,)) * 2 * math.pi], dim=-1)
    blocks = angles.numel() // 4
    tw = torch.empty(shape + (2, 2), dtype=torch.complex64)
    emul.bfly_emul_unitary_fw(P(angles), P(tw), I64(blocks))
    a = angles.clone().requires_grad_(True)
    ref = unitary_chain(a)
    assert_rtol_atol(tw, ref.detach(), "unitary twiddle", rtol=1e-6, atol=1e-6)
    # unitary blocks: T T^H = I
    eye = tw @ tw.conj().transpose(-1, -2)
    assert (eye - torch.eye(2)).abs().max() < 1e-6
    g = torch.randn(shape + (2, 2), dtype=torch.complex64)
    ref.backward(g)
    d = torch.empty_like(angles)
    emul.bfly_emul_unitary_bw(P(angles), P(g), P(d), I64(blocks))
    assert_rtol_atol(d, a.grad, "unitary twiddle gradient", rtol=1e-5, atol=1e-6)


def _glue_reference(oracle_mod, tw, x, inc, in_perm, out_diag, out_perm, out_real):
    """The pipeline the glue forward replaces, operator by operator on the oracle."""
    xin = x.to(tw.dtype)
    if in_perm is not None:
        xin = xin[..., in_perm.long()]
    y = oracle_mod.multiply_fw(tw, xin.contiguous(), inc)
    if out_diag is not None:
        y = y * out_diag
    if out_perm is not None:
        y = y[..., out_perm.long()]
    return y.real.contiguous() if out_real else y


@pytest.mark.parametrize("cplx", [False, True])
def test_forward_with_glue_operators(emul, oracle_mod, cplx):
    """Gather before, diagonal and gather after, real input / output: the kernel's passes on the
    tile (emulated thread by thread) against the chain of separate operators."""
    torch.manual_seed(8)
    dtype = torch.complex64 if cplx else torch.float32
    for log_n, nb, B, S in ((6, 1, 5, 1), (9, 2, 9, 2), (11, 1, 3, 1)):
        n = 1 << log_n
        tw = torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dtype) / 2 ** 0.5
        for combo in range(8 if cplx else 4):
            use_in, use_out = bool(combo & 1), bool(combo & 2)
            real_io = bool(combo & 4)
            x = torch.randn(B, S, n, dtype=torch.float32 if real_io else dtype)
            in_perm = torch.randperm(n, dtype=torch.int32) if use_in else None
            out_perm = torch.randperm(n, dtype=torch.int32) if use_out else None
            out_diag = torch.randn(n, dtype=dtype) if use_out else None
            out = torch.full((B, S, n), float("nan"), dtype=torch.float32 if real_io else dtype)
            rc = emul.bfly_emul_fw_glue(int(cplx), P(tw), P(x), int(real_io), I64(x.stride(0)), I64(x.stride(1)), P(out), int(real_io),
                                        P(in_perm), P(out_diag), P(out_perm), B, S, log_n, nb, n, n, 1, 256)
            assert rc == 0, (log_n, combo, rc)
            want = _glue_reference(oracle_mod, tw, x, True, in_perm, out_diag, out_perm, real_io)
            assert_rtol_atol(out, want, "glue forward n=%d combo=%d" % (n, combo), rtol=1e-4, atol=1e-4)
    # rows wider than a tile, gathers on ragged sizes: refused
    n = 1 << 13
    tw = torch.randn(1, 1, 13, n // 2, 2, 2)
    x = torch.randn(2, 1, n)
    perm = torch.randperm(n, dtype=torch.int32)
    assert emul.bfly_emul_fw_glue(0, P(tw), P(x), 0, I64(n), I64(n), P(torch.empty(2, 1, n)), 0, P(perm), None, None,
                                  2, 1, 13, 1, n, n, 1, 256) == -2
    tw = torch.randn(1, 1, 6, 32, 2, 2)
    x = torch.randn(2, 1, 64)
    perm = torch.randperm(64, dtype=torch.int32)
    assert emul.bfly_emul_fw_glue(0, P(tw), P(x), 0, I64(64), I64(64), P(torch.empty(2, 1, 64)), 0, P(perm), None, None,
                                  2, 1, 6, 1, 60, 64, 1, 256) == -1


def test_packed_pair_forward_on_wide_rows(emul, oracle_mod):
    """float32 rows of 8192 columns run the packed-pair forward in one launch (512-thread CTAs); rows of
    16384 columns pass by pass on 4096-column panels (contiguous for the low bits, 32-column blocks at
    a stride for the top bits); both also as the backward's snapshot pass.  Input that the kernel's
    descriptors cannot cover falls back to the generic kernel."""
    torch.manual_seed(21)
    for log_n, nb, B, inc in ((13, 2, 5, True), (13, 1, 3, False), (14, 2, 2, True)):
        n = 1 << log_n
        tw = torch.randn(1, nb, log_n, n // 2, 2, 2) / 2 ** 0.5
        x = torch.randn(B, 1, n)
        calls = emul.bfly_emul_fw2_calls()
        y = emul_fw(emul, tw, None, x, inc, n - 96, log_n, nb, False, 256, tail_untouched=False)
        assert emul.bfly_emul_fw2_calls() - calls == (1 if log_n == 13 else 3), (log_n, nb)
        assert rel_err(y, oracle_mod.multiply_fw(tw, x, inc, n - 96)) < 2e-5
        g = torch.randn(B, 1, n)
        calls = emul.bfly_emul_fw2_calls()
        d2, _, dx = emul_bw(emul, tw, None, x, g, inc, log_n, nb, False, 256)
        assert emul.bfly_emul_fw2_calls() > calls  # the snapshot pass
        dtr, dxr = oracle_mod.multiply_bw(tw, x, g, inc)
        assert rel_err(d2, dtr) < 2e-5 and rel_err(dx, dxr) < 2e-5
    # two stacks of 8192 columns: still one launch; with the one-launch path refused (input not a
    # multiple of 32 columns) a single stack cannot take the panel passes either: generic passes
    n = 1 << 13
    tw2 = torch.randn(2, 1, 13, n // 2, 2, 2) / 2 ** 0.5
    x2 = torch.randn(3, 2, n)
    calls = emul.bfly_emul_fw2_calls()
    y2 = emul_fw(emul, tw2, None, x2, False, n, 13, 1, False, 256)
    assert emul.bfly_emul_fw2_calls() - calls == 1
    assert rel_err(y2, oracle_mod.multiply_fw(tw2, x2, False, n)) < 2e-5
    tw = torch.randn(1, 1, 13, n // 2, 2, 2) / 2 ** 0.5
    x = torch.randn(3, 1, n - 65)
    calls = emul.bfly_emul_fw2_calls()
    y = emul_fw(emul, tw, None, x, True, n, 13, 1, False, 256)
    assert emul.bfly_emul_fw2_calls() == calls
    assert rel_err(y, oracle_mod.multiply_fw(tw, x, True, n)) < 2e-5
