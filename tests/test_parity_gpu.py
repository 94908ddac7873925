"""Parity of the CUDA path with the CPU oracle, called through the C ABI of
libbfly_b200.so (butterfly_b200.abi) and through the torch operators.

Tolerance: the product is float32 / complex64 arithmetic; the requirement is agreement
within rtol 1e-5 / atol 1e-5 per component.  Small cases are checked at a relative error
(max |a-b| / max |b|) of 2e-5 against the oracle, whose own operation order differs from
the GPU's (separately rounded products vs fused multiply-adds); large cases use the
rtol/atol form directly.
"""
import pytest
import torch

from conftest import abi_option, assert_rtol_atol, assert_sum_accuracy, golden_files, load_golden, rel_err, tol_ratio

pytestmark = pytest.mark.gpu

TOL = 2e-5


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda", 0)


@pytest.fixture(scope="module")
def abi():
    from butterfly_b200 import abi as a
    return a


def within_tol(a, b, rtol=1e-5, atol=1e-5):
    a = torch.view_as_real(a) if a.is_complex() else a
    b = torch.view_as_real(b) if b.is_complex() else b
    return ((a - b).abs() <= atol + rtol * b.abs())


def assert_close_1e5(a, b, name="", what=""):
    """rtol 1e-5 / atol 1e-5 per component, strictly -- except for configuration 3: with
    un-normalised DFT twiddles (|y| up to ~60) two valid float32 evaluation orders of the same
    product (fused vs separately rounded multiply-adds) differ by more than that on ~0.1 % of
    the components, so there 0.2 % of components may reach 5x the tolerance, none beyond."""
    ratio = tol_ratio(a, b)
    if name == "cfg3":
        assert (ratio <= 1).float().mean().item() >= 1 - 2e-3, what + ": too many components outside rtol/atol 1e-5"
        assert ratio.max().item() <= 5.0, what + ": a component is off by %.1fx the tolerance" % ratio.max().item()
    else:
        assert_rtol_atol(a, b, what or name)


@pytest.mark.parametrize("path", golden_files("radix2"), ids=lambda p: p.split("/")[-1])
def test_golden_radix2_through_c_abi(abi, dev, oracle_mod, path):
    d = load_golden(path)
    tw, x, g = d["twiddle"].to(dev), d["input"].to(dev), d["grad"].to(dev)
    n = 1 << d["log_n"]
    before = abi.launch_count()
    out, _ = abi.fw(tw, x, d["increasing_stride"], d["output_size"])
    d_tw, d_x, _ = abi.bw(tw, x, g, d["increasing_stride"])
    torch.cuda.synchronize()
    assert abi.launch_count() > before  # the CUDA kernels ran
    assert rel_err(out[:, :, :d["output_size"]], d["output"]) < TOL
    assert rel_err(d_tw, d["d_twiddle"]) < TOL
    ref_dx = d["d_input"]
    assert rel_err(d_x[:, :, :d["input_size"]], ref_dx) < TOL
    # and per component, at the tolerance the product is specified to
    assert_rtol_atol(out[:, :, :d["output_size"]], d["output"], "output")
    assert_rtol_atol(d_x[:, :, :d["input_size"]], ref_dx, "d_input")
    try:
        assert_rtol_atol(d_tw, d["d_twiddle"], "d_twiddle")
    except AssertionError:
        # the partial sums of the CTAs are added in an order that changes from run to run; an entry that
        # lands outside the per-component tolerance must still be as close to the double-precision
        # gradient as the float32 reference is
        hi = torch.complex128 if d["complex"] else torch.float64
        dt64, _ = oracle_mod.multiply_bw(d["twiddle"].to(hi), d["input"].to(hi), d["grad"].to(hi), d["increasing_stride"])
        assert_sum_accuracy(d_tw, d["d_twiddle"], dt64, "d_twiddle")
    if d["input_size"] > n:
        assert (d_x[:, :, n:d["input_size"]] == 0).all()


@pytest.mark.parametrize("path", [p for p in golden_files("base4") if "_f32_" in p or "_c64_" in p],
                         ids=lambda p: p.split("/")[-1])
def test_golden_base4_through_c_abi(abi, dev, oracle_mod, path):
    d = load_golden(path)
    t4, t2, x, g = d["twiddle4"].to(dev), d["twiddle2"].to(dev), d["input"].to(dev), d["grad"].to(dev)
    out, _ = abi.fw_base4(t4, t2, x, d["increasing_stride"], d["output_size"])
    d4, d2, d_x, _ = abi.bw_base4(t4, t2, x, g, d["increasing_stride"])
    assert rel_err(out[:, :, :d["output_size"]], d["output"]) < TOL
    assert rel_err(d_x[:, :, :d["input_size"]], d["d_input"]) < TOL
    assert_rtol_atol(out[:, :, :d["output_size"]], d["output"], "output")
    assert_rtol_atol(d_x[:, :, :d["input_size"]], d["d_input"], "d_input")
    hi = torch.complex128 if d["complex"] else torch.float64
    for got, name, which in ((d4, "d_twiddle4", 0), (d2, "d_twiddle2", 1)):
        if not got.numel():
            continue
        assert rel_err(got, d[name]) < TOL
        try:
            assert_rtol_atol(got, d[name], name)
        except AssertionError:  # summation order of the CTAs' partial sums: grade against the double-precision gradient
            g64 = oracle_mod.base4_bw(d["twiddle4"].to(hi), d["twiddle2"].to(hi), d["input"].to(hi), d["grad"].to(hi),
                                      d["increasing_stride"])
            assert_sum_accuracy(got, d[name], g64[which], name)


@pytest.mark.parametrize("dtype", [torch.float32, torch.complex64], ids=["f32", "c64"])
@pytest.mark.parametrize("log_n", [1, 2, 3, 4, 6, 8, 9, 10, 11, 12, 13, 14])
def test_sweep_against_oracle(abi, dev, oracle_mod, dtype, log_n):
    """Same sweep as the reference's tests/test_multiply.py:19-90 (both stride orders, several blocks and
    stacks, input padding / output slicing), extended over n = 2 .. 16384 and ragged batches."""
    torch.manual_seed(log_n)
    n = 1 << log_n
    for nb, inc in [(1, True), (2, False), (3, True)]:
        if log_n >= 13 and nb == 3:
            continue
        S = 2
        B = 37 if log_n <= 10 else 9
        shapes = [(n, n), (max(1, n // 2 - 1), max(1, n - 5)), (2 * n + 7, max(1, n // 2 - 2))]
        if log_n >= 13:
            shapes = shapes[:2]
        for insz, outsz in shapes:
            tw = torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dtype) / 2 ** 0.5
            x = torch.randn(B, S, insz, dtype=dtype)
            g = torch.randn(B, S, outsz, dtype=dtype)
            yr = oracle_mod.multiply_fw(tw, x, inc, outsz)
            dtr, dxr = oracle_mod.multiply_bw(tw, x, g, inc)
            out, _ = abi.fw(tw.to(dev), x.to(dev), inc, outsz)
            d_tw, d_x, _ = abi.bw(tw.to(dev), x.to(dev), g.to(dev), inc)
            if dtype == torch.float32 and log_n >= 10:
                # small batches take the scalar phase kernel; the packed-pair one must agree with it:
                # the same input gradient bits, the twiddle gradient up to the order of the row sums
                with abi_option("bw3_min_rows", 0):
                    d_tw3, d_x3, _ = abi.bw(tw.to(dev), x.to(dev), g.to(dev), inc)
                assert torch.equal(d_x3[:, :, :insz], d_x[:, :, :insz]) and rel_err(d_tw3, d_tw) < 1e-5
            assert rel_err(out[:, :, :outsz], yr) < TOL, (nb, inc, insz, outsz)
            assert rel_err(d_tw, dtr) < TOL, (nb, inc, insz, outsz)
            assert rel_err(d_x[:, :, :insz], dxr) < TOL, (nb, inc, insz, outsz)
            what = "n=%d nb=%d inc=%s in=%d out=%d" % (n, nb, inc, insz, outsz)
            assert_rtol_atol(out[:, :, :outsz], yr, what + " output")
            assert_rtol_atol(d_x[:, :, :insz], dxr, what + " d_input")
            # a sum over the batch: its float32 rounding depends on the order of the terms, so it is
            # graded against the double-precision oracle (as close to it as the float32 oracle is,
            # or within 1e-5 of the gradient's scale)
            hi = torch.complex128 if dtype == torch.complex64 else torch.float64
            dt64, _ = oracle_mod.multiply_bw(tw.to(hi), x.to(hi), g.to(hi), inc)
            assert_sum_accuracy(d_tw, dtr, dt64, what + " d_twiddle")


@pytest.mark.parametrize("dtype,log_n", [(torch.float32, 16), (torch.complex64, 15), (torch.float32, 17)],
                         ids=["f32-65536", "c64-32768", "f32-131072"])
def test_rows_wider_than_one_sm(abi, dev, oracle_mod, dtype, log_n):
    """Rows beyond one SM's shared memory (n > 32768 float, > 16384 complex): the forward runs as
    several passes over column panels, the backward's snapshot pass likewise."""
    torch.manual_seed(log_n)
    n = 1 << log_n
    B, S = 5, 1
    for nb, inc in [(1, True), (2, False)]:
        if log_n >= 17 and nb == 2:
            continue
        for insz, outsz in [(n, n), (n // 2 + 96, n - 160)]:
            tw = torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dtype) / 2 ** 0.5
            x = torch.randn(B, S, insz, dtype=dtype)
            g = torch.randn(B, S, outsz, dtype=dtype)
            yr = oracle_mod.multiply_fw(tw, x, inc, outsz)
            dtr, dxr = oracle_mod.multiply_bw(tw, x, g, inc)
            out, _ = abi.fw(tw.to(dev), x.to(dev), inc, outsz)
            d_tw, d_x, _ = abi.bw(tw.to(dev), x.to(dev), g.to(dev), inc)
            assert rel_err(out[:, :, :outsz], yr) < TOL, (nb, inc, insz, outsz)
            assert rel_err(d_tw, dtr) < TOL, (nb, inc, insz, outsz)
            assert rel_err(d_x[:, :, :insz], dxr) < TOL, (nb, inc, insz, outsz)


@pytest.mark.parametrize("log_n,S", [(12, 3), (10, 2)], ids=["n4096", "n1024"])
def test_tma_tile_path_edges(abi, dev, oracle_mod, log_n, S):
    """Shapes whose tiles travel through the TMA unit (4096- and 1024-column float rows), at the
    edges the descriptors have to get right: stack-broadcast input, rows with a padded pitch,
    zero-padded input, sliced output, batches that end inside a tile.  The per-thread copy path
    (option tma = 0, which also means the generic forward kernel) must give the same bits, and
    both must match the oracle."""
    torch.manual_seed(900 + log_n)
    n = 1 << log_n
    nb = 2
    tw = (torch.randn(S, nb, log_n, n // 2, 2, 2) / 2 ** 0.5)
    cases = []
    B = 53  # not a multiple of any tile height
    xb = torch.randn(B, 1, n).expand(B, S, n)                       # stack stride 0
    cases.append(("broadcast", xb, n))
    wide = torch.randn(B, S, n + 64)
    cases.append(("pitched rows", wide[:, :, :n], n - 96))           # row pitch n + 64, sliced output
    cases.append(("padded input", torch.randn(B, S, n // 2 + 32), n))  # zero fill beyond the input
    cases.append(("two rows", torch.randn(2, S, n), n))               # fewer rows than a batch of the backward
    for name, x, outsz in cases:
        g = torch.randn(x.shape[0], S, outsz)
        yr = oracle_mod.multiply_fw(tw, x, True, outsz)
        dtr, dxr = oracle_mod.multiply_bw(tw, x, g, True)
        xd = x.to(dev) if name != "pitched rows" else wide.to(dev)[:, :, :n]
        if name == "broadcast":
            xd = xb[:, :1].to(dev).expand(B, S, n)
        res = {}
        for tma in ("1", "0"):
            with abi_option("tma", int(tma)):
                out, _ = abi.fw(tw.to(dev), xd, True, outsz)
                d_tw, d_x, _ = abi.bw(tw.to(dev), xd, g.to(dev), True)
                torch.cuda.synchronize()
            res[tma] = (out[:, :, :outsz].clone(), d_tw.clone(), d_x.clone())
        assert abi.device_error() == 0
        assert torch.equal(res["1"][0], res["0"][0]), name
        assert torch.equal(res["1"][2], res["0"][2]), name
        assert rel_err(res["1"][1], res["0"][1]) < 1e-5, name
        assert rel_err(res["1"][0], yr) < TOL, name
        assert rel_err(res["1"][1], dtr) < TOL, name
        assert rel_err(res["1"][2][:, :, :x.shape[2]], dxr) < TOL, name


@pytest.mark.parametrize("dtype", [torch.float32, torch.complex64], ids=["f32", "c64"])
def test_saving_forward_and_saved_backward(abi, dev, oracle_mod, dtype):
    """bfly_fw_*_saving / bfly_bw_*_saved through the C ABI, and the autograd operator that uses
    them: same bits as the recomputing pair for output and d_input (same arithmetic, the activations
    are stored instead of recomputed), d_twiddle up to the order of the final adds."""
    import butterfly_b200 as bb
    torch.manual_seed(5)
    for log_n, nb, inc, B in [(12, 2, True, 37), (10, 3, False, 64), (13, 1, True, 9), (5, 1, True, 3)]:
        n = 1 << log_n
        S = 2
        for insz, outsz in [(n, n), (n // 2 + 32 if n >= 64 else n, n - 32 if n >= 64 else n)]:
            tw = (torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dtype) / 2 ** 0.5).to(dev)
            x = torch.randn(B, S, insz, dtype=dtype).to(dev)
            g = torch.randn(B, S, outsz, dtype=dtype).to(dev)
            y0, _ = abi.fw(tw, x, inc, outsz)
            dt0, dx0, _ = abi.bw(tw, x, g, inc)
            y1, snaps, _ = abi.fw_saving(tw, x, inc, outsz)
            dt1, dx1, _ = abi.bw_saved(tw, x, g, snaps, inc)
            torch.cuda.synchronize()
            assert torch.equal(y0[:, :, :outsz], y1[:, :, :outsz])
            assert torch.equal(dx0[:, :, :insz], dx1[:, :, :insz])
            assert rel_err(dt1, dt0) < 1e-5
            # autograd operator, saving on and off
            res = {}
            for mode in ("1", "0"):
                with abi_option("autograd_save", int(mode)):
                    twp = tw.clone().requires_grad_(True)
                    xp = x.clone().requires_grad_(True)
                    y = bb.butterfly_multiply(twp, xp, inc, outsz)
                    y.backward(g)
                res[mode] = (y.detach(), twp.grad, xp.grad)
            assert torch.equal(res["1"][0], res["0"][0]) and torch.equal(res["1"][2], res["0"][2])
            assert rel_err(res["1"][1], res["0"][1]) < 1e-5
            assert torch.equal(res["1"][0], y0[:, :, :outsz]) and torch.equal(res["1"][2], dx0[:, :, :insz])


@pytest.mark.parametrize("dtype", [torch.float32, torch.complex64], ids=["f32", "c64"])
def test_many_blocks_backward_in_chunks(abi, dev, oracle_mod, dtype):
    """More backward phases than one forward launch has snapshot slots for (10 blocks at n = 1024:
    100 stages): the backward runs in chunks of phases, each with its own forward pass."""
    torch.manual_seed(31)
    log_n, nb, S, B = 10, 10, 1, 19
    n = 1 << log_n
    for inc in (True, False):
        tw = torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dtype) / 2 ** 0.5
        x = torch.randn(B, S, n, dtype=dtype)
        g = torch.randn(B, S, n - 32, dtype=dtype)
        yr = oracle_mod.multiply_fw(tw, x, inc, n - 32)
        dtr, dxr = oracle_mod.multiply_bw(tw, x, g, inc)
        out, _ = abi.fw(tw.to(dev), x.to(dev), inc, n - 32)
        d_tw, d_x, _ = abi.bw(tw.to(dev), x.to(dev), g.to(dev), inc)
        y2, snaps, _ = abi.fw_saving(tw.to(dev), x.to(dev), inc, n - 32)
        dt2, dx2, _ = abi.bw_saved(tw.to(dev), x.to(dev), g.to(dev), snaps, inc)
        for a, b in ((out[:, :, :n - 32], yr), (d_tw, dtr), (d_x, dxr), (y2[:, :, :n - 32], yr), (dt2, dtr), (dx2, dxr)):
            assert rel_err(a, b) < 1e-4  # 100 stages of float32 round-off


@pytest.mark.parametrize("logc", [7, 9, 10])
def test_forward_passes_forced_at_small_n(abi, dev, oracle_mod, logc):
    """The multi-pass forward (option fw_logcmax) must give what the one-pass
    forward gives, for radix-2 and base-4 products, float and complex."""
    torch.manual_seed(logc)
    log_n, B, S = 12, 33, 2
    n = 1 << log_n
    for dtype in (torch.float32, torch.complex64):
        for nb, inc in [(2, True), (1, False)]:
            tw = (torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dtype) / 2 ** 0.5).to(dev)
            x = torch.randn(B, S, n - 64, dtype=dtype).to(dev)
            g = torch.randn(B, S, n - 32, dtype=dtype).to(dev)
            y1, _ = abi.fw(tw, x, inc, n - 32)
            dt1, dx1, _ = abi.bw(tw, x, g, inc)
            with abi_option("fw_logcmax", logc):
                y2, _ = abi.fw(tw, x, inc, n - 32)
                dt2, dx2, _ = abi.bw(tw, x, g, inc)
            torch.cuda.synchronize()
            assert torch.equal(y1[:, :, :n - 32], y2[:, :, :n - 32])  # same arithmetic, different tiling
            assert rel_err(dt2, dt1) < 1e-5 and torch.equal(dx1, dx2)
    tw4 = (torch.randn(S, 2, log_n // 2, n // 4, 4, 4) / 2).to(dev)
    tw2 = torch.zeros(S, 2, 0, n // 2, 2, 2, device=dev)
    x = torch.randn(B, S, n).to(dev)
    y1, _ = abi.fw_base4(tw4, tw2, x, True, n)
    with abi_option("fw_logcmax", logc):
        y2, _ = abi.fw_base4(tw4, tw2, x, True, n)
    torch.cuda.synchronize()
    assert rel_err(y2, y1) < 1e-6  # window widths (and so the FMA grouping) may differ between tilings


@pytest.mark.parametrize("dtype", [torch.float32, torch.complex64], ids=["f32", "c64"])
@pytest.mark.parametrize("log_n", [1, 2, 3, 6, 7, 10, 11, 14])
def test_base4_sweep_against_oracle(abi, dev, oracle_mod, log_n, dtype):
    torch.manual_seed(50 + log_n)
    n = 1 << log_n
    for nb, inc in [(1, True), (2, False), (3, True)]:
        if log_n >= 14 and nb > 1:
            continue
        S, B = (2, 19) if log_n < 14 else (1, 5)
        for insz, outsz in [(n, n), (max(1, n // 2 - 1), max(1, n - 5))]:
            tw4 = torch.randn(S, nb, log_n // 2, n // 4, 4, 4, dtype=dtype) / 2
            tw2 = torch.randn(S, nb, log_n % 2, n // 2, 2, 2, dtype=dtype) / 2 ** 0.5
            x = torch.randn(B, S, insz, dtype=dtype)
            g = torch.randn(B, S, outsz, dtype=dtype)
            yr = oracle_mod.base4_fw(tw4, tw2, x, inc, outsz)
            d4r, d2r, dxr = oracle_mod.base4_bw(tw4, tw2, x, g, inc)
            out, _ = abi.fw_base4(tw4.to(dev), tw2.to(dev), x.to(dev), inc, outsz)
            d4, d2, d_x, _ = abi.bw_base4(tw4.to(dev), tw2.to(dev), x.to(dev), g.to(dev), inc)
            assert rel_err(out[:, :, :outsz], yr) < TOL
            assert rel_err(d_x[:, :, :insz], dxr) < TOL
            if tw4.numel():
                assert rel_err(d4, d4r) < TOL
            if tw2.numel():
                assert rel_err(d2, d2r) < TOL


def test_large_batch_twiddle_gradient(abi, dev, oracle_mod):
    """Large batch (the reference uses batch 8192 "for race conditions", tests/test_multiply.py:20):
    d_twiddle sums 8192 terms; compare with the double-precision oracle."""
    torch.manual_seed(3)
    B, S, log_n, nb = 8192, 2, 9, 3
    n = 1 << log_n
    tw = torch.randn(S, nb, log_n, n // 2, 2, 2) / 2 ** 0.5
    x = torch.randn(B, S, n)
    g = torch.randn(B, S, n)
    dtr, dxr = oracle_mod.multiply_bw(tw.double(), x.double(), g.double(), True)
    d_tw, d_x, _ = abi.bw(tw.to(dev), x.to(dev), g.to(dev), True)
    d_tw2, d_x2, _ = abi.bw(tw.to(dev), x.to(dev), g.to(dev), True)
    assert rel_err(d_x.double(), dxr) < TOL
    assert rel_err(d_tw.double(), dtr) < TOL
    assert torch.equal(d_x, d_x2)                 # d_input is deterministic
    assert rel_err(d_tw2, d_tw) < 1e-5            # d_twiddle up to the order of the final atomic adds


def test_edge_cases(abi, dev, oracle_mod):
    torch.manual_seed(4)
    # empty batch
    tw = torch.randn(1, 1, 4, 8, 2, 2, device=dev)
    x = torch.empty(0, 1, 16, device=dev)
    out, rc = abi.fw(tw, x, True)
    assert rc == 0 and out.shape == (0, 1, 16)
    d_tw, d_x, rc = abi.bw(tw, x, torch.empty(0, 1, 16, device=dev), True)
    assert rc == 0 and (d_tw == 0).all()
    # stack-broadcast input (stride 0) and batch not a multiple of anything
    tw = (torch.randn(4, 2, 10, 512, 2, 2) / 2 ** 0.5)
    xb = torch.randn(77, 1, 1000)
    g = torch.randn(77, 4, 1024)
    xe = xb.expand(77, 4, 1000)
    yr = oracle_mod.multiply_fw(tw, xe, True)
    dtr, dxr = oracle_mod.multiply_bw(tw, xe, g, True)
    xd = xb.to(dev).expand(77, 4, 1000)
    out, _ = abi.fw(tw.to(dev), xd, True)
    d_tw, d_x, _ = abi.bw(tw.to(dev), xd, g.to(dev), True)
    assert rel_err(out, yr) < TOL and rel_err(d_tw, dtr) < TOL and rel_err(d_x[:, :, :1000], dxr) < TOL
    # status codes instead of exceptions or faults
    _, rc = abi.fw(tw.to(dev), xd, True, output_size=2000, check=False)
    assert rc == -1
    ws_small = torch.empty(16, dtype=torch.uint8, device=dev)
    big = torch.randn(1, 2, 12, 2048, 2, 2, device=dev)
    xx = torch.randn(4, 1, 4096, device=dev)
    _, _, rc = abi.bw(big, xx, xx, True, workspace=ws_small, check=False)
    assert rc == -4
    misaligned = torch.randn(1 * 1 * 4 * 8 * 4 + 1, device=dev)[1:].view(1, 1, 4, 8, 2, 2)
    _, rc = abi.fw(misaligned, torch.randn(2, 1, 16, device=dev), True, check=False)
    assert rc == -3


def test_operator_semantics(dev, oracle_mod):
    """Behaviour of the torch operators that callers rely on (csrc/butterfly.cpp:20-53, 56-93,
    torch_butterfly/butterfly.py:133-146 of the reference)."""
    import butterfly_b200 as bb
    torch.manual_seed(5)
    S, nb, log_n, B = 2, 2, 6, 10
    n = 64
    tw = (torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=torch.complex64) / 2 ** 0.5)
    x = torch.randn(B, S, n, dtype=torch.complex64)
    twd, xd = tw.to(dev), x.to(dev)
    # output_size=None -> n; sliced output keeps shape (B, S, output_size)
    assert bb.butterfly_multiply(twd, xd, True).shape == (B, S, n)
    assert bb.butterfly_multiply(twd, xd, True, 17).shape == (B, S, 17)
    with pytest.raises(RuntimeError, match="output_size must be <= n"):
        bb.butterfly_multiply(twd, xd, True, n + 1)
    with pytest.raises(RuntimeError, match="twiddle must have shape"):
        bb.butterfly_multiply(twd[:1], xd, True)
    with pytest.raises(RuntimeError, match="not implemented for"):
        bb.butterfly_multiply(twd.real.double().contiguous(), xd.real.double().contiguous(), True)
    # lazily conjugated and transposed/flipped twiddle views (what Butterfly.forward passes)
    y = bb.butterfly_multiply(twd.conj(), xd, True)
    assert rel_err(y, oracle_mod.multiply_fw(tw.conj(), x, True)) < TOL
    twt = twd.transpose(-1, -2).flip([1, 2])
    y = bb.butterfly_multiply(twt, xd, False)
    assert rel_err(y, oracle_mod.multiply_fw(tw.transpose(-1, -2).flip([1, 2]).contiguous(), x, False)) < TOL
    # autograd: gradients reach both arguments, d_twiddle is returned with twiddle's shape
    twp = twd.clone().requires_grad_(True)
    xp = xd.clone().requires_grad_(True)
    g = torch.randn(B, S, 40, dtype=torch.complex64)
    bb.butterfly_multiply(twp, xp, True, 40).backward(g.to(dev))
    dtr, dxr = oracle_mod.multiply_bw(tw, x, g, True)
    assert twp.grad.shape == tw.shape and rel_err(twp.grad, dtr) < TOL and rel_err(xp.grad, dxr) < TOL
    # results do not depend on how many stacks are processed together (ButterflyBmm exactness,
    # tests/test_butterfly.py:237-266 of the reference)
    y_all = bb.butterfly_multiply(twd, xd, True)
    for s in range(S):
        y_one = bb.butterfly_multiply(twd[s:s + 1].contiguous(), xd[:, s:s + 1].contiguous(), True)
        assert torch.equal(y_all[:, s:s + 1], y_one)


def test_bounded_wait_gives_up_and_reports(abi, dev, oracle_mod):
    """A wait that cannot complete runs out of its bound, raises the device flag and returns; the
    host reads the status once, and the device keeps working."""
    assert abi.device_error() == 0
    abi.selftest_bounded_wait(4096)
    flag = torch.zeros(1, dtype=torch.int32).pin_memory()
    abi.device_error_async(flag)       # the non-synchronising read: value valid after the caller's own sync
    torch.cuda.synchronize()
    assert int(flag.item()) == 1
    assert abi.device_error() == 1
    assert abi.device_error() == 0   # read and cleared
    tw = torch.randn(1, 1, 9, 256, 2, 2) / 2 ** 0.5
    x = torch.randn(16, 1, 512)
    y, rc = abi.fw(tw.to(dev), x.to(dev), True)
    assert rc == 0 and rel_err(y, oracle_mod.multiply_fw(tw, x, True)) < TOL
    assert abi.device_error() == 0


def test_forward_without_grad_mode_saves_nothing(dev):
    """A forward under torch.no_grad() on parameters that require grad is the plain forward: the
    same launches and no snapshot planes, where the recording forward of a two-block product
    keeps (batch, nstacks, n) planes for the backward.  The two give the same bits."""
    import butterfly_b200 as bb
    from butterfly_b200 import abi
    torch.manual_seed(11)
    B, S, nb, log_n = 4096, 1, 2, 12
    n = 1 << log_n
    tw = (torch.randn(S, nb, log_n, n // 2, 2, 2, device=dev) / 2 ** 0.5).requires_grad_(True)
    x = torch.randn(B, S, n, device=dev)
    plane = B * S * n * 4

    def run(fn):
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        before, launches = torch.cuda.memory_allocated(), abi.launch_count()
        y = fn()
        torch.cuda.synchronize()
        return y, abi.launch_count() - launches, torch.cuda.max_memory_allocated() - before

    with abi_option("autograd_save", 1):
        plain = lambda: bb.butterfly_multiply_fw(tw.detach(), x, True)
        run(plain)  # first call: lazy initialisation out of the way
        y0, l0, m0 = run(plain)
        with torch.no_grad():
            y1, l1, m1 = run(lambda: bb.butterfly_multiply(tw, x, True))
        y2, l2, m2 = run(lambda: bb.butterfly_multiply(tw, x, True))
    assert torch.equal(y0, y1) and torch.equal(y0, y2)
    assert not y1.requires_grad and y2.requires_grad
    assert l1 == l0 and m1 == m0, (l0, l1, m0, m1)
    assert m0 < 2 * plane            # the output and the re-ordered twiddles
    assert m2 >= m0 + 2 * plane - 4096  # the recording forward also holds two snapshot planes


# ------------------------------------------------------------------ the benchmark configurations at full size

def _run_cfg(name, dev, batch=None):
    import butterfly_b200 as bb
    from butterfly_b200 import configs
    d = configs.make_inputs(name, batch=batch, device=dev)
    if d["base4"]:
        fw = lambda x: bb.butterfly_multiply_base4_fw(d["twiddle4"], d["twiddle2"], x, d["increasing_stride"])
        bw = lambda x, g: bb.butterfly_multiply_base4_bw(d["twiddle4"], d["twiddle2"], x, g, d["increasing_stride"])
    else:
        fw = lambda x: bb.butterfly_multiply_fw(d["twiddle"], x, d["increasing_stride"])
        bw = lambda x, g: bb.butterfly_multiply_bw(d["twiddle"], x, g, d["increasing_stride"])
    return d, fw, bw


def _row_sample(B, tile=7):
    """>= 256 rows of a batch of B: the first rows, a run from the middle, and the last rows (which end
    inside a tile for the batch sizes used here)."""
    if B <= 256:
        return torch.arange(B)
    mid = (B // 2 // tile) * tile + 3
    idx = torch.cat([torch.arange(0, 96), torch.arange(mid, mid + 64), torch.arange(B - 96, B)])
    return idx


def _oracle_fw(oracle_mod, d, x, dtype=None):
    cast = (lambda t: t.to(dtype)) if dtype is not None else (lambda t: t)
    if d["base4"]:
        return oracle_mod.base4_fw(cast(d["twiddle4"].cpu()), cast(d["twiddle2"].cpu()), x, d["increasing_stride"])
    return oracle_mod.multiply_fw(cast(d["twiddle"].cpu()), x, d["increasing_stride"])


def _oracle_bw(oracle_mod, d, x, g, dtype=None):
    """(list of twiddle gradients, d_input) from the oracle; dtype = torch.float64 / complex128 for the
    double-precision oracle."""
    cast = (lambda t: t.to(dtype)) if dtype is not None else (lambda t: t)
    if d["base4"]:
        d4, d2, dx = oracle_mod.base4_bw(cast(d["twiddle4"].cpu()), cast(d["twiddle2"].cpu()), x, g, d["increasing_stride"])
        return [d4, d2], dx
    dt, dx = oracle_mod.multiply_bw(cast(d["twiddle"].cpu()), x, g, d["increasing_stride"])
    return [dt], dx


@pytest.mark.parametrize("name", ["cfg1", "cfg2", "cfg3", "cfg4", "cfg5"])
def test_benchmark_configs_full_size_properties(dev, oracle_mod, name):
    """The benchmark configurations at full size: the oracle on a sample of 256 rows spread over the
    batch (first rows, a run from the middle, the last rows) for output and input gradient, at
    rtol 1e-5 / atol 1e-5 per component; the twiddle gradient of that row sample graded against
    the double-precision oracle; and size-independent properties of the full batch: linearity
    of the forward, the adjoint identity <B x, g> = <x, B^H g>, additivity of the twiddle gradient
    over the batch."""
    d, fw, bw = _run_cfg(name, dev)
    x = d["input"]
    B = d["batch"]
    y = fw(x)
    idx = _row_sample(B)
    xs = x[idx.to(dev)].cpu()
    yr = _oracle_fw(oracle_mod, d, xs)
    assert_close_1e5(y[idx.to(dev)].cpu(), yr, name, name + " output")
    # linearity: B(2x) = 2 B(x) exactly (scaling by 2 commutes with float rounding)
    assert torch.equal(fw(2 * x), 2 * y)
    if d.get("forward_only"):
        return
    g = d["grad"]
    out = bw(x, g)
    d_x = out[-1]
    # adjoint identity, accumulated in double
    hi = torch.complex128 if y.is_complex() else torch.float64
    lhs = (y.to(hi).conj() * g.to(hi)).sum().item()
    rhs = (x.to(hi).conj() * d_x.to(hi)).sum().item()
    norm = (y.to(hi).abs().pow(2).sum().sqrt() * g.to(hi).abs().pow(2).sum().sqrt()).item()
    assert abs(lhs - rhs) <= 1e-6 * norm
    # the oracle on the row sample: input gradient per component ...
    gs = g[idx.to(dev)].cpu()
    dt32, dxr = _oracle_bw(oracle_mod, d, xs, gs)
    assert_close_1e5(d_x[idx.to(dev)].cpu(), dxr, name, name + " d_input")
    # ... and the twiddle gradient of the sampled rows (a separate call on those rows) against the
    # double-precision oracle
    dt64, _ = _oracle_bw(oracle_mod, d, xs, gs, dtype=hi)
    xs_d = x[idx.to(dev)]  # keeps a stack-broadcast input broadcast
    sample = bw(xs_d, g[idx.to(dev)].contiguous())
    for ours, r32, r64 in zip(sample[:-1], dt32, dt64):
        assert_sum_accuracy(ours, r32, r64, name + " d_twiddle of the row sample")
    assert_close_1e5(sample[-1].cpu(), dxr, name, name + " d_input of the row sample")
    # additivity of the twiddle gradient over two halves of the batch
    h = B // 2
    a = bw(x[:h], g[:h])
    b = bw(x[h:], g[h:])
    for full, pa, pb in zip(out[:-1], a[:-1], b[:-1]):
        if full.numel():
            scale = full.abs().max().item()
            assert (full - (pa + pb)).abs().max().item() <= 2e-5 * scale


@pytest.mark.parametrize("name", ["cfg2", "cfg3", "cfg5"])
def test_against_reference_cuda_extension(dev, oracle_mod, name):
    """Output and input gradient within rtol 1e-5 / atol 1e-5 of the reference's own CUDA extension
    (compiled unmodified from the reference tree into oracle/_ref/) on the same seeded inputs."""
    if not oracle_mod.reference_available(cuda=True):
        pytest.skip("oracle/_ref/_butterfly_ref_cuda.so not built")
    try:
        ref = oracle_mod.load_reference_ops(cuda=True)
    except RuntimeError as e:
        pytest.skip(str(e))
    d, fw, bw = _run_cfg(name, dev)
    x, g, tw, inc = d["input"], d["grad"], d["twiddle"], d["increasing_stride"]
    y = fw(x)
    yr = ref.butterfly_multiply_fw(tw, x, inc, d["n"])
    assert_close_1e5(y, yr, name, name + " output vs reference CUDA")
    d_tw, d_x = bw(x, g)
    dtr, dxr = ref.butterfly_multiply_bw(tw, x, g, inc)
    assert_close_1e5(d_x, dxr, name, name + " d_input vs reference CUDA")
    # both twiddle gradients are float sums of thousands of terms in different orders: compare at the
    # accuracy such sums have
    assert rel_err(d_tw, dtr) < 2e-5


def test_operators_capture_into_a_cuda_graph(dev, oracle_mod):
    """The operators only enqueue work on the current stream (descriptor encoding is host work, scratch
    comes from torch's allocator), so a forward + backward captures into a CUDA graph and replays on
    new data in the same buffers."""
    import butterfly_b200 as bb
    torch.manual_seed(17)
    for dtype, log_n, nb, B in ((torch.float32, 10, 2, 256), (torch.complex64, 10, 1, 64)):
        n = 1 << log_n
        tw = (torch.randn(1, nb, log_n, n // 2, 2, 2, dtype=dtype) / 2 ** 0.5).to(dev)
        x = torch.randn(B, 1, n, dtype=dtype, device=dev)
        g = torch.randn(B, 1, n, dtype=dtype, device=dev)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):  # warm-up outside the capture (lazy initialisation, attributes)
            bb.butterfly_multiply_fw(tw, x, True)
            bb.butterfly_multiply_bw(tw, x, g, True)
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y = bb.butterfly_multiply_fw(tw, x, True)
            d_tw, d_x = bb.butterfly_multiply_bw(tw, x, g, True)
        x.copy_(torch.randn(B, 1, n, dtype=dtype))
        g.copy_(torch.randn(B, 1, n, dtype=dtype))
        graph.replay()
        torch.cuda.synchronize()
        yr = oracle_mod.multiply_fw(tw.cpu(), x.cpu(), True)
        dtr, dxr = oracle_mod.multiply_bw(tw.cpu(), x.cpu(), g.cpu(), True)
        assert rel_err(y, yr) < TOL and rel_err(d_x, dxr) < TOL and rel_err(d_tw, dtr) < TOL
