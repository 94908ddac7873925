"""The CPU oracle against the reference: committed golden vectors (generated from the
reference's CPU operator and PyTorch definitions by tests/golden/make_golden.py) and, when
it has been built here, the reference's own compiled CPU operator."""
import pytest
import torch

from conftest import golden_files, load_golden, rel_err


@pytest.mark.parametrize("path", golden_files("radix2"), ids=lambda p: p.split("/")[-1])
def test_oracle_matches_reference_cpu_golden(oracle_mod, path):
    d = load_golden(path)
    out = oracle_mod.multiply_fw(d["twiddle"], d["input"], d["increasing_stride"], d["output_size"])
    d_tw, d_x = oracle_mod.multiply_bw(d["twiddle"], d["input"], d["grad"], d["increasing_stride"])
    # same operation order as the reference CPU operator: bit-exact
    assert torch.equal(out, d["output"])
    assert torch.equal(d_tw, d["d_twiddle"])
    assert torch.equal(d_x, d["d_input"])
    # and the reference's PyTorch definition agrees to rounding
    assert rel_err(out, d["output_torch"]) < 5e-6


@pytest.mark.parametrize("path", golden_files("base4"), ids=lambda p: p.split("/")[-1])
def test_oracle_matches_reference_base4_golden(oracle_mod, path):
    d = load_golden(path)
    out = oracle_mod.base4_fw(d["twiddle4"], d["twiddle2"], d["input"], d["increasing_stride"], d["output_size"])
    d4, d2, d_x = oracle_mod.base4_bw(d["twiddle4"], d["twiddle2"], d["input"], d["grad"], d["increasing_stride"])
    assert rel_err(out, d["output"]) < 5e-6
    assert rel_err(d_x, d["d_input"]) < 5e-6
    if d["twiddle4"].numel():
        assert rel_err(d4, d["d_twiddle4"]) < 5e-6
    if d["twiddle2"].numel():
        assert rel_err(d2, d["d_twiddle2"]) < 5e-6


def test_oracle_double_precision_agrees_with_float(oracle_mod):
    torch.manual_seed(1)
    tw = torch.randn(2, 2, 7, 64, 2, 2, dtype=torch.float64)
    x = torch.randn(5, 2, 128, dtype=torch.float64)
    g = torch.randn(5, 2, 128, dtype=torch.float64)
    hi = oracle_mod.multiply_bw(tw, x, g, True)
    lo = oracle_mod.multiply_bw(tw.float(), x.float(), g.float(), True)
    assert rel_err(lo[0].double(), hi[0]) < 1e-5 and rel_err(lo[1].double(), hi[1]) < 1e-5


def test_oracle_against_compiled_reference_cpu_op(oracle_mod):
    if not oracle_mod.reference_available():
        pytest.skip("oracle/_ref/_butterfly_ref_cpu.so not built (reference tree absent)")
    ref = oracle_mod.load_reference_ops()
    torch.manual_seed(2)
    for dt in (torch.float32, torch.float64, torch.complex64, torch.complex128):
        for log_n, S, nb, B, inc in [(1, 1, 1, 2, True), (4, 2, 3, 7, False), (8, 1, 2, 3, True)]:
            n = 1 << log_n
            for insz, outsz in [(n, n), (n // 2 + 1, max(1, n - 3)), (2 * n + 1, max(1, n // 2))]:
                tw = torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dt)
                x = torch.randn(B, S, insz, dtype=dt)
                g = torch.randn(B, S, outsz, dtype=dt)
                assert torch.equal(oracle_mod.multiply_fw(tw, x, inc, outsz), ref.butterfly_multiply_fw(tw, x, inc, outsz))
                a = oracle_mod.multiply_bw(tw, x, g, inc)
                b = ref.butterfly_multiply_bw(tw, x, g, inc)
                assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    # stack-broadcast input (stride 0), as Butterfly.pre_process produces
    tw = torch.randn(3, 2, 5, 16, 2, 2)
    x = torch.randn(4, 1, 32).expand(4, 3, 32)
    assert torch.equal(oracle_mod.multiply_fw(tw, x, True), ref.butterfly_multiply_fw(tw, x, True, 32))
