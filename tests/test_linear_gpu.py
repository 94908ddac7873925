"""The fused linear layer (bias in the forward's store epilogue; input gradient summed over the
stacks and bias gradient collected inside the backward kernels) against the CPU oracle composed
with the reference's PyTorch glue (torch_butterfly/butterfly.py:152-169: expand the input over the
stacks, flatten the stacks, slice, add the bias), through the C ABI and through the module."""
import pytest
import torch

from conftest import assert_rtol_atol, assert_sum_accuracy, rel_err

pytestmark = pytest.mark.gpu

TOL = 2e-5


def _oracle_layer(oracle_mod, tw, x, bias, g, inc, out_size, dtype=None):
    S, n = tw.shape[0], 1 << tw.shape[2]
    B = x.shape[0]
    cast = (lambda t: t.to(dtype)) if dtype is not None else (lambda t: t)
    xe = x.unsqueeze(1).expand(B, S, x.shape[1])
    y = oracle_mod.multiply_fw(cast(tw), xe, inc).reshape(B, S * n)[:, :out_size] + cast(bias)[:out_size]
    gp = torch.zeros(B, S * n, dtype=g.dtype)
    gp[:, :out_size] = g
    dt, dx = oracle_mod.multiply_bw(cast(tw), xe, gp.reshape(B, S, n), inc)
    return y, dt, dx.sum(1), cast(g).sum(0)


@pytest.mark.parametrize("log_n,S", [(10, 4), (11, 2), (12, 1), (9, 3), (13, 2)])
def test_fused_linear_through_c_abi(oracle_mod, log_n, S):
    from butterfly_b200 import abi
    dev = torch.device("cuda", 0)
    torch.manual_seed(70 + log_n)
    n = 1 << log_n
    for nb, inc in [(1, True), (2, True), (2, False)]:
        for B, in_size in [(64, n), (301, n - 64), (7, n // 2)]:
            out_size = S * n
            tw = torch.randn(S, nb, log_n, n // 2, 2, 2) / 2 ** 0.5
            x = torch.randn(B, in_size)
            bias = torch.randn(out_size)
            g = torch.randn(B, out_size)
            yr, dtr, dxr, dbr = _oracle_layer(oracle_mod, tw, x, bias, g, inc, out_size)
            out, _ = abi.linear_fw(tw.to(dev), x.to(dev), bias.to(dev), inc, out_size)
            what = "n=%d S=%d nb=%d inc=%s B=%d in=%d" % (n, S, nb, inc, B, in_size)
            assert_rtol_atol(out[:, :out_size], yr, what + " output")
            d_tw, d_in, d_b, rc = abi.linear_bw(tw.to(dev), x.to(dev), g.to(dev), inc, check=False)
            if log_n < 10:
                assert rc == -2  # panels narrower than 1024 columns: the caller composes the unfused operators
                continue
            if rc == -2:
                # a phase on strided column segments needs rows that are whole groups of segments: only
                # the ragged input widths may be refused, and the composed route must then serve them
                assert in_size != n, what
                import butterfly_b200 as bb
                d_tw, d_in, d_b = bb.butterfly_linear_bw(tw.to(dev), x.to(dev), g.to(dev), inc, True)
            else:
                assert rc == 0, what
            assert_rtol_atol(d_in, dxr, what + " d_input (summed over stacks)")
            assert rel_err(d_tw, dtr) < TOL, what
            y64, dt64, dx64, db64 = _oracle_layer(oracle_mod, tw, x, bias, g, inc, out_size, dtype=torch.float64)
            assert_sum_accuracy(d_tw, dtr, dt64, what + " d_twiddle")
            assert_sum_accuracy(d_b, dbr, db64, what + " d_bias")
    assert abi.device_error() == 0


def test_fused_linear_operator_and_module(oracle_mod):
    """torch operators: fused route and the composed fallback (ragged out_size, ragged in_size) give the
    oracle's results; the Butterfly module uses the operator and its gradients reach all parameters."""
    import butterfly_b200 as bb
    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    for in_size, out_size, nb in [(1024, 4096, 2), (1000, 3000, 1), (2048, 2048, 2)]:
        layer = bb.Butterfly(in_size, out_size, bias=True, nblocks=nb).to(dev)
        B = 333
        x = torch.randn(B, in_size)
        g = torch.randn(B, out_size)
        xd = x.to(dev).requires_grad_(True)
        before = bb.abi.launch_count()
        y = layer(xd)
        y.backward(g.to(dev))
        assert bb.abi.launch_count() > before
        tw, bias = layer.twiddle.detach().cpu(), layer.bias.detach().cpu()
        yr, dtr, dxr, dbr = _oracle_layer(oracle_mod, tw, x, bias, g, True, out_size)
        what = "Butterfly(%d, %d, nblocks=%d)" % (in_size, out_size, nb)
        assert_rtol_atol(y, yr, what + " output")
        assert_rtol_atol(xd.grad, dxr, what + " d_input")
        assert rel_err(layer.twiddle.grad, dtr) < TOL and rel_err(layer.bias.grad, dbr) < TOL, what
        # and the unfused route (expand / multiply / flatten / slice / bias in PyTorch) agrees
        rows = xd.detach().unsqueeze(1).expand(B, layer.nstacks, in_size)
        y2 = bb.butterfly_multiply(layer.twiddle.detach(), rows, True).reshape(B, -1)[:, :out_size] + layer.bias.detach()
        assert torch.equal(y.detach(), y2)  # same kernels, the bias added to the same rounded values
    assert bb.abi.device_error() == 0
