"""The forward with glue operators (gather, diagonal, real <-> complex) folded into its launch:
through the C ABI against the oracle composed with the separate operators, and the fused module
chains of special.py / glue.fuse against their link-by-link form and torch.fft."""
import pytest
import torch
from torch import nn

from conftest import assert_rtol_atol

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda", 0)


def _reference(oracle_mod, tw, x, inc, in_perm, out_diag, out_perm, out_real):
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
@pytest.mark.parametrize("log_n,nblocks,B,S", [(5, 1, 3, 1), (9, 2, 37, 2), (11, 1, 100, 1), (12, 1, 19, 1), (10, 5, 33, 1)])
def test_glue_forward_through_c_abi(dev, oracle_mod, cplx, log_n, nblocks, B, S):
    from butterfly_b200 import abi
    if cplx and log_n > 11:
        pytest.skip("complex rows of more than 2048 columns do not fit a tile")
    torch.manual_seed(log_n * 7 + nblocks)
    dtype = torch.complex64 if cplx else torch.float32
    n = 1 << log_n
    tw = torch.randn(S, nblocks, log_n, n // 2, 2, 2, dtype=dtype) / 2 ** 0.5
    for combo in range(8 if cplx else 4):
        use_in, use_out, real_io = bool(combo & 1), bool(combo & 2), bool(combo & 4)
        for inc in (True, False):
            x = torch.randn(B, S, n, dtype=torch.float32 if real_io else dtype)
            in_perm = torch.randperm(n, dtype=torch.int32) if use_in else None
            out_perm = torch.randperm(n, dtype=torch.int32) if use_out else None
            out_diag = torch.randn(n, dtype=dtype) if use_out else None
            d = lambda t: None if t is None else t.to(dev)
            launches = abi.launch_count()
            y, rc = abi.fw_glue(tw.to(dev), x.to(dev), inc, d(in_perm), d(out_diag), d(out_perm), real_io)
            assert rc == 0 and abi.launch_count() - launches == (1 if nblocks * log_n <= 40 * 3 else 2)
            want = _reference(oracle_mod, tw, x, inc, in_perm, out_diag, out_perm, real_io)
            assert_rtol_atol(y, want, "glue forward n=%d combo=%d" % (n, combo), rtol=1e-4, atol=1e-4)
    assert abi.device_error() == 0
    # no glue at all: the same bits as the plain forward
    x = torch.randn(B, S, n, dtype=dtype, device=dev)
    with_none, _ = abi.fw_glue(tw.to(dev), x, True)
    import butterfly_b200 as bb
    from conftest import abi_option
    with abi_option("fw2", 0):
        plain = bb.butterfly_multiply_fw(tw.to(dev), x, True)
    assert torch.equal(with_none, plain)


def test_glue_refusals(dev):
    from butterfly_b200 import abi
    n = 1 << 13
    tw = torch.randn(1, 1, 13, n // 2, 2, 2, device=dev)
    x = torch.randn(2, 1, n, device=dev)
    perm = torch.randperm(n, dtype=torch.int32, device=dev)
    assert abi.fw_glue(tw, x, True, perm, check=False)[1] == -2       # rows wider than a tile
    tw = torch.randn(1, 1, 6, 32, 2, 2, device=dev)
    perm = torch.randperm(64, dtype=torch.int32, device=dev)
    assert abi.fw_glue(tw, torch.randn(2, 1, 60, device=dev), True, perm, check=False)[1] == -1  # gather on a ragged row


def test_fused_transforms_against_torch_fft(dev):
    import butterfly_b200 as bb
    from butterfly_b200 import abi, special
    torch.manual_seed(0)
    for n in (8, 256, 2048):
        x = torch.randn(5, 3, n, dtype=torch.complex64, device=dev)
        for br_first in (True, False):
            f = special.fft(n, br_first=br_first).to(dev)
            assert isinstance(f[0], bb.glue.ButterflyPipeline) and len(f) == 1
            launches = abi.launch_count()
            y = f(x)
            assert abi.launch_count() - launches == 1
            assert_rtol_atol(y, torch.fft.fft(x), "fused fft n=%d" % n, rtol=1e-4, atol=1e-4 * n ** 0.5)
            assert_rtol_atol(y, special.fft(n, br_first=br_first, fused=False).to(dev)(x), "fused against chained fft", rtol=1e-5, atol=1e-5 * n ** 0.5)
            fi = special.ifft(n, br_first=br_first).to(dev)
            assert_rtol_atol(fi(y), x, "ifft(fft(x))", rtol=1e-4, atol=1e-4)
    # circulant on real input: Real2Complex, fft, diagonal, ifft, Complex2Real in two launches
    n = 512
    col = torch.randn(n)
    x = torch.randn(7, n, device=dev)
    c = special.circulant(col).to(dev)
    launches = abi.launch_count()
    y = c(x)
    assert abi.launch_count() - launches == 2 and y.dtype == torch.float32
    idx = (torch.arange(n).unsqueeze(1) - torch.arange(n).unsqueeze(0)) % n
    want = x @ col.to(dev)[idx.to(dev)].t()
    assert_rtol_atol(y, want, "circulant", rtol=1e-4, atol=2e-4 * n ** 0.5)
    assert_rtol_atol(special.circulant(col, transposed=True).to(dev)(x), x @ col.to(dev)[idx.to(dev)], "transposed circulant", rtol=1e-4, atol=2e-4 * n ** 0.5)
    one = special.circulant(col, separate_diagonal=False).to(dev)
    launches = abi.launch_count()
    assert_rtol_atol(one(x), want, "circulant as one butterfly", rtol=1e-4, atol=2e-4 * n ** 0.5)
    assert abi.launch_count() - launches == 1
    # a length that is not a power of two runs link by link
    m = 12
    colm = torch.randn(m, dtype=torch.complex64)
    xm = torch.randn(4, m, dtype=torch.complex64, device=dev)
    idx = (torch.arange(m).unsqueeze(1) - torch.arange(m).unsqueeze(0)) % m
    assert_rtol_atol(special.circulant(colm).to(dev)(xm), xm @ colm.to(dev)[idx.to(dev)].t(), "circulant n=12", rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("cplx", [False, True])
def test_fused_chain_gradients(dev, cplx):
    """glue.fuse keeps the function and the gradients of the chain it rewrites (parameters shared)."""
    import butterfly_b200 as bb
    from butterfly_b200 import glue
    from butterfly_b200.complex_utils import Complex2Real, Real2Complex
    from butterfly_b200.diagonal import Diagonal
    from butterfly_b200.permutation import FixedPermutation
    torch.manual_seed(1)
    n = 128
    b1 = bb.Butterfly(n, n, False, cplx, True, nblocks=2)
    b2 = bb.Butterfly(n, n, False, cplx, False)
    links = [FixedPermutation(torch.randperm(n)), b1, Diagonal(n, complex=cplx), FixedPermutation(torch.randperm(n)), b2,
             FixedPermutation(torch.randperm(n))]
    if cplx:
        links = [Real2Complex()] + links + [Complex2Real()]
    chain = nn.Sequential(*links).to(dev)
    fused = glue.fuse(chain)
    assert len(fused) == 2 and all(isinstance(m, glue.ButterflyPipeline) for m in fused)
    x = torch.randn(6, 4, n, device=dev, requires_grad=True)
    g = torch.randn(6, 4, n, device=dev)
    y = chain(x)
    y.backward(g)
    want = [y.detach(), x.grad.clone()] + [p.grad.clone() for p in chain.parameters()]
    x.grad = None
    for p in chain.parameters():
        p.grad = None
    y = fused(x)
    y.backward(g)
    got = [y.detach(), x.grad] + [p.grad for p in chain.parameters()]  # the same parameter objects
    assert len(list(fused.parameters())) == len(list(chain.parameters()))
    for a, b in zip(got, want):
        assert a.dtype == b.dtype
        assert_rtol_atol(a, b, "fused chain", rtol=1e-4, atol=2e-4)


def test_glue_falls_back_link_by_link(dev):
    """A product of more stage groups than one launch carries, ending in a real part, is not covered by
    the fused launch (its intermediate rows need a complex buffer): the operator runs the links one by
    one and still differentiates."""
    import butterfly_b200 as bb
    torch.manual_seed(5)
    log_n, nb = 6, 16  # 96 stages = 48 two-stage groups of the complex forward
    n = 1 << log_n
    tw = (torch.randn(1, nb, log_n, n // 2, 2, 2, dtype=torch.complex64) / 2 ** 0.5).to(dev).requires_grad_(True)
    x = torch.randn(5, 1, n, device=dev, requires_grad=True)
    perm = torch.randperm(n, device=dev).to(torch.int32)
    y = bb.butterfly_multiply_glue(tw, x, True, in_perm=perm, out_real=True)
    want = bb.butterfly_multiply(tw, x.to(torch.complex64)[..., perm.long()], True).real
    assert y.dtype == torch.float32
    assert_rtol_atol(y, want.detach(), "fallback output", rtol=1e-5, atol=1e-5)
    g = torch.randn_like(y)
    gx, gt = torch.autograd.grad(y, (x, tw), g)
    wx, wt = torch.autograd.grad(want, (x, tw), g)
    assert_rtol_atol(gx, wx, "fallback d_input", rtol=1e-4, atol=1e-4)
    assert_rtol_atol(gt, wt, "fallback d_twiddle", rtol=1e-4, atol=1e-4)
