"""Seeded random sweep of the CUDA path against the CPU oracle through the C ABI: radix-2 float32 and
complex64, base-4, both directions, ragged batches and stacks, padded / truncated inputs, sliced
outputs, stack-broadcast and pitched rows; for radix-2 also the forward that saves snapshots and the
backward that starts from them.  Relative error bound 3e-5 (float32 arithmetic in a different but
valid order than the oracle's)."""
import random

import pytest
import torch

from conftest import assert_rtol_atol, assert_sum_accuracy, rel_err

pytestmark = pytest.mark.gpu


def _case(rng):
    kind = rng.choice(["f32", "f32", "c64", "b4"])
    log_n = rng.choice([1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 10, 11, 12, 12, 13, 14])
    if kind == "b4":
        log_n = max(log_n, 2)
    n = 1 << log_n
    nb = rng.choice([1, 1, 2, 3])
    S = rng.choice([1, 1, 2, 3])
    B = rng.choice([1, 2, 3, 4, 5, 7, 8, 16, 33, 70]) if log_n <= 11 else rng.choice([1, 3, 4, 9, 16])
    inc = rng.random() < 0.5
    insz = rng.choice([n, n, max(1, n // 2), max(1, n - 3), n + 5, 2 * n, (n // 64) * 32 + 32 if n >= 64 else n])
    outsz = rng.choice([n, n, max(1, n - 1), max(1, n // 2), n - 32 if n >= 64 else n])
    mode = rng.choice(["plain", "plain", "broadcast", "pitched"])
    return kind, log_n, nb, S, B, inc, insz, outsz, mode


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_cases_against_oracle(oracle_mod, seed):
    from butterfly_b200 import abi
    dev = torch.device("cuda", 0)
    rng = random.Random(seed)
    torch.manual_seed(seed)
    for _ in range(60):
        kind, log_n, nb, S, B, inc, insz, outsz, mode = _case(rng)
        n = 1 << log_n
        dtype = torch.complex64 if kind == "c64" else torch.float32
        what = (kind, log_n, nb, S, B, inc, insz, outsz, mode)
        if mode == "broadcast":
            xh = torch.randn(B, 1, insz, dtype=dtype).expand(B, S, insz)
            xd = xh[:, :1].contiguous().to(dev).expand(B, S, insz)
        elif mode == "pitched":
            wide = torch.randn(B, S, insz + 8, dtype=dtype)
            xh, xd = wide[:, :, :insz], wide.to(dev)[:, :, :insz]
        else:
            xh = torch.randn(B, S, insz, dtype=dtype)
            xd = xh.to(dev)
        g = torch.randn(B, S, outsz, dtype=dtype)
        if kind == "b4":
            tw4 = torch.randn(S, nb, log_n // 2, n // 4, 4, 4) / 2
            tw2 = torch.randn(S, nb, log_n % 2, n // 2, 2, 2) / 2 ** 0.5
            yr = oracle_mod.base4_fw(tw4, tw2, xh, inc, outsz)
            d4r, d2r, dxr = oracle_mod.base4_bw(tw4, tw2, xh, g, inc)
            out, _ = abi.fw_base4(tw4.to(dev), tw2.to(dev), xd, inc, outsz)
            d4, d2, dx, _ = abi.bw_base4(tw4.to(dev), tw2.to(dev), xd, g.to(dev), inc)
            assert rel_err(out[:, :, :outsz], yr) < 3e-5, what
            assert rel_err(dx[:, :, :insz], dxr) < 3e-5, what
            assert_rtol_atol(out[:, :, :outsz], yr, str(what), outliers=3e-4, worst_allowed=3.0)
            assert_rtol_atol(dx[:, :, :insz], dxr, str(what), outliers=3e-4, worst_allowed=3.0)
            # twiddle gradients are sums over the batch whose order (atomic additions of the CTAs' partial
            # sums) changes from run to run: graded against the double-precision oracle, not per component
            # against one float32 order
            d4h, d2h, _ = oracle_mod.base4_bw(tw4.double(), tw2.double(), xh.double(), g.double(), inc)
            if tw4.numel():
                assert rel_err(d4, d4r) < 3e-5, what
                assert_sum_accuracy(d4, d4r, d4h, str(what) + " d_twiddle4")
            if tw2.numel():
                assert rel_err(d2, d2r) < 3e-5, what
                assert_sum_accuracy(d2, d2r, d2h, str(what) + " d_twiddle2")
            continue
        tw = torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dtype) / 2 ** 0.5
        yr = oracle_mod.multiply_fw(tw, xh, inc, outsz)
        dtr, dxr = oracle_mod.multiply_bw(tw, xh, g, inc)
        out, _ = abi.fw(tw.to(dev), xd, inc, outsz)
        dt, dx, _ = abi.bw(tw.to(dev), xd, g.to(dev), inc)
        y2, snaps, _ = abi.fw_saving(tw.to(dev), xd, inc, outsz)
        dt2, dx2, _ = abi.bw_saved(tw.to(dev), xd, g.to(dev), snaps, inc)
        for a, b in ((out[:, :, :outsz], yr), (dx[:, :, :insz], dxr), (y2[:, :, :outsz], yr), (dx2[:, :, :insz], dxr)):
            assert rel_err(a, b) < 3e-5, what
            # per component: rtol 1e-5 / atol 1e-5.  The oracle rounds every product, the GPU fuses
            # multiply-adds: over millions of components a handful land just outside
            assert_rtol_atol(a, b, str(what), outliers=3e-4, worst_allowed=3.0)
        # twiddle gradients are sums over the batch whose order (atomic additions of the CTAs' partial
        # sums) changes from run to run: graded against the double-precision oracle, not per component
        # against one float32 order
        hi = torch.complex128 if dtype == torch.complex64 else torch.float64
        dth, _ = oracle_mod.multiply_bw(tw.to(hi), xh.to(hi), g.to(hi), inc)
        for a in (dt, dt2):
            assert rel_err(a, dtr) < 3e-5, what
            assert_sum_accuracy(a, dtr, dth, str(what) + " d_twiddle")
    assert abi.device_error() == 0
