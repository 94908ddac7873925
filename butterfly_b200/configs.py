"""The five benchmark configurations and their seeded synthetic inputs.

No public dataset stands behind these numbers: the workloads are synthetic tensors with
the shapes, sizes and value distributions the benchmark definition names, drawn from a
fixed CPU generator (order of draws: twiddle, input, grad) so that a CPU run and a GPU run
see identical values.
"""
import math

import torch

# name -> description of the operator call
CONFIGS = {
    # Butterfly(1024, 1024), real, nblocks=1, forward only (the one config a CPU can run in full)
    "cfg1": dict(dtype=torch.float32, log_n=10, nblocks=1, nstacks=1, batch=256, increasing_stride=True,
                 base4=False, forward_only=True, twiddle_init="randn"),
    # real fp32 n=4096, two blocks (increasing then decreasing stride), batch 16384
    "cfg2": dict(dtype=torch.float32, log_n=12, nblocks=2, nstacks=1, batch=16384, increasing_stride=True,
                 base4=False, twiddle_init="randn"),
    # complex64 n=2048, DFT twiddles + 1e-3 perturbation, bit-reversed input, batch 8192
    "cfg3": dict(dtype=torch.complex64, log_n=11, nblocks=1, nstacks=1, batch=8192, increasing_stride=True,
                 base4=False, twiddle_init="dft"),
    # base-4, real fp32 n=16384 (7 radix-4 stages), batch 4096
    "cfg4": dict(dtype=torch.float32, log_n=14, nblocks=1, nstacks=1, batch=4096, increasing_stride=True,
                 base4=True, twiddle_init="randn4"),
    # rectangular 1024 -> 4096 layer: 4 stacks, 2 blocks, batch 8192 per GPU (65536 over 8),
    # the input row is shared by the stacks (stack stride 0)
    "cfg5": dict(dtype=torch.float32, log_n=10, nblocks=2, nstacks=4, batch=8192, increasing_stride=True,
                 base4=False, twiddle_init="randn", broadcast_stacks=True),
}


def bit_reversal(n):
    """Bit-reversal permutation of range(n) as a LongTensor."""
    log_n = int(math.log2(n))
    idx = torch.arange(n)
    rev = torch.zeros(n, dtype=torch.long)
    for b in range(log_n):
        rev |= ((idx >> b) & 1) << (log_n - 1 - b)
    return rev


def dft_twiddle(n, dtype=torch.complex64):
    """Twiddles of the unnormalised decimation-in-time FFT (input already bit-reversed):
    stage s (stride 2^s) has blocks [[1, w], [1, -w]] with w = exp(-2*pi*i*k / 2^(s+1)),
    k = position inside the stride.  Shape (1, 1, log_n, n/2, 2, 2)."""
    log_n = int(math.log2(n))
    tw = torch.zeros(1, 1, log_n, n // 2, 2, 2, dtype=torch.complex128)
    for s in range(log_n):
        stride = 1 << s
        k = torch.arange(n // 2) % stride
        w = torch.exp(-2j * math.pi * k.to(torch.float64) / (2 * stride))
        tw[0, 0, s, :, 0, 0] = 1
        tw[0, 0, s, :, 0, 1] = w
        tw[0, 0, s, :, 1, 0] = 1
        tw[0, 0, s, :, 1, 1] = -w
    return tw.to(dtype)


def make_inputs(name, batch=None, seed=0, rank=0, device="cpu", with_grad=True):
    """Returns a dict with the operator arguments of configuration `name`.

    `batch` overrides the configured batch (bounded samples, parity tests); rank r draws its
    rows from seed 1000+r while every rank draws the same twiddle from `seed`.
    """
    c = dict(CONFIGS[name])
    B = c["batch"] if batch is None else batch
    n = 1 << c["log_n"]
    S, nb, log_n, dt = c["nstacks"], c["nblocks"], c["log_n"], c["dtype"]
    g = torch.Generator().manual_seed(seed)
    out = dict(c)
    if c["twiddle_init"] == "randn":
        out["twiddle"] = torch.randn(S, nb, log_n, n // 2, 2, 2, dtype=dt, generator=g) / math.sqrt(2)
    elif c["twiddle_init"] == "dft":
        out["twiddle"] = dft_twiddle(n, dt) + 1e-3 * torch.randn(1, 1, log_n, n // 2, 2, 2, dtype=dt, generator=g)
    elif c["twiddle_init"] == "randn4":
        out["twiddle4"] = torch.randn(S, nb, log_n // 2, n // 4, 4, 4, dtype=dt, generator=g) / 2
        out["twiddle2"] = torch.empty(S, nb, log_n % 2, n // 2, 2, 2, dtype=dt)
        if log_n % 2:
            out["twiddle2"] = torch.randn(S, nb, 1, n // 2, 2, 2, dtype=dt, generator=g) / math.sqrt(2)
    gr = torch.Generator().manual_seed(1000 + rank) if rank or c.get("broadcast_stacks") else g
    if c.get("broadcast_stacks"):
        x = torch.randn(B, 1, n, dtype=dt, generator=gr)
    else:
        x = torch.randn(B, S, n, dtype=dt, generator=gr)
    if c["twiddle_init"] == "dft":
        x = x[..., bit_reversal(n)].contiguous()
    grad = torch.randn(B, S, n, dtype=dt, generator=gr) if with_grad and not c.get("forward_only") else None
    for k in ("twiddle", "twiddle4", "twiddle2"):
        if k in out:
            out[k] = out[k].to(device)
    x = x.to(device)
    out["input"] = x.expand(B, S, n) if c.get("broadcast_stacks") else x
    out["grad"] = grad.to(device) if grad is not None else None
    out["batch"] = B
    out["n"] = n
    return out


def algorithmic_bytes(name, batch=None):
    """(forward bytes, backward bytes): every operator tensor's unique storage touched once.

    fw = sz*(B*Sx*n + B*S*n) + |twiddle| ;  bw = sz*(B*Sx*n + 2*B*S*n) + 2*|twiddle|
    (Sx = 1 when the stacks share one input row; bw reads twiddle and writes d_twiddle).
    """
    c = CONFIGS[name]
    B = c["batch"] if batch is None else batch
    n = 1 << c["log_n"]
    S = c["nstacks"]
    sz = 4 if c["dtype"] == torch.float32 else 8
    Sx = 1 if c.get("broadcast_stacks") else S
    if c["base4"]:
        tw = S * c["nblocks"] * ((c["log_n"] // 2) * (n // 4) * 16 + (c["log_n"] % 2) * (n // 2) * 4) * sz
    else:
        tw = S * c["nblocks"] * c["log_n"] * (n // 2) * 4 * sz
    fw = sz * (B * Sx * n + B * S * n) + tw
    bw = sz * (B * Sx * n + 2 * B * S * n) + 2 * tw
    return fw, bw
