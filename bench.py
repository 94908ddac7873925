#!/usr/bin/env python
"""Benchmark of the butterfly multiply (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config cfg2]

A "step" is one forward plus one backward of the operator over one batch of synthetic
input (configs.py; default cfg2: real fp32, n=4096, two blocks, batch 16384 per GPU).
With N > 1 (launched by torchrun, one rank per GPU) every rank processes its own batch of
the same size (weak scaling), nothing crosses GPUs in the forward, and the backward ends
with one NCCL all-reduce(sum) of the twiddle gradient.

One JSON line is printed by rank 0:
  value      algorithmic GB/s of fw+bw over all ranks, inputs resident in HBM
  e2e        the same metric through the public torch operator with HOST buffers: every
             step copies input and grad from pinned host memory and copies output,
             input gradient and twiddle gradient back
  roofline   the dominant kernel's algorithmic bytes per launch / its CUDA-event duration,
             against the measured HBM copy bandwidth (MEASURED_PEAKS.json)
  cpu_baseline  the reference's CPU implementation timed on a bounded sample of the rows

--impl reference times the reference's own CPU path (its compiled CPU operator when
oracle/_ref holds it, else the C oracle) on the host cores instead.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0


def measured_hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        return self.snapshot()

    def snapshot(self):
        """Summary of the samples taken so far."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in list(self.lines):
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def load_configs():
    """The configuration table, loaded by path: importing the package would map the product's
    libraries into a process that is only meant to run the reference."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bfly_bench_configs", os.path.join(ROOT, "butterfly_b200", "configs.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


# ------------------------------------------------------------------------------ CPU reference arm

def _cpu_reference_runner():
    """Returns (kind, fw_bw_callable).  Prefers the reference's own CPU operator."""
    import oracle
    if oracle.reference_available(cuda=False) or oracle.reference_available(cuda=True):
        ops = oracle.load_reference_ops(cuda=not oracle.reference_available(cuda=False))

        def run(tw, x, g, inc):
            n = 1 << tw.shape[2]
            y = ops.butterfly_multiply_fw(tw, x, inc, n)
            d_tw, d_x = ops.butterfly_multiply_bw(tw, x, g, inc)
            return y, d_tw, d_x
        return "reference", run
    oracle.build()

    def run(tw, x, g, inc):
        y = oracle.multiply_fw(tw, x, inc)
        d_tw, d_x = oracle.multiply_bw(tw, x, g, inc)
        return y, d_tw, d_x
    return "port", run


_CPU_INPUTS = {}


def cpu_reference_time(cfg_name, rows, cores, reps=1):
    """Times fw+bw of the reference CPU path on `rows` rows of the workload, split over `cores` threads.

    The reference CPU kernels are single-threaded loops (csrc/cpu/butterfly_cpu.cpp:33-60);
    rows are independent, so the sample is cut into `cores` row chunks that run concurrently
    (the operator call releases the GIL) and the twiddle gradients of the chunks are summed.
    """
    from concurrent.futures import ThreadPoolExecutor
    configs = load_configs()
    kind, run = _cpu_reference_runner()
    torch.set_num_threads(1)
    if (cfg_name, rows) not in _CPU_INPUTS:
        _CPU_INPUTS[(cfg_name, rows)] = configs.make_inputs(cfg_name, batch=rows)
    d = _CPU_INPUTS[(cfg_name, rows)]
    tw, x, g, inc = d["twiddle"], d["input"].contiguous(), d["grad"], d["increasing_stride"]
    chunks = [c for c in torch.arange(rows).chunk(cores) if c.numel()]
    pool = ThreadPoolExecutor(max_workers=len(chunks))

    def work(idx):
        return run(tw, x[idx[0]:idx[-1] + 1], g[idx[0]:idx[-1] + 1], inc)
    run(tw, x[:2], g[:2], inc)  # warm-up (page in the library)
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        res = list(pool.map(work, chunks))
        d_tw = res[0][1]
        for r in res[1:]:
            d_tw = d_tw + r[1]
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    pool.shutdown()
    return kind, best, len(chunks)


def run_reference_arm(args):
    configs = load_configs()
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    rows = args.ref_rows
    fwb, bwb = configs.algorithmic_bytes(args.config, batch=rows)
    times = []
    kind = None
    for i in range(args.warmup + args.steps):
        kind, t, used = cpu_reference_time(args.config, rows, cores)
        if i >= args.warmup:
            times.append(t)
    tsum = sum(times)
    n = configs.CONFIGS[args.config]
    value = (fwb + bwb) * len(times) / tsum / 1e9
    line = {
        "impl": "reference", "metric": "fw+bw butterfly multiply GB/s", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * tsum / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32" if n["dtype"] == torch.float32 else "c64", "data": "synthetic",
        "config": {"workload": args.config, "n": 1 << n["log_n"], "nblocks": n["nblocks"], "nstacks": n["nstacks"],
                   "batch_per_step": rows, "note": "bounded sample of the workload's rows per step"},
        "batch_n_per_s": rows * n["nstacks"] * (1 << n["log_n"]) * len(times) / tsum,
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": used, "kind": kind,
                         "sample": "%d of %d rows per step, fw+bw, %d row chunks on %d threads" % (rows, n["batch"], used, used)},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------ GPU arm

# (config, kernel) -> (dram__bytes_read.sum + dram__bytes_write.sum per launch, batch of the capture):
# mean over the phase launches of one backward call in the ncu capture summarised under profiles/
NCU_DRAM_BYTES = {("cfg2", "bfly_bw3_kernel"): (569.9e6, 12288), ("cfg2", "bfly_bw2_kernel"): (165.1e6, 4096),
                  ("cfg2", "bfly_fw2_kernel"): (85.9e6, 4096)}


def fp32_ceiling_gbs(cfg, B, step_bytes, sm_mhz, sms=148):
    """Algorithmic GB/s of fw+bw if only the FP32 pipes limited it (real radix-2 products).

    Per element and stage: forward 2 multiply-add lane operations; backward 4 (twiddle gradient and
    input gradient) + 2 for each recomputed stage (the snapshot pass covers all but the last phase,
    the phases recompute all but their last sub-group; 3/4 and 2/3 of the stages for 24 stages),
    at 128 lanes per SM and the SM clock sampled during the run."""
    import torch
    if cfg["base4"] or cfg["dtype"] != torch.float32 or not sm_mhz:
        return None
    stages = cfg["nblocks"] * cfg["log_n"]
    elem_stages = float(B) * cfg["nstacks"] * (1 << cfg["log_n"]) * stages
    lane_ops = elem_stages * (2 + 4 + 2 * 0.75 + 2 * (2.0 / 3.0))
    seconds = lane_ops / (sms * 128 * sm_mhz * 1e6)
    return step_bytes / seconds / 1e9


def _events_ms(fn, iters, warm):
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def _graph_us_per_call(fn, iters=200):
    """Device time of one operator call replayed from a CUDA graph (no host work per call)."""
    import torch
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return _events_ms(graph.replay, iters, 20) * 1e3


def _host_us_per_call(fn, iters=200):
    """Host time of one operator call (enqueue only: the stream is drained before and after)."""
    import torch
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    t1 = time.perf_counter()
    torch.cuda.synchronize()
    return 1e6 * (t1 - t0) / iters


def measure_config(bb, configs, name, dev, peak, make=None, iters=5, warm=3, ref_ops=None):
    """fw and bw of one configuration, timed separately with CUDA events (inputs resident in HBM):
    ms, algorithmic GB/s and the fraction of the HBM peak; with `ref_ops` the same through the
    reference's CUDA extension."""
    import torch
    d = make() if make else configs.make_inputs(name, device=dev)
    inc = d["increasing_stride"]
    x, g = d["input"], d.get("grad")
    fwb, bwb = d["bytes"] if "bytes" in d else configs.algorithmic_bytes(name, batch=d["batch"])
    if d.get("base4"):
        t4, t2 = d["twiddle4"], d["twiddle2"]
        fw = lambda: bb.butterfly_multiply_base4_fw(t4, t2, x, inc)
        bw = (lambda: bb.butterfly_multiply_base4_bw(t4, t2, x, g, inc)) if g is not None else None
    else:
        tw = d["twiddle"]
        fw = lambda: bb.butterfly_multiply_fw(tw, x, inc)
        bw = (lambda: bb.butterfly_multiply_bw(tw, x, g, inc)) if g is not None else None
    out = {"name": name, "n": d["n"], "batch": d["batch"], "nstacks": int(x.shape[1]),
           "dtype": "f32" if x.dtype == torch.float32 else "c64"}
    fw_ms = _events_ms(fw, iters, warm)
    out.update(fw_ms=fw_ms, fw_gbs=fwb / fw_ms / 1e6, fw_frac_of_hbm_peak=fwb / fw_ms / 1e6 / peak)
    if bw is not None:
        bw_ms = _events_ms(bw, iters, warm)
        out.update(bw_ms=bw_ms, bw_gbs=bwb / bw_ms / 1e6,
                   fw_bw_gbs=(fwb + bwb) / (fw_ms + bw_ms) / 1e6,
                   fw_bw_frac_of_hbm_peak=(fwb + bwb) / (fw_ms + bw_ms) / 1e6 / peak)
    else:
        out["fw_host_us_per_call"] = _host_us_per_call(fw)  # latency-bound case: the launch path matters
        out["fw_graph_replay_us"] = _graph_us_per_call(fw)  # the same call captured once into a CUDA graph
    if ref_ops is not None and not d.get("base4"):
        n = d["n"]
        rfw = lambda: ref_ops.butterfly_multiply_fw(tw, x, inc, n)
        out["reference_cuda_fw_ms"] = _events_ms(rfw, 3, 1)
        if g is not None:
            rbw = lambda: ref_ops.butterfly_multiply_bw(tw, x, g, inc)
            out["reference_cuda_bw_ms"] = _events_ms(rbw, 3, 1)
    return out


def measure_linear_layer(bb, configs, dev, peak, rank=0, iters=5, warm=3):
    """Configuration 5 as what it is in a model -- a 1024 -> 4096 linear layer with bias: the fused
    operators (bias in the forward's store, input gradient summed over the stacks and bias
    gradient inside the backward kernels) beside the same layer through the multiply operators
    plus PyTorch glue (expand, flatten, bias add; sum over stacks, column sum of grad)."""
    import torch
    d = configs.make_inputs("cfg5", rank=rank, device=dev)
    tw, inc, S, n = d["twiddle"], d["increasing_stride"], 4, d["n"]
    B = d["batch"]
    x2 = d["input"][:, 0].contiguous()          # (B, 1024)
    g2 = d["grad"].reshape(B, S * n)            # (B, 4096)
    bias = torch.randn(S * n, device=dev)
    twb = tw.numel() * 4
    fwb = 4 * (B * n + B * S * n + S * n) + twb
    bwb = 4 * (B * n + B * S * n + B * n + S * n) + 2 * twb
    fused_fw = lambda: bb.butterfly_linear_fw(tw, x2, bias, inc, S * n)
    fused_bw = lambda: bb.butterfly_linear_bw(tw, x2, g2, inc, True)

    def glue_fw():
        rows = x2.unsqueeze(1).expand(B, S, n)
        return bb.butterfly_multiply_fw(tw, rows, inc).reshape(B, S * n) + bias

    def glue_bw():
        rows = x2.unsqueeze(1).expand(B, S, n)
        d_tw, d_x = bb.butterfly_multiply_bw(tw, rows, g2.view(B, S, n), inc)
        return d_tw, d_x.sum(1), g2.sum(0)
    out = {"name": "cfg5 as a linear layer with bias (1024 -> 4096)", "n": n, "batch": B, "nstacks": S, "dtype": "f32",
           "fw_ms": _events_ms(fused_fw, iters, warm), "bw_ms": _events_ms(fused_bw, iters, warm),
           "unfused_fw_ms": _events_ms(glue_fw, iters, warm), "unfused_bw_ms": _events_ms(glue_bw, iters, warm),
           "fw_algorithmic_bytes": fwb, "bw_algorithmic_bytes": bwb}
    out["fw_bw_gbs"] = (fwb + bwb) / (out["fw_ms"] + out["bw_ms"]) / 1e6
    out["fw_bw_frac_of_hbm_peak"] = out["fw_bw_gbs"] / peak
    return out


def measure_glue_rows(bb, dev, peak, iters=5, warm=3):
    """The layers next to the multiply, fused against link by link, on inputs larger than L2:
    an FFT with its bit-reversal and a circulant on real rows (glue operators inside the forward
    launch), a 2-D butterfly map (one multiply over the flattened image against two passes around a
    transpose), and the unitary twiddle synthesis (one kernel each way against the torch chain)."""
    import torch
    from butterfly_b200 import special, combine
    out = []
    with torch.no_grad():
        n, B = 2048, 16384  # 268 MB of complex64 rows
        x = torch.randn(B, n, dtype=torch.complex64, device=dev)
        fused, chained = special.fft(n).to(dev), special.fft(n, fused=False).to(dev)
        e = {"name": "fft n=2048 complex64 with bit reversal", "batch": B,
             "fused_fw_ms": _events_ms(lambda: fused(x), iters, warm), "link_by_link_fw_ms": _events_ms(lambda: chained(x), iters, warm),
             "algorithmic_bytes": 2 * B * n * 8}
        e["fused_gbs"] = e["algorithmic_bytes"] / e["fused_fw_ms"] / 1e6
        e["fused_frac_of_hbm_peak"] = e["fused_gbs"] / peak
        out.append(e)
        del x
        n, B = 2048, 32768  # 268 MB of float32 rows in, the same out
        x = torch.randn(B, n, device=dev)
        col = torch.randn(n)
        fused, chained = special.circulant(col).to(dev), special.circulant(col, fused=False).to(dev)
        e = {"name": "circulant n=2048 on float32 rows (real to complex, fft, diagonal, ifft, real part)", "batch": B,
             "fused_fw_ms": _events_ms(lambda: fused(x), iters, warm), "link_by_link_fw_ms": _events_ms(lambda: chained(x), iters, warm),
             "algorithmic_bytes": 2 * B * n * 4}
        e["fused_gbs"] = e["algorithmic_bytes"] / e["fused_fw_ms"] / 1e6
        e["fused_frac_of_hbm_peak"] = e["fused_gbs"] / peak
        out.append(e)
        del x
        h = w = 64
        B = 8192  # 268 MB of complex64 images
        x = torch.randn(B, h, w, dtype=torch.complex64, device=dev)
        b1 = bb.Butterfly(w, w, False, True, True).to(dev)
        b2 = bb.Butterfly(h, h, False, True, True).to(dev)
        one, two = combine.TensorProduct(b1, b2), combine.TensorProduct(b1, b2, fused=False)
        e = {"name": "tensor product of two butterflies on 64x64 complex64 images", "batch": B,
             "fused_fw_ms": _events_ms(lambda: one(x), iters, warm), "link_by_link_fw_ms": _events_ms(lambda: two(x), iters, warm),
             "algorithmic_bytes": 2 * B * h * w * 8}
        e["fused_gbs"] = e["algorithmic_bytes"] / e["fused_fw_ms"] / 1e6
        e["fused_frac_of_hbm_peak"] = e["fused_gbs"] / peak
        out.append(e)
        del x
    layer = bb.ButterflyUnitary(4096, 4096, bias=False, nblocks=2).to(dev)
    angles = layer.twiddle.detach().clone().requires_grad_(True)
    g = torch.randn(angles.shape[:-1] + (2, 2), dtype=torch.complex64, device=dev)

    def chain():
        phi, alpha, psi, chi = torch.unbind(angles, -1)
        c, s_ = torch.cos(phi), torch.sin(phi)
        pol = lambda r, a: torch.stack((r * torch.cos(a), r * torch.sin(a)), dim=-1)
        tw = torch.stack([torch.stack([pol(c, alpha + psi), pol(s_, alpha + chi)], dim=-2),
                          torch.stack([pol(-s_, alpha - chi), pol(c, alpha - psi)], dim=-2)], dim=-3)
        torch.view_as_complex(tw).backward(g)
        angles.grad = None

    def kernels():
        bb.unitary_twiddle(angles).backward(g)
        angles.grad = None
    out.append({"name": "unitary twiddle synthesis and its backward, n=4096, two blocks", "blocks_2x2": angles.numel() // 4,
                "fused_fw_bw_ms": _events_ms(kernels, iters, warm), "link_by_link_fw_bw_ms": _events_ms(chain, iters, warm)})
    return out


def two_block_inputs(log_n, dev, elements=1 << 26):
    """Real fp32 two-block product (increasing then decreasing stride) over `elements` elements."""
    import math
    import torch
    n = 1 << log_n
    B = elements // n
    g = torch.Generator().manual_seed(log_n)
    tw = (torch.randn(1, 2, log_n, n // 2, 2, 2, generator=g) / math.sqrt(2)).to(dev)
    x = torch.randn(B, 1, n, generator=g).to(dev)
    gr = torch.randn(B, 1, n, generator=g).to(dev)
    twb = tw.numel() * 4
    plane = B * n * 4
    return dict(twiddle=tw, input=x, grad=gr, increasing_stride=True, n=n, batch=B, base4=False,
                bytes=(2 * plane + twb, 3 * plane + 2 * twb))


def run_gpu_arm(args):
    import torch.distributed as dist
    import butterfly_b200 as bb
    from butterfly_b200 import abi, configs
    from butterfly_b200.distributed import AsyncTwiddleReducer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the GPU arm has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    cfg = configs.CONFIGS[args.config]
    if cfg["base4"] or cfg.get("forward_only"):
        raise SystemExit("bench.py's headline loop times fw+bw of a radix-2 config (cfg2, cfg3, cfg5); "
                         "cfg1 and cfg4 are measured in other_configs")
    d = configs.make_inputs(args.config, batch=args.batch, rank=rank, device=dev)
    tw, x, g, inc = d["twiddle"], d["input"], d["grad"], d["increasing_stride"]
    B, S, n = d["batch"], cfg["nstacks"], d["n"]
    fwb, bwb = configs.algorithmic_bytes(args.config, batch=args.batch)
    step_bytes = fwb + bwb
    # the twiddle gradient of step k is all-reduced on a side stream while step k+1 computes
    reducer = AsyncTwiddleReducer(dev) if world > 1 else None

    def step():
        y = bb.butterfly_multiply_fw(tw, x, inc)
        d_tw, d_x = bb.butterfly_multiply_bw(tw, x, g, inc)
        if reducer is not None:
            reducer.submit(d_tw)
        return y, d_tw, d_x

    def barrier():
        if reducer is not None:
            reducer.wait()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    nwarm = args.warmup if args.batch is not None else max(args.warmup, 3)  # small profiling cases may use fewer
    for _ in range(nwarm):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    launches0 = abi.launch_count()
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    if reducer is not None:
        reducer.wait()  # the timed region ends when the last all-reduce has finished
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = abi.launch_count() - launches0
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    value = step_bytes * world / (ms_per_step * 1e-3) / 1e9

    # ---- per-kernel durations (separate untimed passes, CUDA events around every launch): the
    # forward calls and the backward calls apart, so that the backward's own forward pass (the
    # snapshot pass) is not mixed up with the forward operator
    NPROF = 3
    abi.profile_enable(True)
    for _ in range(NPROF):
        bb.butterfly_multiply_fw(tw, x, inc)
    torch.cuda.synchronize()
    prof_fw = abi.profile_collect()
    for _ in range(NPROF):
        bb.butterfly_multiply_bw(tw, x, g, inc)
    torch.cuda.synchronize()
    prof_bw = abi.profile_collect()
    abi.profile_enable(False)
    peak, peak_src = measured_hbm_peak()

    clocks_mid = sampler.snapshot() if rank == 0 else None
    # dominant kernel = largest time share of a step.  Its algorithmic bytes: the operator's
    # algorithmic bytes (forward: input + output + twiddle; backward: input + grad + d_input +
    # twiddle + d_twiddle -- each tensor once, never the design's own snapshot traffic) divided
    # over the launches of that kernel which do the operator's work
    shares = {}
    for k, (nl, tms) in prof_fw.items():
        if nl:
            shares[("fw", k)] = (nl / NPROF, tms / NPROF)
    for k, (nl, tms) in prof_bw.items():
        if nl:
            shares[("bw", k)] = (nl / NPROF, tms / NPROF)
    (dom_op, dom), (dom_launches, dom_ms) = max(shares.items(), key=lambda kv: kv[1][1])
    # the backward's phase launches carry the backward's algorithmic bytes; its forward pass
    # (snapshots) is extra work of the design and gets none
    phase_kernels = [k for (op, k) in shares if op == "bw" and k.startswith("bfly_bw")]
    if dom_op == "fw":
        alg = fwb / dom_launches
    elif dom in phase_kernels:
        alg = bwb / sum(shares[("bw", k)][0] for k in phase_kernels)
    else:
        alg = 0.0
    avg_ms = dom_ms / dom_launches
    achieved = alg / (avg_ms * 1e-3) / 1e9
    traffic = None
    cap = NCU_DRAM_BYTES.get((args.config, dom))
    if cap is not None:
        traffic = cap[0] * B / cap[1]
    kernel_ms = {"forward: " + k: v[1] for (op, k), v in shares.items() if op == "fw"}
    kernel_ms.update({"backward: " + k: v[1] for (op, k), v in shares.items() if op == "bw"})
    bw_total_ms = sum(v[1] for (op, k), v in shares.items() if op == "bw")
    roofline = {"bound": "hbm", "kernel": dom, "operator": "forward" if dom_op == "fw" else "backward",
                "achieved": achieved, "peak": peak, "peak_source": peak_src,
                "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
                "traffic_over_algorithmic": (traffic / alg) if (traffic and alg) else None,
                "traffic_source": ("ncu dram__bytes_read+write of a batch-%d capture, scaled by rows" % cap[1]) if cap else None,
                "launches_per_step": dom_launches, "avg_launch_ms": avg_ms, "algorithmic_bytes_per_launch": alg,
                "kernel_ms_per_step": kernel_ms,
                "forward_frac_of_hbm_peak": fwb / (sum(v[1] for (op, k), v in shares.items() if op == "fw") * 1e-3) / 1e9 / peak,
                "backward_frac_of_hbm_peak": bwb / (bw_total_ms * 1e-3) / 1e9 / peak,
                "op_frac_of_hbm_peak": (step_bytes / (ms_per_step * 1e-3) / 1e9) / peak}

    # ---- end to end through the public operator with host buffers
    e2e = None
    if not args.no_e2e:
        hx = torch.empty(x.shape if not cfg.get("broadcast_stacks") else (B, 1, n), dtype=x.dtype).pin_memory()
        hx.copy_(x[:, :1] if cfg.get("broadcast_stacks") else x)
        hg = torch.empty(g.shape, dtype=g.dtype).pin_memory(); hg.copy_(g)
        hy = torch.empty((B, S, n), dtype=x.dtype).pin_memory()
        hdx = torch.empty((B, S, n), dtype=x.dtype).pin_memory()
        hdt = torch.empty(tw.shape, dtype=tw.dtype).pin_memory()
        sz = 4 if cfg["dtype"] == torch.float32 else 8

        from butterfly_b200.host import HostPipeline
        pipe = HostPipeline(dev, chunks=args.e2e_chunks)

        def e2e_step():
            # public host-side API: chunked upload / fw+bw / download on three streams
            d_tw = pipe.fw_bw(tw, hx, hg, inc, hy, hdx, hdt)
            if reducer is not None:
                reducer.submit(d_tw)
        h2d = hx.numel() * sz + hg.numel() * sz
        d2h = (hy.numel() + hdx.numel() + hdt.numel()) * sz
        e2e_steps = max(1, min(args.steps, 20))
        for _ in range(2):
            e2e_step()
        barrier()
        a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(e2e_steps):
            e2e_step()
        if reducer is not None:
            reducer.wait()
        pipe.join()  # the last downloads belong to the timed region
        b.record()
        barrier()
        ems = a.elapsed_time(b)
        # the two copy directions alone (same pinned buffers, same chunking), to show what bounds the pipeline
        h2d_ms = _events_ms(lambda: pipe.upload_only(hx, hg), 3, 1)
        d2h_ms = _events_ms(lambda: pipe.download_only(hy, hdx), 3, 1)
        if world > 1:
            t = torch.tensor([ems, h2d_ms, d2h_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ems, h2d_ms, d2h_ms = [float(v) for v in t.tolist()]
        e2e = {"value": step_bytes * world / (ems / e2e_steps * 1e-3) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ems / e2e_steps,
               "steps": e2e_steps, "api": "butterfly_b200.host.HostPipeline.fw_bw (%d row chunks, 3 streams)" % args.e2e_chunks,
               "h2d_alone_gbs_per_rank": h2d / h2d_ms / 1e6, "d2h_alone_gbs_per_rank": (d2h - hdt.numel() * sz) / d2h_ms / 1e6,
               "pcie_gbs_aggregate": (h2d + d2h) * world / (ems / e2e_steps) / 1e6}

    # ---- the other configurations and the reference's CUDA extension (the kernel to beat), untimed
    # by the headline loop
    other, ref_cuda_note = None, None
    if rank == 0 and world == 1 and not args.no_other and args.batch is None:
        ref_ops = None
        if not args.no_refcuda:
            try:
                import oracle
                if oracle.reference_available(cuda=True):
                    ref_ops = oracle.load_reference_ops(cuda=True)
                else:
                    ref_cuda_note = {"kind": "unavailable", "why": "oracle/_ref/_butterfly_ref_cuda.so not built"}
            except Exception as e:  # the comparison column is optional
                ref_cuda_note = {"kind": "unavailable", "why": repr(e)[:200]}
        other = []
        for name in ("cfg1", "cfg2", "cfg3", "cfg4", "cfg5"):
            other.append(measure_config(bb, configs, name, dev, peak, ref_ops=ref_ops))
        for log_n in (10, 11, 13):
            other.append(measure_config(bb, configs, "two-block n=%d" % (1 << log_n), dev, peak,
                                        make=lambda: two_block_inputs(log_n, dev), ref_ops=ref_ops if log_n <= 11 else None))
        other.append(measure_linear_layer(bb, configs, dev, peak))
        other.extend(measure_glue_rows(bb, dev, peak))
        if ref_ops is not None:
            ref_cuda_note = {"kind": "reference", "library": "oracle/_ref/_butterfly_ref_cuda.so",
                             "what": "csrc/cuda/butterfly_cuda.cu of the reference compiled unmodified for sm_100; "
                                     "reference_cuda_*_ms in other_configs"}
    elif rank == 0 and world > 1 and not args.no_other:
        # the multi-GPU configuration: this rank's shard of cfg5 (8192 rows, stack-broadcast input)
        other = [measure_config(bb, configs, "cfg5", dev, peak,
                                make=lambda: configs.make_inputs("cfg5", rank=rank, device=dev)),
                 measure_linear_layer(bb, configs, dev, peak, rank=rank)]

    # the sampler ran through the kernel-timed loop, the per-kernel pass and the end-to-end loop
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        roofline["fp32_ceiling_gbs"] = fp32_ceiling_gbs(cfg, B, step_bytes, (clocks_mid or clocks or {}).get("sm_mhz"))

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        try:
            rows = args.ref_rows
            cores = os.cpu_count() or 1
            kind, t, used = cpu_reference_time(args.config, rows, cores)
            rfw, rbw = configs.algorithmic_bytes(args.config, batch=rows)
            cpu_baseline = {"value": (rfw + rbw) / t / 1e9, "unit": "GB/s", "cores": used, "kind": kind,
                            "sample": "%d of %d rows, one fw+bw, %d row chunks on %d threads, %.2f s"
                                      % (rows, B, used, used, t)}
        except Exception as e:  # the baseline is reported, never needed by the GPU path
            cpu_baseline = {"value": None, "unit": "GB/s", "cores": 0, "kind": "unavailable", "sample": repr(e)}

    if rank == 0:
        line = {
            "metric": "fw+bw butterfly multiply GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": nwarm, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32" if cfg["dtype"] == torch.float32 else "c64", "data": "synthetic",
            "config": {"workload": args.config, "n": n, "nblocks": cfg["nblocks"], "nstacks": S,
                       "batch_per_gpu": B, "global_batch": B * world, "parallelism": "batch-sharded x%d" % world,
                       "l2": "inputs (%.0f MB per step per GPU) exceed the 126 MB L2; no flush" % (step_bytes / 1e6),
                       "collective": ("one NCCL all-reduce(sum) of d_twiddle per step, on a side stream while the next "
                                      "step computes") if world > 1 else "none"},
            "batch_n_per_s": B * S * n * world / (ms_per_step * 1e-3),
            "frac_of_hbm_peak": value / world / peak,
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "clocks": clocks,
            "gpu_launches": launches, "other_configs": other, "reference_cuda": ref_cuda_note,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="cfg2", choices=["cfg2", "cfg3", "cfg5"])
    ap.add_argument("--ref-rows", type=int, default=4096, help="rows of the bounded CPU sample")
    ap.add_argument("--batch", type=int, default=None, help="override the batch per GPU (profiling a small case)")
    ap.add_argument("--e2e-chunks", type=int, default=8, help="row chunks of the host-memory pipeline")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-other", action="store_true", help="skip the other configurations (other_configs)")
    ap.add_argument("--no-refcuda", action="store_true", help="skip the reference's CUDA extension in other_configs")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
