"""Forward + backward of the butterfly multiply for operands that live in HOST memory.

A caller whose tensors sit in (pinned) host memory -- the situation of a CPU-resident
pipeline that offloads this operator to the GPU -- pays for two PCIe transfers per step that
dwarf the kernels.  `HostPipeline` cuts the batch into row chunks and runs three CUDA streams
(host->device copies, the operators, device->host copies) so that uploads, compute and
downloads of different chunks overlap and both PCIe directions are busy at once.  The twiddle
gradient is additive over rows, so the chunks' partial gradients are summed on the device.
"""
import torch

from . import abi
from .multiply import butterfly_multiply_bw, butterfly_multiply_fw


class HostPipeline:
    """fw+bw over host-resident input / grad / outputs.

        pipe = HostPipeline(device, chunks=8)
        pipe.fw_bw(twiddle_dev, x_host, grad_host, increasing_stride, out_host, d_x_host, d_twiddle_host)

    x_host (B, Sx, n) with Sx = 1 (one row shared by all stacks) or Sx = nstacks; grad_host,
    out_host, d_x_host (B, nstacks, n); all pinned.

    fw_bw only ENQUEUES the work: when it returns, the caller's current stream has been made to
    wait for the kernels (the returned device tensor), not for the downloads, and the host has not
    waited for anything.  Call ``wait()`` before reading out_host / d_x_host / d_twiddle_host on
    the CPU, ``join()`` before device work that must follow the downloads.  Consecutive calls
    overlap: the uploads of the next call run while the downloads of this one drain (downloads are
    ordered among themselves, so re-using the same host buffers keeps the last call's results).
    """

    def __init__(self, device, chunks=8):
        self.device = torch.device(device)
        self.chunks = chunks
        self.s_in = torch.cuda.Stream(self.device)
        self.s_comp = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.flag = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.inflight = []

    def fw_bw(self, twiddle, x_host, grad_host, increasing_stride, out_host, d_x_host, d_twiddle_host):
        B = x_host.shape[0]
        S = grad_host.shape[1]
        n = grad_host.shape[2]
        dev = self.device
        cur = torch.cuda.current_stream(dev)
        # at most two calls in flight: the host waits for the call before the previous one, so that
        # device buffers are recycled instead of growing with every call enqueued ahead
        while len(self.inflight) >= 2:
            self.inflight.pop(0).synchronize()
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_stream(cur)
        bounds = [(B * c // self.chunks, B * (c + 1) // self.chunks) for c in range(self.chunks)]
        d_tw_total = None
        keep = []  # device tensors stay referenced until their stream is done
        for lo, hi in bounds:
            if hi == lo:
                continue
            with torch.cuda.stream(self.s_in):
                xd = x_host[lo:hi].to(dev, non_blocking=True)
                gd = grad_host[lo:hi].to(dev, non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(self.s_in)
            with torch.cuda.stream(self.s_comp):
                self.s_comp.wait_event(ev_in)
                xd.record_stream(self.s_comp)
                gd.record_stream(self.s_comp)
                xr = xd.expand(hi - lo, S, n) if xd.shape[1] != S else xd
                y = butterfly_multiply_fw(twiddle, xr, increasing_stride)
                d_tw, d_x = butterfly_multiply_bw(twiddle, xr, gd, increasing_stride)
                d_tw_total = d_tw if d_tw_total is None else d_tw_total.add_(d_tw)
                ev_c = torch.cuda.Event()
                ev_c.record(self.s_comp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_c)
                y.record_stream(self.s_out)
                d_x.record_stream(self.s_out)
                out_host[lo:hi].copy_(y, non_blocking=True)
                d_x_host[lo:hi].copy_(d_x[:, :, :d_x_host.shape[2]], non_blocking=True)
            keep.append((xd, gd, y, d_x))
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_stream(self.s_comp)
            if d_tw_total is not None:
                d_tw_total.record_stream(self.s_out)
                d_twiddle_host.copy_(d_tw_total, non_blocking=True)
            # the kernels' give-up flag travels with the last download; wait() looks at it
            abi.device_error_async(self.flag)
            self.done = torch.cuda.Event()
            self.done.record(self.s_out)
            self.inflight.append(self.done)
        # The caller's stream waits for the compute stream only (the returned device tensor is final
        # there); it does not wait for the downloads, so that the uploads of the next call overlap them.
        # Host code reads the host buffers after wait(); device work that must follow the downloads
        # calls join().
        cur.wait_stream(self.s_comp)
        return d_tw_total

    def join(self):
        """Makes the current stream wait for the downloads enqueued so far (no host synchronisation)."""
        torch.cuda.current_stream(self.device).wait_stream(self.s_out)

    def wait(self):
        """Blocks the host until the downloads of the last fw_bw call have landed in host memory; raises if
        a kernel of that call gave up on a bounded wait (its results are then invalid)."""
        if getattr(self, "done", None) is not None:
            self.done.synchronize()
            if int(self.flag.item()) != 0:
                code = abi.device_error()  # clears the flag
                raise RuntimeError("butterfly_b200: a kernel gave up on a bounded wait (flag %d); the results of the "
                                   "last fw_bw call are invalid" % code)

    # The two copy directions alone, with the same chunking and streams: what each direction of the
    # host link sustains without the other (benchmarks report them beside the pipelined number).
    def upload_only(self, x_host, grad_host):
        B = x_host.shape[0]
        cur = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(cur)
        with torch.cuda.stream(self.s_in):
            for c in range(self.chunks):
                lo, hi = B * c // self.chunks, B * (c + 1) // self.chunks
                if hi > lo:
                    x_host[lo:hi].to(self.device, non_blocking=True)
                    grad_host[lo:hi].to(self.device, non_blocking=True)
        cur.wait_stream(self.s_in)

    def download_only(self, out_host, d_x_host):
        B = out_host.shape[0]
        cur = torch.cuda.current_stream(self.device)
        self.s_out.wait_stream(cur)
        with torch.cuda.stream(self.s_out):
            for c in range(self.chunks):
                lo, hi = B * c // self.chunks, B * (c + 1) // self.chunks
                if hi > lo:
                    src = torch.empty((hi - lo,) + tuple(out_host.shape[1:]), dtype=out_host.dtype, device=self.device)
                    out_host[lo:hi].copy_(src, non_blocking=True)
                    d_x_host[lo:hi].copy_(src, non_blocking=True)
        cur.wait_stream(self.s_out)
