"""Forward + backward of the sliding-window 2-simplicial attention for tensors that live in HOST memory.

The reference's operator takes CUDA tensors only
(simplicial_attention/triton_two_simplicial_attention.py:729); a caller whose
activations sit in pinned host memory pays a host->device copy before and a
device->host copy after every call.  Batch elements are independent, so
``HostPipeline`` cuts a call into batch chunks and runs three streams: chunk
``c+1`` is copied in while chunk ``c`` is computed and chunk ``c-1`` is copied
out.  Calls may be queued back to back (the host tensors must already hold their
data when ``run`` is called); ``synchronize()`` waits for all of them.
PCIe is full duplex, so in steady state a call costs the larger of its compute
time and one direction's copy time instead of their sum.

Everything is computed by the CUDA library behind the C ABI (``sa2_fwd`` /
``sa2_bwd``); this file only schedules copies and launches.
"""
from __future__ import annotations

import torch

from .attention import check_device, sa2_backward, sa2_forward


def bind_to_device_cpus(device) -> list | None:
    """Restrict this process to the CPUs that NVML reports as local to ``device`` (a read-only query),
    intersected with the CPUs it may already use.  Pinned host buffers allocated afterwards, and the thread
    that queues the copies, then sit on the GPU's side of the machine: with several ranks on a two-socket
    host, copies from the far socket ran at a fifth of the near one's rate.  Returns the CPUs, or None when
    nothing was changed (no NVML, no local CPU in the allowed set, not Linux)."""
    import os
    try:
        import pynvml as n
        n.nvmlInit()
        index = torch.device(device).index or 0
        uuid = str(torch.cuda.get_device_properties(index).uuid)
        handle = None
        for k in range(n.nvmlDeviceGetCount()):
            h = n.nvmlDeviceGetHandleByIndex(k)
            u = n.nvmlDeviceGetUUID(h)
            u = u.decode() if isinstance(u, bytes) else u
            if uuid in u:
                handle = h
        if handle is None:
            return None
        allowed = os.sched_getaffinity(0)
        words = n.nvmlDeviceGetCpuAffinity(handle, (max(allowed) + 64) // 64)
        local = {64 * w + bit for w, word in enumerate(words) for bit in range(64) if (int(word) >> bit) & 1}
        cpus = sorted(local & allowed)
        if not cpus or len(cpus) == len(allowed):
            return None
        os.sched_setaffinity(0, cpus)
        return cpus
    except Exception:
        return None


class HostPipeline:
    """``run(inputs, outputs)`` with ``inputs = (q, k1, k2, v1, v2, dout)`` and
    ``outputs = (out, dq, dk1, dk2, dv1, dv2)``, all pinned host tensors of
    layout ``(b, n, h, d)``; results are valid after ``synchronize()``."""

    def __init__(self, device, w1=512, w2=32, chunk=2, slots=2, kernel="auto"):
        self.device = torch.device(device)
        self.w1, self.w2, self.chunk, self.kernel = int(w1), int(w2), int(chunk), kernel
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.slots = [None] * slots          # device copies of one chunk's six inputs
        self.free = [None] * slots           # event: the slot's inputs are no longer read
        self.results = [None] * slots        # device copies of one chunk's six results, reused from call to call
        self.copied = [None] * slots         # event: the slot's results have been copied out
        self.turn = 0
        self.timed = False                   # record_copies(): events around every chunk's copies
        self._copies = []                    # (direction, bytes, start event, end event)

    def record_copies(self, on=True):
        """Time every chunk's host->device and device->host copies with events on the copy streams;
        ``copy_stats()`` turns them into GB/s per direction (the time each copy stream was busy)."""
        self.timed = bool(on)
        self._copies = []

    def copy_stats(self):
        """``{"h2d_gbs", "d2h_gbs", "h2d_bytes", "d2h_bytes"}`` over the copies recorded since
        ``record_copies()``; call after ``synchronize()``."""
        res = {}
        for name in ("h2d", "d2h"):
            rows = [(nb, a.elapsed_time(b)) for d, nb, a, b in self._copies if d == name]
            nbytes, ms = sum(r[0] for r in rows), sum(r[1] for r in rows)
            res[name + "_bytes"] = nbytes
            res[name + "_gbs"] = nbytes / (ms * 1e-3) / 1e9 if ms > 0 else None
        return res

    def _stage(self, slot, parts):
        bufs = self.slots[slot]
        if bufs is None or any(b.shape != p.shape or b.dtype != p.dtype for b, p in zip(bufs, parts)):
            bufs = [torch.empty(p.shape, dtype=p.dtype, device=self.device) for p in parts]
            self.slots[slot] = bufs
        return bufs

    def _result_buffers(self, slot, dev, outputs, sl):
        """out and the five gradients of the slot: allocated once per chunk shape, so that steady-state calls
        allocate nothing on the device but their scratch (which is returned to the pool on the compute stream)."""
        shapes = [dev[0].shape] + [t.shape for t in dev[:5]]
        bufs = self.results[slot]
        if bufs is None or any(b.shape != s_ or b.dtype != o[sl].dtype for b, s_, o in zip(bufs, shapes, outputs)):
            bufs = [torch.empty(s_, dtype=o.dtype, device=self.device) for s_, o in zip(shapes, outputs)]
            self.results[slot] = bufs
            self.copied[slot] = None
        return bufs

    def run(self, inputs, outputs):
        assert len(inputs) == 6 and len(outputs) == 6
        assert all(t.is_pinned() for t in (*inputs, *outputs)), "host tensors must be pinned"
        b = inputs[0].shape[0]
        for b0 in range(0, b, self.chunk):
            sl = slice(b0, min(b, b0 + self.chunk))
            slot = self.turn % len(self.slots)
            self.turn += 1
            parts = [t[sl] for t in inputs]
            with torch.cuda.stream(self.s_in):
                if self.free[slot] is not None:
                    self.s_in.wait_event(self.free[slot])
                dev = self._stage(slot, parts)
                if self.timed:
                    t0 = torch.cuda.Event(enable_timing=True)
                    t0.record(self.s_in)
                for d_, p_ in zip(dev, parts):
                    d_.copy_(p_, non_blocking=True)
                ready = torch.cuda.Event(enable_timing=self.timed)
                ready.record(self.s_in)
                if self.timed:
                    self._copies.append(("h2d", sum(p_.numel() * p_.element_size() for p_ in parts), t0, ready))
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(ready)
                q, k1, k2, v1, v2, dout = dev
                res = self._result_buffers(slot, dev, outputs, sl)
                if self.copied[slot] is not None:
                    self.s_run.wait_event(self.copied[slot])      # the last results of this slot are on the host
                out, lse = sa2_forward(q, k1, k2, v1, v2, self.w1, self.w2, kernel=self.kernel, out=res[0])
                grads = sa2_backward(q, k1, k2, v1, v2, out, lse, dout, self.w1, self.w2, kernel=self.kernel,
                                     grad_dtype=res[1].dtype, grads=res[1:])
                done = torch.cuda.Event()
                done.record(self.s_run)
                self.free[slot] = done
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                if self.timed:
                    t0 = torch.cuda.Event(enable_timing=True)
                    t0.record(self.s_out)
                for h_, d_ in zip(outputs, (out, *grads)):
                    h_[sl].copy_(d_, non_blocking=True)
                copied = torch.cuda.Event()
                copied.record(self.s_out)
                self.copied[slot] = copied
                if self.timed:
                    t1 = torch.cuda.Event(enable_timing=True)
                    t1.record(self.s_out)
                    self._copies.append(("d2h", sum(d_.numel() * d_.element_size() for d_ in (out, *grads)), t0, t1))

    def join(self):
        """Make the caller's current stream wait for everything queued so far."""
        end = torch.cuda.Event()
        end.record(self.s_out)
        torch.cuda.current_stream(self.device).wait_event(end)

    def synchronize(self, check=True):
        """Block the host until every queued call has delivered its results, then (``check``) raise
        ``Sa2Error`` if any kernel gave up on a bounded wait - its rows would hold NaN."""
        self.s_out.synchronize()
        if check:
            check_device()
