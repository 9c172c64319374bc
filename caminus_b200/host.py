"""The per-layer glue over HOST buffers: the call a caller without device-resident activations makes.

HostLayerGlue owns pinned host buffers for one batch of token rows and runs, per call, every row through the three glue ops
on the device: the rows are cut into chunks, each chunk's inputs are copied in on one stream, computed on a second and its
outputs copied back on a third, two chunks in flight, so the copies of one chunk overlap the kernels of another. All bytes
cross the host link in both directions on every call; device memory holds two chunks, not the batch."""
import contextlib
import os

import torch

from . import glue


@contextlib.contextmanager
def near_gpu(dev):
    """Inside the block the calling thread runs on the CPUs next to GPU `dev` (NVML's CPU affinity of the device), so that pinned
    host memory allocated there lands on that GPU's NUMA node and its copies do not cross the socket interconnect; the thread's
    previous affinity is restored afterwards. Changes nothing on the GPU; without NVML, or where the call fails, it does nothing."""
    old = None
    try:
        import pynvml as nv
        nv.nvmlInit()
        index = torch.device(dev).index or 0
        vis = os.environ.get('CUDA_VISIBLE_DEVICES')
        idx = int(vis.split(',')[index]) if vis and all(v.strip().isdigit() for v in vis.split(',')) else index
        h = nv.nvmlDeviceGetHandleByIndex(idx)
        ncpu = os.cpu_count() or 1
        words = nv.nvmlDeviceGetCpuAffinity(h, (ncpu + 63) // 64)
        cpus = {64 * w + b for w, m in enumerate(words) for b in range(64) if (int(m) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        if cpus & allowed:
            old = allowed
            os.sched_setaffinity(0, cpus & allowed)
    except Exception:
        old = None
    try:
        yield
    finally:
        if old is not None:
            try: os.sched_setaffinity(0, old)
            except Exception: pass


class HostLayerGlue:
    def __init__(self, T, hidden, nh, nkv, inter, nw, par, dev, chunk=1024, eps=1e-6, yarn=False):
        self.T, self.dev, self.chunk = int(T), torch.device(dev), int(min(chunk, T))
        self.layer = glue.LayerGlue(nw, par, eps, yarn)
        pin = lambda *s, dt=torch.float16: torch.empty(*s, dtype=dt, pin_memory=True).zero_()      # (touched where it is allocated)
        with near_gpu(self.dev):
            self.x, self.resid = pin(T, hidden), pin(T, hidden)
            self.q, self.k = pin(T, nh, 128), pin(T, nkv, 128)
            self.gate, self.up = pin(T, inter), pin(T, inter)
            self.h16 = pin(T, hidden)
            self.yq = pin(T, inter // 32 * 36, dt=torch.uint8)
        C = self.chunk
        dv = lambda *s, dt=torch.float16: torch.empty(*s, dtype=dt, device=self.dev)
        self.bufs = [dict(x=dv(C, hidden), resid=dv(C, hidden), q=dv(C, nh, 128), k=dv(C, nkv, 128), gate=dv(C, inter), up=dv(C, inter),
                          h16=dv(C, hidden), yq=dv(C * (inter // 32 * 36), dt=torch.uint8)) for _ in range(2)]
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(self.dev) for _ in range(3))
        ins = (self.x, self.resid, self.q, self.k, self.gate, self.up); outs = (self.x, self.h16, self.q, self.k, self.yq)
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in ins)
        self.d2h_bytes = sum(t.numel() * t.element_size() for t in outs)

    def fill_from(self, x, resid, q, k, gate, up):
        """the first T rows of device tensors into the pinned inputs"""
        T = self.T
        for h, d in ((self.x, x), (self.resid, resid), (self.q, q), (self.k, k), (self.gate, gate), (self.up, up)): h.copy_(d[:T])
        torch.cuda.synchronize(self.dev)

    def run(self, pos0=0):
        """one pass: x, q, k are updated in place in the host buffers; h16 and yq are written. Returns when all of it is back."""
        C, T = self.chunk, self.T
        free = [None, None]
        for i, a in enumerate(range(0, T, C)):
            b = min(T, a + C); n = b - a; B = self.bufs[i & 1]
            with torch.cuda.stream(self.s_in):
                if free[i & 1] is not None: self.s_in.wait_event(free[i & 1])
                for name in ('x', 'resid', 'q', 'k', 'gate', 'up'): B[name][:n].copy_(getattr(self, name)[a:b], non_blocking=True)
                ready = torch.cuda.Event(); ready.record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(ready)
                self.layer(B['x'][:n], B['resid'][:n], B['q'][:n], B['k'][:n], B['gate'][:n], B['up'][:n], B['h16'][:n],
                           B['yq'][:n * self.yq.shape[1]], pos0=pos0 + a)
                done = torch.cuda.Event(); done.record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                for name in ('x', 'h16', 'q', 'k'): getattr(self, name)[a:b].copy_(B[name][:n], non_blocking=True)
                self.yq[a:b].copy_(B['yq'][:n * self.yq.shape[1]].view(n, -1), non_blocking=True)
                f = torch.cuda.Event(); f.record(self.s_out); free[i & 1] = f
        self.s_out.synchronize()

    def copies_only(self):
        """the copies of one pass without its kernels: every input chunk host -> device on one stream while every output chunk goes
        device -> host on another (the bytes and buffers of run()). Returns when all of it has finished. What the host link alone
        costs for a pass: the floor under run()'s time"""
        C, T = self.chunk, self.T
        for i, a in enumerate(range(0, T, C)):
            b = min(T, a + C); n = b - a; B = self.bufs[i & 1]
            with torch.cuda.stream(self.s_in):
                for name in ('x', 'resid', 'q', 'k', 'gate', 'up'): B[name][:n].copy_(getattr(self, name)[a:b], non_blocking=True)
            with torch.cuda.stream(self.s_out):
                for name in ('x', 'h16', 'q', 'k'): getattr(self, name)[a:b].copy_(B[name][:n], non_blocking=True)
                self.yq[a:b].copy_(B['yq'][:n * self.yq.shape[1]].view(n, -1), non_blocking=True)
        self.s_in.synchronize(); self.s_out.synchronize()
