"""Forward + backward of power retention for tensors that live in (pinned) host memory.

The layer is independent across kv heads, so the heads are cut into slices and the slices are
pipelined over three streams: while slice i computes, slice i+1 is copied in and the results
of slice i-1 are copied out.  PCIe is full duplex, so the step costs about
max(copy in, copy out, compute) instead of their sum.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .retention import power_retention


def _copy2d(dst, dst_off_bytes, dst_pitch, src, src_off_bytes, src_pitch, width, rows, to_device, dev_index, stream):
    _lib.check(_lib.lib().pr_copy_2d(ctypes.c_void_p(dst.data_ptr() + dst_off_bytes), ctypes.c_longlong(dst_pitch),
                                     ctypes.c_void_p(src.data_ptr() + src_off_bytes), ctypes.c_longlong(src_pitch),
                                     ctypes.c_longlong(width), ctypes.c_longlong(rows), ctypes.c_int(to_device),
                                     ctypes.c_int(dev_index), ctypes.c_void_p(stream.cuda_stream)), "pr_copy_2d")


class HostPipeline:
    """Reusable buffers and streams for `fwd_bwd` on host tensors of one fixed shape."""

    def __init__(self, b, t, h, d, dtype, device, chunk_size, n_slices=4, gated=True, ratio=1, slices=None):
        """`slices`: kv heads per slice, in order (sum = h).  Default: n_slices equal slices.  A short first
        slice starts the compute and the copy-out stream earlier; `default_slices(h)` gives such a split."""
        if slices is None:
            assert h % n_slices == 0
            slices = [h // n_slices] * n_slices
        assert sum(slices) == h and min(slices) > 0
        self.b, self.t, self.h, self.d, self.ratio = b, t, h, d, ratio
        self.slices = list(slices)
        self.offs = [sum(self.slices[:i]) for i in range(len(self.slices))]
        self.hs = max(self.slices)
        self.n_slices, self.chunk, self.gated = len(self.slices), chunk_size, gated
        self.dev = torch.device(device)
        self.idx = self.dev.index if self.dev.index is not None else torch.cuda.current_device()
        self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(self.dev) for _ in range(3))
        # two sets of device buffers per tensor, sized for the largest slice; a slice of fewer heads uses a
        # dense [b, t, heads, d] view of the same memory
        mk = lambda hh: [torch.empty(b * t * hh * d, device=self.dev, dtype=dtype) for _ in range(2)]
        self.Q, self.dO = mk(self.hs * ratio), mk(self.hs * ratio)
        self.K, self.V = mk(self.hs), mk(self.hs)
        self.G = torch.empty(b, t, h, device=self.dev, dtype=torch.float32) if gated else None
        self.dG = torch.empty(b, t, h, device=self.dev, dtype=torch.float32) if gated else None
        self.res = [None, None]  # results of the slice in flight per parity (kept alive until copied out)
        self.ev_in = [torch.cuda.Event() for _ in range(self.n_slices)]
        self.ev_cmp = [torch.cuda.Event() for _ in range(self.n_slices)]
        self.ev_qkv = [torch.cuda.Event() for _ in range(self.n_slices)]
        self.ev_fwd = [torch.cuda.Event() for _ in range(self.n_slices)]
        self.ev_out = [torch.cuda.Event() for _ in range(self.n_slices)]

    @staticmethod
    def default_slices(h):
        """Two one-head slices first (the pipeline fills after one head has arrived), pairs after that."""
        if h < 4:
            return [1] * h
        rest = h - 2
        return [1, 1] + [2] * (rest // 2) + ([1] if rest % 2 else [])

    def fwd_bwd(self, Qh, Kh, Vh, Gh, dOh, out):
        """Qh, dOh [b,t,h*ratio,d], Kh, Vh [b,t,h,d], Gh [b,t,h] pinned host tensors; `out` = dict of
        pinned host tensors O, dQ, dK, dV (and dlog_G) that receive the results.  Returns after
        everything has been enqueued; synchronise the device (or `self.s_out`) before reading `out`."""
        b, t, h, d, r = self.b, self.t, self.h, self.d, self.ratio
        es = Qh.element_size()
        rows = b * t
        cur = torch.cuda.current_stream(self.dev)
        for s in (self.s_in, self.s_cmp, self.s_out):
            s.wait_stream(cur)
        if self.gated:
            with torch.cuda.stream(self.s_in):
                self.G.copy_(Gh, non_blocking=True)
        for i in range(self.n_slices):
            p = i & 1
            hs, off = self.slices[i], self.offs[i]
            view = lambda buf, heads: buf[:b * t * heads * d].view(b, t, heads, d)
            Qd, dOd = view(self.Q[p], hs * r), view(self.dO[p], hs * r)
            Kd, Vd = view(self.K[p], hs), view(self.V[p], hs)
            if i >= 2:  # the buffers of this parity are free once slice i-2 has been computed
                self.s_in.wait_event(self.ev_cmp[i - 2])
            # Q, K, V first: the forward starts as soon as they are in, the upstream gradient follows
            for host, devbuf, heads, hoff, full in ((Qh, Qd, hs * r, off * r, h * r), (Kh, Kd, hs, off, h),
                                                    (Vh, Vd, hs, off, h)):
                _copy2d(devbuf, 0, heads * d * es, host, hoff * d * es, full * d * es, heads * d * es, rows, 1,
                        self.idx, self.s_in)
            self.ev_qkv[i].record(self.s_in)
            _copy2d(dOd, 0, hs * r * d * es, dOh, off * r * d * es, h * r * d * es, hs * r * d * es, rows, 1, self.idx,
                    self.s_in)
            self.ev_in[i].record(self.s_in)
            self.s_cmp.wait_event(self.ev_qkv[i])
            if i >= 2:  # results of slice i-2 must have left before their tensors are dropped
                self.s_cmp.wait_event(self.ev_out[i - 2])
            with torch.cuda.stream(self.s_cmp):
                q, k, v = (x.detach().requires_grad_(True) for x in (Qd, Kd, Vd))
                g = None
                if self.gated:
                    g = self.G[:, :, off:off + hs].contiguous().requires_grad_(True)
                O = power_retention(q, k, v, g, deg=2, chunk_size=self.chunk)
            # the output leaves while the backward runs
            self.ev_fwd[i].record(self.s_cmp)
            self.s_out.wait_event(self.ev_fwd[i])
            Od = O.detach()
            _copy2d(out["O"], off * r * d * es, h * r * d * es, Od, 0, hs * r * d * es, hs * r * d * es, rows, 0,
                    self.idx, self.s_out)
            self.s_cmp.wait_event(self.ev_in[i])
            with torch.cuda.stream(self.s_cmp):
                O.backward(dOd)
                if self.gated:
                    self.dG[:, :, off:off + hs].copy_(g.grad)
                self.res[p] = (Od, q.grad, k.grad, v.grad)
            self.ev_cmp[i].record(self.s_cmp)
            self.s_out.wait_event(self.ev_cmp[i])
            for name, src, heads, hoff, full in (("dQ", self.res[p][1], hs * r, off * r, h * r),
                                                 ("dK", self.res[p][2], hs, off, h), ("dV", self.res[p][3], hs, off, h)):
                _copy2d(out[name], hoff * d * es, full * d * es, src, 0, heads * d * es, heads * d * es, rows, 0,
                        self.idx, self.s_out)
            self.ev_out[i].record(self.s_out)
        if self.gated:
            self.s_out.wait_event(self.ev_cmp[self.n_slices - 1])
            with torch.cuda.stream(self.s_out):
                out["dlog_G"].copy_(self.dG, non_blocking=True)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_cmp)
