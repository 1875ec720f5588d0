"""Stream- and graph-level runtime around a compiled forward: CUDA-graph replay for
launch-bound chains (:class:`GraphedCallable`) and row-streamed execution from pinned host
memory on three CUDA streams (:class:`HostStreamedModule`).

Every chain this package fuses is independent per row of the activation matrix (that is
also why rows can be sharded over GPUs with no collective).  When the activations start
in pinned host memory and the result is wanted back there, the batch can therefore be cut
into row chunks and the three phases — host->device copy, fused kernels, device->host
copy — run on three CUDA streams, chunk *i+1* being copied in while chunk *i* computes and
chunk *i-1* is copied out.  The reference launches on torch's current stream only
(fuseml/codegen/kernel_launcher.py:622-633 has an unused ``_get_launch_stream``); this is
the stream-level runtime the B200 build adds around the same compiled callable.

    runner = HostStreamedModule(torch.compile(model, backend=FuseMLCompiler()), rows_per_chunk=2048)
    runner.submit(x_pinned, y_pinned)      # returns at once; everything is enqueued
    runner.synchronize()                   # y_pinned is complete

``submit`` may be called again before ``synchronize``: successive batches pipeline into
each other.  Outputs may be one tensor or a tuple of tensors.  An output whose first
dimension is the batch rows is copied out chunk by chunk; any other output (a scalar metric
such as a global sum) is copied whole, which is only meaningful when the batch is one chunk.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


class GraphedCallable:
    """A fused forward captured once in a CUDA graph and replayed.

    Chains of microsecond-scale kernels are bound by the host's launch path (Python, the
    descriptor fill, the driver call); a captured graph replays the same launches with one
    driver call.  Launchers allocate their outputs through torch, which is capturable: the
    outputs live in the graph's private pool and are overwritten by every replay.

    ``fn`` is called with ``args`` (static device tensors: update them in place, then replay).
    The first calls run eagerly on a side stream (kernel attributes and symbol look-ups happen
    there, outside the capture).
    """

    def __init__(self, fn: Callable, *args: torch.Tensor, warmup: int = 3) -> None:
        self.args = args
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(1, warmup)):
                fn(*args)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.outputs = fn(*args)

    def __call__(self):
        self.graph.replay()
        return self.outputs


class HostStreamedModule:
    def __init__(self, fn: Callable, rows_per_chunk: int = 2048, n_buffers: int = 3,
                 device: torch.device | str | None = None) -> None:
        if rows_per_chunk <= 0 or n_buffers < 2:
            raise ValueError("rows_per_chunk must be positive and n_buffers at least 2")
        self.fn = fn
        self.rows_per_chunk = int(rows_per_chunk)
        self.n_buffers = int(n_buffers)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._h2d = torch.cuda.Stream(self.device)
        self._compute = torch.cuda.Stream(self.device)
        self._d2h = torch.cuda.Stream(self.device)
        self._in_bufs: list[torch.Tensor] = []
        self._in_free: list[torch.cuda.Event | None] = [None] * self.n_buffers   # compute finished reading buffer k
        self._slot = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def _buffers_for(self, x_host: torch.Tensor) -> None:
        shape = (self.rows_per_chunk, *x_host.shape[1:])
        if self._in_bufs and self._in_bufs[0].shape == shape and self._in_bufs[0].dtype == x_host.dtype:
            return
        self._in_bufs = [torch.empty(shape, dtype=x_host.dtype, device=self.device) for _ in range(self.n_buffers)]
        self._in_free = [None] * self.n_buffers

    def submit(self, x_host: torch.Tensor, out_host: torch.Tensor | Sequence[torch.Tensor]) -> None:
        """Enqueue one batch.  ``x_host`` and the output buffer(s) must be pinned host tensors."""
        if x_host.is_cuda or not x_host.is_pinned():
            raise ValueError("x_host must be a pinned host tensor")
        outs = [out_host] if isinstance(out_host, torch.Tensor) else list(out_host)
        for o in outs:
            if o.is_cuda or not o.is_pinned():
                raise ValueError("output buffers must be pinned host tensors")
        self._buffers_for(x_host)
        rows = x_host.shape[0]
        # the caller may have produced x_host / consumed out_host on the current stream
        here = torch.cuda.current_stream(self.device)
        self._h2d.wait_stream(here)
        for r0 in range(0, rows, self.rows_per_chunk):
            r1 = min(r0 + self.rows_per_chunk, rows)
            k = self._slot
            self._slot = (self._slot + 1) % self.n_buffers
            buf = self._in_bufs[k][: r1 - r0]
            with torch.cuda.stream(self._h2d):
                if self._in_free[k] is not None:
                    self._h2d.wait_event(self._in_free[k])     # previous user of this buffer is done
                buf.copy_(x_host[r0:r1], non_blocking=True)
                copied = torch.cuda.Event()
                copied.record(self._h2d)
            with torch.cuda.stream(self._compute):
                self._compute.wait_event(copied)
                with torch.no_grad():
                    res = self.fn(buf)
                done = torch.cuda.Event()
                done.record(self._compute)
                self._in_free[k] = done
            res_list = [res] if isinstance(res, torch.Tensor) else list(res)
            if len(res_list) != len(outs):
                raise ValueError(f"module returned {len(res_list)} tensors, {len(outs)} output buffers given")
            with torch.cuda.stream(self._d2h):
                self._d2h.wait_event(done)
                for t, o in zip(res_list, outs):
                    t.record_stream(self._d2h)                # allocated on the compute stream, read here
                    if t.dim() > 0 and t.shape[0] == r1 - r0 and o.dim() == t.dim() and o.shape[0] == rows:
                        o[r0:r1].copy_(t, non_blocking=True)
                    elif rows <= self.rows_per_chunk:
                        o.copy_(t.reshape(o.shape), non_blocking=True)   # a per-batch value (metric)
                    else:
                        raise ValueError("an output that does not follow the batch rows needs the batch in one chunk")
                    self.d2h_bytes += t.numel() * t.element_size()
            self.h2d_bytes += buf.numel() * buf.element_size()

    def synchronize(self) -> None:
        self._d2h.synchronize()
        self._compute.synchronize()

    def wait_on(self, stream: torch.cuda.Stream | None = None) -> None:
        """Make ``stream`` (default: the current one) wait for everything submitted so far,
        without blocking the host."""
        s = stream or torch.cuda.current_stream(self.device)
        s.wait_stream(self._d2h)
        s.wait_stream(self._compute)

    def __call__(self, x_host: torch.Tensor, out_host) -> None:
        self.submit(x_host, out_host)
        self.synchronize()
