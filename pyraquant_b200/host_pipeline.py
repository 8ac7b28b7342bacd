"""Host-buffer entry to the Linear path: pinned host rows in, pinned host rows out.

Rows are independent, so the call is a three-stage software pipeline over row chunks on three CUDA
streams -- host->device copy of chunk i+1, forward of chunk i, device->host copy of chunk i-1 -- with
two device input buffers.  PCIe is full duplex, so the steady state costs max(H2D, D2H, compute).
"""
from __future__ import annotations

from typing import Callable, List

import torch


class HostRowPipeline:
    def __init__(self, forward: Callable[[torch.Tensor], torch.Tensor], in_features: int, dtype: torch.dtype,
                 device: torch.device, chunk_rows: int = 8192):
        self.forward = forward
        self.device = device
        self.chunk_rows = int(chunk_rows)
        self.s_in = torch.cuda.Stream(device)
        self.s_run = torch.cuda.Stream(device)
        self.s_out = torch.cuda.Stream(device)
        self.xbuf = [torch.empty((self.chunk_rows, in_features), dtype=dtype, device=device) for _ in range(2)]

    def __call__(self, x_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """x_host [M,K] and out_host [M,N] are pinned CPU tensors; returns when out_host is complete."""
        self.start(x_host, out_host)
        self.finish()

    def start(self, x_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """Enqueues the whole pipeline and returns at once; several pipelines started back to back share the
        copy engines (PCIe is full duplex, so a read-heavy and a write-heavy layer overlap well)."""
        assert x_host.is_pinned() and out_host.is_pinned()
        M = x_host.shape[0]
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        ran: List[torch.cuda.Event] = []
        for i, r0 in enumerate(range(0, M, self.chunk_rows)):
            r1 = min(M, r0 + self.chunk_rows)
            buf = self.xbuf[i & 1][: r1 - r0]
            with torch.cuda.stream(self.s_in):
                if i >= 2:
                    self.s_in.wait_event(ran[i - 2])            # the forward that read this buffer is done
                buf.copy_(x_host[r0:r1], non_blocking=True)
                loaded = torch.cuda.Event(); loaded.record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(loaded)
                y = self.forward(buf)
                done = torch.cuda.Event(); done.record(self.s_run)
                ran.append(done)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                out_host[r0:r1].copy_(y, non_blocking=True)
                y.record_stream(self.s_out)

    def finish(self) -> None:
        """Blocks until every output row of the last `start` has reached host memory."""
        torch.cuda.current_stream(self.device).wait_stream(self.s_out)
        self.s_out.synchronize()
