"""Host-buffer front end: the call a CPU-side user of the reference makes.

The reference's ``fc_Q4A`` takes and returns host memory.  ``HostFC`` keeps the
packed weight resident on the GPU (as the reference keeps it resident in RAM
after ``llmop_fc_q4a.__init__``) and, per call, copies the activations from
pinned host memory to the device, runs the FC and copies the result back to
pinned host memory."""
from __future__ import annotations

import numpy as np
import torch

from . import llmops


class HostFC:
    """``y_host = HostFC(wq, N)(x_host)``.

    With ``graph=True`` (default) the three steps of a call -- copy in, FC kernel, copy out -- are captured
    once per row count into a CUDA graph over fixed pinned staging buffers and replayed, which takes the
    per-call cost on the CPU from several framework calls to one graph launch.  ``stream``: the stream the
    call runs on (default: a stream of its own); independent FCs on different streams overlap their copies
    and kernels.  With ``sync=False`` the caller synchronizes ``stream`` before reading the result or
    calling the same object again."""

    def __init__(self, wq: torch.Tensor, N: int, max_rows: int = 8, graph: bool = True,
                 stream: "torch.cuda.Stream | None" = None, **fc_kwargs) -> None:
        self.wq, self.N = wq, int(N)
        self.fc_kwargs = fc_kwargs
        Kg, bs = wq.shape[1], wq.shape[2]
        from . import _cabi

        self.qtype, self.G = _cabi.infer_variant(bs)
        self.K = Kg * self.G
        dev = wq.device
        self.device = dev
        self.stream = stream if stream is not None else torch.cuda.Stream(dev)
        self._x_dev = torch.empty((1, max_rows, self.K), dtype=torch.float32, device=dev)
        self._y_dev = torch.empty((1, max_rows, self.N), dtype=torch.float32, device=dev)
        self._x_host = torch.empty((1, max_rows, self.K), dtype=torch.float32).pin_memory()
        self._y_host = torch.empty((1, max_rows, self.N), dtype=torch.float32).pin_memory()
        self.max_rows = max_rows
        self.use_graph = bool(graph)
        self._graphs: dict[int, torch.cuda.CUDAGraph] = {}

    def x_staging(self, M: int) -> torch.Tensor:
        """The pinned input buffer ``[1, M, K]`` a call with ``M`` rows reads: writing the activations
        straight into it and passing it to ``__call__`` saves the host-side copy."""
        return self._x_host[:, :M]

    def _enqueue(self, M: int) -> None:
        xd, yd = self._x_dev[:, :M], self._y_dev[:, :M]
        xd.copy_(self._x_host[:, :M], non_blocking=True)
        llmops.fc_Q4A(xd, self.wq, self.N, out=yd, **self.fc_kwargs)
        self._y_host[:, :M].copy_(yd, non_blocking=True)

    def _graph(self, M: int) -> torch.cuda.CUDAGraph:
        g = self._graphs.get(M)
        if g is None:
            with torch.cuda.stream(self.stream):
                self._enqueue(M)  # eager once: kernel attributes and lazy look-ups happen outside the capture
                self.stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.stream):
                    self._enqueue(M)
            self._graphs[M] = g
        return g

    def __call__(self, x_host: torch.Tensor, sync: bool = True) -> torch.Tensor:
        """x_host: fp32 [1, M, K] on the CPU -> fp32 [1, M, N] in pinned host memory (valid once the
        stream has been synchronized, which ``sync=True`` does)."""
        M = x_host.shape[1]
        if M > self.max_rows or x_host.shape[2] != self.K:
            raise RuntimeError(f"HostFC: input {tuple(x_host.shape)} does not fit [1, <={self.max_rows}, {self.K}]")
        stage = self._x_host[:, :M]
        if x_host.data_ptr() != stage.data_ptr():
            stage.copy_(x_host)
        if self.use_graph:
            g = self._graph(M)
            with torch.cuda.stream(self.stream):
                g.replay()
        else:
            with torch.cuda.stream(self.stream):
                self._enqueue(M)
        if sync:
            self.stream.synchronize()
        return self._y_host[:, :M]

    def h2d_bytes(self, M: int) -> int:
        return 4 * M * self.K

    def d2h_bytes(self, M: int) -> int:
        return 4 * M * self.N
