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
    def __init__(self, wq: torch.Tensor, N: int, max_rows: int = 8, **fc_kwargs) -> None:
        self.wq, self.N = wq, int(N)
        self.fc_kwargs = fc_kwargs
        Kg, bs = wq.shape[1], wq.shape[2]
        from . import _cabi

        self.qtype, self.G = _cabi.infer_variant(bs)
        self.K = Kg * self.G
        dev = wq.device
        self._x_dev = torch.empty((1, max_rows, self.K), dtype=torch.float32, device=dev)
        self._y_dev = torch.empty((1, max_rows, self.N), dtype=torch.float32, device=dev)
        self._y_host = torch.empty((1, max_rows, self.N), dtype=torch.float32).pin_memory()
        self.max_rows = max_rows

    def __call__(self, x_host: torch.Tensor, sync: bool = True) -> torch.Tensor:
        """x_host: pinned (or pageable) fp32 [1, M, K] on the CPU -> fp32 [1, M, N] in pinned host memory."""
        M = x_host.shape[1]
        if M > self.max_rows or x_host.shape[2] != self.K:
            raise RuntimeError(f"HostFC: input {tuple(x_host.shape)} does not fit [1, <={self.max_rows}, {self.K}]")
        xd = self._x_dev[:, :M]
        xd.copy_(x_host, non_blocking=True)
        yd = self._y_dev[:, :M]
        llmops.fc_Q4A(xd, self.wq, self.N, out=yd, **self.fc_kwargs)
        yh = self._y_host[:, :M]
        yh.copy_(yd, non_blocking=True)
        if sync:
            torch.cuda.current_stream(self.wq.device).synchronize()
        return yh

    def h2d_bytes(self, M: int) -> int:
        return 4 * M * self.K

    def d2h_bytes(self, M: int) -> int:
        return 4 * M * self.N
