"""Host-buffer front end: the call a CPU-side user of the reference makes.

The reference's ``fc_Q4A`` takes and returns host memory.  ``HostFC`` keeps the
packed weight resident on the GPU (as the reference keeps it resident in RAM
after ``llmop_fc_q4a.__init__``) and, per call, copies the activations from
pinned host memory to the device, runs the FC and copies the result back to
pinned host memory."""
from __future__ import annotations

import numpy as np
import torch

from . import _cabi, llmops


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
        if self.fc_kwargs.get("workspace") is None:
            # captured graphs hold the workspace's address: own one, sized once for the largest call
            with torch.cuda.device(dev):
                need = int(_cabi.lib().q4fc_fc_workspace_bytes(max_rows, self.K, self.N, self.qtype, self.G))
            self.fc_kwargs["workspace"] = llmops.Workspace(need, dev)

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


class HostFCGroup:
    """Several independent host-buffer FCs submitted together: ``ys = group(xs)``.

    ``members`` are ``HostFC`` objects (or ``tp.HostFusedFC``), each with its own staging buffers and stream.
    One call copies every member's activations in, runs every FC and copies every result out as ONE replayed
    CUDA graph whose branches are the members' streams, so the per-call cost on the CPU is paid once for the
    whole group and copies of one member overlap kernels of another.  The graph is captured once per tuple of
    row counts.  Returns the members' pinned output buffers, valid after ``sync`` (default: waited for here)."""

    def __init__(self, members) -> None:
        self.members = list(members)
        if not self.members:
            raise RuntimeError("HostFCGroup: no members")
        dev = self.members[0].device if hasattr(self.members[0], "device") else self.members[0].stream.device
        self.device = dev
        self.stream = torch.cuda.Stream(dev)
        self._graphs: dict = {}

    def _enqueue(self, Ms) -> None:
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        seen = []
        for h, M in zip(self.members, Ms):
            if h.stream not in seen:
                h.stream.wait_event(start)
                seen.append(h.stream)
            with torch.cuda.stream(h.stream):
                h._enqueue(M)
        for st in seen:
            cur.wait_stream(st)

    def __call__(self, xs, sync: bool = True):
        if len(xs) != len(self.members):
            raise RuntimeError(f"HostFCGroup: {len(xs)} inputs for {len(self.members)} members")
        Ms = tuple(int(x.shape[1]) for x in xs)
        for h, x, M in zip(self.members, xs, Ms):
            if M > h.max_rows or x.shape[2] != h.K:
                raise RuntimeError(f"HostFCGroup: input {tuple(x.shape)} does not fit [1, <={h.max_rows}, {h.K}]")
            stage = h.x_staging(M)
            if x.data_ptr() != stage.data_ptr():
                stage.copy_(x)
        with torch.cuda.stream(self.stream):
            g = self._graphs.get(Ms)
            if g is None:
                self._enqueue(Ms)  # eager once: lazy look-ups and kernel attributes happen outside the capture
                torch.cuda.synchronize(self.device)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.stream):
                    self._enqueue(Ms)
                self._graphs[Ms] = g
            g.replay()
        if sync:
            self.stream.synchronize()
        return [h._y_host[:, :M] for h, M in zip(self.members, Ms)]


class HostFCBatch:
    """A fixed batch of independent host-buffer FCs over ONE pinned staging block each way: ``ys = batch(xs)``.

    ``members``: tuples ``(wq, N, rows)`` -- packed weights resident on the GPU, output width, rows of that call's
    input.  All inputs live in one pinned host block and one device block, all outputs likewise; the calls are
    grouped by row count into ``q4fc_fc_decode_batch`` launches, and the members of a launch lie back to back in the
    blocks.  A step is a pipeline over the launches, largest row count first: its slice of the input block goes up
    (one host-to-device copy per launch), its quantizers and its FC launch run, its slice of the output block comes
    down (one device-to-host copy per launch) -- uploads, kernels and downloads of different launches overlap, and
    the last download is the smallest.  Captured once as a CUDA graph and replayed.  ``x_staging(i)`` is the pinned
    view ``[1, rows, K]`` of input i: writing activations straight into it saves the host-side copy.  Returns the
    pinned output views ``[1, rows, N]``, valid after ``sync`` (default: waited for here)."""

    def __init__(self, members, *, graph: bool = True) -> None:
        self.members = [(wq, int(N), int(rows)) for wq, N, rows in members]
        if not self.members:
            raise RuntimeError("HostFCBatch: no members")
        dev = self.members[0][0].device
        self.device = dev
        self.stream = torch.cuda.Stream(dev)
        self.side = torch.cuda.Stream(dev)  # quantizers
        self.up = torch.cuda.Stream(dev)    # host-to-device copies
        self.down = torch.cuda.Stream(dev)  # device-to-host copies
        shapes = []
        for wq, N, rows in self.members:
            q, G = _cabi.infer_variant(wq.shape[2])
            shapes.append((rows, int(wq.shape[1]) * G, N, G))
        self._shapes = shapes
        nx = sum(r * K for r, K, _, _ in shapes)
        ny = sum(r * N for r, _, N, _ in shapes)
        self._x_host = torch.empty(nx, dtype=torch.float32).pin_memory()
        self._y_host = torch.empty(ny, dtype=torch.float32).pin_memory()
        self._x_dev = torch.empty(nx, dtype=torch.float32, device=dev)
        self._y_dev = torch.empty(ny, dtype=torch.float32, device=dev)
        # one launch per row count (sixteen calls at most): calls of one launch share the size of their code buffers
        by_rows: dict = {}
        for i, (r, _, _, _) in enumerate(shapes):
            by_rows.setdefault(r, []).append(i)
        parts = []
        for _, idx in sorted(by_rows.items(), reverse=True):
            parts += [idx[j: j + 16] for j in range(0, len(idx), 16)]
        n = len(shapes)
        self._xs_host, self._ys_host, self._xs_dev, ys_dev = [None] * n, [None] * n, [None] * n, [None] * n
        self._xq = [llmops.QuantizedActivations(1, r, K, G, False, dev) for r, K, _, G in shapes]
        self._batches = []  # (members, FCBatch, slice of the input block, slice of the output block)
        ox = oy = 0
        for part in parts:
            x0, y0 = ox, oy
            for i in part:
                r, K, N, _ = shapes[i]
                self._xs_host[i] = self._x_host[ox: ox + r * K].view(1, r, K)
                self._xs_dev[i] = self._x_dev[ox: ox + r * K].view(1, r, K)
                self._ys_host[i] = self._y_host[oy: oy + r * N].view(1, r, N)
                ys_dev[i] = self._y_dev[oy: oy + r * N].view(1, r, N)
                ox, oy = ox + r * K, oy + r * N
            fb = llmops.FCBatch([(self._xq[i], self.members[i][0], self.members[i][1], ys_dev[i]) for i in part],
                                pdl=True)
            qb = llmops.QuantizeBatch([(self._xs_dev[i], self._xq[i]) for i in part])  # the launch's quantizers as one
            self._batches.append((part, fb, slice(x0, ox), slice(y0, oy), qb))
        self.use_graph = bool(graph)
        self._graph = None

    def x_staging(self, i: int) -> torch.Tensor:
        return self._xs_host[i]

    def _enqueue(self) -> None:
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.up, self.side, self.down):
            s.wait_event(start)
        for part, fb, xs, ys, qb in self._batches:
            with torch.cuda.stream(self.up):
                self._x_dev[xs].copy_(self._x_host[xs], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(self.up)
            with torch.cuda.stream(self.side):
                self.side.wait_event(arrived)
                qb.run()
                quantized = torch.cuda.Event()
                quantized.record(self.side)
            cur.wait_event(quantized)
            fb.run()
            computed = torch.cuda.Event()
            computed.record(cur)
            with torch.cuda.stream(self.down):
                self.down.wait_event(computed)
                self._y_host[ys].copy_(self._y_dev[ys], non_blocking=True)
        for s in (self.up, self.side, self.down):  # every branch joins the step's stream again
            ev = torch.cuda.Event()
            ev.record(s)
            cur.wait_event(ev)

    def __call__(self, xs=None, sync: bool = True):
        if xs is not None:
            if len(xs) != len(self.members):
                raise RuntimeError(f"HostFCBatch: {len(xs)} inputs for {len(self.members)} members")
            for x, stage in zip(xs, self._xs_host):
                if tuple(x.shape) != tuple(stage.shape):
                    raise RuntimeError(f"HostFCBatch: input {tuple(x.shape)} where {tuple(stage.shape)} is expected")
                if x.data_ptr() != stage.data_ptr():
                    stage.copy_(x)
        with torch.cuda.stream(self.stream):
            if not self.use_graph:
                self._enqueue()
            else:
                if self._graph is None:
                    self._enqueue()  # eager once: lazy look-ups and kernel attributes happen outside the capture
                    torch.cuda.synchronize(self.device)
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=self.stream):
                        self._enqueue()
                    self._graph = g
                self._graph.replay()
        if sync:
            self.stream.synchronize()
        return self._ys_host

    def h2d_bytes(self) -> int:
        return self._x_host.numel() * 4

    def d2h_bytes(self) -> int:
        return self._y_host.numel() * 4
