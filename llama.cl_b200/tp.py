"""N-split of one quantized FC over the GPUs of a node.

Every 32-column stripe ``nb`` of the packed tensor ``[Ng, Kg, BS]`` is
independent (own weights, own outputs) and the tensor is contiguous along
``Ng``, so a rank's shard is a contiguous byte slice of the reference's packed
tensor and packing shards rank by rank gives the same bytes as packing the
whole matrix.  Activations are replicated; each rank computes ``y[:, n0:n1]``.
Two ways to join the slices:

``TPLinearQ4``       one all-gather after the FC (NCCL over NVLink on GPUs; any ``torch.distributed`` backend
                     works, which is how the host logic is tested on CPU).
``FusedTPLinearQ4``  the FC kernel itself stores its columns, stamped with a step counter, into every rank's
                     output buffer over NVLink (``q4fc_fc_decode_tp``); consumers wait word by word for the
                     current stamp.  No collective call, no extra launch.  After a synchronization the caller
                     checks ``TPArena.check()``: a bounded wait on another rank that ran out leaves a status
                     word set and the results of that step invalid.

The reference has no multi-device code; this module has no counterpart there.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

from . import _cabi


def stripes_per_rank(Ng: int, world: int) -> int:
    """Stripes per rank (the last ranks may hold fewer, or none)."""
    return (Ng + world - 1) // world


def shard_bounds(Ng: int, world: int, rank: int) -> tuple[int, int]:
    """Half-open stripe range [nb0, nb1) owned by ``rank``."""
    c = stripes_per_rank(Ng, world)
    nb0 = min(Ng, rank * c)
    return nb0, min(Ng, nb0 + c)


def shard_packed(wq: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """The rank's contiguous slice of a full packed tensor (a view, no copy)."""
    nb0, nb1 = shard_bounds(wq.shape[0], world, rank)
    return wq[nb0:nb1]


def shard_rows(N: int, world: int, rank: int) -> tuple[int, int]:
    """Half-open range of output columns / weight rows [n0, n1) owned by ``rank``."""
    nb0, nb1 = shard_bounds((N + 31) // 32, world, rank)
    return min(N, nb0 * 32), min(N, nb1 * 32)


class TPLinearQ4:
    """One FC whose weight is split along N across the ranks of ``group``.

    ``wq_shard`` is this rank's slice ``[nb0:nb1]`` of the packed tensor.
    ``local_fc(x, wq_shard, n_local) -> y_local`` defaults to the CUDA
    ``fc_Q4A``; tests inject a CPU stand-in to exercise the sharding and
    gathering logic under the gloo backend."""

    def __init__(self, wq_shard: torch.Tensor, N: int, group=None,
                 local_fc: Callable | None = None, **fc_kwargs) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.N = int(N)
        self.Ng = (self.N + 31) // 32
        self.cols = stripes_per_rank(self.Ng, self.world) * 32  # padded columns per rank
        self.n0, self.n1 = shard_rows(self.N, self.world, self.rank)
        nb0, nb1 = shard_bounds(self.Ng, self.world, self.rank)
        if wq_shard.shape[0] != nb1 - nb0:
            raise RuntimeError(f"rank {self.rank}: shard has {wq_shard.shape[0]} stripes, expected {nb1 - nb0}")
        self.weight = wq_shard
        self.qtype, self.group_k = _cabi.infer_variant(wq_shard.shape[2])
        self.fc_kwargs = fc_kwargs
        self._default_fc = local_fc is None
        if local_fc is None:
            from . import llmops

            local_fc = llmops.fc_Q4A
        self.local_fc = local_fc
        self._bufs: dict = {}

    @classmethod
    def from_full_weight(cls, W: torch.Tensor, group=None, *, qtype="q4_1", group_k: int = 32, **kw):
        """Pack only this rank's rows of the fp32 weight ``[N, K]``."""
        from . import llmops

        world, rank = dist.get_world_size(group), dist.get_rank(group)
        n0, n1 = shard_rows(W.shape[0], world, rank)
        shard = llmops.offline_FC_quant_Q4A(W[n0:n1].contiguous(), qtype=qtype, group_k=group_k)
        return cls(shard, W.shape[0], group, **kw)

    def _buffers(self, B: int, M: int, device, dtype):
        key = (B, M, device)
        if key not in self._bufs:
            local = torch.zeros((B * M, self.cols), dtype=dtype, device=device)
            gathered = torch.empty((self.world * B * M, self.cols), dtype=dtype, device=device)
            self._bufs[key] = (local, gathered)
        return self._bufs[key]

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        """x fp32 [B, M, K] (replicated) -> y fp32 [B, M, N] (replicated)."""
        B, M, _ = x.shape
        rows = B * M
        local, gathered = self._buffers(B, M, x.device, torch.float32)
        n_local = self.n1 - self.n0
        if n_local > 0:
            if self._default_fc and n_local == self.cols:
                # the kernel writes straight into the gather source
                self.local_fc(x, self.weight, n_local, out=local.view(B, M, self.cols), **self.fc_kwargs)
            else:
                y = self.local_fc(x, self.weight, n_local, **self.fc_kwargs)
                local[:, :n_local].copy_(y.reshape(rows, n_local))
        dist.all_gather_into_tensor(gathered, local, group=self.group)  # rank-major concatenation along dim 0
        return self.assemble(gathered.view(self.world, rows, self.cols), B, M)

    def assemble(self, gathered: torch.Tensor, B: int, M: int) -> torch.Tensor:
        """[world, rows, cols] -> [B, M, N]; a pure view when rows == 1 and N == world * cols."""
        rows = B * M
        if rows == 1 and self.world * self.cols == self.N:
            return gathered.reshape(B, M, self.N)
        # chunks are in column order and padding sits only at the tail, so the
        # valid columns of the concatenation are exactly [0, N)
        y = gathered.permute(1, 0, 2).reshape(rows, self.world * self.cols)
        return y[:, : self.N].reshape(B, M, self.N).contiguous()


# --------------------------------------------------------------------------
# Fused form: the FC kernel itself delivers its columns to every rank.
# --------------------------------------------------------------------------
class _DeviceView:
    """Minimal ``__cuda_array_interface__`` carrier so that torch can view arena memory as a tensor."""

    def __init__(self, ptr: int, shape: tuple[int, ...], typestr: str) -> None:
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 3,
                                         "strides": None}


class TPArena:
    """Peer-mapped device memory with the same layout on every rank of ``group``.

    Each rank allocates ``nbytes`` through the C-ABI (``q4fc_tp_arena_create``), the 64-byte IPC handles
    travel by ``all_gather_object`` and every rank maps all the others (``q4fc_tp_arena_open``).  ``alloc``
    is a bump allocator: ranks must make the same calls in the same order, which gives symmetric offsets.
    The first 256 bytes hold the status word."""

    STATUS, HEADER = 8, 256

    def __init__(self, nbytes: int, device: torch.device, group=None) -> None:
        import ctypes as C

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if not 1 <= self.world <= 8:
            raise RuntimeError(f"TPArena: world size {self.world} outside 1..8")
        self.device = torch.device(device)
        self.nbytes = int(nbytes)
        self._top = self.HEADER
        L = _cabi.lib()
        base = C.c_void_p()
        handle = C.create_string_buffer(64)
        with torch.cuda.device(self.device):
            _cabi.check(L.q4fc_tp_arena_create(self.nbytes, C.byref(base), handle), "tp_arena_create")
        self.local = int(base.value)
        handles: list = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.bases: list[int] = []
        self._opened: list[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.bases.append(self.local)
                continue
            peer = C.c_void_p()
            with torch.cuda.device(self.device):
                _cabi.check(L.q4fc_tp_arena_open(h, C.byref(peer)), f"tp_arena_open(rank {r})")
            self.bases.append(int(peer.value))
            self._opened.append(int(peer.value))
        dist.barrier(group=group)  # every rank has mapped every arena before anyone stores into one

    # ---- layout
    def alloc(self, nbytes: int, align: int = 256) -> int:
        off = (self._top + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise RuntimeError(f"TPArena: {nbytes} bytes requested, {self.nbytes - off} left of {self.nbytes}")
        self._top = off + int(nbytes)
        return off

    def peers(self, off: int) -> list[int]:
        return [b + off for b in self.bases]

    def tensor(self, off: int, shape: tuple[int, ...], dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """This rank's arena memory at ``off`` as a tensor (no copy)."""
        typestr = {torch.float32: "<f4", torch.int32: "<i4", torch.int64: "<i8", torch.uint8: "|u1"}[dtype]
        return torch.as_tensor(_DeviceView(self.local + off, tuple(shape), typestr), device=self.device)

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def status(self) -> int:
        """The status word (synchronizes the device): non-zero after a bounded wait ran out."""
        torch.cuda.synchronize(self.device)
        return int(self.tensor(self.STATUS, (1,), torch.int32).item())

    def check(self) -> None:
        st = self.status()
        if st != 0:
            raise RuntimeError(f"TP status word = {st:#x}: a bounded wait on the other ranks ran out")

    def close(self) -> None:
        """Collective: unmap the peers' arenas, then free this one after everybody has unmapped it."""
        L = _cabi.lib()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for p in self._opened:
            L.q4fc_tp_arena_close(p)
        self._opened = []
        dist.barrier(group=self.group)
        if self.local:
            L.q4fc_tp_arena_destroy(self.local)
            self.local = 0


class TPSchedule:
    """A fixed set of fused FCs that always run together, once each per step, with its own step counter.

    Outputs are stamped with the schedule's epoch and readers wait for the current stamp, so every FC of
    the schedule must run in every step of the schedule and in no other.  Independent pieces of work
    (another model, a stand-alone FC) get their own schedule."""

    def __init__(self, arena: TPArena) -> None:
        import ctypes as C

        self.arena = arena
        off = arena.alloc(256, 256)
        self.epoch_off, self.barrier_off = off, off + 128
        self._barrier_peers = (C.c_void_p * 8)(*arena.peers(self.barrier_off))

    def step_begin(self) -> None:
        """Advance the epoch and meet the other ranks (one tiny kernel on the current stream)."""
        a = self.arena
        _cabi.check(_cabi.lib().q4fc_tp_step_begin(a.local + self.epoch_off, self._barrier_peers,
                                                   a.local + self.barrier_off, a.world, a.local + a.STATUS,
                                                   a._stream()), "tp_step_begin")


class StampedOutput:
    """What a fused FC returns: this rank's buffer of (value, epoch) words, ``[rows, ld]``, filled by all
    ranks' kernels.  Feed it to the next fused FC as it is (that kernel waits word by word), or call
    ``tensor()`` for plain fp32."""

    def __init__(self, layer: "FusedTPLinearQ4", B: int, M: int) -> None:
        self.layer, self.B, self.M = layer, B, M
        self.rows, self.N, self.ld = B * M, layer.N, layer.ldy
        self.ptr = layer.arena.local + layer.y_off

    @property
    def shape(self) -> tuple[int, int, int]:
        return (self.B, self.M, self.N)

    def tensor(self, out: torch.Tensor | None = None) -> torch.Tensor:
        """fp32 ``[B, M, N]`` on the current stream: one small kernel that waits for every word of this
        step and unpacks it.  ``out`` (contiguous) is reused when given."""
        lay, a = self.layer, self.layer.arena
        if out is None:
            out = torch.empty((self.B, self.M, self.N), dtype=torch.float32, device=a.device)
        elif out.shape != self.shape or out.dtype != torch.float32 or not out.is_contiguous():
            raise RuntimeError("StampedOutput.tensor: out must be a contiguous fp32 [B, M, N] tensor")
        _cabi.check(_cabi.lib().q4fc_tp_collect(self.ptr, self.rows, self.N, self.ld, out.data_ptr(), self.N,
                                                a.local + lay.schedule.epoch_off, a.local + a.STATUS,
                                                a._stream()), "tp_collect")
        return out


class FusedTPLinearQ4:
    """N-split FC whose kernel stores its columns into every rank's output buffer (``q4fc_fc_decode_tp``).

    A layer belongs to a ``TPSchedule`` and runs exactly once in each of its steps, after ``step_begin()``.
    ``y = layer(x)``: ``x`` is a replicated fp32 ``[B, M, K]`` tensor, or the ``StampedOutput`` of another
    layer of the same schedule -- then this layer's kernel waits for the other ranks' columns itself, word
    by word, and nothing else is launched between the two FCs.  Rows per call are limited to 8 (the decode
    kernel)."""

    def __init__(self, schedule: TPSchedule, wq_shard: torch.Tensor, N: int, *, max_rows: int = 8,
                 pdl: bool = False, nibble_signed: bool = False, prequant: bool = False) -> None:
        arena = schedule.arena
        self.schedule = schedule
        self.arena = arena
        self.world, self.rank = arena.world, arena.rank
        self.N = int(N)
        self.Ng = (self.N + 31) // 32
        self.nb0, self.nb1 = shard_bounds(self.Ng, self.world, self.rank)
        self.n0, self.n1 = shard_rows(self.N, self.world, self.rank)
        if wq_shard.shape[0] != self.nb1 - self.nb0:
            raise RuntimeError(f"rank {self.rank}: shard has {wq_shard.shape[0]} stripes, expected {self.nb1 - self.nb0}")
        self.weight = wq_shard
        self.Kg = int(wq_shard.shape[1])
        self.qtype, self.group_k = _cabi.infer_variant(wq_shard.shape[2])
        self.max_rows = int(max_rows)
        self.ldy = self.Ng * 32
        self.y_off = arena.alloc(self.max_rows * self.ldy * 8)
        self.flags = (_cabi.FLAG_PDL if pdl else 0) | (_cabi.FLAG_NIBBLE_SIGNED if nibble_signed else 0)
        # with a plain fp32 input: quantize it once in a small launch in front of the kernel (less repeated work
        # when several FCs run side by side); inputs that are another layer's output are quantized in the kernel
        self._xq = None
        if prequant:
            K = self.Kg * self.group_k
            with torch.cuda.device(arena.device):
                nbytes = int(_cabi.lib().q4fc_xq_bytes(self.max_rows, K, self.group_k))
            self._xq = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=arena.device)
        self._sites: dict = {}

    def _site(self, stamped: bool) -> "_cabi.TpSite":
        if stamped not in self._sites:
            a = self.arena
            s = _cabi.TpSite()
            s.world = self.world
            s.x_stamped = 1 if stamped else 0
            s.col_off = self.nb0 * 32
            for r in range(self.world):
                s.y_peer[r] = a.bases[r] + self.y_off
            s.epoch = a.local + self.schedule.epoch_off
            s.status = a.local + a.STATUS
            s.xq_scratch = self._xq.data_ptr() if (self._xq is not None and not stamped) else None
            self._sites[stamped] = s
        return self._sites[stamped]

    def _site_plain(self) -> "_cabi.TpSite":
        """Site for a plain fp32 input that is quantized inside the kernel (no scratch)."""
        if "plain" not in self._sites:
            src = self._site(False)
            s = _cabi.TpSite()
            s.world, s.x_stamped, s.col_off = src.world, 0, src.col_off
            for r in range(self.world):
                s.y_peer[r] = src.y_peer[r]
            s.epoch, s.status, s.xq_scratch = src.epoch, src.status, None
            self._sites["plain"] = s
        return self._sites["plain"]

    def __call__(self, x: "torch.Tensor | StampedOutput") -> StampedOutput:
        import ctypes as C

        stamped = isinstance(x, StampedOutput)
        if stamped:
            if x.layer.schedule is not self.schedule:
                raise RuntimeError("FusedTPLinearQ4: the input was produced under another schedule")
            B, M, K = x.shape
            rows, ldx, xptr = x.rows, x.ld, x.ptr
        else:
            B, M, K = x.shape
            rows = B * M
            if x.dtype != torch.float32 or x.stride(-1) != 1:
                raise RuntimeError("FusedTPLinearQ4: x must be fp32 with unit stride along K")
            x2 = x.reshape(rows, K)
            ldx, xptr = (x2.stride(0) if rows > 1 else K), x2.data_ptr()
        if rows > self.max_rows:
            raise RuntimeError(f"FusedTPLinearQ4: {rows} rows exceed max_rows={self.max_rows}")
        if (K + self.group_k - 1) // self.group_k != self.Kg:
            raise RuntimeError(f"FusedTPLinearQ4: K={K} does not match the packed tensor's {self.Kg} groups")
        _cabi.check(_cabi.lib().q4fc_fc_decode_tp(
            xptr, rows, K, ldx, self.weight.data_ptr(), self.nb1 - self.nb0, self.Kg, self.qtype, self.group_k,
            self.n1 - self.n0, self.ldy, C.byref(self._site(stamped)), self.flags, self.arena._stream()),
            "fc_decode_tp")
        return StampedOutput(self, B, M)


def _site_array(sites):
    import ctypes as C

    return (C.POINTER(_cabi.TpSite) * len(sites))(*[C.pointer(s) for s in sites])


class FusedTPBatch:
    """Up to four fused N-split FCs of one schedule as ONE launch, each on its own pre-quantized input
    (``q4fc_fc_decode_tp_batch``): the multi-GPU counterpart of ``llmops.FCBatch``.  ``layers``:
    ``FusedTPLinearQ4`` objects of the same schedule and block type; ``xqs``: one ``QuantizedActivations`` per
    layer (replicated on every rank).  The argument block is built once; ``run()`` only launches and returns the
    layers' ``StampedOutput``s."""

    def __init__(self, layers, xqs) -> None:
        if not 1 <= len(layers) <= 4 or len(xqs) != len(layers):
            raise RuntimeError("FusedTPBatch: one to four layers, with one quantized input each")
        self.layers, self.xqs = list(layers), list(xqs)
        sched = layers[0].schedule
        self._calls = (_cabi.TpCall * len(layers))()
        self._sites = []
        for i, (l, xq) in enumerate(zip(layers, xqs)):
            if l.schedule is not sched or (l.qtype, l.group_k) != (layers[0].qtype, layers[0].group_k):
                raise RuntimeError("FusedTPBatch: the layers differ in schedule or block type")
            if xq.group_k != l.group_k or xq.Kg != l.Kg or xq.rows > l.max_rows:
                raise RuntimeError(f"FusedTPBatch: input {i} does not fit its layer")
            c = self._calls[i]
            c.x, c.xq, c.rows, c.K, c.ldx = None, xq.buf.data_ptr(), xq.rows, xq.K, xq.K
            c.wq, c.Ng, c.Kg, c.N, c.ldy = l.weight.data_ptr(), l.nb1 - l.nb0, l.Kg, l.n1 - l.n0, l.ldy
            s = _cabi.TpSite()
            a = l.arena
            s.world, s.x_stamped, s.col_off = l.world, 0, l.nb0 * 32
            for r in range(l.world):
                s.y_peer[r] = a.bases[r] + l.y_off
            s.epoch, s.status, s.xq_scratch = a.local + sched.epoch_off, a.local + a.STATUS, None
            self._sites.append(s)
        self._site_ptrs = _site_array(self._sites)
        self.flags = layers[0].flags
        self.outs = [StampedOutput(l, xq.B, xq.M) for l, xq in zip(layers, xqs)]

    def run(self):
        l0 = self.layers[0]
        _cabi.check(_cabi.lib().q4fc_fc_decode_tp_batch(self._calls, self._site_ptrs, len(self.layers), l0.qtype,
                                                        l0.group_k, self.flags, l0.arena._stream()),
                    "fc_decode_tp_batch")
        return self.outs


def fused_multi(layers, x):
    """Several fused N-split FCs on ONE input as one launch (q/k/v, gate/up): ``x`` is a replicated fp32
    ``[B, M, K]`` tensor or the ``StampedOutput`` of another layer of the same schedule."""
    if not 1 <= len(layers) <= 4:
        raise RuntimeError("fused_multi: one to four layers")
    l0 = layers[0]
    stamped = isinstance(x, StampedOutput)
    if stamped:
        B, M, K = x.shape
        rows, ldx, xptr = x.rows, x.ld, x.ptr
    else:
        B, M, K = x.shape
        rows = B * M
        x2 = x.reshape(rows, K)
        ldx, xptr = (x2.stride(0) if rows > 1 else K), x2.data_ptr()
    calls = (_cabi.TpCall * len(layers))()
    sites = []
    for i, l in enumerate(layers):
        if l.schedule is not l0.schedule or (l.qtype, l.group_k, l.Kg) != (l0.qtype, l0.group_k, l0.Kg):
            raise RuntimeError("fused_multi: the layers differ in schedule, block type or K")
        c = calls[i]
        c.x, c.xq, c.rows, c.K, c.ldx = xptr, None, rows, K, ldx
        c.wq, c.Ng, c.Kg, c.N, c.ldy = l.weight.data_ptr(), l.nb1 - l.nb0, l.Kg, l.n1 - l.n0, l.ldy
        s = l._site(stamped)
        if not stamped and s.xq_scratch:
            s = l._site_plain()
        sites.append(s)
    _cabi.check(_cabi.lib().q4fc_fc_decode_tp_batch(calls, _site_array(sites), len(layers), l0.qtype, l0.group_k,
                                                    l0.flags, l0.arena._stream()), "fc_decode_tp_batch")
    return [StampedOutput(l, B, M) for l in layers]


def collect_many(outs, dsts=None) -> None:
    """``StampedOutput.tensor`` for up to 16 outputs of one schedule in ONE launch (``q4fc_tp_collect_multi``).
    ``dsts[i]``: contiguous fp32 ``[B, M, N]`` tensor, or None to only wait until output i is complete."""
    import ctypes as C

    n = len(outs)
    if not 1 <= n <= 16:
        raise RuntimeError("collect_many: one to sixteen outputs")
    a = outs[0].layer.arena
    sched = outs[0].layer.schedule
    i64 = C.c_int64
    src = (C.c_void_p * n)(*[o.ptr for o in outs])
    rows = (i64 * n)(*[o.rows for o in outs])
    N = (i64 * n)(*[o.N for o in outs])
    ld = (i64 * n)(*[o.ld for o in outs])
    dst = (C.c_void_p * n)(*[(d.data_ptr() if d is not None else None) for d in (dsts or [None] * n)])
    ldd = (i64 * n)(*[o.N for o in outs])
    for o, d in zip(outs, dsts or []):
        if o.layer.schedule is not sched:
            raise RuntimeError("collect_many: the outputs belong to different schedules")
        if d is not None and (d.shape != o.shape or d.dtype != torch.float32 or not d.is_contiguous()):
            raise RuntimeError("collect_many: every dst must be a contiguous fp32 [B, M, N] tensor")
    _cabi.check(_cabi.lib().q4fc_tp_collect_multi(src, rows, N, ld, dst, ldd, n, a.local + sched.epoch_off,
                                                  a.local + a.STATUS, a._stream()), "tp_collect_multi")


class HostFusedFC:
    """Host buffers in, host buffers out, over an N-split FC (the multi-GPU counterpart of ``host.HostFC``).

    Every rank makes the same call with the same activations.  Per call: copy in from pinned host memory,
    step barrier, the fused FC, unpacking of the gathered output, copy out to pinned host memory -- captured
    once per row count into a CUDA graph and replayed.  The FC is a schedule of its own, so calls need no
    coordination with other layers; ``stream`` defaults to a stream of its own."""

    def __init__(self, arena: TPArena, wq_shard: torch.Tensor, N: int, max_rows: int = 8, graph: bool = True,
                 stream: "torch.cuda.Stream | None" = None, **layer_kwargs) -> None:
        self.schedule = TPSchedule(arena)
        self.layer = FusedTPLinearQ4(self.schedule, wq_shard, N, max_rows=max_rows, **layer_kwargs)
        dev = arena.device
        self.device = dev
        self.N, self.K, self.max_rows = int(N), self.layer.Kg * self.layer.group_k, int(max_rows)
        self.stream = stream if stream is not None else torch.cuda.Stream(dev)
        self._x_dev = torch.empty((1, max_rows, self.K), dtype=torch.float32, device=dev)
        self._y_dev = torch.empty((1, max_rows, self.N), dtype=torch.float32, device=dev)
        self._x_host = torch.empty((1, max_rows, self.K), dtype=torch.float32).pin_memory()
        self._y_host = torch.empty((1, max_rows, self.N), dtype=torch.float32).pin_memory()
        self.use_graph = bool(graph)
        self._graphs: dict[int, torch.cuda.CUDAGraph] = {}

    def x_staging(self, M: int) -> torch.Tensor:
        return self._x_host[:, :M]

    def _enqueue(self, M: int) -> None:
        xd = self._x_dev[:, :M]
        xd.copy_(self._x_host[:, :M], non_blocking=True)
        self.schedule.step_begin()
        yd = self.layer(xd).tensor(out=self._y_dev[:, :M])  # the leading dimension is 1: a contiguous slice
        self._y_host[:, :M].copy_(yd, non_blocking=True)

    def __call__(self, x_host: torch.Tensor, sync: bool = True) -> torch.Tensor:
        M = x_host.shape[1]
        if M > self.max_rows or x_host.shape[2] != self.K:
            raise RuntimeError(f"HostFusedFC: input {tuple(x_host.shape)} does not fit [1, <={self.max_rows}, {self.K}]")
        stage = self._x_host[:, :M]
        if x_host.data_ptr() != stage.data_ptr():
            stage.copy_(x_host)
        with torch.cuda.stream(self.stream):
            if self.use_graph:
                g = self._graphs.get(M)
                if g is None:
                    # eager once (every rank does: the step barrier pairs up), then capture
                    self._enqueue(M)
                    self.stream.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=self.stream):
                        self._enqueue(M)
                    self._graphs[M] = g
                g.replay()
            else:
                self._enqueue(M)
        if sync:
            self.stream.synchronize()
            self.layer.arena.check()  # a bounded wait on another rank that ran out makes the result invalid
        return self._y_host[:, :M]


class HostFusedBatch:
    """``host.HostFCBatch`` over N-split weights: a fixed batch of independent host-buffer FCs over one pinned block
    each way.  Every rank makes the same call with the same activations.  ``members``: ``(wq_shard, N, rows)``.
    The members are grouped by row count into ``q4fc_fc_decode_tp_batch`` launches of up to four, largest row count
    first; a step is the step barrier and then a pipeline over those launches: the launch's slice of the input block
    goes up, its quantizers and the N-split launch run, one unpacking launch waits for the other ranks' columns of
    its outputs, its slice of the output block comes down -- copies and kernels of different launches overlap.
    Captured once as a CUDA graph and replayed."""

    def __init__(self, arena: TPArena, members, *, graph: bool = True) -> None:
        from . import llmops

        self.arena = arena
        self.schedule = TPSchedule(arena)
        self.members = [(wq, int(N), int(rows)) for wq, N, rows in members]
        dev = arena.device
        self.device = dev
        self.stream = torch.cuda.Stream(dev)
        self.side = torch.cuda.Stream(dev)  # quantizers
        self.up = torch.cuda.Stream(dev)    # host-to-device copies
        self.down = torch.cuda.Stream(dev)  # device-to-host copies
        self.layers = [FusedTPLinearQ4(self.schedule, wq, N, max_rows=rows, pdl=True) for wq, N, rows in self.members]
        shapes = [(rows, l.Kg * l.group_k, N, l.group_k) for (wq, N, rows), l in zip(self.members, self.layers)]
        self._shapes = shapes
        nx = sum(r * K for r, K, _, _ in shapes)
        ny = sum(r * N for r, _, N, _ in shapes)
        self._x_host = torch.empty(nx, dtype=torch.float32).pin_memory()
        self._y_host = torch.empty(ny, dtype=torch.float32).pin_memory()
        self._x_dev = torch.empty(nx, dtype=torch.float32, device=dev)
        self._y_dev = torch.empty(ny, dtype=torch.float32, device=dev)
        by_rows: dict = {}
        for i, (r, _, _, _) in enumerate(shapes):
            by_rows.setdefault(r, []).append(i)
        parts = []
        for _, idx in sorted(by_rows.items(), reverse=True):
            parts += [idx[j: j + 4] for j in range(0, len(idx), 4)]
        n = len(shapes)
        self._xs_host, self._ys_host, self._xs_dev, self._ys_dev = [None] * n, [None] * n, [None] * n, [None] * n
        self._xq = [llmops.QuantizedActivations(1, r, K, G, False, dev) for r, K, _, G in shapes]
        self._batches = []  # (members, FusedTPBatch, slice of the input block, slice of the output block)
        ox = oy = 0
        for part in parts:
            x0, y0 = ox, oy
            for i in part:
                r, K, N, _ = shapes[i]
                self._xs_host[i] = self._x_host[ox: ox + r * K].view(1, r, K)
                self._xs_dev[i] = self._x_dev[ox: ox + r * K].view(1, r, K)
                self._ys_host[i] = self._y_host[oy: oy + r * N].view(1, r, N)
                self._ys_dev[i] = self._y_dev[oy: oy + r * N].view(1, r, N)
                ox, oy = ox + r * K, oy + r * N
            fb = FusedTPBatch([self.layers[i] for i in part], [self._xq[i] for i in part])
            qb = llmops.QuantizeBatch([(self._xs_dev[i], self._xq[i]) for i in part])  # the launch's quantizers as one
            self._batches.append((part, fb, slice(x0, ox), slice(y0, oy), qb))
        self.use_graph = bool(graph)
        self._graph = None

    def x_staging(self, i: int) -> torch.Tensor:
        return self._xs_host[i]

    def _enqueue(self) -> None:
        from . import llmops

        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.up, self.side, self.down):
            s.wait_event(start)
        self.schedule.step_begin()
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
            collect_many(fb.run(), [self._ys_dev[i] for i in part])
            computed = torch.cuda.Event()
            computed.record(cur)
            with torch.cuda.stream(self.down):
                self.down.wait_event(computed)
                self._y_host[ys].copy_(self._y_dev[ys], non_blocking=True)
        for s in (self.up, self.side, self.down):  # every branch joins the step's stream again
            ev = torch.cuda.Event()
            ev.record(s)
            cur.wait_event(ev)

    def __call__(self, xs=None, sync: bool = True, check: bool = True):
        """``check`` (with ``sync``): read the status word after the step and raise if a bounded wait on another
        rank ran out; a caller that checks ``arena.check()`` itself at a coarser grain passes False."""
        if xs is not None:
            for x, stage in zip(xs, self._xs_host):
                if x.data_ptr() != stage.data_ptr():
                    stage.copy_(x)
        with torch.cuda.stream(self.stream):
            if not self.use_graph:
                self._enqueue()
            else:
                if self._graph is None:
                    self._enqueue()  # eager once (every rank does: the step barrier pairs up), then capture
                    torch.cuda.synchronize(self.device)
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=self.stream):
                        self._enqueue()
                    self._graph = g
                self._graph.replay()
        if sync:
            self.stream.synchronize()
            if check:
                self.arena.check()  # a bounded wait on another rank that ran out makes the results invalid
        return self._ys_host

    def h2d_bytes(self) -> int:
        return self._x_host.numel() * 4

    def d2h_bytes(self) -> int:
        return self._y_host.numel() * 4
