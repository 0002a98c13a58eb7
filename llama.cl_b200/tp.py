"""N-split of one quantized FC over the GPUs of a node.

Every 32-column stripe ``nb`` of the packed tensor ``[Ng, Kg, BS]`` is
independent (own weights, own outputs) and the tensor is contiguous along
``Ng``, so a rank's shard is a contiguous byte slice of the reference's packed
tensor and packing shards rank by rank gives the same bytes as packing the
whole matrix.  Activations are replicated; each rank computes
``y[:, n0:n1]`` with the ordinary FC kernel and the slices are joined with one
all-gather (NCCL over NVLink on GPUs; any ``torch.distributed`` backend works,
which is how the host logic is tested on CPU).  No summation order changes, so
the joined output is bit-equal to the single-GPU output.

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
