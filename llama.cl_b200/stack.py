"""The fixed per-token FC schedule of a Llama block stack, owned and replayed as one CUDA graph.

In the reference a decode step walks ``Model.forward`` (chatllama/main.py:331-380): per layer the seven
``llmop_fc_q4a`` calls q, k, v | o | gate, up | down, and ``lm_head`` at the end -- 225 FC calls for 32 layers,
each quantizing its own input, with ``rmsnorm``, ``iadd``, ``itrans("silu")`` and ``imul`` between them.
``DecodeFCStack`` keeps that schedule resident on the GPU:

* the packed weights of every layer (the reference's own bytes),
* every intermediate buffer and the quantized-activation buffers the FCs read,
* one captured CUDA graph of the whole token, replayed per step.

Two schedules:

``glue="llama"``  the FCs with the in-scope steps between them, as the reference orders them:
    rmsnorm + quantize -> q, k, v (one launch) -> [attention] -> quantize -> o (+ residual) ->
    rmsnorm + quantize -> gate, up (one launch) -> silu(gate) * up + quantize -> down (+ residual);
    final rmsnorm + quantize -> lm_head.  Attention (ops/op_attn.hpp) is not part of the FC path: ``attention``
    is a callable ``(q, k, v, layer) -> tensor`` supplied by the caller; the default passes ``q`` through.
``glue="none"``   the 225 FCs alone, each reading the fp32 output of the one before (q, k, v and gate, up as one
    launch each): the FC-only chain that the per-token benchmark times.

``chain=True`` runs the same schedule through ``llmops.FCChain``: one persistent launch per token (per layer and
attention call when an ``attention`` callable is given) in which the weight stream does not stop between the FCs;
the norms, the residual adds and silu * up are done by that kernel where it quantizes a step's input.

There is no CPU path: every step is a call into the CUDA library.
"""
from __future__ import annotations

from typing import Callable

import torch

from . import llmops

LAYER_FCS = ("q", "k", "v", "o", "gate", "up", "down")


class DecodeFCStack:
    def __init__(self, layers: list[dict], lm_head: torch.Tensor, *, hidden: int, intermediate: int, vocab: int,
                 rows: int = 1, glue: str = "llama", norms: list[dict] | None = None,
                 final_norm: torch.Tensor | None = None, eps: float = 1e-5,
                 attention: Callable | None = None, graph: bool = True, tap: Callable | None = None,
                 chain: bool = False) -> None:
        """``layers[i]``: packed weights under the keys q, k, v, o, gate, up, down.  ``norms[i]``: fp32 weights
        ``input`` and ``post`` of layer i's two rmsnorms (glue="llama"; default ones).  ``rows``: B*M <= 8.
        ``tap(name, layer, tensor)``: called after every step of the llama schedule with the buffer it wrote (for
        tests and debugging; only without a graph, since the buffers are reused from layer to layer)."""
        if glue not in ("llama", "none"):
            raise RuntimeError(f"glue={glue!r}: expected 'llama' or 'none'")
        if not 1 <= rows <= 8:
            raise RuntimeError("DecodeFCStack serves decode steps: 1 <= rows <= 8")
        for i, l in enumerate(layers):
            for k in LAYER_FCS:
                if k not in l:
                    raise RuntimeError(f"layers[{i}] has no weight {k!r}")
        self.layers, self.lm_head = layers, lm_head
        self.H, self.I, self.V, self.rows, self.glue, self.eps = hidden, intermediate, vocab, rows, glue, float(eps)
        self.attention = attention
        self.tap = tap
        if tap is not None and graph:
            raise RuntimeError("tap needs graph=False: a replayed graph makes no Python calls")
        dev = lm_head.device
        self.device = dev
        from . import _cabi

        self.qtype, self.G = _cabi.infer_variant(lm_head.shape[2])
        H, I, V, R = hidden, intermediate, vocab, rows
        f32 = dict(dtype=torch.float32, device=dev)
        self.x = torch.zeros((1, R, H), **f32)  # the step's input: the residual stream
        self.q, self.k, self.v = (torch.empty((1, R, H), **f32) for _ in range(3))
        self.att = torch.empty((1, R, H), **f32)
        self.h1 = torch.empty((1, R, H), **f32)  # residual stream after attention
        self.h2 = torch.empty((1, R, H), **f32)  # residual stream after the MLP
        self.gate, self.up = (torch.empty((1, R, I), **f32) for _ in range(2))
        self.logits = torch.empty((1, R, V), **f32)
        if glue == "llama":
            one = torch.ones(H, **f32)
            self.norms = norms if norms is not None else [dict(input=one, post=one) for _ in layers]
            self.final_norm = final_norm if final_norm is not None else one
            QA = llmops.QuantizedActivations
            self.xq_h = QA(1, R, H, self.G, False, dev)  # normalized residual stream
            self.xq_a = QA(1, R, H, self.G, False, dev)  # attention output
            self.xq_m = QA(1, R, I, self.G, False, dev)  # silu(gate) * up
        self.stream = torch.cuda.Stream(dev)
        self._graph = None
        self.use_graph = bool(graph)
        self.launches_per_token = (8 * len(layers) + 2) if glue == "llama" else (4 * len(layers) + 1)
        self.chains = None
        if chain:
            if tap is not None:
                raise RuntimeError("tap needs chain=False: a chain makes no Python calls between its steps")
            self.chains = self._build_chains()
            self.launches_per_token = len(self.chains)

    # ------------------------------------------------------------------ the schedule as persistent launches
    def _build_chains(self) -> list:
        """The token's steps as ``FCChain`` objects: one for the whole token, or -- with an ``attention`` callable,
        which runs between q, k, v and o -- one in front of every attention call and one behind the last."""
        H, I, V = self.H, self.I, self.V
        if self.glue == "none":
            steps, h = [], self.x
            for l in self.layers:
                steps.append(dict(x=h, jobs=[(l["q"], H, self.q), (l["k"], H, self.k), (l["v"], H, self.v)]))
                steps.append(dict(x=self.q, jobs=[(l["o"], H, self.h1)]))
                steps.append(dict(x=self.h1, jobs=[(l["gate"], I, self.gate), (l["up"], I, self.up)]))
                steps.append(dict(x=self.gate, jobs=[(l["down"], H, self.h2)]))
                h = self.h2
            steps.append(dict(x=h, jobs=[(self.lm_head, V, self.logits)]))
            return [llmops.FCChain(steps)]
        chains, steps, h = [], [], self.x
        # the residual stream alternates between two buffers per half layer, so no step writes the buffer it reads
        for i, (l, nw) in enumerate(zip(self.layers, self.norms)):
            steps.append(dict(x=h, transform="rmsnorm", aux=nw["input"], eps=self.eps,
                              jobs=[(l["q"], H, self.q), (l["k"], H, self.k), (l["v"], H, self.v)]))
            a = self.q
            if self.attention is not None:
                chains.append(llmops.FCChain(steps))
                steps, a = [], self.att
            steps.append(dict(x=a, jobs=[(l["o"], H, self.h1, h)]))
            steps.append(dict(x=self.h1, transform="rmsnorm", aux=nw["post"], eps=self.eps,
                              jobs=[(l["gate"], I, self.gate), (l["up"], I, self.up)]))
            steps.append(dict(x=self.gate, transform="silu_mul", aux=self.up, jobs=[(l["down"], H, self.h2, self.h1)]))
            h = self.h2
        steps.append(dict(x=h, transform="rmsnorm", aux=self.final_norm, eps=self.eps,
                          jobs=[(self.lm_head, V, self.logits)]))
        chains.append(llmops.FCChain(steps))
        return chains

    def _enqueue_chains(self) -> None:
        if self.attention is None or self.glue == "none":
            self.chains[0].run()
            return
        for i, c in enumerate(self.chains):
            c.run()
            if i < len(self.layers):
                a = self.attention(self.q, self.k, self.v, i)
                if a.data_ptr() != self.att.data_ptr():
                    self.att.copy_(a, non_blocking=True)

    def check(self) -> None:
        """Raises if a bounded wait inside a chain launch ran out (host-synchronous)."""
        for c in self.chains or []:
            c.check()

    # ------------------------------------------------------------------ the schedule, enqueued on the current stream
    def _enqueue_llama(self) -> None:
        ops, H, I, G = llmops, self.H, self.I, self.G
        tap = self.tap if self.tap is not None else (lambda name, layer, t: None)
        h = self.x
        for i, (l, nw) in enumerate(zip(self.layers, self.norms)):
            tap("x", i, h)
            ops.rmsnorm_quantize(h, nw["input"], self.eps, G, pdl=True, out=self.xq_h)
            ops.fc_Q4A_multi(self.xq_h, [l["q"], l["k"], l["v"]], [H, H, H], outs=[self.q, self.k, self.v], pdl=True)
            tap("q", i, self.q), tap("k", i, self.k), tap("v", i, self.v)
            a = self.attention(self.q, self.k, self.v, i) if self.attention is not None else self.q
            ops.quantize_activations(a, G, pdl=True, out=self.xq_a)
            # o projection with the residual stream added in the kernel (llmops.iadd, chatllama/main.py:356)
            ops.fc_Q4A_multi(self.xq_a, [l["o"]], [H], outs=[self.h1], addends=[h], pdl=True)
            tap("h1", i, self.h1)
            ops.rmsnorm_quantize(self.h1, nw["post"], self.eps, G, pdl=True, out=self.xq_h)
            ops.fc_Q4A_multi(self.xq_h, [l["gate"], l["up"]], [I, I], outs=[self.gate, self.up], pdl=True)
            tap("gate", i, self.gate), tap("up", i, self.up)
            ops.silu_mul_quantize(self.gate, self.up, G, pdl=True, out=self.xq_m)
            ops.fc_Q4A_multi(self.xq_m, [l["down"]], [H], outs=[self.h2], addends=[self.h1], pdl=True)
            tap("h2", i, self.h2)
            h = self.h2
        ops.rmsnorm_quantize(h, self.final_norm, self.eps, G, pdl=True, out=self.xq_h)
        ops.fc_Q4A_multi(self.xq_h, [self.lm_head], [self.V], outs=[self.logits], pdl=True)

    def _enqueue_none(self) -> None:
        ops, H, I = llmops, self.H, self.I
        h = self.x
        for l in self.layers:
            ops.fc_Q4A_multi(h, [l["q"], l["k"], l["v"]], [H, H, H], outs=[self.q, self.k, self.v], pdl=True)
            ops.fc_Q4A_multi(self.q, [l["o"]], [H], outs=[self.h1], pdl=True)
            ops.fc_Q4A_multi(self.h1, [l["gate"], l["up"]], [I, I], outs=[self.gate, self.up], pdl=True)
            ops.fc_Q4A_multi(self.gate, [l["down"]], [H], outs=[self.h2], pdl=True)
            h = self.h2
        ops.fc_Q4A_multi(h, [self.lm_head], [self.V], outs=[self.logits], pdl=True)

    def enqueue(self) -> None:
        """One token's schedule on the current stream (what the graph holds)."""
        if self.chains is not None:
            self._enqueue_chains()
        else:
            (self._enqueue_llama if self.glue == "llama" else self._enqueue_none)()

    # ------------------------------------------------------------------ a step
    def forward(self, x: torch.Tensor | None = None, sync: bool = False) -> torch.Tensor:
        """``x``: fp32 ``[1, rows, hidden]`` on the device (copied into the stack's input buffer), or None to run
        on what ``self.x`` holds.  Returns ``self.logits`` ``[1, rows, vocab]`` (valid once ``self.stream`` has
        been waited for, which ``sync=True`` does)."""
        with torch.cuda.stream(self.stream):
            if x is not None:
                self.x.copy_(x, non_blocking=True)
            if not self.use_graph:
                self.enqueue()
            else:
                if self._graph is None:
                    self.enqueue()  # eager once: kernel attributes and lazy look-ups happen outside the capture
                    self.stream.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=self.stream):
                        self.enqueue()
                    self._graph = g
                self._graph.replay()
        if sync:
            self.stream.synchronize()
        return self.logits

    __call__ = forward

    def weight_bytes(self) -> int:
        return sum(w.numel() for l in self.layers for w in (l[k] for k in LAYER_FCS)) + self.lm_head.numel()


class FusedTPDecodeFCStack:
    """The FC-only per-token schedule (``DecodeFCStack(glue="none")``) with every weight split along N over the
    ranks of a process group: per layer q, k, v (one launch) | o | gate, up (one launch) | down, then lm_head, each
    FC storing its columns, stamped, into every rank's buffer over NVLink and the next FC reading them from there
    (``tp.FusedTPLinearQ4``) -- no collective call between the FCs.  One step barrier in front, one unpacking launch
    for the logits at the end; captured once as a CUDA graph and replayed.  Every rank constructs it with its shards
    of the same weights and calls ``forward`` with the same input.

    ``layers[i]``: this rank's packed shards (``tp.shard_packed`` or packed from ``tp.shard_rows``) under the keys
    q, k, v, o, gate, up, down; ``lm_head``: this rank's shard."""

    def __init__(self, arena, layers: list[dict], lm_head: torch.Tensor, *, hidden: int, intermediate: int, vocab: int,
                 rows: int = 1, graph: bool = True) -> None:
        from . import tp

        if not 1 <= rows <= 8:
            raise RuntimeError("FusedTPDecodeFCStack serves decode steps: 1 <= rows <= 8")
        self._tp = tp
        self.arena, self.device = arena, arena.device
        self.H, self.I, self.V, self.rows = hidden, intermediate, vocab, rows
        self.schedule = tp.TPSchedule(arena)
        widths = dict(q=hidden, k=hidden, v=hidden, o=hidden, gate=intermediate, up=intermediate, down=hidden)
        self.layers = [{k: tp.FusedTPLinearQ4(self.schedule, l[k], widths[k], max_rows=rows, pdl=True) for k in LAYER_FCS}
                       for l in layers]
        self.head = tp.FusedTPLinearQ4(self.schedule, lm_head, vocab, max_rows=rows, pdl=True)
        self.x = torch.zeros((1, rows, hidden), dtype=torch.float32, device=self.device)
        self.logits = torch.empty((1, rows, vocab), dtype=torch.float32, device=self.device)
        self.stream = torch.cuda.Stream(self.device)
        self.use_graph, self._graph = bool(graph), None
        self.launches_per_token = 4 * len(layers) + 3  # step barrier, 4 per layer, lm_head, unpacking

    def enqueue(self) -> None:
        """One token's schedule on the arena's current stream (what the graph holds)."""
        tp, h = self._tp, self.x
        self.schedule.step_begin()
        for f in self.layers:
            q, _, _ = tp.fused_multi([f["q"], f["k"], f["v"]], h)
            o = f["o"](q)
            g, _ = tp.fused_multi([f["gate"], f["up"]], o)
            h = f["down"](g)
        self.head(h).tensor(out=self.logits)  # the token is done when every rank holds the whole logits row

    def forward(self, x: torch.Tensor | None = None, sync: bool = False) -> torch.Tensor:
        with torch.cuda.stream(self.stream):
            if x is not None:
                self.x.copy_(x, non_blocking=True)
            if not self.use_graph:
                self.enqueue()
            else:
                if self._graph is None:
                    self.enqueue()  # eager once on every rank (the step barrier pairs up), then capture
                    self.stream.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=self.stream):
                        self.enqueue()
                    self._graph = g
                self._graph.replay()
        if sync:
            self.stream.synchronize()
        return self.logits

    __call__ = forward
