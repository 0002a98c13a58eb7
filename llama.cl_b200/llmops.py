"""GPU drop-in for the FC ops of the reference's ``llmops`` module.

Same names, positional arguments and result shapes as the pybind11 functions
registered in ``ops/main.cpp:158-160`` of usstq/llama.cl, on torch CUDA
tensors instead of ``llmops.tensor``:

    offline_FC_quant_Q4A(wei)                  ops/op_fc.hpp:151
    offline_FC_dequant_Q4A(weiq)               ops/op_fc.hpp:124
    fc_Q4A(input, wei_quantized, N)            ops/op_fc.hpp:286

The reference fixes the block type at compile time (``ops/op_fc.hpp:109``);
here it is the keyword ``qtype`` / ``group_k`` of the packer (defaults: the
reference's stock ``q4_1`` / 32) and is recovered from the packed tensor's
last dimension everywhere else.  Errors surface as ``RuntimeError`` like the
reference's ``ASSERT`` (``ops/tensor.hpp:20-36``).  Everything runs on the
CUDA library; there is no CPU path.
"""
from __future__ import annotations

import torch

from . import _cabi
from ._cabi import FLAG_NIBBLE_SIGNED, FLAG_PDL, FLAG_STREAMK, Q4_0, Q4_1

__all__ = ["offline_FC_quant_Q4A", "offline_FC_dequant_Q4A", "fc_Q4A", "FC_dynamic_quantize_x",
           "fc_workspace", "Workspace", "fc_Q4A_multi", "FCBatch", "fc_Q4A_q8", "quantize_activations", "rmsnorm_quantize", "silu_mul_quantize",
           "QuantizedActivations", "QuantizeBatch", "FCChain", "FC_quant_Q8C", "FC_evaluate_Q8C", "embedding_q8c_quant_w", "embedding_q8c", "check_device_status"]


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: torch.Tensor, name: str, dtype: torch.dtype, rank: int) -> None:
    if not isinstance(t, torch.Tensor):
        raise RuntimeError(f"{name}: expected a torch.Tensor, got {type(t).__name__}")
    if t.dtype != dtype or t.dim() != rank:
        # mirrors ASSERT(x.is<T>(rank)) of the reference
        raise RuntimeError(f"assert {name}.is<{str(dtype).replace('torch.', '')}>({rank}) failed: "
                           f"got dtype {t.dtype}, rank {t.dim()}")
    if not t.is_cuda:
        raise RuntimeError(f"{name}: tensor must live on a CUDA device (there is no CPU path)")
    if not t.is_contiguous():
        raise RuntimeError(f"{name}: tensor must be dense row-major (contiguous)")


class Workspace:
    """Scratch for the FC kernels: status word, stripe counters, CTA partials.

    Zeroed once at creation; the kernels leave it clean.  One workspace serves
    any number of calls that are ordered on one stream."""

    def __init__(self, nbytes: int, device: torch.device) -> None:
        self.buf = torch.zeros(max(int(nbytes), 4096), dtype=torch.uint8, device=device)
        self.nbytes = self.buf.numel()

    @property
    def ptr(self) -> int:
        return self.buf.data_ptr()

    def check(self) -> None:
        """Host-synchronous read of the device status word."""
        with torch.cuda.device(self.buf.device):
            _cabi.check(_cabi.lib().q4fc_fc_check_status(self.ptr, _stream_ptr(self.buf.device)), "fc status")


_workspaces: dict = {}
_retired: list = []  # replaced workspaces stay allocated: CUDA graphs captured earlier hold their raw pointers


def fc_workspace(rows: int, K: int, N: int, qtype: int, group_k: int, device: torch.device) -> Workspace:
    """Cached workspace for (device, current stream), grown on demand.

    A decode call is sized for 8 rows whatever it asks for, so that the row count of later calls on the stream
    does not replace the workspace; when a larger one is needed all the same, the old one is kept alive (never
    freed), because graphs captured with it would otherwise replay into freed memory.  Objects that capture
    graphs (``host.HostFC`` and friends) own a workspace sized for their largest call instead of using this
    cache."""
    with torch.cuda.device(device):
        need = int(_cabi.lib().q4fc_fc_workspace_bytes(max(rows, 8) if rows <= 8 else rows, K, N, qtype, group_k))
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.nbytes < need:
        if ws is not None:
            _retired.append(ws)
        ws = Workspace(need, device)
        _workspaces[key] = ws
    return ws


def offline_FC_quant_Q4A(wei: torch.Tensor, *, qtype="q4_1", group_k: int = 32,
                         out: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 ``[N, K]`` -> int8 ``[ceil(N/32), ceil(K/group_k), block_bytes]`` (ops/op_fc.hpp:151-219)."""
    q = _cabi.parse_qtype(qtype)
    _require_cuda(wei, "wei", torch.float32, 2)
    N, K = wei.shape
    bs = _cabi.lib().q4fc_block_bytes(q, group_k)
    if bs < 0:
        raise RuntimeError(f"unsupported block type: qtype={qtype!r}, group_k={group_k}")
    Ng, Kg = (N + 31) // 32, (K + group_k - 1) // group_k
    if out is None:
        out = torch.empty((Ng, Kg, bs), dtype=torch.int8, device=wei.device)
    else:
        _require_cuda(out, "out", torch.int8, 3)
        if tuple(out.shape) != (Ng, Kg, bs):
            raise RuntimeError(f"out: expected shape {(Ng, Kg, bs)}, got {tuple(out.shape)}")
    with torch.cuda.device(wei.device):
        _cabi.check(_cabi.lib().q4fc_pack(wei.data_ptr(), N, K, q, group_k, out.data_ptr(), _stream_ptr(wei.device)),
                    "offline_FC_quant_Q4A")
    return out


def offline_FC_dequant_Q4A(weiq: torch.Tensor, *, nibble_signed: bool = False) -> torch.Tensor:
    """packed -> fp32 ``[Ng*32, Kg*group_k]`` (ops/op_fc.hpp:124-149).

    ``nibble_signed=False`` reads the nibble unsigned for Q4_0 too, as the
    reference does (ops/op_fc.hpp:95-106)."""
    _require_cuda(weiq, "weiq", torch.int8, 3)
    Ng, Kg, bs = weiq.shape
    q, G = _cabi.infer_variant(bs)
    out = torch.empty((Ng * 32, Kg * G), dtype=torch.float32, device=weiq.device)
    with torch.cuda.device(weiq.device):
        _cabi.check(_cabi.lib().q4fc_dequant(weiq.data_ptr(), Ng, Kg, q, G, int(nibble_signed), out.data_ptr(),
                                             _stream_ptr(weiq.device)), "offline_FC_dequant_Q4A")
    return out


def FC_dynamic_quantize_x(input: torch.Tensor, group_k: int, scale: float = 1.0):
    """Q8 activation quantizer (ops/op_fc.hpp:221-272; not exported to Python by the reference).

    fp32 ``[..., K]`` -> (codes int8 ``[..., Kg*group_k]``, scales fp32 ``[..., Kg]``, group sums fp32 ``[..., Kg]``)."""
    if not isinstance(input, torch.Tensor) or input.dtype != torch.float32 or input.dim() < 1:
        raise RuntimeError("input: expected an fp32 tensor of rank >= 1")
    if not input.is_cuda or not input.is_contiguous():
        raise RuntimeError("input: must be a contiguous CUDA tensor")
    K = input.shape[-1]
    rows = input.numel() // K if K else 0
    Kg = (K + group_k - 1) // group_k
    lead = tuple(input.shape[:-1])
    codes = torch.empty(lead + (Kg * group_k,), dtype=torch.int8, device=input.device)
    scales = torch.empty(lead + (Kg,), dtype=torch.float32, device=input.device)
    gsums = torch.empty(lead + (Kg,), dtype=torch.float32, device=input.device)
    with torch.cuda.device(input.device):
        _cabi.check(_cabi.lib().q4fc_quant_x(input.data_ptr(), rows, K, K, group_k, float(scale), codes.data_ptr(),
                                             scales.data_ptr(), gsums.data_ptr(), _stream_ptr(input.device)),
                    "FC_dynamic_quantize_x")
    return codes, scales, gsums


def fc_Q4A(input: torch.Tensor, wei_quantized: torch.Tensor, N: int, *, nibble_signed: bool = False,
           out: torch.Tensor | None = None, workspace: Workspace | None = None, pdl: bool = False,
           path: str = "auto", prequant: bool = False, addend: torch.Tensor | None = None) -> torch.Tensor:
    """``y[b, m, :N] = quantized(input[b, m]) . W`` (ops/op_fc.hpp:286-426).

    input fp32 ``[B, M, K]``, wei_quantized int8 ``[Ng, Kg, block_bytes]`` ->
    fp32 ``[B, M, N]``.  ``path``: "auto" (decode kernel for B*M <= 8, else
    the prefill kernel), "decode", "streamk" (the decode kernel that reduces
    through the workspace) or "prefill".  ``prequant=True`` (decode kernel): quantize the activations in a
    small launch of their own whatever the size -- less total work when several FCs run side by side on
    different streams; by default that happens only for large rows x K.  ``addend`` (decode kernel, B*M <= 8):
    fp32 ``[N]`` (a bias) or ``[B, M, N]`` (a residual; may be ``out``), added to the result inside the kernel
    with one fp32 add per output, as the reference's ``llmops.iadd`` after the FC does."""
    _require_cuda(input, "input", torch.float32, 3)
    _require_cuda(wei_quantized, "wei_quantized", torch.int8, 3)
    if wei_quantized.device != input.device:
        raise RuntimeError("input and wei_quantized live on different devices")
    B, M, K = input.shape
    Ng, Kg, bs = wei_quantized.shape
    q, G = _cabi.infer_variant(bs)
    N = int(N)
    rows = B * M
    if out is None:
        out = torch.empty((B, M, N), dtype=torch.float32, device=input.device)
    else:
        _require_cuda(out, "out", torch.float32, 3)
        if tuple(out.shape) != (B, M, N):
            raise RuntimeError(f"out: expected shape {(B, M, N)}, got {tuple(out.shape)}")
    if workspace is None:
        workspace = fc_workspace(rows, K, N, q, G, input.device)
    flags = (FLAG_NIBBLE_SIGNED if nibble_signed else 0) | (FLAG_PDL if pdl else 0)
    if path == "streamk":
        flags |= FLAG_STREAMK
    if prequant:
        flags |= _cabi.FLAG_PREQUANT
    L = _cabi.lib()
    if addend is not None:
        _require_cuda(addend, "addend", torch.float32, addend.dim())
        if rows > 8 or path in ("streamk", "prefill"):
            raise RuntimeError("addend is folded into the decode kernel only (B*M <= 8, path auto or decode)")
        if tuple(addend.shape) == (N,):
            ld_add = 0
        elif tuple(addend.shape) == (B, M, N) and addend.is_contiguous():
            ld_add = N
        else:
            raise RuntimeError(f"addend: expected contiguous shape {(N,)} or {(B, M, N)}, got {tuple(addend.shape)}")
        with torch.cuda.device(input.device):
            _cabi.check(L.q4fc_fc_decode_add(input.data_ptr(), rows, K, K, wei_quantized.data_ptr(), Ng, Kg, q, G, N,
                                             out.data_ptr(), N, addend.data_ptr(), ld_add, workspace.ptr,
                                             workspace.nbytes, flags, _stream_ptr(input.device)), "fc_Q4A")
        return out
    fn = {"auto": L.q4fc_fc, "decode": L.q4fc_fc_decode, "streamk": L.q4fc_fc_decode,
          "prefill": L.q4fc_fc_prefill}[path]
    with torch.cuda.device(input.device):
        _cabi.check(fn(input.data_ptr(), rows, K, K, wei_quantized.data_ptr(), Ng, Kg, q, G, N, out.data_ptr(), N,
                       workspace.ptr, workspace.nbytes, flags, _stream_ptr(input.device)), "fc_Q4A")
    return out


class QuantizedActivations:
    """Activations quantized once for several FCs (``q4fc_xq_*`` format): int8 codes ``[rows][Kg*G]`` followed
    by ``[Kg][16]`` scales / group sums, in one device buffer.  Made by ``quantize_activations`` or
    ``rmsnorm_quantize``, consumed by ``fc_Q4A_q8``."""

    def __init__(self, B: int, M: int, K: int, group_k: int, signed: bool, device: torch.device) -> None:
        self.B, self.M, self.K, self.group_k, self.signed = B, M, K, group_k, signed
        self.rows = B * M
        with torch.cuda.device(device):
            nbytes = int(_cabi.lib().q4fc_xq_bytes(self.rows, K, group_k))
        if nbytes == 0 and self.rows > 0:
            raise RuntimeError(f"unsupported group_k={group_k}")
        self.buf = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)

    @property
    def Kg(self) -> int:
        return (self.K + self.group_k - 1) // self.group_k

    def codes(self) -> torch.Tensor:
        """int8 ``[rows, Kg*G]`` view of the codes."""
        n = self.rows * self.Kg * self.group_k
        return self.buf[:n].view(torch.int8).view(self.rows, self.Kg * self.group_k)

    def scales_and_sums(self) -> tuple[torch.Tensor, torch.Tensor]:
        """fp32 ``[rows, Kg]`` scales and group sums (views into the ``[Kg][16]`` block)."""
        off = (self.rows * self.Kg * self.group_k + 255) // 256 * 256
        sc = self.buf[off: off + self.Kg * 64].view(torch.float32).view(self.Kg, 8, 2)
        return sc[:, : self.rows, 0].t(), sc[:, : self.rows, 1].t()


def _check_rows(rows: int) -> None:
    if rows > 8:
        raise RuntimeError(f"pre-quantized activations serve the decode kernel: B*M = {rows} exceeds 8")


def quantize_activations(input: torch.Tensor, group_k: int, *, nibble_signed: bool = False, pdl: bool = False,
                         out: QuantizedActivations | None = None) -> QuantizedActivations:
    """FC_dynamic_quantize_x (ops/op_fc.hpp:221-272) once, for every FC that reads ``input`` ``[B, M, K]``."""
    _require_cuda(input, "input", torch.float32, 3)
    B, M, K = input.shape
    _check_rows(B * M)
    xq = out if out is not None else QuantizedActivations(B, M, K, group_k, nibble_signed, input.device)
    with torch.cuda.device(input.device):
        _cabi.check(_cabi.lib().q4fc_quant_x_q8(input.data_ptr(), B * M, K, K, group_k, int(nibble_signed),
                                                xq.buf.data_ptr(), FLAG_PDL if pdl else 0,
                                                _stream_ptr(input.device)), "quantize_activations")
    return xq


class QuantizeBatch:
    """``quantize_activations`` for up to 16 (input, output) pairs as ONE launch (``q4fc_quant_x_q8_batch``).  The
    argument block is built once; ``run()`` only launches (capturable in a CUDA graph)."""

    def __init__(self, pairs, *, pdl: bool = False) -> None:
        if not 1 <= len(pairs) <= 16:
            raise RuntimeError("QuantizeBatch: one to sixteen inputs")
        self.n = len(pairs)
        self._args = (_cabi.XqCall * self.n)()
        self._keep = list(pairs)
        G = signed = None
        for i, (x, xq) in enumerate(pairs):
            _require_cuda(x, f"pairs[{i}] input", torch.float32, 3)
            if not isinstance(xq, QuantizedActivations) or (xq.B, xq.M, xq.K) != tuple(x.shape):
                raise RuntimeError(f"pairs[{i}]: the QuantizedActivations do not fit the input {tuple(x.shape)}")
            if G is None:
                G, signed, self.device = xq.group_k, xq.signed, x.device
            elif (xq.group_k, xq.signed) != (G, signed):
                raise RuntimeError("QuantizeBatch: the outputs differ in group size or signedness")
            a = self._args[i]
            a.x, a.rows, a.K, a.ldx, a.xq = x.data_ptr(), xq.rows, xq.K, xq.K, xq.buf.data_ptr()
        self.group_k, self.signed, self.flags = G, signed, (FLAG_PDL if pdl else 0)

    def run(self) -> None:
        with torch.cuda.device(self.device):
            _cabi.check(_cabi.lib().q4fc_quant_x_q8_batch(self._args, self.n, self.group_k, int(self.signed), self.flags,
                                                          _stream_ptr(self.device)), "quant_x_q8_batch")


def rmsnorm_quantize(input: torch.Tensor, weight: torch.Tensor, eps: float, group_k: int, *,
                     normalized: torch.Tensor | None = None, residual: torch.Tensor | None = None,
                     sum_out: torch.Tensor | None = None, nibble_signed: bool = False, pdl: bool = False,
                     out: QuantizedActivations | None = None) -> QuantizedActivations:
    """``llmops.rmsnorm`` (ops/op_misc.hpp:142-181) and the quantizer of the FCs behind it in one kernel.

    ``input`` fp32 ``[B, M, K]`` is left untouched (the reference normalizes a clone in place,
    chatllama/main.py:345-346); ``normalized`` (same shape), when given, receives the normalized values, which
    are bit-equal to the reference's.  With ``residual`` the row that is normalized is ``input + residual``
    (the reference's ``llmops.iadd`` in front of the norm, chatllama/main.py:359) and ``sum_out`` (may be
    ``input`` or ``residual`` itself) receives that sum."""
    _require_cuda(input, "input", torch.float32, 3)
    _require_cuda(weight, "weight", torch.float32, 1)
    B, M, K = input.shape
    _check_rows(B * M)
    if weight.shape[0] != K:
        raise RuntimeError(f"weight has {weight.shape[0]} elements, the rows {K}")
    if normalized is not None:
        _require_cuda(normalized, "normalized", torch.float32, 3)
        if normalized.shape != input.shape:
            raise RuntimeError("normalized: shape differs from input")
    for name, t in (("residual", residual), ("sum_out", sum_out)):
        if t is not None:
            _require_cuda(t, name, torch.float32, 3)
            if t.shape != input.shape:
                raise RuntimeError(f"{name}: shape differs from input")
    if sum_out is not None and residual is None:
        raise RuntimeError("sum_out without residual")
    xq = out if out is not None else QuantizedActivations(B, M, K, group_k, nibble_signed, input.device)
    with torch.cuda.device(input.device):
        _cabi.check(_cabi.lib().q4fc_add_rmsnorm_quant(
            input.data_ptr(), residual.data_ptr() if residual is not None else None,
            sum_out.data_ptr() if sum_out is not None else None, B * M, K, K, weight.data_ptr(), float(eps),
            normalized.data_ptr() if normalized is not None else None, K, group_k, int(nibble_signed),
            xq.buf.data_ptr(), FLAG_PDL if pdl else 0, _stream_ptr(input.device)), "rmsnorm_quantize")
    return xq


def silu_mul_quantize(gate: torch.Tensor, up: torch.Tensor, group_k: int, *, product: torch.Tensor | None = None,
                      nibble_signed: bool = False, pdl: bool = False,
                      out: QuantizedActivations | None = None) -> QuantizedActivations:
    """``llmops.itrans(gate, "silu")``, ``llmops.imul(up, gate)`` (ops/op_misc.hpp:83-138, chatllama/main.py:365-368)
    and the quantizer of the down projection behind them in one kernel.

    ``gate``, ``up`` fp32 ``[B, M, K]`` are left untouched; ``product`` (same shape), when given, receives
    ``silu(gate) * up``.  The reference's sigmoid uses an approximate reciprocal, so the products agree with
    it to about 4e-4 relative (not bit for bit); the codes are exact given the products."""
    _require_cuda(gate, "gate", torch.float32, 3)
    _require_cuda(up, "up", torch.float32, 3)
    if up.shape != gate.shape:
        raise RuntimeError("up: shape differs from gate")
    B, M, K = gate.shape
    _check_rows(B * M)
    if product is not None:
        _require_cuda(product, "product", torch.float32, 3)
        if product.shape != gate.shape:
            raise RuntimeError("product: shape differs from gate")
    xq = out if out is not None else QuantizedActivations(B, M, K, group_k, nibble_signed, gate.device)
    with torch.cuda.device(gate.device):
        _cabi.check(_cabi.lib().q4fc_silu_mul_quant(
            gate.data_ptr(), up.data_ptr(), B * M, K, K, product.data_ptr() if product is not None else None, K,
            group_k, int(nibble_signed), xq.buf.data_ptr(), FLAG_PDL if pdl else 0, _stream_ptr(gate.device)),
            "silu_mul_quantize")
    return xq


def fc_Q4A_q8(xq: QuantizedActivations, wei_quantized: torch.Tensor, N: int, *, out: torch.Tensor | None = None,
              pdl: bool = False) -> torch.Tensor:
    """``fc_Q4A`` on activations that were quantized beforehand: the same bytes as ``fc_Q4A(input, ...)``."""
    _require_cuda(wei_quantized, "wei_quantized", torch.int8, 3)
    Ng, Kg, bs = wei_quantized.shape
    q, G = _cabi.infer_variant(bs)
    if G != xq.group_k or Kg != xq.Kg:
        raise RuntimeError(f"activations quantized for group {xq.group_k} x {xq.Kg}, weights are group {G} x {Kg}")
    N = int(N)
    if out is None:
        out = torch.empty((xq.B, xq.M, N), dtype=torch.float32, device=wei_quantized.device)
    else:
        _require_cuda(out, "out", torch.float32, 3)
        if tuple(out.shape) != (xq.B, xq.M, N):
            raise RuntimeError(f"out: expected shape {(xq.B, xq.M, N)}, got {tuple(out.shape)}")
    if xq.signed and q != Q4_0:
        # the group-sum slot then holds the bits of 8 * (sum of codes), which a Q4_1 kernel would read as a float
        raise RuntimeError("activations quantized with nibble_signed=True serve Q4_0 weights only")
    flags = (FLAG_PDL if pdl else 0) | (FLAG_NIBBLE_SIGNED if (xq.signed and q == Q4_0) else 0)
    with torch.cuda.device(wei_quantized.device):
        _cabi.check(_cabi.lib().q4fc_fc_decode_q8(xq.buf.data_ptr(), xq.rows, xq.K, wei_quantized.data_ptr(), Ng, Kg,
                                                  q, G, N, out.data_ptr(), N, flags,
                                                  _stream_ptr(wei_quantized.device)), "fc_Q4A_q8")
    return out


def fc_Q4A_multi(input, weights, Ns, *, outs=None, addends=None, workspace: Workspace | None = None,
                 pdl: bool = False, nibble_signed: bool = False):
    """Several ``fc_Q4A`` on one input as ONE launch (``q4fc_fc_decode_multi``): the q/k/v projections, or
    gate/up -- three and two calls on the same tensor in the reference (chatllama/main.py:348-350, 365-367).

    ``input``: fp32 ``[B, M, K]`` with ``B*M <= 8``, or ``QuantizedActivations``.  ``weights``: up to four packed
    tensors of one block type and the same ``Kg``; ``Ns``: their output widths.  Returns the list of outputs,
    each bit-equal to the single call's."""
    prequantized = isinstance(input, QuantizedActivations)
    if prequantized:
        B, M, K, dev = input.B, input.M, input.K, input.buf.device
    else:
        _require_cuda(input, "input", torch.float32, 3)
        B, M, K = input.shape
        dev = input.device
    rows = B * M
    _check_rows(rows)
    if not 1 <= len(weights) <= 4 or len(Ns) != len(weights):
        raise RuntimeError("fc_Q4A_multi: one to four weight tensors, with one N each")
    q = G = Kg = None
    jobs = (_cabi.FcJob * len(weights))()
    outs = list(outs) if outs is not None else [None] * len(weights)
    addends = list(addends) if addends is not None else [None] * len(weights)
    for i, (w, N) in enumerate(zip(weights, Ns)):
        _require_cuda(w, f"weights[{i}]", torch.int8, 3)
        qi, Gi = _cabi.infer_variant(w.shape[2])
        if q is None:
            q, G, Kg = qi, Gi, int(w.shape[1])
        elif (qi, Gi, int(w.shape[1])) != (q, G, Kg):
            raise RuntimeError("fc_Q4A_multi: the weight tensors differ in block type or K")
        N = int(N)
        if outs[i] is None:
            outs[i] = torch.empty((B, M, N), dtype=torch.float32, device=dev)
        else:
            _require_cuda(outs[i], f"outs[{i}]", torch.float32, 3)
            if tuple(outs[i].shape) != (B, M, N):
                raise RuntimeError(f"outs[{i}]: expected shape {(B, M, N)}, got {tuple(outs[i].shape)}")
        jobs[i].wq, jobs[i].Ng, jobs[i].N = w.data_ptr(), int(w.shape[0]), N
        jobs[i].y, jobs[i].ldy = outs[i].data_ptr(), N
        a = addends[i]
        if a is not None:
            _require_cuda(a, f"addends[{i}]", torch.float32, a.dim())
            if tuple(a.shape) == (N,):
                jobs[i].ld_addend = 0
            elif tuple(a.shape) == (B, M, N):
                jobs[i].ld_addend = N
            else:
                raise RuntimeError(f"addends[{i}]: expected shape {(N,)} or {(B, M, N)}, got {tuple(a.shape)}")
            jobs[i].addend = a.data_ptr()
    if (K + G - 1) // G != Kg:
        raise RuntimeError(f"fc_Q4A_multi: K={K} does not match the weights' {Kg} groups of {G}")
    signed = nibble_signed or (prequantized and input.signed)
    if prequantized and input.signed and q != Q4_0:
        raise RuntimeError("activations quantized with nibble_signed=True serve Q4_0 weights only")
    flags = (FLAG_PDL if pdl else 0) | (FLAG_NIBBLE_SIGNED if (signed and q == Q4_0) else 0)
    with torch.cuda.device(dev):
        _cabi.check(_cabi.lib().q4fc_fc_decode_multi(
            None if prequantized else input.data_ptr(), input.buf.data_ptr() if prequantized else None, rows, K, K,
            Kg, q, G, jobs, len(weights), workspace.ptr if workspace is not None else None,
            workspace.nbytes if workspace is not None else 0, flags, _stream_ptr(dev)), "fc_Q4A_multi")
    return outs


class FCBatch:
    """A fixed batch of independent FCs that runs as ONE launch (``q4fc_fc_decode_batch``).

    ``calls``: up to 16 tuples ``(xq, wei_quantized, N)`` or ``(xq, wei_quantized, N, out)`` with ``xq`` a
    ``QuantizedActivations`` (several calls may share one) and the weights all of one block type.  The argument
    block is built once; ``run()`` only launches, so the object is cheap to call per step and safe to capture in
    a CUDA graph.  ``outs`` holds the outputs, each equal to ``fc_Q4A_q8`` of that call alone within the rounding
    of the fp32 sums."""

    def __init__(self, calls, *, pdl: bool = False) -> None:
        if not 1 <= len(calls) <= 16:
            raise RuntimeError("FCBatch: one to sixteen calls")
        self.n = len(calls)
        self._args = (_cabi.FcCall * self.n)()
        self._keep = []
        self.outs = []
        q = G = None
        signed = False
        for i, call in enumerate(calls):
            xq, w, N = call[0], call[1], int(call[2])
            out = call[3] if len(call) > 3 else None
            if not isinstance(xq, QuantizedActivations):
                raise RuntimeError("FCBatch: inputs must be QuantizedActivations (quantize_activations / rmsnorm_quantize)")
            _require_cuda(w, f"calls[{i}] weights", torch.int8, 3)
            qi, Gi = _cabi.infer_variant(w.shape[2])
            if q is None:
                q, G, self.device = qi, Gi, w.device
            elif (qi, Gi) != (q, G):
                raise RuntimeError("FCBatch: the weight tensors differ in block type")
            if Gi != xq.group_k or int(w.shape[1]) != xq.Kg:
                raise RuntimeError(f"calls[{i}]: activations are group {xq.group_k} x {xq.Kg}, weights {Gi} x {w.shape[1]}")
            if xq.signed and q != Q4_0:
                raise RuntimeError("activations quantized with nibble_signed=True serve Q4_0 weights only")
            signed = signed or xq.signed
            if out is None:
                out = torch.empty((xq.B, xq.M, N), dtype=torch.float32, device=w.device)
            else:
                _require_cuda(out, f"calls[{i}] out", torch.float32, 3)
                if tuple(out.shape) != (xq.B, xq.M, N):
                    raise RuntimeError(f"calls[{i}] out: expected shape {(xq.B, xq.M, N)}, got {tuple(out.shape)}")
            a = self._args[i]
            a.xq, a.rows, a.K = xq.buf.data_ptr(), xq.rows, xq.K
            a.wq, a.Ng, a.Kg, a.N = w.data_ptr(), int(w.shape[0]), int(w.shape[1]), N
            a.y, a.ldy = out.data_ptr(), N
            self._keep.append((xq, w))
            self.outs.append(out)
        self.qtype, self.group_k = q, G
        self.flags = (FLAG_PDL if pdl else 0) | (FLAG_NIBBLE_SIGNED if (signed and q == Q4_0) else 0)

    def run(self):
        with torch.cuda.device(self.device):
            _cabi.check(_cabi.lib().q4fc_fc_decode_batch(self._args, self.n, self.qtype, self.group_k, self.flags,
                                                         _stream_ptr(self.device)), "fc_decode_batch")
        return self.outs


class FCChain:
    """A chain of dependent decode FCs that runs as ONE persistent launch (``q4fc_fc_chain_*``): the weight stream
    does not stop between the steps, only the activations wait for the step before.

    ``steps``: a list of dicts, in execution order:
        ``x``          fp32 CUDA tensor ``[1, rows, K]`` (or ``[rows, K]``): the step's input -- an output of an earlier
                       step, or a tensor the caller fills before ``run()``;
        ``transform``  ``"plain"`` (default), ``"rmsnorm"`` (``aux`` = weight ``[K]``, ``eps``) or ``"silu_mul"``
                       (``aux`` = the up projection, same shape as ``x``: the value quantized is ``aux * silu(x)``);
        ``jobs``       ``[(wei_quantized, N, out), ...]`` or ``(wei_quantized, N, out, addend)``: weight tensors that
                       multiply the step's input, ``out`` fp32 ``[1, rows, N]``, ``addend`` a bias ``[N]`` or a tensor of
                       ``out``'s shape (the residual stream) added to the result.
    All weights share one block type; ``rows <= 8``; ``K % 8 == 0``.  The tables are uploaded once; ``run()`` only
    launches (asynchronous on the current stream, capturable in a CUDA graph); ``check()`` waits and raises if a
    bounded wait inside the kernel ran out."""

    _TRANSFORMS = {"plain": _cabi.CHAIN_PLAIN, "rmsnorm": _cabi.CHAIN_RMSNORM, "silu_mul": _cabi.CHAIN_SILU_MUL}

    def __init__(self, steps) -> None:
        if not steps:
            raise RuntimeError("FCChain: no steps")
        njobs = sum(len(s["jobs"]) for s in steps)
        self._steps = (_cabi.ChainStep * len(steps))()
        self._jobs = (_cabi.FcJob * max(njobs, 1))()
        self._keep = []
        self._handle = None
        q = G = rows = None
        jn = 0
        for i, s in enumerate(steps):
            x = s["x"]
            if not isinstance(x, torch.Tensor) or x.dtype != torch.float32 or not x.is_cuda or not x.is_contiguous():
                raise RuntimeError(f"steps[{i}].x: expected a contiguous fp32 CUDA tensor")
            K = int(x.shape[-1])
            r = x.numel() // K
            if rows is None:
                rows, self.device = r, x.device
            elif r != rows:
                raise RuntimeError(f"steps[{i}].x has {r} rows, the chain {rows}")
            tname = s.get("transform", "plain")
            if tname not in self._TRANSFORMS:
                raise RuntimeError(f"steps[{i}].transform={tname!r}: expected one of {sorted(self._TRANSFORMS)}")
            aux = s.get("aux")
            if tname == "rmsnorm":
                _require_cuda(aux, f"steps[{i}].aux", torch.float32, 1)
                if aux.numel() != K:
                    raise RuntimeError(f"steps[{i}].aux: rmsnorm weight of {aux.numel()} values for K={K}")
            elif tname == "silu_mul":
                if not isinstance(aux, torch.Tensor) or aux.dtype != torch.float32 or tuple(aux.shape) != tuple(x.shape) \
                        or not aux.is_cuda or not aux.is_contiguous():
                    raise RuntimeError(f"steps[{i}].aux: silu_mul needs the up projection, a tensor like x")
            elif aux is not None:
                raise RuntimeError(f"steps[{i}]: a plain step takes no aux")
            if not s["jobs"]:
                raise RuntimeError(f"steps[{i}]: no jobs")
            st = self._steps[i]
            st.x, st.ldx, st.K = x.data_ptr(), K, K
            st.transform, st.eps = self._TRANSFORMS[tname], float(s.get("eps", 0.0))
            st.aux, st.njobs = (aux.data_ptr() if aux is not None else None), len(s["jobs"])
            self._keep.append((x, aux))
            for job in s["jobs"]:
                w, N, out = job[0], int(job[1]), job[2]
                addend = job[3] if len(job) > 3 else None
                _require_cuda(w, f"steps[{i}] weights", torch.int8, 3)
                qi, Gi = _cabi.infer_variant(w.shape[2])
                if q is None:
                    q, G = qi, Gi
                elif (qi, Gi) != (q, G):
                    raise RuntimeError("FCChain: the weight tensors differ in block type")
                if int(w.shape[1]) != (K + Gi - 1) // Gi:
                    raise RuntimeError(f"steps[{i}]: weights hold {w.shape[1]} K groups, the input needs {(K + Gi - 1) // Gi}")
                if not isinstance(out, torch.Tensor) or out.dtype != torch.float32 or not out.is_cuda \
                        or not out.is_contiguous() or out.numel() != rows * N or int(out.shape[-1]) != N:
                    raise RuntimeError(f"steps[{i}] out: expected a contiguous fp32 CUDA tensor [..., {rows}, {N}]")
                a = self._jobs[jn]
                a.wq, a.Ng, a.N, a.y, a.ldy = w.data_ptr(), int(w.shape[0]), N, out.data_ptr(), N
                a.addend, a.ld_addend = None, 0
                if addend is not None:
                    if not isinstance(addend, torch.Tensor) or addend.dtype != torch.float32 or not addend.is_cuda \
                            or not addend.is_contiguous():
                        raise RuntimeError(f"steps[{i}] addend: expected a contiguous fp32 CUDA tensor")
                    if addend.numel() == N:
                        a.addend, a.ld_addend = addend.data_ptr(), 0  # one row for all: a bias
                    elif addend.numel() == rows * N and int(addend.shape[-1]) == N:
                        a.addend, a.ld_addend = addend.data_ptr(), N
                    else:
                        raise RuntimeError(f"steps[{i}] addend: expected [{N}] or the shape of out")
                self._keep.append((w, out, addend))
                jn += 1
        self.rows, self.qtype, self.group_k, self.nsteps, self.njobs = rows, q, G, len(steps), njobs
        h = _cabi.C.c_void_p()
        with torch.cuda.device(self.device):
            _cabi.check(_cabi.lib().q4fc_fc_chain_create(self._steps, len(steps), self._jobs, njobs, rows, q, G,
                                                         _cabi.C.byref(h)), "FCChain")
        self._handle = h

    def run(self) -> None:
        with torch.cuda.device(self.device):
            _cabi.check(_cabi.lib().q4fc_fc_chain_run(self._handle, _stream_ptr(self.device)), "FCChain.run")

    def check(self) -> None:
        with torch.cuda.device(self.device):
            _cabi.check(_cabi.lib().q4fc_fc_chain_check(self._handle, _stream_ptr(self.device)), "FCChain.check")

    def close(self) -> None:
        if self._handle is not None:
            h, self._handle = self._handle, None
            with torch.cuda.device(self.device):
                torch.cuda.synchronize(self.device)
                _cabi.lib().q4fc_fc_chain_destroy(h)

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass


# ---- per-channel int8 weights ("Q8C") and the quantized embedding table ---------------------------------------------
_q8c_scratch: dict = {}


def FC_quant_Q8C(wei: torch.Tensor):
    """fp32 ``[N, K]`` -> (int8 ``[ceil(N/32), ceil(K/32), 1024]``, fp32 scales ``[ceil(N/32)*32]``), bit-identical to
    ``FC_quant_Q8C`` of the reference's older extension (ext/llama_ext.cpp:56-113)."""
    _require_cuda(wei, "wei", torch.float32, 2)
    N, K = wei.shape
    Ng, Kg = (N + 31) // 32, (K + 31) // 32
    wq = torch.empty((Ng, Kg, 1024), dtype=torch.int8, device=wei.device)
    ws = torch.empty((Ng * 32,), dtype=torch.float32, device=wei.device)
    with torch.cuda.device(wei.device):
        _cabi.check(_cabi.lib().q4fc_q8c_pack(wei.data_ptr(), N, K, wq.data_ptr(), ws.data_ptr(),
                                              _stream_ptr(wei.device)), "FC_quant_Q8C")
    return wq, ws


def FC_evaluate_Q8C(input: torch.Tensor, wei_quantized: torch.Tensor, wei_scales: torch.Tensor, N: int, *,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """``[B, M, K]`` x Q8C weights -> ``[B, M, N]`` (ext/llama_ext.cpp:336-371).  The scratch for the quantized
    activations is kept per (device, stream) and grows to the largest call; calls on one stream are ordered."""
    _require_cuda(input, "input", torch.float32, 3)
    _require_cuda(wei_quantized, "wei_quantized", torch.int8, 3)
    _require_cuda(wei_scales, "wei_scales", torch.float32, 1)
    B, M, K = input.shape
    Ng, Kg, bs = wei_quantized.shape
    if bs != 1024:
        raise RuntimeError(f"assert wei_quantized.size(2) == sizeof(q8_c_block) failed: got {bs}")
    if Kg != (K + 31) // 32 or N > Ng * 32 or wei_scales.numel() < N:
        raise RuntimeError(f"FC_evaluate_Q8C: weights {tuple(wei_quantized.shape)} / scales {tuple(wei_scales.shape)} "
                           f"do not match K={K}, N={N}")
    dev = input.device
    if out is None:
        out = torch.empty((B, M, N), dtype=torch.float32, device=dev)
    else:
        _require_cuda(out, "out", torch.float32, 3)
        if tuple(out.shape) != (B, M, N):
            raise RuntimeError(f"out: expected shape {(B, M, N)}, got {tuple(out.shape)}")
    L = _cabi.lib()
    need = L.q4fc_q8c_workspace_bytes(B * M, K)
    with torch.cuda.device(dev):
        stream = _stream_ptr(dev)
        key = (dev.index, stream)
        ws = _q8c_scratch.get(key)
        if ws is None or ws.numel() < need:
            ws = torch.empty(max(need, 1 << 16), dtype=torch.uint8, device=dev)
            _q8c_scratch[key] = ws
        _cabi.check(L.q4fc_q8c_fc(input.data_ptr(), B * M, K, K, wei_quantized.data_ptr(), wei_scales.data_ptr(), Ng,
                                  Kg, N, out.data_ptr(), N, ws.data_ptr(), ws.numel(), stream), "FC_evaluate_Q8C")
    return out


def embedding_q8c_quant_w(weight: torch.Tensor):
    """fp32 table ``[V, E]`` -> (int8 codes ``[V, E]``, fp32 scales ``[V]``), bit-identical to the reference's
    ``llmops.embedding_q8c_quant_w`` (ops/op_embedding.hpp:51-78)."""
    _require_cuda(weight, "weight", torch.float32, 2)
    V, E = weight.shape
    codes = torch.empty((V, E), dtype=torch.int8, device=weight.device)
    scales = torch.empty((V,), dtype=torch.float32, device=weight.device)
    with torch.cuda.device(weight.device):
        _cabi.check(_cabi.lib().q4fc_emb_q8c_quant(weight.data_ptr(), V, E, codes.data_ptr(), scales.data_ptr(),
                                                   _stream_ptr(weight.device)), "embedding_q8c_quant_w")
    return codes, scales


def embedding_q8c(output: torch.Tensor, input: torch.Tensor, weight: torch.Tensor, scales: torch.Tensor) -> None:
    """``output[..., :] = scales[id] * weight[id, :]`` for the ids in ``input`` (int32 or int64, any rank), with the
    reference's argument order and in-place result (ops/op_embedding.hpp:108-137).  An id outside the table gives a
    row of zeros and makes ``check_device_status`` raise."""
    _require_cuda(weight, "weight", torch.int8, 2)
    _require_cuda(scales, "scales", torch.float32, 1)
    if not isinstance(input, torch.Tensor) or input.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("assert input.is<int64_t>() failed: ids must be int32 or int64")
    if not input.is_cuda or not input.is_contiguous():
        raise RuntimeError("input: must be a contiguous CUDA tensor")
    V, E = weight.shape
    if not isinstance(output, torch.Tensor) or output.dtype != torch.float32:
        raise RuntimeError("assert output.is<float>() failed")
    if tuple(output.shape) != tuple(input.shape) + (E,):
        raise RuntimeError(f"assert infer_shape() == output.shape() failed: {tuple(output.shape)} vs "
                           f"{tuple(input.shape) + (E,)}")
    if not output.is_cuda or not output.is_contiguous():
        raise RuntimeError("output: must be a contiguous CUDA tensor")
    with torch.cuda.device(weight.device):
        _cabi.check(_cabi.lib().q4fc_emb_q8c(input.data_ptr(), int(input.dtype == torch.int32), input.numel(),
                                             weight.data_ptr(), scales.data_ptr(), V, E, output.data_ptr(), E,
                                             _stream_ptr(weight.device)), "embedding_q8c")


def check_device_status(device: torch.device | None = None) -> None:
    """Raises if a kernel launched without a workspace on this device reported a failure (a bounded wait that ran
    out, an embedding id outside its table).  Host-synchronous on the current stream."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    with torch.cuda.device(dev):
        _cabi.check(_cabi.lib().q4fc_fc_check_status(None, _stream_ptr(dev)), "check_device_status")


def fc_Q4A2(input, wei_quantized, N):
    """Bound by the reference (ops/main.cpp:161) but its body is compiled out (ops/op_fc.hpp:428-623)."""
    raise RuntimeError("fc_Q4A2 has no implementation in the reference; use fc_Q4A")
