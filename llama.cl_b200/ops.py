"""``llmop_fc_q4a``: the callable the reference's model builds for every
``nn.Linear`` (``chatllama/main.py:158-177``), and ``llmop_embedding_q8c``, the
one it builds for the token table (``chatllama/main.py:207-219``), on the GPU
kernels."""
from __future__ import annotations

import torch

from . import llmops


class llmop_fc_q4a:
    """Packs ``linear.weight`` at construction, ``__call__(input)`` runs the FC
    and adds the bias.  Attributes as in the reference: ``weight`` (packed),
    ``bias``, ``N``.  ``qtype`` / ``group_k`` choose the block type that the
    reference fixes at compile time."""

    def __init__(self, linear, *, qtype="q4_1", group_k: int = 32, device=None) -> None:
        w = linear.weight.detach()
        dev = torch.device(device) if device is not None else (w.device if w.is_cuda else torch.device("cuda"))
        w = w.to(device=dev, dtype=torch.float32).contiguous()
        self.weight = llmops.offline_FC_quant_Q4A(w, qtype=qtype, group_k=group_k)
        b = getattr(linear, "bias", None)
        self.bias = b.detach().to(device=dev, dtype=torch.float32).contiguous() if b is not None else None
        self.N = int(linear.weight.shape[0])

    def __call__(self, input: torch.Tensor, **kw) -> torch.Tensor:
        if self.bias is not None and input.shape[0] * input.shape[1] <= 8 and kw.get("path", "auto") in ("auto", "decode"):
            # the reference's llmops.iadd(out, bias), folded into the decode kernel (same single fp32 add)
            return llmops.fc_Q4A(input, self.weight, self.N, addend=self.bias, **kw)
        out = llmops.fc_Q4A(input, self.weight, self.N, **kw)
        if self.bias is not None:
            out.add_(self.bias)  # the reference's llmops.iadd(out, bias)
        return out

    def weight_size(self) -> int:
        size = self.weight.numel() * self.weight.element_size()
        if self.bias is not None:
            size += self.bias.numel() * self.bias.element_size()
        return size

    def __repr__(self) -> str:
        return f"llmop_fc_q4a(weight: {list(self.weight.shape)})"


class llmop_embedding_q8c:
    """Quantizes the table at construction (one scale per row), ``__call__(input_ids)`` looks rows up and
    dequantizes them.  Attributes as in the reference: ``weight`` (int8 codes ``[V, E]``), ``scales`` (``[V]``)."""

    def __init__(self, weight: torch.Tensor, *, device=None) -> None:
        w = weight.detach()
        dev = torch.device(device) if device is not None else (w.device if w.is_cuda else torch.device("cuda"))
        self.weight, self.scales = llmops.embedding_q8c_quant_w(w.to(device=dev, dtype=torch.float32).contiguous())

    def __call__(self, input_ids: torch.Tensor) -> torch.Tensor:
        ids = input_ids.to(self.weight.device).contiguous()
        output = torch.empty(tuple(ids.shape) + (self.weight.shape[1],), dtype=torch.float32, device=self.weight.device)
        llmops.embedding_q8c(output, ids, self.weight, self.scales)
        return output

    def __repr__(self) -> str:
        return f"llmop_embedding_q8c(weight: {list(self.weight.shape)})"
