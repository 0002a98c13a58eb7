"""GPU drop-in for the FC part of the reference's older torch extension
``chatllama.c_ext`` (``ext/llama_ext.cpp:633-654``): ``FC_quant_Q4A``,
``FC_evaluate_Q4A``, the class ``FCQ4A``, and the per-channel int8 pair
``FC_quant_Q8C`` / ``FC_evaluate_Q8C``.  Its Q4A functions only have the
Q4_1 / group-32 block (``ext/llama_ext.cpp:378-400``)."""
from __future__ import annotations

import torch

from . import llmops


def FC_quant_Q4A(weight: torch.Tensor) -> torch.Tensor:
    """ext/llama_ext.cpp:405-471: fp32 [N, K] -> int8 [Ng, Kg, 640]."""
    return llmops.offline_FC_quant_Q4A(weight, qtype="q4_1", group_k=32)


def FC_evaluate_Q4A(input: torch.Tensor, weight: torch.Tensor, N: int) -> torch.Tensor:
    """ext/llama_ext.cpp:484-606: input [B, M, K] -> [B, M, N]."""
    return llmops.fc_Q4A(input, weight, N)


def FC_quant_Q8C(weight: torch.Tensor):
    """ext/llama_ext.cpp:56-113: fp32 [N, K] -> [int8 [Ng, Kg, 1024], fp32 [Ng*32]]."""
    return list(llmops.FC_quant_Q8C(weight))


def FC_evaluate_Q8C(input: torch.Tensor, wei_quantized: torch.Tensor, wei_scales: torch.Tensor, N: int) -> torch.Tensor:
    """ext/llama_ext.cpp:336-371: input [B, M, K] -> [B, M, N]."""
    return llmops.FC_evaluate_Q8C(input, wei_quantized, wei_scales, N)


class FCQ4A:
    """ext/llama_ext.cpp:608-625: packs at construction, ``forward(input)`` evaluates."""

    def __init__(self, weight: torch.Tensor) -> None:
        self._N = int(weight.shape[0])
        self._weight = FC_quant_Q4A(weight)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return FC_evaluate_Q4A(input, self._weight, self._N)

    def __repr__(self) -> str:
        return "FCQ4A()"
