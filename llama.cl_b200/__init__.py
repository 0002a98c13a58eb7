"""B200 (sm_100a) implementation of the quantized fully-connected path of
usstq/llama.cl: Q4_0 / Q4_1 weight packer, Q8 activation quantizer and the
packed-nibble FC product, behind the reference's op names.

    llmops   -- offline_FC_quant_Q4A / offline_FC_dequant_Q4A / fc_Q4A
    c_ext    -- FC_quant_Q4A / FC_evaluate_Q4A / FCQ4A (older extension names)
    ops      -- llmop_fc_q4a (the per-Linear callable of the reference model)
    host     -- host-buffer front ends (copy in, FC, copy out as one replayed graph)
    stack    -- the per-token FC schedule of a Llama block stack as one replayed graph
    tp       -- N-split of one FC over the GPUs of a node: joined by an all-gather, or by
                the FC kernel's own stamped stores into every rank's buffer

All compute runs in ``lib/libq4fc_b200.so`` (see ``include/q4fc_b200.h``).
"""
from . import _cabi, c_ext, host, llmops, ops, stack, tp  # noqa: F401
from .llmops import fc_Q4A, offline_FC_dequant_Q4A, offline_FC_quant_Q4A  # noqa: F401
from .ops import llmop_fc_q4a  # noqa: F401

__version__ = "0.1.0"
