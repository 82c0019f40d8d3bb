"""Convolutions over time of what a sublayer reads.

"causal_depthwise": out_t = y_t + sum_{j < taps} w[:, j] * y_(t - taps + 1 + j) on every channel
of its own, zeros before the sequence's start; the weight is stored [channels, taps], without a
bias. The last taps - 1 inputs of a sequence are its state (float32 [taps - 1, channels] per
sequence, zeros for a new one): a step reads what lies before its first token from there and
moves the state on to its end, so the result does not depend on how a sequence is cut into steps.
The arithmetic is float32; the output has the run's type.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import need, register_part, tensor_name


@register_part("input_conv", "causal_depthwise")
class CausalDepthwiseConv:
    graph_safe = True

    @classmethod
    def tensors(cls, spec):
        p = spec.params
        return {tensor_name(spec): ((int(need(p, "size", "causal_depthwise")),
                                     int(need(p, "taps", "causal_depthwise"))), "matrix")}

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.size, self.taps = int(p["size"]), int(p["taps"])
        if not 1 <= self.taps <= K.CANON_MAX_TAPS:
            raise ValueError(f"a convolution of {self.taps} taps: this kernel takes 1 to {K.CANON_MAX_TAPS}")
        w = weights[tensor_name(spec)].to(device=runtime.device, dtype=torch.float32)
        self.weight = w.t().contiguous()          # [taps, channels]: a tap's weights lie together

    def state_rows(self) -> int:
        return self.taps - 1

    def forward(self, y, state, ctx, out_dtype):
        """y float32 [N, channels]; state float32 [slots + 1, taps - 1, channels] (None with one tap)."""
        return K.canon_conv(y, self.weight, state, ctx.tok_seq, ctx.cu_q, ctx.seq_slot, ctx.B, out_dtype)
