"""RMSNorm, with the residual add that precedes it fused in.

y_i = x_i * 1/sqrt(mean(x^2) + eps) * w_i, everything in float32
(crates/aegisllm-cuda/src/cuda/kernels/blackwell/norm_rope_kv.cu:36-62;
crates/aegisllm-cpu/src/cpu/math.rs:4-8). `weight_offset` 1 gives the (1 + w)
form that the reference folds in for other families (executor/loader.rs:189-194);
it is a parameter, 0 for Qwen3 dense. With `scalar` the stored weight is ONE number
(a tensor without dimensions) that multiplies every coordinate.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import need, register_part, tensor_name


class NormedUpdate:
    """An update of the residual stream that is RMS-normed BEFORE it is added (a norm at a
    sublayer's output): h += rmsnorm(sum of `delta`'s partial sums + `bias`) * `weight`. A block
    hands it on as `pending` like a plain stack of partial sums, and the norm that follows does
    the whole chain, norm of the update, add, its own norm, in one kernel."""
    __slots__ = ("delta", "weight", "eps", "bias")

    def __init__(self, delta, weight, eps, bias=None):
        self.delta, self.weight, self.eps, self.bias = delta, weight, float(eps), bias


@register_part("norm", "rmsnorm")
class RMSNorm:
    @classmethod
    def tensors(cls, spec):
        size = need(spec.params, "size", "rmsnorm")
        return {tensor_name(spec): (() if spec.params.get("scalar") else (size,), "norm")}

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.size = int(need(p, "size", "rmsnorm"))
        self.eps = float(need(p, "eps", "rmsnorm"))
        w = weights[tensor_name(spec)].to(device=runtime.device, dtype=torch.float32)
        if p.get("scalar"):
            w = w.reshape(1).expand(self.size)        # the kernels read one weight a coordinate
        off = float(p.get("weight_offset", 0.0))
        self.weight = (w + off).contiguous() if off else w.contiguous()

    def forward(self, h, delta, out_dtype, rows=None, write_h=True):
        if isinstance(delta, NormedUpdate):
            return K.postnorm_add_rmsnorm(h, delta.delta, delta.bias, delta.weight, delta.eps, self.weight,
                                          self.eps, out_dtype, rows=rows, write_h=write_h)
        return K.add_rmsnorm(h, delta, self.weight, self.eps, out_dtype, rows=rows, write_h=write_h)

    def forward_conv(self, h, delta, conv, state, ctx, out_dtype):
        """The norm and, behind it, an input convolution (parts/conv.py) of the normed rows. A
        step of one token a sequence whose pending update is a NormedUpdate (or nothing) is one
        kernel; everything else is the norm, in float32, and then the convolution."""
        if ctx.is_decode and (delta is None or isinstance(delta, NormedUpdate)):
            d = delta
            return K.postnorm_add_rmsnorm(h, None if d is None else d.delta, None if d is None else d.bias,
                                          None if d is None else d.weight, 0.0 if d is None else d.eps,
                                          self.weight, self.eps, out_dtype,
                                          conv=(conv.weight, state, ctx.seq_slot))
        return conv.forward(self.forward(h, delta, torch.float32), state, ctx, out_dtype)
