"""The attention mixer whose heads talk after the softmax.

In order: q, k, v = y Wq^T + bq, y Wk^T + bk, y Wv^T + bv; ONE RMS norm over the whole query
projection (all heads at once, a weight of heads x dim values) and one over the whole key
projection; no rotation (positions enter the model elsewhere, or not at all); k, v appended to
the cache (keys of `head_dim`, values of `value_dim` values, which may differ); a query at
position p sees key j if j <= p and (p - j < window or j < keep_first); per head an ordinary
softmax of scale * q . k over the visible keys; then the heads' weights are mixed,
m_h = sum_g talk[h, g] w_g, and head h applies m_h to the values of its own kv head
(h // (heads / kv_heads)); o = ctx Wo^T + bo. Scores, weights and the mix are float32.
"""
from __future__ import annotations

import torch

from ..cache.kv import LAYOUT_LINEAR, CacheNeed
from ..ops import kernels as K
from .base import need, register_part
from .linear import Linear


@register_part("mixer", "talking_attention")
class TalkingAttention:
    graph_safe = True

    @classmethod
    def tensors(cls, spec):
        p = spec.params
        D, H, G, d, dv = (int(need(p, k, "talking_attention")) for k in
                          ("hidden_size", "num_heads", "num_kv_heads", "head_dim", "value_dim"))
        pre = spec.prefix
        return {f"{pre}.q": ((H * d, D), "matrix"), f"{pre}.q.b": ((H * d,), "matrix"),
                f"{pre}.k": ((G * d, D), "matrix"), f"{pre}.k.b": ((G * d,), "matrix"),
                f"{pre}.v": ((G * dv, D), "matrix"), f"{pre}.v.b": ((G * dv,), "matrix"),
                f"{pre}.q.norm": ((H * d,), "norm"), f"{pre}.k.norm": ((G * d,), "norm"),
                f"{pre}.talk": ((H, H), "matrix"),
                f"{pre}.o": ((D, H * dv), "matrix"), f"{pre}.o.b": ((D,), "matrix")}

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.runtime = runtime
        self.D = int(p["hidden_size"])
        self.H, self.G = int(p["num_heads"]), int(p["num_kv_heads"])
        self.d, self.dv = int(p["head_dim"]), int(p["value_dim"])
        if self.H % self.G:
            raise ValueError(f"{self.H} heads are not a multiple of {self.G} kv heads")
        self.window = int(need(p, "window", "talking_attention"))
        self.keep_first = int(p.get("keep_first", 0))
        self.scale = float(need(p, "softmax_scale", "talking_attention"))
        self.eps = float(need(p, "norm_eps", "talking_attention"))
        pre = spec.prefix
        f32 = lambda n: weights[n].to(device=runtime.device, dtype=torch.float32).contiguous()
        self.qkv = Linear.stacked([weights[f"{pre}.q"], weights[f"{pre}.k"], weights[f"{pre}.v"]], runtime)
        self.qkv_bias = torch.cat([f32(f"{pre}.q.b"), f32(f"{pre}.k.b"), f32(f"{pre}.v.b")]).contiguous()
        self.q_norm, self.k_norm = f32(f"{pre}.q.norm"), f32(f"{pre}.k.norm")
        self.talk = f32(f"{pre}.talk")
        self.o = Linear(weights[f"{pre}.o"], runtime)
        self.update_bias = f32(f"{pre}.o.b")     # added by whoever adds the update's partial sums

    def cache_need(self):
        # tiles [key][values], keys and values each of their own width
        return CacheNeed(self.G, self.d, self.window, v_dim=self.dv, keep_first=self.keep_first,
                         layout=LAYOUT_LINEAR)

    def state_shape(self):
        return None

    def forward(self, y, ctx, entry, bias_downstream=False):
        """The update as float32 partial sums; with bias_downstream the output projection's bias
        is left to the consumer (`update_bias`), else it is added here."""
        kc, vc, table = entry.cache()
        qkv = self.qkv(y, split_ok=True)
        q = K.qkv_bias_norm_store(qkv, self.qkv_bias, self.q_norm, self.k_norm, self.eps, ctx.cache_pos,
                                  ctx.tok_seq, table, kc, vc, self.H, self.G, self.d, self.dv,
                                  self.runtime.dtype)
        # steps in which sequences bring many tokens go to the tensor cores; one token each, to
        # the kernels that spread a sequence's keys over the device
        prompt = {} if ctx.is_decode else dict(cu_q=ctx.cu_q, seq_start=ctx.seq_start, n_seqs=ctx.B)
        out = K.attn_talk(q, kc, vc, table, ctx.tok_seq, ctx.cache_pos, self.talk, self.window,
                          self.keep_first, self.scale, self.dv, **prompt)
        delta = self.o(out.view(-1, self.H * self.dv), split_ok=True)
        if not bias_downstream:
            (delta[0] if delta.dim() == 3 else delta).add_(self.update_bias)
        return delta
