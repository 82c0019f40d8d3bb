"""A selective state-space mixer ("mamba2"): a linear recurrence over time with a matrix state
per head, in place of attention.

In order, for H heads of P channels, state size N and G groups (inner = H P):
u = y Win^T, laid out [z: inner | x: inner | B: G N | C: G N | dt: H]; x, B and C together go
through a causal convolution over time on each channel of its own (`taps` taps with a bias, the
last tap the current token's, zeros before a sequence's start) and SiLU;
dt = softplus(dt + dt_bias); per head h, with the B and C of group h // (H / G):
S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T (S is N x P), y_t = S_t^T C_t + D_h x_t;
the heads' y side by side are multiplied by silu(z), RMS-normed in `norm_groups` equal parts
(each by its own root mean square) times a weight, and projected back: out = v Wo^T.

A sequence's state is S of every head (float32) and the convolution's last taps - 1 inputs; both
start at zero and are carried from step to step, so a sequence may be fed in any portions.
Everything that enters the recurrence is float32; the two projections run in the run's type.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import need, register_part
from .linear import Linear


@register_part("mixer", "mamba2")
class StateSpaceMixer:
    graph_safe = True

    @staticmethod
    def _sizes(p):
        D, H, P, N, G, taps, parts = (int(need(p, k, "mamba2")) for k in
                                      ("hidden_size", "num_heads", "head_dim", "state_size", "groups", "taps",
                                       "norm_groups"))
        return D, H, P, N, G, taps, parts

    @classmethod
    def tensors(cls, spec):
        D, H, P, N, G, taps, _ = cls._sizes(spec.params)
        inner, C = H * P, H * P + 2 * G * N
        pre = spec.prefix
        return {f"{pre}.in": ((inner + C + H, D), "matrix"), f"{pre}.conv": ((C, taps), "matrix"),
                f"{pre}.conv.b": ((C,), "matrix"), f"{pre}.dt_bias": ((H,), "matrix"),
                f"{pre}.A_log": ((H,), "matrix"), f"{pre}.D": ((H,), "matrix"),
                f"{pre}.norm": ((inner,), "norm"), f"{pre}.o": ((D, inner), "matrix")}

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.runtime = runtime
        self.D, self.H, self.P, self.N, self.G, self.taps, self.parts = self._sizes(p)
        self.inner = self.H * self.P
        self.C = self.inner + 2 * self.G * self.N
        if self.H % self.G or self.inner % self.parts:
            raise ValueError(f"{self.H} heads in {self.G} groups, {self.inner} channels in {self.parts} parts: "
                             "the first must divide evenly")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"a convolution of {self.taps} taps: this kernel takes 1 to 16")
        self.eps = float(need(p, "norm_eps", "mamba2"))
        pre = spec.prefix
        f32 = lambda n: weights[n].to(device=runtime.device, dtype=torch.float32).contiguous()
        self.w_in = Linear(weights[f"{pre}.in"], runtime)
        self.w_out = Linear(weights[f"{pre}.o"], runtime)
        self.conv_w = f32(f"{pre}.conv").t().contiguous()      # [taps, channels]: a tap's weights lie together
        self.conv_b = f32(f"{pre}.conv.b")
        self.dt_bias, self.a_log, self.d_skip = f32(f"{pre}.dt_bias"), f32(f"{pre}.A_log"), f32(f"{pre}.D")
        self.norm_w = f32(f"{pre}.norm")
        self.n_state = self.H * self.N * self.P
        self.n_conv = (self.taps - 1) * self.C

    def cache_need(self):
        return None

    def state_shape(self):
        """One float32 row a sequence: the heads' states [H, N, P], then the convolution's last
        inputs [taps - 1, C]."""
        return ((self.n_state + self.n_conv,), torch.float32)

    adds_residual = True      # forward takes `residual` and may add its update to it in place

    def forward(self, y, ctx, entry, residual=None):
        store = entry.state()
        S = store[:, :self.n_state].unflatten(1, (self.H, self.N, self.P))
        conv_state = store[:, self.n_state:].unflatten(1, (self.taps - 1, self.C)) if self.taps > 1 else None
        u = self.w_in(y, split_ok=True)                     # float32 [N, W], possibly partial sums
        xbc = K.conv_silu(u, self.inner, self.C, self.conv_w, self.conv_b, conv_state, ctx.tok_seq, ctx.cu_q,
                          ctx.seq_slot, ctx.B, ctx.is_decode)
        yh = K.ssm_scan(xbc, self.H, self.P, self.N, self.G, u, self.inner + self.C, self.dt_bias, self.a_log,
                        self.d_skip, S, ctx.cu_q, ctx.seq_slot, ctx.B)
        v = K.gated_part_norm(yh, u, 0, self.norm_w, self.eps, self.parts, self.runtime.dtype)
        return self.w_out(v, split_ok=True, add_to=residual)
