"""A plain, slow implementation of the Rasezen decoder on the CPU, written from the design's
equations, one function per mechanism. It shares no code with the library: whole sequences only,
no cache, no batching, a Python loop over time for the recurrence. The tests compare the engine
with it.

Notation: a sequence of T tokens, width D. Attention: H query heads, G key/value heads,
query/key size d, value size dv. State-space mixer: H heads of P channels, state size N, G
groups of (B, C) vectors. unit(x) = x / sqrt(mean(x^2) + eps) over the last axis.
"""
import json
import math
import struct
from pathlib import Path

import torch

F = torch.float32


def read_safetensors(path):
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    head = json.loads(raw[8:8 + n])
    data = memoryview(raw)[8 + n:]
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16}
    out = {}
    for name, info in head.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
    return out


def load_model(folder, dtype=F):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {k: v.to(dtype) for k, v in read_safetensors(folder / "model.safetensors").items()}
    return cfg, w


# ------------------------------------------------------------------ small pieces

def unit(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose weight is ONE number for all coordinates."""
    return unit(x, eps) * g


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2."""
    ap, aq = softplus(p), 0.5 + softplus(q)
    neg = torch.clamp(z, max=0.0)
    return torch.where(z > 0, ap * z * z + 0.5 * z, aq * (torch.expm1(neg) - neg) + 0.5 * z)


def rotate(x, positions, base, dims):
    """x [T, heads, d]; the first `dims` coordinates of each head are rotated in pairs
    (i, i + dims/2) by the angle position * base^(-2i/dims); the rest pass."""
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = torch.tensor(float(base), dtype=x.dtype) ** (-2.0 * i / dims)
    a = positions.to(x.dtype)[:, None] * freq[None, :]            # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def window_mask(T, size):
    """[T, T] True where query i sees key j: 0 <= i - j < size."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i - j < size)


# ------------------------------------------------------------------ mixers

def attention(h, w, pre, m, eps):
    """h [T, D]; m: the layer's 'mixer' object of config.json; pre: '<layer>.mix'."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w[f"{pre}.q"].T + w[f"{pre}.q.b"]
    k = h @ w[f"{pre}.k"].T + w[f"{pre}.k.b"]
    v = h @ w[f"{pre}.v"].T + w[f"{pre}.v.b"]
    q = unit(q, eps) * w[f"{pre}.q.norm"]              # over the whole projection, all heads at once
    k = unit(k, eps) * w[f"{pre}.k.norm"]
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, dv)
    if m.get("rot") is not None and m["rot"]["dims"]:
        pos = torch.arange(T)
        q = rotate(q, pos, m["rot"]["base"], m["rot"]["dims"])
        k = rotate(k, pos, m["rot"]["base"], m["rot"]["dims"])
    v = unit(v, eps)                                   # each head's value by its own root mean square
    rep = H // G
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihe,jhe->hij", q, k) * m["scale"]
    size = m["mask"]["size"] if m.get("mask") is not None else T          # no mask: every earlier key
    s = s.masked_fill(~window_mask(T, size)[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhe->ihe", p, v).reshape(T, H * dv)
    return o @ w[f"{pre}.o"].T


def causal_conv(x, weight, bias):
    """x [T, C]; weight [C, taps], the last column is the current token's; zeros before the start."""
    T, C = x.shape
    taps = weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x])
    out = bias.expand(T, C).clone()
    for j in range(taps):
        out = out + padded[j:j + T] * weight[:, j]
    return out


def state_space(h, w, pre, m, eps):
    """The selective state-space mixer: per head a state S [N, P] with
    S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T and y_t = S_t^T C_t + D x_t."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    u = h @ w[f"{pre}.in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[f"{pre}.conv"], w[f"{pre}.conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[f"{pre}.dt_bias"])                   # [T, H]
    decay = torch.exp(-torch.exp(w[f"{pre}.A_log"]) * dt)       # [T, H]
    per = H // G
    Bh, Ch = B.repeat_interleave(per, dim=1), C.repeat_interleave(per, dim=1)   # head h reads group h // per
    y = torch.zeros(T, H, P, dtype=h.dtype)
    S = torch.zeros(H, N, P, dtype=h.dtype)
    for t in range(T):                                        # all heads at once, one token at a time
        S = decay[t, :, None, None] * S + dt[t, :, None, None] * Bh[t, :, :, None] * x[t, :, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, Ch[t]) + w[f"{pre}.D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)                          # the gate comes before the norm
    parts = m["norm_groups"]
    y = unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[f"{pre}.norm"]
    return y @ w[f"{pre}.o"].T


# ------------------------------------------------------------------ feed-forwards

def dense_ff(h, w, pre):
    p, q = w[f"{pre}.act"][0], w[f"{pre}.act"][1]
    return xielu(h @ w[f"{pre}.up"].T, p, q) @ w[f"{pre}.down"].T


def gated_ff(h, w, pre):
    return (silu(h @ w[f"{pre}.gate"].T) * (h @ w[f"{pre}.up"].T)) @ w[f"{pre}.down"].T


def route(h, w, pre, r):
    """(indices [T, top], weights [T, top]) of the chosen experts; indices >= experts are the
    identity experts."""
    s = torch.softmax(h @ w[f"{pre}.router"].T, dim=-1)
    idx = torch.topk(s + w[f"{pre}.correction"], r["top"], dim=-1).indices
    return idx, torch.gather(s, 1, idx) * r.get("scale", 1.0)


def expert_mixture(h, w, pre, mlp):
    r = mlp["router"]
    idx, wt = route(h, w, pre, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t]):
            out[t] += a * (h[t] if e >= r["experts"] else gated_ff(h[t:t + 1], w, f"{pre}.e{e}")[0])
    if mlp.get("shared") is not None:
        out = out + gated_ff(h, w, f"{pre}.shared")
    return out


def feed_forward(h, w, pre, mlp):
    if mlp["kind"] == "dense":
        return dense_ff(h, w, pre)
    if mlp["kind"] == "moe":
        return expert_mixture(h, w, pre, mlp)
    raise ValueError(mlp["kind"])


# ------------------------------------------------------------------ the model

def layer(x, w, i, L, eps):
    h = scalar_norm(x, w[f"l{i}.norm1"], eps)
    mix = {"attention": attention, "mamba2": state_space}[L["type"]](h, w, f"l{i}.mix", L["mixer"], eps)
    if L.get("mlp") is not None:
        mix = mix + feed_forward(h, w, f"l{i}.mlp", L["mlp"])
    return x + mix


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and the stream after every layer)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    after = []
    for i, L in enumerate(cfg["layers"]):
        x = layer(x, w, i, L, eps)
        after.append(x)
    logits = scalar_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits


def generate_greedy(cfg, w, prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        out.append(int(forward(cfg, w, toks)[-1].argmax()))
        toks.append(out[-1])
    return out
