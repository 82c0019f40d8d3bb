"""A plain, slow implementation of the Dabevik decoder in float32 on the CPU, written from the
design's equations, one function per mechanism. It shares no code with the library: whole
sequences only, no cache, no batching. The tests compare the engine with it.

Notation: a sequence of T tokens, width D, H query heads, G key/value heads, query/key size d,
value size dv; rms(x) = sqrt(mean(x^2) + eps).
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
        t = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        out[name] = t
    return out


def load_model(folder):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {k: v.to(F) for k, v in read_safetensors(folder / "model.safetensors").items()}
    return cfg, w


def owner_of(cfg, i):
    """Index of the layer whose tensors layer i uses."""
    seen = set()
    while "weights_of" in cfg["layers"][i] and cfg["layers"][i]["weights_of"] is not None:
        if i in seen:
            raise ValueError("layers name each other in a circle")
        seen.add(i)
        i = int(cfg["layers"][i]["weights_of"])
    return i


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def embed(tokens, table, scale, pos_table, positions):
    return table[tokens] * scale + pos_table[positions]


def input_convolution(h, wc):
    """h [T, D], wc [D, taps]: h_t + sum_j wc[:, j] * h_(t - taps + 1 + j), zeros before t = 0."""
    T, D = h.shape
    taps = wc.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += wc[:, j] * h[s]
    return out


def sees(i, j, size, keep_first):
    return j <= i and (i - j < size or j < keep_first)


def talking_attention(h, w, pre, m, eps):
    """The attention mixer on its (already convolved) input h [T, D]; m is the layer's 'mixer'
    entry. Softmax weights of all heads are mixed by the talk matrix before they meet the values."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size, keep = m["mask"]["size"], m["mask"]["keep_first"]
    q = h @ w[pre + "q"].T + w[pre + "q.b"]
    k = h @ w[pre + "k"].T + w[pre + "k.b"]
    v = h @ w[pre + "v"].T + w[pre + "v.b"]
    q = rms_norm(q, w[pre + "q.norm"], eps).view(T, H, d)       # one norm over the whole projection
    k = rms_norm(k, w[pre + "k.norm"], eps).view(T, G, d)
    v = v.view(T, G, dv)
    per = H // G
    probs = torch.zeros(H, T, T)
    for hh in range(H):
        g = hh // per
        for i in range(T):
            js = [j for j in range(T) if sees(i, j, size, keep)]
            s = (k[js, g] @ q[i, hh]) * m["scale"]
            probs[hh, i, js] = torch.softmax(s, dim=0)
    mixed = torch.einsum("hg,gij->hij", w[pre + "talk"], probs)
    out = torch.zeros(T, H, dv)
    for hh in range(H):
        out[:, hh] = mixed[hh] @ v[:, hh // per]
    return out.reshape(T, H * dv) @ w[pre + "o"].T + w[pre + "o.b"]


def polynorm(z, act, eps):
    a, b, c, e = (float(x) for x in act)
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def dense_ffn(h, w, pre, eps):
    return polynorm(h @ w[pre + "up"].T, w[pre + "act"], eps) @ w[pre + "down"].T


def layer(x, cfg, w, i):
    L = cfg["layers"][i]
    p = f"l{owner_of(cfg, i)}."
    eps = cfg["norm"]["eps"]
    if L["type"] != "attention":
        raise ValueError(f"unknown layer type {L['type']!r}")
    h = input_convolution(rms_norm(x, w[p + "norm1"], eps), w[p + "canon1"])
    x = x + rms_norm(talking_attention(h, w, p + "mix.", L["mixer"], eps), w[p + "norm1b"], eps)
    if L.get("mlp") is not None:
        if L["mlp"]["kind"] != "dense":
            raise ValueError(f"unknown feed-forward kind {L['mlp']['kind']!r}")
        h = input_convolution(rms_norm(x, w[p + "norm2"], eps), w[p + "canon2"])
        x = x + rms_norm(dense_ffn(h, w, p + "mlp.", eps), w[p + "norm2b"], eps)
    return x


def forward(cfg, w, tokens, streams=False):
    """Logits [T, vocab] of a whole sequence; with streams also the residual stream after
    every layer run [layers, T, D]."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = embed(tokens, w["embed"], cfg["embedding"]["scale"], w["pos"], torch.arange(len(tokens)))
    after = []
    for i in range(len(cfg["layers"])):
        x = layer(x, cfg, w, i)
        after.append(x)
    logits = rms_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["embed"].T
    return (logits, torch.stack(after)) if streams else logits


def generate_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]
