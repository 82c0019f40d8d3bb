"""Small Dabevik configurations and seeded weights for the tests. The sizes differ from one
another in everything that can differ: heads against kv heads (ratio 2, 1, 4), key size against
value size, heads x size against the width, windows shorter and longer than a cache page (64),
kept first tokens (none, a few, more than the window and more than a page), taps (3, 1, 5), a
layer without feed-forward, layers that run with another layer's tensors, a feed-forward narrower
and wider than the model.
"""
import json
from pathlib import Path

import torch


def attention(heads, kv_heads, dim, vdim, scale, size, keep_first):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "mask": {"size": size, "keep_first": keep_first}}


def layer(mixer, ff, weights_of=None):
    e = {"type": "attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


def config(vocab, width, max_positions, scale, eps, taps, layers):
    return {"architecture": "Dabevik", "vocab": vocab, "width": width, "max_positions": max_positions,
            "embedding": {"scale": scale}, "norm": {"eps": eps}, "canon": {"taps": taps}, "layers": layers}


_A = attention(4, 2, 16, 24, 0.3, 9, 2)
_B1 = attention(6, 6, 32, 32, 0.11, 70, 0)
_B2 = attention(3, 1, 32, 16, 0.2, 1000, 0)
_C1 = attention(8, 2, 64, 64, 0.09, 150, 5)
_C2 = attention(2, 2, 64, 128, 0.15, 33, 70)

SMALL = {
    # a layer with everything, a layer without feed-forward, and the first layer's tensors once more
    "X": config(97, 64, 512, 7.5, 1e-6, 3, [layer(_A, 80), layer(_A, None), layer(_A, 80, weights_of=0)]),
    # one tap (no state), a window that crosses a page border, no kept tokens; then all keys in sight
    "Y": config(160, 96, 640, 1.0, 1e-5, 1, [layer(_B1, 48), layer(_B2, 200)]),
    # five taps, a window of several pages with a few kept tokens; kept tokens beyond a page and
    # beyond the window; the second layer's tensors used twice
    "Z": config(211, 128, 1024, 11.0, 3e-6, 5, [layer(_C1, 96), layer(_C2, 160), layer(_C2, 160, weights_of=1)]),
}


def make_weights(cfg, seed):
    """Seeded bfloat16 tensors by the design's names; norms near 1, the talk matrix near the
    identity, everything else of a size that keeps activations of order one."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *shape, std=1.0: torch.randn(*shape, generator=g) * std
    D, t = cfg["width"], {}
    t["embed"] = rn(cfg["vocab"], D, std=1.0 / cfg["embedding"]["scale"])
    t["pos"] = rn(cfg["max_positions"], D, std=0.3)
    t["final.norm"] = 1 + rn(D, std=0.1)
    for i, L in enumerate(cfg["layers"]):
        if L.get("weights_of") is not None:
            continue
        m, p = L["mixer"], f"l{i}."
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        t[p + "norm1"], t[p + "norm1b"] = 1 + rn(D, std=0.1), 1 + rn(D, std=0.1)
        t[p + "canon1"] = rn(D, cfg["canon"]["taps"], std=0.3)
        for name, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
            t[p + "mix." + name] = rn(rows, D, std=D ** -0.5)
            t[p + "mix." + name + ".b"] = rn(rows, std=0.2)
        t[p + "mix.q.norm"], t[p + "mix.k.norm"] = 1 + rn(H * d, std=0.1), 1 + rn(G * d, std=0.1)
        t[p + "mix.talk"] = torch.eye(H) + rn(H, H, std=0.3)
        t[p + "mix.o"], t[p + "mix.o.b"] = rn(D, H * dv, std=(H * dv) ** -0.5), rn(D, std=0.2)
        if L["mlp"] is not None:
            F = L["mlp"]["ff"]
            t[p + "norm2"], t[p + "norm2b"] = 1 + rn(D, std=0.1), 1 + rn(D, std=0.1)
            t[p + "canon2"] = rn(D, cfg["canon"]["taps"], std=0.3)
            t[p + "mlp.up"], t[p + "mlp.down"] = rn(F, D, std=D ** -0.5), rn(D, F, std=F ** -0.5)
            t[p + "mlp.act"] = torch.tensor([0.7, 0.4, -0.2, 0.1]) + rn(4, std=0.05)
    return {k: v.to(torch.bfloat16) for k, v in t.items()}


def write_model(cfg, folder, seed):
    from lumenllm_b200.weights.safetensors_io import write_file
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_file(folder / "model.safetensors", make_weights(cfg, seed))
    return folder
