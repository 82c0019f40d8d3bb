"""Small Rasezen configurations and seeded weights for the tests. The sizes differ from one
another in everything that can differ: heads against kv heads (ratio 2, 1, 3), key size against
value size, rotation over a part of a head, over all of it and none, windows shorter and longer
than a cache page (64) and none; state-space layers with one group and several, state sizes
that fit one thread and that are spread over two and four, one to five taps, one norm part and
several; dense feed-forwards narrower and wider than the model, expert mixtures with and without
identity experts and shared expert, one choice and several, and layers without feed-forward.
"""
import json
from pathlib import Path

import torch


def attention(heads, kv_heads, dim, vdim, scale, size=None, rot=None, base=10000.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    if rot is not None:
        m["rot"] = {"base": base, "dims": rot}
    return m


def state_space(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, identity, top, scale, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff},
         "router": {"experts": experts, "identity": identity, "scale": scale, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp):
    return {"type": "mamba2" if "state" in mixer else "attention", "mixer": mixer, "mlp": mlp}


def config(vocab, width, eps, layers):
    return {"architecture": "Rasezen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


SMALL = {
    # a short window, rotation over half a head, values wider than keys; one group, one norm part,
    # experts with one identity expert and a shared expert; a layer without feed-forward whose
    # window crosses a page border; a state spread over two threads
    "X": config(97, 64, 1e-6, [
        layer(attention(4, 2, 16, 24, 0.3, size=9, rot=8), dense(80)),
        layer(state_space(4, 16, 8, 1, 4, 1), moe(24, 4, 1, 2, 1.5, shared=32)),
        layer(attention(4, 4, 16, 8, 0.25, size=70, rot=16, base=500.0), None),
        layer(state_space(6, 8, 40, 3, 2, 3), dense(48))]),
    # no window and no rotation; one choice among experts without identity or shared expert; one
    # tap (no convolution state); a feed-forward wider than the model
    "Y": config(160, 96, 1e-5, [
        layer(attention(6, 6, 32, 32, 0.11, rot=32, base=1e6), moe(40, 3, 0, 1, 1.0)),
        layer(state_space(2, 24, 16, 2, 1, 4), None),
        layer(attention(3, 1, 32, 16, 0.2), dense(200)),
        layer(state_space(3, 32, 12, 1, 5, 2), moe(16, 5, 2, 3, 0.7, shared=8))]),
    # head sizes that the tensor-core attention kernels take (64, 128) with windows of several
    # pages and of less than one; a state spread over four threads; more identity experts than
    # choices
    "Z": config(211, 128, 3e-6, [
        layer(attention(4, 2, 64, 64, 0.12, size=150, rot=32), moe(48, 6, 3, 2, 2.0, shared=64)),
        layer(state_space(4, 32, 100, 2, 3, 2), dense(96)),
        layer(attention(2, 1, 128, 128, 0.09, size=33, rot=128, base=1e5), dense(160))]),
}


def make_weights(cfg, seed):
    """Seeded bfloat16 tensors by the design's names, of a size that keeps activations of order
    one; the router's rows are large enough for choices to be clear of ties."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *shape, std=1.0: torch.randn(shape, generator=g) * std
    D, t = cfg["width"], {}
    t["embed"] = rn(cfg["vocab"], D)
    t["head"] = rn(cfg["vocab"], D, std=D ** -0.5)
    t["final.norm"] = torch.tensor(1.0) + rn(std=0.1)
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}."
        t[p + "norm1"] = torch.tensor(1.0) + rn(std=0.1)
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for name, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                t[p + "mix." + name] = rn(rows, D, std=D ** -0.5)
                t[p + "mix." + name + ".b"] = rn(rows, std=0.2)
            t[p + "mix.q.norm"], t[p + "mix.k.norm"] = 1 + rn(H * d, std=0.1), 1 + rn(G * d, std=0.1)
            t[p + "mix.o"] = rn(D, H * dv, std=(H * dv) ** -0.5)
        else:
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, C = H * P, H * P + 2 * G * N
            t[p + "mix.in"] = rn(inner + C + H, D, std=D ** -0.5)
            t[p + "mix.conv"], t[p + "mix.conv.b"] = rn(C, m["conv"], std=0.5), rn(C, std=0.2)
            t[p + "mix.dt_bias"], t[p + "mix.A_log"], t[p + "mix.D"] = rn(H, std=0.5), rn(H, std=0.5) - 1.0, 1 + rn(H, std=0.3)
            t[p + "mix.norm"] = 1 + rn(inner, std=0.1)
            t[p + "mix.o"] = rn(D, inner, std=inner ** -0.5)
        mlp = L["mlp"]
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            F = mlp["ff"]
            t[p + "mlp.up"], t[p + "mlp.down"] = rn(F, D, std=D ** -0.5), rn(D, F, std=F ** -0.5)
            t[p + "mlp.act"] = torch.tensor([0.3, -0.2]) + rn(2, std=0.2)
        else:
            r, F = mlp["router"], mlp["expert"]["ff"]
            E = r["experts"] + r["identity"]
            t[p + "mlp.router"], t[p + "mlp.correction"] = rn(E, D, std=3.0 * D ** -0.5), rn(E, std=0.1)
            names = [f"e{e}" for e in range(r["experts"])] + (["shared"] if mlp.get("shared") else [])
            for name in names:
                Fe = mlp["shared"]["ff"] if name == "shared" else F
                t[f"{p}mlp.{name}.gate"], t[f"{p}mlp.{name}.up"] = rn(Fe, D, std=D ** -0.5), rn(Fe, D, std=D ** -0.5)
                t[f"{p}mlp.{name}.down"] = rn(D, Fe, std=Fe ** -0.5)
    return {k: v.to(torch.bfloat16) for k, v in t.items()}


def write_model(cfg, folder, seed):
    from lumenllm_b200.weights.safetensors_io import write_file
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_file(folder / "model.safetensors", make_weights(cfg, seed))
    return folder
