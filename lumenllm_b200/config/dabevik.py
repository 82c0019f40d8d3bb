"""Typed configuration of Dabevik (config.json key "architecture": "Dabevik").

A small decoder with learned positions and a scaled, tied embedding. Every layer is
x <- x + norm_b(mixer(conv(norm_a(x)))), then the same around a feed-forward (which a layer may
lack): RMS norms before and after each sublayer, and a short causal convolution over time on
each channel of what a sublayer reads. The mixer is attention without rotation: biased
projections, one RMS norm over the whole query (and key) projection, a sliding window that keeps
the first tokens in sight, and softmax weights mixed across heads before they meet the values.
The feed-forward is up -> PolyNorm -> down. A layer may run with another layer's tensors
("weights_of") and a cache and state of its own.

config.json gives every size and every constant; nothing here is a default for them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .registry import eos_ids_of, register_architecture
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _obj(d, key, where):
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object, got {v!r}")
    return v


def _int(d, key, where, least=1):
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < least:
        raise ConfigError(f"config.json: {where}'{key}' must be an integer of at least {least}, got {v!r}")
    return int(v)


def _num(d, key, where):
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class DabevikAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int          # keys a query sees behind it, itself included
    keep_first: int      # first tokens of a sequence that stay in sight

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "DabevikAttention":
        mask = _obj(m, "mask", where)
        a = cls(heads=_int(m, "heads", where), kv_heads=_int(m, "kv_heads", where), dim=_int(m, "dim", where),
                vdim=_int(m, "vdim", where), scale=_num(m, "scale", where),
                window=_int(mask, "size", where + "mask."), keep_first=_int(mask, "keep_first", where + "mask.", 0))
        if a.heads % a.kv_heads:
            raise ConfigError(f"config.json: {where}{a.heads} heads are not a multiple of {a.kv_heads} kv_heads")
        return a

    def to_dict(self) -> dict:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                "scale": self.scale, "mask": {"size": self.window, "keep_first": self.keep_first}}


@dataclass(frozen=True)
class DabevikLayer:
    type: str
    mixer: DabevikAttention
    ff: Optional[int]                 # width of the dense feed-forward; None: the layer has none
    weights_of: Optional[int] = None  # the layer whose tensors this one uses


@register_architecture("Dabevik")
@dataclass(frozen=True)
class DabevikConfig:
    vocab: int
    width: int
    max_positions: int
    embedding_scale: float
    norm_eps: float
    canon_taps: int
    layers: Tuple[DabevikLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    # ------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: dict) -> "DabevikConfig":
        for k in ("vocab", "width", "max_positions", "embedding", "norm", "canon", "layers"):
            if k not in d:
                raise ConfigError(f"config.json: missing key '{k}'")
        entries = d["layers"]
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = e.get("type")
            if kind != "attention":
                raise ConfigError(f"config.json: {where}type {kind!r} is not a mixer of this design "
                                  "(known: 'attention')")
            mixer = DabevikAttention.from_dict(_obj(e, "mixer", where), where + "mixer.")
            mlp = e.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}mlp must be null or an object of kind 'dense', "
                                      f"got {mlp!r}")
                ff = _int(mlp, "ff", where + "mlp.")
            of = e.get("weights_of")
            if of is not None and (isinstance(of, bool) or not isinstance(of, int) or not 0 <= of < len(entries)
                                   or of == i):
                raise ConfigError(f"config.json: {where}weights_of {of!r} names no other layer")
            layers.append(DabevikLayer(kind, mixer, ff, of))
        cfg = cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""),
                  max_positions=_int(d, "max_positions", ""),
                  embedding_scale=_num(_obj(d, "embedding", ""), "scale", "embedding."),
                  norm_eps=_num(_obj(d, "norm", ""), "eps", "norm."),
                  canon_taps=_int(_obj(d, "canon", ""), "taps", "canon."), layers=tuple(layers),
                  eos_token_ids=eos_ids_of(d.get("eos_token_id"), "config.json"),
                  extra={k: v for k, v in d.items() if k not in (
                      "architecture", "vocab", "width", "max_positions", "embedding", "norm", "canon", "layers",
                      "eos_token_id", "torch_dtype")})
        if cfg.norm_eps < 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        for i in range(len(layers)):
            j = cfg.owner_of(i)
            if (layers[j].mixer, layers[j].ff, layers[j].type) != (layers[i].mixer, layers[i].ff, layers[i].type):
                raise ConfigError(f"config.json: layers[{i}] uses the tensors of layer {j} but has other sizes")
        return cfg

    def to_dict(self) -> dict:
        layers = []
        for l in self.layers:
            e = {"type": l.type, "mixer": l.mixer.to_dict(),
                 "mlp": None if l.ff is None else {"kind": "dense", "ff": l.ff}}
            if l.weights_of is not None:
                e["weights_of"] = l.weights_of
            layers.append(e)
        d = {"architecture": "Dabevik", "vocab": self.vocab, "width": self.width,
             "max_positions": self.max_positions, "embedding": {"scale": self.embedding_scale},
             "norm": {"eps": self.norm_eps}, "canon": {"taps": self.canon_taps}, "layers": layers}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ------------------------------------------------------------ meaning
    def owner_of(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself, unless it names another)."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"config.json: layers name each other's tensors in a circle (layer {i})")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    def model_spec(self) -> ModelSpec:
        D, eps = self.width, self.norm_eps
        owners = sorted({self.owner_of(i) for i in range(len(self.layers))})
        index = {o: k for k, o in enumerate(owners)}

        def norm(name):
            return PartSpec("rmsnorm", {"size": D, "eps": eps, "weight_offset": 0.0, "tensor": name})

        def conv(name):
            return PartSpec("causal_depthwise", {"size": D, "taps": self.canon_taps, "tensor": name})

        specs = []
        for o in owners:
            l, p = self.layers[o], f"l{o}"
            a = l.mixer
            mixer = PartSpec("talking_attention", {
                "hidden_size": D, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
                "value_dim": a.vdim, "softmax_scale": a.scale, "window": a.window, "keep_first": a.keep_first,
                "norm_eps": eps}, prefix=f"{p}.mix")
            ffn = None if l.ff is None else PartSpec(
                "polynorm_mlp", {"hidden_size": D, "intermediate_size": l.ff, "eps": eps}, prefix=f"{p}.mlp")
            norms = {"mixer": norm(f"{p}.norm1"), "mixer_out": norm(f"{p}.norm1b")}
            extras = {"mixer_conv": conv(f"{p}.canon1")}
            if ffn is not None:
                norms.update({"ffn": norm(f"{p}.norm2"), "ffn_out": norm(f"{p}.norm2b")})
                extras["ffn_conv"] = conv(f"{p}.canon2")
            specs.append(LayerSpec("sandwich_conv", mixer, ffn, norms, prefix=p, extras=extras))
        spec = ModelSpec(
            architecture="Dabevik", vocab_size=self.vocab, hidden_size=D, max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": D,
                                                   "scale": self.embedding_scale, "tensor": "embed",
                                                   "position_tensor": "pos",
                                                   "max_positions": self.max_positions}),
            layers=tuple(specs),
            schedule=tuple(ScheduleEntry(index[self.owner_of(i)]) for i in range(len(self.layers))),
            final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": D, "tied_to": "embed",
                                          "own_tensor": False}),
            eos_token_ids=self.eos_token_ids)
        spec.validate()
        return spec
