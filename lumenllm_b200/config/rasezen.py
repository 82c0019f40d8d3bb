"""Typed configuration of Rasezen (config.json key "architecture": "Rasezen").

A small decoder whose layers are parallel blocks, x <- x + (mixer(n) + ff(n)) with n = norm(x):
one RMS norm a layer, with ONE number as its weight, read by both sublayers. A layer's mixer is
either attention (biased projections, an RMS norm over the whole query and the whole key
projection, rotation of part of every head, values divided by their root mean square, a sliding
window, ordinary softmax) or a selective state-space recurrence ("mamba2": input projection,
short causal convolution with SiLU, a decaying matrix state per head, a gate, an RMS norm in
equal parts, output projection). Its feed-forward is dense with the xIELU activation, or a
mixture of small gated experts (some of which hand their input on unchanged) chosen by a softmax
router with a correction of the choice, plus a shared expert; or the layer has none. The head is
a matrix of its own.

config.json gives every size and every constant, layer by layer; nothing here is a default for
them. There is no limit on positions in the design: `max_positions`, if config.json has it,
bounds a sequence, else only the cache does.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .dabevik import _int, _num, _obj
from .registry import eos_ids_of, register_architecture
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

UNBOUNDED_POSITIONS = 1 << 30


@dataclass(frozen=True)
class RasezenAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int          # keys a query sees behind it, itself included; 0: all of them
    rot_dims: int        # rotated values of a head; 0: none
    rot_base: float

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "RasezenAttention":
        window = _int(_obj(m, "mask", where), "size", where + "mask.") if m.get("mask") is not None else 0
        rot = m.get("rot")
        a = cls(heads=_int(m, "heads", where), kv_heads=_int(m, "kv_heads", where), dim=_int(m, "dim", where),
                vdim=_int(m, "vdim", where), scale=_num(m, "scale", where), window=window,
                rot_dims=_int(rot, "dims", where + "rot.", 0) if rot is not None else 0,
                rot_base=_num(rot, "base", where + "rot.") if rot is not None else 1.0)
        if a.heads % a.kv_heads:
            raise ConfigError(f"config.json: {where}{a.heads} heads are not a multiple of {a.kv_heads} kv_heads")
        if a.rot_dims % 2 or a.rot_dims > a.dim:
            raise ConfigError(f"config.json: {where}rot.dims {a.rot_dims} must be even and at most dim {a.dim}")
        return a

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return d


@dataclass(frozen=True)
class RasezenStateSpace:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "RasezenStateSpace":
        s = cls(*(_int(m, k, where) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")))
        if s.heads % s.groups:
            raise ConfigError(f"config.json: {where}{s.heads} heads are not a multiple of {s.groups} groups")
        if (s.heads * s.vdim) % s.norm_groups:
            raise ConfigError(f"config.json: {where}{s.heads * s.vdim} channels do not divide into "
                              f"{s.norm_groups} norm_groups")
        return s

    def to_dict(self) -> dict:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups,
                "conv": self.conv, "norm_groups": self.norm_groups}


@dataclass(frozen=True)
class RasezenMlp:
    kind: str                       # "dense" or "moe"
    ff: int                         # dense: its width; moe: an expert's width
    experts: int = 0
    identity: int = 0
    top: int = 0
    scale: float = 1.0
    shared_ff: int = 0              # 0: no shared expert

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "RasezenMlp":
        kind = m.get("kind")
        if kind == "dense":
            return cls("dense", _int(m, "ff", where))
        if kind == "moe":
            r = _obj(m, "router", where)
            shared = m.get("shared")
            x = cls("moe", _int(_obj(m, "expert", where), "ff", where + "expert."),
                    experts=_int(r, "experts", where + "router."),
                    identity=_int(r, "identity", where + "router.", 0) if "identity" in r else 0,
                    top=_int(r, "top", where + "router."), scale=_num(r, "scale", where + "router.") if "scale" in r else 1.0,
                    shared_ff=_int(shared, "ff", where + "shared.") if shared is not None else 0)
            if x.top > x.experts + x.identity:
                raise ConfigError(f"config.json: {where}router.top {x.top} exceeds the {x.experts + x.identity} experts")
            return x
        raise ConfigError(f"config.json: {where}kind {kind!r} is not a feed-forward of this design "
                          "(known: 'dense', 'moe')")

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d = {"kind": "moe", "expert": {"ff": self.ff},
             "router": {"experts": self.experts, "identity": self.identity, "scale": self.scale, "top": self.top}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class RasezenLayer:
    type: str                                   # "attention" or "mamba2"
    mixer: Any                                  # RasezenAttention or RasezenStateSpace
    mlp: Optional[RasezenMlp]


@register_architecture("Rasezen")
@dataclass(frozen=True)
class RasezenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[RasezenLayer, ...]
    max_positions: int = UNBOUNDED_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    MIXERS = {"attention": RasezenAttention, "mamba2": RasezenStateSpace}

    @classmethod
    def from_dict(cls, d: dict) -> "RasezenConfig":
        for k in ("vocab", "width", "norm", "layers"):
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
            if kind not in cls.MIXERS:
                raise ConfigError(f"config.json: {where}type {kind!r} is not a mixer of this design "
                                  f"(known: {sorted(cls.MIXERS)})")
            mixer = cls.MIXERS[kind].from_dict(_obj(e, "mixer", where), where + "mixer.")
            mlp = e.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"config.json: {where}mlp must be null or an object, got {mlp!r}")
            layers.append(RasezenLayer(kind, mixer, None if mlp is None else RasezenMlp.from_dict(mlp, where + "mlp.")))
        known = ("architecture", "vocab", "width", "norm", "layers", "max_positions", "eos_token_id", "torch_dtype")
        cfg = cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""),
                  norm_eps=_num(_obj(d, "norm", ""), "eps", "norm."), layers=tuple(layers),
                  max_positions=_int(d, "max_positions", "") if "max_positions" in d else UNBOUNDED_POSITIONS,
                  eos_token_ids=eos_ids_of(d.get("eos_token_id"), "config.json"),
                  extra={k: v for k, v in d.items() if k not in known})
        if cfg.norm_eps < 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        return cfg

    def to_dict(self) -> dict:
        d = {"architecture": "Rasezen", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                        for l in self.layers]}
        if self.max_positions != UNBOUNDED_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ------------------------------------------------------------ meaning
    def model_spec(self) -> ModelSpec:
        D, eps = self.width, self.norm_eps

        def norm(name):
            return PartSpec("rmsnorm", {"size": D, "eps": eps, "weight_offset": 0.0, "tensor": name, "scalar": True})

        specs = []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}", l.mixer
            if l.type == "attention":
                position = (PartSpec("rotary", {"head_dim": m.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                                                "wide_frequencies": True})
                            if m.rot_dims else PartSpec("none", {}))
                mixer = PartSpec("wide_norm_attention", {
                    "hidden_size": D, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                    "value_dim": m.vdim, "softmax_scale": m.scale, "window": m.window, "norm_eps": eps,
                    "value_norm": True, "position": position}, prefix=f"{p}.mix")
            else:
                mixer = PartSpec("mamba2", {
                    "hidden_size": D, "num_heads": m.heads, "head_dim": m.vdim, "state_size": m.state,
                    "groups": m.groups, "taps": m.conv, "norm_groups": m.norm_groups, "norm_eps": eps},
                    prefix=f"{p}.mix")
            ffn = None
            if l.mlp is not None and l.mlp.kind == "dense":
                ffn = PartSpec("xielu_mlp", {"hidden_size": D, "intermediate_size": l.mlp.ff}, prefix=f"{p}.mlp")
            elif l.mlp is not None:
                x = l.mlp
                ffn = PartSpec("routed_experts", {
                    "hidden_size": D, "expert_size": x.ff, "num_experts": x.experts, "identity_experts": x.identity,
                    "top": x.top, "scale": x.scale, "shared_size": x.shared_ff}, prefix=f"{p}.mlp")
            specs.append(LayerSpec("parallel", mixer, ffn, {"input": norm(f"{p}.norm1")}, prefix=p))
        spec = ModelSpec(
            architecture="Rasezen", vocab_size=self.vocab, hidden_size=D, max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": D, "tensor": "embed"}),
            layers=tuple(specs), schedule=tuple(ScheduleEntry(i) for i in range(len(specs))),
            final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": D, "tensor": "head"}),
            eos_token_ids=self.eos_token_ids)
        spec.validate()
        return spec
