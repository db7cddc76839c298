"""Mubasun: typed configuration and its layout as parts.

A decoder whose layers are listed one by one in ``config.json``.  A learned vector per position is added to the
embedded token; a layer norms the stream once and adds the sum of its two sublayers, which both read that normed row:
``h = norm(x); x += mixer(h) + ff(h)``; every norm is an RMS norm taken in groups.

    {"architecture": "Mubasun", "vocab": V, "width": W, "max_positions": P, "norm": {"eps": e, "groups": g},
     "layers": [
       {"type": "attention",
        "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"} (optional), "kv_from": j (optional)},
        "mlp": {"kind": "dense", "ff"}
             | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "identity", "top", "scale"},
                "shared": {"ff"} (optional)}
             | null}]}

``attention``: grouped-query softmax attention without biases and without a rotation. Queries and keys pass an RMS
norm over their whole projection (all heads at once). A penalty ``slope_h * (i - j)`` is subtracted from the score of
query position i and key position j, ``slope_h = 2^(-8 (h + 1) / heads)``; ``mask.size`` is a sliding window (absent:
every earlier position). The concatenated heads are multiplied by ``sigmoid(W_g h)`` before the output product. With
``kv_from`` the layer has no keys and values and reads those of layer j.

Feed-forwards: ``dense`` is down(xIELU(up(h))) with two learned numbers per layer; ``moe`` is a router (softmax over
experts and identity experts; the choice adds a learned correction to the scores, the weights are the scores times
``router.scale``, with no renormalisation over the chosen ones), experts down(silu(gate(h)) * up(h)), identity experts
(an entry that contributes weight * h and owns no parameters) and a shared expert of the same form scaled by
sigmoid(w . h).

Checkpoint names: ``embed``, ``pos``, ``final.norm``, ``head``; layer i: ``l<i>.norm1``, ``l<i>.mix.q|k|v|g|o``,
``l<i>.mix.q.norm``, ``l<i>.mix.k.norm``, ``l<i>.mlp.up|down|act`` or ``l<i>.mlp.router``, ``l<i>.mlp.correction``,
``l<i>.mlp.e<n>.gate|up|down``, ``l<i>.mlp.shared.gate|up|down|sg``.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Dict, List, Optional, Tuple

from ..parts.spec import EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .base import Architecture, ModelConfig, as_float, as_int, register_architecture

LAYER_TYPES = ("attention",)
MLP_KINDS = ("dense", "moe")


def _obj(v: Any, what: str) -> Dict[str, Any]:
    if not isinstance(v, dict):
        raise TypeError(f"{what} must be an object, got {v!r}")
    return v


def distance_slopes(heads: int) -> Tuple[float, ...]:
    """The design's slope per head: 2^(-8 (h + 1) / heads), h = 0 .. heads - 1."""
    return tuple(2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads))


@dataclasses.dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int] = None
    kv_from: Optional[int] = None

    @classmethod
    def parse(cls, m: Dict[str, Any]) -> "AttentionConfig":
        mask = m.get("mask")
        size = None if mask is None else _obj(mask, "mixer.mask").get("size")
        src = m.get("kv_from")
        return cls(heads=as_int(m.get("heads")), kv_heads=as_int(m.get("kv_heads")), dim=as_int(m.get("dim")),
                   vdim=as_int(m.get("vdim")), scale=as_float(m.get("scale")),
                   window=None if size is None else as_int(size), kv_from=None if src is None else as_int(src))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out

    def problems(self, where: str) -> List[str]:
        p: List[str] = []
        for name in ("heads", "kv_heads", "dim", "vdim"):
            if getattr(self, name) < 1:
                p.append(f"{where}.{name} must be >= 1 (got {getattr(self, name)})")
        if self.kv_heads >= 1 and self.heads % self.kv_heads:
            p.append(f"{where}: {self.kv_heads} kv_heads do not divide {self.heads} heads")
        if not (self.scale > 0 and math.isfinite(self.scale)):
            p.append(f"{where}.scale must be > 0 (got {self.scale})")
        if self.window is not None and self.window < 1:
            p.append(f"{where}.mask.size must be >= 1 (got {self.window})")
        return p


@dataclasses.dataclass(frozen=True)
class MlpConfig:
    kind: str
    ff: int                          # inner width: of the dense feed-forward, or of one expert
    experts: int = 0
    identity: int = 0
    top: int = 0
    route_scale: float = 1.0
    shared_ff: Optional[int] = None  # inner width of the shared expert; None: no shared expert

    @classmethod
    def parse(cls, v: Any) -> Optional["MlpConfig"]:
        if v is None:
            return None
        v = _obj(v, "mlp")
        kind = v.get("kind")
        if kind not in MLP_KINDS:
            raise ValueError(f"mlp.kind must be one of {MLP_KINDS} (got {kind!r})")
        if kind == "dense":
            return cls(kind, as_int(v.get("ff")))
        r = _obj(v.get("router"), "mlp.router")
        shared = v.get("shared")
        return cls(kind, as_int(_obj(v.get("expert"), "mlp.expert").get("ff")), experts=as_int(r.get("experts")),
                   identity=as_int(r.get("identity", 0)), top=as_int(r.get("top")),
                   route_scale=as_float(r.get("scale", 1.0)),
                   shared_ff=None if shared is None else as_int(_obj(shared, "mlp.shared").get("ff")))

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        out: Dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff},
                               "router": {"experts": self.experts, "identity": self.identity, "top": self.top,
                                          "scale": self.route_scale}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out

    def problems(self, where: str) -> List[str]:
        p: List[str] = []
        if self.ff < 1:
            p.append(f"{where}: the inner width must be >= 1 (got {self.ff})")
        if self.kind == "moe":
            if self.experts < 1 or self.identity < 0:
                p.append(f"{where}.router: experts >= 1 and identity >= 0 (got {self.experts}, {self.identity})")
            elif not (1 <= self.top <= min(16, self.experts + self.identity)):
                p.append(f"{where}.router.top must lie between 1 and min(16, experts + identity) (got {self.top})")
            if not math.isfinite(self.route_scale):
                p.append(f"{where}.router.scale must be finite (got {self.route_scale})")
            if self.shared_ff is not None and self.shared_ff < 1:
                p.append(f"{where}.shared.ff must be >= 1 (got {self.shared_ff})")
        return p


@dataclasses.dataclass(frozen=True)
class LayerConfig:
    type: str
    attention: AttentionConfig
    mlp: Optional[MlpConfig]

    @classmethod
    def parse(cls, v: Any) -> "LayerConfig":
        v = _obj(v, "a layer")
        kind = v.get("type")
        if kind not in LAYER_TYPES:
            raise ValueError(f"layer type must be one of {LAYER_TYPES} (got {kind!r})")
        return cls(kind, AttentionConfig.parse(_obj(v.get("mixer"), "mixer")), MlpConfig.parse(v.get("mlp")))

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.attention.to_dict(),
                "mlp": None if self.mlp is None else self.mlp.to_dict()}


def _layers(v: Any) -> Tuple[LayerConfig, ...]:
    if not isinstance(v, (list, tuple)) or not v:
        raise TypeError("layers must be a list with at least one entry")
    return tuple(LayerConfig.parse(x) for x in v)


def _norm(v: Any) -> Tuple[float, int]:
    v = _obj(v, "norm")
    return as_float(v.get("eps")), as_int(v.get("groups", 1))


def _req(conv, key=None):
    md = {"convert": conv, "required": True}
    if key:
        md["key"] = key
    return dataclasses.field(default=None, metadata=md)


@dataclasses.dataclass(frozen=True)
class MubasunConfig(ModelConfig):
    vocab: int = _req(as_int)
    width: int = _req(as_int)
    max_positions: int = _req(as_int)
    layers: Tuple[LayerConfig, ...] = _req(_layers)
    norm: Tuple[float, int] = _req(_norm)                      # (eps, groups)
    architecture: str = dataclasses.field(default="Mubasun", metadata={"convert": str})
    initializer_range: float = dataclasses.field(default=0.02, metadata={"convert": as_float})

    @classmethod
    def architecture_names(cls) -> Tuple[str, ...]:
        return ("Mubasun",)

    @property
    def norm_eps(self) -> float:
        return self.norm[0]

    @property
    def norm_groups(self) -> int:
        return self.norm[1]

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
                "layers": [l.to_dict() for l in self.layers], "initializer_range": self.initializer_range}

    def problems(self) -> List[str]:
        p: List[str] = []
        if self.vocab < 1 or self.width < 1:
            p.append(f"vocab and width must be >= 1 (got {self.vocab}, {self.width})")
        if self.max_positions < 1:
            p.append(f"max_positions must be >= 1 (got {self.max_positions})")
        if not self.norm_eps > 0:
            p.append(f"norm.eps must be > 0 (got {self.norm_eps})")
        if self.norm_groups < 1 or (self.width >= 1 and self.width % self.norm_groups):
            p.append(f"norm.groups must be >= 1 and divide the width {self.width} (got {self.norm_groups})")
        if not (1 <= len(self.layers) <= 1024):
            p.append(f"between 1 and 1024 layers (got {len(self.layers)})")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            a = layer.attention
            p.extend(a.problems(where + ".mixer"))
            if layer.mlp is not None:
                p.extend(layer.mlp.problems(where + ".mlp"))
            if a.kv_from is not None:
                j = a.kv_from
                src = self.layers[j].attention if 0 <= j < i else None
                if src is None or src.kv_from is not None:
                    p.append(f"{where}.mixer.kv_from must name an earlier layer with keys and values of its own (got {j})")
                elif (src.kv_heads, src.dim, src.vdim) != (a.kv_heads, a.dim, a.vdim):
                    p.append(f"{where}.mixer.kv_from: layer {j}'s kv_heads, dim and vdim differ from this layer's")
        if not self.initializer_range > 0:
            p.append(f"initializer_range must be > 0 (got {self.initializer_range})")
        return p


def _attention_part(cfg: MubasunConfig, a: AttentionConfig, pre: str):
    shared = a.kv_from is not None
    spec = PartSpec("attention", {
        "hidden_size": cfg.width, "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
        "scale": a.scale, "softcap": None, "window": a.window, "bias": False,
        "qk_norm": {"eps": cfg.norm_eps, "over": "projection"}, "distance_slopes": distance_slopes(a.heads),
        "out_gate": True, "shared_kv": shared, "position": PartSpec("none", {"head_dim": a.dim})})
    names = {"mixer.q_proj": pre + "q", "mixer.o_proj": pre + "o", "mixer.g_proj": pre + "g", "mixer.q_norm": pre + "q.norm"}
    if not shared:
        names.update({"mixer.k_proj": pre + "k", "mixer.v_proj": pre + "v", "mixer.k_norm": pre + "k.norm"})
    return spec, names


def _gated_names(local: str, pre: str) -> Dict[str, str]:
    return {f"{local}gate_proj": pre + "gate", f"{local}up_proj": pre + "up", f"{local}down_proj": pre + "down"}


def _mlp_part(cfg: MubasunConfig, m: MlpConfig, pre: str):
    W = cfg.width
    if m.kind == "dense":
        spec = PartSpec("mlp", {"hidden_size": W, "intermediate_size": m.ff, "activation": "xielu"})
        return spec, {"ff.up_proj": pre + "up", "ff.down_proj": pre + "down", "ff.act_params": pre + "act"}
    shared = None
    names = {"ff.router": pre + "router", "ff.correction": pre + "correction"}
    if m.shared_ff is not None:
        shared = PartSpec("gated_mlp", {"hidden_size": W, "intermediate_size": m.shared_ff, "activation": "silu"})
        names.update(_gated_names("ff.shared.", pre + "shared."))
        names["ff.shared_gate"] = pre + "shared.sg"
    for e in range(m.experts):
        names.update(_gated_names(f"ff.experts.{e}.", f"{pre}e{e}."))
    spec = PartSpec("routed_experts", {
        "hidden_size": W, "intermediate_size": m.ff, "experts": m.experts, "top": m.top, "activation": "silu",
        "score": "softmax", "renormalize": False, "weight_on": "output", "correction": True, "identity": m.identity,
        "route_scale": m.route_scale, "shared": shared, "shared_gate": shared is not None})
    return spec, names


def mubasun_spec(cfg: MubasunConfig) -> ModelSpec:
    W = cfg.width
    norm = PartSpec("group_rmsnorm", {"size": W, "eps": cfg.norm_eps, "groups": cfg.norm_groups})
    layers, schedule = [], []
    for i, lc in enumerate(cfg.layers):
        pre = f"l{i}."
        tensors = {"norms.pre.weight": pre + "norm1"}
        mixer, names = _attention_part(cfg, lc.attention, pre + "mix.")
        tensors.update(names)
        ff = None
        if lc.mlp is not None:
            ff, names = _mlp_part(cfg, lc.mlp, pre + "mlp.")
            tensors.update(names)
        layers.append(LayerSpec(block=PartSpec("parallel", {}), mixer=mixer, feed_forward=ff, norms={"pre": norm},
                                tensors=tensors))
        if lc.attention.kv_from is not None:     # the cache line of the layer whose keys and values it reads
            schedule.append(ScheduleEntry(layer=i, cache=lc.attention.kv_from, writes_cache=False))
        else:
            schedule.append(ScheduleEntry(layer=i, cache=i, writes_cache=True))
    return ModelSpec(
        name="Mubasun", hidden_size=W,
        embedding=EmbeddingSpec(cfg.vocab, W, 1.0, "embed", position_tensor="pos", n_positions=cfg.max_positions),
        layers=tuple(layers), schedule=tuple(schedule),
        head=HeadSpec(cfg.vocab, W, tied=False, tensor="head", softcap=None, norm=norm, norm_tensor="final.norm"),
        max_positions=cfg.max_positions, stop_ids=(), init_std=cfg.initializer_range, init_norm_std=0.1)


MUBASUN = register_architecture(Architecture(
    name="Mubasun", config_cls=MubasunConfig, build_spec=mubasun_spec, aliases=("mubasun",)))
