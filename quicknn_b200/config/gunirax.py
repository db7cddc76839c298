"""Gunirax: typed configuration and its layout as parts.

A decoder whose layers are listed one by one in ``config.json``; a stretch of them may run several times over with
the same weights.  Layers are pre-norm and every norm is a dynamic tanh (``tanh(alpha x) * w + b``).

    {"architecture": "Gunirax", "vocab": V, "width": W, "embedding": {"scale": s}, "norm": {"eps": e},
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [
       {"type": "parallel",
        "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"},
                           "rot": {"base", "dims", "scaling": {"factor", "low", "high", "original"}}},
                  "right": {"heads", "dim", "vdim", "decay": [per head]}},
        "mlp": {"kind": "dense", "ff"}
             | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale", "groups": {"count", "keep"}},
                "shared": {"ff"}}
             | null},
       {"type": "hgrn2", "mixer": {"heads", "dim", "vdim"}, "mlp": ...}]}

``loop``: layers a .. b-1 run n times in a row, every pass with cache lines and states of its own; before every pass but
the first the embedded rows are added to the stream.  ``parallel``: a chunked sigmoid attention whose values are its
keys (left: biases on q and k, an interleaved rotation with frequencies rescaled by wavelength, an RMS norm without
weights per head after the rotation, a bias per head on the scores, weights mixed over the heads, a gate per head)
beside a matrix memory with a fixed decay per head (right); both outputs RMS-normed over the width and averaged.
``hgrn2``: a matrix memory whose forget gate also decides what is written.  Feed-forwards: ``dense`` is
down(silu(gate(h)) * up(h)); ``moe`` has a sigmoid router with a correction for the choice, a choice limited to the best
groups of experts, weights renormalised over the chosen experts and scaled, experts and a shared expert of the form
down(relu(up(h))^2).  ``norm.eps`` is the eps of every RMS norm inside the mixers.

Checkpoint names: ``embed``, ``final.norm`` (+ ``.alpha``, ``.b``), ``head``; layer i: ``l<i>.norm1``, ``l<i>.norm2``
(+ ``.alpha``, ``.b``); ``l<i>.mix.left.q|k`` (+ ``.b``), ``.talk``, ``.pb``, ``.g``, ``.o``, ``.out``;
``l<i>.mix.right.q|k|v|g|o|norm|out``; ``l<i>.mix.q|f|v|o|norm|lower`` and ``f.b``; ``l<i>.mlp.gate|up|down`` or
``l<i>.mlp.router``, ``l<i>.mlp.correction``, ``l<i>.mlp.e<n>.up|down``, ``l<i>.mlp.shared.up|down``.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Dict, List, Optional, Tuple

from ..parts.spec import EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .base import Architecture, ModelConfig, as_float, as_int, register_architecture
from .tumudra import RotaryConfig

LAYER_TYPES = ("parallel", "hgrn2")
MLP_KINDS = ("dense", "moe")
MAX_POSITIONS = 1 << 20          # rotations have no table; this only bounds a cache's longest sequence


def _obj(v: Any, what: str) -> Dict[str, Any]:
    if not isinstance(v, dict):
        raise TypeError(f"{what} must be an object, got {v!r}")
    return v


@dataclasses.dataclass(frozen=True)
class SigmoidAttentionConfig:
    """The left branch of ``parallel``."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotaryConfig
    chunk: Optional[int] = None              # mask.size; None: every earlier position

    @classmethod
    def parse(cls, m: Dict[str, Any], where: str) -> "SigmoidAttentionConfig":
        mask = m.get("mask")
        size = None if mask is None else _obj(mask, where + ".mask").get("size")
        return cls(heads=as_int(m.get("heads")), kv_heads=as_int(m.get("kv_heads")), dim=as_int(m.get("dim")),
                   vdim=as_int(m.get("vdim")), scale=as_float(m.get("scale")),
                   rot=RotaryConfig.parse(m.get("rot"), where + ".rot"), chunk=None if size is None else as_int(size))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale, "rot": self.rot.to_dict()}
        if self.chunk is not None:
            out["mask"] = {"size": self.chunk}
        return out

    def problems(self, where: str) -> List[str]:
        p: List[str] = []
        for name in ("heads", "kv_heads", "dim", "vdim"):
            if getattr(self, name) < 1:
                p.append(f"{where}.{name} must be >= 1 (got {getattr(self, name)})")
        if self.kv_heads >= 1 and self.heads % self.kv_heads:
            p.append(f"{where}: {self.kv_heads} kv_heads do not divide {self.heads} heads")
        if self.vdim != self.dim:
            p.append(f"{where}.vdim must equal dim, the values being the keys (got {self.vdim} and {self.dim})")
        if not math.isfinite(self.scale):
            p.append(f"{where}.scale must be finite (got {self.scale})")
        if self.chunk is not None and self.chunk < 1:
            p.append(f"{where}.mask.size must be >= 1 (got {self.chunk})")
        p.extend(self.rot.problems(where + ".rot", self.dim))
        return p


@dataclasses.dataclass(frozen=True)
class MemoryConfig:
    """A matrix memory: the right branch of ``parallel`` (with ``decay``) or the ``hgrn2`` mixer (without)."""

    heads: int
    dim: int
    vdim: int
    decay: Optional[Tuple[float, ...]] = None

    @classmethod
    def parse(cls, m: Dict[str, Any], where: str, with_decay: bool) -> "MemoryConfig":
        decay = None
        if with_decay:
            d = m.get("decay")
            if not isinstance(d, (list, tuple)):
                raise TypeError(f"{where}.decay must be a list, got {d!r}")
            decay = tuple(as_float(x) for x in d)
        return cls(heads=as_int(m.get("heads")), dim=as_int(m.get("dim")), vdim=as_int(m.get("vdim")), decay=decay)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}
        if self.decay is not None:
            out["decay"] = list(self.decay)
        return out

    def problems(self, where: str) -> List[str]:
        p: List[str] = []
        for name in ("heads", "dim", "vdim"):
            if getattr(self, name) < 1:
                p.append(f"{where}.{name} must be >= 1 (got {getattr(self, name)})")
        if self.dim > 256:
            p.append(f"{where}.dim must be at most 256 (got {self.dim})")
        if self.decay is not None:
            if len(self.decay) != self.heads:
                p.append(f"{where}.decay needs one number per head ({len(self.decay)} for {self.heads})")
            if any(not (0.0 <= d <= 1.0) for d in self.decay):
                p.append(f"{where}.decay: every decay lies in [0, 1]")
        return p


@dataclasses.dataclass(frozen=True)
class MlpConfig:
    kind: str
    ff: int                          # inner width: of the dense feed-forward, or of one expert
    experts: int = 0
    top: int = 0
    route_scale: float = 1.0
    groups: int = 1                  # equal groups of neighbouring experts
    keep: int = 1                    # groups whose experts can be chosen
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
        g = r.get("groups")
        count, keep = (1, 1) if g is None else (as_int(_obj(g, "mlp.router.groups").get("count")), as_int(g.get("keep")))
        shared = v.get("shared")
        return cls(kind, as_int(_obj(v.get("expert"), "mlp.expert").get("ff")), experts=as_int(r.get("experts")),
                   top=as_int(r.get("top")), route_scale=as_float(r.get("scale", 1.0)), groups=count, keep=keep,
                   shared_ff=None if shared is None else as_int(_obj(shared, "mlp.shared").get("ff")))

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        out: Dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff},
                               "router": {"experts": self.experts, "top": self.top, "scale": self.route_scale,
                                          "groups": {"count": self.groups, "keep": self.keep}}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out

    def problems(self, where: str) -> List[str]:
        p: List[str] = []
        if self.ff < 1:
            p.append(f"{where}: the inner width must be >= 1 (got {self.ff})")
        if self.kind == "moe":
            if self.experts < 1:
                p.append(f"{where}.router.experts must be >= 1 (got {self.experts})")
            elif not (1 <= self.top <= min(16, self.experts)):
                p.append(f"{where}.router.top must lie between 1 and min(16, experts) (got {self.top})")
            elif self.groups < 1 or self.experts % self.groups or not (1 <= self.keep <= self.groups):
                p.append(f"{where}.router.groups: count must divide the experts and keep lie between 1 and count "
                         f"(got {self.groups}, {self.keep} for {self.experts} experts)")
            elif self.keep * (self.experts // self.groups) < self.top:
                p.append(f"{where}.router.groups: {self.keep} groups of {self.experts // self.groups} experts cannot "
                         f"give {self.top} experts")
            if not math.isfinite(self.route_scale):
                p.append(f"{where}.router.scale must be finite (got {self.route_scale})")
            if self.shared_ff is not None and self.shared_ff < 1:
                p.append(f"{where}.shared.ff must be >= 1 (got {self.shared_ff})")
        return p


@dataclasses.dataclass(frozen=True)
class LayerConfig:
    type: str
    mlp: Optional[MlpConfig]
    attention: Optional[SigmoidAttentionConfig] = None       # parallel: the left branch
    memory: Optional[MemoryConfig] = None                    # parallel: the right branch; hgrn2: the mixer

    @classmethod
    def parse(cls, v: Any) -> "LayerConfig":
        v = _obj(v, "a layer")
        kind = v.get("type")
        if kind not in LAYER_TYPES:
            raise ValueError(f"layer type must be one of {LAYER_TYPES} (got {kind!r})")
        m = _obj(v.get("mixer"), "mixer")
        mlp = MlpConfig.parse(v.get("mlp"))
        if kind == "hgrn2":
            return cls(kind, mlp, memory=MemoryConfig.parse(m, "mixer", with_decay=False))
        return cls(kind, mlp, attention=SigmoidAttentionConfig.parse(_obj(m.get("left"), "mixer.left"), "mixer.left"),
                   memory=MemoryConfig.parse(_obj(m.get("right"), "mixer.right"), "mixer.right", with_decay=True))

    def to_dict(self) -> Dict[str, Any]:
        mixer = self.memory.to_dict() if self.type == "hgrn2" else {"left": self.attention.to_dict(),
                                                                     "right": self.memory.to_dict()}
        return {"type": self.type, "mixer": mixer, "mlp": None if self.mlp is None else self.mlp.to_dict()}

    def problems(self, where: str) -> List[str]:
        p: List[str] = []
        if self.attention is not None:
            p.extend(self.attention.problems(where + ".mixer.left"))
        p.extend(self.memory.problems(where + (".mixer.right" if self.type == "parallel" else ".mixer")))
        if self.mlp is not None:
            p.extend(self.mlp.problems(where + ".mlp"))
        return p


def _layers(v: Any) -> Tuple[LayerConfig, ...]:
    if not isinstance(v, (list, tuple)) or not v:
        raise TypeError("layers must be a list with at least one entry")
    return tuple(LayerConfig.parse(x) for x in v)


def _eps(v: Any) -> float:
    return as_float(_obj(v, "norm").get("eps"))


def _embedding_scale(v: Any) -> float:
    return as_float(_obj(v, "embedding").get("scale"))


def _loop(v: Any) -> Tuple[int, int, int]:
    if v is None:
        return (0, 0, 1)
    v = _obj(v, "loop")
    return as_int(v.get("start")), as_int(v.get("stop")), as_int(v.get("times"))


def _req(conv, key=None):
    md = {"convert": conv, "required": True}
    if key:
        md["key"] = key
    return dataclasses.field(default=None, metadata=md)


@dataclasses.dataclass(frozen=True)
class GuniraxConfig(ModelConfig):
    vocab: int = _req(as_int)
    width: int = _req(as_int)
    layers: Tuple[LayerConfig, ...] = _req(_layers)
    norm_eps: float = _req(_eps, key="norm")
    embedding_scale: float = _req(_embedding_scale, key="embedding")
    loop: Tuple[int, int, int] = dataclasses.field(default=(0, 0, 1), metadata={"convert": _loop})   # start, stop, times
    architecture: str = dataclasses.field(default="Gunirax", metadata={"convert": str})
    initializer_range: float = dataclasses.field(default=0.02, metadata={"convert": as_float})

    @classmethod
    def architecture_names(cls) -> Tuple[str, ...]:
        return ("Gunirax",)

    def to_dict(self) -> Dict[str, Any]:
        start, stop, times = self.loop
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "loop": {"start": start, "stop": stop, "times": times},
                "layers": [l.to_dict() for l in self.layers], "initializer_range": self.initializer_range}

    def problems(self) -> List[str]:
        p: List[str] = []
        if self.vocab < 1 or self.width < 1:
            p.append(f"vocab and width must be >= 1 (got {self.vocab}, {self.width})")
        if not self.norm_eps > 0:
            p.append(f"norm.eps must be > 0 (got {self.norm_eps})")
        if not math.isfinite(self.embedding_scale):
            p.append(f"embedding.scale must be finite (got {self.embedding_scale})")
        if not (1 <= len(self.layers) <= 1024):
            p.append(f"between 1 and 1024 layers (got {len(self.layers)})")
        start, stop, times = self.loop
        if not (0 <= start <= stop <= len(self.layers)) or not (1 <= times <= 64):
            p.append(f"loop: 0 <= start <= stop <= {len(self.layers)} layers and 1 <= times <= 64 "
                     f"(got start {start}, stop {stop}, times {times})")
        for i, layer in enumerate(self.layers):
            p.extend(layer.problems(f"layers[{i}]"))
        if not self.initializer_range > 0:
            p.append(f"initializer_range must be > 0 (got {self.initializer_range})")
        return p

    def layer_runs(self) -> Tuple[Tuple[int, bool], ...]:
        """The executed layers in order, as (layer, whether the embedded rows are added to the stream first)."""
        start, stop, times = self.loop
        runs: List[Tuple[int, bool]] = [(i, False) for i in range(start)]
        for k in range(times if stop > start else 0):
            runs += [(i, k > 0 and i == start) for i in range(start, stop)]
        runs += [(i, False) for i in range(stop, len(self.layers))]
        return tuple(runs)


def _dyt(cfg: GuniraxConfig) -> PartSpec:
    return PartSpec("dynamic_tanh", {"size": cfg.width})


def _norm_names(local: str, name: str) -> Dict[str, str]:
    return {f"{local}.weight": name, f"{local}.alpha": name + ".alpha", f"{local}.b": name + ".b"}


def _feed_forward(cfg: GuniraxConfig, m: MlpConfig, pre: str):
    W = cfg.width
    if m.kind == "dense":
        spec = PartSpec("gated_mlp", {"hidden_size": W, "intermediate_size": m.ff, "activation": "silu"})
        return spec, {"ff.gate_proj": pre + "gate", "ff.up_proj": pre + "up", "ff.down_proj": pre + "down"}
    names = {"ff.router": pre + "router", "ff.correction": pre + "correction"}
    for e in range(m.experts):
        names[f"ff.experts.{e}.up_proj"] = f"{pre}e{e}.up"
        names[f"ff.experts.{e}.down_proj"] = f"{pre}e{e}.down"
    shared = None
    if m.shared_ff is not None:
        shared = PartSpec("mlp", {"hidden_size": W, "intermediate_size": m.shared_ff, "activation": "relu2"})
        names["ff.shared.up_proj"] = pre + "shared.up"
        names["ff.shared.down_proj"] = pre + "shared.down"
    spec = PartSpec("routed_experts", {
        "hidden_size": W, "experts": m.experts, "top": m.top, "intermediate_size": m.ff, "gated": False,
        "activation": "relu2", "score": "sigmoid", "correction": True, "renormalize": True, "route_scale": m.route_scale,
        "groups": (m.groups, m.keep), "weight_on": "output", "shared": shared})
    return spec, names


def gunirax_spec(cfg: GuniraxConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = _dyt(cfg)
    layers, optional = [], []
    for i, lc in enumerate(cfg.layers):
        pre = f"l{i}."
        tensors = _norm_names("norms.pre_mixer", pre + "norm1")
        m = lc.memory
        if lc.type == "hgrn2":
            mixer = PartSpec("hgrn2", {"hidden_size": W, "n_heads": m.heads, "dim": m.dim, "vdim": m.vdim, "eps": eps})
            tensors.update({f"mixer.{n}": f"{pre}mix.{n}" for n in ("q", "f", "v", "o", "norm", "lower")})
            tensors["mixer.f_bias"] = pre + "mix.f.b"
        else:
            a = lc.attention
            left = PartSpec("sigmoid_attention", {
                "hidden_size": W, "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim, "scale": a.scale,
                "mask": {"kind": "causal", "size": 0} if a.chunk is None else {"kind": "chunk", "size": a.chunk},
                "bias": True, "qk_norm": {"eps": eps}, "head_bias": True, "talk": True, "out_gate": True,
                "values_from_keys": True, "position": a.rot.part(a.dim, "interleaved")})
            lp = pre + "mix.left."
            tensors.update({"mixer.left.q_proj": lp + "q", "mixer.left.q_bias": lp + "q.b", "mixer.left.k_proj": lp + "k",
                            "mixer.left.k_bias": lp + "k.b", "mixer.left.talk": lp + "talk", "mixer.left.head_bias": lp + "pb",
                            "mixer.left.g_proj": lp + "g", "mixer.left.o_proj": lp + "o", "mixer.left.out": lp + "out"})
            right = PartSpec("lightning", {"hidden_size": W, "n_heads": m.heads, "dim": m.dim, "vdim": m.vdim,
                                           "decay": m.decay, "eps": eps})
            rp = pre + "mix.right."
            tensors.update({f"mixer.right.{n}": rp + n for n in ("q", "k", "v", "o", "norm", "out")})
            tensors["mixer.right.gate"] = rp + "g"
            mixer = PartSpec("parallel", {"hidden_size": W, "eps": eps, "branches": {"left": left, "right": right}})
        ff = None
        norms = {"pre_mixer": norm}
        if lc.mlp is not None:
            ff, names = _feed_forward(cfg, lc.mlp, pre + "mlp.")
            tensors.update(names)
            tensors.update(_norm_names("norms.pre_ff", pre + "norm2"))
            norms["pre_ff"] = norm
        else:                                                # a layer without a feed-forward may still carry its second norm
            optional += [pre + "norm2", pre + "norm2.alpha", pre + "norm2.b"]
        layers.append(LayerSpec(block=PartSpec("prenorm", {}), mixer=mixer, feed_forward=ff, norms=norms, tensors=tensors))
    # every executed layer has a cache line of its own: a pass of the loop keeps its own keys, values and states
    schedule = tuple(ScheduleEntry(layer=i, cache=n, add_embedding=again) for n, (i, again) in enumerate(cfg.layer_runs()))
    return ModelSpec(
        name="Gunirax", hidden_size=W,
        embedding=EmbeddingSpec(cfg.vocab, W, cfg.embedding_scale, "embed"),
        layers=tuple(layers), schedule=schedule,
        head=HeadSpec(cfg.vocab, W, tied=False, tensor="head", softcap=None, norm=norm, norm_tensor="final.norm"),
        max_positions=MAX_POSITIONS, stop_ids=(), init_std=cfg.initializer_range, init_norm_std=0.1,
        optional_tensors=tuple(optional))


GUNIRAX = register_architecture(Architecture(
    name="Gunirax", config_cls=GuniraxConfig, build_spec=gunirax_spec, aliases=("gunirax",)))
