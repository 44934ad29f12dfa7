"""Fifudra configuration, from the keys of its config.json.

The file lists the layers one by one, says which run of them is repeated, and how many residual streams there are::

    {"architecture": "Fifudra", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "streams": S | null, "loop": {"start": a, "stop": b, "times": n} | null,
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads": H, "dim": d, "rot_dim": r, "vdim": dv, "q_rank": Rq, "kv_rank": Rkv, "scale": s,
                           "rot": {"base": b, "dims": r, "scaling": {"factor": f, "original": L, "fast": x, "slow": y} | null}},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "delta", "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "conv": taps},
                 "mlp": {"kind": "moe", "expert": {"ff": F},
                         "router": {"experts": E, "top": k, "scale": c, "groups": {"count": n, "keep": m} | null}}},
                {"type": "hgrn2", "mixer": {"heads": H, "dim": d, "vdim": dv}, "mlp": null}, ...]}

Every size and constant is read from there; a layer may differ from the next in all of them.  ``streams`` left out or
null means one plain residual stream, ``loop`` left out no repetition, ``embedding.scale`` and ``router.scale`` left
out 1, ``groups`` left out a router that may choose among all experts, ``scaling`` left out plain rotary frequencies,
``mlp`` null a layer without a feed-forward.  ``max_positions`` (optional) bounds a sequence's length.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .base import ConfigError, KeyReader, ModelConfig

MIXER_TYPES = ("latent_attention", "delta", "hgrn2")
MLP_KINDS = ("dense", "moe")
DEFAULT_MAX_POSITIONS = 1 << 20      # the design itself has no limit: positions are turned into angles on the fly


@dataclass(frozen=True)
class RotarySpec:
    base: float
    dims: int
    factor: float = 0.0        # 0: no scaling of the frequencies
    original: float = 0.0
    fast: float = 0.0
    slow: float = 0.0

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        out = dict(base=r.number("base", positive=True), dims=r.integer("dims", minimum=0))
        sc = data.get("scaling")
        if sc is not None:
            s = KeyReader(sc, where + ".scaling")
            out.update(factor=s.number("factor", positive=True), original=s.number("original", positive=True),
                       fast=s.number("fast", positive=True), slow=s.number("slow", positive=True))
        if out["dims"] % 2:
            raise ConfigError(f"{where}: 'dims' must be even (lanes turn in pairs)")
        return cls(**out)

    def to_dict(self):
        d = {"base": self.base, "dims": self.dims}
        if self.factor:
            d["scaling"] = {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}
        return d


@dataclass(frozen=True)
class LatentAttentionSpec:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: RotarySpec

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        if not isinstance(data.get("rot"), dict):
            raise ConfigError(f"{where}: required key 'rot' is missing")
        out = cls(heads=r.integer("heads", minimum=1), dim=r.integer("dim", minimum=1), rot_dim=r.integer("rot_dim", minimum=0),
                  vdim=r.integer("vdim", minimum=1), q_rank=r.integer("q_rank", minimum=1), kv_rank=r.integer("kv_rank", minimum=1),
                  scale=r.number("scale"), rot=RotarySpec.from_dict(data["rot"], where + ".rot"))
        if out.rot.dims != out.rot_dim:
            raise ConfigError(f"{where}: 'rot.dims' must equal 'rot_dim' (the whole rotated part turns)")
        return out

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "q_rank": self.q_rank,
                "kv_rank": self.kv_rank, "scale": self.scale, "rot": self.rot.to_dict()}


@dataclass(frozen=True)
class DeltaSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        heads = r.integer("heads", minimum=1)
        out = cls(heads=heads, kv_heads=r.integer("kv_heads", heads, minimum=1), dim=r.integer("dim", minimum=1),
                  vdim=r.integer("vdim", minimum=1), conv=r.integer("conv", minimum=1))
        if out.heads % out.kv_heads:
            raise ConfigError(f"{where}: 'kv_heads' must divide 'heads'")
        return out

    def to_dict(self):
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class Hgrn2Spec:
    heads: int
    dim: int
    vdim: int

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        return cls(heads=r.integer("heads", minimum=1), dim=r.integer("dim", minimum=1), vdim=r.integer("vdim", minimum=1))

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}


MIXER_SPECS = {"latent_attention": LatentAttentionSpec, "delta": DeltaSpec, "hgrn2": Hgrn2Spec}


@dataclass(frozen=True)
class FifudraMlp:
    kind: str                  # "dense" or "moe"
    ff: int = 0                # dense: hidden size; moe: an expert's hidden size
    experts: int = 0
    top: int = 0
    scale: float = 1.0         # on the chosen experts' weights
    groups: int = 0            # 0: the router chooses among all experts
    keep: int = 0

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        kind = r.string("kind")
        if kind not in MLP_KINDS:
            raise ConfigError(f"{where}: kind '{kind}' is not one of {MLP_KINDS}")
        if kind == "dense":
            return cls(kind, ff=r.integer("ff", minimum=1))
        for key in ("router", "expert"):
            if not isinstance(data.get(key), dict):
                raise ConfigError(f"{where}: required key '{key}' is missing")
        router = KeyReader(data["router"], where + ".router")
        groups = keep = 0
        if data["router"].get("groups") is not None:
            g = KeyReader(data["router"]["groups"], where + ".router.groups")
            groups, keep = g.integer("count", minimum=1), g.integer("keep", minimum=1)
        out = cls(kind, ff=KeyReader(data["expert"], where + ".expert").integer("ff", minimum=1),
                  experts=router.integer("experts", minimum=1), top=router.integer("top", minimum=1),
                  scale=router.number("scale", 1.0), groups=groups, keep=keep)
        if out.top > out.experts:
            raise ConfigError(f"{where}.router: 'top' exceeds 'experts'")
        if groups and (out.experts % groups or keep > groups or keep * (out.experts // groups) < out.top):
            raise ConfigError(f"{where}.router.groups: {groups} groups of which {keep} are kept cannot serve "
                              f"{out.top} of {out.experts} experts")
        return out

    def to_dict(self):
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        router = {"experts": self.experts, "top": self.top, "scale": self.scale}
        if self.groups:
            router["groups"] = {"count": self.groups, "keep": self.keep}
        return {"kind": "moe", "router": router, "expert": {"ff": self.ff}}


@dataclass(frozen=True)
class FifudraLayer:
    type: str
    mixer: Any
    mlp: FifudraMlp | None = None

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        kind = r.string("type")
        if kind not in MIXER_TYPES:
            raise ConfigError(f"{where}: layer type '{kind}' is not one of {MIXER_TYPES}")
        if not isinstance(data.get("mixer"), dict):
            raise ConfigError(f"{where}: required key 'mixer' is missing")
        mlp = data.get("mlp")
        return cls(kind, MIXER_SPECS[kind].from_dict(data["mixer"], where + ".mixer"),
                   None if mlp is None else FifudraMlp.from_dict(mlp, where + ".mlp"))

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class FifudraConfig(ModelConfig):
    vocab: int
    width: int
    layers: tuple
    norm_eps: float = 1e-5
    embedding_scale: float = 1.0
    streams: int = 0                 # 0: one plain residual stream
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1              # layers loop_start .. loop_stop - 1 run this many times in a row
    max_positions: int = DEFAULT_MAX_POSITIONS
    architecture: str = "Fifudra"
    extra: dict = field(default_factory=dict, compare=False)

    def __post_init__(self):
        object.__setattr__(self, "layers", tuple(self.layers))
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        if not (0 <= self.loop_start <= self.loop_stop <= len(self.layers)) or self.loop_times < 1:
            raise ConfigError(f"config.json.loop: layers {self.loop_start} .. {self.loop_stop} x {self.loop_times} "
                              f"of {len(self.layers)} layers")

    def run_order(self) -> tuple:
        """The layers in the order they run, the looped ones as often as they run."""
        n = len(self.layers)
        a, b = self.loop_start, self.loop_stop
        return tuple(range(a)) + tuple(range(a, b)) * self.loop_times + tuple(range(b, n))

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "FifudraConfig":
        r = KeyReader(data)
        layers = data.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        norm = KeyReader(data.get("norm") or {}, "config.json.norm")
        emb = KeyReader(data.get("embedding") or {}, "config.json.embedding")
        loop = dict(loop_start=0, loop_stop=0, loop_times=1)
        if data.get("loop") is not None:
            lr = KeyReader(data["loop"], "config.json.loop")
            loop = dict(loop_start=lr.integer("start", minimum=0), loop_stop=lr.integer("stop", minimum=0),
                        loop_times=lr.integer("times", 1, minimum=1))
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   layers=tuple(FifudraLayer.from_dict(l, f"config.json.layers[{i}]") for i, l in enumerate(layers)),
                   norm_eps=norm.number("eps", positive=True), embedding_scale=emb.number("scale", 1.0),
                   streams=r.integer("streams", 0, minimum=0) or 0,
                   max_positions=r.integer("max_positions", DEFAULT_MAX_POSITIONS, minimum=1),
                   architecture=r.string("architecture", "Fifudra"), **loop)

    def to_dict(self) -> dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "embedding": {"scale": self.embedding_scale}, "layers": [l.to_dict() for l in self.layers]}
        if self.streams:
            d["streams"] = self.streams
        if self.loop_times != 1 or self.loop_stop > self.loop_start:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d
